"""Build step: turn the interpreter's C++ ``switch`` into a real jump table at the PTX level.

nvcc lowers a dense C++ ``switch`` to a balanced tree of compare-and-branch pairs (no ``brx.idx`` is ever emitted),
which for the interpreter's ~950 (opcode, stack depth) cases means about ten dependent branches per interpreted
instruction. The kernels therefore leave two kinds of marker comments in their PTX (see ``interpret`` in
``csrc/gint_interp.cuh``):

    // GINT_DISPATCH %rN site S depth D;   at the end of every handler (and once at loop entry): %rN holds the next opcode
    // GINT_TARGET <key>;      first statement of the case for <key>   (``default`` for the default case)

This module rewrites the PTX text of one kernel: after the DISPATCH marker it inserts

    $gint_targets_D: .branchtargets L_op0, L_op1, ...;      (one table per stack depth D)
    brx.idx.uni %rN, $gint_targets_D;

where ``L_op`` is the label of the basic block that starts with ``GINT_TARGET D*n_ops+op`` (the default block for
combinations without a case) and D is the stack depth after the handler the marker sits in -- programs are straight
line, so the depth before every instruction is static and only the opcode has to be looked up at run time. Restricting
each branch to the ~142 targets of one depth also keeps the control-flow graph ptxas has to digest small. The compare tree that follows becomes unreachable and is dropped by ptxas. The key is warp-uniform by
construction (every lane of a warp interprets the same program), hence ``.uni``.

The rewrite is validated structurally (exactly one DISPATCH marker, unique TARGET keys, every marker at the head of a
labelled block) and the build fails if any check does not hold -- it never guesses.
"""
from __future__ import annotations

import re

_LABEL = re.compile(r"^(\$L__BB\d+_\d+):\s*$")
_TARGET = re.compile(r"^\s*// GINT_TARGET (\w+);")
_DISPATCH = re.compile(r"^\s*// GINT_DISPATCH (%r\d+) site (\w+) depth (\w+);")
_CONTROL = re.compile(r"^\s*(@%p\d+\s+)?(bra|brx|ret|exit|call|trap)\b")


class PtxDispatchError(RuntimeError):
    pass


SMALL_HANDLER_INSNS = 64


def cluster_small_handlers(lines: list[str], limit: int = SMALL_HANDLER_INSNS, order=None, always=None) -> tuple[list[str], int]:
    """Move every small single-block handler next to the others, ahead of the large ones.

    The compiler emits handlers in key order, so the few-instruction handlers a program actually runs (moves, arithmetic,
    register loads and stores, lane permutes) lie scattered between tile accesses and inlined math routines of several
    kilobytes each: the hot code of a program is a few hundred instructions spread over megabytes, every jump lands on a
    different cache line and the lines fetched after it belong to cold handlers. A handler that is ONE basic block -- label,
    GINT_TARGET marker, straight-line code, its own ``brx.idx`` (or ``ret``) -- can be moved freely: control only ever enters
    it through a jump table and leaves it through its terminator. Such blocks of at most ``limit`` instructions are cut out
    and re-emitted together, in key order (stack depth, then opcode), right after the entry dispatch. Everything else stays
    where it was. Returns (lines, number of handlers moved)."""
    def is_code(t: str) -> bool:
        t = t.strip()
        return bool(t) and not t.startswith("//") and not t.startswith(".") and t not in ("{", "}") and not t.endswith(":")

    entry = next((i for i, t in enumerate(lines) if t.lstrip().startswith("brx.idx.uni") and i > 0 and "$gint_targets" in t), None)
    if entry is None:
        return lines, 0
    label_at = [i for i, t in enumerate(lines) if _LABEL.match(t.strip())]
    moved: list[tuple[int, int, int]] = []     # (key, start line, end line exclusive)
    for n, start in enumerate(label_at):
        end = label_at[n + 1] if n + 1 < len(label_at) else None
        if end is None or start < entry:
            continue
        body = lines[start + 1:end]
        key = next((m.group(1) for t in body if (m := _TARGET.match(t))), None)
        if key is None or key == "default":
            continue
        code = [t.strip() for t in body if is_code(t)]
        if not code or (len(code) > limit and not (always and int(key) in always)):
            continue
        if not (code[-1].startswith("brx.idx.uni") or code[-1].startswith("ret;")):
            continue                                          # falls through or ends otherwise: leave it
        if any(_CONTROL.match(t) for t in code[:-1]):
            continue                                          # internal control flow
        # nothing may fall through INTO the block: the last code line before its label must be an unconditional transfer
        j = start - 1
        while j >= 0 and not is_code(lines[j]):
            j -= 1
        prev = lines[j].strip() if j >= 0 else ""
        if not (prev.startswith("brx.idx.uni") or prev.startswith("ret;") or re.match(r"^bra(\.uni)?\s", prev)):
            continue
        moved.append((int(key), start, end))
    if not moved:
        return lines, 0
    cut = set()
    for _, a, b in moved:
        cut.update(range(a, b))
    out: list[str] = []
    for i, t in enumerate(lines):
        if i in cut:
            continue
        out.append(t)
        if i == entry:
            for _, a, b in sorted(moved, key=(lambda m: order(m[0])) if order else None):
                out.extend(lines[a:b])
    return out, len(moved)


def rewrite(ptx: str, n_keys: int, n_ops: int = 142, cluster: bool = True, hot: set | None = None, hot_any_size: bool = False) -> tuple[str, dict]:
    """Return (rewritten PTX, stats). ``n_keys`` is the size of the dispatch key space. ``hot_any_size``: single-block handlers
    in ``hot`` join the cluster whatever their length (kernels whose hot handlers are long fused sequences)."""
    lines = ptx.split("\n")
    # depth -1 stands for "all": the non-threaded form, one table over every (depth, opcode) key
    dispatch = [(i, m.group(1), m.group(2), -1 if m.group(3) == "all" else int(m.group(3)))
                for i, line in enumerate(lines) if (m := _DISPATCH.match(line))]
    sites = [d[2] for d in dispatch]
    if sites.count("entry") != 1:
        raise PtxDispatchError(f"expected exactly one entry GINT_DISPATCH marker, found {sites.count('entry')}")
    if len(set(sites)) != len(sites):
        raise PtxDispatchError("a GINT_DISPATCH site appears twice (the compiler duplicated a handler)")

    targets: dict[str, str] = {}
    for i, line in enumerate(lines):
        m = _TARGET.match(line)
        if not m:
            continue
        key = m.group(1)
        if key in targets:
            raise PtxDispatchError(f"GINT_TARGET {key} appears twice (the compiler duplicated the dispatch loop)")
        # the marker must head a labelled basic block: walk back over non-control statements to the label
        j = i - 1
        label = None
        while j >= 0:
            prev = lines[j].strip()
            lm = _LABEL.match(prev)
            if lm:
                label = lm.group(1)
                break
            if _CONTROL.match(prev) or prev.startswith("{") or prev.startswith("}"):
                break
            j -= 1
        if label is None:
            raise PtxDispatchError(f"GINT_TARGET {key} (line {i + 1}) is not at the head of a labelled block")
        targets[key] = label
    if "default" not in targets:
        raise PtxDispatchError("no GINT_TARGET default marker")
    numeric = {int(k): v for k, v in targets.items() if k != "default"}
    if not numeric or max(numeric) >= n_keys:
        raise PtxDispatchError("dispatch keys out of range")

    threaded = len(sites) > 1
    if threaded:
        n_halt = sum(1 for k in numeric if k % n_ops == 0)   # Halt handlers return instead of dispatching
        if len(sites) - 1 + n_halt != len(numeric):
            raise PtxDispatchError(f"{len(numeric)} handlers but {len(sites) - 1} dispatch sites and {n_halt} Halt handlers")

    n_depths = n_keys // n_ops
    indent = "\t"

    def table_name(depth: int) -> str:
        return "$gint_targets_all" if depth < 0 else f"$gint_targets_{depth}"

    def table_decl(depth: int) -> list[str]:
        keys = range(n_keys) if depth < 0 else range(depth * n_ops, (depth + 1) * n_ops)
        labs = [numeric.get(k, targets["default"]) for k in keys]
        decl = [f"{indent}{table_name(depth)}: .branchtargets"]
        for i in range(0, len(labs), 8):
            chunk = labs[i:i + 8]
            decl.append(f"{indent}{indent}" + ", ".join(chunk) + (";" if i + 8 >= len(labs) else ","))
        return decl

    first = min(d[0] for d in dispatch)
    used_depths = sorted({d[3] for d in dispatch})
    if max(used_depths) >= n_depths:
        raise PtxDispatchError("dispatch depth out of range")
    # Where each branch goes. The entry site sits just before the switch: its brx follows the marker and the compare tree
    # after it becomes unreachable. A handler's marker is the last statement of the handler; whatever the compiler put
    # between it and the block's terminator (copies for the fallback loop) must still run, so the brx REPLACES the
    # terminator, which has to be the unconditional branch back to the loop header.
    insert_after: dict[int, str] = {}
    replace: dict[int, str] = {}
    for d_line, key_reg, site, depth in dispatch:
        brx = f"{indent}brx.idx.uni {key_reg}, {table_name(depth)};"
        if site == "entry":
            insert_after[d_line] = brx
            continue
        j = d_line + 1
        while j < len(lines) and not _CONTROL.match(lines[j]) and not _LABEL.match(lines[j].strip()):
            j += 1
        if j >= len(lines) or not re.match(r"^\s*bra(\.uni)?\s+\$L__BB\d+_\d+;", lines[j]):
            raise PtxDispatchError(f"handler {site}: expected an unconditional branch after its dispatch marker, found: "
                                   f"{lines[j].strip() if j < len(lines) else 'end of file'}")
        replace[j] = brx
    out = []
    for i, line in enumerate(lines):
        if i in replace:
            out.append(replace[i])
            continue
        out.append(line)
        if i == first:                      # all tables are declared once, before their first use in the text
            for depth in used_depths:
                out.extend(table_decl(depth))
        if i in insert_after:
            out.append(insert_after[i])
    n_moved = 0
    if cluster and threaded:
        # profile-guided order: the handlers that recorded programs run (gint_b200/hot_handlers.py) first, next to each
        # other, then the other small ones; within each group by stack depth and opcode
        hot_keys = {d * n_ops + o for d, o in (hot or ())}

        def order(key: int):
            return (0 if key in hot_keys else 1, key)
        out, n_moved = cluster_small_handlers(out, order=order, always=hot_keys if hot_any_size else None)
    return "\n".join(out), {"cases": len(numeric), "keys": n_keys, "sites": len(sites), "tables": len(used_depths), "clustered": n_moved}
