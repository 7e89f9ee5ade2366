"""Which (stack depth, opcode) handlers do real programs run? -- input for the kernels' code layout.

    python -m gint_b200.hot_handlers          # rewrites gint_b200/csrc/hot_handlers.json

The interpreter kernels hold one handler per (opcode, stack depth): well over a thousand blocks of code, of which any one
program runs a few dozen. Which ones are run is far from uniform -- frontend- and conductor-generated programs live at small
stack depths and use a few dozen opcodes -- and the instruction cache works best when the handlers a program jumps between lie
close together. The build step (``gint_b200/ptx_dispatch.py``) therefore emits the handlers listed here first, next to each
other, before all others: a profile-guided layout, with the recorded programs of ``gint_b200/data/programs.json`` (streams
recorded from the reference's frontend, small-matrix helpers and torch.compile backend at many sizes) as the profile.

The list is derived with the library's own pre-decoder (``gint_debug_transform``), i.e. it names the handlers of the streams the
kernels actually run (early-issued loads, fast accesses, fused handlers), and it is keyed by opcode NUMBERS: it has to be
regenerated whenever the internal opcode numbering changes (a CPU test compares the file with a fresh derivation).
"""
from __future__ import annotations

import ctypes
import json
import os
import re

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
TABLE = os.path.join(HERE, "csrc", "hot_handlers.json")


def _header_int(name: str, file: str) -> int:
    with open(os.path.join(HERE, "csrc", file)) as f:
        return int(re.search(rf"#define {name} (\d+)", f.read()).group(1))


def _effects() -> dict[int, int]:
    """Net stack effect of every non-fused dispatch opcode, from the X-macro lists of gint_opcodes.h."""
    with open(os.path.join(HERE, "csrc", "gint_opcodes.h")) as f:
        text = f.read()
    return {int(num): int(net) for _, num, _, net in re.findall(r"X\((\w+), (\d+), (-?\d+), (-?\d+)\)", text)}


def derive() -> dict:
    from .host import capi
    from .host.utils import fill_tensor_info
    from .programs import load_records, recorded
    lib = capi.load_library()
    fused_first = _header_int("GINT_FUSED_FIRST", "gint_fused.h")
    n_dispatch = _header_int("GINT_N_DISPATCH_PLAIN", "gint_opcodes.h")
    n_dispatch_rf = _header_int("GINT_N_DISPATCH_RF", "gint_opcodes.h")     # the register-file kernels dispatch on more opcodes
    n_dispatch_vec = _header_int("GINT_N_DISPATCH_VEC", "gint_opcodes.h")   # and so do the vector-layout kernels
    buf = (ctypes.c_int32 * (256 * 10))()
    n_fused = lib.gint_debug_fused_table(buf, 256)
    assert n_fused > 0
    members = {buf[10 * k]: [buf[10 * k + 2 + j] for j in range(buf[10 * k + 1])] for k in range(n_fused)}
    net = _effects()

    def net_of(op: int) -> int:
        return sum(net[m] for m in members[op]) if op in members else net[op]

    keys: set[tuple[int, int]] = set()       # handlers of the ordinary streams
    rf_keys: set[tuple[int, int]] = set()    # handlers of the streams with the virtual registers in shared memory (their own kernels)
    vec_keys: set[tuple[int, int]] = set()   # handlers of the vector-layout streams (their own kernels)
    for name in load_records():
        if name == "execute_everything":      # refused by the library (deeper than any kernel's stack)
            continue
        prog = recorded(name)
        code = np.ascontiguousarray(prog.bytecode)
        ti = capi.HTensorInfo()
        fill_tensor_info(ti, prog.tensor_infos)
        cap = code.size + 64
        ops, operands = (ctypes.c_int32 * cap)(), (ctypes.c_uint32 * cap)()
        for early in (0, 1, 2, 3, 5):         # bit 0: early-issue pass; bit 1: registers in shared memory; bit 2: vector layout
            n = lib.gint_debug_transform(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(code.size), ctypes.byref(ti),
                                         len(prog.tensor_infos), early, 1, ops, operands, cap)
            if n == 0 and early & 6:          # the program does not qualify for that stream
                continue
            assert n > 0, (name, n)
            depth = 0
            for i in range(n):
                op = ops[i]
                if op < 0:                    # absorbed into the fused handler before it
                    continue
                (rf_keys if early & 2 else vec_keys if early & 4 else keys).add((depth, op))
                depth += net_of(op)
    return {"n_dispatch": n_dispatch, "n_dispatch_rf": n_dispatch_rf, "fused_first": fused_first,
            "n_dispatch_vec": n_dispatch_vec, "keys": sorted([d, o] for d, o in keys), "rf_keys": sorted([d, o] for d, o in rf_keys),
            "vec_keys": sorted([d, o] for d, o in vec_keys)}


def load(family: str = "plain") -> set[tuple[int, int]]:
    """The committed list as a set of (depth, opcode); empty if the file is absent or was made for another numbering.
    ``family``: "plain", "rf" (the kernels that keep the virtual registers in shared memory) or "vec" (vector layout)."""
    if family not in ("plain", "rf", "vec"):
        raise ValueError(f"unknown kernel family {family!r}")
    try:
        with open(TABLE) as f:
            t = json.load(f)
        if t["n_dispatch"] != _header_int("GINT_N_DISPATCH_PLAIN", "gint_opcodes.h") or t["fused_first"] != _header_int("GINT_FUSED_FIRST", "gint_fused.h") or \
                t["n_dispatch_rf"] != _header_int("GINT_N_DISPATCH_RF", "gint_opcodes.h") or \
                t["n_dispatch_vec"] != _header_int("GINT_N_DISPATCH_VEC", "gint_opcodes.h"):
            return set()
        keys = t[{"plain": "keys", "rf": "rf_keys", "vec": "vec_keys"}[family]]
    except (OSError, KeyError, ValueError):
        return set()
    return {(d, o) for d, o in keys}


def main() -> None:
    t = derive()
    with open(TABLE, "w") as f:
        json.dump(t, f)
    print(f"{TABLE}: {len(t['keys'])} handlers, {len(t['rf_keys'])} for the register-file kernels, {len(t['vec_keys'])} for the vector-layout kernels")


if __name__ == "__main__":
    main()
