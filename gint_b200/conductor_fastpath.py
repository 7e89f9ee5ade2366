"""Run a conductor-compiled graph's bytecode steps through ``gint_execute_plan``: one library call per run of consecutive
subgraph steps instead of one Python-level ``executor.execute`` per subgraph.

The reference's torch.compile backend ends in a closure ``execute(*args)`` that walks a flat step list in Python
(``gint/conductor/compiler.py:1442-1485``): per subgraph it allocates the outputs, writes base pointers into
``TensorInterface`` skeletons and calls ``executor.execute``. The conductor stays unchanged here; ``accelerate(execute)`` reads
that closure's own step list (its free variables ``plan`` / ``sg_dispatch``), and returns a callable with the same behaviour
in which

* every subgraph program is created once, up front, and its handle and descriptor-slot order are kept in a C array of
  ``gint_plan_step`` records,
* a call writes the fresh tensors' addresses straight into that array (no skeleton objects, no per-call cache lookup) and
* consecutive subgraph steps are launched by ONE ``gint_execute_plan`` call (eager fallback steps in between split the runs,
  so stream order is what the original loop produced), and
* a row gather that the conductor leaves to torch eager -- ``g = table[idx]`` (``aten.index.Tensor``, not lowered:
  ``gint/conductor/op_registry.py:1058-1132``) -- whose only consumer is one subgraph that reads ``g`` one row per logical program
  is folded into that subgraph's launch (``gint_execute_gathered``): the program reads ``table[idx[b]]`` in place, the gather
  kernel and the intermediate tensor disappear (``fold_gathers=False`` keeps them).

``install(accelerate_conductor=True)`` (``gint_b200/dropin.py``) applies this to every graph the conductor compiles afterwards,
by wrapping ``GintCompiler.compile``; nothing of the conductor's source is modified. Falls back to the original closure when
its shape is not the one described above (a different conductor version).
"""
from __future__ import annotations

import ctypes
from typing import Callable

import torch

from .host import capi
from .host.executor import B200Executor
from .opcodes import MAX_N_TENSORS

# step kinds of the conductor's flat plan (gint/conductor/compiler.py:1296-1302)
STEP_PH, STEP_SUBGRAPH, STEP_GET_ATTR, STEP_EAGER, STEP_OUT_NODE, STEP_OUT_CONST, STEP_OUT_SEQ = range(7)


def _closure_vars(fn) -> dict:
    names = fn.__code__.co_freevars
    cells = fn.__closure__ or ()
    out = {}
    for n, c in zip(names, cells):
        try:
            out[n] = c.cell_contents
        except ValueError:       # empty cell
            pass
    return out


class _Ref:
    """Stands for ``results[i]`` while a step's argument resolvers are evaluated symbolically."""
    __slots__ = ("i",)

    def __init__(self, i: int) -> None:
        self.i = i


def _refs_in(value, out: set) -> None:
    if isinstance(value, _Ref):
        out.add(value.i)
    elif isinstance(value, (list, tuple)):
        for v in value:
            _refs_in(v, out)
    elif isinstance(value, dict):
        for v in value.values():
            _refs_in(v, out)


def _find_foldable_gathers(plan, sg_dispatch, results_size) -> dict:
    """{position of the eager step in `plan`: (results index of g, of the table, of the index, sg_dispatch position)} for every
    ``g = aten.index.Tensor(table, [idx])`` whose result is read by exactly one subgraph, as one of its inputs with no offset,
    and by nothing else."""
    try:
        index_op = torch.ops.aten.index.Tensor
    except AttributeError:
        return {}
    probe = [_Ref(i) for i in range(results_size)]
    found = {}
    for pos, step in enumerate(plan):
        if step[0] != STEP_EAGER or step[2] is not index_op or step[4]:
            continue
        try:
            args = [r(probe) for r in step[3]]
        except Exception:
            continue
        if len(args) != 2 or not isinstance(args[0], _Ref) or not isinstance(args[1], (list, tuple)) or len(args[1]) != 1 or not isinstance(args[1][0], _Ref):
            continue
        g_idx, table_idx, index_idx = step[1], args[0].i, args[1][0].i
        users_sg, other_use = [], False
        for pos2, st in enumerate(plan):
            if pos2 == pos:
                continue
            k = st[0]
            if k == STEP_SUBGRAPH:
                for in_idx, _, off in sg_dispatch[st[1]][2]:
                    if in_idx == g_idx:
                        users_sg.append((st[1], off))
            elif k == STEP_EAGER:
                used: set = set()
                try:
                    _refs_in([r(probe) for r in st[3]], used)
                    _refs_in({k_: r(probe) for k_, r in st[4]}, used)
                except Exception:
                    other_use = True
                other_use = other_use or g_idx in used
            elif k == STEP_OUT_NODE:
                other_use = other_use or st[1] == g_idx
            elif k == STEP_OUT_SEQ:
                other_use = other_use or any(is_node and v == g_idx for is_node, v in st[1])
        if other_use or len(users_sg) != 1 or users_sg[0][1] != 0:
            continue
        found[pos] = (g_idx, table_idx, index_idx, users_sg[0][0])
    return found


def accelerate(execute: Callable, executor: B200Executor, fold_gathers: bool = True) -> Callable:
    """A drop-in replacement for the conductor's ``execute`` closure (see the module docstring); ``execute`` itself is returned
    when it cannot be taken apart."""
    env = _closure_vars(execute)
    plan, sg_dispatch, results_size = env.get("plan"), env.get("sg_dispatch"), env.get("results_size")
    if not isinstance(plan, list) or not isinstance(sg_dispatch, list) or not isinstance(results_size, int):
        return execute
    if any(not (isinstance(s, tuple) and s and isinstance(s[0], int) and 0 <= s[0] <= STEP_OUT_SEQ) for s in plan):
        return execute

    lib = executor._lib
    n_sg = sum(1 for s in plan if s[0] == STEP_SUBGRAPH)
    if n_sg == 0:
        return execute
    steps_c = (capi.PlanStepC * n_sg)()
    state = {"ctx": None, "device": None}

    # per subgraph: where each tensor's address goes in the C array
    lowered = []       # parallel to the subgraph steps, in plan order
    fast_plan = []     # the new step list: subgraph runs are (KIND_RUN, first, count, [alloc/patch records])
    KIND_RUN, KIND_GATHERED = 100, 101
    gathers = _find_foldable_gathers(plan, sg_dispatch, results_size) if fold_gathers else {}
    gather_of_sg = {v[3]: (pos, v) for pos, v in gathers.items()}      # sg_dispatch position -> the eager step folded into it
    k = 0
    for pos, step in enumerate(plan):
        if pos in gathers:
            continue                      # the gather itself: folded into its consumer (or replayed there, see _run_gathered)
        if step[0] != STEP_SUBGRAPH:
            fast_plan.append(step)
            continue
        comp_sg, ti_skeletons, input_writes, output_writes, output_shapes, ref_idx = sg_dispatch[step[1]]
        rec = {"comp_sg": comp_sg, "skeletons": ti_skeletons, "k": k, "ref": ref_idx,
               "outs": [(out_idx, skel_idx, tuple(shape)) for (out_idx, skel_idx), shape in zip(output_writes, output_shapes)],
               "ins": [(in_idx, skel_idx, off) for in_idx, skel_idx, off in input_writes], "slots_of": None}
        lowered.append(rec)
        if step[1] in gather_of_sg:
            gpos, (g_idx, table_idx, index_idx, _) = gather_of_sg[step[1]]
            rec.update(gather=(g_idx, table_idx, index_idx), gather_step=plan[gpos], gather_ok=None)
            fast_plan.append((KIND_GATHERED, k, rec))
            k += 1
            continue
        if fast_plan and fast_plan[-1][0] == KIND_RUN:
            fast_plan[-1][2].append(rec)
        else:
            first_ptr = ctypes.cast(ctypes.byref(steps_c, k * ctypes.sizeof(capi.PlanStepC)), ctypes.POINTER(capi.PlanStepC))
            fast_plan.append((KIND_RUN, k, [rec], first_ptr))
        k += 1

    def _prepare():
        """First call (a CUDA context exists now): create the programs and fix the slot order of every step."""
        device, ctx = executor._ctx()
        for rec in lowered:
            _, line = executor._cacheline(rec["comp_sg"], rec["skeletons"], {})
            st = steps_c[rec["k"]]
            st.handle = line.handle
            st.n_tensors = line.n
            st.grid_dim = rec["comp_sg"].grid_dim
            slots_of: dict[int, list[int]] = {}
            for slot, arg in enumerate(line.indices):      # descriptor slot -> argument (skeleton) index
                slots_of.setdefault(arg, []).append(slot)
            rec["slots_of"] = slots_of
        state["ctx"], state["device"] = ctx, device

    torch_empty = torch.empty
    current_stream = torch.cuda.current_stream
    run_plan = lib.gint_execute_plan
    run_gathered = lib.gint_execute_gathered

    def _gather_layout_ok(rec) -> bool:
        """Static half of the folding condition: every descriptor slot that reads g maps logical program b to row b -- one
        batch dimension, one tile per logical program -- so that replacing b by idx[b] reads row idx[b] of the table."""
        g_idx = rec["gather"][0]
        skel = next(skel_idx for in_idx, skel_idx, _ in rec["ins"] if in_idx == g_idx)
        pd = rec["comp_sg"].get_program(*rec["skeletons"])
        indices = pd.input_indices if pd.input_indices is not None else list(range(len(pd.input_infos)))
        slots = [s_ for s_, a_ in enumerate(indices) if a_ == skel]
        if not slots:
            return False
        rows, stride = None, None
        for s_ in slots:
            info = pd.input_infos[s_]
            if len(info.batch_shape) != 1 or list(info.block_grid_dims) != [1, 1] or info.elm_size != 4:
                return False
            if rows not in (None, info.batch_shape[0]) or stride not in (None, info.batch_strides[0]):
                return False
            rows, stride = info.batch_shape[0], info.batch_strides[0]
        rec["gather_rows"], rec["gather_stride"], rec["gather_skel"] = rows, stride, skel
        return rows == rec["comp_sg"].grid_dim

    def _run_gathered(rec, results, args, stream_handle):
        g_idx, table_idx, index_idx = rec["gather"]
        table, index = results[table_idx], results[index_idx]
        if rec["gather_ok"] is None:
            rec["gather_ok"] = _gather_layout_ok(rec)
        ok = (rec["gather_ok"] and table.dim() == 2 and index.dim() == 1 and index.dtype == torch.int64 and table.dtype == torch.float32
              and table.is_contiguous() and index.is_contiguous() and index.numel() == rec["gather_rows"]
              and table.stride(0) == rec["gather_stride"] and table.numel() < 2 ** 31 and table.shape[0] > 0)
        if not ok:                        # run the gather as torch would have, then the subgraph as usual
            st = rec["gather_step"]
            results[g_idx] = st[2](*tuple(r(results) for r in st[3]))
        ref = table if rec["ref"] == g_idx and ok else (results[rec["ref"]] if rec["ref"] >= 0 else args[0])
        dtype, device = ref.dtype, ref.device
        c = steps_c[rec["k"]]
        ptrs, slots_of = c.base_ptrs, rec["slots_of"]
        for out_idx, skel_idx, shape in rec["outs"]:
            t = torch_empty(shape, dtype=dtype, device=device)
            results[out_idx] = t
            for s_ in slots_of.get(skel_idx, ()):
                ptrs[s_] = t.data_ptr()
        mask = 0
        for in_idx, skel_idx, off in rec["ins"]:
            if ok and in_idx == g_idx:
                p = table.data_ptr()
                for s_ in slots_of.get(skel_idx, ()):
                    mask |= 1 << s_
            else:
                p = results[in_idx].data_ptr() + off
            for s_ in slots_of.get(skel_idx, ()):
                ptrs[s_] = p
        if ok:
            rc = run_gathered(state["ctx"], c.handle, ptrs, c.n_tensors, c.grid_dim, mask, ctypes.c_void_p(index.data_ptr()), table.shape[0],
                              table.numel() * 4, stream_handle)
        else:
            rc = lib.gint_execute(state["ctx"], c.handle, ptrs, c.n_tensors, c.grid_dim, stream_handle)
        if rc != 0:
            executor._check(state["ctx"], rc, "gint_execute_gathered" if ok else "gint_execute")
        executor.launches += 1
        fast_execute.gathers_folded += 1 if ok else 0

    def fast_execute(*args):
        if state["ctx"] is None or state["device"] != torch.cuda.current_device():
            _prepare()
        results = [None] * results_size
        stream_handle = current_stream().cuda_stream
        for step in fast_plan:
            kind = step[0]
            if kind == KIND_RUN:
                first, recs = step[1], step[2]
                for rec in recs:
                    ref = results[rec["ref"]] if rec["ref"] >= 0 else args[0]
                    dtype, device = ref.dtype, ref.device
                    ptrs = steps_c[rec["k"]].base_ptrs
                    slots_of = rec["slots_of"]
                    for out_idx, skel_idx, shape in rec["outs"]:
                        t = torch_empty(shape, dtype=dtype, device=device)
                        results[out_idx] = t
                        p = t.data_ptr()
                        for s in slots_of.get(skel_idx, ()):
                            ptrs[s] = p
                    for in_idx, skel_idx, off in rec["ins"]:
                        p = results[in_idx].data_ptr() + off
                        for s in slots_of.get(skel_idx, ()):
                            ptrs[s] = p
                rc = run_plan(state["ctx"], step[3], len(recs), stream_handle)
                if rc != 0:
                    executor._check(state["ctx"], rc, "gint_execute_plan")
                executor.launches += len(recs)
            elif kind == KIND_GATHERED:
                _run_gathered(step[2], results, args, stream_handle)
            elif kind == STEP_PH:
                results[step[2]] = args[step[1]]
            elif kind == STEP_EAGER:
                target, arg_rs, kw_rs = step[2], step[3], step[4]
                results[step[1]] = target(*tuple(r(results) for r in arg_rs), **{k_: r(results) for k_, r in kw_rs})
            elif kind == STEP_GET_ATTR:
                results[step[1]] = step[2]
            elif kind == STEP_OUT_NODE:
                return results[step[1]]
            elif kind == STEP_OUT_CONST:
                return step[1]
            else:  # STEP_OUT_SEQ
                return tuple(results[v] if is_node else v for is_node, v in step[1])

    fast_execute.num_gint_subgraphs = getattr(execute, "num_gint_subgraphs", n_sg)
    fast_execute.original = execute
    fast_execute.plan_runs = sum(1 for s in fast_plan if s[0] == KIND_RUN)
    fast_execute.foldable_gathers = len(gathers)
    fast_execute.gathers_folded = 0
    return fast_execute


ACCELERATED: list = []     # every closure `patch_conductor` has replaced so far (newest last), for inspection and tests


def patch_conductor(executor: B200Executor) -> bool:
    """Wrap ``gint.conductor.compiler.GintCompiler.compile`` so that every graph compiled from now on runs through
    ``accelerate``. Returns False when the conductor cannot be imported."""
    try:
        import gint.conductor.compiler as cc
    except Exception:
        return False
    if getattr(cc.GintCompiler.compile, "_gint_b200_wrapped", False):
        return True
    original = cc.GintCompiler.compile

    def compile_and_accelerate(self, *a, **kw):
        fast = accelerate(original(self, *a, **kw), executor)
        ACCELERATED.append(fast)
        return fast

    compile_and_accelerate._gint_b200_wrapped = True
    compile_and_accelerate._gint_b200_original = original
    cc.GintCompiler.compile = compile_and_accelerate
    return True


def unpatch_conductor() -> None:
    import sys
    cc = sys.modules.get("gint.conductor.compiler")
    if cc is not None and getattr(cc.GintCompiler.compile, "_gint_b200_wrapped", False):
        cc.GintCompiler.compile = cc.GintCompiler.compile._gint_b200_original
