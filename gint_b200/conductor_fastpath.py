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
  so stream order is what the original loop produced).

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


def accelerate(execute: Callable, executor: B200Executor) -> Callable:
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
    KIND_RUN = 100
    k = 0
    for step in plan:
        if step[0] != STEP_SUBGRAPH:
            fast_plan.append(step)
            continue
        comp_sg, ti_skeletons, input_writes, output_writes, output_shapes, ref_idx = sg_dispatch[step[1]]
        rec = {"comp_sg": comp_sg, "skeletons": ti_skeletons, "k": k, "ref": ref_idx,
               "outs": [(out_idx, skel_idx, tuple(shape)) for (out_idx, skel_idx), shape in zip(output_writes, output_shapes)],
               "ins": [(in_idx, skel_idx, off) for in_idx, skel_idx, off in input_writes], "slots_of": None}
        lowered.append(rec)
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
    return fast_execute


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
        return accelerate(original(self, *a, **kw), executor)

    compile_and_accelerate._gint_b200_wrapped = True
    compile_and_accelerate._gint_b200_original = original
    cc.GintCompiler.compile = compile_and_accelerate
    return True


def unpatch_conductor() -> None:
    import sys
    cc = sys.modules.get("gint.conductor.compiler")
    if cc is not None and getattr(cc.GintCompiler.compile, "_gint_b200_wrapped", False):
        cc.GintCompiler.compile = cc.GintCompiler.compile._gint_b200_original
