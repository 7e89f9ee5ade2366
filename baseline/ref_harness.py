"""Run recorded bytecode programs through the UNMODIFIED reference executor and kernels installed under ``baseline/_ref``.

Used by the GPU parity tests and by ``bench.py`` to put the reference's own ``geval_s7`` / ``geval_l12`` (built for sm_100 by
``baseline/build_ref.py``) beside this repository's kernels on the same buffers. Nothing under ``gint_b200/`` imports this.

The reference package is imported from ``baseline/_ref`` only; when that folder is absent ``available()`` is False and callers
skip. The reference executor is ``gint.host.cuda.executor_impl.CudaExecutor`` exactly as shipped: per-call 608-byte descriptor
upload, ``cuLaunchKernel`` of its fatbin's kernel with its own warps-per-block heuristic (``executor_impl.py:51-74``).
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")

_state: dict = {}


def available() -> bool:
    return os.path.exists(os.path.join(REF_DIR, "gint", "host", "cuda", "gint.fatbin.xz"))


def why_unavailable() -> str:
    if not os.path.isdir(os.path.join(REF_DIR, "gint")):
        return "baseline/_ref is absent (run baseline/build_ref.py where the reference checkout is)"
    if not available():
        return "baseline/_ref/gint/host/cuda/gint.fatbin.xz is absent (baseline/build_ref.py did not finish)"
    return ""


def import_reference():
    """The reference's ``gint`` package (from ``baseline/_ref``)."""
    if "gint" not in _state:
        if REF_DIR not in sys.path:
            sys.path.insert(0, REF_DIR)
        import gint  # noqa: F401
        import gint.host.executor as gx
        if not os.path.abspath(gx.__file__).startswith(REF_DIR):
            raise RuntimeError(f"another gint package is imported from {gx.__file__}")
        _state["gint"] = gint
        _state["gx"] = gx
    return _state["gint"]


def reference_executor():
    """A fresh-once ``CudaExecutor`` of the reference (not installed into its global: callers pass it around)."""
    if "executor" not in _state:
        import_reference()
        from gint.host.cuda.executor_impl import CudaExecutor
        _state["executor"] = CudaExecutor()
    return _state["executor"]


def as_reference_program(recorded):
    """Wrap a ``gint_b200.programs.RecordedProgram`` (bytecode + descriptors) as a reference ``BaseExecutableProgram``."""
    import_reference()
    gx = _state["gx"]
    cache = _state.setdefault("programs", {})
    key = id(recorded)
    if key not in cache:
        infos = [gx.ProgramTensorInfo(**vars(t)) for t in recorded.tensor_infos]
        pd = gx.ProgramData(recorded.bytecode.copy(), infos, list(recorded.input_indices))

        class _Fixed(gx.BaseExecutableProgram):
            def get_program(self, *args, **kw):
                return pd

            def cache_policy(self, *args, **kw):
                return None

        cache[key] = (_Fixed(), recorded)     # keep `recorded` alive so its id stays unique
    return cache[key][0]


def wrap_program_data(program, infos, input_indices=None):
    """A reference ``BaseExecutableProgram`` for an int32 stream and descriptor records (objects with ProgramTensorInfo's fields)."""
    import numpy
    import_reference()
    gx = _state["gx"]
    ref_infos = [gx.ProgramTensorInfo(**{k: getattr(t, k) for k in ("elm_size", "batch_strides", "batch_shape", "block_shape_stride_1",
                                                                   "block_shape_stride_2", "block_grid_dims", "block_grid_steps")}) for t in infos]
    pd = gx.ProgramData(numpy.ascontiguousarray(numpy.asarray(program, dtype=numpy.int32).reshape(-1)), ref_infos,
                        list(input_indices) if input_indices is not None else None)

    class _Fixed(gx.BaseExecutableProgram):
        def get_program(self, *args, **kw):
            return pd

        def cache_policy(self, *args, **kw):
            return None

    return _Fixed()


def execute(program, tensors, grid_dim: int, stream: int = 0) -> None:
    """``CudaExecutor.execute`` of the reference on torch tensors."""
    gx = _state.get("gx") or (import_reference() and _state["gx"])
    reference_executor().execute(program, [gx._convert_arg(t) for t in tensors], grid_dim, cuda_stream=stream)


def run_workload(wl, stream: int = 0) -> int:
    """One pass of a ``gint_b200.workloads.Workload`` through the reference executor; returns the launches issued."""
    gx = _state.get("gx") or (import_reference() and _state["gx"])
    ex = reference_executor()
    if wl.pre is not None:
        wl.pre(wl.tensors)
    for st in wl.steps:
        ex.execute(as_reference_program(st.program), [gx._convert_arg(wl.tensors[r]) for r in st.roles], st.grid_dim, cuda_stream=stream)
    return len(wl.steps)


def variant_of(recorded) -> str:
    import_reference()
    return _state["gx"].select_variant(as_reference_program(recorded).get_program())
