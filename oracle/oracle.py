"""ctypes loader for the CPU oracle (oracle/gint_oracle.c). TEST INFRASTRUCTURE ONLY.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg import this module; the product package
(gint_b200/) never does. The oracle executes bytecode on HOST memory (numpy / CPU torch tensors).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy

HERE = os.path.dirname(os.path.abspath(__file__))
LIB = os.path.join(HERE, "libgint_oracle.so")

MAX_N_TENSORS = 8


class OracleTensorInfo(ctypes.Structure):
    _fields_ = [
        ("base_ptr", ctypes.c_int64 * MAX_N_TENSORS),
        ("elm_size", ctypes.c_int32 * MAX_N_TENSORS),
        ("batch_strides", (ctypes.c_int32 * 4) * MAX_N_TENSORS),
        ("batch_shape", (ctypes.c_int32 * 4) * MAX_N_TENSORS),
        ("block_shape_stride_1", (ctypes.c_int32 * 2) * MAX_N_TENSORS),
        ("block_shape_stride_2", (ctypes.c_int32 * 2) * MAX_N_TENSORS),
        ("block_grid_dims", (ctypes.c_int32 * 2) * MAX_N_TENSORS),
        ("block_grid_steps", (ctypes.c_int32 * 2) * MAX_N_TENSORS),
    ]


class OracleStats(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int32) for n in ("num_instructions", "max_stack", "max_reg_idx", "min_pool_size",
                                              "regs_used_mask", "error_index")]


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "gint_oracle.c")
    if force or not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(src):
        subprocess.run(["make", "-C", HERE, "-B" if force else "-s"], check=True, capture_output=True)
    return LIB


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(LIB)
        L.gint_oracle_analyze.restype = ctypes.c_int
        L.gint_oracle_analyze.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_int, ctypes.POINTER(OracleStats)]
        L.gint_oracle_pool_size.restype = ctypes.c_int
        L.gint_oracle_pool_size.argtypes = [ctypes.POINTER(OracleStats)]
        L.gint_oracle_execute.restype = ctypes.c_int
        L.gint_oracle_execute.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_int, ctypes.POINTER(OracleTensorInfo),
                                          ctypes.c_int, ctypes.c_uint32, ctypes.c_int, ctypes.c_int]
        L.gint_oracle_execute_range.restype = ctypes.c_int
        L.gint_oracle_execute_range.argtypes = [ctypes.POINTER(ctypes.c_int32), ctypes.c_int, ctypes.POINTER(OracleTensorInfo),
                                                ctypes.c_int, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_int, ctypes.c_int]
        L.gint_oracle_execute_indirect.restype = ctypes.c_int
        L.gint_oracle_execute_indirect.argtypes = [ctypes.POINTER(ctypes.POINTER(ctypes.c_int32)), ctypes.POINTER(ctypes.c_int32),
                                                   ctypes.POINTER(ctypes.POINTER(OracleTensorInfo)), ctypes.c_int,
                                                   ctypes.c_uint32, ctypes.c_int]
        L.gint_oracle_sizeof_tensor_info.restype = ctypes.c_int
        assert L.gint_oracle_sizeof_tensor_info() == ctypes.sizeof(OracleTensorInfo) == 608
        _lib = L
    return _lib


def _code(program) -> numpy.ndarray:
    return numpy.ascontiguousarray(numpy.asarray(program, dtype=numpy.int32).reshape(-1))


def _fill(ti: OracleTensorInfo, infos, ptrs) -> None:
    """Same packing rule as the product's fill_tensor_info, restated: batch dims reversed, padded (0, 1)
    (reference gint/host/utils.py:6-27)."""
    for s, t in enumerate(infos):
        get = (lambda k: t[k]) if isinstance(t, dict) else (lambda k: getattr(t, k))
        ti.base_ptr[s] = int(ptrs[s])
        ti.elm_size[s] = int(get("elm_size"))
        bs, bsh = list(get("batch_strides"))[::-1], list(get("batch_shape"))[::-1]
        for j in range(4):
            ti.batch_strides[s][j] = bs[j] if j < len(bs) else 0
            ti.batch_shape[s][j] = bsh[j] if j < len(bsh) else 1
        for f in ("block_shape_stride_1", "block_shape_stride_2", "block_grid_dims", "block_grid_steps"):
            v = get(f)
            getattr(ti, f)[s][0] = int(v[0])
            getattr(ti, f)[s][1] = int(v[1])


def analyze(program) -> dict:
    code = _code(program)
    st = OracleStats()
    rc = lib().gint_oracle_analyze(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(code.size), ctypes.byref(st))
    out = {n: getattr(st, n) for n, _ in OracleStats._fields_}
    out["status"] = rc
    out["pool_size"] = lib().gint_oracle_pool_size(ctypes.byref(st)) if rc == 0 else 0
    return out


def _host_ptr(t) -> int:
    if hasattr(t, "data_ptr"):
        assert t.device.type == "cpu", "the oracle runs on host memory"
        return t.data_ptr()
    return t.ctypes.data


def execute(program, infos, tensors, grid_dim: int, input_indices=None, pool_size: int = 0, threads: int = 1) -> None:
    """Run `grid_dim` logical programs on host tensors (CPU torch tensors or numpy arrays), in place.
    tensors[input_indices[i]] backs descriptor slot i."""
    code = _code(program)
    idx = list(range(len(infos))) if input_indices is None else list(input_indices)
    ti = OracleTensorInfo()
    _fill(ti, infos, [_host_ptr(tensors[i]) for i in idx])
    rc = lib().gint_oracle_execute(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(code.size), ctypes.byref(ti),
                                   len(infos), int(grid_dim), int(pool_size), int(threads))
    if rc != 0:
        raise RuntimeError(f"oracle: status {rc}")


def execute_range(program, infos, ptrs, first: int, count: int, pool_size: int = 0, threads: int = 1) -> None:
    """Run logical programs [first, first + count) with explicit base addresses (ints), e.g. biased shard pointers."""
    code = _code(program)
    ti = OracleTensorInfo()
    _fill(ti, infos, ptrs)
    rc = lib().gint_oracle_execute_range(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(code.size), ctypes.byref(ti),
                                         len(infos), int(first), int(count), int(pool_size), int(threads))
    if rc != 0:
        raise RuntimeError(f"oracle: status {rc}")


def execute_indirect(programs, infos_list, tensors_list, indices, input_indices_list=None) -> None:
    """Indirect mode: logical program i runs programs[indices[i]] on tensors_list[indices[i]]."""
    codes = [_code(p) for p in programs]
    tis = []
    for k, (infos, tensors) in enumerate(zip(infos_list, tensors_list)):
        idx = list(range(len(infos))) if not input_indices_list or input_indices_list[k] is None else list(input_indices_list[k])
        ti = OracleTensorInfo()
        _fill(ti, infos, [_host_ptr(tensors[i]) for i in idx])
        tis.append(ti)
    n = len(indices)
    code_ptrs = (ctypes.POINTER(ctypes.c_int32) * n)(*[codes[i].ctypes.data_as(ctypes.POINTER(ctypes.c_int32)) for i in indices])
    n_words = (ctypes.c_int32 * n)(*[int(codes[i].size) for i in indices])
    ti_ptrs = (ctypes.POINTER(OracleTensorInfo) * n)(*[ctypes.pointer(tis[i]) for i in indices])
    max_t = max(len(x) for x in infos_list)
    rc = lib().gint_oracle_execute_indirect(code_ptrs, n_words, ti_ptrs, max_t, n, 0)
    if rc != 0:
        raise RuntimeError(f"oracle: status {rc}")
