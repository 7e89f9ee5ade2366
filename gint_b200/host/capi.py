"""ctypes binding of libgint_b200.so (declared in include/gint_b200.h).

The library is built in-tree by ``python -m gint_b200.build``. There is no CPU fallback: if the library is
missing or no sm_100 device is usable the calls raise.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_char_p, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p

MAX_N_TENSORS = 8

LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "libgint_b200.so")


class GintError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, status: int, message: str):
        super().__init__(f"gint_b200: {message} (status {status})")
        self.status = status


class HTensorInfo(ctypes.Structure):
    """608-byte descriptor block; same layout as the reference's ``gint/kernel/interpreter/structs.py:19-30``."""
    _fields_ = [
        ("base_ptr", c_int64 * MAX_N_TENSORS),
        ("elm_size", c_int32 * MAX_N_TENSORS),
        ("batch_strides", (c_int32 * 4) * MAX_N_TENSORS),
        ("batch_shape", (c_int32 * 4) * MAX_N_TENSORS),
        ("block_shape_stride_1", (c_int32 * 2) * MAX_N_TENSORS),
        ("block_shape_stride_2", (c_int32 * 2) * MAX_N_TENSORS),
        ("block_grid_dims", (c_int32 * 2) * MAX_N_TENSORS),
        ("block_grid_steps", (c_int32 * 2) * MAX_N_TENSORS),
    ]


class BytecodeStatsC(ctypes.Structure):
    _fields_ = [(n, c_int32) for n in ("num_instructions", "max_stack", "max_reg_idx", "min_pool_size", "regs_used_mask",
                                       "error_index", "pool_size", "reserved")]


class LaunchInfoC(ctypes.Structure):
    _fields_ = [(n, c_int32) for n in ("pool_size", "tiles_per_warp", "warps_per_block", "grid_blocks", "smem_bytes",
                                       "regs_per_thread", "blocks_per_sm", "num_sms", "early_loads", "registers_in_smem", "vector_layout")] + \
               [("reserved", c_int32 * 5)]


GINT_OK = 0
GINT_ERR_INVALID_ARGUMENT = -1
GINT_ERR_UNKNOWN_OPCODE = -2
GINT_ERR_STACK_UNDERFLOW = -3
GINT_ERR_STACK_OVERFLOW = -4
GINT_ERR_NO_HALT = -5
GINT_ERR_BAD_HANDLE = -6
GINT_ERR_ARG_COUNT = -7
GINT_ERR_CUDA = -8
GINT_ERR_NO_DEVICE = -9
GINT_ERR_TOO_LARGE = -10
GINT_ERR_OUT_OF_MEMORY = -11

class DeviceStatusC(ctypes.Structure):
    """gint_device_status"""
    _fields_ = [("code", c_int32), ("slot", c_int32), ("logical_program", c_uint32), ("instruction", c_uint32), ("address", c_uint64),
                ("lane", c_uint32), ("count", c_uint32)]


DEVICE_CODES = {0: "ok", 1: "load out of range", 2: "store out of range", 3: "instruction budget exhausted", 4: "bad dispatch"}


class PlanStepC(ctypes.Structure):
    """gint_plan_step"""
    _fields_ = [("handle", c_uint64), ("base_ptrs", c_uint64 * 8), ("n_tensors", c_int32), ("grid_dim", c_uint32)]


# every symbol include/gint_b200.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "gint_version": (c_int, []),
    "gint_status_string": (c_char_p, [c_int]),
    "gint_sizeof_tensor_info": (c_int, []),
    "gint_analyze": (c_int, [POINTER(c_int32), c_int, POINTER(BytecodeStatsC)]),
    "gint_predecode": (c_int, [POINTER(c_int32), c_int, POINTER(c_uint32), c_int]),
    "gint_debug_transform": (c_int, [POINTER(c_int32), c_int, POINTER(HTensorInfo), c_int, c_int, c_int, POINTER(c_int32), POINTER(c_uint32), c_int]),
    "gint_debug_fused_table": (c_int, [POINTER(c_int32), c_int]),
    "gint_create": (c_int, [c_int, POINTER(c_void_p)]),
    "gint_destroy": (None, [c_void_p]),
    "gint_last_error": (c_char_p, [c_void_p]),
    "gint_program_create": (c_int, [c_void_p, POINTER(c_int32), c_int, POINTER(HTensorInfo), c_int, POINTER(c_uint64)]),
    "gint_program_destroy": (c_int, [c_void_p, c_uint64]),
    "gint_program_launch_info": (c_int, [c_void_p, c_uint64, c_uint32, POINTER(LaunchInfoC)]),
    "gint_execute": (c_int, [c_void_p, c_uint64, POINTER(c_uint64), c_int, c_uint32, c_void_p]),
    "gint_execute_range": (c_int, [c_void_p, c_uint64, POINTER(c_uint64), c_int, c_uint32, c_uint32, c_void_p]),
    "gint_execute_plan": (c_int, [c_void_p, POINTER(PlanStepC), c_int, c_void_p]),
    "gint_execute_gathered": (c_int, [c_void_p, c_uint64, POINTER(c_uint64), c_int, c_uint32, c_uint32, c_void_p, c_uint32, c_uint64, c_void_p]),
    "gint_execute_batch": (c_int, [c_void_p, POINTER(c_int32), c_int, c_int, POINTER(HTensorInfo), c_int, POINTER(c_uint64), c_int, c_uint64, POINTER(c_int32), c_void_p]),
    "gint_execute_checked": (c_int, [c_void_p, c_uint64, POINTER(c_uint64), POINTER(c_uint64), POINTER(c_uint64), c_int, c_uint32, c_void_p]),
    "gint_device_status_read": (c_int, [c_void_p, POINTER(DeviceStatusC), c_int]),
    "gint_execute_indirect": (c_int, [c_void_p, POINTER(c_uint64), c_int, POINTER(c_uint64), POINTER(c_int32), c_uint32, c_void_p]),
    "gint_execute_indirect_static": (c_int, [c_void_p, POINTER(c_uint64), c_int, POINTER(c_uint64), POINTER(c_int32), c_uint32, c_void_p]),
    "gint_set_option": (c_int, [c_void_p, c_char_p, c_int]),
}

_lib = None


def load_library(path: str | None = None) -> ctypes.CDLL:
    """Load libgint_b200.so and set the prototypes. Raises if the library has not been built."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise GintError(GINT_ERR_NO_DEVICE, f"{p} not found: build it with `python -m gint_b200.build`")
    lib = ctypes.CDLL(p)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    if lib.gint_sizeof_tensor_info() != ctypes.sizeof(HTensorInfo):
        raise GintError(GINT_ERR_INVALID_ARGUMENT, "descriptor struct layout mismatch between Python and the library")
    if path is None:
        _lib = lib
    return lib


def status_string(status: int) -> str:
    return load_library().gint_status_string(status).decode()
