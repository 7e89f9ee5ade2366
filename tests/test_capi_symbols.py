"""The C-ABI shared library loads without a GPU and exports every symbol include/gint_b200.h declares; its
host-only entry points (analysis, pre-decode, status strings) behave as documented. No compute calls here."""
import ctypes
import os
import re

import numpy as np
import pytest

from gint_b200.host import capi
from gint_b200 import opcodes as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "gint_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gint_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound():
    lib = capi.load_library()
    declared = _declared_symbols()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/gint_b200.h but not exported"
    assert sorted(capi.SIGNATURES) == declared, "ctypes binding and header disagree"


def test_struct_layout():
    lib = capi.load_library()
    assert lib.gint_sizeof_tensor_info() == ctypes.sizeof(capi.HTensorInfo) == 608
    off = {n: getattr(capi.HTensorInfo, n).offset for n, _ in capi.HTensorInfo._fields_}
    assert off == dict(base_ptr=0, elm_size=64, batch_strides=96, batch_shape=224, block_shape_stride_1=352,
                       block_shape_stride_2=416, block_grid_dims=480, block_grid_steps=544)
    assert lib.gint_version() >= 100


def test_status_strings():
    lib = capi.load_library()
    assert lib.gint_status_string(0) == b"ok"
    for code in range(-11, 0):
        assert lib.gint_status_string(code) not in (b"", b"unknown status")
    assert lib.gint_status_string(-999) == b"unknown status"


def _analyze(pairs):
    lib = capi.load_library()
    code = np.array(pairs, dtype=np.int32).reshape(-1)
    st = capi.BytecodeStatsC()
    rc = lib.gint_analyze(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), code.size, ctypes.byref(st))
    return rc, st


def test_analyze_error_codes():
    assert _analyze([[O.LoadImm, 0], [O.Halt, 0]])[0] == capi.GINT_OK
    rc, st = _analyze([[O.LoadImm, 0], [999, 0], [O.Halt, 0]])
    assert rc == capi.GINT_ERR_UNKNOWN_OPCODE and st.error_index == 1
    rc, st = _analyze([[O.LoadImm, 0], [O.FAdd, 0], [O.Halt, 0]])
    assert rc == capi.GINT_ERR_STACK_UNDERFLOW and st.error_index == 1
    rc, st = _analyze([[O.LoadImm, 0]] * 9 + [[O.Halt, 0]])
    assert rc == capi.GINT_ERR_STACK_OVERFLOW and st.error_index == 8
    assert _analyze([[O.LoadImm, 0], [O.Pop, 0]])[0] == capi.GINT_ERR_NO_HALT
    lib = capi.load_library()
    assert lib.gint_analyze(None, 0, None) == capi.GINT_ERR_INVALID_ARGUMENT
    code = np.zeros(3, dtype=np.int32)
    st = capi.BytecodeStatsC()
    assert lib.gint_analyze(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), 3, ctypes.byref(st)) == capi.GINT_ERR_INVALID_ARGUMENT


def test_predecode_keys_carry_the_stack_depth():
    lib = capi.load_library()
    prog = [[O.LoadImm, 0], [O.Dup, 0], [O.FAdd, 0], [O.FStoreReg0, 0], [O.FLoadReg0, 0], [O.Pop, 0], [O.Halt, 0]]
    code = np.array(prog, dtype=np.int32).reshape(-1)
    keys = (ctypes.c_uint32 * 16)()
    n = lib.gint_predecode(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), code.size, keys, 16)
    assert n == 7
    depth_before = [0, 1, 2, 1, 0, 1, 0]
    assert list(keys[:n]) == [d * O.N_OPCODES + op for d, (op, _) in zip(depth_before, prog)]
    # too small an output buffer
    assert lib.gint_predecode(code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), code.size, keys, 3) == capi.GINT_ERR_INVALID_ARGUMENT


def test_context_creation_fails_loudly_without_a_device():
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    lib = capi.load_library()
    out = ctypes.c_void_p()
    assert lib.gint_create(0, ctypes.byref(out)) == capi.GINT_ERR_NO_DEVICE
    assert not out.value
    from gint_b200.host.executor import B200Executor
    from gint_b200 import TensorInterface
    import cases
    ex = B200Executor()
    t = TensorInterface("f", 4, 0, (128,), (1,))
    with pytest.raises(Exception):
        ex.execute(cases.VectorAddProgram(), [t, t, t], 1)
