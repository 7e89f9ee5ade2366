"""The allocation-free indirect launch (gint_execute_indirect_static) gives the same bits as gint_execute_indirect.

Some callers may not allocate device memory at the moment they launch (all device memory belongs to another allocator,
a deadline rules out the stall an allocation can cause, or the permitted driver calls are restricted). For them the
library keeps the per-launch tables of an indirect launch in a fixed array of its own. This file is collected last on
purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

import cases as C
from conftest import bits_equal, mismatch_report
from gint_b200 import get_executor
from gint_b200.host import capi
from gint_b200.host.executor import _convert_arg

pytestmark = pytest.mark.gpu


def _inputs(seed: int, n: int):
    g = torch.Generator().manual_seed(seed)
    return [[torch.randn(n, generator=g).cuda(), torch.randn(n, generator=g).cuda(), torch.zeros(n).cuda()] for _ in range(2)]


def test_static_indirect_matches_indirect_twice_in_a_row():
    ex = get_executor()
    n = 128 * 6
    tiles = n // 128
    indices = [0] * tiles + [1] * tiles + [0] * 3          # program 0 over its tiles, program 1 over its tiles, a few repeats
    progs = [C.vec_add_128, C.vec_mul_128]
    for call in range(2):                                  # two calls in a row share the static array
        ref = _inputs(100 + call, n)
        got = _inputs(100 + call, n)
        ex.execute_indirect(progs, ref, indices)
        before = torch.cuda.memory_allocated()
        ex.execute_indirect(progs, got, indices, static_tables=True)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        for p in range(2):
            assert bits_equal(got[p][2], ref[p][2]), f"call {call}, program {p}: " + mismatch_report(got[p][2], ref[p][2])
        torch.testing.assert_close(got[0][2], got[0][0] + got[0][1])
        torch.testing.assert_close(got[1][2], got[1][0] * got[1][1])


def test_static_indirect_rejects_oversized_batches():
    ex = get_executor()
    a, b, c = (torch.zeros(128, device="cuda") for _ in range(3))
    with pytest.raises(capi.GintError) as e1:
        ex.execute_indirect([C.vec_add_128], [(a, b, c)], [0] * 4097, static_tables=True)
    assert e1.value.status == capi.GINT_ERR_TOO_LARGE and "4096" in str(e1.value)
    with pytest.raises(capi.GintError) as e2:
        ex.execute_indirect([C.vec_add_128] * 65, [(a, b, c)] * 65, [0], static_tables=True)
    assert e2.value.status == capi.GINT_ERR_TOO_LARGE and "64" in str(e2.value)
    torch.cuda.synchronize()
    assert torch.equal(c, torch.zeros(128, device="cuda"))     # nothing was launched


def test_static_indirect_through_the_raw_c_abi():
    """Same check with the handles and pointer arrays built by hand, as a non-Python caller would."""
    ex = get_executor()
    lib = capi.load_library()
    _, ctx = ex._ctx()
    n = 128
    g = torch.Generator().manual_seed(7)
    a, b = torch.randn(n, generator=g).cuda(), torch.randn(n, generator=g).cuda()
    out_ref, out_new = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    _, line = ex._cacheline(C.vec_mul_128, [_convert_arg(t) for t in (a, b, out_ref)], {})
    handles = (ctypes.c_uint64 * 1)(line.handle)
    idx = (ctypes.c_int32 * 1)(0)
    for out, fn in ((out_ref, lib.gint_execute_indirect), (out_new, lib.gint_execute_indirect_static)):
        ptrs = (ctypes.c_uint64 * capi.MAX_N_TENSORS)(a.data_ptr(), b.data_ptr(), out.data_ptr())
        assert fn(ctx, handles, 1, ptrs, idx, 1, None) == 0, lib.gint_last_error(ctx)
    torch.cuda.synchronize()
    assert bits_equal(out_new, out_ref)
    torch.testing.assert_close(out_new, a * b)
