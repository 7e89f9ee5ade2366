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
        ex.execute_indirect(progs, got, indices, static_tables=True)
        torch.cuda.synchronize()
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


def test_static_indirect_allocates_no_device_memory():
    """Free device memory as the DRIVER reports it (cudaMemGetInfo; torch's own counters only see torch's allocator) does not
    move across static launches, not even when the batch grows from the smallest to the largest the entry point takes -- the
    point at which scratch that is grown on demand would have to allocate. A first, small call comes before the measurement:
    it loads the kernel and resolves the array's address."""
    ex = get_executor()
    lib = capi.load_library()
    device = torch.cuda.current_device()
    ctx = ctypes.c_void_p()
    assert lib.gint_create(device, ctypes.byref(ctx)) == 0     # a context of its own: no indirect launch has grown its scratch
    try:
        n = 128
        a, b, c = torch.randn(n, device="cuda"), torch.randn(n, device="cuda"), torch.zeros(n, device="cuda")
        pd = C.vec_add_128.get_program(*[_convert_arg(t) for t in (a, b, c)])
        code = pd.program
        ti = capi.HTensorInfo()
        from gint_b200.host.utils import fill_tensor_info
        fill_tensor_info(ti, pd.input_infos)
        handle = ctypes.c_uint64()
        assert lib.gint_program_create(ctx, code.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), int(code.size), ctypes.byref(ti), 3,
                                       ctypes.byref(handle)) == 0

        def launch(n_programs: int, grid: int):
            handles = (ctypes.c_uint64 * n_programs)(*([handle.value] * n_programs))
            ptrs = (ctypes.c_uint64 * (n_programs * capi.MAX_N_TENSORS))()
            for p in range(n_programs):
                ptrs[p * capi.MAX_N_TENSORS + 0], ptrs[p * capi.MAX_N_TENSORS + 1], ptrs[p * capi.MAX_N_TENSORS + 2] = a.data_ptr(), b.data_ptr(), c.data_ptr()
            idx = (ctypes.c_int32 * grid)(*[i % n_programs for i in range(grid)])
            assert lib.gint_execute_indirect_static(ctx, handles, n_programs, ptrs, idx, grid, None) == 0, lib.gint_last_error(ctx)

        launch(1, 1)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info(device)
        launch(64, 4096)                                         # every logical program writes the same values to the same place
        launch(3, 17)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info(device)
        assert free_after == free_before, f"driver-reported free memory moved by {free_before - free_after} bytes"
        torch.testing.assert_close(c, a + b)
    finally:
        torch.cuda.synchronize()
        lib.gint_destroy(ctx)


def test_static_indirect_refuses_a_capturing_stream():
    """The tables are uploaded from a host image that the next call overwrites, so the launch cannot be part of a graph: on a
    stream that is being captured both indirect entry points return an error and queue nothing (the capture stays valid)."""
    ex = get_executor()
    lib = capi.load_library()
    _, ctx = ex._ctx()
    n = 128
    a, b, out = torch.randn(n, device="cuda"), torch.randn(n, device="cuda"), torch.zeros(n, device="cuda")
    _, line = ex._cacheline(C.vec_add_128, [_convert_arg(t) for t in (a, b, out)], {})
    handles = (ctypes.c_uint64 * 1)(line.handle)
    idx = (ctypes.c_int32 * 1)(0)
    ptrs = (ctypes.c_uint64 * capi.MAX_N_TENSORS)(a.data_ptr(), b.data_ptr(), out.data_ptr())
    assert lib.gint_execute_indirect_static(ctx, handles, 1, ptrs, idx, 1, None) == 0      # set-up happens outside any capture
    torch.cuda.synchronize()
    out.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        rc_static = lib.gint_execute_indirect_static(ctx, handles, 1, ptrs, idx, 1, stream)
        msg_static = lib.gint_last_error(ctx).decode()
        rc_plain = lib.gint_execute_indirect(ctx, handles, 1, ptrs, idx, 1, stream)
        out.add_(1.0)                                            # so that the captured graph is not empty
    assert rc_static == capi.GINT_ERR_INVALID_ARGUMENT and "captured" in msg_static
    assert rc_plain == capi.GINT_ERR_INVALID_ARGUMENT
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, torch.ones(n, device="cuda"))       # only the torch op was captured


_FIRST_CALL_FROM_TWO_THREADS = r"""
import ctypes, sys, threading
import torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {tests!r})
import cases as C
from gint_b200 import get_executor
from gint_b200.host import capi
from gint_b200.host.executor import _convert_arg
ex = get_executor(); lib = capi.load_library(); _, ctx = ex._ctx()
n = 128
sets = []
for t in range(2):
    g = torch.Generator().manual_seed(t)
    a, b = torch.randn(n, generator=g).cuda(), torch.randn(n, generator=g).cuda()
    sets.append((a, b, torch.zeros(n, device="cuda")))
prog = [C.vec_add_128, C.vec_mul_128]
lines = [ex._cacheline(prog[t], [_convert_arg(x) for x in sets[t]], {{}})[1] for t in range(2)]
torch.cuda.synchronize()
gate = threading.Barrier(2); rcs = [None, None]
def work(t):
    handles = (ctypes.c_uint64 * 1)(lines[t].handle); idx = (ctypes.c_int32 * 1)(0)
    ptrs = (ctypes.c_uint64 * capi.MAX_N_TENSORS)(*[x.data_ptr() for x in sets[t]])
    gate.wait()
    # the same (default) stream in both threads: the launches are ordered on the GPU, only the host side is concurrent
    rcs[t] = lib.gint_execute_indirect_static(ctx, handles, 1, ptrs, idx, 1, None)
th = [threading.Thread(target=work, args=(t,)) for t in range(2)]
[t.start() for t in th]; [t.join() for t in th]
torch.cuda.synchronize()
assert rcs == [0, 0], rcs
assert torch.equal(sets[0][2], sets[0][0] + sets[0][1]) and torch.equal(sets[1][2], sets[1][0] * sets[1][1])
print("ok")
"""


def test_static_indirect_first_call_from_two_threads():
    """In a fresh process the very first static launch comes from two threads at once: the one-time set-up runs under the
    library's lock, so both launches see a complete set-up and neither disturbs the other's tables."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = _FIRST_CALL_FROM_TWO_THREADS.format(root=root, tests=os.path.join(root, "tests"))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout[-2000:] + r.stderr[-4000:]
