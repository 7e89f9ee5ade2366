"""Guards against silent performance regressions of the five named programs at their full sizes.

Two kinds of check. (1) The launch geometry each program gets -- pool size, tiles per warp, whether its virtual registers live in
shared memory, how many loads are issued early -- is deterministic and is what the measured numbers depend on: a change to the
pre-decoder or to the tiles-per-warp rules that silently sends a program down another path shows up here. (2) The achieved
bandwidth, with CUDA events, must stay above a floor set a quarter below what this build measures on a B200 (1965 MHz, no
throttling): loose enough for another board of the same kind, tight enough to catch a fall back to the untransformed stream or
to the wrong kernel (the 4x4 inverse on the 12-slot pool kernel runs at 0.97 TB/s, below its floor).
"""
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from gint_b200 import get_executor  # noqa: E402
from gint_b200.workloads import FULL_SIZES, make_workload  # noqa: E402

pytestmark = pytest.mark.gpu

# program -> (pool size, tiles per warp, registers in shared memory, early loads of the first step, floor in GB/s of algorithmic bytes)
EXPECTED = {
    "rmsnorm": (4, 1, 0, 96, 3650.0),
    "bmm4x4": (7, 2, 0, 0, 3700.0),
    "inv4x4": (7, 2, 8, 0, 1300.0),
    "graph": (4, 2, 0, 32, 3500.0),
    "graph_gathered": (4, 2, 0, 32, 3400.0),
}


def _time_us(wl, ex, stream, n=10):
    for _ in range(3):
        wl.run(ex, stream)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(n):
        wl.run(ex, stream)
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / n


@pytest.mark.parametrize("name", list(EXPECTED))
def test_named_program_keeps_its_geometry_and_its_speed(name):
    pool, k, smem_regs, early, floor = EXPECTED[name]
    ex = get_executor()
    wl = make_workload(name, *FULL_SIZES[name], device="cuda")
    st = wl.steps[0]
    info = ex.launch_info(st.program, [wl.tensors[r] for r in st.roles], st.grid_dim)
    assert (info["pool_size"], info["tiles_per_warp"], info["registers_in_smem"], info["early_loads"]) == (pool, k, smem_regs, early), info
    us = _time_us(wl, ex, torch.cuda.current_stream().cuda_stream)
    gbs = wl.algorithmic_bytes / us / 1e3
    assert gbs >= floor, f"{name}: {us:.1f} us per pass = {gbs:.0f} GB/s, below the floor of {floor:.0f} GB/s"


def test_small_add_stays_a_single_short_launch():
    """a+b over 2^20 elements: four tiles per warp (a latency-bound launch), the program inside the kernel parameters, and at most
    12 us per launch through the executor with 22 rotating buffer sets (measured: 7.5 us, of which 5.5 on the device)."""
    ex = get_executor()
    wls = [make_workload("add", *FULL_SIZES["add"], device="cuda", seed=i) for i in range(22)]
    st = wls[0].steps[0]
    info = ex.launch_info(st.program, [wls[0].tensors[r] for r in st.roles], st.grid_dim)
    assert (info["pool_size"], info["tiles_per_warp"]) == (4, 4), info
    s = torch.cuda.current_stream().cuda_stream
    for w in wls:
        w.run(ex, s)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        for w in wls:
            w.run(ex, s)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / (10 * len(wls))
    assert us <= 12.0, f"a+b: {us:.1f} us per launch"
