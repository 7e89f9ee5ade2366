"""Executor-level behaviour on the GPU: the drop-in surface of gint.host (errors, caching, streams, CUDA-graph capture,
indirect dispatch, range launches for sharding)."""
import ctypes

import numpy as np
import pytest
import torch

import cases as C
from conftest import bits_equal, mismatch_report
from gint_b200 import ProgramData, ProgramTensorInfo, TensorInterface, bytecode, cdiv, get_executor
from gint_b200.host import capi
from gint_b200.host.executor import BaseExecutableProgram, _convert_arg
from gint_b200.host.frontend import *  # noqa: F401,F403
from gint_b200.programs import recorded
from oracle import oracle

pytestmark = pytest.mark.gpu


def test_wrong_argument_count_raises_value_error():
    # reference: gint/host/cuda/executor_impl.py:93-94
    a = torch.zeros(256, device="cuda")
    with pytest.raises(ValueError, match="Number of arguments"):
        get_executor().execute(recorded("add_n4096"), [_convert_arg(a)] * 2, 1)


def test_invalid_programs_raise_before_any_launch():
    class Bad(BaseExecutableProgram):
        def __init__(self, bc):
            self.bc = bc

        def get_program(self, *args):
            return ProgramData(np.array(self.bc, dtype=np.int32).reshape(-1),
                               [ProgramTensorInfo(4, [], [], [128, 1], [1, 0], [1, 1], [0, 0])])
    x = torch.zeros(128, device="cuda")
    with pytest.raises(ValueError, match="unknown opcode"):
        Bad([[200, 0], [0, 0]])(x, grid_dim=1)
    with pytest.raises(ValueError, match="needs depth"):
        Bad([[FAdd, 0], [0, 0]])(x, grid_dim=1)
    with pytest.raises(ValueError):                      # deeper than any kernel geometry
        Bad([[LoadImm, 0]] * 9 + [[0, 0]])(x, grid_dim=1)
    with pytest.raises(Exception):                       # tensor slot 3 of a 1-tensor program
        Bad([[LoadGlobal1DF32, 3], [Pop, 0], [0, 0]])(x, grid_dim=1)
    torch.cuda.synchronize()
    assert torch.equal(x, torch.zeros(128, device="cuda"))


def test_program_is_built_once_per_cache_key():
    prog = C.VectorAddProgram()
    calls = []
    orig = prog.get_program
    prog.get_program = lambda *a, **k: (calls.append(1), orig(*a, **k))[1]
    a, b, c = (torch.randn(1000, device="cuda") for _ in range(3))
    for _ in range(3):
        prog(a, b, c, grid_dim=cdiv(1000, 256))
    a2, b2, c2 = (torch.randn(500, device="cuda") for _ in range(3))
    prog(a2, b2, c2, grid_dim=cdiv(500, 256))
    torch.cuda.synchronize()
    assert len(calls) == 2                               # one per shape, as with program._cu in the reference
    torch.testing.assert_close(c, a + b)
    torch.testing.assert_close(c2, a2 + b2)


def test_launch_on_a_side_stream_is_ordered_with_it():
    s = torch.cuda.Stream()
    a, b = torch.randn(1 << 20, device="cuda"), torch.randn(1 << 20, device="cuda")
    c = torch.zeros(1 << 20, device="cuda")
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        a2 = a * 2                                        # producer on s
        C.VectorAddProgram()(a2, b, c, grid_dim=cdiv(1 << 20, 256), cuda_stream=s.cuda_stream)
        out = c + 1                                       # consumer on s
    s.synchronize()
    torch.testing.assert_close(out, a * 2 + b + 1)


def test_cuda_graph_capture_and_replay():
    """Mirror of the reference's tests/test_cuda_graph_capture.py:31-65."""
    def cubic_ease(x):
        shape = x.shape
        x = x.view(-1)
        y = torch.empty_like(x)
        C.vector_expr2(x, y, grid_dim=cdiv(len(x), 256), BLOCK=256, cuda_stream=torch.cuda.current_stream().cuda_stream)
        return (x ** 2 * (3 - 2 * x)).view(shape), y.view(shape)

    torch.manual_seed(42)
    x1 = torch.rand(12938, 3, device="cuda")
    x2 = torch.rand(12938, 3, device="cuda")
    graphed = torch.cuda.make_graphed_callables(cubic_ease, (x2,))
    r1, y1 = graphed(x1)
    r1, y1 = r1.clone(), y1.clone()
    r2, y2 = graphed(x2)
    torch.testing.assert_close(y1, x1 ** 2 * (3 - 2 * x1))
    torch.testing.assert_close(y2, x2 ** 2 * (3 - 2 * x2))
    torch.testing.assert_close(r2, x2 ** 2 * (3 - 2 * x2))
    # an eager call in between must not disturb what the graph captured (descriptors are kernel parameters)
    _, ye = cubic_ease(torch.rand(12938, 3, device="cuda"))
    _, y1b = graphed(x1)
    torch.testing.assert_close(y1b, x1 ** 2 * (3 - 2 * x1))


def test_manual_graph_capture_allocates_nothing():
    a, b, c = (torch.randn(4096, device="cuda") for _ in range(3))
    prog = recorded("add_n4096")
    args = [_convert_arg(t) for t in (c, a, b)]           # roles: out, a, b
    ex = get_executor()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        ex.execute(prog, args, prog.grid_dim, cuda_stream=s.cuda_stream)   # warm-up: builds the program
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    before = torch.cuda.memory_allocated()
    with torch.cuda.graph(g, stream=s):
        ex.execute(prog, args, prog.grid_dim, cuda_stream=torch.cuda.current_stream().cuda_stream)
    assert torch.cuda.memory_allocated() == before
    c.zero_()
    a.copy_(torch.arange(4096.0, device="cuda"))
    g.replay()
    torch.cuda.synchronize()
    assert torch.equal(c, a + b)


def test_indirect_dispatch_two_programs_one_launch():
    """Mirror of the reference's tests/test_indirect.py:34-62, plus a bit-exact check against the oracle's indirect mode."""
    ex = get_executor()
    N = 128 * 5
    g = torch.Generator().manual_seed(0)
    host = [[torch.randn(N, generator=g), torch.randn(N, generator=g), torch.zeros(N)] for _ in range(2)]
    dev = [[t.cuda() for t in ts] for ts in host]
    wpp = cdiv(N, 128)
    # warp i decodes its descriptors with logical index i (main.py:182-194); with a 5-tile grid, i % 5 is the tile, so
    # warps 0..4 run program 0 over tiles 0..4 and warps 5..9 run program 1 over tiles 0..4
    indices = [0] * wpp + [1] * wpp
    ex.execute_indirect(programs=[C.vec_add_128, C.vec_mul_128], args_list=dev, indices=indices)
    torch.cuda.synchronize()
    pds = [p.get_program(*[_convert_arg(t) for t in ts]) for p, ts in zip((C.vec_add_128, C.vec_mul_128), host)]
    oracle.execute_indirect([pd.program for pd in pds], [[vars(t) for t in pd.input_infos] for pd in pds], host, indices,
                            [pd.input_indices for pd in pds])
    for p in range(2):
        assert bits_equal(dev[p][2], host[p][2]), mismatch_report(dev[p][2], host[p][2])
    torch.testing.assert_close(dev[0][2], dev[0][0] + dev[0][1])
    torch.testing.assert_close(dev[1][2], dev[1][0] * dev[1][1])


def test_indirect_dispatch_single_tile_programs():
    """The shape the reference's test uses: N = 128, one warp per program, add then mul."""
    ex = get_executor()
    a1, b1, a2, b2 = (torch.randn(128, device="cuda") for _ in range(4))
    c1, c2 = torch.zeros(128, device="cuda"), torch.zeros(128, device="cuda")
    # both programs address tile 0 only when their logical index is 0; use one launch per order to cover both
    ex.execute_indirect([C.vec_add_128], [(a1, b1, c1)], [0])
    ex.execute_indirect([C.vec_mul_128, C.vec_add_128], [(a2, b2, c2), (a1, b1, c1)], [0])
    torch.cuda.synchronize()
    torch.testing.assert_close(c1, a1 + b1)
    torch.testing.assert_close(c2, a2 * b2)


def test_indirect_many_programs():
    """Many distinct tiny programs in one launch (the superoptimizer's usage pattern): program p computes x * p + p."""
    ex = get_executor()

    def make(p):
        @bytecode
        def prog(x, y, REGW, WARP):
            xb = make_block_1d(x, 128, 1, 4096, 0)       # every logical program reads the same tile
            yb = make_block_1d(y, 128 * 300, 1, 300, 128)
            fldg_1d(0, xb)
            fmulimm(float(p))
            faddimm(float(p))
            fstg_1d(0, yb)
            halt()
        return prog
    n = 300
    x = torch.randn(128, device="cuda")
    y = torch.zeros(n * 128, device="cuda")
    ex.execute_indirect([make(p) for p in range(n)], [(x, y)] * n, list(range(n)))
    torch.cuda.synchronize()
    ref = torch.stack([x * p + p for p in range(n)]).reshape(-1)
    assert torch.equal(y, ref)


def test_execute_range_shards_cover_the_grid():
    """Two half-range launches with biased base pointers give the same bits as one full launch: the multi-GPU
    sharding primitive, exercised on one device."""
    from gint_b200.workloads import make_workload
    ex = get_executor()
    full = make_workload("rmsnorm", 64, 4096, device="cuda")
    full.run(ex)
    torch.cuda.synchronize()
    want = full.tensors["out"].clone()
    st = full.steps[0]
    # shard s owns rows [32 s, 32 s + 32) in its own buffers; pointers are biased so the program's global row r maps there
    for s in range(2):
        rows = slice(32 * s, 32 * s + 32)
        x_loc = full.tensors["x"][rows].clone()
        out_loc = torch.zeros(32, 4096, device="cuda")
        bias = 32 * s * 4096 * 4
        t = {"x": TensorInterface("f", 4, x_loc.data_ptr() - bias, (), ()), "w": _convert_arg(full.tensors["w"]),
             "out": TensorInterface("f", 4, out_loc.data_ptr() - bias, (), ())}
        ex.execute_range(st.program, [t[r] for r in st.roles], 32 * s, 32)
        torch.cuda.synchronize()
        assert torch.equal(out_loc, want[rows])


@pytest.mark.parametrize("name,leading,inner,chunks", [("rmsnorm", 64, 4096, 5), ("rmsnorm", 7, 256, 16), ("add", 4096, 1, 4),
                                                       ("add", 1000, 1, 3), ("bmm4x4", 1000, 16, 7), ("inv4x4", 33, 16, 2)])
def test_execute_streamed_matches_execute(name, leading, inner, chunks):
    """Host data, transfers overlapped with the kernels range by range: same bits as copy-in, one launch, copy-out."""
    from gint_b200.workloads import make_workload
    ex = get_executor()
    wl = make_workload(name, leading, inner, device="cuda")
    st = wl.steps[0]
    host = {r: t.cpu().pin_memory() for r, t in wl.tensors.items()}
    wl.run(ex)
    torch.cuda.synchronize()
    want = {r: wl.tensors[r].cpu() for r in wl.outputs}
    dev = [torch.full_like(wl.tensors[r], float("nan")) for r in st.roles]           # staging buffers hold no data yet
    ins = {i: host[r] for i, r in enumerate(st.roles) if r not in wl.outputs}
    outs = {i: torch.zeros_like(host[r]).pin_memory() for i, r in enumerate(st.roles) if r in wl.outputs}
    launches = ex.launches
    ex.execute_streamed(st.program, dev, st.grid_dim, ins, outs, n_chunks=chunks)
    torch.cuda.synchronize()
    assert ex.launches - launches == min(chunks, st.grid_dim)
    for i, r in enumerate(st.roles):
        if r in wl.outputs:
            assert bits_equal(outs[i], want[r]), mismatch_report(outs[i], want[r])


def test_plan_runs_all_steps_with_one_call():
    """The conductor graph's two bytecode programs as a plan: same bits as one execute() per step; set_arg re-points an
    output; a bad step is reported with its index."""
    from gint_b200.workloads import make_workload
    ex = get_executor()
    wl = make_workload("graph", 8192, 1024, device="cuda")
    wl.run(ex)
    torch.cuda.synchronize()
    want = {r: wl.tensors[r].clone() for r in wl.outputs}
    for r in wl.outputs:
        wl.tensors[r].zero_()
    plan = wl.plan(ex)
    assert len(plan) == len(wl.steps) == 2
    wl.pre(wl.tensors)
    launches = ex.launches
    plan.run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert ex.launches - launches == 2
    for r in wl.outputs:
        assert bits_equal(wl.tensors[r], want[r])
    # re-point the last step's output at another buffer
    last = wl.steps[-1]
    out_role = "s"   # the row sums: written by the last step only
    other = torch.zeros_like(wl.tensors[out_role])
    plan.set_arg(len(wl.steps) - 1, last.roles.index(out_role), other)
    plan.run(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert bits_equal(other, want[out_role])
    # a step whose handle is unknown fails with its position in the message, after the steps before it were queued
    plan._steps[1].handle = 0xDEAD
    with pytest.raises(capi.GintError, match="plan step 1 of 2"):
        plan.run()
    torch.cuda.synchronize()


def test_launch_info_reports_geometry():
    from gint_b200.workloads import make_workload
    ex = get_executor()
    # (the inverse needs 12 slots with its 8 registers in the pool; they live in shared memory instead and the pool is its stack)
    for name, pool, smem_regs in (("rmsnorm", 4, 0), ("bmm4x4", 7, 0), ("inv4x4", 7, 8)):
        wl = make_workload(name, {"rmsnorm": 64}.get(name, 1000), {"rmsnorm": 4096}.get(name, 16), device="cuda")
        st = wl.steps[0]
        info = ex.launch_info(st.program, [wl.tensors[r] for r in st.roles], st.grid_dim)
        assert info["pool_size"] == pool and info["registers_in_smem"] == smem_regs
        assert info["tiles_per_warp"] in (1, 2, 4)
        assert info["num_sms"] == torch.cuda.get_device_properties(0).multi_processor_count
        assert info["grid_blocks"] >= 1 and info["regs_per_thread"] > 0 and info["smem_bytes"] > 0


@pytest.mark.parametrize("name,leading", [("inv4x4", 1000), ("inv4x4", 33), ("inv4x4", 524288)])
def test_registers_in_shared_memory_give_the_bits_of_the_pool(name, leading):
    """The same program on the kernel that keeps the virtual registers in shared memory (default for programs that would need
    the 12-slot pool) and on the 12-slot pool kernel, which lays stack and registers out as the reference does."""
    from gint_b200.workloads import make_workload
    ex = get_executor()
    rf, pool = make_workload(name, leading, 16, device="cuda"), make_workload(name, leading, 16, device="cuda")
    st = rf.steps[0]
    assert ex.launch_info(st.program, [rf.tensors[r] for r in st.roles], st.grid_dim)["registers_in_smem"] == 8
    rf.run(ex, torch.cuda.current_stream().cuda_stream)
    ex.set_option("register_file", 0)
    try:
        assert ex.launch_info(st.program, [pool.tensors[r] for r in st.roles], st.grid_dim)["pool_size"] == 12
        pool.run(ex, torch.cuda.current_stream().cuda_stream)
    finally:
        ex.set_option("register_file", 1)
    torch.cuda.synchronize()
    for role in rf.outputs:
        assert bits_equal(rf.tensors[role], pool.tensors[role]), mismatch_report(rf.tensors[role], pool.tensors[role])


def test_vector_layout_gives_the_bits_of_the_natural_layout():
    """The conductor graph's fused program on the vector-layout kernel (an option: its full 1-D tiles live in the pool as four
    consecutive elements per lane, one rearrangement in front of the warp reduction) and on the ordinary kernel."""
    from gint_b200.workloads import make_workload
    ex = get_executor()
    outs = []
    try:
        for on in (1, 0):
            ex.set_option("vector_layout", on)
            wl = make_workload("graph", 8192, 1024, device="cuda")
            st = wl.steps[0]
            info = ex.launch_info(st.program, [wl.tensors[r] for r in st.roles], st.grid_dim)
            assert info["vector_layout"] == on and info["pool_size"] == 4
            assert ex.launch_info(wl.steps[1].program, [wl.tensors[r] for r in wl.steps[1].roles], wl.steps[1].grid_dim)["vector_layout"] == 0
            wl.run(ex, torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            outs.append({r: wl.tensors[r].clone() for r in wl.outputs})
    finally:
        ex.set_option("vector_layout", 0)
    for r in outs[0]:
        assert bits_equal(outs[0][r], outs[1][r]), mismatch_report(outs[0][r], outs[1][r])


def test_vector_layout_with_a_reduced_scale_matches_the_oracle():
    """sum over a 2048-element row (lanes, then width values), then every tile of the row scaled by that sum: the scale is uniform, so
    the tiles stay in the vector layout; one rearrangement in front of the reduction. Bit-exact against the CPU oracle."""
    # (-(sum * x + 0.5) * 3, so that the program is not one of those that run one tile per warp: they keep the natural layout)
    import numpy as np
    from gint_b200.host import frontend as fe
    from gint_b200.host.executor import BaseExecutableProgram, ProgramData, ProgramTensorInfo
    from oracle import oracle
    n_tiles, rows = 16, 300

    class RowScale(BaseExecutableProgram):
        def get_program(self, x, y):
            bc = [[fe.LoadGlobal1DF32, 0]]
            for i in range(1, n_tiles):
                bc += [[fe.LoadGlobal1DF32, 16 * 128 * i], [fe.FAdd, 0]]
            bc += [[fe.WarpAllReduceSum, 0], [fe.Dup, 0], [fe.FPermW, 0x01000302], [fe.FAdd, 0], [fe.Dup, 0], [fe.FPermW, 0x02030001], [fe.FAdd, 0],
                   [fe.FStoreReg0, 0]]
            for i in range(n_tiles):
                bc += [[fe.LoadGlobal1DF32, 16 * 128 * i], [fe.FLoadReg0, 0], [fe.FMul, 0], [fe.FAddImm, 0x3F000000], [fe.FMulImm, 0x40400000], [fe.FNeg, 0],
                       [fe.StoreGlobal1DF32, 16 * 128 * i + 1]]      # (enough arithmetic per tile for two tiles per warp)
            bc += [[0, 0]]
            infos = [ProgramTensorInfo(4, [128 * n_tiles], [rows], [128 * n_tiles, 1], [1, 0], [1, 1], [0, 0]) for _ in (x, y)]
            return ProgramData(np.array(bc, dtype=np.int32), infos)

    prog = RowScale()
    x = torch.randn(rows, 128 * n_tiles, generator=torch.Generator().manual_seed(5))
    want = [x.clone(), torch.zeros_like(x)]
    pd = prog.get_program(*C.to_interfaces(want))
    oracle.execute(pd.program, [vars(t) for t in pd.input_infos], want, rows)
    ex = get_executor()
    xd, yd = x.cuda(), torch.zeros_like(x).cuda()
    ex.set_option("vector_layout", 1)       # (off by default; applies to programs created from here on)
    try:
        assert ex.launch_info(prog, [xd, yd], rows)["vector_layout"] == 1
        prog(xd, yd, grid_dim=rows)
        torch.cuda.synchronize()
    finally:
        ex.set_option("vector_layout", 0)
    assert bits_equal(yd.cpu(), want[1]), mismatch_report(yd.cpu(), want[1])


def test_register_pressure_case_runs_on_the_register_file_kernel():
    import cases as C
    ex = get_executor()
    case = [c for c in C.build_cases() if c.name == "register_pressure_n1000"][0]
    ts = [t.cuda() for t in case.make(torch.Generator().manual_seed(3))]
    info = ex.launch_info(case.program, ts, case.grid_dim)
    assert info["pool_size"] == 7 and info["registers_in_smem"] == 8


def test_indirect_launch_runs_lane_broadcasts_of_a_small_pool_program():
    """bmm4x4 needs 7 pool slots, so its DupBroadcastW instructions are pre-decoded into their index-in-the-opcode form; the
    indirect kernel (12 slots) must carry those handlers too. Same bits as the direct launch."""
    import cases as C
    ex = get_executor()
    g = torch.Generator().manual_seed(11)
    a, b = torch.randn(64, 16, generator=g).cuda(), torch.randn(64, 16, generator=g).cuda()
    direct, indirect = torch.zeros(64, 16, device="cuda"), torch.zeros(64, 16, device="cuda")
    C.bmm4x4(a, b, direct, grid_dim=2)
    ex.execute_indirect([C.bmm4x4], [(a, b, indirect)], [0, 0])       # both warps run logical programs 0 and 1 of the same program
    torch.cuda.synchronize()
    assert bits_equal(indirect, direct), mismatch_report(indirect, direct)
    torch.testing.assert_close(direct, torch.bmm(a.view(-1, 4, 4), b.view(-1, 4, 4)).reshape(-1, 16), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("leading,inner", [(10, 256), (96, 1024), (8192, 1024)])
def test_gathered_rows_equal_gather_then_launch(leading, inner):
    """The conductor graph with x_full[idx] read in place (gint_execute_gathered) gives the bits of the three-kernel form
    (torch gather into g, fused program, row sum), and matches torch eager."""
    from gint_b200.workloads import EAGER, check_outputs, make_workload
    ex = get_executor()
    three = make_workload("graph", leading, inner, device="cuda")
    two = make_workload("graph_gathered", leading, inner, device="cuda")
    three.run(ex, torch.cuda.current_stream().cuda_stream)
    launches = ex.launches
    two.run(ex, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert ex.launches - launches == 2
    for role in two.outputs:
        assert bits_equal(two.tensors[role], three.tensors[role]), f"{role}: " + mismatch_report(two.tensors[role], three.tensors[role])
    assert torch.equal(two.tensors["g"], torch.zeros_like(two.tensors["g"]))      # the intermediate was never written
    check_outputs(two, EAGER["graph"]({k: v.cpu() for k, v in two.tensors.items()}))
