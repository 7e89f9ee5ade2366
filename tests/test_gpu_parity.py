"""GPU parity: the CUDA interpreter, called through the executor API and the C ABI, against the CPU oracle on the same
seeded inputs (bit-exact for everything that is not transcendental math) and against the torch-eager expressions.

Every case runs at each tiles-per-warp setting (1, 2, 4 and automatic): the kernels for K logical programs per warp
must give the same bits as one program per warp.
"""
import math

import numpy as np
import pytest
import torch

from cases import Case, build_cases, to_interfaces
from conftest import bits_equal, mismatch_report, oracle_run_workload
from fuzz import FuzzProgram, N_IN, N_OUT
from gint_b200 import get_executor
from gint_b200.workloads import EAGER, FULL_SIZES, check_outputs, make_workload
from oracle import oracle

pytestmark = pytest.mark.gpu

CASES = build_cases()
KS = [0, 1, 2, 4]


@pytest.fixture(autouse=True)
def _reset_options():
    yield
    if torch.cuda.is_available():
        get_executor().set_option("tiles_per_warp", 0)


def _run_both(case: Case, k: int, seed: int = 42):
    g = torch.Generator().manual_seed(seed)
    host = case.make(g)
    dev = [t.cuda() for t in host]
    if case.view:
        host, dev = case.view(host), case.view(dev)
    pd = case.program.get_program(*to_interfaces(host), **case.kwargs)
    oracle.execute(pd.program, [vars(t) for t in pd.input_infos], host, case.grid_dim, input_indices=pd.input_indices, threads=4)
    ex = get_executor()
    ex.set_option("tiles_per_warp", k)
    case.program(*dev, grid_dim=case.grid_dim, **case.kwargs)
    torch.cuda.synchronize()
    return host, dev


@pytest.mark.parametrize("k", KS)
@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_case_matches_oracle(case, k):
    host, dev = _run_both(case, k)
    for i in case.outputs:
        if case.exact:
            assert bits_equal(dev[i], host[i]), f"{case.name} output {i}: " + mismatch_report(dev[i], host[i])
        else:
            torch.testing.assert_close(dev[i].cpu().float(), host[i].float(), rtol=max(case.rtol, 2e-5), atol=max(case.atol, 2e-5))
    if case.expect is not None:
        for i, ref in case.expect(host).items():
            got = dev[i].cpu()
            torch.testing.assert_close(got.float(), ref.reshape(got.shape).float(), rtol=max(case.rtol, 1.3e-6), atol=max(case.atol, 1e-5))


@pytest.mark.parametrize("k", KS)
def test_fused_handlers_keep_separate_roundings(k):
    """mul followed by add inside one fused handler must stay two roundings (the bytecode has an FMA opcode for the other
    meaning): outputs 0 and 1 of fused_idioms contain no transcendental and must equal the oracle bit for bit."""
    case = next(c for c in CASES if c.name == "fused_idioms_n1000")
    host, dev = _run_both(case, k)
    assert bits_equal(dev[3], host[3]), mismatch_report(dev[3], host[3])
    assert bits_equal(dev[4], host[4]), mismatch_report(dev[4], host[4])
    a, b, c = host[0], host[1], host[2]
    n = a.numel()
    pad = torch.zeros(((n + 127) // 128) * 128)
    pad[:n] = b
    bt = pad.view(-1, 4, 32)[:, [1, 2, 1, 2], :].reshape(-1)[:n]
    assert torch.equal(host[3], (a * bt) + c)


def test_inputs_are_left_untouched():
    case = next(c for c in CASES if c.name == "vector_add_s12345")
    host, dev = _run_both(case, 0)
    assert bits_equal(dev[0], host[0]) and bits_equal(dev[1], host[1])


# ------------------------------------------------------------------------------------------------ the five named programs, small

SMALL = [("add", 4096, 1), ("add", 1000, 1), ("rmsnorm", 64, 4096), ("rmsnorm", 7, 256), ("rmsnorm", 5, 200), ("rmsnorm", 3, 64),
         ("bmm4x4", 1000, 16), ("bmm4x4", 33, 16), ("bmm4x4", 1, 16), ("inv4x4", 1000, 16), ("inv4x4", 33, 16), ("inv4x4", 1, 16),
         ("graph", 96, 1024), ("graph", 10, 256)]


@pytest.mark.parametrize("k", KS)
@pytest.mark.parametrize("name,leading,inner", SMALL)
def test_named_program_small(name, leading, inner, k):
    cpu = make_workload(name, leading, inner, device="cpu")
    gpu = make_workload(name, leading, inner, device="cuda")
    oracle_run_workload(cpu)
    ex = get_executor()
    ex.set_option("tiles_per_warp", k)
    gpu.run(ex, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for role in gpu.outputs:
        if name in ("add", "bmm4x4", "inv4x4"):   # add/mul/div/moves only: the GPU must reproduce the oracle bit for bit
            assert bits_equal(gpu.tensors[role], cpu.tensors[role]), f"{name}.{role}: " + mismatch_report(gpu.tensors[role], cpu.tensors[role])
        else:                                      # rsqrt / exp are approximate on the GPU
            torch.testing.assert_close(gpu.tensors[role].cpu(), cpu.tensors[role], rtol=1e-5, atol=1e-6)
    check_outputs(gpu, EAGER[name](cpu.tensors))   # tolerances of the benchmark definition: rtol 1e-5 / atol 1e-6 (1e-4 for inv4x4)


# ------------------------------------------------------------------------------------------------ the five named programs, full size

@pytest.mark.parametrize("name", ["add", "rmsnorm", "bmm4x4", "inv4x4", "graph"])
def test_named_program_full_size(name):
    """Full benchmark sizes: compared with torch eager on the GPU, plus size-independent properties."""
    wl = make_workload(name, device="cuda")
    ex = get_executor()
    wl.run(ex, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    ref = EAGER[name](wl.tensors)
    if name == "add":
        assert torch.equal(wl.tensors["out"], ref["out"])
    else:
        for role in wl.outputs:
            torch.testing.assert_close(wl.tensors[role], ref[role].reshape(wl.tensors[role].shape), rtol=wl.rtol, atol=wl.atol)
    if name == "inv4x4":
        A, X = wl.tensors["a"].view(-1, 4, 4), wl.tensors["c"].view(-1, 4, 4)
        resid = (torch.bmm(A, X) - torch.eye(4, device="cuda")).abs().max().item()
        assert resid < 1e-5, resid
    if name == "rmsnorm":   # scale invariance: rmsnorm(2x) == rmsnorm(x) up to eps; rows are independent
        y1 = wl.tensors["out"].clone()
        wl.tensors["x"].mul_(2.0)
        wl.run(ex, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        torch.testing.assert_close(wl.tensors["out"], y1, rtol=1e-5, atol=1e-6)
    if name == "graph":     # the row sum is consistent with z
        torch.testing.assert_close(wl.tensors["s"], wl.tensors["z"].sum(-1), rtol=1e-5, atol=1e-4)
    # a sample of rows/elements is also checked against the CPU oracle bit-for-bit or within tolerance
    if name in ("bmm4x4", "inv4x4"):
        small = make_workload(name, 1000, 16, device="cpu")
        small.tensors["a"].copy_(wl.tensors["a"][:1000].cpu())
        if "b" in small.tensors:
            small.tensors["b"].copy_(wl.tensors["b"][:1000].cpu())
        oracle_run_workload(small)
        assert bits_equal(wl.tensors["c"][:1000], small.tensors["c"])


@pytest.mark.parametrize("name,leading,inner", [("add", 131072, 1), ("rmsnorm", 2048, 4096), ("bmm4x4", 524288, 16), ("inv4x4", 524288, 16),
                                                ("graph", 8192, 1024)])
def test_transformed_streams_give_the_same_bits_as_the_plain_stream(name, leading, inner):
    """Early-issued loads, fast accesses, staged row blocks and fused handlers only reschedule the program: at sizes where
    all of them apply (full tiles, aligned, 32 matrices per tile), the outputs equal those of the untransformed stream."""
    ex = get_executor()
    outs = []
    try:
        for early, fuse in ((1, 1), (0, 0)):
            ex.set_option("early_issue", early)
            ex.set_option("fuse", fuse)
            wl = make_workload(name, leading, inner, device="cuda")      # a fresh program object: built with these options
            wl.run(ex, torch.cuda.current_stream().cuda_stream)
            torch.cuda.synchronize()
            outs.append({r: wl.tensors[r].clone() for r in wl.outputs})
    finally:
        ex.set_option("early_issue", 1)
        ex.set_option("fuse", 1)
    for r in outs[0]:
        assert bits_equal(outs[0][r], outs[1][r]), mismatch_report(outs[0][r], outs[1][r])


@pytest.mark.parametrize("name,leading,inner,out_role,in_role", [("rmsnorm", 2048, 4096, "out", "x"), ("bmm4x4", 524288, 16, "c", "a"),
                                                                  ("add", 131072, 1, "out", "a"), ("inv4x4", 524288, 16, "c", "a")])
def test_output_aliasing_an_input_runs_the_program_as_written(name, leading, inner, out_role, in_role):
    """The output tensor IS one of the inputs. Loads that the pre-decoder moved ahead of stores (the ring of early-issued
    loads, the staged row blocks) would then read stale data, so such a launch must fall back to the untransformed stream;
    the result has to equal the oracle's, which executes the program as written on the same aliased buffers. Checked on a
    sample of the leading units (the oracle is slow) after the whole launch has run."""
    sample = {"rmsnorm": 64, "bmm4x4": 1000, "add": 4096, "inv4x4": 1000}[name]
    gpu = make_workload(name, leading, inner, device="cuda")
    cpu = make_workload(name, sample, inner, device="cpu")
    for r, t in cpu.tensors.items():
        if r != out_role:    # the first `sample` leading units of every sharded input, broadcast operands whole
            src = gpu.tensors[r]
            t.copy_((src[:sample] if src.shape[0] == leading else src).cpu())
    gpu.tensors[out_role] = gpu.tensors[in_role]
    cpu.tensors[out_role] = cpu.tensors[in_role]
    gpu.run(get_executor(), torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    oracle_run_workload(cpu)
    got = gpu.tensors[out_role][:sample]
    if name == "rmsnorm":      # rsqrt: a few ulp between libm and the GPU
        torch.testing.assert_close(got.cpu(), cpu.tensors[out_role], rtol=1e-5, atol=1e-6)
    else:
        assert bits_equal(got, cpu.tensors[out_role]), mismatch_report(got, cpu.tensors[out_role])


# ------------------------------------------------------------------------------------------------ random programs

def _fuzz_inputs(prog: FuzzProgram, seed: int):
    g = torch.Generator().manual_seed(seed)
    r, c = prog.rows, prog.cols
    if prog.family == "float":
        ins = [torch.randn(r, c, generator=g) for _ in range(N_IN)]
        ins[1][ins[1].abs() < 0.05] = 0.0       # exact zeros: division by zero, signed zeros
    else:
        ins = [torch.randint(-2 ** 31, 2 ** 31 - 1, (r, c), generator=g, dtype=torch.int64).to(torch.int32).view(torch.float32) for _ in range(N_IN)]
        ins[1] = torch.randint(-40, 40, (r, c), generator=g, dtype=torch.int64).to(torch.int32).view(torch.float32)
    return ins + [torch.zeros(r, c) for _ in range(N_OUT)]


@pytest.mark.parametrize("family", ["float", "int"])
@pytest.mark.parametrize("seed", range(24))
def test_random_programs_bit_exact(seed, family):
    depth, regs = [(3, 1), (4, 0), (6, 1), (7, 4), (8, 4), (4, 8), (5, 7), (2, 2)][seed % 8]
    rows, cols = [(4, 32), (37, 100), (64, 128), (5, 8), (129, 36), (33, 4)][seed % 6]
    prog = FuzzProgram(seed, family, depth, regs, length=60 + 7 * seed, rows=rows, cols=cols)
    host = _fuzz_inputs(prog, seed)
    pd = prog.get_program()
    oracle.execute(pd.program, [vars(t) for t in pd.input_infos], host, prog.grid_dim)
    ex = get_executor()
    for k in KS:
        dev = [t.cuda() for t in _fuzz_inputs(prog, seed)]
        ex.set_option("tiles_per_warp", k)
        prog(*dev, grid_dim=prog.grid_dim)
        torch.cuda.synchronize()
        for i in range(N_IN, N_IN + N_OUT):
            assert bits_equal(dev[i], host[i]), f"seed {seed} {family} K={k} layout={prog.layout} out {i}: " + mismatch_report(dev[i], host[i])
