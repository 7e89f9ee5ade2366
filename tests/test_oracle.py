"""Pin the CPU oracle (oracle/gint_oracle.c) before anything is compared against it.

1. Known-answer tests the reference keeps for this path: packed immediates -> [1,2,3,4] / [16,32,48,64], int32 add,
   gather and scatter exact (reference tests/test_frontend.py:166-208,245-291).
2. Bytecode streams produced by the reference's own frontend / conductor (gint_b200/data/programs.json), executed by the
   oracle and compared with the torch-eager expressions the reference's tests use.
3. Operand order and lane mapping of every opcode family against independent numpy/torch expectations.
"""
import math

import numpy as np
import pytest
import torch

from cases import Case, build_cases, to_interfaces
from conftest import bits_equal, mismatch_report, oracle_run_workload
from gint_b200.programs import recorded
from gint_b200.workloads import EAGER, check_outputs, make_workload
from oracle import oracle

CASES = build_cases()


def run_case_on_oracle(case: Case, seed: int = 42):
    g = torch.Generator().manual_seed(seed)
    tensors = case.make(g)
    if case.view:
        tensors = case.view(tensors)
    args = to_interfaces(tensors)
    pd = case.program.get_program(*args, **case.kwargs)
    oracle.execute(pd.program, [vars(t) for t in pd.input_infos], tensors, case.grid_dim, input_indices=pd.input_indices)
    return tensors


@pytest.mark.parametrize("case", [c for c in CASES if c.expect is not None], ids=lambda c: c.name)
def test_oracle_matches_torch_eager(case):
    tensors = run_case_on_oracle(case)
    expected = case.expect(tensors)
    for i, ref in expected.items():
        if case.rtol == 0 and case.atol == 0:
            assert bits_equal(tensors[i], ref.reshape(tensors[i].shape)), mismatch_report(tensors[i], ref.reshape(tensors[i].shape))
        else:
            torch.testing.assert_close(tensors[i], ref.reshape(tensors[i].shape).to(tensors[i].dtype), rtol=case.rtol, atol=case.atol)


# ------------------------------------------------------------------------------------------------ golden programs (from the reference)

@pytest.mark.parametrize("name,leading,inner", [
    ("add", 4096, 1), ("add", 1000, 1),
    ("rmsnorm", 64, 4096), ("rmsnorm", 7, 256), ("rmsnorm", 5, 200), ("rmsnorm", 3, 64),
    ("bmm4x4", 1000, 16), ("bmm4x4", 33, 16), ("bmm4x4", 1, 16),
    ("inv4x4", 1000, 16), ("inv4x4", 33, 16), ("inv4x4", 1, 16),
    ("graph", 96, 1024), ("graph", 10, 256),
])
def test_reference_generated_programs_match_eager(name, leading, inner):
    wl = make_workload(name, leading, inner, device="cpu")
    oracle_run_workload(wl)
    errs = check_outputs(wl, EAGER[name](wl.tensors))
    assert all(math.isfinite(e) for e in errs.values())
    if name == "inv4x4":  # A @ X ~ I, the reference's second criterion (tests/test_inv4x4.py)
        A = wl.tensors["a"].view(-1, 4, 4)
        X = wl.tensors["c"].view(-1, 4, 4)
        torch.testing.assert_close(torch.bmm(A, X), torch.eye(4).expand_as(A), rtol=0, atol=1e-5)


def test_recorded_hand_written_programs_match_eager():
    """Streams recorded from the reference's own test programs (not re-typed here)."""
    g = torch.Generator().manual_seed(42)
    p = recorded("basic_expr1_s1000_p64")
    a, b, c = torch.rand(1000, 64, generator=g) + 1e-6, torch.rand(1000, 64, generator=g) + 1e-6, torch.zeros(1000, 64)
    oracle.execute(p.bytecode, [vars(t) for t in p.tensor_infos], [a, b, c], p.grid_dim, input_indices=p.input_indices)
    torch.testing.assert_close(c, -((a + b + b) / b - b))
    p = recorded("vector_expr2_z100000")
    x, y = torch.rand(100000, generator=g), torch.zeros(100000)
    oracle.execute(p.bytecode, [vars(t) for t in p.tensor_infos], [x, y], p.grid_dim, input_indices=p.input_indices)
    torch.testing.assert_close(y, x ** 2 * (3 - 2 * x))
    p = recorded("rmsnorm_bf16_b4_t800_nh12_h64")
    x = (torch.randn(4, 800, 12, 64, generator=g) * 1.5 + 0.5).bfloat16().transpose(1, 2)
    y, w = torch.zeros_like(x), torch.rand(64, generator=g).bfloat16()
    oracle.execute(p.bytecode, [vars(t) for t in p.tensor_infos], [x, y, w], p.grid_dim, input_indices=p.input_indices, threads=4)
    torch.testing.assert_close(y, torch.nn.functional.rms_norm(x, (64,), w, eps=1e-5))


def test_frontend_mirror_reproduces_reference_bytecode():
    """Programs re-expressed with this repository's frontend give the same int32 stream and descriptors as the
    reference's frontend did for the same shapes."""
    import cases as C
    from gint_b200 import TensorInterface

    def ti(shape, elm=4, strides=None):
        if strides is None:
            strides, acc = [], 1
            for e in reversed(shape):
                strides.append(acc)
                acc *= e
            strides = tuple(reversed(strides))
        return TensorInterface("f", elm, 0, tuple(shape), tuple(strides))

    def same(prog, args, rec_name, **kw):
        rec = recorded(rec_name)
        pd = prog.get_program(*args, **kw)
        assert np.array_equal(pd.program, rec.bytecode), rec_name
        assert [vars(t) for t in pd.input_infos] == [vars(t) for t in rec.tensor_infos], rec_name
        assert list(pd.input_indices or range(len(pd.input_infos))) == rec.input_indices, rec_name

    same(C.basic_expr1, [ti((31, 256)) for _ in range(3)], "basic_expr1_s31_p256")
    same(C.vector_expr2, [ti((1023,)) for _ in range(2)], "vector_expr2_z1023", BLOCK=256)
    same(C.BatchAddProgram(), [ti((9999, 32)) for _ in range(3)], "batch_add_s9999_p32")
    same(C.VectorAddProgram(), [ti((12345,)) for _ in range(3)], "vector_add_s12345")
    same(C.bmm4x4, [ti((1000, 16)) for _ in range(3)], "bmm4x4_b1000")
    same(C.indirect_arith, [ti((1, 32)), ti((1, 32)), ti((1, 32)), ti((1, 100)), ti((1, 32)), ti((1, 32)), ti((1, 100))], "indirect_arith")
    same(C.packed_imm, [ti((1, 100)), ti((1, 100))], "packed_imm")
    xs = (1 * 12 * 6 * 80, 80, 6 * 80, 1)   # (B, NH, T, H) view of a (B, T, NH, H) tensor
    same(C.rmsnorm_bf16, [ti((1, 6, 12, 80), 2, xs), ti((1, 6, 12, 80), 2, xs), ti((80,), 2)], "rmsnorm_bf16_b1_t12_nh6_h80")


# ------------------------------------------------------------------------------------------------ independent expectations

def _tiles(x: torch.Tensor):
    """(G, 4, 32) view of a 1-D tensor under the 1-D tile mapping: element = 128*g + lane + 32*w, zero padded."""
    n = x.numel()
    G = (n + 127) // 128
    pad = torch.zeros(G * 128, dtype=x.dtype)
    pad[:n] = x
    return pad.view(G, 4, 32), n


def _untile(t: torch.Tensor, n: int):
    return t.reshape(-1)[:n]


@pytest.mark.parametrize("n", [1, 127, 128, 129, 5000])
def test_alu_mix_expectation(n):
    case = next(c for c in CASES if c.name == f"alu_mix_n{n}")
    t = run_case_on_oracle(case)
    x, y = t[0].double(), t[1].double()
    f = (y * x + y).float().double()                       # fma(y, x, y): one rounding
    d = (t[0] - t[1])                                      # x - y in fp32
    o0 = ((d / t[0]) + 0.5) * -3.0
    m = f > d.double()
    o1 = torch.where(m, t[0], t[1])
    o2 = torch.fmod(t[1], t[0])
    p = ((t[1] - (-t[0])).abs() < 0.25).float()
    q = (t[1] <= t[0]).float()
    o3 = (p + q) / (1.0 / t[0])
    torch.testing.assert_close(t[2], o0, rtol=0, atol=0)
    assert (t[3] != o1).sum() <= max(1, n // 1000)         # a borderline compare may flip under double rounding of the fma model
    torch.testing.assert_close(t[4], o2, rtol=0, atol=0)
    torch.testing.assert_close(t[5], o3, rtol=0, atol=0)


@pytest.mark.parametrize("n", [1, 127, 128, 129, 5000])
def test_int_mix_expectation(n):
    case = next(c for c in CASES if c.name == f"int_mix_n{n}")
    t = run_case_on_oracle(case)
    a = t[0].view(torch.int32).numpy().astype(np.int64)
    b = t[1].view(torch.int32).numpy().astype(np.int64)
    wrap = lambda v: ((v + 2 ** 31) % 2 ** 32) - 2 ** 31
    ba = wrap(b * a)
    d = wrap(a - ba)
    v = wrap((d ^ b) | a)
    s = b & 31
    o0 = wrap((v % 2 ** 32) >> s)                          # logical shift right of the 32-bit pattern
    # C-style truncating division; /0 -> -1, %0 -> dividend (the values the GPU path defines)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(b == 0, -1, np.trunc(a / np.where(b == 0, 1, b)).astype(np.int64))
        r = np.where(b == 0, a, a - np.where(b == 0, 0, q) * b)
    w = (np.arange(n) % 128) // 32                         # width lane of each element
    o1 = wrap(((q + r) % 2 ** 32) << w)
    assert np.array_equal(t[2].view(torch.int32).numpy().astype(np.int64), o0)
    assert np.array_equal(t[3].view(torch.int32).numpy().astype(np.int64), o1)


@pytest.mark.parametrize("n", [1, 127, 128, 129, 5000])
def test_width_ops_expectation(n):
    case = next(c for c in CASES if c.name == f"width_ops_n{n}")
    t = run_case_on_oracle(case)
    xt, _ = _tiles(t[0])                                   # (G, w, lane)
    x0, x1, x2, x3 = xt[:, 0], xt[:, 1], xt[:, 2], xt[:, 3]
    o0 = torch.stack([x0, x1, x0, x2], dim=1)              # fperm_w(3,0,2,1) then fshuf2(1,3,0,2)
    o1 = xt + x2.unsqueeze(1)
    mx = xt.max(dim=2, keepdim=True).values
    mn = xt.min(dim=2, keepdim=True).values
    tot = xt.double().sum(dim=(1, 2), keepdim=True).float()
    o2 = (mx + mn + tot).expand_as(xt)
    assert torch.equal(t[1], _untile(o0, n))
    assert torch.equal(t[2], _untile(o1, n))
    torch.testing.assert_close(t[3], _untile(o2, n), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("r,c", [(1, 1), (7, 33), (64, 100)])
def test_dtype_tiles_expectation(r, c):
    case = next(k for k in CASES if k.name == f"dtype_tiles_r{r}_c{c}")
    t = run_case_on_oracle(case)
    h = t[0].float() + t[1].float()
    prod = h.half().float() * 0 + h * t[2].float()         # fp32 product of the un-narrowed sum and the u8 value
    assert torch.equal(t[3], h.half())
    assert torch.equal(t[4], prod.bfloat16())
    assert torch.equal(t[5], prod)


NARROW = [c.name for c in CASES if c.name.startswith(("dtype_tiles_1d", "dtype_tiles_2dw"))]


@pytest.mark.parametrize("name", NARROW)
def test_narrow_type_tiles_expectation(name):
    """1-D and 2DW f16 / bf16 / u8 loads and f16 / bf16 stores against an independent torch expression: widening is exact,
    narrowing is round-to-nearest-even (ties, overflow to inf, NaN stays NaN), and Nop / Pop2 leave the values alone."""
    case = next(k for k in CASES if k.name == name)
    t = run_case_on_oracle(case)
    h = t[0].float() + t[1].float()
    prod = h * t[2].float()
    for got, want in ((t[3], h.half()), (t[4], prod.bfloat16()), (t[5], prod)):
        assert got.shape == want.shape
        nan = torch.isnan(want.float())
        assert torch.equal(torch.isnan(got.float()), nan)
        assert torch.equal(got.float()[~nan], want.float()[~nan])
        # signed zeros too
        assert torch.equal(torch.signbit(got.float()[~nan]), torch.signbit(want.float()[~nan]))


def test_narrowing_ties_go_to_even():
    """Known answers for the special values in front of the narrow-type inputs."""
    case = next(k for k in CASES if k.name == "dtype_tiles_1d_n127")
    t = run_case_on_oracle(case)
    oh = t[3].float()
    assert oh[0] == 1.0                      # 1 + 2^-11 is halfway between 1 and 1 + 2^-10: even mantissa wins
    assert oh[1] == 1.0 + 2.0 ** -9          # 1 + 3 * 2^-11 is halfway between 1 + 2^-10 and 1 + 2^-9
    assert oh[2] == 1.0                      # 1 + 2^-12 is below the tie
    assert oh[3] == float("inf")             # 65504 + 16 is the tie between 65504 (odd mantissa) and 2^16: even wins, which overflows
    assert oh[4] == 65504.0                  # 65504 + 8 is below that tie
    assert torch.isnan(oh[7]) and torch.isnan(oh[11]) and oh[6] == float("inf") and oh[10] == float("-inf")


def test_advance_alias_expectation():
    """Stores through a moved slot are seen by the loads that follow them in program order."""
    case = next(k for k in CASES if k.name == "advance_alias")
    g = torch.Generator().manual_seed(42)
    orig = case.make(g)[0].clone()
    t = run_case_on_oracle(case)
    a0, a1 = orig[128:256], orig[256:384]
    assert torch.equal(t[0][:128], 2 * a0)
    assert torch.equal(t[1], 3 * (2 * a0))
    assert torch.equal(t[0][128:], a1 + 2 * a0)


def test_special_math_close_to_libm():
    case = next(c for c in CASES if c.name == "special_math_n777")
    t = run_case_on_oracle(case)
    x = t[0].double()
    torch.testing.assert_close(t[1].double(), x.sqrt() + x.rsqrt(), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(t[2].double(), x.exp() + x.exp2(), rtol=1e-6, atol=1e-6)
    torch.testing.assert_close(t[3].double(), x.log() + x.log2(), rtol=1e-6, atol=2e-6)
    torch.testing.assert_close(t[4].double(), x.sin() + x.cos() + (x.float() * 0.3).double().tan(), rtol=1e-6, atol=2e-6)
    xs = (x.float() * 0.2).double()
    misc = xs.asin() + xs.acos() + x.atan() + x.erf() + torch.atan2(torch.full_like(x, 2.0), x) + x.pow(1.5)
    torch.testing.assert_close(t[5].double(), misc, rtol=2e-6, atol=4e-6)


# ------------------------------------------------------------------------------------------------ edge cases

def test_empty_grid_is_a_no_op():
    c = torch.full((16,), 5.0)
    import cases as C
    pd = C.VectorAddProgram().get_program(*to_interfaces([c, c, c]))
    oracle.execute(pd.program, [vars(t) for t in pd.input_infos], [c, c, c], 0)
    assert torch.equal(c, torch.full((16,), 5.0))


def test_nan_propagating_min_max_and_signed_zero():
    from gint_b200 import bytecode
    from gint_b200.host.frontend import fldg_1d, fstg_1d, halt, make_block_1d, warp_allreduce_fmax, warp_allreduce_fmin

    @bytecode
    def prog(x, mx, mn, REGW, WARP):
        xb, a, b = [make_block_1d(t, 128, 1) for t in (x, mx, mn)]
        fldg_1d(0, xb); warp_allreduce_fmax(); fstg_1d(0, a)
        fldg_1d(0, xb); warp_allreduce_fmin(); fstg_1d(0, b)
        halt()
    x = torch.zeros(128)
    x[:32] = torch.arange(32.0)
    x[5] = float("nan")                      # width lane 0 has a NaN -> both reductions give NaN there
    x[32:64] = -0.0
    x[40] = 0.0                              # width lane 1: max(-0, +0) = +0, min = -0
    mx, mn = torch.zeros(128), torch.zeros(128)
    pd = prog.get_program(*to_interfaces([x, mx, mn]))
    oracle.execute(pd.program, [vars(t) for t in pd.input_infos], [x, mx, mn], 1)
    assert torch.isnan(mx[:32]).all() and torch.isnan(mn[:32]).all()
    assert (mx[32:64].view(torch.int32) == 0).all()                 # +0.0
    assert (mn[32:64].view(torch.int32) == -2 ** 31).all()          # -0.0


def test_gather_does_not_reject_negative_indices():
    """idx < shape1 is a signed compare with no lower bound (load_store.py:266-288): index -1 reads the element below."""
    from gint_b200 import bytecode
    from gint_b200.host.frontend import fldg_1d_ind, fstg_1d, halt, ipush4, make_block_1d

    @bytecode
    def prog(data, out, REGW, WARP):
        d = make_block_1d(data, 4, 1)
        o = make_block_1d(out, 128, 1)
        ipush4(0x7f0300ff)        # indices (-1, 0, 3, 127): -1 passes, 127 >= shape -> 0.0
        fldg_1d_ind(d)
        fstg_1d(0, o)
        halt()
    backing = torch.arange(10.0)
    data, out = backing[1:5], torch.zeros(128)
    pd = prog.get_program(*to_interfaces([data, out]))
    oracle.execute(pd.program, [vars(t) for t in pd.input_infos], [data, out], 1)
    assert out[0] == 0.0 and out[32] == 1.0 and out[64] == 4.0 and out[96] == 0.0   # backing[0], data[0], data[3], masked


def test_register_aliasing_follows_pool_layout():
    """Register n is pool[P-1-n] (state.py:38-41). With the reference's largest layout (P = 12) a stack 8 deep overwrites
    register 7 = pool[4]; the oracle reproduces that layout when told to use it."""
    import gint_b200.host.frontend as fe
    bc = [[fe.LoadImm, fe._f32_bits(7.0)], [fe.FStoreReg0 + 7, 0]]
    bc += [[fe.LoadImm, fe._f32_bits(float(i))] for i in range(8)]          # depth 8: slot 4 is clobbered by value 4.0
    bc += [[fe.Pop2, 0]] * 4
    bc += [[fe.FLoadReg0 + 7, 0], [fe.StoreGlobal1DF32, 0], [fe.Halt, 0]]
    out = torch.zeros(128)
    info = dict(elm_size=4, batch_strides=[], batch_shape=[], block_shape_stride_1=[128, 1], block_shape_stride_2=[1, 0],
                block_grid_dims=[1, 1], block_grid_steps=[0, 0])
    st = oracle.analyze(np.array(bc, dtype=np.int32))
    assert st["pool_size"] == 12 and st["max_stack"] == 8 and st["max_reg_idx"] == 7
    oracle.execute(np.array(bc, dtype=np.int32), [info], [out], 1)
    assert torch.equal(out, torch.full((128,), 4.0))
