"""Program cases shared by the oracle tests (CPU) and the GPU parity tests.

Each case is a program written with this repository's frontend mirror (so it reads like the reference's tests),
seeded host inputs, and -- where one exists -- the torch-eager expectation the reference's tests use.
`exact` says whether the GPU and the CPU oracle must agree bit for bit (everything except transcendental math).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import numpy as np
import torch

from gint_b200 import TensorInterface, bytecode, cdiv
from gint_b200.host.executor import BaseExecutableProgram, ProgramData, ProgramTensorInfo
from gint_b200.host.frontend import *  # noqa: F401,F403

REGW = 4


@dataclass
class Case:
    name: str
    program: BaseExecutableProgram
    make: Callable[[torch.Generator], list]           # -> list of CPU tensors (inputs and zeroed outputs)
    grid_dim: int
    outputs: list                                      # indices into the tensor list
    expect: Optional[Callable[[list], dict]] = None    # tensors -> {output index: expected tensor}
    exact: bool = True
    kwargs: dict = field(default_factory=dict)
    view: Optional[Callable[[list], list]] = None      # applied after `make` (and after moving to the device): strided views
    rtol: float = 1.3e-6
    atol: float = 1e-5


# ------------------------------------------------------------------------------------------------ programs

@bytecode
def basic_expr1(a, b, c, REGW, WARP):
    """-((a + b + b) / b - b) on 2DT tiles; operand order of fadd/fdiv/fsub/fneg (reference tests/test_frontend.py:8-26)."""
    B, C = a.shape
    a, b, c = [make_block_2d(t, [C, B], [t.strides[1], t.strides[0]], [1, cdiv(B, REGW)], [0, REGW]) for t in (a, b, c)]
    for i in range(0, C, WARP):
        fldg_2dt(i, b)
        dup()
        dup2()
        fldg_2dt(i, a)
        fadd()
        fadd()
        fdiv()
        fsub()
        fneg()
        fstg_2dt(i, c)
    halt()


@bytecode
def vector_expr2(x, y, REGW, WARP, BLOCK):
    """Cubic ease x^2 (3 - 2x) via fmaimm (reference tests/test_frontend.py:28-43)."""
    C, = x.shape
    x, y = [make_block_1d(t, C, t.strides[-1], cdiv(C, BLOCK), BLOCK) for t in (x, y)]
    for i in range(0, BLOCK, WARP * REGW):
        fldg_1d(i, x)
        dup()
        dup()
        fmaimm(-2.0, 3.0)
        fmul()
        fmul()
        fstg_1d(i, y)
    halt()


@bytecode
def vec_add_128(a, b, c, REGW, WARP):
    """One 128-element tile per logical program (block shape = full extent, so later tiles are not masked)."""
    N, = a.shape
    a, b, c = [make_block_1d(t, N, t.strides[0], cdiv(N, WARP * REGW), WARP * REGW) for t in (a, b, c)]
    fldg_1d(0, a)
    fldg_1d(0, b)
    fadd()
    fstg_1d(0, c)
    halt()


@bytecode
def vec_mul_128(a, b, c, REGW, WARP):
    N, = a.shape
    a, b, c = [make_block_1d(t, N, t.strides[0], cdiv(N, WARP * REGW), WARP * REGW) for t in (a, b, c)]
    fldg_1d(0, a)
    fldg_1d(0, b)
    fmul()
    fstg_1d(0, c)
    halt()


class BatchAddProgram(BaseExecutableProgram):
    """Raw-opcode 2DT batch add (reference tests/test_a_plus_b_executor.py:10-33)."""

    def get_program(self, a, b, c) -> ProgramData:
        B, C = a.shape
        bc = []
        for i in range(0, C, 32):
            bc.extend([70, 16 * i, 70, 16 * i + 1, 2, 0, 71, 16 * i + 2])
        bc.extend([0, 0])
        return ProgramData(np.array(bc, dtype=np.int32),
                           [ProgramTensorInfo(4, [], [], [C, t.strides[1]], [B, t.strides[0]], [1, cdiv(B, self.REGW)], [0, self.REGW])
                            for t in (a, b, c)])


class VectorAddProgram(BaseExecutableProgram):
    """Raw-opcode 1D add, 256 elements per logical program (reference tests/test_a_plus_b_executor.py:36-61)."""

    def get_program(self, a, b, c) -> ProgramData:
        C, = a.shape
        bc, block = [], 256
        for i in range(0, block, 32 * self.REGW):
            bc.extend([15, 16 * i, 15, 16 * i + 1, 2, 0, 16, 16 * i + 2])
        bc.extend([0, 0])
        return ProgramData(np.array(bc, dtype=np.int32),
                           [ProgramTensorInfo(4, [], [], [C, t.strides[0]], [1, 0], [cdiv(C, block), 1], [block, 0]) for t in (a, b, c)])


@bytecode
def indirect_arith(a, b, c, data, indices, out_load, out_store, REGW, WARP):
    """Integer add, gather and scatter (reference tests/test_frontend.py:166-188)."""
    a, b, c, data, indices, out_load, out_store = [make_block_1d(t, t.shape[-1], t.strides[-1])
                                                  for t in (a, b, c, data, indices, out_load, out_store)]
    fldg_1d(0, a)
    fldg_1d(0, b)
    iadd()
    fstg_1d(0, c)
    fldg_1d(0, indices)
    fldg_1d_ind(data)
    fstg_1d(0, out_load)
    fldg_1d(0, out_load)
    fldg_1d(0, indices)
    fstg_1d_ind(out_store)
    halt()


@bytecode
def packed_imm(packed_f_out, packed_i_out, REGW, WARP):
    """Packed immediates written through a scatter (reference tests/test_frontend.py:191-208)."""
    packed_f_out, packed_i_out = [make_block_1d(t, t.shape[-1], t.strides[-1]) for t in (packed_f_out, packed_i_out)]
    fpush4(0x04030201)
    ipush4(0x03020100)
    fstg_1d_ind(packed_f_out)
    ipush4(0x40302010)
    ipush4(0x03020100)
    fstg_1d_ind(packed_i_out)
    halt()


@bytecode
def rmsnorm_bf16(x, y, w, REGW, WARP):
    """Hand-written bf16 RMSNorm over (B, NH, T, H) with arbitrary strides (reference tests/test_rmsnorm.py:112-151)."""
    B, NH, T, H = x.shape
    xb, yb = [make_block_2d(t, [H, T], [t.strides[-1], t.strides[-2]], [1, cdiv(T, REGW)], [0, REGW],
                            [t.strides[0], t.strides[1]], [B, NH]) for t in (x, y)]
    wb = make_block_2d(w, [H, T], [w.strides[-1], 0], [1, cdiv(T, REGW)], [0, REGW], [0, 0], [B, NH])
    fpush(0.0)
    for c in range(0, H, WARP):
        fldg_2dt_bf16(c, xb)
        dup()
        fma()
    warp_allreduce_fsum()
    fmaimm(1 / H, 1e-5)
    frsqrt()
    for c in range(0, H, WARP):
        dup()
        fldg_2dt_bf16(c, xb)
        fmul()
        fldg_2dt_bf16(c, wb)
        fmul()
        fstg_2dt_bf16(c, yb)
    halt()


@bytecode
def bmm4x4(a, b, c, REGW, WARP):
    """Batched 4x4 matmul, one matrix per lane (reference gint/host/matrix.py:35-56, tests/test_bmm4x4.py:7-37)."""
    B, _ = a.shape
    ab, bb, cb = [make_block_2d(t, [B, 16], [t.strides[0], t.strides[1]], [cdiv(B, 32), 1], [32, 0]) for t in (a, b, c)]
    for i in range(4):
        fldg_2dw(4 * i, ab)
        for k in range(4):
            dup_broadcast_w(k)
            fldg_2dw(4 * k, bb)
            fmul()
            swap()
        pop()
        for _ in range(3):
            fadd()
        fstg_2dw(4 * i, cb)
    halt()


@bytecode
def alu_mix(x, y, o0, o1, o2, o3, REGW, WARP):
    """Float ALU, compares, select, immediates, stack shuffles and registers in one program (exact ops only)."""
    N, = x.shape
    xb, yb, b0, b1, b2, b3 = [make_block_1d(t, N, t.strides[0], cdiv(N, 128), 128) for t in (x, y, o0, o1, o2, o3)]
    fldg_1d(0, xb)          # x
    fldg_1d(0, yb)          # x y
    dup2()                  # x y x y
    fma()                   # x  (y*x + y)           T=y,S=x,U=y -> y*x+y
    fstore_reg(0)           # x            r0 = y*x+y
    dup()                   # x x
    fldg_1d(0, yb)          # x x y
    frsub()                 # x  (x - y)             S - T
    dupx1()                 # (x-y) x (x-y)
    fdiv()                  # (x-y)  ((x-y)/x)       T / S
    faddimm(0.5)
    fmulimm(-3.0)
    fstg_1d(0, b0)          # (x-y)
    fload_reg(0)            # (x-y) r0
    fgt()                   # [r0 > (x-y)]
    fldg_1d(0, xb)          # m x
    fldg_1d(0, yb)          # m x y
    dupx2()                 # y m x y
    pop()                   # y m x
    swap()                  # y x m
    fselect()               # m > 0 ? x : y
    fstg_1d(0, b1)
    fldg_1d(0, xb)
    fldg_1d(0, yb)
    frem()                  # fmod(y, x)
    fstg_1d(0, b2)
    fldg_1d(0, xb)
    fneg()
    fldg_1d(0, yb)
    fapprox(0.25)           # |y - (-x)| < 0.25
    fldg_1d(0, xb)
    fldg_1d(0, yb)
    fle()                   # y <= x
    fadd()
    fldg_1d(0, xb)
    frcp()
    frdiv()                 # S / T = (cmp sum) / (1/x)
    fstg_1d(0, b3)
    halt()


@bytecode
def int_mix(a, b, o0, o1, REGW, WARP):
    """Every integer opcode on int32 bit patterns; shifts by the low bits of b."""
    N, = a.shape
    ab, bb, b0, b1 = [make_block_1d(t, N, t.strides[0], cdiv(N, 128), 128) for t in (a, b, o0, o1)]
    fldg_1d(0, ab)
    fldg_1d(0, bb)
    imul()                  # b*a
    fldg_1d(0, ab)
    isub()                  # a - b*a
    fldg_1d(0, bb)
    ixor()
    fldg_1d(0, ab)
    ior()
    fldg_1d(0, bb)
    ipush4(0x1f1f1f1f)
    iand()                  # b & 31  (T=31, S=b -> 31 & b)
    swap()                  # shift value
    ishr()                  # value >> (b&31)   T=value? see expectation
    fstg_1d(0, b0)
    fldg_1d(0, bb)          # b
    fldg_1d(0, ab)          # b a
    idiv()                  # a / b
    fldg_1d(0, bb)          # q b
    fldg_1d(0, ab)          # q b a
    irem()                  # q (a % b)
    iadd()
    ipush4(0x03020100)      # shift amounts 0,1,2,3 per width lane
    swap()
    ishl()                  # (q + r) << lane_w
    fstg_1d(0, b1)
    halt()


@bytecode
def width_ops(x, o0, o1, o2, REGW, WARP):
    """Width-lane permutes and the reduction + width-combine idiom of the conductor (op_registry.py:346-359)."""
    N, = x.shape
    xb, b0, b1, b2 = [make_block_1d(t, N, t.strides[0], cdiv(N, 128), 128) for t in (x, o0, o1, o2)]
    fldg_1d(0, xb)
    fperm_w(3, 0, 2, 1)
    fldg_1d(0, xb)
    fshuf2(1, 3, 0, 2)      # (perm[1], perm[3], x[0], x[2])
    fstg_1d(0, b0)
    fldg_1d(0, xb)
    dup_broadcast_w(2)
    fadd()
    fstg_1d(0, b1)
    fldg_1d(0, xb)
    warp_allreduce_fmax()
    fldg_1d(0, xb)
    warp_allreduce_fmin()
    fadd()
    fldg_1d(0, xb)
    warp_allreduce_fsum()
    dup()
    fperm_w(2, 3, 0, 1)
    fadd()
    dup()
    fperm_w(1, 0, 3, 2)
    fadd()
    fadd()
    fstg_1d(0, b2)
    halt()


@bytecode
def dtype_tiles(xh, xb, xu, oh, ob, of, REGW, WARP):
    """f16 / bf16 / u8 tiles through all three layouts, with AdvanceBlock2D and AdvanceBase."""
    R, C = xh.shape                                  # R rows (width dim), C columns (thread dim)
    th = [make_block_2d(t, [C, R], [t.strides[1], t.strides[0]], [1, cdiv(R, REGW)], [0, REGW]) for t in (xh, xb, xu, oh, ob, of)]
    h, b, u, ohb, obb, ofb = th
    for i in range(0, C, WARP):
        fldg_2dt_f16(i, h)
        fldg_2dt_bf16(i, b)
        fadd()
        dup()
        fstg_2dt_f16(i, ohb)
        fldg_2dt_u8(i, u)
        fmul()
        dup()
        fstg_2dt_bf16(i, obb)
        fstg_2dt(i, ofb)
    halt()


@bytecode
def advance_walk(x, y, REGW, WARP, STEPS):
    """Walk a (T, 4)-tiled 2D tensor with AdvanceBlock2D on the thread dim and AdvanceBase on the output pointer."""
    T, W = x.shape
    xb = make_block_2d(x, [T, W], [x.strides[0], x.strides[1]], [1, 1], [0, 0])
    yb = make_block_2d(y, [T, W], [y.strides[0], y.strides[1]], [1, 1], [0, 0])
    for s in range(STEPS):
        fldg_2dw(0, xb)
        fmulimm(2.0)
        fstg_2dw(0, yb)
        adv_block_2d(32, xb)
        adv_base(32 * y.strides[0] * 4, yb)
    halt()


@bytecode
def dtype_tiles_1d(xh, xb, xu, oh, ob, of, REGW, WARP):
    """f16 / bf16 / u8 tiles through the 1-D layout (element = offset + lane + 32 w), with Nop and Pop2 along the way."""
    N, = xh.shape
    h, b, u, ohb, obb, ofb = [make_block_1d(t, N, t.strides[0], cdiv(N, 256), 256) for t in (xh, xb, xu, oh, ob, of)]
    for i in range(0, 256, WARP * REGW):
        nop()
        fldg_1d_f16(i, h)
        fldg_1d_bf16(i, b)
        fadd()
        dup()
        fstg_1d_f16(i, ohb)
        fpush(3.0)
        fpush(4.0)
        pop2()                 # drops both immediates
        fldg_1d_u8(i, u)
        fmul()
        dup()
        fstg_1d_bf16(i, obb)
        fstg_1d(i, ofb)
    halt()


@bytecode
def dtype_tiles_2dw(xh, xb, xu, oh, ob, of, REGW, WARP):
    """f16 / bf16 / u8 tiles through the 2DW layout: thread = row (dim 1), width lane = column (dim 2)."""
    T, W = xh.shape
    h, b, u, ohb, obb, ofb = [make_block_2d(t, [T, W], [t.strides[0], t.strides[1]], [cdiv(T, WARP), 1], [WARP, 0])
                              for t in (xh, xb, xu, oh, ob, of)]
    for j in range(0, W, REGW):
        fldg_2dw_f16(j, h)
        fldg_2dw_bf16(j, b)
        fadd()
        dup()
        fstg_2dw_f16(j, ohb)
        fldg_2dw_u8(j, u)
        fmul()
        dup()
        fstg_2dw_bf16(j, obb)
        fstg_2dw(j, ofb)
    halt()


@bytecode
def advance_alias(a, out, REGW, WARP):
    """A store through a slot that AdvanceBase has moved OUTSIDE the extent its descriptor gives lands on what a later load of
    another slot reads: the load must see the stored values, so it may not be started ahead of the store. (`out` is described
    as 128 elements that do not overlap `a`; moved by 512 bytes it covers a[0:128].)"""
    ab, ob = make_block_1d(a, 256, 1), make_block_1d(out, 128, 1)
    fldg_1d(0, ab); fmulimm(2.0); adv_base(512, ob); fstg_1d(0, ob)       # a[0:128] = 2 a[0:128], through the moved `out`
    fldg_1d(0, ab); fmulimm(3.0); adv_base(-512, ob); fstg_1d(0, ob)      # out[0:128] = 3 * (the new a[0:128])
    fldg_1d(128, ab); fldg_1d(0, ab); fadd(); adv_base(1024, ob); fstg_1d(0, ob)   # a[128:256] += a[0:128]
    halt()


def narrow_special_values(n: int, g: torch.Generator):
    """Inputs for the narrow-type cases: random values with, in front, sums that are exact ties of the f16 / bf16 roundings,
    values beyond the f16 range, signed zeros, infinities and NaN."""
    h = torch.randn(n, generator=g).half()
    b = torch.randn(n, generator=g).bfloat16()
    u = torch.randint(0, 256, (n,), generator=g, dtype=torch.int64).to(torch.uint8)
    sp_h = torch.tensor([1.0, 1.0, 1.0, 65504.0, 65504.0, -0.0, float("inf"), float("nan"), 6.1e-5, 2.0 ** -24, 0.0, 1.0]).half()
    sp_b = torch.tensor([2.0 ** -11, 3 * 2.0 ** -11, 2.0 ** -12, 16.0, 8.0, 0.0, 1.0, 1.0, -6.1e-5, 2.0 ** -25, float("-inf"), float("nan")]).bfloat16()
    sp_u = torch.tensor([1, 1, 1, 1, 255, 7, 0, 3, 1, 1, 2, 0], dtype=torch.uint8)
    k = min(n, sp_h.numel())
    h[:k], b[:k], u[:k] = sp_h[:k], sp_b[:k], sp_u[:k]
    return h, b, u


@bytecode
def special_math(x, o_sqrt, o_exp, o_log, o_trig, o_misc, REGW, WARP):
    """Transcendental opcodes (approximate on the GPU; compared with a tolerance)."""
    N, = x.shape
    xb, bs, be, bl, bt, bm = [make_block_1d(t, N, t.strides[0], cdiv(N, 128), 128) for t in (x, o_sqrt, o_exp, o_log, o_trig, o_misc)]
    fldg_1d(0, xb); fsqrt(); fldg_1d(0, xb); frsqrt(); fadd(); fstg_1d(0, bs)
    fldg_1d(0, xb); fexp(); fldg_1d(0, xb); fexp2(); fadd(); fstg_1d(0, be)
    fldg_1d(0, xb); flog(); fldg_1d(0, xb); flog2(); fadd(); fstg_1d(0, bl)
    fldg_1d(0, xb); fsin(); fldg_1d(0, xb); fcos(); fadd(); fldg_1d(0, xb); fmulimm(0.3); ftan(); fadd(); fstg_1d(0, bt)
    fldg_1d(0, xb); fmulimm(0.2); fasin(); fldg_1d(0, xb); fmulimm(0.2); facos(); fadd()
    fldg_1d(0, xb); fatan(); fadd(); fldg_1d(0, xb); ferf(); fadd()
    fldg_1d(0, xb); fpush(2.0); fatan2(); fadd()        # atan2(2, x)
    fldg_1d(0, xb); fpush(1.5); swap(); fpow(); fadd()   # x ** 1.5  (T=x, S=1.5)
    fstg_1d(0, bm)
    halt()


@bytecode
def fused_idioms(a, b, c, o0, o1, o2, REGW, WARP):
    """Instruction sequences that the pre-decoder replaces by fused handlers, in contexts where a contracted
    multiply-add would show (the product's other factor comes from a permute, a register, an immediate)."""
    N, = a.shape
    ab, bb, cb, b0, b1, b2 = [make_block_1d(t, N, 1, cdiv(N, 128), 128) for t in (a, b, c, o0, o1, o2)]
    fldg_1d(0, cb); fldg_1d(0, ab); fldg_1d(0, bb); fperm_w(1, 2, 1, 2); fmul(); fadd(); fstg_1d(0, b0)      # perm; [mul, add]
    fldg_1d(0, cb); fstore_reg(1); fldg_1d(0, ab); fload_reg(1); fmul(); fldg_1d(0, bb); fsub(); fstg_1d(0, b1)  # mul; [load, sub]
    fldg_1d(0, ab); dup(); fneg(); fexp(); faddimm(1.0); frdiv()                                              # SiLU idiom
    fldg_1d(0, bb); fmulimm(0.3); faddimm(-1.25); fmul(); fldg_1d(0, cb); fadd(); fstg_1d(0, b2)              # mulimm; addimm; [mul] [load, add, store]
    halt()


STATIC_FPERM = [(0, 0, 0, 0), (2, 3, 0, 1), (1, 0, 3, 2), (0, 0, 1, 1), (1, 1, 1, 1), (2, 1, 2, 1), (1, 1, 2, 2), (2, 2, 2, 2),
                (3, 3, 2, 2), (3, 0, 3, 0), (0, 3, 0, 3), (0, 2, 1, 3), (3, 3, 0, 0), (3, 3, 3, 3), (3, 2, 1, 0), (1, 3, 0, 2)]
STATIC_FSHUF2 = [(0, 1, 0, 1), (3, 1, 3, 1), (2, 0, 2, 0), (0, 2, 0, 2), (1, 3, 1, 3), (2, 3, 2, 3), (3, 3, 0, 1), (0, 0, 0, 0)]


@bytecode
def permute_selectors(a, b, out, REGW, WARP):
    """FPermW / FShuf2 with the selectors that have handlers of their own (the first 14 / 6 of each list) and with two that do
    not; every result is scaled by a different constant and accumulated, so a wrong lane shows in the sum."""
    N, = a.shape
    ab, bb, ob = [make_block_1d(t, N, 1, cdiv(N, 128), 128) for t in (a, b, out)]
    fpush(0.0)
    for i, sel in enumerate(STATIC_FPERM):
        fldg_1d(0, ab); fperm_w(*sel); fmulimm(float(i + 1)); fadd()
    for i, sel in enumerate(STATIC_FSHUF2):
        fldg_1d(0, ab); fldg_1d(0, bb); fshuf2(*sel); fmulimm(float(2 * i + 3)); fadd()
    fstg_1d(0, ob)
    halt()


@bytecode
def shifted_in_place(a, out, REGW, WARP):
    """out[i] = 2 a[i], chunk by chunk, where `out` is the same memory as `a` one chunk further on: every store changes
    what the next load reads. A launch that had started the loads early would see the old values."""
    N, = a.shape
    ab, ob = make_block_1d(a, N, 1), make_block_1d(out, N, 1)
    for off in range(0, N, 128):
        fldg_1d(off, ab); fmulimm(2.0); fstg_1d(off, ob)
    halt()


@bytecode
def register_pressure(a, b, o0, o1, REGW, WARP):
    """Eight registers and a stack five deep: the 12-slot pool in the reference (register 7 and stack slot 4 are the same pool
    entry there, which this program never notices), the register-file kernels here. Register loads feed permutes, shuffles and
    products in the combinations those kernels fuse, and a few that they do not."""
    N, = a.shape
    ab, bb, o0b, o1b = [make_block_1d(t, N, 1, cdiv(N, 128), 128) for t in (a, b, o0, o1)]
    fldg_1d(0, ab); fstore_reg(0)
    fldg_1d(0, bb); fstore_reg(1)
    for n in range(2, 8):                                     # r[n] = r[n-1] * 0.5 + r[n-2]
        fload_reg(n - 2); fload_reg(n - 1); fmulimm(0.5); fadd(); fstore_reg(n)
    fload_reg(7); fperm_w(1, 0, 3, 2); fload_reg(6); fperm_w(2, 3, 0, 1); fmul()      # load, permute, load, permute, multiply
    fload_reg(5); fperm_w(3, 3, 0, 0); fload_reg(4); fmul()                           # load, permute, load, multiply
    fload_reg(3); fload_reg(2); fperm_w(0, 2, 1, 3); fmul()                           # load, load, permute, multiply
    fload_reg(1); fload_reg(0); fshuf2(3, 1, 2, 0)                                    # load, load, shuffle   (depth 4)
    fload_reg(6); fmul()                                                              # load, multiply (register 7 is gone by now:
                                                                                      # the fifth stack slot is the same pool entry)
    fadd(); fadd(); fsub(); fstore_reg(3)                                             # depth 0
    fload_reg(0); fload_reg(1); dup2(); fshuf2(0, 1, 0, 1); fstore_reg(4); fshuf2(2, 3, 2, 3); fstore_reg(5)
    fload_reg(3); fload_reg(4); fload_reg(5); fload_reg(6); fload_reg(2)               # depth 5
    fmul(); frsub(); fstore_reg(6)                                                    # multiply, reverse subtract, store
    fmul()
    fload_reg(6); fperm_w(2, 2, 1, 1); fadd()
    fstg_1d(0, o0b)
    fload_reg(3); fload_reg(5); fmul(); fload_reg(4); frsub(); fstg_1d(0, o1b)
    halt()


# ------------------------------------------------------------------------------------------------ case list

def _z(*shape, dtype=torch.float32):
    return torch.zeros(*shape, dtype=dtype)


def build_cases() -> list[Case]:
    cases: list[Case] = []

    for s, p in [(1, 1), (4, 16), (6, 18), (31, 32), (32, 64), (1000, 18), (257, 256)]:
        def mk(g, s=s, p=p):
            return [torch.rand(s, p, generator=g) + 1e-6, torch.rand(s, p, generator=g) + 1e-6, _z(s, p)]
        cases.append(Case(f"basic_expr1_s{s}_p{p}", basic_expr1, mk, cdiv(s, REGW), [2],
                          expect=lambda t: {2: -((t[0] + t[1] + t[1]) / t[1] - t[1])}))

    for z in [1, 5, 16, 17, 31, 32, 33, 1023, 1024, 100001]:
        def mk(g, z=z):
            return [torch.rand(z, generator=g), _z(z)]
        cases.append(Case(f"vector_expr2_z{z}", vector_expr2, mk, cdiv(z, 256), [1], kwargs=dict(BLOCK=256),
                          expect=lambda t: {1: t[0] ** 2 * (3 - 2 * t[0])}))

    for s, p in [(1, 1), (6, 18), (31, 32), (9999, 32), (200, 256)]:
        def mk(g, s=s, p=p):
            return [torch.randn(s, p, generator=g), torch.randn(s, p, generator=g), _z(s, p)]
        cases.append(Case(f"batch_add_s{s}_p{p}", BatchAddProgram(), mk, cdiv(s, REGW), [2], expect=lambda t: {2: t[0] + t[1]}))

    for s in [1, 32, 33, 256, 12345, 100000]:
        def mk(g, s=s):
            return [torch.randn(s, generator=g), torch.randn(s, generator=g), _z(s)]
        cases.append(Case(f"vector_add_s{s}", VectorAddProgram(), mk, cdiv(s, 256), [2], expect=lambda t: {2: t[0] + t[1]}))

    # strided 1-D views (stride 3) and an empty grid
    def mk_strided(g):
        return [torch.randn(3000, generator=g) for _ in range(2)] + [_z(3000)]
    cases.append(Case("vector_add_strided", VectorAddProgram(), mk_strided, cdiv(1000, 256), [2], expect=lambda t: {2: t[0] + t[1]},
                      view=lambda ts: [b[::3] for b in ts]))

    def mk_ind(g):
        a = torch.randint(0, 100, (1, 32), generator=g, dtype=torch.int32)
        b = torch.randint(0, 100, (1, 32), generator=g, dtype=torch.int32)
        idx = torch.randint(0, 100, (1, 32), generator=g, dtype=torch.int32)
        return [a.view(torch.float32), b.view(torch.float32), torch.zeros(1, 32, dtype=torch.int32).view(torch.float32),
                torch.rand(1, 100, generator=g), idx.view(torch.float32), _z(1, 32), _z(1, 100)]

    def exp_ind(t):
        a, b, idx = t[0].view(torch.int32), t[1].view(torch.int32), t[4].view(torch.int32).long()
        gathered = t[3][0][idx[0]].view(1, 32)
        scat = torch.zeros(100)
        # duplicate indices: any of the written values is legal; every duplicate carries the same value here
        scat[idx[0]] = gathered[0]
        return {2: (a + b).view(torch.float32), 5: gathered, 6: scat.view(1, 100)}
    cases.append(Case("indirect_arith", indirect_arith, mk_ind, 1, [2, 5, 6], expect=exp_ind, rtol=0, atol=0))

    def exp_imm(t):
        f = torch.zeros(1, 100)
        f[0, :4] = torch.tensor([1.0, 2.0, 3.0, 4.0])
        i = torch.zeros(1, 100, dtype=torch.int32)
        i[0, :4] = torch.tensor([16, 32, 48, 64], dtype=torch.int32)
        return {0: f, 1: i.view(torch.float32)}
    cases.append(Case("packed_imm", packed_imm, lambda g: [_z(1, 100), _z(1, 100)], 1, [0, 1], expect=exp_imm, rtol=0, atol=0))

    for bb, t_, nh, h in [(1, 12, 1, 16), (1, 12, 6, 80), (4, 100, 3, 64), (1, 300, 2, 128)]:
        def mk(g, bb=bb, t_=t_, nh=nh, h=h):
            x = (torch.randn(bb, t_, nh, h, generator=g) * 1.5 + 0.5).to(torch.bfloat16)
            return [x, torch.zeros_like(x), torch.rand(h, generator=g).to(torch.bfloat16)]
        cases.append(Case(f"rmsnorm_bf16_b{bb}_t{t_}_nh{nh}_h{h}", rmsnorm_bf16, mk, bb * nh * cdiv(t_, REGW), [1], exact=False,
                          view=lambda ts: [ts[0].transpose(1, 2), ts[1].transpose(1, 2), ts[2]],
                          expect=lambda t: {1: torch.nn.functional.rms_norm(t[0].float(), (t[0].shape[-1],), t[2].float(), eps=1e-5).to(torch.bfloat16)},
                          rtol=1.6e-2, atol=1e-2))

    for B in [1, 31, 32, 64, 1000, 40000]:
        def mk(g, B=B):
            return [torch.randn(B, 16, generator=g), torch.randn(B, 16, generator=g), _z(B, 16)]
        cases.append(Case(f"bmm4x4_B{B}", bmm4x4, mk, cdiv(B, 32), [2], rtol=1e-5, atol=1e-5,
                          expect=lambda t: {2: torch.bmm(t[0].view(-1, 4, 4), t[1].view(-1, 4, 4)).reshape(-1, 16)}))

    for n in [1, 127, 128, 129, 5000]:
        def mk(g, n=n):
            return [torch.randn(n, generator=g), torch.randn(n, generator=g)] + [_z(n) for _ in range(4)]
        cases.append(Case(f"alu_mix_n{n}", alu_mix, mk, cdiv(n, 128), [2, 3, 4, 5]))

        def mki(g, n=n):
            a = torch.randint(-2 ** 31, 2 ** 31 - 1, (n,), generator=g, dtype=torch.int64).to(torch.int32)
            b = torch.randint(-50, 50, (n,), generator=g, dtype=torch.int64).to(torch.int32)   # includes zeros: division by zero
            return [a.view(torch.float32), b.view(torch.float32), _z(n), _z(n)]
        cases.append(Case(f"int_mix_n{n}", int_mix, mki, cdiv(n, 128), [2, 3]))

        def mkw(g, n=n):
            return [torch.randn(n, generator=g)] + [_z(n) for _ in range(3)]
        cases.append(Case(f"width_ops_n{n}", width_ops, mkw, cdiv(n, 128), [1, 2, 3]))

    cases.append(Case("shifted_in_place_n1024", shifted_in_place, lambda g: [torch.randn(1024 + 128, generator=g)], 1, [1],
                      view=lambda ts: [ts[0][:1024], ts[0][128:]]))

    for n in [128, 1000]:
        def mkp(g, n=n):
            return [torch.randn(n, generator=g), torch.randn(n, generator=g), _z(n)]
        cases.append(Case(f"permute_selectors_n{n}", permute_selectors, mkp, cdiv(n, 128), [2]))

    for n in [128, 1000, 40000]:
        def mkr(g, n=n):
            return [torch.randn(n, generator=g), torch.randn(n, generator=g), _z(n), _z(n)]
        cases.append(Case(f"register_pressure_n{n}", register_pressure, mkr, cdiv(n, 128), [2, 3]))

    for n in [1, 128, 1000]:
        def mkf(g, n=n):
            return [torch.randn(n, generator=g) for _ in range(3)] + [_z(n) for _ in range(3)]
        cases.append(Case(f"fused_idioms_n{n}", fused_idioms, mkf, cdiv(n, 128), [3, 4, 5], exact=False, rtol=2e-6, atol=2e-6))

    for r, c in [(1, 1), (7, 33), (64, 100)]:
        def mk(g, r=r, c=c):
            return [torch.randn(r, c, generator=g).half(), torch.randn(r, c, generator=g).bfloat16(),
                    torch.randint(0, 256, (r, c), generator=g, dtype=torch.int64).to(torch.uint8),
                    _z(r, c, dtype=torch.float16), _z(r, c, dtype=torch.bfloat16), _z(r, c)]
        cases.append(Case(f"dtype_tiles_r{r}_c{c}", dtype_tiles, mk, cdiv(r, REGW), [3, 4, 5]))

    # narrow types through the 1-D and 2DW layouts (partial tiles, a strided view, rounding ties, NaN / inf / overflow)
    for n in [1, 127, 256, 1000]:
        def mk(g, n=n):
            h, b, u = narrow_special_values(n, g)
            return [h, b, u, _z(n, dtype=torch.float16), _z(n, dtype=torch.bfloat16), _z(n)]
        cases.append(Case(f"dtype_tiles_1d_n{n}", dtype_tiles_1d, mk, cdiv(n, 256), [3, 4, 5]))

    def mk_1d_strided(g):
        h, b, u = narrow_special_values(900, g)
        return [h, b, u, _z(900, dtype=torch.float16), _z(900, dtype=torch.bfloat16), _z(900)]
    cases.append(Case("dtype_tiles_1d_strided", dtype_tiles_1d, mk_1d_strided, cdiv(300, 256), [3, 4, 5], view=lambda ts: [t[::3] for t in ts]))

    for t_, w_ in [(1, 4), (33, 6), (100, 16)]:
        def mk(g, t_=t_, w_=w_):
            h, b, u = narrow_special_values(t_ * w_, g)
            return [h.view(t_, w_), b.view(t_, w_), u.view(t_, w_), _z(t_, w_, dtype=torch.float16), _z(t_, w_, dtype=torch.bfloat16), _z(t_, w_)]
        cases.append(Case(f"dtype_tiles_2dw_t{t_}_w{w_}", dtype_tiles_2dw, mk, cdiv(t_, 32), [3, 4, 5]))

    def mk_2dw_strided(g):
        h, b, u = narrow_special_values(64 * 24, g)
        return [h.view(64, 24), b.view(64, 24), u.view(64, 24), _z(64, 24, dtype=torch.float16), _z(64, 24, dtype=torch.bfloat16), _z(64, 24)]
    cases.append(Case("dtype_tiles_2dw_strided", dtype_tiles_2dw, mk_2dw_strided, cdiv(64, 32), [3, 4, 5],
                      view=lambda ts: [t[1::2, ::2] for t in ts]))

    def mk_adv(g):
        return [torch.randn(100, 4, generator=g), torch.full((128, 4), 7.0)]
    cases.append(Case("advance_walk", advance_walk, mk_adv, 1, [1], kwargs=dict(STEPS=4),
                      expect=lambda t: {1: torch.cat([t[0] * 2.0, torch.zeros(28, 4)])}))

    cases.append(Case("advance_alias", advance_alias, lambda g: [torch.randn(384, generator=g)], 1, [0, 1],
                      view=lambda ts: [ts[0][128:384], ts[0][0:128]]))

    for n in [1, 128, 777]:
        def mk(g, n=n):
            return [torch.rand(n, generator=g) * 3 + 0.1] + [_z(n) for _ in range(5)]
        cases.append(Case(f"special_math_n{n}", special_math, mk, cdiv(n, 128), [1, 2, 3, 4, 5], exact=False, rtol=2e-5, atol=2e-5))

    return cases


def to_interfaces(tensors) -> list[TensorInterface]:
    from gint_b200.host.executor import _convert_arg
    return [_convert_arg(t) for t in tensors]
