"""Bytecode emitters: the ``@bytecode`` DSL vocabulary of gint (mirror of ``gint/host/frontend.py``).

Inside a function decorated with ``gint_b200.bytecode`` every call below appends one ``[opcode, operand]`` pair to
the program being recorded; outside of one it just returns that pair. ``make_block_1d`` / ``make_block_2d``
register a tensor descriptor and return it; passing the descriptor object where an ``arg_i`` is expected resolves
to its slot number. Operand encodings are the bytecode format's (``gint/host/frontend.py:104-482``):

* tile loads/stores:  ``16 * offset + slot``
* ``fpush``/``faddimm``/``fmulimm``/``fapprox``: the float32 bit pattern
* ``fmaimm``: two float16 packed as (mul = low half, add = high half)
* ``fperm_w`` / ``fshuf2`` / ``fpush4`` / ``ipush4``: four bytes, little endian, one per width lane
"""
from __future__ import annotations

import functools
from contextvars import ContextVar
from typing import Optional, Sequence

import numpy

from .. import opcodes as _op
from ..opcodes import *  # noqa: F401,F403  (Halt, FAdd, ... as module constants, like the reference's star import)
from .executor import ProgramTensorInfo, TensorInterface

REG_WIDTH = _op.REG_WIDTH


class FrontendState:
    """What one ``@bytecode`` function call has recorded so far."""

    def __init__(self, fn_args: Sequence[TensorInterface]) -> None:
        self.bc: list[list[int]] = []
        self.tis: list[ProgramTensorInfo] = []
        self.tis_arg_ids: list[int] = []
        self.fn_args = fn_args
        self._arg_pos = {id(a): i for i, a in enumerate(fn_args)}
        self._slot_of: dict[int, int] = {}

    def add_tensor(self, source, info: ProgramTensorInfo) -> None:
        key = source if isinstance(source, int) else id(source)
        self._slot_of[id(info)] = len(self.tis)
        self.tis.append(info)
        self.tis_arg_ids.append(self._arg_pos[key])

    def resolve(self, x):
        return self._slot_of.get(id(x), x)


_frontend_state: ContextVar[Optional[FrontendState]] = ContextVar("_frontend_state", default=None)


def _emitter(fn):
    @functools.wraps(fn)
    def wrapper(*args):
        st = _frontend_state.get()
        if st is None:
            return fn(*args)
        pair = fn(*(st.resolve(a) for a in args))
        st.bc.append([int(pair[0]), int(pair[1])])
        return pair
    return wrapper


def _descriptor(fn):
    @functools.wraps(fn)
    def wrapper(*args, **kwargs):
        info = fn(*args, **kwargs)
        st = _frontend_state.get()
        if st is not None:
            st.add_tensor(args[0], info)
        return info
    return wrapper


@_descriptor
def make_block_1d(t: TensorInterface, block1d_shape: int, block1d_stride: int, block1d_grid_dim: int = 1,
                  block1d_grid_step: int = 0, batch_strides: Sequence[int] = (), batch_shape: Sequence[int] = ()) -> ProgramTensorInfo:
    return ProgramTensorInfo(elm_size=t.elm_size, batch_strides=list(batch_strides), batch_shape=list(batch_shape),
                             block_shape_stride_1=[block1d_shape, block1d_stride], block_shape_stride_2=[1, 0],
                             block_grid_dims=[block1d_grid_dim, 1], block_grid_steps=[block1d_grid_step, 0])


@_descriptor
def make_block_2d(t: TensorInterface, block2d_shape: Sequence[int], block2d_stride: Sequence[int],
                  block2d_grid_dims: Sequence[int] = (1, 1), block2d_grid_steps: Sequence[int] = (0, 0),
                  batch_strides: Sequence[int] = (), batch_shape: Sequence[int] = ()) -> ProgramTensorInfo:
    """``block2d_shape`` / ``block2d_stride`` are given as (thread dim, width dim)."""
    return ProgramTensorInfo(elm_size=t.elm_size, batch_strides=list(batch_strides), batch_shape=list(batch_shape),
                             block_shape_stride_1=[block2d_shape[0], block2d_stride[0]],
                             block_shape_stride_2=[block2d_shape[1], block2d_stride[1]],
                             block_grid_dims=list(block2d_grid_dims), block_grid_steps=list(block2d_grid_steps))


def _f32_bits(v: float) -> int:
    return int(numpy.float32(v).view(numpy.int32))


def _bytes4(a: int, b: int, c: int, d: int) -> int:
    return (a & 0xFF) | ((b & 0xFF) << 8) | ((c & 0xFF) << 16) | ((d & 0xFF) << 24)


def _define(name: str, opcode: int, kind: str):
    if kind == "none":
        def fn():
            return [opcode, 0]
    elif kind == "f32":
        def fn(val: float):
            return [opcode, _f32_bits(val)]
    elif kind == "tile":
        def fn(offset, arg_i):
            return [opcode, 16 * offset + arg_i]
    elif kind == "slot":
        def fn(arg_i):
            return [opcode, arg_i]
    elif kind == "raw":
        def fn(value: int):
            return [opcode, value]
    elif kind == "bytes4":
        def fn(i0: int, i1: int, i2: int, i3: int):
            return [opcode, _bytes4(i0, i1, i2, i3)]
    else:  # pragma: no cover
        raise ValueError(kind)
    fn.__name__ = fn.__qualname__ = name
    globals()[name] = _emitter(fn)


_EMITTERS = [
    # name, opcode, operand kind
    ("halt", Halt, "none"), ("nop", Nop, "none"),
    ("fadd", FAdd, "none"), ("fmul", FMul, "none"), ("fma", FMA, "none"), ("fsub", FSub, "none"), ("frsub", FRSub, "none"),
    ("fneg", FNeg, "none"), ("fdiv", FDiv, "none"), ("frdiv", FRDiv, "none"), ("frem", FRem, "none"),
    ("fpush", LoadImm, "f32"), ("faddimm", FAddImm, "f32"), ("fmulimm", FMulImm, "f32"),
    ("fldg_1d", LoadGlobal1DF32, "tile"), ("fstg_1d", StoreGlobal1DF32, "tile"),
    ("fldg_1d_f16", LoadGlobal1DF16, "tile"), ("fstg_1d_f16", StoreGlobal1DF16, "tile"),
    ("fldg_1d_bf16", LoadGlobal1DBF16, "tile"), ("fstg_1d_bf16", StoreGlobal1DBF16, "tile"),
    ("fldg_1d_u8", LoadGlobal1DU8, "tile"),
    ("pop", Pop, "none"), ("pop2", Pop2, "none"), ("dup", Dup, "none"), ("dupx1", DupX1, "none"), ("dupx2", DupX2, "none"),
    ("dup2", Dup2, "none"), ("swap", Swap, "none"),
    ("fgt", FGt, "none"), ("flt", FLt, "none"), ("fge", FGe, "none"), ("fle", FLe, "none"), ("feq", FEq, "none"), ("fne", FNe, "none"),
    ("fapprox", FApprox, "f32"), ("fselect", Select, "none"),
    ("warp_allreduce_fsum", WarpAllReduceSum, "none"), ("warp_allreduce_fmax", WarpAllReduceMax, "none"),
    ("warp_allreduce_fmin", WarpAllReduceMin, "none"), ("warp_allreduce_fprod", WarpAllReduceProd, "none"),
    ("fsqrt", FSqrt, "none"), ("fsin", FSin, "none"), ("fcos", FCos, "none"), ("ftan", FTan, "none"), ("fasin", FArcSin, "none"),
    ("facos", FArcCos, "none"), ("fatan", FArcTan, "none"), ("fatan2", FArcTan2, "none"), ("fpow", FPow, "none"),
    ("fexp", FExp, "none"), ("fexp2", FExp2, "none"), ("flog", FLog, "none"), ("flog2", FLog2, "none"), ("frsqrt", FRSqrt, "none"),
    ("ferf", FErf, "none"), ("frcp", FRcp, "none"),
    ("iadd", IAdd, "none"), ("imul", IMul, "none"), ("isub", ISub, "none"), ("idiv", IDiv, "none"), ("irem", IRem, "none"),
    ("ishl", IShl, "none"), ("ishr", IShr, "none"), ("iand", IAnd, "none"), ("ior", IOr, "none"), ("ixor", IXor, "none"),
    ("fldg_1d_ind", LoadGlobal1DF32Indirect, "slot"), ("fstg_1d_ind", StoreGlobal1DF32Indirect, "slot"),
    ("fpush4", LoadImm4F, "raw"), ("ipush4", LoadImm4I, "raw"),
    ("fldg_2dt", LoadGlobal2DTF32, "tile"), ("fstg_2dt", StoreGlobal2DTF32, "tile"),
    ("fldg_2dt_f16", LoadGlobal2DTF16, "tile"), ("fstg_2dt_f16", StoreGlobal2DTF16, "tile"),
    ("fldg_2dt_bf16", LoadGlobal2DTBF16, "tile"), ("fstg_2dt_bf16", StoreGlobal2DTBF16, "tile"),
    ("fldg_2dt_u8", LoadGlobal2DTU8, "tile"),
    ("fldg_2dw", LoadGlobal2DWF32, "tile"), ("fstg_2dw", StoreGlobal2DWF32, "tile"),
    ("fldg_2dw_f16", LoadGlobal2DWF16, "tile"), ("fstg_2dw_f16", StoreGlobal2DWF16, "tile"),
    ("fldg_2dw_bf16", LoadGlobal2DWBF16, "tile"), ("fstg_2dw_bf16", StoreGlobal2DWBF16, "tile"),
    ("fldg_2dw_u8", LoadGlobal2DWU8, "tile"),
    ("adv_block_2d", AdvanceBlock2D, "tile"), ("adv_base", AdvanceBase, "tile"),
    ("dup_broadcast_w", DupBroadcastW, "raw"),
    ("fperm_w", FPermW, "bytes4"), ("fshuf2", FShuf2, "bytes4"),
]
for _name, _opc, _kind in _EMITTERS:
    _define(_name, _opc, _kind)


@_emitter
def fmaimm(mul: float, add: float):
    """top * mul + add with both immediates rounded to float16."""
    return [FMAImm, int(numpy.array([mul, add], dtype=numpy.float16).view(numpy.int32).item())]


@_emitter
def fload_reg(n: int):
    return [LOAD_REGS[n], 0]


@_emitter
def fstore_reg(n: int):
    return [STORE_REGS[n], 0]


__all__ = (["FrontendState", "make_block_1d", "make_block_2d", "fmaimm", "fload_reg", "fstore_reg", "REG_WIDTH"]
           + [e[0] for e in _EMITTERS] + list(_op.__all__))
