"""Random straight-line bytecode programs with valid stack discipline, for GPU-vs-oracle bit-exact comparison.

Two families that never mix, so that NaN payload differences between x86 and the GPU cannot leak into integer bit
operations: `float` (IEEE add/sub/mul/fma/div, compares, select, immediates, reductions) and `int` (two's-complement ops).
Both use every stack/width-lane move, the virtual registers, and 1-D / 2-D-T / 2-D-W tile loads and stores.
"""
from __future__ import annotations

import numpy as np

from gint_b200 import opcodes as O
from gint_b200.host.executor import BaseExecutableProgram, ProgramData, ProgramTensorInfo
from gint_b200.host.frontend import _bytes4, _f32_bits

N_IN, N_OUT = 3, 3


class FuzzProgram(BaseExecutableProgram):
    """Tensors: N_IN inputs and N_OUT outputs, all fp32 of shape (rows, cols) row-major; tiles of 32 columns x 4 rows
    (2DT), 32 rows x 4 columns (2DW), or 128 consecutive elements (1D)."""

    def __init__(self, seed: int, family: str, max_depth: int, n_regs: int, length: int, rows: int, cols: int):
        super().__init__()
        self.seed, self.family, self.max_depth, self.n_regs, self.length = seed, family, max_depth, n_regs, length
        self.rows, self.cols = rows, cols
        self.layout = ["1d", "2dt", "2dw"][seed % 3]
        self._pd = self._generate()

    def cache_policy(self, *a, **k):
        return None

    def get_program(self, *args, **kw) -> ProgramData:
        return self._pd

    # grid: number of logical programs needed to cover the tensor under the chosen layout
    @property
    def grid_dim(self) -> int:
        r, c = self.rows, self.cols
        if self.layout == "1d":
            return -(-(r * c) // 128)
        if self.layout == "2dt":
            return -(-c // 32) * -(-r // 4)
        return -(-r // 32) * -(-c // 4)

    def _infos(self):
        r, c = self.rows, self.cols
        if self.layout == "1d":
            mk = lambda: ProgramTensorInfo(4, [], [], [r * c, 1], [1, 0], [-(-(r * c) // 128), 1], [128, 0])
        elif self.layout == "2dt":   # thread dim = columns (stride 1), width dim = rows
            mk = lambda: ProgramTensorInfo(4, [], [], [c, 1], [r, c], [-(-c // 32), -(-r // 4)], [32, 4])
        else:                        # thread dim = rows, width dim = columns (stride 1): 16-byte rows when c % 4 == 0
            mk = lambda: ProgramTensorInfo(4, [], [], [r, c], [c, 1], [-(-r // 32), -(-c // 4)], [32, 4])
        return [mk() for _ in range(N_IN + N_OUT)]

    def _generate(self) -> ProgramData:
        rng = np.random.default_rng(self.seed)
        ld = {"1d": O.LoadGlobal1DF32, "2dt": O.LoadGlobal2DTF32, "2dw": O.LoadGlobal2DWF32}[self.layout]
        st = {"1d": O.StoreGlobal1DF32, "2dt": O.StoreGlobal2DTF32, "2dw": O.StoreGlobal2DWF32}[self.layout]
        bc: list[list[int]] = []
        depth = 0
        out_next = 0
        regs_written: set[int] = set()

        def emit(op, operand=0):
            nonlocal depth
            need, net = O.STACK_EFFECTS[op]
            assert depth >= need, (O.NAMES[op], depth)
            depth += net
            assert depth <= self.max_depth
            bc.append([op, int(np.int32(np.uint32(operand & 0xFFFFFFFF)))])

        def perm():
            return _bytes4(*rng.integers(0, 4, 4).tolist())

        if self.family == "float":
            binary = [O.FAdd, O.FMul, O.FSub, O.FRSub, O.FDiv, O.FRDiv, O.FGt, O.FLt, O.FGe, O.FLe, O.FEq, O.FNe]
            unary = [O.FNeg, O.FRcp]
            reduce_ = [O.WarpAllReduceSum, O.WarpAllReduceMax, O.WarpAllReduceMin, O.WarpAllReduceProd]
        else:
            binary = [O.IAdd, O.IMul, O.ISub, O.IDiv, O.IRem, O.IShl, O.IShr, O.IAnd, O.IOr, O.IXor]
            unary, reduce_ = [], []

        for _ in range(self.length):
            choices = []
            if depth < self.max_depth:
                choices += ["load", "load", "imm"]
                if regs_written:
                    choices.append("regload")
            if depth >= 1:
                choices += ["unary", "perm", "store", "immop"]
                if reduce_ and rng.random() < 0.3:
                    choices.append("reduce")
                if self.n_regs:
                    choices.append("regstore")
                if depth < self.max_depth:
                    choices += ["dup", "bcast"]
            if rng.random() < 0.05:
                choices.append("nop")
            if depth >= 2:
                choices += ["binary", "binary", "binary", "swap", "shuf"]
                if depth >= 3 and rng.random() < 0.2:
                    choices.append("pop2")
                if depth < self.max_depth:
                    choices.append("dupx1")
                if depth + 2 <= self.max_depth:
                    choices.append("dup2")
            if depth >= 3:
                choices += ["tern"]
                if depth < self.max_depth:
                    choices.append("dupx2")
            kind = choices[rng.integers(len(choices))]
            if kind == "load":
                emit(ld, 16 * 0 + int(rng.integers(N_IN)))
            elif kind == "imm":
                if self.family == "float":
                    which = rng.integers(3)
                    if which == 0:
                        emit(O.LoadImm, _f32_bits(float(rng.normal())))
                    elif which == 1:
                        emit(O.LoadImm4F, _bytes4(*rng.integers(-8, 8, 4).tolist()))
                    else:
                        emit(O.LoadImm, _f32_bits(float(rng.choice([0.0, -0.0, 1.0, 0.5, 1e-30, 3e38]))))
                else:
                    emit(O.LoadImm4I, _bytes4(*rng.integers(-128, 128, 4).tolist()))
            elif kind == "regload":
                emit(O.LOAD_REGS[int(rng.choice(sorted(regs_written)))])
            elif kind == "regstore":
                r = int(rng.integers(self.n_regs))
                regs_written.add(r)
                emit(O.STORE_REGS[r])
            elif kind == "unary":
                if unary:
                    emit(unary[rng.integers(len(unary))])
            elif kind == "immop":
                if self.family == "float":
                    which = rng.integers(3)
                    if which == 0:
                        emit(O.FAddImm, _f32_bits(float(rng.normal())))
                    elif which == 1:
                        emit(O.FMulImm, _f32_bits(float(rng.normal())))
                    else:
                        emit(O.FMAImm, int(np.array(rng.normal(size=2), dtype=np.float16).view(np.int32).item()))
            elif kind == "perm":
                emit(O.FPermW, perm())
            elif kind == "shuf":
                emit(O.FShuf2, perm())
            elif kind == "bcast":
                emit(O.DupBroadcastW, int(rng.integers(4)))
            elif kind == "reduce":
                emit(reduce_[rng.integers(len(reduce_))])
            elif kind == "store":
                emit(st, 16 * 0 + N_IN + (out_next % N_OUT))
                out_next += 1
            elif kind == "dup":
                emit(O.Dup)
            elif kind == "dupx1":
                emit(O.DupX1)
            elif kind == "dupx2":
                emit(O.DupX2)
            elif kind == "dup2":
                emit(O.Dup2)
            elif kind == "swap":
                emit(O.Swap)
            elif kind == "nop":
                emit(O.Nop)
            elif kind == "pop2":
                emit(O.Pop2)
            elif kind == "binary":
                emit(binary[rng.integers(len(binary))])
            elif kind == "tern":
                if self.family == "float":
                    emit(O.FMA if rng.random() < 0.5 else O.Select)
                else:
                    emit(O.Pop)
        # flush: fold what is left on the stack and in the registers into the outputs
        fold = O.FAdd if self.family == "float" else O.IXor
        for r in sorted(regs_written):
            if depth < self.max_depth:
                emit(O.LOAD_REGS[r])
                if depth >= 2:
                    emit(fold)
        while depth >= 2:
            emit(fold)
        if depth == 1:
            emit(st, N_IN + (out_next % N_OUT))
        bc.append([O.Halt, 0])
        return ProgramData(np.array(bc, dtype=np.int32).reshape(-1), self._infos())
