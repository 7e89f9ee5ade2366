"""Opcode numbering and stack effects of the gint bytecode format.

The bytecode format is the contract with the unchanged gint frontend and conductor: a stream of
int32 pairs ``[opcode, operand]`` terminated by opcode 0 (``gint/kernel/interpreter/main.py:61-168``
for the numbering, ``gint/host/analyzer.py:24-135`` for the stack effects). The numbers below are
checked against a dump of the reference's own tables in ``gint_b200/data/opcodes.json``.

The same table exists three times in this repository on purpose, each written independently and
cross-checked by tests: here (host Python), in ``gint_b200/csrc/gint_opcodes.h`` (the C-ABI library's
pre-decoder) and in ``oracle/gint_oracle.c`` (the CPU checker).
"""
from __future__ import annotations

REG_WIDTH = 4            # values per thread per stack slot ("width lanes")
WARP_SIZE = 32
MAX_N_TENSORS = 8
MAX_STACK = 8
NUM_REGS = 8
TILE_ELEMS = WARP_SIZE * REG_WIDTH

# (name, min stack depth before, net stack effect)
_TABLE = [
    ("Halt", 0, 0), ("Nop", 0, 0),
    ("FAdd", 2, -1), ("FMul", 2, -1), ("FMA", 3, -2), ("FSub", 2, -1), ("FRSub", 2, -1), ("FNeg", 1, 0),
    ("FDiv", 2, -1), ("FRDiv", 2, -1), ("FRem", 2, -1),
    ("LoadImm", 0, 1), ("FAddImm", 1, 0), ("FMulImm", 1, 0), ("FMAImm", 1, 0),
    ("LoadGlobal1DF32", 0, 1), ("StoreGlobal1DF32", 1, -1), ("LoadGlobal1DF16", 0, 1), ("StoreGlobal1DF16", 1, -1),
    ("LoadGlobal1DBF16", 0, 1), ("StoreGlobal1DBF16", 1, -1), ("LoadGlobal1DU8", 0, 1),
    ("Pop", 1, -1), ("Pop2", 2, -2), ("Dup", 1, 1), ("DupX1", 2, 1), ("DupX2", 3, 1), ("Dup2", 2, 2),
    ("FGt", 2, -1), ("FLt", 2, -1), ("FGe", 2, -1), ("FLe", 2, -1), ("FEq", 2, -1), ("FNe", 2, -1),
    ("FApprox", 2, -1), ("Select", 3, -2),
    ("WarpAllReduceSum", 1, 0), ("WarpAllReduceMax", 1, 0), ("WarpAllReduceMin", 1, 0), ("WarpAllReduceProd", 1, 0),
    ("FSqrt", 1, 0), ("FSin", 1, 0), ("FCos", 1, 0), ("FTan", 1, 0), ("FArcSin", 1, 0), ("FArcCos", 1, 0),
    ("FArcTan", 1, 0), ("FArcTan2", 2, -1), ("FPow", 2, -1), ("FExp", 1, 0), ("FExp2", 1, 0), ("FLog", 1, 0),
    ("FLog2", 1, 0), ("FRSqrt", 1, 0), ("FErf", 1, 0),
    ("Swap", 2, 0),
    ("IAdd", 2, -1), ("IMul", 2, -1), ("ISub", 2, -1), ("IDiv", 2, -1), ("IRem", 2, -1), ("IShl", 2, -1),
    ("IShr", 2, -1), ("IAnd", 2, -1), ("IOr", 2, -1), ("IXor", 2, -1),
    ("LoadGlobal1DF32Indirect", 1, 0), ("StoreGlobal1DF32Indirect", 2, -2),
    ("LoadImm4F", 0, 1), ("LoadImm4I", 0, 1),
    ("LoadGlobal2DTF32", 0, 1), ("StoreGlobal2DTF32", 1, -1), ("LoadGlobal2DTF16", 0, 1), ("StoreGlobal2DTF16", 1, -1),
    ("LoadGlobal2DTBF16", 0, 1), ("StoreGlobal2DTBF16", 1, -1), ("LoadGlobal2DTU8", 0, 1),
    ("LoadGlobal2DWF32", 0, 1), ("StoreGlobal2DWF32", 1, -1), ("LoadGlobal2DWF16", 0, 1), ("StoreGlobal2DWF16", 1, -1),
    ("LoadGlobal2DWBF16", 0, 1), ("StoreGlobal2DWBF16", 1, -1), ("LoadGlobal2DWU8", 0, 1),
    ("AdvanceBlock2D", 0, 0), ("AdvanceBase", 0, 0), ("DupBroadcastW", 1, 1),
] + [(f"FLoadReg{n}", 0, 1) for n in range(NUM_REGS)] + [(f"FStoreReg{n}", 1, -1) for n in range(NUM_REGS)] + [
    ("FRcp", 1, 0), ("FPermW", 1, 0), ("FShuf2", 2, -1),
]

NAMES: list[str] = [t[0] for t in _TABLE]
OPCODES: dict[str, int] = {name: i for i, name in enumerate(NAMES)}
STACK_EFFECTS: dict[int, tuple[int, int]] = {i: (t[1], t[2]) for i, t in enumerate(_TABLE)}
N_OPCODES = len(_TABLE)

FLOAD_REG_BASE = OPCODES["FLoadReg0"]
FSTORE_REG_BASE = OPCODES["FStoreReg0"]

# module-level constants Halt, Nop, FAdd, ... so programs can be written with symbolic opcodes
globals().update(OPCODES)
LOAD_REGS = [FLOAD_REG_BASE + n for n in range(NUM_REGS)]
STORE_REGS = [FSTORE_REG_BASE + n for n in range(NUM_REGS)]

__all__ = ["REG_WIDTH", "WARP_SIZE", "MAX_N_TENSORS", "MAX_STACK", "NUM_REGS", "TILE_ELEMS", "NAMES", "OPCODES",
           "STACK_EFFECTS", "N_OPCODES", "LOAD_REGS", "STORE_REGS"] + NAMES
