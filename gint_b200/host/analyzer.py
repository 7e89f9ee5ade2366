"""Static analysis of a straight-line bytecode program (mirror of ``gint/host/analyzer.py``).

The walk is done in Python here so program authors get the same ``BytecodeStats`` object and the same
``ValueError`` messages as with the reference; the C-ABI library repeats the walk on every program it is given
(``gint_analyze``) and the two are cross-checked by the tests.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Sequence, Union

import numpy

from ..opcodes import FLOAD_REG_BASE, FSTORE_REG_BASE, NUM_REGS, STACK_EFFECTS

BytecodeInput = Union[Sequence[Sequence[int]], numpy.ndarray]


@dataclass
class BytecodeStats:
    num_instructions: int      # up to, not including, the first Halt
    max_stack: int             # peak depth
    max_reg_idx: int           # highest virtual register touched, -1 if none
    regs_used: frozenset
    min_pool_size: int         # worst stack depth + (highest register seen so far + 1)


def _pairs(bc: BytecodeInput) -> Iterable[tuple[int, int]]:
    arr = numpy.asarray(bc)
    if arr.ndim == 1:
        if arr.size % 2:
            raise AssertionError("flat bytecode must have even length")
        arr = arr.reshape(-1, 2)
    for op, operand in arr:
        yield int(op), int(operand)


def analyze_bytecode(bc: BytecodeInput) -> BytecodeStats:
    depth = peak_depth = pool = n = 0
    max_reg = -1
    regs: set[int] = set()
    for op, _ in _pairs(bc):
        if op == 0:
            break
        n += 1
        if op not in STACK_EFFECTS:
            raise ValueError(f"unknown opcode {op}")
        need, net = STACK_EFFECTS[op]
        if depth < need:
            raise ValueError(f"insn {n - 1} (opcode {op}) needs depth {need}, have {depth}")
        for base in (FLOAD_REG_BASE, FSTORE_REG_BASE):
            if base <= op < base + NUM_REGS:
                regs.add(op - base)
                max_reg = max(max_reg, op - base)
        here = max(depth, depth + net)
        peak_depth = max(peak_depth, here)
        pool = max(pool, here + max_reg + 1)
        depth += net
    return BytecodeStats(n, peak_depth, max_reg, frozenset(regs), pool)


def stack_effect(opcode: int) -> tuple[int, int]:
    return STACK_EFFECTS[opcode]


def known_opcodes() -> frozenset:
    return frozenset(STACK_EFFECTS)


def select_pool_size(stats: BytecodeStats) -> int:
    """Pool geometry the B200 kernels use: 4, 7 or 12 slots (see ``gint_analyze`` in include/gint_b200.h)."""
    need = stats.max_stack + stats.max_reg_idx + 1
    return 4 if need <= 4 else 7 if need <= 7 else 12
