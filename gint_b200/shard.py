"""Sharding a program over several GPUs by its independent leading dimension (no collective).

Every logical program of a gint launch is independent, so rank r of N can run a contiguous range of the logical grid on
its own device: ``gint_execute_range(first, count)`` with base pointers *biased* so that the addresses the full-size
program computes for logical program ``first`` land at the start of the rank's local buffers. The bias per tensor is the
byte offset the descriptor decode assigns to logical program ``first`` (zero for broadcast operands such as a weight
vector, which are replicated instead of sharded).

The offset rule restates the device-side decode (reference: ``gint/kernel/interpreter/instructions/load_tensor_infos.py:23-40``):
``b1 = i % gd1; i //= gd1; b2 = i % gd2; i //= gd2; off = b1*step1*stride1 + b2*step2*stride2 + sum_j bstride[j] * (i % bshape[j])``
with batch dims taken innermost first.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

from .host.executor import ProgramTensorInfo

U32 = 0xFFFFFFFF


def shard_range(grid_dim: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced split of ``grid_dim`` logical programs: returns (first, count) of ``rank``."""
    if not 0 <= rank < world:
        raise ValueError("rank out of range")
    base, extra = divmod(grid_dim, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def element_offset(info: ProgramTensorInfo, index: int) -> int:
    """Element offset of logical program ``index`` from the tensor's base pointer (32-bit unsigned arithmetic)."""
    r = index & U32
    gd1, gd2 = info.block_grid_dims
    b1 = r % gd1 if gd1 else 0
    r = r // gd1 if gd1 else 0
    b2 = r % gd2 if gd2 else 0
    r = r // gd2 if gd2 else 0
    off = b1 * info.block_grid_steps[0] * info.block_shape_stride_1[1] + b2 * info.block_grid_steps[1] * info.block_shape_stride_2[1]
    for stride, extent in zip(reversed(info.batch_strides), reversed(info.batch_shape)):
        idx = r % extent if extent else 0
        r = r // extent if extent else 0
        off += stride * idx
    return off & U32


@dataclass
class ShardPlan:
    first: int
    count: int
    byte_bias: list[int]      # per descriptor slot: subtract from the local buffer's address to get the base pointer to pass

    def biased(self, local_ptrs: Sequence[int]) -> list[int]:
        return [p - b for p, b in zip(local_ptrs, self.byte_bias)]


def plan_shard(infos: Sequence[ProgramTensorInfo], grid_dim: int, world: int, rank: int) -> ShardPlan:
    """Range and pointer biases for ``rank``. A tensor whose offset at ``first`` is zero is treated as replicated."""
    first, count = shard_range(grid_dim, world, rank)
    return ShardPlan(first, count, [element_offset(t, first) * t.elm_size for t in infos])
