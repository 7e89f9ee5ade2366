"""Batched execution of candidate programs: the executor side of a bytecode superoptimizer.

Mirror of ``BatchRunner`` in the reference's example application (``examples/superopt/executor.py:61-186``): many short programs
that share their input tensors and write one output row each are run by ONE launch. There the batch is assembled in Python --
a 608-byte descriptor block is packed per candidate, bytecode, blocks and two pointer tables are uploaded with four
allocations, and the reference's own kernel is launched through its raw handle (``geval_func_handle``), which ties the caller to
that kernel's ABI. Here the same call is one library entry point, ``gint_execute_batch``: candidates are analysed and pre-decoded
in C, one descriptor block is shared by all of them and the per-candidate output pointer travels in the launch table.

    runner = BatchRunner(n_inputs=2, test_size=128)
    out = runner.run(bytecodes, [a, b], output_buffer)      # bytecodes: int32 [N, words]; out = output_buffer[:N]
    runner.last_status                                      # int32 [N]: 0, or the negative gint status of a skipped candidate
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy
import torch

from .host import capi
from .host.executor import B200Executor, ProgramTensorInfo, get_executor
from .host.utils import fill_tensor_info


def contiguous_f32_info(test_size: int) -> ProgramTensorInfo:
    """Descriptor of a 1-D contiguous f32 tensor of ``test_size`` elements seen by one logical program
    (``examples/superopt/executor.py:36-46``)."""
    return ProgramTensorInfo(elm_size=4, batch_strides=[], batch_shape=[], block_shape_stride_1=[test_size, 1], block_shape_stride_2=[1, 0],
                             block_grid_dims=[1, 1], block_grid_steps=[test_size, 0])


class BatchRunner:
    """Run many candidate programs that share ``n_inputs`` input tensors and each write one row of an output buffer.
    Slot order of every candidate: the inputs, then the output."""

    def __init__(self, n_inputs: int, test_size: int = 128, executor: Optional[B200Executor] = None) -> None:
        self.n_inputs, self.test_size, self.n_tensors = n_inputs, test_size, n_inputs + 1
        self._ex = executor or get_executor()
        self._ti = capi.HTensorInfo()
        fill_tensor_info(self._ti, [contiguous_f32_info(test_size)] * self.n_tensors)
        self.last_status: Optional[numpy.ndarray] = None

    def run(self, bytecodes_np: numpy.ndarray, input_tensors: Sequence[torch.Tensor], output_buffer: torch.Tensor, cuda_stream: int = 0) -> torch.Tensor:
        """``bytecodes_np``: int32 [N, words], complete programs; ``output_buffer``: device tensor [>= N, test_size] whose rows
        0..N-1 receive the candidates' outputs (rows of skipped candidates are left as they are). Asynchronous."""
        n, words = bytecodes_np.shape
        if n == 0:
            return output_buffer[:0]
        if len(input_tensors) != self.n_inputs:
            raise ValueError("Number of arguments don't match the program.")
        if output_buffer.shape[0] < n or output_buffer.shape[-1] != self.test_size or not output_buffer.is_contiguous():
            raise ValueError("output_buffer must be contiguous with at least N rows of test_size elements")
        codes = numpy.ascontiguousarray(bytecodes_np, dtype=numpy.int32)
        ptrs = (ctypes.c_uint64 * capi.MAX_N_TENSORS)(*[t.data_ptr() for t in input_tensors], output_buffer.data_ptr())
        status = numpy.zeros(n, dtype=numpy.int32)
        _, ctx = self._ex._ctx()
        rc = self._ex._lib.gint_execute_batch(ctx, codes.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), n, words, ctypes.byref(self._ti),
                                              self.n_tensors, ptrs, self.n_inputs, self.test_size * 4,
                                              status.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)), cuda_stream)
        self._ex._check(ctx, rc, "gint_execute_batch")
        self._ex.launches += 1
        self.last_status = status
        return output_buffer[:n]
