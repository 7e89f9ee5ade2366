"""``@bytecode``: turn a Python function that calls frontend emitters into an executable program
(mirror of ``gint/host/sugar.py``)."""
from __future__ import annotations

import functools
from typing import Callable, Hashable, Optional

import numpy

from .executor import BaseExecutableProgram, ProgramData, TensorInterface
from .frontend import FrontendState, _frontend_state


class SugarProgram(BaseExecutableProgram):
    """Records the decorated function once per cache key; the recording is the program."""

    def __init__(self, func: Callable, cache_policy_fn: Optional[Callable[..., Hashable]] = None) -> None:
        super().__init__()
        self.func = func
        self.cache_policy_fn = cache_policy_fn
        functools.update_wrapper(self, func)

    def cache_policy(self, *args: TensorInterface, **extra_kwargs) -> Hashable:
        if self.cache_policy_fn is not None:
            return self.cache_policy_fn(*args, **extra_kwargs)
        return super().cache_policy(*args, **extra_kwargs)

    def record(self, *args: TensorInterface, **extra_kwargs) -> FrontendState:
        state = FrontendState(args)
        token = _frontend_state.set(state)
        try:
            self.func(*args, REGW=self.REGW, WARP=self.executor_warp_size(), **extra_kwargs)
        finally:
            _frontend_state.reset(token)
        return state

    def get_program(self, *args: TensorInterface, **extra_kwargs) -> ProgramData:
        st = self.record(*args, **extra_kwargs)
        return ProgramData(numpy.array(st.bc, dtype=numpy.int32).reshape(-1), st.tis, st.tis_arg_ids)

    def executor_warp_size(self) -> int:
        return 32  # fixed by the bytecode format (32 lanes x 4 width values per tile); no GPU needed to record


def bytecode(func: Optional[Callable] = None, cache_policy: Optional[Callable[..., Hashable]] = None):
    """Decorator. The function receives its tensor arguments as ``TensorInterface`` plus ``REGW`` and ``WARP``."""
    if func is None:
        return functools.partial(bytecode, cache_policy=cache_policy)
    return SugarProgram(func, cache_policy)
