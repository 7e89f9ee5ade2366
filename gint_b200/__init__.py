"""gint_b200: the gint GPU bytecode interpreter path, rebuilt for B200 (sm_100a).

Drop-in for the interpreter path of eliphatfs/gint: same bytecode format, same ``gint.host`` executor API
(``get_executor().execute(program, tensor_interfaces, grid_dim, cuda_stream=...)``), same ``@bytecode`` frontend.
The kernels and the launch layer are new (``gint_b200/csrc``, C ABI in ``include/gint_b200.h``).
"""
from .host.utils import cdiv
from .host.sugar import bytecode
from .host.executor import (BaseExecutableProgram, BaseExecutor, B200Executor, ProgramData, ProgramTensorInfo,
                            TensorInterface, get_executor)
from .host.analyzer import analyze_bytecode, BytecodeStats
from .dropin import install, uninstall

__version__ = "0.1.0"

__all__ = ["cdiv", "bytecode", "BaseExecutableProgram", "BaseExecutor", "B200Executor", "ProgramData", "ProgramTensorInfo",
           "TensorInterface", "get_executor", "install", "uninstall", "analyze_bytecode", "BytecodeStats", "__version__"]
