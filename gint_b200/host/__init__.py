from .executor import (BaseExecutor, BaseExecutableProgram, B200Executor, ProgramData, ProgramTensorInfo,  # noqa: F401
                       TensorInterface, get_executor, select_variant)
from .analyzer import analyze_bytecode, BytecodeStats  # noqa: F401
from .sugar import bytecode, SugarProgram  # noqa: F401
from .utils import cdiv  # noqa: F401
