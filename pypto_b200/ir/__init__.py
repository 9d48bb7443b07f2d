"""``ir.compile`` and ``CompiledProgram`` (python/pypto/ir/compile.py:194-432,
python/pypto/ir/compiled_program.py:559-705, 1364-1414)."""

from .pass_manager import OptimizationStrategy  # noqa: F401
from .compiled_program import CompiledProgram, compile  # noqa: F401,A004
from .distributed_compiled_program import DistributedCompiledProgram, DistributedConfig  # noqa: F401,E402
