"""Only the strategy enum of python/pypto/ir/pass_manager.py survives here: there is no pass
pipeline, programs are mapped to fused kernels."""

import enum


class OptimizationStrategy(enum.Enum):
    Default = 0
    DebugTileOptimization = 1
    TileCCEOptimization = 2
