"""Launch surface: the names user programs import from ``pypto.runtime``
(python/pypto/runtime/__init__.py of the reference): ``run``, ``RunConfig``, ``ChipWorker``,
``DeviceTensor``, ``TensorSpec``, ``validate_golden``, ``benchmark``."""

from .device_tensor import DeviceTensor, StackedDeviceTensor  # noqa: F401
from .run_config import RunConfig  # noqa: F401
from .tensor_spec import TensorSpec  # noqa: F401
from .worker import ChipWorker, RegistrationHandle  # noqa: F401
from .runner import RunResult, benchmark, BenchmarkStats, run, validate_golden  # noqa: F401
from .distributed_runner import DistributedRunHandle, DistributedWorker  # noqa: F401
from . import fused_programs  # noqa: F401
