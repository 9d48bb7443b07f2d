"""pypto_b200: B200 (sm_100a) kernels for the fused operators of pypto's model examples,
behind pypto's program / launch surface.  See ``include/pypto_b200.h`` for the C ABI."""

from ._lib import BackendUnavailable, PtoError  # noqa: F401

__version__ = "0.1.0"
