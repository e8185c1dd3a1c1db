"""B200-native kernels for CINN's fused op groups behind the CINN runtime ABI."""
from ._lib import CinnB200Error, lib  # noqa: F401
from .runtime import FusedGroup  # noqa: F401
from . import common, frontend  # noqa: F401,E402
