"""Target-plugin protocol, API-compatible with ``tileops.backend``
(``src/tileops/backend/__init__.py:38-69`` in the reference): a third-party distribution
registers a device detector and one ``build_kernel`` per op under a target name."""

from .dispatch import default_target, load_failures, registered_targets, set_default_target
from .errors import AmbiguousTargetError, BackendError, OpNotAvailableError, UnknownTargetError
from .protocol import BUILTIN, BuildKernel, KernelResult, Target, TensorSpec
from .registry import register_detector, register_kernel_builder

__all__ = [
    "BUILTIN", "AmbiguousTargetError", "BackendError", "BuildKernel", "KernelResult",
    "OpNotAvailableError", "Target", "TensorSpec", "UnknownTargetError", "default_target",
    "load_failures", "register_detector", "register_kernel_builder", "registered_targets",
    "set_default_target",
]
