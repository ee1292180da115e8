"""Target-plugin protocol of TileOPs (``src/tileops/backend/__init__.py:38-69`` in the reference): a
third-party distribution registers a device detector and one ``build_kernel`` per op under a target name.

When a TileOPs installation is importable, this package IS ``tileops.backend``: its ``registry``,
``dispatch``, ``protocol`` and ``errors`` submodules are aliased to the installed ones, so the operators of
this package and the operators of that installation share one registry and one default target.  Without
one (this repository's tests, a GPU box with only this package), condensed private copies of the same four
modules serve.
"""

import sys as _sys

try:
    import tileops.backend as _installed
    from tileops.backend import dispatch, errors, protocol, registry
except Exception:  # noqa: BLE001 - no TileOPs installation (or one that does not import here)
    _installed = None

if _installed is not None:
    for _name, _mod in (("dispatch", dispatch), ("errors", errors), ("protocol", protocol), ("registry", registry)):
        _sys.modules[__name__ + "." + _name] = _mod
else:
    from . import dispatch, errors, protocol, registry  # noqa: F401

#: True when the registry in use belongs to an installed TileOPs
USES_INSTALLED_TILEOPS = _installed is not None

from .dispatch import default_target, load_failures, registered_targets, set_default_target  # noqa: E402
from .errors import AmbiguousTargetError, BackendError, OpNotAvailableError, UnknownTargetError  # noqa: E402
from .protocol import BUILTIN, BuildKernel, KernelResult, Target, TensorSpec  # noqa: E402
from .registry import register_detector, register_kernel_builder  # noqa: E402

__all__ = [
    "BUILTIN", "AmbiguousTargetError", "BackendError", "BuildKernel", "KernelResult",
    "OpNotAvailableError", "Target", "TensorSpec", "UnknownTargetError", "default_target",
    "load_failures", "register_detector", "register_kernel_builder", "registered_targets",
    "set_default_target", "USES_INSTALLED_TILEOPS",
]
