"""Which target serves a call; condensed from ``src/tileops/backend/dispatch.py:15-129`` of the reference
(used only when ``tileops.backend`` itself is not importable):
explicit ``target=`` first, then the process default, then detection on the first tensor's
device; ``None`` means the in-tree kernels run."""

from __future__ import annotations

import torch

from . import registry
from .errors import AmbiguousTargetError, BackendError, UnknownTargetError
from .protocol import BUILTIN, Target


def detect_target(device: torch.device):
    registry.ensure_loaded()
    claimed = []
    for target, detect in list(registry.DETECTORS.items()):
        try:
            if detect(device):
                claimed.append(target)
        except Exception as exc:
            raise BackendError(
                f"detector for target {target!r} ({registry.describe(detect)}) raised on device "
                f"{device}: {exc!r}. A detector must return False for devices it does not serve."
                f"{registry.load_failure_suffix()}") from exc
    if not claimed:
        return None
    if len(claimed) > 1:
        raise AmbiguousTargetError(
            f"device {device} is claimed by {sorted(claimed)}; pass target= to choose"
            f"{registry.load_failure_suffix()}")
    return claimed[0]


def _check_known(target: Target) -> None:
    if target is not None and target is not BUILTIN and target not in registry.known_targets():
        raise UnknownTargetError(
            f"no backend registered target {target!r}; known targets: "
            f"{sorted(registry.known_targets())}{registry.load_failure_suffix()}")


def select_target(requested: Target, device) -> Target:
    registry.ensure_loaded()
    if requested is not None:
        _check_known(requested)
        return requested
    if registry.default_target is not None:
        return registry.default_target
    if device is None:
        return None
    return detect_target(device)


def registered_kernel_builder(op: str, target: str):
    registry.ensure_loaded()
    return registry.BUILDERS.get((op, target))


def registered_targets(op=None) -> list:
    registry.ensure_loaded()
    if op is None:
        return sorted(registry.known_targets())
    return sorted(t for name, t in registry.BUILDERS if name == op)


def set_default_target(target: Target) -> None:
    registry.ensure_loaded()
    _check_known(target)
    registry.default_target = target


def default_target() -> Target:
    return registry.default_target


def load_failures() -> tuple:
    registry.ensure_loaded()
    return tuple(registry.LOAD_FAILURES)
