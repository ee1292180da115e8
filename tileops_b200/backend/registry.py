"""Process-wide tables of target detectors and kernel builders.

Condensed from ``src/tileops/backend/registry.py:42-194`` of the reference (same globals, functions and
messages, so that this package runs without a TileOPs installation; when ``tileops.backend`` is
importable the package uses that one instead, see ``backend/__init__.py``).  The contract: one detector
per target, one builder per ``(op, target)``, duplicates are an error, plugins are discovered
from the ``tileops.backends`` entry-point group exactly once, and a plugin that fails to
import is recorded and skipped rather than fatal.
"""

from __future__ import annotations

import threading
import traceback
import warnings
from importlib.metadata import entry_points
from typing import Callable, NamedTuple

from .errors import BackendError
from .protocol import BuildKernel, DetectFn, Target

ENTRY_POINT_GROUP = "tileops.backends"

DETECTORS: dict = {}
BUILDERS: dict = {}
LOAD_FAILURES: list = []
default_target: Target = None
_loaded = False
LOCK = threading.RLock()
_LOADING = threading.local()


def describe(fn: Callable) -> str:
    return f"{getattr(fn, '__module__', '?')}.{getattr(fn, '__qualname__', fn)}"


def register_detector(target: str, detect: DetectFn) -> None:
    """Record how *target* recognises its devices. A second detector for it is an error."""
    with LOCK:
        if target in DETECTORS:
            raise BackendError(
                f"target {target!r} already has detector {describe(DETECTORS[target])}; "
                f"{describe(detect)} cannot replace it.")
        DETECTORS[target] = detect


def register_kernel_builder(op: str, target: str, build_kernel: BuildKernel) -> None:
    """Record how *target* builds a kernel for *op* (manifest key). Duplicates are an error."""
    with LOCK:
        if (op, target) in BUILDERS:
            raise BackendError(
                f"{(op, target)} is already registered to {describe(BUILDERS[(op, target)])}; "
                f"{describe(build_kernel)} cannot take it.")
        BUILDERS[(op, target)] = build_kernel


def known_targets() -> set:
    return set(DETECTORS) | {t for _, t in BUILDERS}


class RegistryState(NamedTuple):
    detectors: dict
    builders: dict
    load_failures: list
    default_target: Target
    loaded: bool


def snapshot() -> RegistryState:
    with LOCK:
        return RegistryState(dict(DETECTORS), dict(BUILDERS), list(LOAD_FAILURES), default_target, _loaded)


def restore(state: RegistryState) -> None:
    global default_target, _loaded
    with LOCK:
        DETECTORS.clear(); DETECTORS.update(state.detectors)
        BUILDERS.clear(); BUILDERS.update(state.builders)
        LOAD_FAILURES[:] = state.load_failures
        default_target = state.default_target
        _loaded = state.loaded


def _load_all() -> list:
    failed = []
    for ep in sorted(entry_points(group=ENTRY_POINT_GROUP), key=lambda e: (e.name, e.value)):
        checkpoint = snapshot()
        try:
            ep.load()
        except Exception as exc:  # noqa: BLE001 - a broken plugin must not take the process down
            restore(checkpoint)
            reason = "".join(traceback.format_exception_only(type(exc), exc)).strip()
            failure = f"{ep.name} ({ep.value}): {reason}"
            LOAD_FAILURES.append(failure)
            failed.append(failure)
        except BaseException:
            restore(checkpoint)
            raise
    return failed


def ensure_loaded() -> None:
    """Import every declared plugin module, once per process."""
    global _loaded
    if _loaded or getattr(_LOADING, "active", False):
        return
    with LOCK:
        if _loaded:
            return
        _LOADING.active = True
        try:
            failed = _load_all()
            _loaded = True
        finally:
            _LOADING.active = False
    for failure in failed:
        warnings.warn(f"backend failed to load and was skipped: {failure}", RuntimeWarning, stacklevel=3)


def load_failure_suffix() -> str:
    return f" ({len(LOAD_FAILURES)} backend(s) failed to load)" if LOAD_FAILURES else ""
