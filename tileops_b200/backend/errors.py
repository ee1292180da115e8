"""Errors of the target-plugin layer (mirrors ``tileops.backend.errors``,
``src/tileops/backend/errors.py:1-23`` in the reference)."""


class BackendError(Exception):
    """Root of everything this layer raises."""


class UnknownTargetError(BackendError):
    """``target=`` named something nobody registered."""


class AmbiguousTargetError(BackendError):
    """Two detectors claimed one device."""


class OpNotAvailableError(BackendError):
    """The chosen target has no kernel for this op; there is no silent fall back."""
