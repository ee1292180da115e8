"""Errors of the target-plugin layer; condensed from ``src/tileops/backend/errors.py:1-23`` of the
reference (used only when ``tileops.backend`` itself is not importable)."""


class BackendError(Exception):
    """Root of everything this layer raises."""


class UnknownTargetError(BackendError):
    """``target=`` named something nobody registered."""


class AmbiguousTargetError(BackendError):
    """Two detectors claimed one device."""


class OpNotAvailableError(BackendError):
    """The chosen target has no kernel for this op; there is no silent fall back."""
