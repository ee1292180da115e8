"""Types that cross the op/target boundary; condensed from ``src/tileops/backend/protocol.py:10-53`` of the
reference (used only when ``tileops.backend`` itself is not importable)."""

from __future__ import annotations

from typing import Callable, Final, NamedTuple, Union

import torch


class TensorSpec(NamedTuple):
    """A tensor's device, dtype and shape without its storage."""

    device: torch.device
    dtype: torch.dtype
    shape: tuple

    @staticmethod
    def of(tensor: torch.Tensor) -> "TensorSpec":
        return TensorSpec(tensor.device, tensor.dtype, tuple(tensor.shape))


KernelResult = Union[torch.Tensor, tuple, None]
BuildKernel = Callable[..., Callable[..., KernelResult]]
DetectFn = Callable[[torch.device], bool]


class _Builtin:
    __slots__ = ()

    def __repr__(self) -> str:
        return "BUILTIN"


#: Forces the in-tree kernels whatever plugins are installed; compared by identity.
BUILTIN: Final = _Builtin()
Target = Union[str, _Builtin, None]
