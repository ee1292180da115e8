"""Kernel-class protocol the op layer dispatches over.

The subset of ``tileops.kernels.kernel_base.Kernel``
(``src/tileops/kernels/kernel_base.py:47-160`` in the reference) that ``kernel_map=`` overrides
and ``Op.select_kernel_key`` rely on: ``supported_archs``, ``general``, ``applies``,
``refusal``, a ``config`` dict, ``autotune()`` and ``__call__ = forward``.  There is no JIT and
no autotuner here: the kernels are compiled ahead of time and their tunables are fixed.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any, Dict, Optional

import torch

from ..utils import get_sm_version


class Kernel(ABC):
    dtype: Optional[torch.dtype] = None
    config: Dict[str, Any]
    autotune_configs: Optional[list] = None
    #: architectures (major*10+minor) the kernel runs on; ``None`` = anywhere
    supported_archs: Optional[list] = None
    #: the implementation that serves whatever no specialised sibling claims
    general: bool = False

    def __init__(self, *args: Any, device_index: "int | None" = None, **kwargs: Any) -> None:
        self.device_index = device_index
        self._check_arch()
        self.config = {}

    @classmethod
    def applies(cls, call: Any) -> bool:
        """Whether this class serves *call* (architecture aside)."""
        return True

    @classmethod
    def refusal(cls, call: Any) -> Optional[str]:
        """Why this class cannot serve *call*, or ``None`` when it can."""
        archs = cls.supported_archs
        if archs is not None and call.arch not in archs:
            return f"built for architectures {sorted(archs)}, device reports {call.arch}"
        if not cls.applies(call):
            return "does not serve this call"
        return None

    def _check_arch(self) -> None:
        cls = type(self)
        if cls.supported_archs is None:
            return
        arch = get_sm_version(self.device_index)
        if arch not in cls.supported_archs:
            where = "the current device" if self.device_index is None else f"cuda:{self.device_index}"
            raise ValueError(
                f"{cls.__name__} is built for architectures {sorted(cls.supported_archs)}, "
                f"but {where} reports {arch}")

    def _require_cuda(self, **tensors: Optional[torch.Tensor]) -> None:
        for name, tensor in tensors.items():
            if tensor is not None and not tensor.is_cuda:
                raise ValueError(
                    f"{type(self).__name__} is a CUDA kernel; got {name} on {tensor.device}. "
                    "Another target's backend serves other devices.")

    @property
    def default_config(self) -> Dict[str, Any]:
        return {}

    def init_config(self, config: Optional[Dict[str, Any]] = None, tune: bool = False) -> None:
        self.config = dict(self.default_config)
        if config:
            self.config.update(config)

    def autotune(self) -> None:
        """Ahead-of-time kernels have nothing to tune; kept for interface parity."""

    @abstractmethod
    def forward(self, *args: Any, **kwargs: Any):
        raise NotImplementedError

    def __call__(self, *args: Any, **kwargs: Any):
        return self.forward(*args, **kwargs)
