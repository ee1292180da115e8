"""Cached device facts (condensed from ``src/tileops/utils/utils.py:19-53`` of the reference)."""

import functools

import torch

#: architecture reported when no CUDA device can be queried (construction and selection must
#: still work on a CPU-only host; launching does not)
NO_DEVICE_ARCH = 0


@functools.lru_cache(maxsize=16)
def _sm_version(index: int) -> int:
    major, minor = torch.cuda.get_device_capability(index)
    return major * 10 + minor


@functools.lru_cache(maxsize=16)
def _sm_count(index: int) -> int:
    return torch.cuda.get_device_properties(index).multi_processor_count


def get_sm_version(index=None) -> int:
    """``major*10 + minor`` of the device (current by default); 0 without a CUDA device."""
    if not torch.cuda.is_available():
        return NO_DEVICE_ARCH
    return _sm_version(torch.cuda.current_device() if index is None else index)


def get_sm_count(index=None) -> int:
    if not torch.cuda.is_available():
        return 0
    return _sm_count(torch.cuda.current_device() if index is None else index)


def is_h200(index=None) -> bool:
    if not torch.cuda.is_available():
        return False
    i = torch.cuda.current_device() if index is None else index
    return "H200" in torch.cuda.get_device_name(i).upper()


def forget_device_properties() -> None:
    _sm_version.cache_clear()
    _sm_count.cache_clear()
