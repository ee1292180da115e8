"""ctypes binding of ``libtileops_b200.so`` (the C ABI declared in ``include/tileops_b200.h``).

There is no fallback: if the library has not been built, importing a kernel raises.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_lib", "libtileops_b200.so")


def use_library(path: str) -> None:
    """Load another build of the same library instead of the in-tree one (comparing kernel variants).
    Must be called before the first kernel call."""
    global _LIB_PATH, _lib
    _LIB_PATH, _lib = path, None

OK = 0
F16, BF16, E4M3, F32 = 0, 1, 2, 3
# variant flags of tb200_gqa_decode (TB200_DECODE_* in include/tileops_b200.h)
DECODE_WIDE_ON, DECODE_WIDE_OFF, DECODE_FP8_MMA, DECODE_NO_TMA = 1, 2, 4, 8
DECODE_CHUNK_TILES_SHIFT = 8
PREFILL_TWO_TILES = 1


def prefill_flags(config: "dict | None") -> int:
    """Variant flags of the prefill entry points from a kernel ``config`` dict: ``tiles_per_cta`` 2 asks for
    the kernel with two Q tiles per CTA (head dim 128, dense); 1, the default, is the kernel with one."""
    if config and int(config.get("tiles_per_cta") or 1) == 2:
        return PREFILL_TWO_TILES
    return 0


def decode_flags(config: "dict | None") -> int:
    """Variant flags from a kernel ``config`` dict: ``wide`` (True / False / absent = the library's
    choice), ``fp8_mma``, ``tma`` (False keeps the cp.async kernel), ``chunk_tiles`` (fixed split-KV
    run length in 64-token tiles)."""
    if not config:
        return 0
    flags = 0
    wide = config.get("wide")
    if wide is not None:
        flags |= DECODE_WIDE_ON if wide else DECODE_WIDE_OFF
    if config.get("fp8_mma"):
        flags |= DECODE_FP8_MMA
    if config.get("tma") is False:
        flags |= DECODE_NO_TMA
    chunk = int(config.get("chunk_tiles") or 0)
    if not 0 <= chunk <= 0xFFFF:
        raise ValueError(f"chunk_tiles={chunk} is outside [0, 65535]")
    return flags | (chunk << DECODE_CHUNK_TILES_SHIFT)

_DTYPE_CODE = {torch.float16: F16, torch.bfloat16: BF16, torch.float32: F32}
if hasattr(torch, "float8_e4m3fn"):
    _DTYPE_CODE[torch.float8_e4m3fn] = E4M3

#: every symbol ``include/tileops_b200.h`` declares: (restype, argtypes)
SIGNATURES = {
    "tb200_last_error": (c_char_p, []),
    "tb200_version": (c_int, []),
    "tb200_gqa_decode_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int]),
    "tb200_gqa_decode": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,      # q k v o lse
        c_void_p, c_int32, c_void_p, c_int32,                  # lens uniform bt bt_stride
        c_void_p, c_void_p,                                    # k_scale v_scale
        c_int, c_int, c_int,                                   # q/kv/o dtype
        c_int, c_int, c_int, c_int, c_int,                     # batch heads heads_kv dim page
        c_int64, c_int64, c_int64,                             # strides
        c_float, c_float, c_int64, c_int,                      # sm_scale softcap kv_pool_tokens flags
        c_void_p, c_size_t, c_void_p]),                        # workspace bytes stream
    "tb200_gqa_decode_noalloc": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
        c_void_p, c_int32, c_void_p, c_int32,
        c_void_p, c_void_p,
        c_int, c_int, c_int,
        c_int, c_int, c_int, c_int, c_int,
        c_int64, c_int64, c_int64,
        c_float, c_float,
        c_void_p]),                                            # stream (no workspace arguments)
    "tb200_gqa_decode_sharded": (c_int, [
        c_void_p, c_void_p, c_void_p,                          # q k v
        c_void_p, c_int32, c_void_p, c_int32,                  # lens uniform bt bt_stride
        c_void_p, c_void_p, c_int, c_int,                      # k_scale v_scale q/kv dtype
        c_int, c_int, c_int, c_int, c_int,                     # batch heads heads_kv dim page
        c_int64, c_int64, c_int64, c_float, c_float,           # strides sm_scale softcap
        c_int64, c_int,                                        # kv_pool_tokens flags
        c_void_p, c_void_p, c_void_p, c_int, c_int,            # peer_buffers peer_flags step_counter world rank
        c_void_p, c_size_t, c_void_p]),                        # workspace bytes stream
    "tb200_gqa_lse_merge_wait": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int, c_int64, c_int64, c_int64, c_int,
        c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),     # flags step_counter status wait_cycles stream
    "tb200_gqa_lse_merge": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64, c_int,
                                    c_int64, c_int64, c_int, c_void_p]),
    "tb200_gqa_prefill_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, c_int]),
    "tb200_gqa_prefill": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,      # q k v o lse
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int,  # dtype B Sq Skv H Hkv D causal
        c_float, c_float, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),   # sm_scale softcap win_l win_r flags ws bytes stream
    "tb200_gqa_prefill_paged": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # q k_new v_new k_pages v_pages o lse
        c_void_p, c_void_p, c_void_p, c_void_p, c_int64,        # cu_seqlens_q cu_seqlens_kv cache_seqlens block_table stride
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int,  # dtype total_q total_kv B maxq H Hkv D page pool causal
        c_float, c_float, c_int, c_int, c_int, c_void_p, c_size_t, c_void_p]),
    "tb200_gqa_prefill_paged_e4m3_cache": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,  # q k_new v_new k_pages v_pages k_scale v_scale o lse
        c_void_p, c_void_p, c_void_p, c_int64,                  # cu_seqlens_q cache_seqlens block_table stride
        c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int64, c_int,  # dtype total_q B maxq H Hkv D page pool causal
        c_float, c_float, c_void_p, c_size_t, c_void_p]),
    "tb200_rope_neox_packed": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,      # x y cos sin cu_seqlens_q cache_seqlens
        c_int, c_int, c_int, c_int, c_int, c_int, c_int,              # dtype tokens B H D rotary_dim max_position
        c_void_p, c_void_p]),                                        # status stream
    "tb200_fp8_cache_gather": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,      # k_pages v_pages k_new v_new k_out v_out
        c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,  # cu_q cu_kv cache bt stride k_scale v_scale
        c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),          # dtype total_kv B Hkv D page stream
    "tb200_mma_issue_probe": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p]),
    "tb200_gqa_decode_last_kernel": (c_int, []),
    "tb200_fp8_cache_append": (c_int, [
        c_void_p, c_void_p, c_void_p, c_void_p,                         # k_new v_new k_pages v_pages
        c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p,      # cu_q cache bt stride k_scale v_scale
        c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]),          # dtype total_q B Hkv D page stream
}

_lib = None


class NativeLibraryError(RuntimeError):
    """The CUDA library is missing or a call into it failed."""


def lib() -> ctypes.CDLL:
    """Load the shared library once; raise if it is not there."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise NativeLibraryError(
                f"{_LIB_PATH} not found: build it with `python -m tileops_b200.build` "
                "(there is no CPU or eager fallback)")
        handle = ctypes.CDLL(_LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"dtype {dtype} has no kernel") from None


def check(status: int, what: str) -> None:
    if status != OK:
        msg = lib().tb200_last_error().decode(errors="replace")
        if status in (1, 2):
            raise ValueError(f"{what}: {msg}")
        raise NativeLibraryError(f"{what} failed with status {status}: {msg}")


def ptr(t: "torch.Tensor | None") -> "int | None":
    return None if t is None else t.data_ptr()


def current_stream(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream
