"""sm_100a kernel classes for GQA decode (L1 of the operator stack).

Drop-in replacements, by ``kernel_map`` slot, for the reference's TileLang classes:
``GQADecodeKernel`` (``src/tileops/kernels/attention/gqa_decode.py:415-615``) and
``GQADecodePagedKernel`` (``src/tileops/kernels/attention/gqa_decode_paged.py:514-746``).
Constructor and ``forward`` signatures are the reference's, so the same classes can be handed
to a stock TileOPs op through ``kernel_map=``.  All three call one CUDA kernel through the
C ABI (``tb200_gqa_decode``); there is no host synchronisation and no per-call allocation
besides the output.
"""

from __future__ import annotations

from typing import Optional

import torch

from .. import functional as F
from .call_spec import ATTENTION_DTYPES, fp8_dtype
from .kernel_base import Kernel

__all__ = [
    "GQADecodeSm100Kernel",
    "GQADecodePagedSm100Kernel",
    "GQADecodePagedFp8Sm100Kernel",
    "gqa_decode_paged_block_ns",
]

_SUPPORTED_DIMS = (64, 128)
_TILE = 64  # tokens per shared-memory tile of the CUDA kernel


def gqa_decode_paged_block_ns(page_size: int) -> tuple:
    """Token-tile heights that never straddle a page, widest first.

    Same admission rule as the reference (``gqa_decode_paged.py:21-33``): pages that are a
    multiple of 64 tokens, or shorter than 64.  The CUDA kernel itself addresses every row
    through the block table and could serve any page size; the rule is kept so that a page
    layout the reference rejects is rejected here with the same error.
    """
    if page_size <= 0:
        raise ValueError("page_size must be positive")
    if page_size % _TILE == 0:
        return (_TILE,)
    if page_size < _TILE:
        return (page_size,)
    raise ValueError(f"page_size={page_size} matches no supported block_N")


class _DecodeBase(Kernel):
    supported_archs = [100]
    general = True

    @classmethod
    def applies(cls, call) -> bool:
        return call.dim in _SUPPORTED_DIMS and call.dtype in ATTENTION_DTYPES

    def _common_init(self, batch, heads, heads_kv, seqlen_kv, dim, dtype, sm_scale, softcap, tune):
        if heads % heads_kv != 0:
            raise ValueError("heads must be divisible by heads_kv")
        if dim not in _SUPPORTED_DIMS:
            raise ValueError(f"{type(self).__name__} supports head dims {_SUPPORTED_DIMS}, got {dim}")
        self.batch, self.heads, self.heads_kv = batch, heads, heads_kv
        self.seqlen_kv, self.dim, self.dtype = seqlen_kv, dim, dtype
        self.groups = heads // heads_kv
        self.sm_scale = dim ** -0.5 if sm_scale is None else sm_scale
        self.softcap = 0.0 if softcap is None else softcap
        self.tune = tune

    @property
    def default_config(self) -> dict:
        """``block_N`` / ``threads`` / ``num_stages`` / ``num_split`` describe the compiled kernel (the
        reference's tunables, ``gqa_decode.py:520-553``; fixed here).  The entries a caller may set through
        ``config=`` select a compiled variant and travel to the library as flags, never as environment
        variables: ``wide`` (True / False / None = the library's choice: 3 CTAs per SM with a 2-stage ring
        for long 16-bit contexts), ``tma`` (False keeps the cp.async kernel where the TMA-producer kernel
        would apply), ``fp8_mma`` (e4m3 tensor-core path of an FP8 cache), ``chunk_tiles`` (fixed split-KV
        run length in 64-token tiles; 0 = the device-side cost model)."""
        return {"block_N": _TILE, "threads": 128, "num_stages": 3, "num_split": "device-balanced",
                "wide": None, "tma": True, "fp8_mma": False, "chunk_tiles": 0}


class GQADecodeSm100Kernel(_DecodeBase):
    """Contiguous-cache decode: ``forward(Q[B,H,D], K[B,S,Hkv,D], V, real_seqlen_kv:int)``."""

    def __init__(self, batch, heads, heads_kv, seqlen_kv, dim, dtype, sm_scale=None, softcap=0.0,
                 config: Optional[dict] = None, tune: bool = False, device_index=None) -> None:
        super().__init__(device_index=device_index)
        self._common_init(batch, heads, heads_kv, seqlen_kv, dim, dtype, sm_scale, softcap, tune)
        self.init_config(config, tune)

    def forward(self, Q: torch.Tensor, K: torch.Tensor, V: torch.Tensor, real_seqlen_kv: int,
                return_lse: bool = False):
        self._require_cuda(Q=Q, K=K, V=V)
        return F.gqa_decode(Q, K, V, real_seqlen_kv=int(real_seqlen_kv), sm_scale=self.sm_scale,
                            softcap=self.softcap, return_lse=return_lse, config=self.config)


class GQADecodePagedSm100Kernel(_DecodeBase):
    """Paged decode: ``forward(Q[B,H,D], K[N,Hkv,D], V, real_seqlen_kv[B] i32, block_table[B,W] i32)``."""

    def __init__(self, batch, heads, heads_kv, seqlen_kv, dim, page_size, dtype, sm_scale=None,
                 softcap=0.0, config: Optional[dict] = None, tune: bool = False, device_index=None) -> None:
        super().__init__(device_index=device_index)
        self._common_init(batch, heads, heads_kv, seqlen_kv, dim, dtype, sm_scale, softcap, tune)
        if seqlen_kv % page_size != 0:
            raise ValueError(f"seqlen_kv={seqlen_kv} must be a multiple of page_size={page_size}")
        self.page_size = page_size
        self._block_ns = gqa_decode_paged_block_ns(page_size)
        self.autotune_configs = [{"block_N": n} for n in self._block_ns]
        self.init_config(config, tune)
        self.config["block_N"] = self._block_ns[0]

    def forward(self, Q, K, V, real_seqlen_kv: torch.Tensor, block_table: torch.Tensor,
                return_lse: bool = False, out_dtype=None):
        self._require_cuda(Q=Q, K=K, V=V, real_seqlen_kv=real_seqlen_kv, block_table=block_table)
        return F.gqa_decode(Q, K, V, real_seqlen_kv=real_seqlen_kv, block_table=block_table,
                            page_size=self.page_size, sm_scale=self.sm_scale, softcap=self.softcap,
                            return_lse=return_lse, out_dtype=out_dtype, config=self.config)


class GQADecodePagedFp8Sm100Kernel(GQADecodePagedSm100Kernel):
    """Paged decode over an e4m3 cache with fp32 scales per (page, KV head):
    ``forward(Q, K_fp8, V_fp8, k_scale[P,Hkv], v_scale[P,Hkv], real_seqlen_kv, block_table)``.
    No reference counterpart (the reference has FP8 caches only in paged *prefill*, with one
    scalar scale, ``src/tileops/kernels/attention/gqa_fwd.py:1005-1305``)."""

    def forward(self, Q, K, V, k_scale, v_scale, real_seqlen_kv, block_table,
                return_lse: bool = False, out_dtype=None):
        self._require_cuda(Q=Q, K=K, V=V, k_scale=k_scale, v_scale=v_scale,
                           real_seqlen_kv=real_seqlen_kv, block_table=block_table)
        if K.dtype != fp8_dtype() or V.dtype != fp8_dtype():
            raise ValueError("K and V must be torch.float8_e4m3fn")
        return F.gqa_decode(Q, K, V, real_seqlen_kv=real_seqlen_kv, block_table=block_table,
                            page_size=self.page_size, k_scale=k_scale, v_scale=v_scale,
                            sm_scale=self.sm_scale, softcap=self.softcap, return_lse=return_lse,
                            out_dtype=out_dtype, config=self.config)
