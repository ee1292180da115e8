"""Tensor-level wrappers over the C ABI: argument checks, workspace cache, launch.

These are what the kernel classes (``tileops_b200.kernels``) call.  They allocate the output
with torch, hand raw pointers and the current torch CUDA stream to the library, and never
synchronise with the device.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _native as N

# One workspace per (device, stream, problem shape).  The kernel leaves its counters zeroed, so
# the buffer is zero-filled only when it is created.  Keyed by stream because two launches that
# overlap on the GPU must not share scheduler counters, and by shape because the position of
# the counters inside the buffer depends on (batch, heads, heads_kv, dim): partial results of
# one shape would otherwise land on the counters of another.
_WORKSPACES: dict = {}


def _decode_workspace(device: torch.device, batch: int, heads: int, heads_kv: int, dim: int) -> torch.Tensor:
    need = N.lib().tb200_gqa_decode_workspace_bytes(batch, heads, heads_kv, dim)
    if need == 0:
        raise ValueError("invalid decode problem size")
    key = (device, torch.cuda.current_stream(device).cuda_stream, "decode", batch, heads, heads_kv, dim)
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


def release_workspaces() -> None:
    """Drop every cached workspace (e.g. before measuring memory)."""
    _WORKSPACES.clear()


def _require_cuda(**tensors: Optional[torch.Tensor]) -> None:
    for name, t in tensors.items():
        if t is not None and not t.is_cuda:
            raise ValueError(f"{name} must be on a cuda device, got {t.device}")


def gqa_decode(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    *,
    real_seqlen_kv: "torch.Tensor | int",
    block_table: Optional[torch.Tensor] = None,
    page_size: int = 0,
    k_scale: Optional[torch.Tensor] = None,
    v_scale: Optional[torch.Tensor] = None,
    sm_scale: Optional[float] = None,
    softcap: float = 0.0,
    out_dtype: Optional[torch.dtype] = None,
    return_lse: bool = False,
    out: Optional[torch.Tensor] = None,
    lse_out: Optional[torch.Tensor] = None,
    config: Optional[dict] = None,
) -> "torch.Tensor | Tuple[torch.Tensor, torch.Tensor]":
    """Single-token GQA decode.

    q ``[B,H,D]``; paged cache (``block_table`` given): k/v ``[N,Hkv,D]``; contiguous cache:
    k/v ``[B,S,Hkv,D]``.  ``real_seqlen_kv`` is an int32 device tensor ``[B]`` or one int for
    all sequences.  An e4m3 cache needs ``k_scale``/``v_scale`` ``[N/page,Hkv]`` fp32.
    Returns o ``[B,H,D]`` (and the log2-domain LSE ``[B,H]`` fp32 when asked).  ``out`` /
    ``lse_out`` are optional preallocated contiguous destinations (e.g. slices of a
    communication buffer).  ``config`` selects a kernel variant (see ``_native.decode_flags``).
    """
    _require_cuda(q=q, k=k, v=v, block_table=block_table, k_scale=k_scale, v_scale=v_scale)
    if q.dim() != 3:
        raise ValueError(f"q must have shape [B, H, D], got {tuple(q.shape)}")
    B, H, D = q.shape
    paged = block_table is not None
    if paged:
        if k.dim() != 3 or v.shape != k.shape or k.shape[2] != D:
            raise ValueError(f"paged k/v must have shape [N, Hkv, {D}], got {tuple(k.shape)} / {tuple(v.shape)}")
        Hkv = k.shape[1]
        if block_table.dtype != torch.int32 or block_table.dim() != 2 or block_table.shape[0] != B:
            raise ValueError("block_table must be int32 with shape [B, num_pages]")
        if page_size <= 0:
            raise ValueError("page_size must be positive")
        block_table = block_table.contiguous()
    else:
        if k.dim() != 4 or v.shape != k.shape or k.shape[0] != B or k.shape[3] != D:
            raise ValueError(f"k/v must have shape [{B}, S, Hkv, {D}], got {tuple(k.shape)} / {tuple(v.shape)}")
        Hkv = k.shape[2]
    if H % Hkv != 0:
        raise ValueError("heads must be divisible by heads_kv")
    q = q.contiguous()
    k = k.contiguous()
    v = v.contiguous()
    fp8 = k.dtype == getattr(torch, "float8_e4m3fn", None)
    if fp8:
        if k_scale is None or v_scale is None:
            raise ValueError("an float8_e4m3fn cache needs k_scale and v_scale")
        if k_scale.dtype != torch.float32 or v_scale.dtype != torch.float32:
            raise ValueError("k_scale/v_scale must be torch.float32")
        k_scale, v_scale = k_scale.contiguous(), v_scale.contiguous()
    elif k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError(f"k/v dtype {k.dtype} must equal q dtype {q.dtype} (or be float8_e4m3fn)")

    lens_t = None
    uniform = 0
    if isinstance(real_seqlen_kv, torch.Tensor):
        _require_cuda(real_seqlen_kv=real_seqlen_kv)
        if real_seqlen_kv.dtype != torch.int32 or tuple(real_seqlen_kv.shape) != (B,):
            raise ValueError("real_seqlen_kv must be int32 with shape [B]")
        lens_t = real_seqlen_kv.contiguous()
    else:
        uniform = int(real_seqlen_kv)
        if not paged and uniform > k.shape[1]:
            raise ValueError(f"real_seqlen_kv {uniform} exceeds the cache length {k.shape[1]}")

    if out is not None:
        if tuple(out.shape) != (B, H, D) or not out.is_contiguous() or out.device != q.device:
            raise ValueError("out must be a contiguous [B, H, D] tensor on q's device")
        out_dtype = out.dtype
    out_dtype = q.dtype if out_dtype is None else out_dtype
    o = torch.empty((B, H, D), dtype=out_dtype, device=q.device) if out is None else out
    if lse_out is not None:
        if tuple(lse_out.shape) != (B, H) or lse_out.dtype != torch.float32 or not lse_out.is_contiguous():
            raise ValueError("lse_out must be a contiguous float32 [B, H] tensor")
        return_lse = True
    lse = lse_out if lse_out is not None else (
        torch.empty((B, H), dtype=torch.float32, device=q.device) if return_lse else None)
    ws = _decode_workspace(q.device, B, H, Hkv, D)
    scale = D ** -0.5 if sm_scale is None else float(sm_scale)
    if paged:
        tok_stride, head_stride, batch_stride = k.stride(0), k.stride(1), 0
    else:
        tok_stride, head_stride, batch_stride = k.stride(1), k.stride(2), k.stride(0)
    with torch.cuda.device(q.device):
        st = N.lib().tb200_gqa_decode(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), N.ptr(lse),
            N.ptr(lens_t), uniform, N.ptr(block_table), block_table.shape[1] if paged else 0,
            N.ptr(k_scale) if fp8 else None, N.ptr(v_scale) if fp8 else None,
            N.dtype_code(q.dtype), N.dtype_code(k.dtype), N.dtype_code(out_dtype),
            B, H, Hkv, D, int(page_size),
            tok_stride, head_stride, batch_stride,
            scale, float(softcap or 0.0), k.shape[0] if paged else 0, N.decode_flags(config),
            ws.data_ptr(), ws.numel(), N.current_stream(q.device))
    N.check(st, "tb200_gqa_decode")
    return (o, lse) if return_lse else o


def gqa_lse_merge(o_parts: torch.Tensor, lse_parts: torch.Tensor, out_dtype: torch.dtype,
                  return_lse: bool = False):
    """o_parts ``[R, ..., D]`` fp32 and lse_parts ``[R, ...]`` fp32 (log2 domain) -> merged o.

    Each part must be contiguous; the parts themselves may be strided along dim 0 (views into
    an all-gather buffer)."""
    _require_cuda(o_parts=o_parts, lse_parts=lse_parts)
    if o_parts.dtype != torch.float32 or lse_parts.dtype != torch.float32:
        raise ValueError("o_parts and lse_parts must be torch.float32")
    if tuple(o_parts.shape[:-1]) != tuple(lse_parts.shape):
        raise ValueError("o_parts must have shape lse_parts.shape + [D]")
    if not o_parts[0].is_contiguous():
        o_parts = o_parts.contiguous()
    if not lse_parts[0].is_contiguous():
        lse_parts = lse_parts.contiguous()
    R, D = o_parts.shape[0], o_parts.shape[-1]
    rows = lse_parts[0].numel()
    o_stride = o_parts.stride(0) if R > 1 else 0
    l_stride = lse_parts.stride(0) if R > 1 else 0
    o = torch.empty(o_parts.shape[1:], dtype=out_dtype, device=o_parts.device)
    lse = torch.empty(lse_parts.shape[1:], dtype=torch.float32, device=o_parts.device) if return_lse else None
    with torch.cuda.device(o_parts.device):
        st = N.lib().tb200_gqa_lse_merge(o_parts.data_ptr(), lse_parts.data_ptr(), o.data_ptr(), N.ptr(lse),
                                         R, rows, D, o_stride, l_stride, N.dtype_code(out_dtype),
                                         N.current_stream(o_parts.device))
    N.check(st, "tb200_gqa_lse_merge")
    return (o, lse) if return_lse else o


def _prefill_status(device: torch.device, need: int) -> torch.Tensor:
    """Zeroed status buffer of the prefill kernels, one per device (a kernel writes it only when a bounded
    device-side wait runs out).  A wait that ran out makes the launch - and, the word being sticky, every
    later launch on the device - return with its outputs unwritten.  So that this cannot pass unnoticed, the
    word has a mirror in pinned host memory: every prefill call first looks at the mirror (a plain host
    read, no synchronisation; it shows what launches that have completed by now left there), raises
    ``NativeLibraryError`` and clears the word if it is set, and after its launch queues a 4-byte copy of the
    word into the mirror on the same stream."""
    key = (device, "prefill_status")
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(max(need, 256), dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
        _WORKSPACES[(device, "prefill_status_mirror")] = torch.zeros(1, dtype=torch.int32).pin_memory()
    mirror = _WORKSPACES[(device, "prefill_status_mirror")]
    code = int(mirror[0])
    if code:
        mirror.zero_()
        ws[:4].zero_()
        raise N.NativeLibraryError(
            f"an earlier prefill launch on {device} gave up on a device-side wait (code {code}); its outputs and "
            "those of the launches after it are not valid.  The status word has been cleared.")
    return ws


def _mirror_prefill_status(device: torch.device) -> None:
    ws = _WORKSPACES.get((device, "prefill_status"))
    mirror = _WORKSPACES.get((device, "prefill_status_mirror"))
    if ws is not None and mirror is not None:
        mirror.copy_(ws[:4].view(torch.int32), non_blocking=True)


def _device_of(device: "torch.device | str | int | None") -> torch.device:
    """A device with an explicit index (``"cuda"`` means the current device)."""
    d = torch.device("cuda" if device is None else device)
    if d.type == "cuda" and d.index is None:
        d = torch.device("cuda", torch.cuda.current_device())
    return d


def prefill_status(device: "torch.device | str | int | None" = None, reset: bool = False) -> int:
    """0 if no prefill launch on ``device`` (default: the current CUDA device) has timed out on a
    device-side wait, else the code of the wait that gave up (synchronises with the device).

    The word is sticky: once set, every later prefill launch on the device returns at once with its
    outputs unwritten, so after a suspected timeout poll this before using any output.  ``reset=True``
    clears the word after reading it."""
    ws = _WORKSPACES.get((_device_of(device), "prefill_status"))
    if ws is None:
        return 0
    code = int(ws[:4].view(torch.int32).item())
    if reset and code:
        ws[:4].zero_()
        _WORKSPACES[(_device_of(device), "prefill_status_mirror")].zero_()
    return code


def decode_status(device: "torch.device | str | int | None" = None) -> int:
    """Largest non-zero status word left by a decode launch in any cached workspace of ``device`` (601-603:
    a bounded wait of the TMA decode kernel ran out), else 0.  Synchronises.  A workspace whose status is set
    is dropped from the cache (its counters are no longer trustworthy); the next call allocates a fresh one."""
    dev, worst = _device_of(device), 0
    for key in [k for k in _WORKSPACES if len(k) > 2 and k[2] == "decode" and k[0] == dev]:
        code = int(_WORKSPACES[key][8:12].view(torch.int32).item())
        if code:
            worst = max(worst, code)
            del _WORKSPACES[key]
    return worst


def decode_last_kernel() -> str:
    """Name of the kernel that served this thread's last decode call: ``"tma"`` (TMA producer warp + math
    warps), ``"cp_async"``, or ``""`` before the first call."""
    return {1: "tma", 2: "cp_async"}.get(int(N.lib().tb200_gqa_decode_last_kernel()), "")


def gqa_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, is_causal: bool = True,
                sm_scale: Optional[float] = None, softcap: float = 0.0, return_lse: bool = False,
                window_size_left: int = -1, window_size_right: int = -1, config: Optional[dict] = None):
    """Dense BSHD prefill: q ``[B,Sq,H,D]``, k/v ``[B,Skv,Hkv,D]`` -> o ``[B,Sq,H,D]`` (+ LSE
    ``[B,H,Sq]`` fp32, log2 domain)."""
    _require_cuda(q=q, k=k, v=v)
    if q.dim() != 4 or k.dim() != 4 or v.shape != k.shape:
        raise ValueError("q must be [B,Sq,H,D] and k/v [B,Skv,Hkv,D]")
    B, Sq, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    if k.shape[0] != B or k.shape[3] != D:
        raise ValueError("k/v batch and head dim must match q")
    if H % Hkv != 0:
        raise ValueError("heads must be divisible by heads_kv")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q/k/v dtypes must match")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    o = torch.empty_like(q)
    lse = torch.empty((B, H, Sq), dtype=torch.float32, device=q.device) if return_lse else None
    need = N.lib().tb200_gqa_prefill_workspace_bytes(B, H, Hkv, Sq, Skv, D)
    ws = _prefill_status(q.device, need)
    scale = D ** -0.5 if sm_scale is None else float(sm_scale)
    with torch.cuda.device(q.device):
        st = N.lib().tb200_gqa_prefill(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), N.ptr(lse),
                                       N.dtype_code(q.dtype), B, Sq, Skv, H, Hkv, D, int(bool(is_causal)),
                                       scale, float(softcap or 0.0), int(window_size_left),
                                       int(window_size_right), N.prefill_flags(config), N.ptr(ws), need,
                                       N.current_stream(q.device))
    N.check(st, "tb200_gqa_prefill")
    _mirror_prefill_status(q.device)
    return (o, lse) if return_lse else o


def gqa_prefill_paged(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor,
                      k_pages: Optional[torch.Tensor], v_pages: Optional[torch.Tensor],
                      cu_seqlens_q: torch.Tensor, cache_seqlens: Optional[torch.Tensor],
                      block_table: Optional[torch.Tensor], max_seqlen_q: int, *, page_size: int = 0,
                      is_causal: bool = True, sm_scale: Optional[float] = None, softcap: float = 0.0,
                      return_lse: bool = False, cu_seqlens_kv: Optional[torch.Tensor] = None,
                      window_size_left: int = -1, window_size_right: int = -1, config: Optional[dict] = None):
    """Packed prefill of one chunk per request over a paged cache, appending the chunk in place.

    q ``[total_q,H,D]``, k_new/v_new ``[total_q,Hkv,D]``, k_pages/v_pages ``[pool_tokens,Hkv,D]``
    (modified in place), cu_seqlens_q ``[B+1]``, cache_seqlens ``[B]``, block_table ``[B,W]`` (int32)
    -> o ``[total_q,H,D]`` (+ LSE ``[H,total_q]`` fp32, log2 domain).  With the three cache arguments
    ``None`` it is the packed varlen prefill without a cache; only then may ``cu_seqlens_kv``
    give k_new/v_new their own row ranges (bottom-right aligned causal mask per request).
    """
    _require_cuda(q=q, k_new=k_new, v_new=v_new, cu_seqlens_q=cu_seqlens_q)
    if q.dim() != 3 or k_new.dim() != 3 or v_new.shape != k_new.shape:
        raise ValueError("q must be [total_q,H,D] and k_new/v_new [total_kv,Hkv,D]")
    if cu_seqlens_kv is None and k_new.shape[0] != q.shape[0]:
        raise ValueError("k_new/v_new must have the rows of q unless cu_seqlens_kv is given")
    if cu_seqlens_kv is not None:
        if k_pages is not None:
            raise ValueError("cu_seqlens_kv cannot be combined with a cache")
        _require_cuda(cu_seqlens_kv=cu_seqlens_kv)
        if cu_seqlens_kv.dtype != torch.int32 or cu_seqlens_kv.shape != cu_seqlens_q.shape:
            raise ValueError("cu_seqlens_kv must be int32 with the shape of cu_seqlens_q")
        cu_seqlens_kv = cu_seqlens_kv.contiguous()
    total_q, H, D = q.shape
    Hkv = k_new.shape[1]
    if k_new.shape[2] != D or H % Hkv != 0:
        raise ValueError("head dim must match and heads must be divisible by heads_kv")
    if k_new.dtype != q.dtype or v_new.dtype != q.dtype:
        raise ValueError("q/k_new/v_new dtypes must match")
    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_q.dim() != 1:
        raise ValueError("cu_seqlens_q must be a 1-D int32 tensor")
    B = cu_seqlens_q.numel() - 1
    has_cache = k_pages is not None
    pool_tokens, bt_stride = 0, 0
    if has_cache:
        if v_pages is None or cache_seqlens is None or block_table is None:
            raise ValueError("k_pages, v_pages, cache_seqlens and block_table come together")
        _require_cuda(k_pages=k_pages, v_pages=v_pages, cache_seqlens=cache_seqlens, block_table=block_table)
        if k_pages.dtype != q.dtype or v_pages.dtype != q.dtype:
            raise ValueError("k_pages/v_pages must have the dtype of q")
        if not (k_pages.is_contiguous() and v_pages.is_contiguous()):
            raise ValueError("k_pages and v_pages must be contiguous (they are written in place)")
        if k_pages.dim() != 3 or tuple(k_pages.shape[1:]) != (Hkv, D) or v_pages.shape != k_pages.shape:
            raise ValueError("k_pages/v_pages must be [pool_tokens,Hkv,D]")
        if cache_seqlens.dtype != torch.int32 or block_table.dtype != torch.int32:
            raise ValueError("cache_seqlens and block_table must be int32")
        if cache_seqlens.shape != (B,) or block_table.dim() != 2 or block_table.shape[0] != B:
            raise ValueError("cache_seqlens must be [B] and block_table [B,W]")
        if block_table.stride(1) != 1:
            block_table = block_table.contiguous()
        pool_tokens, bt_stride = k_pages.shape[0], block_table.stride(0)
    q, k_new, v_new = q.contiguous(), k_new.contiguous(), v_new.contiguous()
    cu_seqlens_q = cu_seqlens_q.contiguous()
    o = torch.empty_like(q)
    lse = torch.empty((H, total_q), dtype=torch.float32, device=q.device) if return_lse else None
    if total_q == 0:
        return (o, lse) if return_lse else o
    need = N.lib().tb200_gqa_prefill_workspace_bytes(B, H, Hkv, int(max_seqlen_q), 0, D)
    ws = _prefill_status(q.device, need)
    scale = D ** -0.5 if sm_scale is None else float(sm_scale)
    with torch.cuda.device(q.device):
        st = N.lib().tb200_gqa_prefill_paged(
            q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), N.ptr(k_pages), N.ptr(v_pages), o.data_ptr(),
            N.ptr(lse), cu_seqlens_q.data_ptr(), N.ptr(cu_seqlens_kv), N.ptr(cache_seqlens) if has_cache else None,
            N.ptr(block_table) if has_cache else None, bt_stride, N.dtype_code(q.dtype), total_q,
            k_new.shape[0], B,
            int(max_seqlen_q), H, Hkv, D, int(page_size), pool_tokens, int(bool(is_causal)), scale,
            float(softcap or 0.0), int(window_size_left), int(window_size_right), N.prefill_flags(config),
            N.ptr(ws), need, N.current_stream(q.device))
    N.check(st, "tb200_gqa_prefill_paged")
    _mirror_prefill_status(q.device)
    return (o, lse) if return_lse else o


def rope_neox_packed(x: torch.Tensor, cos_table: torch.Tensor, sin_table: torch.Tensor,
                     cu_seqlens_q: torch.Tensor, cache_seqlens: Optional[torch.Tensor],
                     rotary_dim: Optional[int] = None) -> torch.Tensor:
    """GPT-NeoX rotary embedding of packed ``x [T,H,D]`` at positions ``cache_seqlens[b] + i`` for the
    i-th token of request b; tables ``[max_position, rotary_dim/2]`` in x's dtype.  Returns a new tensor."""
    _require_cuda(x=x, cos_table=cos_table, sin_table=sin_table, cu_seqlens_q=cu_seqlens_q)
    if x.dim() != 3:
        raise ValueError("x must be [tokens, heads, dim]")
    T, H, D = x.shape
    rotary_dim = D if rotary_dim is None else int(rotary_dim)
    if cos_table.dtype != x.dtype or sin_table.dtype != x.dtype:
        raise ValueError("cos/sin tables must have x's dtype")
    if cos_table.shape != sin_table.shape or cos_table.dim() != 2 or cos_table.shape[1] != rotary_dim // 2:
        raise ValueError(f"cos/sin tables must be [max_position, {rotary_dim // 2}]")
    if cu_seqlens_q.dtype != torch.int32 or (cache_seqlens is not None and cache_seqlens.dtype != torch.int32):
        raise ValueError("cu_seqlens_q and cache_seqlens must be int32")
    x = x.contiguous()
    y = torch.empty_like(x)
    # positions are range-checked by the caller (the operator does, on the host); no status word is passed
    with torch.cuda.device(x.device):
        st = N.lib().tb200_rope_neox_packed(
            x.data_ptr(), y.data_ptr(), cos_table.contiguous().data_ptr(), sin_table.contiguous().data_ptr(),
            cu_seqlens_q.contiguous().data_ptr(), N.ptr(cache_seqlens), N.dtype_code(x.dtype), T,
            cu_seqlens_q.numel() - 1, H, D, rotary_dim, cos_table.shape[0], None, N.current_stream(x.device))
    N.check(st, "tb200_rope_neox_packed")
    return y


def gqa_prefill_paged_fp8_cache(q: torch.Tensor, k_new: torch.Tensor, v_new: torch.Tensor, k_pages: torch.Tensor,
                                v_pages: torch.Tensor, k_scale: torch.Tensor, v_scale: torch.Tensor,
                                cu_seqlens_q: torch.Tensor, cache_seqlens: torch.Tensor, block_table: torch.Tensor,
                                max_seqlen_q: int, *, page_size: int, is_causal: bool = True,
                                sm_scale: Optional[float] = None, softcap: float = 0.0,
                                fused: Optional[bool] = None) -> torch.Tensor:
    """Packed prefill of one chunk per request over an FP8-e4m3 paged cache with scalar scales
    (``k_scale`` / ``v_scale``: fp32 tensors of shape (1,)).

    Default (``fused=False``): three launches - the cached tokens are dequantised into a packed 16-bit K/V next
    to the chunk's own rows, the packed prefill runs on it, and the chunk is quantised into the pages (the
    packed buffer is sized by the capacity of the block table).  ``fused=True`` (head dim 128): ONE launch - the
    prefill kernel reads the e4m3 pages by TMA, four converter warps expand each tile in shared memory, the
    scalar scales are folded into the softmax, and the appending CTAs quantise the chunk into the pages.  It
    needs no packed copy of the cache but measured 20-30 % slower (every CTA that shares a KV head converts
    the same tiles again on schedulers the softmax already fills).  Nothing is read back from the
    device either way."""
    _require_cuda(q=q, k_new=k_new, v_new=v_new, k_pages=k_pages, v_pages=v_pages, k_scale=k_scale, v_scale=v_scale,
                  cu_seqlens_q=cu_seqlens_q, cache_seqlens=cache_seqlens, block_table=block_table)
    f8 = getattr(torch, "float8_e4m3fn")
    if k_pages.dtype != f8 or v_pages.dtype != f8:
        raise ValueError("k_pages and v_pages must be torch.float8_e4m3fn")
    if k_scale.dtype != torch.float32 or v_scale.dtype != torch.float32 or k_scale.numel() != 1 or v_scale.numel() != 1:
        raise ValueError("k_scale and v_scale must be fp32 tensors with one element")
    if not (k_pages.is_contiguous() and v_pages.is_contiguous()):
        raise ValueError("k_pages and v_pages must be contiguous (they are written in place)")
    total_q, H, D = q.shape
    Hkv = k_new.shape[1]
    B = cu_seqlens_q.numel() - 1
    q, k_new, v_new = q.contiguous(), k_new.contiguous(), v_new.contiguous()
    cu_seqlens_q, cache_seqlens = cu_seqlens_q.contiguous(), cache_seqlens.contiguous()
    if block_table.stride(1) != 1:
        block_table = block_table.contiguous()
    fused = bool(fused)
    if fused:
        if D != 128:
            raise ValueError("the fused e4m3-page prefill serves head dim 128")
        if k_pages.dim() != 3 or tuple(k_pages.shape[1:]) != (Hkv, D) or v_pages.shape != k_pages.shape:
            raise ValueError("k_pages/v_pages must be [pool_tokens,Hkv,D]")
        o = torch.empty_like(q)
        if total_q == 0:
            return o
        need = N.lib().tb200_gqa_prefill_workspace_bytes(B, H, Hkv, int(max_seqlen_q), 0, D)
        ws = _prefill_status(q.device, need)
        scale = D ** -0.5 if sm_scale is None else float(sm_scale)
        with torch.cuda.device(q.device):
            st = N.lib().tb200_gqa_prefill_paged_e4m3_cache(
                q.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                k_scale.data_ptr(), v_scale.data_ptr(), o.data_ptr(), None, cu_seqlens_q.data_ptr(),
                cache_seqlens.data_ptr(), block_table.data_ptr(), block_table.stride(0), N.dtype_code(q.dtype),
                total_q, B, int(max_seqlen_q), H, Hkv, D, int(page_size), k_pages.shape[0], int(bool(is_causal)),
                scale, float(softcap or 0.0), N.ptr(ws), need, N.current_stream(q.device))
        N.check(st, "tb200_gqa_prefill_paged_e4m3_cache")
        _mirror_prefill_status(q.device)
        return o
    kv_lens = cache_seqlens + (cu_seqlens_q[1:] - cu_seqlens_q[:-1])
    cu_kv = torch.zeros(B + 1, dtype=torch.int32, device=q.device)
    cu_kv[1:] = torch.cumsum(kv_lens, 0)
    # The packed K/V is sized by what the block table can describe (its width x the page size per request)
    # plus the chunk: an upper bound known on the host, so that no length is read back from the device.
    # The buffers are kept per shape (a chunked prefill calls this with the same shapes over and over).
    total_kv = B * block_table.shape[1] * int(page_size) + total_q
    key = (q.device, torch.cuda.current_stream(q.device).cuda_stream, "fp8_cache_packed", total_kv, Hkv, D, q.dtype)
    bufs = _WORKSPACES.get(key)
    if bufs is None:
        bufs = (torch.empty((total_kv, Hkv, D), dtype=q.dtype, device=q.device),
                torch.empty((total_kv, Hkv, D), dtype=q.dtype, device=q.device))
        _WORKSPACES[key] = bufs
    k_all, v_all = bufs
    lib, stream = N.lib(), N.current_stream(q.device)
    with torch.cuda.device(q.device):
        st = lib.tb200_fp8_cache_gather(
            k_pages.data_ptr(), v_pages.data_ptr(), k_new.data_ptr(), v_new.data_ptr(), k_all.data_ptr(),
            v_all.data_ptr(), cu_seqlens_q.data_ptr(), cu_kv.data_ptr(), cache_seqlens.data_ptr(),
            block_table.data_ptr(), block_table.stride(0), k_scale.data_ptr(), v_scale.data_ptr(),
            N.dtype_code(q.dtype), total_kv, B, Hkv, D, int(page_size), stream)
        N.check(st, "tb200_fp8_cache_gather")
        o = gqa_prefill_paged(q, k_all, v_all, None, None, cu_seqlens_q, None, None, int(max_seqlen_q),
                              is_causal=is_causal, sm_scale=sm_scale, softcap=softcap, cu_seqlens_kv=cu_kv)
        st = lib.tb200_fp8_cache_append(
            k_new.data_ptr(), v_new.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), cu_seqlens_q.data_ptr(),
            cache_seqlens.data_ptr(), block_table.data_ptr(), block_table.stride(0), k_scale.data_ptr(),
            v_scale.data_ptr(), N.dtype_code(q.dtype), total_q, B, Hkv, D, int(page_size), stream)
        N.check(st, "tb200_fp8_cache_append")
    return o


def mma_issue_probe(n: int = 128, a_in_tmem: bool = False, repetitions: int = 200, device=None) -> "tuple[float, float]":
    """Clocks one ``tcgen05.mma`` (M = 128, K = 16, N = ``n``) takes to be accepted / to complete on the
    tensor pipe of ``device`` (``tb200_mma_issue_probe``; synchronises)."""
    dev = _device_of(device)
    out = torch.zeros(2, dtype=torch.int64, device=dev)
    with torch.cuda.device(dev):
        st = N.lib().tb200_mma_issue_probe(out.data_ptr(), int(n), int(bool(a_in_tmem)), int(repetitions),
                                           N.current_stream(dev))
    N.check(st, "tb200_mma_issue_probe")
    issued, done = (int(x) for x in out.cpu())
    if done < 0:
        raise N.NativeLibraryError("tb200_mma_issue_probe: the bounded wait for the last MMA ran out")
    return issued / (8.0 * repetitions), done / (8.0 * repetitions)
