"""CPU oracle for the GQA attention-forward path. TEST INFRASTRUCTURE ONLY.

This module restates, in plain fp32 torch / numpy on the CPU, the torch reference
programs that tile-ai/TileOPs itself checks its GQA kernels against.  It exists so
that the CUDA kernels of ``tileops_b200`` can be compared with the reference's
arithmetic on a machine where the reference tree is absent.  Nothing in the
product package imports it: only the tests, the smoke entry and the benchmark's
CPU-baseline leg do, and only as the checker.

Pinning: every function below is checked against the reference's own code run in
the build container (fixtures under ``tests/golden/`` produced by
``tests/golden/make_golden.py``, which imports the reference's workloads and test
references: decode, paged decode, dense / packed / sliding-window prefill, paged prefill with append and
its FP8-cache form, GPT-NeoX RoPE, the FP8 quantiser, the roofline formulas).  Two functions have no
reference counterpart and are therefore
*parity unpinned* beyond their own definition: the per-(page, KV-head) FP8
quantiser/dequantiser (the reference only has one scalar scale per cache,
``tests/ops/attention/test_gqa_prefill_paged.py:348-356``) and the multi-shard
O/LSE merge (the reference merges splits only inside one kernel,
``src/tileops/kernels/attention/gqa_decode_paged.py:344-374``).

All LSE values are in the log2 domain, as in the reference
(``workloads/attention/gqa.py:29``): ``lse = log2(sum_j exp(score_j))`` with
``score`` already multiplied by ``sm_scale``.
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

LOG2E = math.log2(math.e)
FP8_MAX = 448.0


def _scale(dim: int, sm_scale: Optional[float]) -> float:
    # src/tileops/ops/attention/gqa.py:81-82
    return dim ** -0.5 if sm_scale is None else float(sm_scale)


def _softcap(scores: torch.Tensor, softcap: Optional[float]) -> torch.Tensor:
    # workloads/attention/gqa.py:171-172 ; tests/ops/attention/test_gqa.py:127-128
    if softcap is not None and softcap > 0:
        return softcap * torch.tanh(scores / softcap)
    return scores


# ---------------------------------------------------------------------------
# contiguous single-token decode
# ---------------------------------------------------------------------------

def decode_ref(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sm_scale: Optional[float] = None,
    softcap: Optional[float] = None,
    return_lse: bool = False,
):
    """q [B,H,D], k/v [B,S,Hkv,D] -> o [B,H,D] (q dtype).

    Follows ``GroupedQueryAttentionDecodeWorkload.ref_program``
    (``workloads/attention/gqa.py:165-175``): expand KV heads, fp32 scores,
    optional softcap, softmax, fp32 PV, cast to the q dtype.
    """
    B, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    qf = q.float().unsqueeze(2)                                   # [B,H,1,D]
    kf = k.float().repeat_interleave(g, dim=2).permute(0, 2, 1, 3)  # [B,H,S,D]
    vf = v.float().repeat_interleave(g, dim=2).permute(0, 2, 1, 3)
    scores = torch.matmul(qf, kf.transpose(-2, -1)) * _scale(D, sm_scale)
    scores = _softcap(scores, softcap)
    probs = torch.softmax(scores, dim=-1)
    out = torch.matmul(probs, vf).squeeze(2).to(q.dtype).contiguous()
    if return_lse:
        lse = torch.logsumexp(scores, dim=-1).squeeze(2) * LOG2E   # [B,H]
        return out, lse
    return out


# ---------------------------------------------------------------------------
# paged decode
# ---------------------------------------------------------------------------

def paged_gather(
    pool: np.ndarray, block_table_row: np.ndarray, real_len: int, page_size: int
) -> np.ndarray:
    """Logical view of one sequence: logical page i <- physical page block_table[i].

    Pure integer indexing (bit-exact by construction).  Follows the reassembly
    loop of ``tests/ops/attention/test_gqa_decode_paged.py:45-58``: copy whole
    pages in logical order, then truncate to ``real_len`` tokens.
    """
    n_pages = -(-int(real_len) // page_size)
    if n_pages == 0:
        return pool[:0]
    rows = (
        block_table_row[:n_pages].astype(np.int64)[:, None] * page_size
        + np.arange(page_size, dtype=np.int64)[None, :]
    ).reshape(-1)[: int(real_len)]
    return pool[rows]


def physical_rows(block_table_row: np.ndarray, real_len: int, page_size: int) -> np.ndarray:
    """Physical pool row of every logical token 0..real_len-1 (int64)."""
    t = np.arange(int(real_len), dtype=np.int64)
    return block_table_row.astype(np.int64)[t // page_size] * page_size + t % page_size


def paged_decode_ref(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    real_seqlen_kv: torch.Tensor,
    block_table: torch.Tensor,
    page_size: int,
    sm_scale: Optional[float] = None,
    softcap: Optional[float] = None,
    return_lse: bool = False,
):
    """q [B,H,D], k/v pool [N,Hkv,D], real_seqlen_kv [B] i32, block_table [B,W] i32.

    Reassemble-then-attend, as ``GroupedQueryAttentionDecodePagedTest.ref_program``
    (``tests/ops/attention/test_gqa_decode_paged.py:30-72``).  A sequence of
    length 0 yields a zero row (the reference kernels' empty guard,
    ``src/tileops/kernels/attention/gqa_decode_paged.py:160-163``) and an LSE of
    ``-inf``.
    """
    B, H, D = q.shape
    Hkv = k.shape[1]
    g = H // Hkv
    group_id = torch.arange(H) // g
    outs, lses = [], []
    bt = block_table.cpu().numpy()
    lens = real_seqlen_kv.cpu().numpy()
    for b in range(B):
        L = int(lens[b])
        if L == 0:
            outs.append(torch.zeros(1, H, D, dtype=q.dtype))
            lses.append(torch.full((1, H), float("-inf")))
            continue
        rows = torch.from_numpy(physical_rows(bt[b], L, page_size))
        kl = k[rows].float()[:, group_id, :].permute(1, 0, 2)      # [H,L,D]
        vl = v[rows].float()[:, group_id, :].permute(1, 0, 2)
        qb = q[b].float().unsqueeze(1)                            # [H,1,D]
        scores = torch.matmul(qb, kl.transpose(-2, -1)) * _scale(D, sm_scale)
        scores = _softcap(scores, softcap)
        probs = torch.softmax(scores, dim=-1)
        outs.append(torch.matmul(probs, vl).squeeze(1).unsqueeze(0).to(q.dtype))
        lses.append((torch.logsumexp(scores, dim=-1).squeeze(1) * LOG2E).unsqueeze(0))
    out = torch.cat(outs, dim=0).contiguous()
    if return_lse:
        return out, torch.cat(lses, dim=0)
    return out


# ---------------------------------------------------------------------------
# FP8-e4m3 KV cache with one fp32 scale per (page, KV head)
# ---------------------------------------------------------------------------

def quantize_kv_per_page(x: torch.Tensor, page_size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """x pool [N,Hkv,D] (N multiple of page_size) -> (e4m3 pool, scale [N/page,Hkv] f32).

    The arithmetic of ``quantize_kv_fa3_descale`` (``workloads/gqa_fp8_utils.py:4-17``:
    ``scale = clamp(amax, 1e-4) / 448``; ``x_q = clamp(x / scale, +-448).to(e4m3)``)
    with the amax taken per (page, KV head) instead of per (batch, KV head).
    """
    N, Hkv, D = x.shape
    assert N % page_size == 0
    xp = x.float().reshape(N // page_size, page_size, Hkv, D)
    scale = xp.abs().amax(dim=(1, 3)).clamp(min=1e-4) / FP8_MAX       # [P,Hkv]
    xq = torch.clamp(xp / scale[:, None, :, None], -FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return xq.reshape(N, Hkv, D).contiguous(), scale.float().contiguous()


def dequantize_kv_per_page(
    xq: torch.Tensor, scale: torch.Tensor, page_size: int, dtype: torch.dtype
) -> torch.Tensor:
    """``(fp8.float() * scale).to(dtype)``: the dequantise step of the reference's FP8
    cache test (``tests/ops/attention/test_gqa_prefill_paged.py:355-356``), with the
    scale broadcast per (page, KV head)."""
    N, Hkv, D = xq.shape
    xf = xq.float().reshape(N // page_size, page_size, Hkv, D) * scale[:, None, :, None]
    return xf.reshape(N, Hkv, D).to(dtype)


def paged_decode_fp8_ref(
    q, k_fp8, v_fp8, k_scale, v_scale, real_seqlen_kv, block_table, page_size,
    sm_scale=None, softcap=None, return_lse=False,
):
    """Dequantise-then-attend: the pool is dequantised to the q dtype and the paged
    reference above is applied."""
    kd = dequantize_kv_per_page(k_fp8, k_scale, page_size, q.dtype)
    vd = dequantize_kv_per_page(v_fp8, v_scale, page_size, q.dtype)
    return paged_decode_ref(q, kd, vd, real_seqlen_kv, block_table, page_size,
                            sm_scale, softcap, return_lse)


# ---------------------------------------------------------------------------
# prefill
# ---------------------------------------------------------------------------

def prefill_ref(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    is_causal: bool = True,
    sm_scale: Optional[float] = None,
    softcap: Optional[float] = None,
    return_lse: bool = False,
    window_left: int = -1,
    window_right: int = -1,
):
    """q [B,Sq,H,D], k/v [B,Skv,Hkv,D] -> o [B,Sq,H,D] (+ LSE [B,H,Sq] fp32, log2).

    ``window_left`` / ``window_right`` (-1 = unlimited) add the sliding-window conditions of
    the reference's sliding-window reference programs
    (``tests/ops/attention/test_gqa_sliding_window.py:17-54``,
    ``test_gqa_sliding_window_varlen.py:22-84``): with ``d = Skv - Sq``, key j is hidden from
    row i when ``j < i + d - window_left`` or ``j > i + d + window_right``; rows left without
    a key give zeros.

    Follows ``_gqa_prefill_ref`` (``tests/ops/attention/test_gqa.py:109-139``):
    fp32 materialised scores, softcap before the mask, bottom-right aligned causal
    mask ``k_pos <= q_pos + (Skv - Sq)``.  The LSE follows
    ``_compute_gqa_square_lse`` (``workloads/attention/gqa.py:11-29``), generalised
    to the same scale/softcap/mask.  Processed one (batch, head-group) at a time
    to bound memory.
    """
    B, Sq, H, D = q.shape
    Skv, Hkv = k.shape[1], k.shape[2]
    g = H // Hkv
    scale = _scale(D, sm_scale)
    out = torch.empty(B, Sq, H, D, dtype=q.dtype)
    lse = torch.empty(B, H, Sq, dtype=torch.float32)
    q_pos = torch.arange(Sq)[:, None] + (Skv - Sq)
    k_pos = torch.arange(Skv)[None, :]
    mask = torch.ones(Sq, Skv, dtype=torch.bool)
    if is_causal:
        mask &= k_pos <= q_pos
    if window_left >= 0:
        mask &= k_pos >= q_pos - window_left
    if window_right >= 0:
        mask &= k_pos <= q_pos + window_right
    masked = is_causal or window_left >= 0 or window_right >= 0
    for b in range(B):
        for hk in range(Hkv):
            qf = q[b, :, hk * g:(hk + 1) * g, :].float().permute(1, 0, 2)   # [g,Sq,D]
            kf = k[b, :, hk, :].float()                                    # [Skv,D]
            vf = v[b, :, hk, :].float()
            scores = torch.matmul(qf, kf.t()) * scale                       # [g,Sq,Skv]
            scores = _softcap(scores, softcap)
            if masked:
                scores = scores.masked_fill(~mask[None], float("-inf"))
            probs = torch.softmax(scores, dim=-1).nan_to_num()
            o = torch.matmul(probs, vf)                                     # [g,Sq,D]
            out[b, :, hk * g:(hk + 1) * g, :] = o.permute(1, 0, 2).to(q.dtype)
            lse[b, hk * g:(hk + 1) * g, :] = torch.logsumexp(scores, dim=-1) * LOG2E
    if return_lse:
        return out, lse
    return out


def prefill_packed_ref(q, k, v, cu_seqlens_q, cu_seqlens_kv, is_causal=True,
                       sm_scale=None, softcap=None, window_left=-1, window_right=-1):
    """Packed THD form, per request; follows ``_gqa_prefill_varlen_ref``
    (``tests/ops/attention/test_gqa.py:152-191``)."""
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    ck = [int(x) for x in cu_seqlens_kv.tolist()]
    outs = []
    for b in range(len(cq) - 1):
        outs.append(prefill_ref(q[cq[b]:cq[b + 1]].unsqueeze(0), k[ck[b]:ck[b + 1]].unsqueeze(0),
                                v[ck[b]:ck[b + 1]].unsqueeze(0), is_causal, sm_scale, softcap,
                                window_left=window_left, window_right=window_right)[0])
    return torch.cat(outs, dim=0)


def rope_tables_ref(rotary_dim: int, max_position: int, base: float = 10000.0, dtype=torch.float32):
    """cos / sin tables [max_position, rotary_dim/2], computed in fp32 and cast to ``dtype``; follows
    ``base_freqs`` (``src/tileops/ops/rope.py:97-120``)."""
    half = rotary_dim // 2
    freqs = 1.0 / (base ** (torch.arange(0, half, dtype=torch.float32) / half))
    angles = torch.outer(torch.arange(max_position, dtype=torch.float32), freqs)
    return torch.cos(angles).to(dtype), torch.sin(angles).to(dtype)


def rope_neox_packed_ref(x, cos, sin, cu_seqlens_q, cache_seqlens, rotary_dim=None):
    """GPT-NeoX rotation of packed x [T,H,D] at positions ``cache_len[b] + i``; follows
    ``ref_rope_neox_position_ids`` (``tests/ops/test_rope.py:84-102``): fp32 arithmetic on tables held
    in x's dtype, the first ``rotary_dim`` dims rotated about their midpoint, the rest copied."""
    cq = [int(v) for v in cu_seqlens_q.tolist()]
    pos = torch.cat([torch.arange(cq[b + 1] - cq[b]) + (int(cache_seqlens[b]) if cache_seqlens is not None else 0)
                     for b in range(len(cq) - 1)]).long()
    rd = x.shape[-1] if rotary_dim is None else rotary_dim
    cos_full = torch.cat([cos, cos], dim=-1)[pos].unsqueeze(1).float()
    sin_full = torch.cat([sin, sin], dim=-1)[pos].unsqueeze(1).float()
    xr = x[..., :rd]
    rot = torch.cat([-xr[..., rd // 2:], xr[..., :rd // 2]], dim=-1)
    y = (xr.float() * cos_full + rot.float() * sin_full).to(x.dtype)
    return y if rd == x.shape[-1] else torch.cat([y, x[..., rd:]], dim=-1)


def prefill_paged_ref(q, k_new, v_new, k_pages, v_pages, cu_seqlens_q, cache_seqlens, block_table,
                      page_size, is_causal=True, sm_scale=None, softcap=None):
    """Packed prefill of one chunk per request over a paged cache, with append.

    q [total_q,H,D], k_new/v_new [total_q,Hkv,D], k_pages/v_pages [pool_tokens,Hkv,D],
    cu_seqlens_q [B+1], cache_seqlens [B], block_table [B,W] -> (o [total_q,H,D], k_pages_after,
    v_pages_after).  Follows ``_gqa_prefill_paged_ref`` and the append checks of
    ``tests/ops/attention/test_gqa_prefill_paged.py:76-117,288-300``: request b attends to its
    cached tokens (gathered through the table) followed by its new tokens, causal meaning
    ``kv_pos <= cache_len + q_pos`` (the bottom-right alignment of :func:`prefill_ref`); the new
    rows land at logical positions ``cache_len + i``; cached rows are untouched.
    """
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    kp_after, vp_after = k_pages.clone(), v_pages.clone()
    outs = []
    for b in range(len(cq) - 1):
        old = int(cache_seqlens[b])
        n = cq[b + 1] - cq[b]
        bt_row = block_table[b].numpy() if isinstance(block_table, torch.Tensor) else np.asarray(block_table[b])
        rows_old = torch.from_numpy(physical_rows(bt_row, old, page_size).astype(np.int64))
        k_all = torch.cat([k_pages[rows_old].to(q.dtype), k_new[cq[b]:cq[b + 1]]], dim=0)
        v_all = torch.cat([v_pages[rows_old].to(q.dtype), v_new[cq[b]:cq[b + 1]]], dim=0)
        if n > 0:
            outs.append(prefill_ref(q[cq[b]:cq[b + 1]].unsqueeze(0), k_all.unsqueeze(0), v_all.unsqueeze(0),
                                    is_causal, sm_scale, softcap)[0])
            rows_new = torch.from_numpy(physical_rows(bt_row, old + n, page_size)[old:].astype(np.int64))
            kp_after[rows_new] = k_new[cq[b]:cq[b + 1]].to(k_pages.dtype)
            vp_after[rows_new] = v_new[cq[b]:cq[b + 1]].to(v_pages.dtype)
    o = torch.cat(outs, dim=0) if outs else q.new_zeros(q.shape)
    return o, kp_after, vp_after


def prefill_paged_fp8_cache_ref(q, k_new, v_new, k_pages, v_pages, k_scale, v_scale, cu_seqlens_q, cache_seqlens,
                               block_table, page_size, is_causal=True, sm_scale=None, softcap=None):
    """Paged prefill over an FP8-e4m3 cache with scalar scales; follows the reference's FP8-cache test
    (``tests/ops/attention/test_gqa_prefill_paged.py:348-404``): cached tokens enter the attention as
    ``(x8.float() * scale).to(q.dtype)``, the chunk's own k_new / v_new at full precision, and the pages
    receive ``(x.float() / scale).to(float8_e4m3fn)`` at the chunk's positions.  Returns (o, k_pages_after,
    v_pages_after)."""
    f8 = torch.float8_e4m3fn
    ks, vs = float(k_scale.reshape(-1)[0]), float(v_scale.reshape(-1)[0])
    kd = (k_pages.float() * ks).to(q.dtype)
    vd = (v_pages.float() * vs).to(q.dtype)
    o, kd_after, _ = prefill_paged_ref(q, k_new, v_new, kd, vd, cu_seqlens_q, cache_seqlens, block_table, page_size,
                                       is_causal, sm_scale, softcap)
    kp_after, vp_after = k_pages.clone(), v_pages.clone()
    cq = [int(x) for x in cu_seqlens_q.tolist()]
    for b in range(len(cq) - 1):
        old, n = int(cache_seqlens[b]), cq[b + 1] - cq[b]
        if n == 0:
            continue
        bt_row = block_table[b].numpy() if isinstance(block_table, torch.Tensor) else np.asarray(block_table[b])
        rows = torch.from_numpy(physical_rows(bt_row, old + n, page_size)[old:].astype(np.int64))
        kp_after[rows] = (k_new[cq[b]:cq[b + 1]].float() / ks).to(f8)
        vp_after[rows] = (v_new[cq[b]:cq[b + 1]].float() / vs).to(f8)
    return o, kp_after, vp_after


# ---------------------------------------------------------------------------
# split / shard merge (log2-domain LSE)
# ---------------------------------------------------------------------------

def merge_partials_ref(o_parts: torch.Tensor, lse_parts: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """o_parts [R,B,H,D] fp32 (each already normalised by its own sum), lse_parts
    [R,B,H] fp32 log2-domain -> merged (o [B,H,D] fp32, lse [B,H]).

    ``O = sum_r 2^(lse_r - lse_tot) O_r`` with ``lse_tot = log2 sum_r 2^lse_r``: the
    algebra of the reference's combine grid
    (``src/tileops/kernels/attention/gqa_decode_paged.py:344-374``).  A part whose
    LSE is ``-inf`` (or the finite floor ``<= -1e29``) carries no weight; if every
    part is empty the result is zero.  A NaN LSE in any part makes the row NaN (o and lse): a part that
    went wrong must not be mistaken for an empty one.
    """
    bad = torch.isnan(lse_parts).any(dim=0)
    lse_parts = torch.nan_to_num(lse_parts, nan=float("-inf"))
    lse = lse_parts.double()
    m = lse.max(dim=0).values
    m_safe = torch.where(torch.isfinite(m) & (m > -1e29), m, torch.zeros_like(m))
    w = torch.exp2(lse - m_safe[None])
    w = torch.where(lse_parts.double() > -1e29, w, torch.zeros_like(w))
    den = w.sum(dim=0)
    o = (w[..., None] * o_parts.double()).sum(dim=0) / torch.where(den > 0, den, torch.ones_like(den))[..., None]
    lse_tot = torch.where(den > 0, torch.log2(torch.where(den > 0, den, torch.ones_like(den))) + m_safe,
                          torch.full_like(den, float("-inf")))
    o, lse_tot = o.float(), lse_tot.float()
    o[bad] = float("nan")
    lse_tot[bad] = float("nan")
    return o, lse_tot


# ---------------------------------------------------------------------------
# roofline formulas (restated; pinned against the importable originals)
# ---------------------------------------------------------------------------

def _itemsize(dtype) -> int:
    # src/tileops/perf/formulas.py:177-194
    if hasattr(dtype, "itemsize"):
        return int(dtype.itemsize)
    name = str(dtype)
    if "float32" in name or "int32" in name:
        return 4
    if "float64" in name or "int64" in name:
        return 8
    if "int8" in name or "bool" in name:
        return 1
    return 2


def gqa_fwd_roofline_ref(batch, seq_len, heads, heads_kv, dim, is_causal, dtype):
    # src/tileops/perf/formulas.py:152-174
    flops = 4 * batch * heads * seq_len * seq_len * dim
    if is_causal:
        flops //= 2
    q_elems = batch * seq_len * heads * dim
    kv_elems = batch * seq_len * heads_kv * dim
    return int(flops), int(2 * (q_elems + kv_elems) * _itemsize(dtype))


def gqa_decode_roofline_ref(batch, heads, heads_kv, seqlen_kv, dim, dtype):
    # src/tileops/perf/formulas.py:668-687
    e = _itemsize(dtype)
    q_elems = batch * heads * dim
    kv_elems = batch * seqlen_kv * heads_kv * dim
    return int(4 * batch * heads * seqlen_kv * dim), int((2 * q_elems + 2 * kv_elems) * e)


def gqa_decode_paged_roofline_ref(batch, heads, heads_kv, seqlen_kv, dim, page_size, dtype):
    # src/tileops/perf/formulas.py:690-711
    e = _itemsize(dtype)
    q_elems = batch * heads * dim
    kv_elems = seqlen_kv * heads_kv * dim
    meta = batch * 4 + batch * max(1, (seqlen_kv + page_size - 1) // page_size) * 4
    return int(4 * batch * heads * seqlen_kv * dim), int((2 * q_elems + 2 * kv_elems) * e + meta)
