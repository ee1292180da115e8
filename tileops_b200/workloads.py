"""Seeded synthetic inputs for the GQA attention-forward workloads.

The role of the reference's ``workloads/attention/gqa.py`` (``gen_inputs``): tensors of the
Llama-3 attention shapes drawn from N(0,1).  Differences, on purpose: every sequence owns its
own pages (the reference's paged workload aliases one identity block table across the batch,
``workloads/attention/gqa.py:204-218``), lengths need not be page aligned, the block table is
a random permutation of the pool, and everything derives from explicit seeds so that a rank
holding a slice of the problem regenerates exactly its part.

Seeding rule (base seed 1235, the reference's test seed): lengths and the page permutation come
from a CPU generator seeded ``1235 + cfg``; q from a generator seeded ``1235 + 100*cfg``; K and V
of sequence ``b`` from a generator seeded ``1235 + 1000*cfg + b`` (K first, then V, fp32 randn of
``[len_b, Hkv, D]``, then cast) on the device the inputs live on.
"""

from __future__ import annotations

import dataclasses
from typing import List, Optional

import torch

BASE_SEED = 1235
FP8_MAX = 448.0


@dataclasses.dataclass
class PagedDecodeInputs:
    q: torch.Tensor                 # [B,H,D]
    k: torch.Tensor                 # [P*page,Hkv,D]  (cache dtype)
    v: torch.Tensor
    real_seqlen_kv: torch.Tensor    # [B] int32
    block_table: torch.Tensor       # [B,W] int32
    page_size: int
    k_scale: Optional[torch.Tensor] = None   # [P,Hkv] fp32 (e4m3 cache only)
    v_scale: Optional[torch.Tensor] = None
    lens: Optional[List[int]] = None          # host copy of real_seqlen_kv

    @property
    def kv_bytes_needed(self) -> int:
        """Bytes of K and V that the live tokens occupy (what one pass must read)."""
        return 2 * sum(self.lens) * self.k.shape[1] * self.k.shape[2] * self.k.element_size()

    def algorithmic_bytes(self) -> int:
        """K/V of live tokens + q + o + scales + metadata, each counted once."""
        B, H, D = self.q.shape
        pages = sum(-(-n // self.page_size) for n in self.lens)
        scales = 2 * pages * self.k.shape[1] * 4 if self.k_scale is not None else 0
        return self.kv_bytes_needed + 2 * B * H * D * self.q.element_size() + scales + 4 * pages + 4 * B

    def algorithmic_flops(self) -> int:
        _, H, D = self.q.shape
        return 4 * H * D * sum(self.lens)


def _gen(device, seed: int) -> torch.Generator:
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return g


def quantize_kv_per_page(x: torch.Tensor, page_size: int):
    """x ``[N,Hkv,D]`` -> (e4m3 ``[N,Hkv,D]``, fp32 scale ``[N/page,Hkv]``), scale = amax/448.

    The arithmetic of the reference's ``quantize_kv_fa3_descale``
    (``workloads/gqa_fp8_utils.py:4-17``) with pages in the role of the batch dimension.
    """
    N, Hkv, D = x.shape
    xp = x.float().reshape(N // page_size, page_size, Hkv, D)
    scale = xp.abs().amax(dim=(1, 3)).clamp(min=1e-4) / FP8_MAX
    xq = torch.clamp(xp / scale[:, None, :, None], -FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return xq.reshape(N, Hkv, D).contiguous(), scale.float().contiguous()


def draw_lengths(cfg, batch, len_range, generator=None):
    """``batch`` context lengths drawn uniformly from ``len_range`` (inclusive) with the seed stream of
    workload ``cfg``: what :func:`make_paged_decode` draws when it is given no lengths."""
    g = generator if generator is not None else torch.Generator().manual_seed(BASE_SEED + cfg)
    lo, hi = len_range
    return torch.randint(lo, hi + 1, (batch,), generator=g).tolist()


def make_paged_decode(
    cfg: int,
    batch: int,
    heads: int,
    heads_kv: int,
    dim: int,
    page_size: int,
    lens: "List[int] | None" = None,
    len_range: "tuple[int, int] | None" = None,
    dtype: torch.dtype = torch.bfloat16,
    fp8_cache: bool = False,
    device: "torch.device | str" = "cuda",
    tail_fill: float = 0.0,
    spare_pages: int = 0,
    page_begin: int = 0,
    page_end: Optional[int] = None,
) -> PagedDecodeInputs:
    """Build one paged-decode problem.

    ``lens`` fixes the lengths, else they are drawn uniformly from ``len_range`` (inclusive).
    ``tail_fill`` is written to the pool rows of a tail page beyond a sequence's length (NaN
    in tests shows a kernel that reads them).  ``page_begin``/``page_end`` restrict every
    sequence to a range of its LOGICAL pages (a KV-sequence shard): the returned lengths,
    block table and pool describe only that range, in a local pool.
    """
    device = torch.device(device)
    gcpu = torch.Generator().manual_seed(BASE_SEED + cfg)
    if lens is None:
        lens = draw_lengths(cfg, batch, len_range, gcpu)
    lens = [int(x) for x in lens]
    full_pages = [-(-n // page_size) for n in lens]
    # logical page range kept by this shard, per sequence
    kept = []
    for n_pg in full_pages:
        b0 = min(page_begin, n_pg)
        b1 = n_pg if page_end is None else min(page_end, n_pg)
        kept.append((b0, max(b0, b1)))
    local_pages = [b1 - b0 for b0, b1 in kept]
    local_lens = [max(0, min(n, b1 * page_size) - b0 * page_size) for n, (b0, b1) in zip(lens, kept)]
    P = sum(local_pages) + spare_pages
    perm = torch.randperm(max(P, 1), generator=gcpu).to(torch.int32)
    W = max(max(local_pages), 1)
    bt = torch.zeros(batch, W, dtype=torch.int32)
    off = 0
    for b in range(batch):
        bt[b, :local_pages[b]] = perm[off:off + local_pages[b]]
        off += local_pages[b]

    q = torch.randn(batch, heads, dim, generator=_gen(device, BASE_SEED + 100 * cfg), device=device).to(dtype)
    pool_k = torch.full((max(P, 1) * page_size, heads_kv, dim), tail_fill, dtype=dtype, device=device)
    pool_v = torch.full_like(pool_k, tail_fill)
    bt_dev = bt.to(device)
    for b in range(batch):
        g = _gen(device, BASE_SEED + 1000 * cfg + b)
        n = lens[b]
        t0, t1 = kept[b][0] * page_size, kept[b][0] * page_size + local_lens[b]
        # draw in fixed 4096-token blocks so that a shard can skip to its range cheaply and
        # still see the same numbers as the unsharded problem
        blk = 4096
        for s in range(0, n, blk):
            e = min(n, s + blk)
            kb = torch.randn(e - s, heads_kv, dim, generator=g, device=device)
            vb = torch.randn(e - s, heads_kv, dim, generator=g, device=device)
            a, z = max(s, t0), min(e, t1)
            if a >= z:
                continue
            t = torch.arange(a - t0, z - t0, device=device)
            rows = bt_dev[b, t // page_size].long() * page_size + t % page_size
            pool_k[rows] = kb[a - s:z - s].to(dtype)
            pool_v[rows] = vb[a - s:z - s].to(dtype)

    out = PagedDecodeInputs(q=q, k=pool_k, v=pool_v,
                            real_seqlen_kv=torch.tensor(local_lens, dtype=torch.int32, device=device),
                            block_table=bt_dev.contiguous(), page_size=page_size, lens=local_lens)
    if fp8_cache:
        kf = torch.nan_to_num(pool_k.float(), nan=0.0) if tail_fill != tail_fill else pool_k.float()
        vf = torch.nan_to_num(pool_v.float(), nan=0.0) if tail_fill != tail_fill else pool_v.float()
        out.k, out.k_scale = quantize_kv_per_page(kf, page_size)
        out.v, out.v_scale = quantize_kv_per_page(vf, page_size)
    return out


def make_contiguous_decode(cfg, batch, heads, heads_kv, seqlen_kv, dim, dtype=torch.float32, device="cpu"):
    """q ``[B,H,D]``, k/v ``[B,S,Hkv,D]`` ~ N(0,1) (the reference's CPU-runnable decode case draws these on the CPU)."""
    device = torch.device(device)
    q = torch.randn(batch, heads, dim, generator=_gen(device, BASE_SEED + 100 * cfg), device=device).to(dtype)
    ks, vs = [], []
    for b in range(batch):
        g = _gen(device, BASE_SEED + 1000 * cfg + b)
        ks.append(torch.randn(seqlen_kv, heads_kv, dim, generator=g, device=device))
        vs.append(torch.randn(seqlen_kv, heads_kv, dim, generator=g, device=device))
    return q, torch.stack(ks).to(dtype), torch.stack(vs).to(dtype)


def make_prefill(cfg, batch, seqlen_q, seqlen_kv, heads, heads_kv, dim, dtype=torch.bfloat16, device="cuda"):
    """q ``[B,Sq,H,D]``, k/v ``[B,Skv,Hkv,D]`` ~ N(0,1) cast to ``dtype``."""
    device = torch.device(device)
    q = torch.randn(batch, seqlen_q, heads, dim, generator=_gen(device, BASE_SEED + 100 * cfg), device=device).to(dtype)
    ks, vs = [], []
    for b in range(batch):
        g = _gen(device, BASE_SEED + 1000 * cfg + b)
        ks.append(torch.randn(seqlen_kv, heads_kv, dim, generator=g, device=device).to(dtype))
        vs.append(torch.randn(seqlen_kv, heads_kv, dim, generator=g, device=device).to(dtype))
    return q, torch.stack(ks), torch.stack(vs)


def make_paged_prefill(cfg, q_lens, cache_lens, heads, heads_kv, dim, page_size, max_pages_per_req,
                       dtype=torch.float16, device="cuda"):
    """Inputs of one packed prefill chunk per request over a paged cache, in the argument order of
    ``GroupedQueryAttentionPrefillPagedWithKVCacheFwdOp.forward``: (q, k_new, v_new, k_pages, v_pages,
    k_scale, v_scale, cu_seqlens_q, cache_seqlens, block_table, max_seqlen_q).  All ~ N(0,1); the
    block table is a seeded permutation of the pool's pages (every request owns
    ``max_pages_per_req`` of them); every pool row is filled, cached or not."""
    device = torch.device(device)
    g = _gen(device, BASE_SEED + 100 * cfg)
    batch, total_q = len(q_lens), int(sum(q_lens))
    pool = batch * max_pages_per_req * page_size
    q = torch.randn(total_q, heads, dim, generator=g, device=device).to(dtype)
    k_new = torch.randn(total_q, heads_kv, dim, generator=g, device=device).to(dtype)
    v_new = torch.randn(total_q, heads_kv, dim, generator=g, device=device).to(dtype)
    k_pages = torch.randn(pool, heads_kv, dim, generator=g, device=device).to(dtype)
    v_pages = torch.randn(pool, heads_kv, dim, generator=g, device=device).to(dtype)
    bt = torch.randperm(batch * max_pages_per_req, generator=g, device=device).to(torch.int32)
    cu = torch.zeros(batch + 1, dtype=torch.int32)
    cu[1:] = torch.tensor(q_lens, dtype=torch.int32).cumsum(0)
    one = torch.ones(1, dtype=torch.float32, device=device)
    return (q, k_new, v_new, k_pages, v_pages, one, one.clone(), cu.to(device),
            torch.tensor(cache_lens, dtype=torch.int32, device=device),
            bt.reshape(batch, max_pages_per_req).contiguous(), int(max(q_lens)))


# The five benchmark workloads, by number: 1 contiguous fp32 decode (2 x 256 tokens), 2 causal prefill bf16
# (4 x 4096), 3 paged bf16 decode (64 ragged sequences), 4 paged decode over an e4m3 cache (128 x 4096),
# 5 long-context paged decode (8 x 131072, page 128).
def baseline_config(cfg: int, device="cuda", **overrides):
    if cfg == 1:
        return make_contiguous_decode(1, 2, 8, 2, 256, 64, torch.float32, overrides.get("device", "cpu"))
    if cfg == 2:
        return make_prefill(2, 4, 4096, 4096, 32, 8, 128, torch.bfloat16, device)
    if cfg == 3:
        return make_paged_decode(3, 64, 32, 8, 128, 64, len_range=(512, 8192), device=device, **overrides)
    if cfg == 4:
        return make_paged_decode(4, 128, 64, 8, 128, 64, lens=[4096] * 128, fp8_cache=True, device=device,
                                 **overrides)
    if cfg == 5:
        return make_paged_decode(5, 8, 32, 8, 128, 128, lens=[131072] * 8, device=device, **overrides)
    raise ValueError(f"unknown workload number {cfg}")
