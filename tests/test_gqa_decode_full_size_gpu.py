"""Decode parity at the full size of the FP8 and the long-context workloads, the kernel variants
against each other, and the batch sizes that reach the plan's multi-pass code.

* FP8-e4m3 cache, 128 sequences x 4096 tokens, 64 q heads / 8 KV heads: sequences against the
  dequantise-then-attend oracle (<= 3e-2 abs) and the split/merge property on every row.
* 8 sequences x 131072 tokens, page 128: one sequence x one KV-head group against the oracle, and
  the single-launch result against the LSE merge of 2 / 4 / 8 page-range shards computed on the one
  GPU (the exact decomposition the multi-GPU path uses).
* The TMA-producer kernel and the cp.async kernel give the same result (tolerance of bf16 P noise),
  a fixed run length of 1 / 2 / many splits gives the same result as the cost model's choice.

Acceptance forms follow the reference's paged-decode test
(tests/ops/attention/test_gqa_decode_paged.py:17-28,75-151 in tile-ai/TileOPs).
"""

import pytest
import torch

from oracle import gqa_oracle as O
from tileops_b200 import _native as N
from tileops_b200 import functional as F
from tileops_b200 import workloads as W
from tileops_b200.sharded import shard_page_range

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 1e-2
FP8_ATOL = 3e-2


def close(got, want, atol=ATOL, rtol=RTOL):
    got, want = got.float().cpu(), want.float().cpu()
    assert not torch.isnan(got).any(), "NaN in kernel output"
    torch.testing.assert_close(got, want, atol=atol, rtol=rtol)


def decode(inp, lens=None, bt=None, **kw):
    extra = dict(k_scale=inp.k_scale, v_scale=inp.v_scale) if inp.k_scale is not None else {}
    return F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv if lens is None else lens,
                        block_table=inp.block_table if bt is None else bt, page_size=inp.page_size, **extra, **kw)


def test_fp8_workload_at_full_size():
    inp = W.baseline_config(4, "cuda")
    B, H, D = inp.q.shape
    assert (B, H, D, inp.k.shape[1], inp.page_size) == (128, 64, 128, 8, 64)
    o, lse = decode(inp, return_lse=True, out_dtype=torch.float32)
    assert not torch.isnan(o).any()
    kc, vc, ksc, vsc = inp.k.cpu(), inp.v.cpu(), inp.k_scale.cpu(), inp.v_scale.cpu()
    for b in (0, 41, 77, 127):
        ref = O.paged_decode_fp8_ref(inp.q[b:b + 1].cpu(), kc, vc, ksc, vsc, inp.real_seqlen_kv[b:b + 1].cpu(),
                                     inp.block_table[b:b + 1].cpu(), 64)
        close(o[b:b + 1], ref, atol=FP8_ATOL, rtol=0.0)
    # attention over a sequence == LSE merge of attention over its two halves, for every row
    half = torch.full_like(inp.real_seqlen_kv, 2048)
    o1, l1 = decode(inp, lens=half, return_lse=True, out_dtype=torch.float32)
    bt2 = torch.zeros_like(inp.block_table)
    bt2[:, :32] = inp.block_table[:, 32:]
    o2, l2 = decode(inp, lens=half, bt=bt2, return_lse=True, out_dtype=torch.float32)
    merged, ml = F.gqa_lse_merge(torch.stack([o1, o2]), torch.stack([l1, l2]), torch.float32, return_lse=True)
    torch.testing.assert_close(merged, o, atol=2e-3, rtol=1e-2)
    torch.testing.assert_close(ml, lse, atol=1e-4, rtol=1e-5)
    # the bf16 output the operator returns
    close(decode(inp), o, atol=1e-2, rtol=1e-2)


def test_long_context_workload_at_full_size_and_its_shard_merges():
    inp = W.baseline_config(5, "cuda")
    B, H, D = inp.q.shape
    Hkv, page, ctx = inp.k.shape[1], inp.page_size, 131072
    assert (B, H, D, Hkv, page) == (8, 32, 128, 8, 128)
    o, lse = decode(inp, return_lse=True, out_dtype=torch.float32)
    assert not torch.isnan(o).any()
    g = H // Hkv
    for b, hk in ((0, 0), (5, 3), (7, 7)):
        ref, rl = O.paged_decode_ref(inp.q[b:b + 1, hk * g:(hk + 1) * g].cpu().float(), inp.k[:, hk:hk + 1].cpu().float(),
                                     inp.v[:, hk:hk + 1].cpu().float(), inp.real_seqlen_kv[b:b + 1].cpu(),
                                     inp.block_table[b:b + 1].cpu(), page, return_lse=True)
        close(o[b:b + 1, hk * g:(hk + 1) * g], ref)
        torch.testing.assert_close(lse[b:b + 1, hk * g:(hk + 1) * g].cpu(), rl, atol=2e-3, rtol=1e-3)
    # KV-sequence shards over 2 / 4 / 8 ranks, computed on this GPU and merged with the cross-rank merge kernel
    for world in (2, 4, 8):
        parts_o, parts_l = [], []
        for r in range(world):
            p0, p1 = shard_page_range(ctx // page, r, world)
            lens_r = (inp.real_seqlen_kv - p0 * page).clamp(min=0, max=(p1 - p0) * page).to(torch.int32)
            po, pl = decode(inp, lens=lens_r, bt=inp.block_table[:, p0:p1].contiguous(), return_lse=True,
                            out_dtype=torch.float32)
            parts_o.append(po); parts_l.append(pl)
        merged, ml = F.gqa_lse_merge(torch.stack(parts_o), torch.stack(parts_l), torch.float32, return_lse=True)
        torch.testing.assert_close(merged, o, atol=2e-3, rtol=1e-2)
        torch.testing.assert_close(ml, lse, atol=1e-4, rtol=1e-5)


@pytest.mark.parametrize("fp8", [False, True])
def test_tma_kernel_and_cp_async_kernel_agree(fp8):
    inp = W.make_paged_decode(71, 24, 32, 8, 128, 64, len_range=(1, 6000), fp8_cache=fp8, device="cuda", spare_pages=2,
                              tail_fill=float("nan"))
    a, la = decode(inp, return_lse=True, out_dtype=torch.float32, config={"tma": True})
    assert F.decode_last_kernel() == "tma"
    b, lb = decode(inp, return_lse=True, out_dtype=torch.float32, config={"tma": False})
    assert F.decode_last_kernel() == "cp_async"
    assert not torch.isnan(a).any() and not torch.isnan(b).any()
    torch.testing.assert_close(a, b, atol=2e-3, rtol=1e-2)
    torch.testing.assert_close(la, lb, atol=1e-4, rtol=1e-5)
    if not fp8:
        close(a, O.paged_decode_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv.cpu(),
                                    inp.block_table.cpu(), 64))


@pytest.mark.parametrize("page,D,dtype", [(16, 128, torch.bfloat16), (32, 128, torch.float16), (16, 64, torch.bfloat16),
                                          (32, 64, torch.bfloat16)])
def test_small_pages_through_the_tma_kernel(page, D, dtype):
    """Pages of 16 and 32 tokens: a 64-token tile is four or two copies of one page each.  Ragged lengths
    whose last tile reaches past the sequence's own pages, NaN behind every sequence end, and a block table
    that is exactly as wide as the longest sequence needs (a lookup behind a sequence's pages would leave the
    row, or the tensor)."""
    lens = [1, 15, 16, 17, 63, 64, 65, 100, 1000, 2049, 4096 + 33, 0]
    inp = W.make_paged_decode(73, len(lens), 32, 8, D, page, lens=lens, dtype=dtype, device="cuda",
                              tail_fill=float("nan"))
    assert inp.block_table.shape[1] == -(-max(lens) // page)
    a, la = decode(inp, return_lse=True, out_dtype=torch.float32, config={"tma": True})
    assert F.decode_last_kernel() == "tma"
    b, lb = decode(inp, return_lse=True, out_dtype=torch.float32, config={"tma": False})
    assert F.decode_last_kernel() == "cp_async"
    live = [i for i, n in enumerate(lens) if n > 0]
    assert not torch.isnan(a[live]).any() and not torch.isnan(b[live]).any()
    torch.testing.assert_close(a[live], b[live], atol=2e-3, rtol=1e-2)
    torch.testing.assert_close(la[live], lb[live], atol=1e-4, rtol=1e-5)
    close(a[live], O.paged_decode_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv.cpu(),
                                      inp.block_table.cpu(), page)[live])


@pytest.mark.parametrize("page", [16, 32])
def test_small_pages_of_an_fp8_cache_through_the_tma_kernel(page):
    """An e4m3 cache with pages of 16 / 32 tokens has four / two scale pairs per 64-token tile; every page gets
    a scale of its own magnitude here, so a warp that took a neighbouring page's scale would be far off."""
    lens = [1, 17, 64, 100, 1000, 2049, 0]
    inp = W.make_paged_decode(74, len(lens), 64, 8, 128, page, lens=lens, fp8_cache=True, device="cuda")
    # spread the scales over a factor of 8 (downwards, so that the outputs stay O(1)): the oracle and both
    # kernels dequantise with the same (page, head) scales
    g = torch.Generator(device="cuda").manual_seed(5)
    factor = torch.exp2(torch.randint(-3, 1, inp.k_scale.shape, generator=g, device="cuda").float())
    inp.k_scale = (inp.k_scale * factor).contiguous()
    inp.v_scale = (inp.v_scale * factor.flip(0)).contiguous()
    a, la = decode(inp, return_lse=True, out_dtype=torch.float32, config={"tma": True})
    assert F.decode_last_kernel() == "tma"
    b, lb = decode(inp, return_lse=True, out_dtype=torch.float32, config={"tma": False})
    assert F.decode_last_kernel() == "cp_async"
    live = [i for i, n in enumerate(lens) if n > 0]
    assert not torch.isnan(a[live]).any()
    torch.testing.assert_close(a[live], b[live], atol=5e-3, rtol=1e-2)
    torch.testing.assert_close(la[live], lb[live], atol=1e-3, rtol=1e-4)
    ref = O.paged_decode_fp8_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.k_scale.cpu(), inp.v_scale.cpu(),
                                 inp.real_seqlen_kv.cpu(), inp.block_table.cpu(), page)
    close(a[live], ref[live], atol=FP8_ATOL)


@pytest.mark.parametrize("tma", [True, False])
def test_fixed_run_lengths_give_the_result_of_the_cost_model(tma):
    """One run per sequence, two, and as many as the workspace admits: the merged result must not depend
    on the split (up to the bf16 rounding of P, which depends on each run's running maximum)."""
    inp = W.make_paged_decode(72, 6, 32, 8, 128, 64, len_range=(2000, 9000), device="cuda")
    base, lb = decode(inp, return_lse=True, out_dtype=torch.float32, config={"tma": tma})
    for chunk in (4096, 70, 2):
        o, l = decode(inp, return_lse=True, out_dtype=torch.float32, config={"tma": tma, "chunk_tiles": chunk})
        torch.testing.assert_close(o, base, atol=2e-3, rtol=1e-2)
        torch.testing.assert_close(l, lb, atol=1e-4, rtol=1e-5)
        again = decode(inp, out_dtype=torch.float32, config={"tma": tma, "chunk_tiles": chunk})
        assert torch.equal(o, again)          # same split: bit-identical, whoever ran which run


def test_many_short_segments_per_cta_are_bit_reproducible():
    """Forced run lengths of 2 and 3 tiles make every CTA of the TMA kernel walk a dozen short segments, most of
    them partial: 150 launches each must give the same bits (a barrier of the math warps at which only one
    lane per warp arrived let the last stores of the other lanes be read too early: one lane's last 16 head dims
    came out as the previous segment's in 1-10 % of such launches).  Lengths one past a tile boundary make the
    segments shortest."""
    lens = [n // 64 * 64 + 1 for n in W.draw_lengths(72, 6, (2000, 9000))]
    inp = W.make_paged_decode(72, 6, 32, 8, 128, 64, lens=lens, device="cuda")
    want = decode(inp, out_dtype=torch.float32, config={"tma": True, "chunk_tiles": 4096})
    for chunk in (3, 7):
        cfg = {"tma": True, "chunk_tiles": chunk}
        base = decode(inp, out_dtype=torch.float32, config=cfg).clone()
        assert F.decode_last_kernel() == "tma"
        torch.testing.assert_close(base, want, atol=2e-3, rtol=1e-2)
        odd = sum(0 if torch.equal(decode(inp, out_dtype=torch.float32, config=cfg), base) else 1 for _ in range(150))
        assert odd == 0, f"{odd} of 150 launches with runs of {chunk} tiles differ from the first"


def test_contiguous_cache_through_the_tma_kernel():
    B, H, Hkv, S, D = 5, 32, 8, 3000, 128
    q, k, v = W.make_contiguous_decode(73, B, H, Hkv, S, D, torch.bfloat16, "cuda")
    kn, vn = k.clone(), v.clone()
    kn[:, 2777:] = float("nan"); vn[:, 2777:] = float("nan")
    ref = O.decode_ref(q.cpu(), k[:, :2777].cpu(), v[:, :2777].cpu())
    for tma in (True, False):
        close(F.gqa_decode(q, kn, vn, real_seqlen_kv=2777, config={"tma": tma}), ref)
    # the last tile of the last sequence runs past the end of the tensor: the copy engine fills zeros there
    close(F.gqa_decode(q, k, v, real_seqlen_kv=S), O.decode_ref(q.cpu(), k.cpu(), v.cpu()))


def test_large_batches_reach_the_multi_pass_plan():
    # more sequences than planning threads, ragged and short, with empty ones
    g = torch.Generator().manual_seed(9)
    lens = torch.randint(0, 400, (300,), generator=g).tolist()
    lens[3] = 0; lens[299] = 0
    inp = W.make_paged_decode(74, 300, 16, 4, 128, 64, lens=lens, device="cuda", tail_fill=float("nan"))
    ref = O.paged_decode_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv.cpu(), inp.block_table.cpu(), 64)
    for tma in (True, False):
        close(decode(inp, config={"tma": tma}), ref)
    inp8 = W.make_paged_decode(75, 128, 32, 8, 128, 64, len_range=(1, 700), fp8_cache=True, device="cuda")
    ref8 = O.paged_decode_fp8_ref(inp8.q.cpu(), inp8.k.cpu(), inp8.v.cpu(), inp8.k_scale.cpu(), inp8.v_scale.cpu(),
                                  inp8.real_seqlen_kv.cpu(), inp8.block_table.cpu(), 64)
    for tma in (True, False):
        close(decode(inp8, config={"tma": tma}), ref8, atol=FP8_ATOL, rtol=0.0)


def test_batch_beyond_the_plan_capacity_is_refused():
    B = 4097
    q = torch.zeros(B, 8, 64, device="cuda", dtype=torch.bfloat16)
    k = torch.zeros(64, 2, 64, device="cuda", dtype=torch.bfloat16)
    lens = torch.zeros(B, dtype=torch.int32, device="cuda")
    bt = torch.zeros(B, 1, dtype=torch.int32, device="cuda")
    with pytest.raises(ValueError, match="exceeds"):
        F.gqa_decode(q, k, k, real_seqlen_kv=lens, block_table=bt, page_size=64)


def test_merge_wait_gives_up_and_poisons_its_rows():
    """Flags that nothing raises: the bounded wait of the cross-rank merge runs out by itself, records
    code 501 and writes NaN / -inf, and a launch that starts with the status set gives up at once."""
    rows, D, parts = 2, 128, 2
    n = rows * (D + 1)                                                    # one rank's slot: O rows, then their LSEs
    buf = torch.randn(2 * parts * n, device="cuda")                       # [2 parities][parts][slot]
    flags = torch.zeros(parts, dtype=torch.int32, device="cuda")
    step = torch.ones(1, dtype=torch.int32, device="cuda")                # the local decode "finished step 1"
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(rows, D, device="cuda")
    lse = torch.zeros(rows, device="cuda")

    def run(limit):
        st = N.lib().tb200_gqa_lse_merge_wait(buf.data_ptr(), buf.data_ptr() + rows * D * 4, out.data_ptr(), lse.data_ptr(),
                                              parts, rows, D, n, n, parts * n, N.F32, flags.data_ptr(),
                                              step.data_ptr(), status.data_ptr(), limit,
                                              torch.cuda.current_stream().cuda_stream)
        N.check(st, "tb200_gqa_lse_merge_wait")
        torch.cuda.synchronize()

    run(2_000_000)                                    # about a millisecond
    assert int(status.item()) == 501
    assert torch.isnan(out).all() and torch.isinf(lse).all()
    out.zero_()
    run(2_000_000_000)                                # status still set: returns at once, rows poisoned again
    assert torch.isnan(out).all()
    # the passing case: both flags at the step, parts of parity 1 merged
    status.zero_(); flags.fill_(1)
    run(2_000_000)
    assert int(status.item()) == 0
    odd = buf[parts * n:].view(parts, n).cpu()                           # step 1 uses the buffers of parity 1
    want, wl = O.merge_partials_ref(odd[:, :rows * D].reshape(parts, 1, rows, D), odd[:, rows * D:].reshape(parts, 1, rows))
    torch.testing.assert_close(out.cpu(), want[0], atol=1e-5, rtol=1e-5)
