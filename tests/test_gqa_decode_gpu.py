"""GPU parity tests of the decode path: op (-> kernel class -> C ABI -> CUDA kernel) against
the CPU oracle on identical seeded inputs.

Tolerances: bf16/fp16 outputs within 2e-2 abs / 1e-2 rel of the fp32 reference; FP8-cache
outputs within 3e-2 abs of dequantise-then-attend; block-table gathers bit-exact.  The shapes
follow the reference's own tests (tests/ops/attention/test_gqa_decode.py:16-38,
test_gqa_decode_paged.py:75-151 in tile-ai/TileOPs) plus ragged, empty and permuted cases.
"""

import numpy as np
import pytest
import torch

from oracle import gqa_oracle as O
from tileops_b200 import functional as F
from tileops_b200 import workloads as W
from tileops_b200.ops import (
    GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp,
    GroupedQueryAttentionDecodePagedWithKVCacheFwdOp,
    GroupedQueryAttentionDecodeWithKVCacheFwdOp,
)

pytestmark = pytest.mark.gpu
ATOL, RTOL = 2e-2, 1e-2
FP8_ATOL = 3e-2


def close(got, want, atol=ATOL, rtol=RTOL):
    got, want = got.float().cpu(), want.float().cpu()
    assert not torch.isnan(got).any(), "NaN in kernel output"
    torch.testing.assert_close(got, want, atol=atol, rtol=rtol)


def cpu(inp):
    return (inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv.cpu(), inp.block_table.cpu())


# ---------------------------------------------------------------- contiguous decode
@pytest.mark.parametrize("B,H,Hkv,S,D,dtype", [
    (2, 8, 2, 256, 64, torch.bfloat16),          # the reference's CPU-runnable decode case
    (1, 32, 8, 8192, 128, torch.float16),
    (1, 32, 8, 8192, 128, torch.bfloat16),
    (1, 16, 2, 8192, 128, torch.float16),
    (8, 64, 16, 1024, 128, torch.float16),
    (1, 32, 4, 6000, 128, torch.float16),        # unaligned length
    (3, 8, 8, 77, 64, torch.bfloat16),           # MHA (group 1), ragged tile
    (1, 128, 8, 300, 128, torch.bfloat16),       # group 16: two head tiles
    (1, 96, 2, 130, 64, torch.float16),          # group 48: three head blocks
])
def test_decode_op_matches_oracle(B, H, Hkv, S, D, dtype):
    q, k, v = W.make_contiguous_decode(1, B, H, Hkv, S, D, dtype, "cuda")
    op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(B, H, Hkv, S, D)
    o = op(q, k, v)
    assert o.shape == q.shape and o.dtype == dtype
    close(o, O.decode_ref(q.cpu(), k.cpu(), v.cpu()))
    assert op.eval_roofline()[0] == 4 * B * H * S * D


@pytest.mark.parametrize("sm_scale,softcap", [(0.25, None), (None, 2.0), (0.3, 50.0)])
def test_decode_op_scale_and_softcap(sm_scale, softcap):
    B, H, Hkv, S, D = 2, 32, 8, 1000, 128
    q, k, v = W.make_contiguous_decode(2, B, H, Hkv, S, D, torch.float16, "cuda")
    op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(B, H, Hkv, S, D, sm_scale=sm_scale, softcap=softcap)
    close(op(q, k, v), O.decode_ref(q.cpu(), k.cpu(), v.cpu(), sm_scale, softcap))


def test_decode_live_length_below_capacity_reads_no_padding():
    B, H, Hkv, S, D = 2, 8, 2, 256, 64
    q, k, v = W.make_contiguous_decode(1, B, H, Hkv, S, D, torch.bfloat16, "cuda")
    op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(B, H, Hkv, S, D)
    close(op(q, k[:, :100], v[:, :100]), O.decode_ref(q.cpu(), k[:, :100].cpu(), v[:, :100].cpu()))
    kn, vn = k.clone(), v.clone()
    kn[:, 100:] = float("nan"); vn[:, 100:] = float("nan")
    o = F.gqa_decode(q, kn, vn, real_seqlen_kv=100)
    close(o, O.decode_ref(q.cpu(), k[:, :100].cpu(), v[:, :100].cpu()))


def test_decode_golden_config1():
    import os
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "gqa_golden.npz"))
    q, k, v = (torch.from_numpy(G[n]).cuda().bfloat16() for n in ("dec_q", "dec_k", "dec_v"))
    op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(2, 8, 2, 256, 64)
    close(op(q, k, v), torch.from_numpy(G["dec_o"]))       # fp32 reference output of the reference
    op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(2, 8, 2, 256, 64, softcap=2.0)
    close(op(q, k, v), torch.from_numpy(G["dec_o_softcap2"]))


# ---------------------------------------------------------------- paged decode
@pytest.mark.parametrize("B,H,Hkv,D,page,lens,dtype", [
    (1, 16, 8, 128, 128, [512], torch.float16),
    (2, 8, 4, 64, 256, [1024, 700], torch.float16),
    (1, 32, 8, 128, 64, [256], torch.float16),
    (2, 16, 8, 128, 128, [512, 300], torch.bfloat16),
    (1, 16, 4, 128, 512, [2048], torch.float16),
    (1, 32, 16, 64, 128, [512], torch.float16),
    (1, 16, 4, 128, 192, [3072], torch.float16),            # page 192: 64-token tiles inside a page
    (3, 8, 2, 64, 16, [37, 64, 5], torch.bfloat16),         # small pages, several pages per tile
    (4, 64, 8, 128, 64, [4096, 100, 2049, 777], torch.bfloat16),
    (3, 32, 8, 128, 64, [1000, 0, 1], torch.bfloat16),      # empty sequence, single token
    (2, 32, 8, 128, 32, [513, 31], torch.float16),
    (16, 32, 8, 128, 64, None, torch.bfloat16),             # ragged batch, split-KV merge
])
def test_paged_decode_op_matches_oracle(B, H, Hkv, D, page, lens, dtype):
    kw = dict(lens=lens) if lens is not None else dict(len_range=(1, 3000))
    inp = W.make_paged_decode(11, B, H, Hkv, D, page, dtype=dtype, device="cuda",
                              tail_fill=float("nan"), spare_pages=3, **kw)
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(B, H, Hkv, inp.k.shape[0], D, page)
    o = op(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    assert o.shape == inp.q.shape and o.dtype == dtype
    close(o, O.paged_decode_ref(*cpu(inp), page))
    # reference's own acceptance form: max-abs and per-sequence cosine (test_gqa_decode_paged.py:17-28)
    ref = O.paged_decode_ref(*cpu(inp), page).float()
    live = torch.tensor(inp.lens) > 0
    cos = torch.nn.functional.cosine_similarity(o.float().cpu().reshape(B, -1)[live], ref.reshape(B, -1)[live], dim=-1)
    assert cos.min() > 0.99


def test_paged_decode_reversed_block_table():
    # tests/ops/attention/test_gqa_decode_paged.py:122-140: reversed page order
    B, H, Hkv, D, page, n_pages = 1, 16, 4, 128, 192, 16
    q = torch.randn(B, H, D, device="cuda", dtype=torch.float16)
    k = torch.randn(n_pages * page, Hkv, D, device="cuda", dtype=torch.float16)
    v = torch.randn_like(k)
    lens = torch.full((B,), n_pages * page, dtype=torch.int32, device="cuda")
    bt = torch.arange(n_pages, device="cuda", dtype=torch.int32).flip(0).unsqueeze(0).contiguous()
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(B, H, Hkv, n_pages * page, D, page)
    assert page % op._get_kernel((), torch.float16).config["block_N"] == 0
    close(op(q, k, v, lens, bt), O.paged_decode_ref(q.cpu(), k.cpu(), v.cpu(), lens.cpu(), bt.cpu(), page))


def test_paged_gather_is_bit_exact_on_integer_coded_pages():
    """With one-hot attention (one key dominates) the output row IS a V row of the pool, so a
    wrong page or row index shows up as a wrong integer code, not as a tolerance question."""
    B, H, Hkv, D, page = 4, 8, 2, 64, 16
    lens = [70, 16, 33, 129]
    inp = W.make_paged_decode(12, B, H, Hkv, D, page, lens=lens, dtype=torch.bfloat16, device="cuda",
                              spare_pages=5)
    N = inp.k.shape[0]
    codes = torch.arange(N, device="cuda") % 251
    inp.v[:] = codes[:, None, None].to(torch.bfloat16)              # V row = its physical row code
    inp.k.zero_()
    inp.q.zero_(); inp.q[..., 0] = 1.0
    g = torch.Generator().manual_seed(5)
    want = torch.empty(B, dtype=torch.int64)
    for b in range(B):
        t = int(torch.randint(0, lens[b], (1,), generator=g))
        row = int(O.physical_rows(inp.block_table[b].cpu().numpy(), lens[b], page)[t])
        inp.k[row, :, 0] = 200.0                                      # this token wins the softmax
        want[b] = row % 251
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(B, H, Hkv, N, D, page, sm_scale=1.0)
    o = op(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table).float().cpu()
    for b in range(B):
        assert torch.all(o[b] == float(want[b])), (b, o[b, 0, :4], want[b])


def test_paged_decode_scale_softcap_and_lse():
    inp = W.make_paged_decode(13, 3, 32, 8, 128, 64, lens=[700, 64, 2000], device="cuda")
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(3, 32, 8, inp.k.shape[0], 128, 64, sm_scale=0.2, softcap=2.0)
    close(op(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table),
          O.paged_decode_ref(*cpu(inp), 64, sm_scale=0.2, softcap=2.0))
    o, lse = F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv, block_table=inp.block_table,
                          page_size=64, return_lse=True, out_dtype=torch.float32)
    ro, rl = O.paged_decode_ref(inp.q.cpu().float(), inp.k.cpu().float(), inp.v.cpu().float(),
                                inp.real_seqlen_kv.cpu(), inp.block_table.cpu(), 64, return_lse=True)
    close(o, ro)
    torch.testing.assert_close(lse.cpu(), rl, atol=2e-3, rtol=1e-3)


def test_paged_decode_repeated_calls_are_bit_identical_per_work_split():
    """The scheduler is dynamic; the merge order of split-KV partials is fixed, so the result
    must not depend on which CTA ran which run."""
    inp = W.make_paged_decode(14, 8, 32, 8, 128, 64, len_range=(3000, 9000), device="cuda")
    op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(8, 32, 8, inp.k.shape[0], 128, 64)
    a = op(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    for _ in range(3):
        b = op(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
        assert torch.equal(a, b)


# ---------------------------------------------------------------- FP8 cache
@pytest.mark.parametrize("B,H,Hkv,D,page,lens,dtype", [
    (2, 64, 8, 128, 64, [300, 1024], torch.bfloat16),
    (3, 32, 8, 128, 64, [64, 65, 2000], torch.bfloat16),
    (2, 16, 4, 64, 16, [100, 33], torch.bfloat16),
    (2, 64, 8, 128, 128, [4096, 0], torch.float16),
    (1, 128, 8, 128, 64, [777], torch.bfloat16),
])
def test_paged_decode_fp8_cache_matches_dequantise_then_attend(B, H, Hkv, D, page, lens, dtype):
    inp = W.make_paged_decode(15, B, H, Hkv, D, page, lens=lens, dtype=dtype, fp8_cache=True,
                              device="cuda", spare_pages=2)
    op = GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp(B, H, Hkv, inp.k.shape[0], D, page)
    o = op(inp.q, inp.k, inp.v, inp.k_scale, inp.v_scale, inp.real_seqlen_kv, inp.block_table)
    ref = O.paged_decode_fp8_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.k_scale.cpu(), inp.v_scale.cpu(),
                                 inp.real_seqlen_kv.cpu(), inp.block_table.cpu(), page)
    close(o, ref, atol=FP8_ATOL, rtol=0.0)


def test_fp8_expansion_is_exact_for_every_byte():
    """All 256 e4m3 codes (NaN codes excluded) pass through the in-register expansion: a
    one-hot softmax returns V rows, which must equal float(code) * scale exactly in bf16."""
    H, Hkv, D, page = 8, 1, 128, 64
    codes = torch.arange(256, dtype=torch.uint8)
    codes = codes[(codes & 0x7F) != 0x7F]                               # 0x7F / 0xFF are NaN
    vals = codes.view(torch.float8_e4m3fn)
    n = codes.numel()
    rows = 2 * page
    v = torch.zeros(rows, Hkv, D, dtype=torch.uint8)
    for r in range(rows):
        v[r, 0] = codes[(torch.arange(D) + r * 7) % n]
    v8 = v.view(torch.float8_e4m3fn).cuda()
    k8 = torch.zeros_like(v8)
    scale = torch.tensor([[0.5], [0.015625]], device="cuda")
    q = torch.zeros(1, H, D, device="cuda", dtype=torch.bfloat16); q[..., 0] = 64  # score >= 448: one-hot
    for r in (0, 63, 64, 127):
        kk = k8.clone().view(torch.uint8); kk[r, 0, 0] = 0x7E            # 448: wins the softmax
        out = F.gqa_decode(q, kk.view(torch.float8_e4m3fn), v8, real_seqlen_kv=torch.tensor([rows], dtype=torch.int32, device="cuda"),
                           block_table=torch.tensor([[0, 1]], dtype=torch.int32, device="cuda"), page_size=page,
                           k_scale=scale, v_scale=scale, sm_scale=1.0, out_dtype=torch.float32)
        want = v8[r, 0].float().cpu() * float(scale[r // page, 0])
        assert torch.equal(out[0, 0].cpu(), want), r


# ---------------------------------------------------------------- full-size properties
def test_split_merge_property_at_config3_size():
    """The paged bf16 decode workload (64 ragged sequences) at full size: (a) three sequences against the oracle; (b) attention
    over a sequence equals the LSE-merge of attention over its two halves, for every row."""
    inp = W.baseline_config(3, "cuda")
    B = 64
    o, lse = F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv, block_table=inp.block_table,
                          page_size=64, return_lse=True, out_dtype=torch.float32)
    for b in (0, 17, 63):
        ref = O.paged_decode_ref(inp.q[b:b + 1].cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv[b:b + 1].cpu(),
                                 inp.block_table[b:b + 1].cpu(), 64)
        close(o[b:b + 1], ref)
    half = (inp.real_seqlen_kv // 128) * 64                                # page-aligned first half
    o1, l1 = F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=half.to(torch.int32), block_table=inp.block_table,
                          page_size=64, return_lse=True, out_dtype=torch.float32)
    bt2 = torch.zeros_like(inp.block_table)
    for b in range(B):
        s = int(half[b]) // 64
        bt2[b, :inp.block_table.shape[1] - s] = inp.block_table[b, s:]
    o2, l2 = F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=(inp.real_seqlen_kv - half).to(torch.int32),
                          block_table=bt2, page_size=64, return_lse=True, out_dtype=torch.float32)
    merged, ml = F.gqa_lse_merge(torch.stack([o1, o2]), torch.stack([l1, l2]), torch.float32, return_lse=True)
    # P is rounded to bf16 before the PV product, differently for different running maxima,
    # so the two evaluations agree to bf16-P noise, not to fp32 round-off
    torch.testing.assert_close(merged, o, atol=2e-3, rtol=1e-2)
    torch.testing.assert_close(ml, lse, atol=1e-4, rtol=1e-5)
    mo, _ = O.merge_partials_ref(torch.stack([o1, o2]).cpu(), torch.stack([l1, l2]).cpu())
    torch.testing.assert_close(merged.cpu(), mo, atol=1e-5, rtol=1e-5)


def test_merge_handles_empty_parts():
    o_parts = torch.randn(3, 4, 8, 64, device="cuda")
    lse = torch.randn(3, 4, 8, device="cuda")
    lse[1] = float("-inf"); lse[2, 0] = -1e30
    lse[:, 3] = float("-inf")
    got, gl = F.gqa_lse_merge(o_parts, lse, torch.float32, return_lse=True)
    want, wl = O.merge_partials_ref(o_parts.cpu(), lse.cpu())
    torch.testing.assert_close(got.cpu(), want, atol=1e-6, rtol=1e-5)
    assert torch.all(got[3] == 0) and torch.all(torch.isinf(gl[3]))


def test_sharded_decode_graph_replay_matches_eager():
    # single rank: the captured step is the decode launch and the merge launch (the all-gather joins at
    # world size > 1); a replay must see tensors updated in place
    from tileops_b200.sharded import KVSequenceShardedPagedDecode
    inp = W.make_paged_decode(61, 4, 32, 8, 128, 64, len_range=(300, 3000), device="cuda")
    op = KVSequenceShardedPagedDecode(4, 32, 8, 128, 64)
    args = (inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    eager = op(*args).clone()
    replay = op.graphed(*args)
    assert torch.equal(replay(), eager)
    inp.q.mul_(0.5)
    want = op(*args).clone()
    assert torch.equal(replay(), want) and not torch.equal(want, eager)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_wide_variant_for_long_capacity_caches(dtype):
    # 3 CTAs per SM with a 2-stage ring: chosen by the library when a sequence may hold >= 16k tokens;
    # forced here on a ragged batch, and reached naturally by a table with 16k-token capacity
    inp = W.make_paged_decode(62, 6, 32, 8, 128, 64, len_range=(100, 5000), dtype=dtype, device="cuda")
    ref = O.paged_decode_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv.cpu(), inp.block_table.cpu(), 64)
    o = F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv, block_table=inp.block_table, page_size=64,
                     config={"wide": True})
    close(o, ref)
    long = W.make_paged_decode(63, 2, 16, 4, 128, 128, lens=[16384, 9000], dtype=dtype, device="cuda")
    assert long.block_table.shape[1] * 128 >= 16384
    o = F.gqa_decode(long.q, long.k, long.v, real_seqlen_kv=long.real_seqlen_kv, block_table=long.block_table,
                     page_size=128)
    close(o, O.paged_decode_ref(long.q.cpu(), long.k.cpu(), long.v.cpu(), long.real_seqlen_kv.cpu(),
                                long.block_table.cpu(), 128))
