"""Seeded random paged-decode problems against the oracle: every combination of the dimensions that select a
code path (page size 16 ... 256, head dim 64 / 128, 1 ... 16 q heads per KV head, 16-bit or e4m3 cache, softcap,
ragged lengths from 0 up, a block table wider than needed) that a hand-written case list would not enumerate.

Acceptance as in the reference's paged-decode test (tests/ops/attention/test_gqa_decode_paged.py:75-151 in
tile-ai/TileOPs): 2e-2 abs / 1e-2 rel for 16-bit caches, 3e-2 abs for an e4m3 cache.
"""

import random

import pytest
import torch

from oracle import gqa_oracle as O
from tileops_b200 import functional as F
from tileops_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _case(seed: int):
    rng = random.Random(1235 + seed)
    dim = rng.choice([64, 128])
    fp8 = dim == 128 and rng.random() < 0.35
    heads_kv = rng.choice([1, 2, 4, 8])
    group = rng.choice([1, 2, 4, 5, 8, 12, 16])
    page = rng.choice([16, 32, 64, 128, 256])
    batch = rng.choice([1, 2, 3, 7, 19])
    top = rng.choice([40, 300, 1500, 5000])
    lens = [rng.choice([0, 1, page - 1, page, page + 1, rng.randint(1, top)]) for _ in range(batch)]
    if max(lens) == 0:
        lens[0] = rng.randint(1, top)
    dtype = torch.float16 if fp8 or rng.random() < 0.5 else torch.bfloat16
    softcap = rng.choice([0.0, 0.0, 30.0])
    return dict(dim=dim, fp8=fp8, heads_kv=heads_kv, heads=heads_kv * group, page=page, lens=lens, dtype=dtype,
                softcap=softcap, spare=rng.choice([0, 3]))


@pytest.mark.parametrize("seed", range(32))
def test_random_paged_decode_matches_the_oracle(seed):
    c = _case(seed)
    inp = W.make_paged_decode(200 + seed, len(c["lens"]), c["heads"], c["heads_kv"], c["dim"], c["page"], lens=c["lens"],
                              dtype=c["dtype"], fp8_cache=c["fp8"], device="cuda", spare_pages=c["spare"],
                              tail_fill=float("nan"))
    kw = dict(k_scale=inp.k_scale, v_scale=inp.v_scale) if c["fp8"] else {}
    got, lse = F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv, block_table=inp.block_table,
                            page_size=c["page"], softcap=c["softcap"], return_lse=True, out_dtype=torch.float32, **kw)
    live = [i for i, n in enumerate(c["lens"]) if n > 0]
    dead = [i for i, n in enumerate(c["lens"]) if n == 0]
    assert not torch.isnan(got[live]).any(), f"NaN in the output of {c} (kernel {F.decode_last_kernel()})"
    if c["fp8"]:
        want = O.paged_decode_fp8_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.k_scale.cpu(), inp.v_scale.cpu(),
                                      inp.real_seqlen_kv.cpu(), inp.block_table.cpu(), c["page"],
                                      softcap=c["softcap"] or None)
        tol = dict(atol=3e-2, rtol=1e-2)
    else:
        want = O.paged_decode_ref(inp.q.cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv.cpu(), inp.block_table.cpu(),
                                  c["page"], softcap=c["softcap"] or None)
        tol = dict(atol=2e-2, rtol=1e-2)
    torch.testing.assert_close(got[live].cpu().float(), want[live].float(), **tol)
    if dead:   # a sequence without a token: zeros, LSE -inf
        assert torch.count_nonzero(got[dead]) == 0
        assert torch.isinf(lse[dead]).all()
    # the other kernel agrees (whichever served the call first)
    first = F.decode_last_kernel()
    other = F.gqa_decode(inp.q, inp.k, inp.v, real_seqlen_kv=inp.real_seqlen_kv, block_table=inp.block_table,
                         page_size=c["page"], softcap=c["softcap"], out_dtype=torch.float32,
                         config={"tma": first != "tma"}, **kw)
    torch.testing.assert_close(other[live], got[live], atol=4e-3, rtol=1e-2)
