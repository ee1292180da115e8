"""World-size-2 (and 3) CPU ranks over gloo exercise the KV-sequence sharding protocol:
page-range partition, local problem construction, packing into the communication buffer,
all-gather layout and the merge of (O, LSE) including an empty shard.  The compute callables
are the CPU oracle here (test-only injection); on GPUs the same class runs the CUDA kernels."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gqa_oracle as O
from tileops_b200 import workloads as W
from tileops_b200.sharded import KVSequenceShardedPagedDecode, shard_page_range

B, H, HKV, D, PAGE = 3, 8, 2, 32, 8
LENS = [100, 9, 41]          # 13, 2 and 6 pages: with 3 ranks the middle sequence leaves a rank empty


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        max_pages = max(-(-n // PAGE) for n in LENS)
        p0, p1 = shard_page_range(max_pages, rank, world)
        loc = W.make_paged_decode(21, B, H, HKV, D, PAGE, lens=LENS, dtype=torch.float32, device="cpu",
                                  page_begin=p0, page_end=p1, tail_fill=float("nan"))

        def decode_fn(q, k, v, lens, bt, out, lse_out):
            k2, v2 = torch.nan_to_num(k), torch.nan_to_num(v)
            o, l = O.paged_decode_ref(q, k2, v2, lens, bt, PAGE, return_lse=True)
            out.copy_(o); lse_out.copy_(l)

        def merge_fn(o_parts, lse_parts, dtype):
            return O.merge_partials_ref(o_parts.reshape(o_parts.shape[0], -1, D).contiguous(),
                                        lse_parts.reshape(lse_parts.shape[0], -1).contiguous())[0].reshape(B, H, D).to(dtype)

        op = KVSequenceShardedPagedDecode(B, H, HKV, D, PAGE, decode_fn=decode_fn, merge_fn=merge_fn)
        out = op(loc.q, loc.k, loc.v, loc.real_seqlen_kv, loc.block_table)
        full = W.make_paged_decode(21, B, H, HKV, D, PAGE, lens=LENS, dtype=torch.float32, device="cpu")
        ref = O.paged_decode_ref(full.q, full.k, full.v, full.real_seqlen_kv, full.block_table, PAGE)
        ret[rank] = float((out - ref).abs().max())
        if rank == world - 1:
            ret["lens_last"] = loc.lens
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_decode_protocol_over_gloo(world):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        for r in range(world):
            assert ret[r] < 1e-5, (r, ret[r])
        if world == 3:
            assert ret["lens_last"][1] == 0        # the short sequence has no page on the last rank


def test_shard_page_range_covers_everything_once():
    for n in (0, 1, 7, 8, 1024):
        for world in (1, 2, 3, 8):
            cuts = [shard_page_range(n, r, world) for r in range(world)]
            assert cuts[0][0] == 0 and cuts[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(cuts[:-1], cuts[1:]))
            assert max(e - b for b, e in cuts) - min(e - b for b, e in cuts) <= 1


# ---------------------------------------------------------------------------------------------
# failure paths, made on the host: a rank whose partial is poisoned, a rank that is late, a rank that
# raises before the exchange.  No GPU is involved; the survivors must either get the right answer or an
# error, never a silently wrong result and never a hang.
# ---------------------------------------------------------------------------------------------

def _failure_worker(rank, world, port, ret, mode):
    import datetime
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    try:
        max_pages = max(-(-n // PAGE) for n in LENS)
        p0, p1 = shard_page_range(max_pages, rank, world)
        loc = W.make_paged_decode(21, B, H, HKV, D, PAGE, lens=LENS, dtype=torch.float32, device="cpu",
                                  page_begin=p0, page_end=p1)

        def decode_fn(q, k, v, lens, bt, out, lse_out):
            if mode == "raise" and rank == 1:
                raise RuntimeError("injected: this rank fails before the exchange")
            if mode == "late" and rank == 1:
                time.sleep(1.5)
            o, l = O.paged_decode_ref(q, k, v, lens, bt, PAGE, return_lse=True)
            if mode == "nan_lse" and rank == 1:
                l = torch.full_like(l, float("nan"))
            if mode == "neg_inf_lse" and rank == 1:
                l = torch.full_like(l, float("-inf"))       # "this rank saw no token": a legal, empty part
                o = torch.full_like(o, 123.0)                # whatever it carries must not reach the result
            out.copy_(o); lse_out.copy_(l)

        def merge_fn(o_parts, lse_parts, dtype):
            return O.merge_partials_ref(o_parts.reshape(o_parts.shape[0], -1, D).contiguous(),
                                        lse_parts.reshape(lse_parts.shape[0], -1).contiguous())[0].reshape(B, H, D).to(dtype)

        op = KVSequenceShardedPagedDecode(B, H, HKV, D, PAGE, decode_fn=decode_fn, merge_fn=merge_fn)
        try:
            out = op(loc.q, loc.k, loc.v, loc.real_seqlen_kv, loc.block_table)
            ret[rank] = ("ok", out)
        except Exception as exc:  # noqa: BLE001 - the test inspects what each rank saw
            ret[rank] = ("error", type(exc).__name__ + ": " + str(exc)[:200])
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001 - a group whose peer died may refuse a clean shutdown
            pass


def _run_failure(mode, world=2):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_failure_worker, args=(world, port, ret, mode), nprocs=world, join=True)
        return {r: ret[r] for r in range(world)}


def _reference():
    full = W.make_paged_decode(21, B, H, HKV, D, PAGE, lens=LENS, dtype=torch.float32, device="cpu")
    return full, O.paged_decode_ref(full.q, full.k, full.v, full.real_seqlen_kv, full.block_table, PAGE)


def test_a_rank_with_nan_lse_poisons_the_result_on_every_rank():
    res = _run_failure("nan_lse")
    for r, (kind, out) in res.items():
        assert kind == "ok" and torch.isnan(out).all(), (r, kind)      # loud, and the same on every rank


def test_a_rank_with_an_empty_part_is_ignored():
    # rank 1 claims to have seen no token: the merge must equal attention over rank 0's pages alone
    res = _run_failure("neg_inf_lse")
    max_pages = max(-(-n // PAGE) for n in LENS)
    p0, p1 = shard_page_range(max_pages, 0, 2)
    loc = W.make_paged_decode(21, B, H, HKV, D, PAGE, lens=LENS, dtype=torch.float32, device="cpu", page_begin=p0, page_end=p1)
    want = O.paged_decode_ref(loc.q, loc.k, loc.v, loc.real_seqlen_kv, loc.block_table, PAGE)
    for r, (kind, out) in res.items():
        assert kind == "ok", (r, out)
        torch.testing.assert_close(out, want, atol=1e-5, rtol=1e-5)


def test_a_late_rank_only_delays_the_step():
    _, ref = _reference()
    res = _run_failure("late")
    for r, (kind, out) in res.items():
        assert kind == "ok", (r, out)
        torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-5)


def test_a_rank_that_raises_before_the_exchange_fails_the_others_within_the_group_timeout():
    res = _run_failure("raise")
    assert res[1][0] == "error" and "injected" in res[1][1]
    assert res[0][0] == "error", "the surviving rank must see an error from the collective, not a result"
