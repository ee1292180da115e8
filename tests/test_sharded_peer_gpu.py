"""KV-sequence sharded decode with the exchange fused into the decode kernel (stores over NVLink into
every rank's symmetric buffer, flag, bounded wait in the merge): two ranks on two GPUs, compared bit for bit
with the NCCL all-gather path, eagerly and replayed from a CUDA graph.  Needs two GPUs (skipped otherwise)."""

import os
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, faulthandler, torch, torch.distributed as dist
    faulthandler.dump_traceback_later(150, exit=True)
    sys.path.insert(0, os.getcwd())
    from tileops_b200 import workloads as W
    from tileops_b200.sharded import KVSequenceShardedPagedDecode, shard_page_range
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    B, H, Hkv, D, page, ctx = 4, 32, 8, 128, 128, 8192
    p0, p1 = shard_page_range(ctx // page, rank, world)
    inp = W.make_paged_decode(5, B, H, Hkv, D, page, lens=[ctx, 5000, 300, 8000], device=dev, page_begin=p0, page_end=p1)
    nccl = KVSequenceShardedPagedDecode(B, H, Hkv, D, page)
    peer = KVSequenceShardedPagedDecode(B, H, Hkv, D, page)
    peer.enable_peer_exchange(dev)
    args = (inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    for step in range(5):                       # consecutive steps alternate the buffer parity
        inp.q.mul_(0.9).add_(0.01 * step)
        a = nccl(*args).clone()
        b = peer(*args).clone()
        assert torch.equal(a, b), f"step {step}: fused exchange differs from the all-gather path"
    g = peer.graphed(*args)
    for step in range(3):
        inp.q.mul_(1.05)
        assert torch.equal(g().clone(), nccl(*args)), f"graph replay {step} differs"
    assert peer.peer_status() == 0
    del g
    peer._peer = None
    # a slot whose size is no multiple of 16 bytes (batch * heads * (D + 1) floats with batch * heads = 18): the
    # decode kernel then stores its result to the peers in 4-byte pieces instead of 16-byte ones
    B2, H2, Hkv2 = 3, 6, 2
    p0, p1 = shard_page_range(4096 // page, rank, world)
    inp2 = W.make_paged_decode(6, B2, H2, Hkv2, D, page, lens=[4096, 1000, 130], device=dev, page_begin=p0, page_end=p1)
    nccl2 = KVSequenceShardedPagedDecode(B2, H2, Hkv2, D, page)
    peer2 = KVSequenceShardedPagedDecode(B2, H2, Hkv2, D, page)
    peer2.enable_peer_exchange(dev)
    args2 = (inp2.q, inp2.k, inp2.v, inp2.real_seqlen_kv, inp2.block_table)
    for step in range(3):
        inp2.q.mul_(0.9).add_(0.01 * step)
        assert torch.equal(nccl2(*args2), peer2(*args2)), f"odd slot size, step {step}: fused exchange differs"
    assert peer2.peer_status() == 0
    peer2._peer = None
    torch.cuda.synchronize()
    dist.barrier()
    dist.destroy_process_group()
    print("PEER-OK", rank, flush=True)
""")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_peer_exchange_matches_nccl_path(tmp_path):
    script = tmp_path / "peer_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run(
        [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", "29541", str(script)],
        cwd=ROOT, env=env, capture_output=True, text=True, timeout=280)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count("PEER-OK") == 2
