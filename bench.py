#!/usr/bin/env python
"""Benchmark of the GQA attention-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The headline
workload is BASELINE config 3 (paged bf16 decode, batch 64, 32/8 heads, D=128, context uniform
in [512, 8192], page 64, random-permutation block table); the metric is achieved HBM GB/s over
the algorithmic bytes (live K/V + q + o + block-table entries + lengths, each once).  The other
BASELINE configurations are timed too and reported under ``"others"`` in the same JSON line.

For N > 1 (launched by ``python -m torch.distributed.run``, one rank per GPU) every rank decodes
its own batch of the same shape (weak scaling; the path partitions by sequence with no
data-path collective); ``value`` is all ranks' bytes over the slowest rank's time.  The
KV-sequence-sharded long-context decode (config 5), which does have one exchange step, is
reported under ``"others"``.

``--impl reference`` times the reference's CPU implementation of the same workload (its torch
reference program, restated in ``oracle/`` because the reference tree is not on the GPU box)
on the host cores, on a bounded sample.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "paged_decode_hbm_gbs"
UNIT = "GB/s"
FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0

# DRAM traffic per launch relative to the algorithmic bytes, from the ncu capture summarised in
# profiles/ (dram__bytes_read.sum + dram__bytes_write.sum of gqa_decode_kernel on a scaled-down
# config-3 case; traffic grows in proportion to the live tokens).
NCU_TRAFFIC_RATIO = {"cfg3": 1.026}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS,
            "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def time_steps(fn, steps: int, warmup: int, world: int, sampler=None):
    """W untimed steps, then exactly K steps between a barrier+synchronize on both sides, timed
    with CUDA events on the launching (current) stream.  Returns this rank's elapsed ms.

    With a clock sampler the untimed part is stretched to about 1.5 s of the same step, the
    sampler running from its start to the end of the timed region: the timed region itself
    lasts only milliseconds, far less than one nvidia-smi sampling period, so the samples
    describe the clocks the GPU holds under this load when the timed steps run."""
    import torch.distributed as dist
    if sampler:
        sampler.start()
        t_end = time.perf_counter() + 1.5
        while time.perf_counter() < t_end:
            for _ in range(20):
                fn()
            torch.cuda.synchronize()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def max_over_ranks(ms: float, world: int, device) -> float:
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sum_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


# ------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------

def build_paged(cfg: int, rank: int, device):
    from tileops_b200 import workloads as W
    from tileops_b200.ops import (GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp,
                                  GroupedQueryAttentionDecodePagedWithKVCacheFwdOp)
    # every rank has its own batch (own data and block table from its own seed stream) with the SAME
    # context lengths, so that the work per GPU is identical at every N (weak scaling)
    if cfg == 3:
        inp = W.make_paged_decode(3 + 10 * rank, 64, 32, 8, 128, 64, lens=W.draw_lengths(3, 64, (512, 8192)),
                                  device=device)
    elif cfg == 4:
        inp = W.make_paged_decode(4 + 10 * rank, 128, 64, 8, 128, 64, lens=[4096] * 128, fp8_cache=True,
                                  device=device)
    else:
        raise ValueError(cfg)
    B, H, D = inp.q.shape
    cls = GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp if cfg == 4 else GroupedQueryAttentionDecodePagedWithKVCacheFwdOp
    op = cls(B, H, inp.k.shape[1], inp.k.shape[0], D, inp.page_size)
    if cfg == 4:
        args = (inp.q, inp.k, inp.v, inp.k_scale, inp.v_scale, inp.real_seqlen_kv, inp.block_table)
    else:
        args = (inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    return inp, op, args


def run_paged_device(cfg, rank, world, device, steps, warmup, sampler=None):
    inp, op, args = build_paged(cfg, rank, device)
    ms = time_steps(lambda: op(*args), steps, warmup, world, sampler)
    return inp, op, args, ms


def run_e2e_paged(op, args, steps, warmup, world, device):
    """Same op, inputs in pinned HOST memory: every step copies them to the device, runs the op
    and reads the result back."""
    host = [a.cpu().pin_memory() for a in args]
    dev = [torch.empty_like(a) for a in args]
    out_host = torch.empty(args[0].shape, dtype=args[0].dtype).pin_memory()
    h2d = sum(a.numel() * a.element_size() for a in host)
    d2h = out_host.numel() * out_host.element_size()

    def step():
        for h, d in zip(host, dev):
            d.copy_(h, non_blocking=True)
        out_host.copy_(op(*dev), non_blocking=True)

    ms = time_steps(step, steps, warmup, world)
    return ms, h2d, d2h


def cpu_baseline_paged(cfg: int, budget_s: float = 15.0):
    """Reference CPU path (oracle port of the reference's torch ref_program) on a bounded sample
    of the workload: whole sequences of the config, as many as fit the time budget."""
    from oracle import gqa_oracle as O
    from tileops_b200 import workloads as W
    n_seq = 4
    if cfg == 3:
        inp = W.make_paged_decode(3, n_seq, 32, 8, 128, 64, len_range=(512, 8192), device="cpu")
    else:
        inp = W.make_paged_decode(4, n_seq, 64, 8, 128, 64, lens=[4096] * n_seq, fp8_cache=True, device="cpu")

    def run():
        if cfg == 4:
            return O.paged_decode_fp8_ref(inp.q, inp.k, inp.v, inp.k_scale, inp.v_scale, inp.real_seqlen_kv,
                                          inp.block_table, inp.page_size)
        return O.paged_decode_ref(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table, inp.page_size)

    run()
    t0 = time.perf_counter()
    reps = 0
    while True:
        run()
        reps += 1
        if time.perf_counter() - t0 > budget_s or reps >= 50:
            break
    sec = (time.perf_counter() - t0) / reps
    by = inp.algorithmic_bytes()
    return {"value": by / sec / 1e9, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{n_seq} sequences of the config-{cfg} workload (sum of lengths {sum(inp.lens)} tokens), "
                      f"{reps} repetitions, {sec * 1e3:.1f} ms each",
            "ms_per_step_sample": sec * 1e3}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-others", action="store_true", help="time only the headline workload")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--case", default=None,
                    choices=["decode_small", "decode_fp8_small", "prefill_small", "prefill_paged"],
                    help="run only a reduced case of one kernel (a few hundred MB on the device: the "
                         "size an ncu capture of all sections can handle) and print its timing")
    a = ap.parse_args()
    if a.case:
        return run_small_case(a.case, a.steps, max(a.warmup, 1))
    rank, world, local = dist_env()
    warmup = max(a.warmup, 3)
    workload = ("BASELINE config 3: GQA paged decode bf16, batch 64, 32 q heads / 8 KV heads, head_dim 128, "
                "context ~U[512,8192], page 64, random-permutation block table")
    config = {"workload": workload, "per_gpu_batch": 64, "l2_policy": "inputs (1.3 GB per step) exceed the 126 MB L2",
              "partition": "by sequence, one batch per GPU" if a.gpus > 1 else "single GPU"}

    if a.impl == "reference":
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)
        base = cpu_baseline_paged(3, budget_s=max(5.0, min(60.0, 2.0 * a.steps)))
        line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": a.gpus,
                "steps": a.steps, "warmup": warmup, "ms_per_step": base["ms_per_step_sample"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    peaks = measured_peaks()

    sampler = ClockSampler(local) if rank == 0 else None
    inp, op, args, ms_local = run_paged_device(3, rank, world, device, a.steps, warmup, sampler)
    clocks = sampler.stop() if sampler else None
    ms = max_over_ranks(ms_local, world, device)
    bytes_all = sum_over_ranks(float(inp.algorithmic_bytes()), world, device)
    tokens_all = sum_over_ranks(float(inp.q.shape[0]), world, device)
    ms_step = ms / a.steps
    value = bytes_all / (ms_step * 1e-3) / 1e9
    # roofline of the dominant kernel on this rank (one launch per step)
    achieved = inp.algorithmic_bytes() / (ms_local / a.steps * 1e-3) / 1e9
    ratio = NCU_TRAFFIC_RATIO.get("cfg3")
    roofline = {"bound": "hbm", "kernel": "gqa_decode_kernel<128,bf16>", "achieved": achieved,
                "peak": peaks["hbm_gbs"], "unit": UNIT, "frac": achieved / peaks["hbm_gbs"],
                "peak_source": f"of {peaks['source']}", "frac_of_nominal_8000": achieved / 8000.0,
                "algorithmic_bytes_per_launch": inp.algorithmic_bytes(),
                "traffic": None if ratio is None else ratio * inp.algorithmic_bytes()}

    e2e_ms, h2d, d2h = run_e2e_paged(op, args, max(3, min(a.steps, 10)), 3, world, device)
    e2e_ms = max_over_ranks(e2e_ms, world, device) / max(3, min(a.steps, 10))
    e2e = {"value": bytes_all / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms}

    others = {}
    del inp, op, args
    torch.cuda.empty_cache()
    if not a.no_others:
        others = run_others(rank, world, device, max(5, a.steps // 2), warmup, peaks)

    cpu_base = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        cpu_base = cpu_baseline_paged(3)

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps,
                "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "tokens_per_s": tokens_all / (ms_step * 1e-3), "roofline": roofline, "e2e": e2e,
                "gpu_launches": a.steps, "clocks": clocks, "others": others}
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_small_case(case: str, steps: int, warmup: int):
    """Reduced single-kernel cases for profiler captures: same kernels and code path as the
    BASELINE configurations, a quarter of the batch (inputs still exceed the L2)."""
    from tileops_b200 import workloads as W
    from tileops_b200.ops import (GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp,
                                  GroupedQueryAttentionDecodePagedWithKVCacheFwdOp,
                                  GroupedQueryAttentionFwdOp)
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if case == "decode_small":
        inp = W.make_paged_decode(3, 16, 32, 8, 128, 64, len_range=(512, 8192), device=device)
        op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(16, 32, 8, inp.k.shape[0], 128, 64)
        fn = lambda: op(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)  # noqa: E731
        work, unit = inp.algorithmic_bytes(), "GB/s"
    elif case == "decode_fp8_small":
        inp = W.make_paged_decode(4, 32, 64, 8, 128, 64, lens=[4096] * 32, fp8_cache=True, device=device)
        op = GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp(32, 64, 8, inp.k.shape[0], 128, 64)
        fn = lambda: op(inp.q, inp.k, inp.v, inp.k_scale, inp.v_scale, inp.real_seqlen_kv, inp.block_table)  # noqa: E731
        work, unit = inp.algorithmic_bytes(), "GB/s"
    elif case == "prefill_paged":
        fn, work = paged_prefill_step(device, 0)
        unit = "TFLOP/s"
    else:
        q, k, v = W.make_prefill(2, 1, 4096, 4096, 32, 8, 128, torch.bfloat16, device)
        op = GroupedQueryAttentionFwdOp(1, 32, 8, 4096, 128, is_causal=True)
        fn = lambda: op(q, k, v)  # noqa: E731
        fn()
        work, unit = op.eval_roofline()[0], "TFLOP/s"
    ms = time_steps(fn, steps, warmup, 1) / steps
    rate = work / (ms * 1e-3) / (1e9 if unit == "GB/s" else 1e12)
    print(json.dumps({"case": case, "ms_per_step": ms, "work_per_step": work, "rate": rate, "unit": unit,
                      "steps": steps, "warmup": warmup}))


def run_others(rank, world, device, steps, warmup, peaks):
    """The remaining BASELINE configurations, each timed with the same protocol."""
    out = {}
    # config 4: FP8-e4m3 KV cache, batch 128 per GPU
    try:
        inp, op, args, ms = run_paged_device(4, rank, world, device, steps, warmup)
        ms = max_over_ranks(ms, world, device) / steps
        by = sum_over_ranks(float(inp.algorithmic_bytes()), world, device)
        out["cfg4_paged_decode_fp8kv"] = {
            "gbs": by / (ms * 1e-3) / 1e9, "frac_of_peak": by / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "ms_per_step": ms, "tokens_per_s": 128 * world / (ms * 1e-3), "gpu_launches": steps}
        del inp, op, args
        torch.cuda.empty_cache()
    except Exception as exc:  # noqa: BLE001 - report, never hide
        out["cfg4_paged_decode_fp8kv"] = {"error": repr(exc)}
    # config 5: long context, KV-sequence sharded over the ranks, NCCL (O, LSE) exchange
    try:
        out["cfg5_long_context_sharded"] = run_cfg5(rank, world, device, steps, warmup, peaks)
        torch.cuda.empty_cache()
    except Exception as exc:  # noqa: BLE001
        out["cfg5_long_context_sharded"] = {"error": repr(exc)}
    # config 2: causal prefill
    try:
        out["cfg2_causal_prefill"] = run_cfg2(rank, world, device, steps, warmup, peaks)
    except Exception as exc:  # noqa: BLE001
        out["cfg2_causal_prefill"] = {"error": repr(exc)}
    # the step that fills the pages decode reads: one 512-token chunk per request over a 4k prefix
    try:
        fn, flops = paged_prefill_step(device, rank)
        ms = max_over_ranks(time_steps(fn, steps, warmup, world), world, device) / steps
        tf = flops * world / (ms * 1e-3) / 1e12
        out["paged_prefill_llama8b_chunk512"] = {
            "tflops": tf, "frac_of_peak_burst": tf / world / peaks["bf16_tflops"], "ms_per_step": ms,
            "tokens_per_s": 8 * 512 * world / (ms * 1e-3), "gpu_launches": steps}
    except Exception as exc:  # noqa: BLE001
        out["paged_prefill_llama8b_chunk512"] = {"error": repr(exc)}
    return out


def paged_prefill_step(device, rank):
    """Manifest workload "llama-8b-prefill-paged-b8-prefix4k-chunk512-p64" (fp16, no fused RoPE): the
    kernel class is called directly, because the operator's own argument checks read the length
    tensors on the host (as the reference's do) and would put a sync into every timed step."""
    from tileops_b200 import workloads as W
    from tileops_b200.kernels import GQAPrefillPagedSm100Kernel
    from tileops_b200.perf.formulas import gqa_prefill_paged_with_kv_cache_fwd_roofline
    B, H, Hkv, D, page, W_pages, old, n = 8, 32, 8, 128, 64, 72, 4096, 512
    args = W.make_paged_prefill(6 + 10 * rank, [n] * B, [old] * B, H, Hkv, D, page, W_pages, torch.float16, device)
    kern = GQAPrefillPagedSm100Kernel(B, H, Hkv, W_pages, page, D, True, torch.float16)
    flops, _ = gqa_prefill_paged_with_kv_cache_fwd_roofline(
        total_q=B * n, batch=B, q_lens=[n] * B, cache_lens=[old] * B, heads=H, heads_kv=Hkv, dim=D,
        page_size=page, max_pages_per_req=W_pages, max_seqlen_q=n, is_causal=True, dtype=torch.float16)
    return (lambda: kern(*args)), flops


def run_cfg5(rank, world, device, steps, warmup, peaks):
    from tileops_b200 import workloads as W
    from tileops_b200.sharded import KVSequenceShardedPagedDecode, shard_page_range
    B, H, Hkv, D, page, ctx = 8, 32, 8, 128, 128, 131072
    p0, p1 = shard_page_range(ctx // page, rank, world)
    inp = W.make_paged_decode(5, B, H, Hkv, D, page, lens=[ctx] * B, device=device, page_begin=p0, page_end=p1)
    op = KVSequenceShardedPagedDecode(B, H, Hkv, D, page)
    fn = lambda: op(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)  # noqa: E731
    # one CUDA graph per step (decode launch + NCCL all-gather + merge launch): at 4+ GPUs the GPU work of a
    # step is shorter than the time Python needs to issue the three calls.  Every rank takes the same branch.
    graphed = os.environ.get("TB200_BENCH_GRAPH", "1") != "0"
    # exchange: stores over NVLink from the decode kernel into every rank's symmetric buffer (fused compute +
    # exchange); falls back to the NCCL all-gather if symmetric memory cannot be set up.  All ranks agree.
    exchange = "nccl_all_gather"
    if world > 1 and os.environ.get("TB200_BENCH_PEER", "1") != "0":
        import torch.distributed as dist
        ok = torch.ones(1, device=device)
        try:
            op.enable_peer_exchange(device)
        except Exception as exc:  # noqa: BLE001 - reported below, never hidden
            ok.zero_()
            print(f"[bench] rank {rank}: peer exchange unavailable ({exc!r}); using the NCCL all-gather", file=sys.stderr)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() > 0:
            exchange = "peer_stores"
        else:
            op._peer = None
    if graphed:
        fn = op.graphed(inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    ms = max_over_ranks(time_steps(fn, steps, warmup, world), world, device) / steps
    peer_status = op.peer_status()
    # drop the graph and the symmetric buffer before the process group is torn down
    del fn
    op._peer = None
    torch.cuda.synchronize(device)
    total = 2 * B * ctx * Hkv * D * 2 + 2 * B * H * D * 2 + 4 * B * (ctx // page) + 4 * B
    return {"gbs": total / (ms * 1e-3) / 1e9, "frac_of_peak": total / world / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3), "scaling": "strong",
            "exchange_bytes_per_rank": B * H * (D + 1) * 4 * world, "cuda_graph": graphed, "exchange": exchange,
            "peer_wait_status": peer_status,
            "gpu_launches": steps * (2 if world > 1 else 2)}


def run_cfg2(rank, world, device, steps, warmup, peaks):
    from tileops_b200 import workloads as W
    from tileops_b200.ops import GroupedQueryAttentionFwdOp
    B, S, H, Hkv, D = 4, 4096, 32, 8, 128
    q, k, v = W.make_prefill(2 + 10 * rank, B, S, S, H, Hkv, D, torch.bfloat16, device)
    op = GroupedQueryAttentionFwdOp(B, H, Hkv, S, D, is_causal=True)
    ms = max_over_ranks(time_steps(lambda: op(q, k, v), steps, warmup, world), world, device) / steps
    flops, _ = op.eval_roofline()
    tf = flops * world / (ms * 1e-3) / 1e12
    return {"tflops": tf, "frac_of_peak_burst": tf / world / peaks["bf16_tflops"],
            "frac_of_peak_sustained": tf / world / peaks["bf16_tflops_sustained"],
            "frac_of_nominal_2250": tf / world / 2250.0, "ms_per_step": ms,
            "tokens_per_s": B * S * world / (ms * 1e-3), "gpu_launches": steps}


if __name__ == "__main__":
    main()
