#!/usr/bin/env python
"""Benchmark of the GQA attention-forward hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-others] [--no-manifest]

One "step" is one pass of the hot path over one batch of seeded synthetic input.  The headline
workload is the paged bf16 decode of a Llama-3-8B attention layer (batch 64, 32 q heads / 8 KV heads,
head dim 128, context uniform in [512, 8192], 64-token pages, random-permutation block table); the
metric is achieved HBM GB/s over the algorithmic bytes (live K/V + q + o + block-table entries +
lengths, each once).  The FP8-cache decode, the long-context KV-sharded decode, the causal prefill and
a paged-prefill chunk are timed with the same protocol and reported under ``"others"``, each with its
own clock record, per-launch medians, roofline block and a one-shot comparison with the CPU oracle.

For N > 1 (launched by ``python -m torch.distributed.run``, one rank per GPU) every rank decodes
its own batch of the same shape (weak scaling; the path partitions by sequence with no data-path
collective); ``value`` is all ranks' bytes over the slowest rank's time.  The KV-sequence-sharded
long-context decode, which does have one exchange step, is reported under ``"others"`` together with a
bit-identity check of its fused exchange against the NCCL all-gather path.

``--impl reference`` times the reference's CPU implementation of the same workload (its torch
reference program, restated in ``oracle/`` because the reference tree does not travel with this
repository) on the host cores, on a bounded sample.
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
PER_LAUNCH_SAMPLES = 100

# DRAM traffic per launch relative to the algorithmic bytes (dram__bytes.sum of one ncu capture of
# gqa_decode_tma_kernel on the quarter-batch case ``--case decode_small``: 374.8 MB against 368.07 MB; traffic
# grows in proportion to the live tokens, so the ratio carries over to the full launch).
NCU_TRAFFIC_RATIO = {"paged_decode_bf16": 1.018}


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


def time_steps(fn, steps: int, warmup: int, world: int, sampler=None, soak_s: float = 0.0):
    """W untimed steps, then exactly K steps between a barrier+synchronize on both sides, timed
    with CUDA events on the launching (current) stream.  Returns this rank's elapsed ms.

    With a clock sampler the untimed part is stretched to ``soak_s`` seconds of the same step, the
    sampler running from its start to the end of the timed region: the timed region itself
    lasts only milliseconds, far less than one nvidia-smi sampling period, so the samples
    describe the clocks the GPU holds under this load when the timed steps run."""
    import torch.distributed as dist
    if sampler:
        sampler.start()
    if soak_s > 0:
        # the same number of soak steps on every rank (a step may hold an exchange that all ranks must run in
        # lockstep): the slowest rank's time for 10 steps sizes the soak
        for _ in range(5):                   # first calls pay one-time costs (maps, attributes, workspaces)
            fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(10):
            fn()
        torch.cuda.synchronize()
        per_step = max((time.perf_counter() - t0) / 10, 1e-6)
        if world > 1:
            t = torch.tensor([per_step], device="cuda", dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            per_step = float(t.item())
        for _ in range(min(int(soak_s / per_step), 100000) // 20):
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
    torch.cuda.profiler.start()          # a profiler started with --profile-from-start off lists the timed launches only
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def per_launch_us(fn, samples: int = PER_LAUNCH_SAMPLES):
    """``samples`` steps, each between its own pair of CUDA events on the launching stream (all queued,
    one synchronize at the end): (median, min) microseconds of one step."""
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(samples)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    us = [a.elapsed_time(b) * 1e3 for a, b in evs]
    return statistics.median(us), min(us)


def measure(fn, steps, warmup, world, device, local_index, sample_clocks=True):
    """The timing protocol of every entry: clock sampler over a soak and the timed region, K steps timed as
    one region (max over ranks), then per-launch medians over 100 more steps."""
    sampler = ClockSampler(local_index) if sample_clocks else None
    ms_local = time_steps(fn, steps, warmup, world, sampler, soak_s=1.5 if sample_clocks else 0.0)
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    med, mn = per_launch_us(fn)
    clocks = sampler.stop() if sampler else None
    ms = max_over_ranks(ms_local, world, device) / steps
    out = {"ms_per_step": ms, "ms_per_step_local": ms_local / steps, "per_launch_us_median": med,
           "per_launch_us_min": mn, "per_launch_samples": PER_LAUNCH_SAMPLES, "clocks": clocks}
    if clocks and clocks.get("sm_mhz"):
        # time x clock: comparable between boxes that settle at different SM clocks under the power cap
        out["us_x_sm_mhz"] = med * clocks["sm_mhz"]
    return out


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


def hbm_roofline(kernel, bytes_per_launch, us_per_launch, peaks, traffic_ratio=None):
    achieved = bytes_per_launch / (us_per_launch * 1e-6) / 1e9
    return {"bound": "hbm", "kernel": kernel, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": achieved / peaks["hbm_gbs"], "peak_source": f"of {peaks['source']}",
            "frac_of_nominal_8000": achieved / 8000.0, "algorithmic_bytes_per_launch": bytes_per_launch,
            "traffic": None if traffic_ratio is None else traffic_ratio * bytes_per_launch}


def tensor_roofline(kernel, flops_per_launch, us_per_launch, peaks):
    achieved = flops_per_launch / (us_per_launch * 1e-6) / 1e12
    return {"bound": "tensor", "kernel": kernel, "achieved": achieved, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
            "frac": achieved / peaks["bf16_tflops"], "peak_source": f"of {peaks['source']} (cuBLAS bf16 burst)",
            "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"], "frac_of_nominal_2250": achieved / 2250.0,
            "algorithmic_flops_per_launch": flops_per_launch, "traffic": None}


# ------------------------------------------------------------------------------------------
# workloads
# ------------------------------------------------------------------------------------------

def build_paged(kind: str, rank: int, device):
    from tileops_b200 import workloads as W
    from tileops_b200.ops import (GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp,
                                  GroupedQueryAttentionDecodePagedWithKVCacheFwdOp)
    # every rank has its own batch (own data and block table from its own seed stream) with the SAME
    # context lengths, so that the work per GPU is identical at every N (weak scaling)
    if kind == "bf16":
        inp = W.make_paged_decode(3 + 10 * rank, 64, 32, 8, 128, 64, lens=W.draw_lengths(3, 64, (512, 8192)),
                                  device=device)
    elif kind == "fp8":
        inp = W.make_paged_decode(4 + 10 * rank, 128, 64, 8, 128, 64, lens=[4096] * 128, fp8_cache=True,
                                  device=device)
    else:
        raise ValueError(kind)
    B, H, D = inp.q.shape
    cls = GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp if kind == "fp8" else GroupedQueryAttentionDecodePagedWithKVCacheFwdOp
    op = cls(B, H, inp.k.shape[1], inp.k.shape[0], D, inp.page_size)
    if kind == "fp8":
        args = (inp.q, inp.k, inp.v, inp.k_scale, inp.v_scale, inp.real_seqlen_kv, inp.block_table)
    else:
        args = (inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    return inp, op, args


def paged_parity_spot(inp, out, b: int = 0) -> float:
    """Max abs error of sequence ``b`` of a paged decode result against the CPU oracle."""
    from oracle import gqa_oracle as O
    sl = slice(b, b + 1)
    if inp.k_scale is not None:
        ref = O.paged_decode_fp8_ref(inp.q[sl].cpu(), inp.k.cpu(), inp.v.cpu(), inp.k_scale.cpu(), inp.v_scale.cpu(),
                                     inp.real_seqlen_kv[sl].cpu(), inp.block_table[sl].cpu(), inp.page_size)
    else:
        ref = O.paged_decode_ref(inp.q[sl].cpu(), inp.k.cpu(), inp.v.cpu(), inp.real_seqlen_kv[sl].cpu(),
                                 inp.block_table[sl].cpu(), inp.page_size)
    return float((out[sl].float().cpu() - ref.float()).abs().max())


def run_e2e_paged(op, args, steps, warmup, world, device, resident: bool):
    """Same op through the operator call with HOST buffers: every step copies its inputs from pinned host
    memory to the device, runs the op and reads the result back.  ``resident=False`` copies everything
    (the KV pool included: what a caller holding its cache in host memory pays); ``resident=True`` is the
    serving step, cache resident on the device, only q, lengths and block table copied in."""
    moved = [i for i, a in enumerate(args) if not resident or a.numel() * a.element_size() < (64 << 20)]
    host = {i: args[i].cpu().pin_memory() for i in moved}
    dev = list(args)
    for i in moved:
        dev[i] = torch.empty_like(args[i])
    out_host = torch.empty(args[0].shape, dtype=args[0].dtype).pin_memory()
    h2d = sum(h.numel() * h.element_size() for h in host.values())
    d2h = out_host.numel() * out_host.element_size()

    def step():
        for i in moved:
            dev[i].copy_(host[i], non_blocking=True)
        out_host.copy_(op(*dev), non_blocking=True)

    ms = time_steps(step, steps, warmup, world)
    return ms, h2d, d2h


def cpu_baseline_paged(kind: str, budget_s: float = 15.0):
    """Reference CPU path (oracle port of the reference's torch ref_program) on a bounded sample
    of the workload: whole sequences of the workload, as many repetitions as fit the time budget."""
    from oracle import gqa_oracle as O
    from tileops_b200 import workloads as W
    n_seq = 4
    if kind == "bf16":
        inp = W.make_paged_decode(3, n_seq, 32, 8, 128, 64, len_range=(512, 8192), device="cpu")
    else:
        inp = W.make_paged_decode(4, n_seq, 64, 8, 128, 64, lens=[4096] * n_seq, fp8_cache=True, device="cpu")

    def run():
        if kind == "fp8":
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
            "sample": f"{n_seq} sequences of the paged {kind} decode workload (sum of lengths {sum(inp.lens)} tokens), "
                      f"{reps} repetitions, {sec * 1e3:.1f} ms each",
            "ms_per_step_sample": sec * 1e3}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-others", action="store_true", help="time only the headline workload")
    ap.add_argument("--no-manifest", action="store_true", help="skip the decode workloads of the operator manifest")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="long-context sharded step: eager launches instead of a CUDA graph")
    ap.add_argument("--nccl-exchange", action="store_true", help="long-context sharded step: NCCL all-gather instead of the fused exchange")
    ap.add_argument("--case", default=None,
                    choices=["decode_small", "decode_fp8_small", "prefill_small", "prefill_two_tile_small", "prefill_paged",
                             "rope_small", "fp8_cache_small", "fp8_cache_fused", "merge_small", "mma_issue"],
                    help="run only a reduced case of one kernel (a few hundred MB on the device: the "
                         "size an ncu capture of all sections can handle) and print its timing")
    a = ap.parse_args()
    if a.case:
        return run_small_case(a.case, a.steps, max(a.warmup, 1))
    rank, world, local = dist_env()
    warmup = max(a.warmup, 3)
    workload = ("GQA paged decode bf16 (Llama-3-8B attention): batch 64, 32 q heads / 8 KV heads, head_dim 128, "
                "context ~U[512,8192], page 64, random-permutation block table")
    config = {"workload": workload, "per_gpu_batch": 64, "l2_policy": "inputs (1.3 GB per step) exceed the 126 MB L2",
              "partition": "by sequence, one batch per GPU" if a.gpus > 1 else "single GPU"}

    if a.impl == "reference":
        if rank != 0:
            return
        torch.set_num_threads(os.cpu_count() or 1)
        base = cpu_baseline_paged("bf16", budget_s=max(5.0, min(60.0, 2.0 * a.steps)))
        line = {"impl": "reference", "metric": METRIC, "value": base["value"], "unit": UNIT, "n_gpus": a.gpus,
                "steps": a.steps, "warmup": warmup, "ms_per_step": base["ms_per_step_sample"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": config, "cpu_baseline": base,
                "e2e": {"value": base["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback for the product path)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    peaks = measured_peaks()

    inp, op, args = build_paged("bf16", rank, device)
    m = measure(lambda: op(*args), a.steps, warmup, world, device, local, sample_clocks=True)
    bytes_all = sum_over_ranks(float(inp.algorithmic_bytes()), world, device)
    tokens_all = sum_over_ranks(float(inp.q.shape[0]), world, device)
    ms_step = m["ms_per_step"]
    value = bytes_all / (ms_step * 1e-3) / 1e9
    # roofline of the dominant kernel on this rank (one launch per step), from the timed region
    roofline = hbm_roofline("gqa_decode_tma_kernel<128, bf16>", inp.algorithmic_bytes(), m["ms_per_step_local"] * 1e3,
                            peaks, NCU_TRAFFIC_RATIO.get("paged_decode_bf16"))
    roofline["achieved_per_launch_median"] = inp.algorithmic_bytes() / (m["per_launch_us_median"] * 1e-6) / 1e9
    parity_spot = paged_parity_spot(inp, op(*args)) if rank == 0 else None

    n_e2e = max(3, min(a.steps, 10))
    e2e_ms, h2d, d2h = run_e2e_paged(op, args, n_e2e, 3, world, device, resident=False)
    e2e_ms = max_over_ranks(e2e_ms, world, device) / n_e2e
    e2e = {"value": bytes_all / (e2e_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms}
    n_res = max(10, min(a.steps, 50))
    res_ms, h2d_r, d2h_r = run_e2e_paged(op, args, n_res, 3, world, device, resident=True)
    res_ms = max_over_ranks(res_ms, world, device) / n_res
    e2e_resident = {"value": bytes_all / (res_ms * 1e-3) / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d_r,
                    "d2h_bytes_per_step": d2h_r, "ms_per_step": res_ms,
                    "what": "KV pool resident on the device; q, lengths and block table copied in, o copied out"}

    others = {}
    del inp, op, args
    torch.cuda.empty_cache()
    if not a.no_others:
        others = run_others(rank, world, local, device, max(5, a.steps // 2), warmup, peaks, a)
    if not a.no_manifest and world == 1:
        try:
            others["manifest_decode_workloads"] = run_manifest_decode(device, peaks)
        except Exception as exc:  # noqa: BLE001 - report, never hide
            others["manifest_decode_workloads"] = {"error": repr(exc)}

    cpu_base = None
    if rank == 0 and world == 1 and not a.no_cpu_baseline:
        cpu_base = cpu_baseline_paged("bf16")

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps,
                "warmup": warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
                "tokens_per_s": tokens_all / (ms_step * 1e-3), "roofline": roofline, "e2e": e2e,
                "e2e_resident": e2e_resident, "gpu_launches": a.steps, "clocks": m["clocks"],
                "per_launch_us_median": m["per_launch_us_median"], "per_launch_us_min": m["per_launch_us_min"],
                "us_x_sm_mhz": m.get("us_x_sm_mhz"), "parity_spot": parity_spot, "others": others}
        if cpu_base is not None:
            line["cpu_baseline"] = cpu_base
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def run_small_case(case: str, steps: int, warmup: int):
    """Reduced single-kernel cases for profiler captures: same kernels and code path as the
    benchmarked workloads, a fraction of the batch (inputs still exceed the L2)."""
    from tileops_b200 import functional as F
    from tileops_b200 import workloads as W
    from tileops_b200.ops import (GroupedQueryAttentionDecodePagedFp8KVCacheFwdOp,
                                  GroupedQueryAttentionDecodePagedWithKVCacheFwdOp,
                                  GroupedQueryAttentionFwdOp)
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    if case == "mma_issue":
        # what one tcgen05.mma instruction costs on the tensor pipe, by N and by the place of the A operand
        rows = {}
        for n in (64, 128, 256):
            for tmem_a in (False, True):
                issued, done = F.mma_issue_probe(n, tmem_a, 200, device)
                rows[f"N={n},A={'tmem' if tmem_a else 'smem'}"] = {"clocks_per_mma": round(done, 1),
                                                                    "arithmetic_clocks": n // 2}
        print(json.dumps({"case": case, "M": 128, "K": 16, "kind": "f16", "rows": rows}))
        return
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
    elif case == "rope_small":
        # the rotation pass of the fused-RoPE paged prefill: 64k tokens x 32 heads x 128 dims, bf16 (read + write 1 GB)
        T, H, D = 65536, 32, 128
        x = torch.randn(T, H, D, device=device, dtype=torch.bfloat16)
        pos = torch.arange(8192, device=device, dtype=torch.float32)[:, None]
        inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=device, dtype=torch.float32) / D))
        cos, sin = torch.cos(pos * inv).to(x.dtype), torch.sin(pos * inv).to(x.dtype)
        cu = torch.arange(0, T + 1, 8192, device=device, dtype=torch.int32)
        cache = torch.zeros(cu.numel() - 1, device=device, dtype=torch.int32)
        fn = lambda: F.rope_neox_packed(x, cos, sin, cu, cache)  # noqa: E731
        work, unit = 2 * x.numel() * 2, "GB/s"
    elif case == "fp8_cache_small":
        # gather + packed prefill + append of the paged prefill over an FP8 cache (8 x 512 new over 8 x 4096 cached)
        B, H, Hkv, D, page, Wp, old, n = 8, 32, 8, 128, 64, 72, 4096, 512
        args = list(W.make_paged_prefill(6, [n] * B, [old] * B, H, Hkv, D, page, Wp, torch.float16, device))
        f8 = torch.float8_e4m3fn
        args[3], args[4] = args[3].to(f8), args[4].to(f8)
        fn = lambda: F.gqa_prefill_paged_fp8_cache(*args[:10], args[10], page_size=page)  # noqa: E731
        work, unit = 2 * B * old * Hkv * D + 2 * B * n * Hkv * D * 3, "GB/s"
    elif case == "fp8_cache_fused":
        # the same workload through the one-launch variant (e4m3 pages expanded inside the prefill kernel)
        B, H, Hkv, D, page, Wp, old, n = 8, 32, 8, 128, 64, 72, 4096, 512
        args = list(W.make_paged_prefill(6, [n] * B, [old] * B, H, Hkv, D, page, Wp, torch.float16, device))
        f8 = torch.float8_e4m3fn
        args[3], args[4] = args[3].to(f8), args[4].to(f8)
        fn = lambda: F.gqa_prefill_paged_fp8_cache(*args[:10], args[10], page_size=page, fused=True)  # noqa: E731
        work, unit = 4 * B * H * D * (n * old + n * (n + 1) // 2), "TFLOP/s"
    elif case == "merge_small":
        # the cross-rank merge: 8 parts of 256 rows x 128 dims
        parts, rows, D = 8, 256, 128
        o_parts = torch.randn(parts, rows, D, device=device)
        lse_parts = torch.randn(parts, rows, device=device)
        fn = lambda: F.gqa_lse_merge(o_parts, lse_parts, torch.bfloat16)  # noqa: E731
        work, unit = parts * rows * (D + 1) * 4 + rows * D * 2, "GB/s"
    elif case == "prefill_two_tile_small":
        # the opt-in prefill kernel with two Q tiles per CTA, same inputs as prefill_small
        q, k, v = W.make_prefill(2, 1, 4096, 4096, 32, 8, 128, torch.bfloat16, device)
        fn = lambda: F.gqa_prefill(q, k, v, is_causal=True, config={"tiles_per_cta": 2})  # noqa: E731
        work, unit = 4 * 32 * 4096 * 4096 * 128 // 2, "TFLOP/s"
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


def run_others(rank, world, local, device, steps, warmup, peaks, a):
    """The remaining workloads, each timed with the same protocol and its own clock record."""
    out = {}
    # FP8-e4m3 KV cache (Llama-3-70B attention), batch 128 per GPU
    try:
        inp, op, args = build_paged("fp8", rank, device)
        m = measure(lambda: op(*args), steps, warmup, world, device, local)
        by = sum_over_ranks(float(inp.algorithmic_bytes()), world, device)
        out["paged_decode_fp8kv"] = {
            "workload": "batch 128, 64 q heads / 8 KV heads, head_dim 128, context 4096, page 64, e4m3 cache with "
                        "fp32 scales per (page, KV head)",
            "gbs": by / (m["ms_per_step"] * 1e-3) / 1e9, "tokens_per_s": 128 * world / (m["ms_per_step"] * 1e-3),
            "gpu_launches": steps,
            "roofline": hbm_roofline("gqa_decode_tma_kernel<128, e4m3>", inp.algorithmic_bytes(),
                                     m["ms_per_step_local"] * 1e3, peaks),
            "parity_spot": paged_parity_spot(inp, op(*args)) if rank == 0 else None, **m}
        del inp, op, args
        torch.cuda.empty_cache()
    except Exception as exc:  # noqa: BLE001 - report, never hide
        out["paged_decode_fp8kv"] = {"error": repr(exc)}
    # long context, KV-sequence sharded over the ranks, (O, LSE) exchange
    try:
        out["long_context_sharded"] = run_long_context(rank, world, local, device, steps, warmup, peaks, a)
        torch.cuda.empty_cache()
    except Exception as exc:  # noqa: BLE001
        out["long_context_sharded"] = {"error": repr(exc)}
    # causal prefill
    try:
        out["causal_prefill"] = run_causal_prefill(rank, world, local, device, steps, warmup, peaks)
    except Exception as exc:  # noqa: BLE001
        out["causal_prefill"] = {"error": repr(exc)}
    # the step that fills the pages decode reads: one 512-token chunk per request over a 4k prefix
    try:
        fn, flops = paged_prefill_step(device, rank)
        m = measure(fn, steps, warmup, world, device, local)
        tf = flops * world / (m["ms_per_step"] * 1e-3) / 1e12
        out["paged_prefill_llama8b_chunk512"] = {
            "workload": "manifest llama-8b-prefill-paged-b8-prefix4k-chunk512-p64 (fp16)",
            "tflops": tf, "tokens_per_s": 8 * 512 * world / (m["ms_per_step"] * 1e-3), "gpu_launches": steps,
            "roofline": tensor_roofline("gqa_prefill_kernel<f16, 128, paged>", flops, m["ms_per_step_local"] * 1e3, peaks),
            **m}
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


def run_long_context(rank, world, local, device, steps, warmup, peaks, a):
    from oracle import gqa_oracle as O
    from tileops_b200 import workloads as W
    from tileops_b200.sharded import KVSequenceShardedPagedDecode, shard_page_range
    B, H, Hkv, D, page, ctx = 8, 32, 8, 128, 128, 131072
    p0, p1 = shard_page_range(ctx // page, rank, world)
    inp = W.make_paged_decode(5, B, H, Hkv, D, page, lens=[ctx] * B, device=device, page_begin=p0, page_end=p1)
    op = KVSequenceShardedPagedDecode(B, H, Hkv, D, page)
    call = (inp.q, inp.k, inp.v, inp.real_seqlen_kv, inp.block_table)
    reference_out = op(*call).clone()            # NCCL all-gather path (or the plain merge on one GPU)
    # one CUDA graph per step (decode launch [+ exchange] + merge launch): at 4+ GPUs the GPU work of a
    # step is shorter than the time Python needs to issue the calls.  Every rank takes the same branch.
    graphed = not a.no_graph
    # exchange: stores over NVLink from the decode kernel into every rank's symmetric buffer (fused compute +
    # exchange); falls back to the NCCL all-gather if symmetric memory cannot be set up.  All ranks agree.
    exchange, exchange_check = "nccl_all_gather", None
    if world > 1 and not a.nccl_exchange:
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
            # the fused exchange against the all-gather path on the same inputs, on every rank
            diff = (op(*call).float() - reference_out.float()).abs().max().reshape(1)
            dist.all_reduce(diff, op=dist.ReduceOp.MAX)
            exchange_check = "bit-identical" if float(diff.item()) == 0.0 else float(diff.item())
        else:
            op._peer = None
    # one sequence x one KV-head group of the merged result against the CPU oracle over the whole context
    parity_spot = None
    if rank == 0:
        full = W.make_paged_decode(5, 1, H, Hkv, D, page, lens=[ctx], device=device)   # sequence 0: same K/V stream
        g = H // Hkv
        ref = O.paged_decode_ref(inp.q[0:1, 0:g].cpu().float(), full.k[:, 0:1].cpu().float(), full.v[:, 0:1].cpu().float(),
                                 full.real_seqlen_kv.cpu(), full.block_table.cpu(), page)
        parity_spot = float((reference_out[0:1, 0:g].float().cpu() - ref).abs().max())
        del full
    fn = op.graphed(*call) if graphed else (lambda: op(*call))
    m = measure(fn, steps, warmup, world, device, local)
    peer_status = op.peer_status()
    # drop the graph and the symmetric buffer before the process group is torn down
    del fn
    op._peer = None
    torch.cuda.synchronize(device)
    total = 2 * B * ctx * Hkv * D * 2 + 2 * B * H * D * 2 + 4 * B * (ctx // page) + 4 * B
    ms = m["ms_per_step"]
    return {"workload": "batch 8, 32 q heads / 8 KV heads, head_dim 128, context 131072 per sequence, page 128, bf16; "
                        "KV positions sharded over the ranks",
            "gbs": total / (ms * 1e-3) / 1e9, "tokens_per_s": B / (ms * 1e-3), "scaling": "strong",
            "exchange_bytes_per_rank": B * H * (D + 1) * 4 * world, "cuda_graph": graphed, "exchange": exchange,
            "exchange_check": exchange_check, "parity_spot": parity_spot, "peer_wait_status": peer_status,
            "gpu_launches": steps * 2,
            "roofline": hbm_roofline("gqa_decode_kernel<128, bf16> + lse_merge_kernel", total // world,
                                     m["ms_per_step_local"] * 1e3, peaks), **m}


def run_causal_prefill(rank, world, local, device, steps, warmup, peaks):
    from oracle import gqa_oracle as O
    from tileops_b200 import workloads as W
    from tileops_b200.ops import GroupedQueryAttentionFwdOp
    B, S, H, Hkv, D = 4, 4096, 32, 8, 128
    q, k, v = W.make_prefill(2 + 10 * rank, B, S, S, H, Hkv, D, torch.bfloat16, device)
    op = GroupedQueryAttentionFwdOp(B, H, Hkv, S, D, is_causal=True)
    m = measure(lambda: op(q, k, v), steps, warmup, world, device, local)
    flops, _ = op.eval_roofline()
    tf = flops * world / (m["ms_per_step"] * 1e-3) / 1e12
    parity_spot = None
    if rank == 0:
        g = H // Hkv
        ref = O.prefill_ref(q[0:1, :, 0:g].cpu(), k[0:1, :, 0:1].cpu(), v[0:1, :, 0:1].cpu(), True)
        parity_spot = float((op(q, k, v)[0:1, :, 0:g].float().cpu() - ref.float()).abs().max())
    return {"workload": "batch 4, seqlen 4096, 32 q heads / 8 KV heads, head_dim 128, causal, bf16",
            "tflops": tf, "tokens_per_s": B * S * world / (m["ms_per_step"] * 1e-3), "gpu_launches": steps,
            "roofline": tensor_roofline("gqa_prefill_kernel<bf16, 128>", flops, m["ms_per_step_local"] * 1e3, peaks),
            "parity_spot": parity_spot, **m}


def run_manifest_decode(device, peaks):
    """The decode and paged-decode workloads of the operator manifest (the reference's benchmark shapes,
    ``src/tileops/manifest/attention.yaml`` of tile-ai/TileOPs, incl. the batch-1 1k..256k contexts), one
    launch each between its own events.  These inputs are small (most fit the L2), so two figures are given:
    launches back to back on resident data (graph replay), and launches after a write larger than the L2."""
    from tileops_b200 import workloads as W
    from tileops_b200.manifest import load_workloads
    from tileops_b200.ops import (GroupedQueryAttentionDecodePagedWithKVCacheFwdOp,
                                  GroupedQueryAttentionDecodeWithKVCacheFwdOp)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    rows = {}

    def timed(fn, cold: bool, n: int = 30):
        """cold: a write larger than the L2 before every launch, each launch between its own events.
        warm: ``n`` launches replayed from one CUDA graph (what a decode loop does; no host launch latency
        inside the events, which for the small shapes is several times the kernel); the average of the launches."""
        for _ in range(3):
            fn()
        if not cold:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream(device))
            with torch.cuda.stream(side):
                fn()                                 # workspaces of this stream exist before the capture
            torch.cuda.current_stream(device).wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(n):
                    fn()
            graph.replay()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) * 1e3 / n
        us = []
        for _ in range(n):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            us.append(e0.elapsed_time(e1) * 1e3)
        return statistics.median(us)

    for wl in load_workloads("GroupedQueryAttentionDecodeWithKVCacheFwdOp"):
        B, H, D = wl["q_shape"]
        _, S, Hkv, _ = wl["kv_shape"]
        dtype = getattr(torch, wl["dtypes"][0])
        q, k, v = W.make_contiguous_decode(20, B, H, Hkv, S, D, dtype, device)
        op = GroupedQueryAttentionDecodeWithKVCacheFwdOp(B, H, Hkv, S, D, softcap=wl.get("softcap"))
        fn = lambda: op(q, k, v)  # noqa: E731
        by = 2 * B * S * Hkv * D * 2 + 2 * B * H * D * 2
        warm, cold = timed(fn, False), timed(fn, True)
        rows["decode/" + wl["label"]] = {"us_warm": warm, "us_cold": cold, "gbs_cold": by / cold / 1e3,
                                         "frac_of_peak_cold": by / cold / 1e3 / peaks["hbm_gbs"], "bytes": by}
        del q, k, v, op
    for wl in load_workloads("GroupedQueryAttentionDecodePagedWithKVCacheFwdOp"):
        if wl.get("own_pages"):
            continue            # the headline and long-context workloads: timed above with their own protocol
        B, H, D = wl["q_shape"]
        pool, Hkv, _ = wl["kv_shape"]
        page = wl["page_size"]
        dtype = getattr(torch, wl["dtypes"][0])
        # the reference's paged workload: one pool of `pool` tokens, every sequence reads all of it through
        # the same identity block table (workloads/attention/gqa.py:204-218)
        q = torch.randn(B, H, D, device=device).to(dtype)
        k = torch.randn(pool, Hkv, D, device=device).to(dtype)
        v = torch.randn(pool, Hkv, D, device=device).to(dtype)
        lens = torch.full((B,), pool, dtype=torch.int32, device=device)
        bt = torch.arange(pool // page, dtype=torch.int32, device=device).repeat(B, 1).contiguous()
        op = GroupedQueryAttentionDecodePagedWithKVCacheFwdOp(B, H, Hkv, pool, D, page, softcap=wl.get("softcap"))
        fn = lambda: op(q, k, v, lens, bt)  # noqa: E731
        by = 2 * pool * Hkv * D * 2 + 2 * B * H * D * 2          # the pool is shared: each byte once from HBM
        warm, cold = timed(fn, False), timed(fn, True)
        rows["paged/" + wl["label"]] = {"us_warm": warm, "us_cold": cold, "bytes_from_hbm": by,
                                        "gbs_l2_warm": B * 2 * pool * Hkv * D * 2 / warm / 1e3}
        del q, k, v, op
    return rows


if __name__ == "__main__":
    main()
