#!/usr/bin/env python3
"""Benchmark of the fused Q/K RMSNorm + RoPE + causal GQA attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C4|C5|C2] [--impl reference]

A step is one pass of the operator (row-prepare of K + attention, two kernel
launches, output and prepared-K buffers preallocated) over the named
workload.  With N > 1 (launched by torch.distributed.run, one rank per GPU)
the workload is sharded by KV-head group: every rank owns Hkv/N whole GQA
groups, there is no collective on the data path, and the reported value is
the whole job's FLOPs over the slowest rank's device time.

Prints one JSON line (rank 0).  `--impl reference` times the CPU FP32 oracle
(the reference's own CPU path for this operator) on the host cores instead.
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
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

from kernelfuser_b200.inputs import WORKLOADS, make_workload_inputs  # noqa: E402
from kernelfuser_b200.roofline import attention_flops, load_peaks, prepare_bytes  # noqa: E402
from kernelfuser_b200.shard import head_shard, shard_inputs  # noqa: E402

METRIC = "Fused QKnorm+RoPE+attn prefill TFLOP/s"
UNIT = "TFLOP/s"
DTYPE_NAME = {torch.bfloat16: "bf16", torch.float16: "fp16", torch.float32: "fp32"}
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of ONE launch at the full single-GPU size of the
# workload, from a one-launch ncu capture of this program (three metrics, --clock-control none); keyed by
# (workload name, kernel).  None where no full-size capture has been taken.
NCU_DRAM_BYTES_FULL = {
    ("C4", "attention"): 808484864 + 505497088,    # read + write; algorithmic bytes 1 342 177 280
    ("C4", "prepare"): 136419840 + 76488960,       # algorithmic bytes 268 435 456 (part of the output is still in L2)
    ("C5", "attention"): 1102489344 + 509574400,   # algorithmic bytes 1 610 612 736
    ("C5", "prepare"): 283977472 + 210954240,      # algorithmic bytes 536 870 912
}


# ----------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clock, power and clock-event (throttle) reasons of one GPU through
    NVML from a background thread while the timed region runs.  Reading only:
    nothing on the GPU is changed."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
               0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, torch_device_index: int, period_s: float = 0.002):
        self.period = period_s
        self.samples = []  # (time, sm_mhz, power_w, reasons_bitmask)
        self.t0 = self.t1 = None
        self._stop = threading.Event()
        self.thread = None
        self.handle = None
        self.max_mhz = None
        try:
            import pynvml
            self.nvml = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode() if hasattr(uuid, "encode") else uuid)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # pragma: no cover - depends on the box
            self.err = f"nvml unavailable: {e}"
            self.handle = None

    def _loop(self):
        nv = self.nvml
        while not self._stop.is_set():
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    power = nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                except Exception:
                    power = float("nan")
                try:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    reasons = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((time.perf_counter(), mhz, power, reasons))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.handle is None:
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def mark_begin(self):
        self.t0 = time.perf_counter()

    def mark_end(self):
        self.t1 = time.perf_counter()

    def stop(self) -> dict:
        if self.handle is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [getattr(self, "err", "nvml unavailable")]}
        self._stop.set()
        self.thread.join(timeout=2)
        inside = [s for s in self.samples if self.t0 is not None and self.t0 <= s[0] <= (self.t1 or 1e30)]
        scope = "timed region"
        if len(inside) < 3:  # a very short timed region: fall back to every sample taken under load (warm-up too)
            inside = self.samples
            scope = "warm-up + timed region"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["no samples"]}
        mask = 0
        for s in inside:
            mask |= s[3]
        reasons = sorted(name for bit, name in self.REASONS.items() if mask & bit)
        powers = [s[2] for s in inside if s[2] == s[2]]
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": self.max_mhz, "reasons": reasons,
                "samples": len(inside), "scope": scope, "power_w_max": max(powers) if powers else None}


def physical_gpu_index(local: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        parts = [p for p in vis.split(",") if p.strip()]
        if local < len(parts) and parts[local].strip().isdigit():
            return int(parts[local])
    return local


# ----------------------------------------------------------------------------
def use_all_host_cores() -> int:
    """Give torch's CPU kernels every core this process may run on.  Launchers such as torch.distributed.run
    export OMP_NUM_THREADS=1 to their children, which would time the CPU arm on a single thread."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover - non-Linux
        n = os.cpu_count() or 1
    torch.set_num_threads(max(n, 1))
    return torch.get_num_threads()


def cpu_oracle_rate(w, seconds_budget: float = 15.0):
    """Times the CPU FP32 oracle on a bounded sample (batch 1 of the workload)
    and returns (TFLOP/s, threads, description)."""
    from oracle import oracle as orc
    nthreads = use_all_host_cores()
    xs = make_workload_inputs(w, seed=0, B=1, dtype=torch.float32)
    flops = attention_flops(1, w.Hq, w.S, w.D, w.causal)
    orc.oracle_fp32(*xs, w.causal)  # warm-up
    times = []
    t_end = time.perf_counter() + seconds_budget
    while len(times) < 3 or (time.perf_counter() < t_end and len(times) < 50):
        t0 = time.perf_counter()
        orc.oracle_fp32(*xs, w.causal)
        times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    desc = (f"{w.name} at B=1 (1/{w.B} of the batch), fp32 oracle, median of {len(times)} runs, "
            f"{t * 1e3:.0f} ms per run")
    return flops / t / 1e12, nthreads, desc


def run_reference(args, w, rank):
    """The reference arm: the CPU FP32 oracle on the host cores (rank 0 only)."""
    if rank != 0:
        return
    from oracle import oracle as orc
    nthreads = use_all_host_cores()
    xs = make_workload_inputs(w, seed=0, B=1, dtype=torch.float32)
    flops = attention_flops(1, w.Hq, w.S, w.D, w.causal)
    for _ in range(max(args.warmup, 1)):
        orc.oracle_fp32(*xs, w.causal)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        orc.oracle_fp32(*xs, w.causal)
    dt = (time.perf_counter() - t0) / args.steps
    val = flops / dt / 1e12
    sample = f"each step = {w.name} at B=1 (1/{w.B} of the batch) through the CPU FP32 oracle"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
        "config": workload_config(w, args.gpus),
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": nthreads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def workload_config(w, n):
    return {"workload": f"{w.name}: B={w.B} S={w.S} Hq={w.Hq} Hkv={w.Hkv} D={w.D} causal theta={w.theta:g}",
            "flops_convention": "2*B*Hq*S^2*D (causal)", "sharding": f"kv-head groups, {w.Hkv // n} per GPU",
            "l2": "flushed between steps (256 MiB write); inputs also exceed L2",
            "step": "row-prepare(K) + attention, buffers preallocated"}


# ----------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="C4", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=3)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--variant", type=int, default=0)
    ap.add_argument("--batch", type=int, default=0, help="override the workload batch (profiling on a smaller case)")
    ap.add_argument("--seq", type=int, default=0, help="override the workload sequence length (profiling only)")
    ap.add_argument("--no-graph", action="store_true", help="skip the graph-replay protocol")
    ap.add_argument("--sustained-s", type=float, default=2.5, help="seconds of back-to-back steps (0 = skip)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    w = WORKLOADS[args.workload]
    if args.batch > 0:
        import dataclasses
        w = dataclasses.replace(w, B=args.batch, name=f"{w.name}(batch {args.batch})")
    if args.seq > 0:
        import dataclasses
        w = dataclasses.replace(w, S=args.seq, name=f"{w.name}(S {args.seq})")
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operator has no CPU path")

    import torch.distributed as dist
    import kernelfuser_b200 as kf

    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- inputs: generated once on the CPU from the seed, this rank's head groups only
    sh = head_shard(w.Hq, w.Hkv, rank, world)
    q, k, v, gq, gk, cos, sin = make_workload_inputs(w, seed=0)
    q, k, v = shard_inputs(q, k, v, sh, contiguous=True)
    host = [t.pin_memory() for t in (q, k, v)]
    small = [t.to(dev) for t in (gq, gk, cos, sin)]
    dq, dk, dv = (torch.empty_like(t, device=dev) for t in host)
    for d, h in zip((dq, dk, dv), host):
        d.copy_(h, non_blocking=True)
    out = torch.empty_like(dq)
    kn = torch.empty_like(dk)
    host_out = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    torch.cuda.synchronize()

    def op():
        return kf.optimized_attention(dq, dk, dv, *small, causal=w.causal, eps=w.eps, out=out, kn=kn,
                                      variant=args.variant)

    def op_split(ev):
        # same two launches, with an event between them to time each kernel
        kf.prepare_rows(dk, small[1], small[2], small[3], eps=w.eps, out=kn)
        ev.record()
        kf.attention_forward(dq, kn, dv, small[0], small[2], small[3], out, causal=w.causal, eps=w.eps,
                             variant=args.variant)

    flops_total = attention_flops(w.B, w.Hq, w.S, w.D, w.causal)
    flops_rank = flops_total / world

    # ---- warm-up (the clock sampler already runs, so a short timed region still has samples under load)
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    for _ in range(args.warmup):
        flush.zero_()
        op()
    torch.cuda.synchronize()
    kf.check_status(dev)

    # ---- timed region: K steps, device time of the operator only (flush excluded).  The operator call makes
    # its two launches back to back (the attention kernel dependent on the prepare), so it is timed as a whole.
    # Each timed step is followed by a "split" step - the same two launches with an event between them - whose
    # only purpose is the per-kernel time of the rooflines; interleaving keeps both under the same clock and
    # power conditions (taken afterwards, the split steps ran 5 % slower: the GPU leaves its burst clocks
    # within tens of milliseconds).  `ms_per_step` and `value` come from the K operator calls alone.
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(2)] for _ in range(args.steps)]
    ev2 = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    if sampler:
        sampler.mark_begin()
    wall0 = time.perf_counter()
    for i in range(args.steps):
        flush.zero_()
        ev[i][0].record()
        op()
        ev[i][1].record()
        flush.zero_()
        ev2[i][0].record()
        op_split(ev2[i][1])
        ev2[i][2].record()
    barrier()
    wall = time.perf_counter() - wall0
    if sampler:
        sampler.mark_end()
    clocks = sampler.stop() if sampler else None
    kf.check_status(dev)
    t_step = sum(e[0].elapsed_time(e[1]) for e in ev) / args.steps
    t_prep = sum(e[0].elapsed_time(e[1]) for e in ev2) / args.steps
    t_attn = sum(e[1].elapsed_time(e[2]) for e in ev2) / args.steps
    times = torch.tensor([t_step, t_prep, t_attn], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    t_step, t_prep, t_attn = (float(x) for x in times.tolist())

    # ---- end to end: pinned host inputs -> device, operator, output -> pinned host
    e2e_steps = max(args.e2e_steps, 1)

    def e2e_step():
        # public host-buffer API: pinned host q/k/v -> device (chunked over the batch, copies overlapped
        # with the kernels), operator, output -> pinned host
        kf.optimized_attention_host(host[0], host[1], host[2], *small, causal=w.causal, eps=w.eps,
                                    out=host_out, device=dev)

    e2e_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    t_e2e = torch.tensor([e0.elapsed_time(e1) / e2e_steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t_e2e, op=dist.ReduceOp.MAX)
    t_e2e = float(t_e2e.item())
    kf.check_status(dev)
    h2d = sum(t.numel() * t.element_size() for t in host)
    d2h = host_out.numel() * host_out.element_size()

    # ---- where the end-to-end time goes: this rank's copies alone, each direction by itself
    def timed(fn, reps=3):
        fn()
        torch.cuda.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        a0.record()
        for _ in range(reps):
            fn()
        a1.record()
        barrier()
        return a0.elapsed_time(a1) / reps

    def copy_in():
        for d, h in zip((dq, dk, dv), host):
            d.copy_(h, non_blocking=True)

    t_h2d = timed(copy_in)
    t_d2h = timed(lambda: host_out.copy_(out, non_blocking=True))
    parts = torch.tensor([t_h2d, t_d2h], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(parts, op=dist.ReduceOp.MAX)
    t_h2d, t_d2h = (float(x) for x in parts.tolist())

    # ---- the reference's protocol beside the flushed per-step number: CUDA graphs of 20 back-to-back
    # operator calls, fresh captures in each of 5 rounds, 7 replays per round, L2-warm (fixed buffers)
    from kernelfuser_b200.timing import paired
    gp = None
    if not args.no_graph:
        g = paired({"op": op}, rounds=5, samples=7, replays=20)
        stats = torch.tensor([g["op"]["median_us"], g["op"]["p10_us"], g["op"]["p90_us"]], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        med, p10, p90 = (float(x) for x in stats.tolist())
        gp = {"median_us": med, "p10_us": p10, "p90_us": p90, "tflops": flops_total / (med * 1e-6) / 1e12,
              "protocol": g["protocol"], "reduction": "max over ranks of each statistic"}

    # ---- sustained: the same step back to back for a few seconds (no flush), clocks and power sampled
    sus = None
    if args.sustained_s > 0:
        n_sus = max(int(args.sustained_s * 1e3 / max(t_step, 1e-3)), 10)
        s_sampler = ClockSampler(local, period_s=0.01) if rank == 0 else None
        if s_sampler:
            s_sampler.start()
        barrier()
        if s_sampler:
            s_sampler.mark_begin()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(n_sus):
            op()
        b1.record()
        barrier()
        if s_sampler:
            s_sampler.mark_end()
        s_clocks = s_sampler.stop() if s_sampler else None
        t_sus = torch.tensor([b0.elapsed_time(b1) / n_sus], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t_sus, op=dist.ReduceOp.MAX)
        t_sus = float(t_sus.item())
        kf.check_status(dev)
        sus = {"steps": n_sus, "ms_per_step": t_sus, "seconds": n_sus * t_sus * 1e-3,
               "value": flops_total / (t_sus * 1e-3) / 1e12, "unit": UNIT, "clocks": s_clocks}

    if rank == 0:
        peaks = load_peaks(ROOT)
        tag = "of measured" if peaks["source"] == "measured" else "of fallback"
        value = flops_total / (t_step * 1e-3) / 1e12
        attn_tf = flops_rank / (t_attn * 1e-3) / 1e12
        prep_b = prepare_bytes(w.B, sh.n_kv, w.S, w.D)
        # algorithmic bytes of the attention launch: Q and O once, prepared K and V once (16-bit elements)
        attn_bytes = 2.0 * w.B * w.S * w.D * (2 * sh.n_q + 2 * sh.n_kv)
        prep_gbs = prep_b / (t_prep * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": t_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": DTYPE_NAME[w.dtype], "data": "synthetic",
            "config": workload_config(w, world),
            "pct_of_nominal_bf16_peak": 100.0 * value / (2250.0 * world),
            "roofline": {"kernel": "attention", "bound": "tensor", "achieved": attn_tf, "peak": peaks["bf16_tflops"],
                         "unit": "TFLOP/s", "frac": attn_tf / peaks["bf16_tflops"],
                         "traffic": NCU_DRAM_BYTES_FULL.get((w.name, "attention")) if world == 1 else None,
                         "algorithmic_bytes": attn_bytes,
                         "traffic_source": "ncu dram read+write of one launch at this size (N=1 only)",
                         "peak_source": f"{tag} (cuBLAS bf16 burst)", "ms_per_launch": t_attn,
                         "flops_per_launch": flops_rank},
            "roofline_prepare": {"kernel": "prepare_rows(K)", "bound": "hbm", "achieved": prep_gbs,
                                 "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": prep_gbs / peaks["hbm_gbs"],
                                 "traffic": NCU_DRAM_BYTES_FULL.get((w.name, "prepare")) if world == 1 else None,
                                 "peak_source": tag, "ms_per_launch": t_prep,
                                 "bytes_per_launch": prep_b},
            "e2e": {"value": flops_total / (t_e2e * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d * world,
                    "d2h_bytes_per_step": d2h * world, "ms_per_step": t_e2e, "steps": e2e_steps,
                    "breakdown_ms": {"h2d_alone": t_h2d, "d2h_alone": t_d2h, "kernels": t_step,
                                     "note": "slowest rank; each direction copied by itself, all ranks at once"},
                    "h2d_gbs_per_rank": h2d / (t_h2d * 1e-3) / 1e9, "d2h_gbs_per_rank": d2h / (t_d2h * 1e-3) / 1e9},
            "gpu_launches": 4 * args.steps,  # row-prepare + attention per timed step, and per interleaved split step
            "clocks": clocks,
            "wall_s_timed_region": wall,
        }
        if gp is not None:
            line["graph_protocol"] = gp
        if sus is not None:
            sus["frac_of_sustained_peak"] = sus["value"] / (peaks.get("bf16_tflops_sustained") or peaks["bf16_tflops"]) / world
            sus["peak"] = peaks.get("bf16_tflops_sustained")
            line["sustained"] = sus
        if world == 1 and not args.no_cpu_baseline:
            val, cores, desc = cpu_oracle_rate(w)
            line["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
