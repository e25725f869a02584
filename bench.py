#!/usr/bin/env python
"""Benchmark of the Similarity + MEX hot path: forward + backward samples/s of the data-parallel
SimNet configuration (cfg5: 3x32x32 inputs, global batch 2048 split over the GPUs, Similarity(64, 3x3)
-> 3 x [MEX + 2x2 sum-pool] -> MEX(10), softmax cross-entropy, parameter gradients all-reduced).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg5|cfg3]

N > 1 is launched by torch.distributed.run, one rank per GPU.  Rank 0 prints ONE JSON line.
Data are synthetic (seeded uniform images, random labels) and parameters randomly initialised.

`--impl reference` times the reference project's own CPU operators (oracle/_ref, else the CPU
restatement) on the host cores, on a bounded sample of the same workload per step.
"""
import argparse
import json
import os
import re
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GLOBAL_BATCH = {"cfg5": 2048, "cfg3": 256}
DATA_SEED = {"cfg5": 4, "cfg3": 2}
FALLBACK_HBM_GBS = 6650.0          # earlier measurement on this pool, used only without MEASURED_PEAKS.json
NOMINAL_FP32_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12
# dram__bytes_read.sum + dram__bytes_write.sum of one whole library call, per sample, from ncu at batch 512
# (kernel by kernel in profiles/mex_backward_cfg5_mex1.md); key = operator signature without its batch.  The step
# runs the call on the forward pass's workspace, which skips its two prepasses: their 134.9 MB are taken out.
NCU_DRAM_BYTES_PER_SAMPLE = {"mex_backward[C64 32x32 M128 K64 N1024 R4 dy/4]": (1249.5e6 - 134.9e6) / 512}


def make_data(workload, spec):
    rng = np.random.default_rng(DATA_SEED[workload])
    n = GLOBAL_BATCH[workload]
    x = rng.uniform(-0.5, 0.5, size=(n,) + tuple(spec["input_shape"])).astype(np.float32)
    labels = rng.integers(0, spec["classes"], size=n).astype(np.int64)
    return x, labels


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": FALLBACK_HBM_GBS}, "fallback"


class ClockSampler(object):
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu, self.proc = gpu_index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons, power = [], [], set(), []
        for line in out.splitlines():
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2])); power.append(float(f[3]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------- CPU legs
def cpu_net(workload, threads):
    from oracle import oracle
    from oracle.simnet_cpu import CpuSimNet
    from simnets_tf_b200.netspec import SPECS
    if not oracle.available("port") and not oracle.available("reference"):
        oracle.build()
    kind = "reference" if oracle.available("reference") else "port"
    return CpuSimNet(SPECS[workload], oracle.load(kind), seed=DATA_SEED[workload], threads=threads), kind


def cpu_step_time(net, x, labels, sample, global_batch):
    t0 = time.perf_counter()
    net.step(x[:sample], labels[:sample], global_batch)
    return time.perf_counter() - t0


def cpu_baseline(workload, x, labels, budget_s=20.0):
    """The CPU operators on all host cores over a bounded sample (a few samples per core), ~budget_s of work."""
    from oracle.simnet_cpu import host_cores
    cores = host_cores()
    net, kind = cpu_net(workload, cores)
    probe = min(len(x), cores)
    t = cpu_step_time(net, x, labels, probe, GLOBAL_BATCH[workload])
    per_round = max(t, 1e-3)
    rounds = int(max(1, min(8, budget_s / per_round - 1)))
    sample = min(len(x), probe * rounds)
    t = cpu_step_time(net, x, labels, sample, GLOBAL_BATCH[workload])
    return {"value": sample / t, "unit": "samples/s", "cores": cores, "kind": kind,
            "sample": "%d of %d samples of one %s step (fwd+bwd), batch split over %d threads, %.1f s" % (
                sample, GLOBAL_BATCH[workload], workload, cores, t)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle.simnet_cpu import host_cores
    from simnets_tf_b200.netspec import SPECS
    workload = args.workload
    x, labels = make_data(workload, SPECS[workload])
    cores = host_cores()
    net, kind = cpu_net(workload, cores)
    sample = min(len(x), args.ref_sample if args.ref_sample > 0 else max(8, cores))
    for _ in range(args.warmup):
        cpu_step_time(net, x, labels, sample, GLOBAL_BATCH[workload])
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_step_time(net, x, labels, sample, GLOBAL_BATCH[workload])
    dt = time.perf_counter() - t0
    value = sample * args.steps / dt
    line = {
        "impl": "reference", "metric": "similarity_mex_fwd_bwd_samples_per_s", "value": value, "unit": "samples/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "global_batch": GLOBAL_BATCH[workload], "parallelism": "cpu threads over the batch",
                   "sample_per_step": sample},
        "cpu_baseline": {"value": value, "unit": "samples/s", "cores": cores, "kind": kind,
                         "sample": "%d of %d samples per step, batch split over %d threads" % (sample, GLOBAL_BATCH[workload], cores)},
        "e2e": {"value": value, "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------- GPU leg
def run_ours(args):
    import torch
    import torch.distributed as dist
    from simnets_tf_b200 import _lib, dp
    from simnets_tf_b200._torch_glue import PROFILE
    from simnets_tf_b200.simnet import SPECS, SimNet

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit("--gpus %d but WORLD_SIZE=%d: launch N>1 with torch.distributed.run" % (args.gpus, world))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()   # fail loudly here if the CUDA library is missing

    workload = args.workload
    spec = SPECS[workload]
    gb = GLOBAL_BATCH[workload]
    x_all, l_all = make_data(workload, spec)
    lo, hi = dp.shard_bounds(gb, world, rank)
    x_host = torch.from_numpy(x_all[lo:hi]).pin_memory()
    l_host = torch.from_numpy(l_all[lo:hi]).pin_memory()
    x_dev, l_dev = x_host.to(dev), l_host.to(dev)
    net = SimNet(spec, seed=DATA_SEED[workload], device=dev)
    bucket = dp.GradBucket(net.parameters())

    def compute(xd, ld):
        bucket.zero()
        loss = net.loss(xd, ld, gb)
        loss.backward()
        return loss

    def step(xd, ld):
        loss = compute(xd, ld)
        bucket.all_reduce()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- forward + backward as ONE CUDA graph: at 256 samples per GPU the step is a few ms of device time behind
    # ~600 launches, so replaying a graph keeps the host off the critical path.  The bucket all-reduce is enqueued
    # eagerly right behind each replay (one launch), on the same stream; it is not part of the capture.
    graph, loss_static, launches_per_step = None, None, 0
    for _ in range(args.warmup):
        step(x_dev, l_dev)
    barrier()
    if not args.no_graph:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(2):
                compute(x_dev, l_dev)
        torch.cuda.current_stream().wait_stream(side)
        barrier()
        graph = torch.cuda.CUDAGraph()
        n0 = _lib.launch_count()
        with torch.cuda.graph(graph):
            loss_static = compute(x_dev, l_dev)
        launches_per_step = _lib.launch_count() - n0
        barrier()

    def run_step():
        if graph is not None:
            graph.replay()
            bucket.all_reduce()
            return loss_static
        return step(x_dev, l_dev)

    for _ in range(2):
        run_step()
    barrier()

    # ---- device-resident timing (inputs already in HBM)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    barrier()
    ms = max_over_ranks(e0.elapsed_time(e1))
    launches = launches_per_step * args.steps if graph is not None else _lib.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None

    # ---- per-operator device time: the same K steps again, launched eagerly with CUDA events around every call of
    # the library (events cannot bracket kernels inside a replayed graph)
    PROFILE.start()
    for _ in range(args.steps):
        step(x_dev, l_dev)
    ops = PROFILE.stop()
    barrier()

    # ---- end to end: pinned host inputs -> device, step, loss back to the host, every step
    h2d = x_host.numel() * x_host.element_size() + l_host.numel() * l_host.element_size()
    loss_host = torch.empty((), dtype=torch.float32).pin_memory()

    def e2e_step():
        x_dev.copy_(x_host, non_blocking=True)        # the graph reads these two buffers
        l_dev.copy_(l_host, non_blocking=True)
        loss = run_step()
        loss_host.copy_(loss.detach(), non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return float(loss_host)

    for _ in range(min(args.warmup, 2)):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(args.steps):
        last_loss = e2e_step()
    e1.record()
    barrier()
    ms_e2e = max_over_ranks(e0.elapsed_time(e1))

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_src = measured_peaks()
    hbm_peak = float(peaks["hbm_gbs"])
    # dominant operator call group by device time inside the timed region
    table = []
    for key, r in ops.items():
        avg_ms = r["ms"] / r["calls"]
        table.append({"op": key, "calls": r["calls"], "ms_total": round(r["ms"], 4), "ms_per_call": round(avg_ms, 5),
                      "GBps": round(r["bytes"] / r["calls"] / (avg_ms * 1e-3) / 1e9, 2),
                      "Gterms_per_s": round(r["terms"] / r["calls"] / (avg_ms * 1e-3) / 1e9, 2)})
    table.sort(key=lambda r: -r["ms_total"])
    top = table[0]
    # DRAM traffic of the dominant call from one ncu capture at a smaller batch, scaled to this batch (every byte these
    # kernels touch belongs to one sample); null for an op that has no capture
    m = re.match(r"(\w+)\[B(\d+) (.*)\]$", top["op"])
    per_sample = NCU_DRAM_BYTES_PER_SAMPLE.get("%s[%s]" % (m.group(1), m.group(3))) if m else None
    traffic = int(per_sample * int(m.group(2))) if per_sample else None
    roofline = {"kernel": top["op"], "bound": "hbm", "achieved": top["GBps"], "peak": hbm_peak, "unit": "GB/s",
                "frac": round(top["GBps"] / hbm_peak, 4), "peak_source": "of " + peak_src, "traffic": traffic,
                "share_of_step": round(top["ms_total"] / ms, 4),
                "fp32": {"Gterms_per_s": top["Gterms_per_s"], "nominal_fp32_tflops": round(NOMINAL_FP32_TFLOPS, 2)}}

    line = {
        "metric": "similarity_mex_fwd_bwd_samples_per_s", "value": gb * args.steps / (ms * 1e-3), "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "global_batch": gb, "per_gpu_batch": hi - lo, "parallelism": "dp%d" % world, "launch": "eager" if graph is None else "cuda graph replay",
                   "input": list(spec["input_shape"]), "l2": "per-step working set (>0.5 GB of activations per 256 samples) exceeds the 126 MB L2",
                   "grad_bucket_bytes": bucket.nbytes()},
        "clocks": clocks,
        "e2e": {"value": gb * args.steps / (ms_e2e * 1e-3), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                "ms_per_step": ms_e2e / args.steps, "loss": last_loss},
        "gpu_launches": launches,
        "roofline": roofline,
        "ops": table[:12],
    }
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(workload, x_all, l_all)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(GLOBAL_BATCH), default="cfg5")
    ap.add_argument("--ref-sample", type=int, default=0, help="samples per reference step (default: one per host core, at least 8)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying one CUDA graph")
    ap.add_argument("--global-batch", type=int, default=0,
                    help="diagnostics only: another global batch than the configuration's (e.g. 256 on one GPU = the per-GPU share of 8)")
    args = ap.parse_args()
    if args.global_batch:
        GLOBAL_BATCH[args.workload] = args.global_batch
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
