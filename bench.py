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
# runs the call on the forward pass's workspace, which skips its two prepasses, so they are left out: input-gradient
# kernel 472.2 MB read + 106.9 MB written, offsets-gradient kernel 472.5 MB read + 0.2 MB written, partial-sum
# reduce 9.9 MB, the three gated exact kernels 0.1 MB.
NCU_DRAM_BYTES_PER_SAMPLE = {"mex_backward[C64 32x32 M128 K64 N1024 R4 dy/4]": 1061.8e6 / 512}


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
    sample = min(len(x), args.ref_sample if args.ref_sample > 0 else 8 * cores)      # eight samples per thread: ~2.5 s per step
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
TF32_FRACTION_OF_BF16 = 0.5      # dense TF32 tensor throughput is half the BF16 figure of MEASURED_PEAKS.json (no TF32 peak is measured)
# arithmetic FP32 lane operations per (instance, tap, position) term of the Similarity kernels, by op and function
SIM_OPS_PER_TERM = {"similarity_forward": 3, "similarity_input_grad": 3, "similarity_params_grad": 5}


def op_roofline(key, r, hbm_gbs, tf32_tflops, fp32_tfma):
    """Which roofline binds one operator call and what fraction of it the call reaches.
    MEX: the slower of HBM time for the algorithmic bytes and tensor-core time for the three split-TF32 products of
    every term.  Similarity: HBM time against FP32-pipe time at SIM_OPS_PER_TERM lane operations per term."""
    ms = r["ms"] / r["calls"]
    nbytes, terms = r["bytes"] / r["calls"], r["terms"] / r["calls"]
    name = key.split("[")[0]
    t_hbm = nbytes / (hbm_gbs * 1e9) * 1e3
    out = {"hbm_GBps": round(nbytes / (ms * 1e-3) / 1e9, 1), "hbm_frac": round(t_hbm / ms, 4)}
    if name.startswith("mex"):
        t_alt = terms * 2 * 3 / (tf32_tflops * 1e12) * 1e3
        out.update(bound="tensor" if t_alt > t_hbm else "hbm", tensor_frac=round(t_alt / ms, 4),
                   tensor_TFLOPs=round(terms * 6 / (ms * 1e-3) / 1e12, 1))
    else:
        t_alt = terms * SIM_OPS_PER_TERM.get(name, 3) / (fp32_tfma * 1e12) * 1e3 if fp32_tfma else 0.0
        out.update(bound="fp32" if t_alt > t_hbm else "hbm", fp32_frac=round(t_alt / ms, 4))
    out["frac"] = round(max(t_hbm, t_alt) / ms, 4)
    return out


def fp32_peak(torch, dev):
    """Measured FP32 fused multiply-adds per second (scalar and packed instruction), by the library's probe kernel."""
    from simnets_tf_b200 import _lib
    scratch = torch.zeros(4, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream
    out = {}
    for name, packed in (("scalar", 0), ("packed", 1)):
        best = 0.0
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            n = _lib.lib().simnets_fp32_fma_probe(packed, 4096, scratch.data_ptr(), stream)
            e1.record()
            e1.synchronize()
            if n > 0:
                best = max(best, n / (e0.elapsed_time(e1) * 1e-3))
        out[name] = best / 1e12
    return out


def cfg4_section(torch, dev, hbm_gbs, tf32_tflops):
    """The op pair of BASELINE configs[3] (N=256, C=64, 32x32, 20 % NaN; Similarity 256 x 3x3 then MEX 256 x [4,2,2]) through
    the C ABI at the configuration's batch: device time per call, terms/s and fractions of the FP32 pipe and of HBM.
    (4a = L2 with NaN-aware normalisation, the variant of the invalid literal config that the reference accepts.)"""
    from simnets_tf_b200 import opbench
    peak = fp32_peak(torch, dev)
    fma = max(peak.values())
    out = {"fp32_peak_TFMAs": {k: round(v, 2) for k, v in peak.items()}, "fp32_nominal_TFMAs": round(148 * 128 * 1.965e9 / 1e12, 2),
           "batch": 256, "sim": {}, "mex": {}}
    for layer, group, ops in (("cfg4_sim", "sim", ("forward", "input_grad", "params_grad")),
                              ("cfg4_mex", "mex", ("forward", "input_grad", "offsets_grad"))):
        for op in ops:
            r = opbench.run(layer, op, 256, 10, 3)
            row = {"calls": 1, "ms": r["ms_per_call"], "bytes": r["algorithmic_bytes"], "terms": r["terms"]}
            rf = op_roofline(r["op"], row, hbm_gbs, tf32_tflops, fma)
            rf.update(ms=round(r["ms_per_call"], 4), Tterms_per_s=round(r["Gterms_per_s"] / 1e3, 3))
            out[group][op] = rf
    return out


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

    # ---- do the N-way sharded gradients, summed by NCCL, equal the gradients of the whole batch on one GPU?
    # 64 samples: every rank differentiates its shard, the bucket is all-reduced, rank 0 differentiates all 64 as well.
    grad_check = None
    if world > 1:
        nchk = 64
        clo, chi = dp.shard_bounds(nchk, world, rank)
        xc, lc = torch.from_numpy(x_all[:nchk]).to(dev), torch.from_numpy(l_all[:nchk]).to(dev)
        bucket.zero()
        if chi > clo:
            net.loss(xc[clo:chi], lc[clo:chi], nchk).backward()
        bucket.all_reduce()
        summed = bucket.flat.clone()
        bucket.zero()
        worst = 0.0
        if rank == 0:
            net.loss(xc, lc, nchk).backward()
            off = 0
            for p in bucket.params:
                a, b = summed[off:off + p.numel()], bucket.flat[off:off + p.numel()]
                worst = max(worst, float((a - b).abs().max() / b.abs().max().clamp_min(1e-30)))
                off += p.numel()
        barrier()
        grad_check = {"samples": nchk, "max_rel_err": worst, "tolerance": 1e-4, "ok": bool(worst <= 1e-4),
                      "what": "per parameter tensor, max |sum over ranks - one GPU| / max |one GPU|"}

    # ---- forward + backward as two CUDA graphs around the cut of dp.OverlappedStep (at 256 samples per GPU the step is
    # about a millisecond behind ~60 launches, so replaying graphs keeps the host off the critical path); the two
    # all-reduces are enqueued eagerly, the first on a second stream while the second graph runs.
    for _ in range(args.warmup):
        bucket.zero()
        net.loss(x_dev, l_dev, gb).backward()
        bucket.all_reduce()
    barrier()
    n0 = _lib.launch_count()
    stepper = dp.OverlappedStep(net, bucket, x_dev, l_dev, gb, graphs=not args.no_graph)
    launches_per_step = (_lib.launch_count() - n0) // 3 if not args.no_graph else 0      # two warm-up passes + the capture
    for _ in range(2):
        stepper.run()
    barrier()

    # ---- device-resident timing (inputs already in HBM): R repeats of K steps, each repeat bracketed by a barrier and
    # a device synchronisation; the reported time is the median repeat (max over ranks per repeat)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    repeat_ms = []
    # at least R repeats, and more while the timed windows add up to less than two seconds (short steps on many GPUs), so
    # that the clock sampler sees the device under load; every rank takes the same decision (the times are maxima over ranks)
    while len(repeat_ms) < args.repeats or (sum(repeat_ms) < 2000.0 and len(repeat_ms) < 40 * args.repeats):
        barrier()
        e0.record()
        for _ in range(args.steps):
            stepper.run()
        e1.record()
        barrier()
        repeat_ms.append(max_over_ranks(e0.elapsed_time(e1)))
    ms = statistics.median(repeat_ms)
    launches = launches_per_step * args.steps if not args.no_graph else (_lib.launch_count() - launches0) // len(repeat_ms)
    clocks = sampler.stop() if rank == 0 else None

    # ---- per-operator device time: K steps launched eagerly with CUDA events around every call of the library
    # (events cannot bracket kernels inside a replayed graph)
    eager = dp.OverlappedStep(net, bucket, x_dev, l_dev, gb, graphs=False)
    eager.run()
    PROFILE.start()
    for _ in range(args.steps):
        eager.run()
    ops = PROFILE.stop()
    barrier()

    # ---- end to end: pinned host inputs -> device, step, loss back to the host, every step.  The next step's inputs
    # travel on a copy stream while the current step computes; a device-to-device copy hands them to the graphs' buffers.
    h2d = x_host.numel() * x_host.element_size() + l_host.numel() * l_host.element_size()
    loss_host = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(2)]
    loss_ready = [torch.cuda.Event(), torch.cuda.Event()]
    copy_stream = torch.cuda.Stream(device=dev)
    x_next, l_next = torch.empty_like(x_dev), torch.empty_like(l_dev)
    arrived, consumed = torch.cuda.Event(), torch.cuda.Event()

    def prefetch():
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed)              # the staging buffers have been handed over
            x_next.copy_(x_host, non_blocking=True)
            l_next.copy_(l_host, non_blocking=True)
            arrived.record(copy_stream)

    def e2e_launch(i):
        """Enqueue step i: inputs from the staging buffers, the step, its loss on the way to pinned host memory."""
        main = torch.cuda.current_stream()
        main.wait_event(arrived)
        x_dev.copy_(x_next, non_blocking=True)            # the graphs read these two buffers
        l_dev.copy_(l_next, non_blocking=True)
        consumed.record(main)
        prefetch()                                        # the step after this one
        loss = stepper.run()
        loss_host[i & 1].copy_(loss.detach(), non_blocking=True)
        loss_ready[i & 1].record(main)

    def e2e_read(i):
        """The host reads step i's loss (waits for it to arrive)."""
        loss_ready[i & 1].synchronize()
        return float(loss_host[i & 1])

    def e2e_steps(k):
        """k steps; every step's loss is read on the host, the one of step i while step i + 1 is already running, so that
        the host's work of launching a step is not serialised with the device's work of running one."""
        for i in range(k):
            e2e_launch(i)
            if i > 0:
                e2e_read(i - 1)
        return e2e_read(k - 1)

    consumed.record(torch.cuda.current_stream())
    prefetch()
    e2e_steps(2)
    e2e_ms = []
    for _ in range(max(1, args.repeats // 5)):
        barrier()
        e0.record()
        last_loss = e2e_steps(args.steps)                 # returns after the last loss has been read
        e1.record()
        barrier()
        e2e_ms.append(max_over_ranks(e0.elapsed_time(e1)))
    ms_e2e = statistics.median(e2e_ms)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_src = measured_peaks()
    hbm_peak = float(peaks["hbm_gbs"])
    tf32_peak = float(peaks.get("bf16_tflops", 1590.0)) * TF32_FRACTION_OF_BF16
    fma_peak = max(fp32_peak(torch, dev).values())
    # operator call groups by device time inside the eager pass, each with the roofline that binds it
    table = []
    for key, r in ops.items():
        avg_ms = r["ms"] / r["calls"]
        row = {"op": key, "calls": r["calls"], "ms_total": round(r["ms"], 4), "ms_per_call": round(avg_ms, 5),
               "Gterms_per_s": round(r["terms"] / r["calls"] / (avg_ms * 1e-3) / 1e9, 2)}
        row.update(op_roofline(key, r, hbm_peak, tf32_peak, fma_peak))
        table.append(row)
    table.sort(key=lambda r: -r["ms_total"])
    top = table[0]
    # DRAM traffic of the dominant call from one ncu capture at a smaller batch, scaled to this batch (every byte these
    # kernels touch belongs to one sample); null for an op that has no capture
    m = re.match(r"(\w+)\[B(\d+) (.*)\]$", top["op"])
    per_sample = NCU_DRAM_BYTES_PER_SAMPLE.get("%s[%s]" % (m.group(1), m.group(3))) if m else None
    traffic = int(per_sample * int(m.group(2))) if per_sample else None
    if top["bound"] == "tensor":
        roofline = {"kernel": top["op"], "bound": "tensor", "achieved": top["tensor_TFLOPs"], "peak": tf32_peak, "unit": "TFLOP/s",
                    "frac": top["tensor_frac"], "peak_source": "half the BF16 burst of " + peak_src + " peaks (TF32)", "traffic": traffic}
    elif top["bound"] == "fp32":
        # a Similarity call bound by the FP32 pipe (a small batch can put it first): lane operations per second against
        # the FFMA rate measured on this device
        ops_per_term = SIM_OPS_PER_TERM.get(top["op"].split("[")[0], 3)
        roofline = {"kernel": top["op"], "bound": "fp32", "achieved": round(top["Gterms_per_s"] * ops_per_term / 1e3, 2),
                    "peak": round(fma_peak, 2), "unit": "T lane-ops/s", "frac": top["fp32_frac"],
                    "peak_source": "FFMA issue rate measured by the library's probe on this device", "traffic": traffic}
    else:
        roofline = {"kernel": top["op"], "bound": "hbm", "achieved": top["hbm_GBps"], "peak": hbm_peak, "unit": "GB/s",
                    "frac": top["hbm_frac"], "peak_source": "of " + peak_src, "traffic": traffic}
    roofline["share_of_step"] = round(top["ms_total"] / args.steps / (ms / args.steps), 4)

    line = {
        "metric": "similarity_mex_fwd_bwd_samples_per_s", "value": gb * args.steps / (ms * 1e-3), "unit": "samples/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload, "global_batch": gb, "per_gpu_batch": hi - lo, "parallelism": "dp%d" % world,
                   "launch": "eager" if args.no_graph else "two cuda graphs per step, all-reduce of the deep layers' gradients overlapped with the rest of the backward pass",
                   "input": list(spec["input_shape"]), "l2": "per-step working set (>0.5 GB of activations per 256 samples) exceeds the 126 MB L2",
                   "grad_bucket_bytes": bucket.nbytes(), "repeats": len(repeat_ms),
                   "timing": "median over %d repeats of %d steps (min %.3f, max %.3f ms per step)" % (
                       len(repeat_ms), args.steps, min(repeat_ms) / args.steps, max(repeat_ms) / args.steps)},
        "clocks": clocks,
        "e2e": {"value": gb * args.steps / (ms_e2e * 1e-3), "unit": "samples/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4,
                "ms_per_step": ms_e2e / args.steps, "loss": last_loss,
                "how": "inputs prefetched from pinned memory on a copy stream one step ahead; every step's loss is copied to pinned memory and read by the host, step i's while step i + 1 runs, the last one before the closing event"},
        "gpu_launches": launches,
        "roofline": roofline,
        "ops": table[:12],
    }
    if grad_check is not None:
        line["grad_check"] = grad_check
    if world == 1 and not args.no_cfg4:
        line["cfg4"] = cfg4_section(torch, dev, hbm_peak, tf32_peak)
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
    ap.add_argument("--ref-sample", type=int, default=0, help="samples per reference step (default: eight per host core)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="launch every step eagerly instead of replaying CUDA graphs")
    ap.add_argument("--repeats", type=int, default=25, help="timed repeats of the K steps; the median repeat is reported")
    ap.add_argument("--no-cfg4", action="store_true", help="skip the single-operator section of the large op pair")
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
