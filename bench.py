#!/usr/bin/env python
"""Benchmark of the B200Acc hot path: int8 ResNet-50 images/s at global batch 256 (the headline configuration).

    python bench.py [--gpus N] [--steps K] [--warmup W]            the B200 arm
    python bench.py --impl reference [--steps K] [--warmup W]      the reference's own CpuRef on host cores

One "step" = one pass of the whole ResNet-50 graph (batch 256 in total, sharded by batch rows over the N ranks,
no collective on the data path).  Prints ONE JSON line on rank 0:
  value      images/s with the input batch already resident in HBM (CUDA events on the network's stream,
             barrier + synchronize on both sides, max over ranks)
  e2e        images/s through LoadedNetwork.EnqueueAsync / WaitOutputs with pinned HOST buffers: every request's H2D
             copy of the image batch and D2H read of the class scores are inside the timed region; the copy of the next
             request overlaps the compute of the current one
  roofline   the dominant kernel family's achieved int8 throughput against the measured tensor peak
  cpu_baseline  the reference's CpuRef timed on this box's host cores on a bounded sample (N = 1 only)
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GLOBAL_BATCH = 256
IMAGE = 224


# dram__bytes_read.sum + dram__bytes_write.sum per convolution launch, averaged over the 53 convolution launches of
# one batch-256 step, from an ncu capture of this file's own command
CONV_DRAM_BYTES_PER_LAUNCH = 102.1e6


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) >= 9:
                for i, nme in enumerate(names):
                    if r[5 + i].lower().startswith("active"):
                        reasons.add(nme)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CpuRef, one single-threaded instance per host core
# ---------------------------------------------------------------------------------------------------------------

def _cpuref_worker(args):
    """Child process: build the batch-1 ResNet-50 graph, load it on CpuRef, run `passes` timed inferences."""
    passes, warm = args
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    from armnn_b200 import configs
    net, info = configs.resnet50(1, IMAGE)
    x = np.random.default_rng(0).integers(-128, 128, size=info["input_shape"]).astype(np.int8)
    import hostnet
    import q8util
    if q8util.have_cpuref():
        runner = hostnet.ArmnnNetwork(net, "CpuRef")
        kind = "reference"
    else:
        from armnn_b200 import network
        os.environ["OMP_NUM_THREADS"] = "1"
        runner = hostnet.OracleNetwork(network.Optimize(net))
        kind = "port"
    times = []
    for i in range(warm + passes):
        t = time.perf_counter()
        runner.run({0: x})
        if i >= warm:
            times.append(time.perf_counter() - t)
    return kind, times


def cpuref_images_per_s(steps, warmup, cores=None):
    """Every step: each of `cores` worker processes pushes ONE 224x224 image through CpuRef (batch rows are
    independent, CpuRef itself is single-threaded).  images/s = cores / slowest worker's mean step time."""
    import multiprocessing as mp
    cores = cores or min(len(os.sched_getaffinity(0)), 64)        # bounded: each worker is a whole process
    ctx = mp.get_context("spawn")
    with ctx.Pool(cores) as pool:
        res = pool.map(_cpuref_worker, [(steps, warmup)] * cores)
    kind = res[0][0]
    per_step = [max(r[1][i] for r in res) for i in range(steps)]           # slowest worker per step
    mean = sum(per_step) / len(per_step)
    return {"value": cores / mean, "unit": "images/s", "cores": cores, "kind": kind,
            "sample": "%d step(s) of 1 image per core (batch-1 ResNet-50 224x224 graph, %d single-threaded "
                      "CpuRef instances in parallel)" % (steps, cores), "ms_per_step": mean * 1e3}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    base = cpuref_images_per_s(args.steps, max(args.warmup, 0))
    line = {"impl": "reference", "metric": "int8 ResNet-50 images/s", "value": base["value"], "unit": "images/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": base["ms_per_step"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32 (CpuRef dequantises int8 to float)",
            "data": "synthetic", "config": _config(args.gpus),
            "cpu_baseline": {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")},
            "e2e": {"value": base["value"], "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def _config(n_gpus):
    return {"workload": "ResNet-50 int8 (QAsymmS8 activations, per-channel QSymmS8 weights), 224x224, random-init, "
                        "global batch 256 sharded by rows", "global_batch": GLOBAL_BATCH, "per_gpu_batch": GLOBAL_BATCH // n_gpus,
            "image": IMAGE, "parallelism": "replica-per-GPU batch sharding x%d, no collective" % n_gpus,
            "l2": "no explicit flush: one step writes and re-reads %.2f GB of layer tensors per GPU (16.8 MB per image), "
                  "above the 126 MB L2" % (16.8e-3 * (GLOBAL_BATCH // n_gpus))}


# ---------------------------------------------------------------------------------------------------------------
# the B200 arm
# ---------------------------------------------------------------------------------------------------------------

def run_b200(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from armnn_b200 import configs, network

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torchrun with %d ranks" % (args.gpus, args.gpus))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200Acc kernels have no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    per_gpu = GLOBAL_BATCH // world

    net, info = configs.resnet50(per_gpu, IMAGE)
    rt = network.IRuntime.Create(local)
    nid = rt.LoadNetwork(network.Optimize(net, ["B200Acc"]))
    ln = rt.GetLoadedNetwork(nid)
    rng = np.random.default_rng(1000 + rank)
    host_in = torch.from_numpy(rng.integers(-128, 128, size=info["input_shape"]).astype(np.int8)).pin_memory()
    host_out = torch.empty(info["output_shape"], dtype=torch.int8).pin_memory()
    ln.input_tensor(0).copy_(host_in.cuda(), non_blocking=False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(seconds):
        if world == 1:
            return seconds
        t = torch.tensor([seconds], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident throughput ----
    ln.Execute()
    torch.cuda.synchronize()
    ln.CaptureGraph()          # the whole workload queue as one CUDA graph: no per-workload host launch in the step
    for _ in range(args.warmup):
        ln.Execute()
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    with torch.cuda.stream(ln.stream):
        e0.record()
        for _ in range(args.steps):
            launches += ln.Execute()
        e1.record()
    barrier()
    dev_s = max_over_ranks(e0.elapsed_time(e1) / 1e3)
    clocks = sampler.stop() if rank == 0 else None

    # ---- end to end with host buffers ----
    # Requests are pipelined as a serving loop would: the H2D copy of request i + 1 runs on a copy stream while request i
    # computes (it starts once request i's first workload has consumed the input tensor); every request's H2D copy and
    # D2H read are inside the timed region.
    ln.CapturePipelined()
    for _ in range(min(args.warmup, 3)):
        ln.WaitOutputs(ln.EnqueueAsync({0: host_in}), {0: host_out})
    barrier()
    t0 = time.perf_counter()
    prev = None
    for _ in range(args.steps):
        ticket = ln.EnqueueAsync({0: host_in})
        if prev is not None:
            ln.WaitOutputs(prev, {0: host_out})
        prev = ticket
    ln.WaitOutputs(prev, {0: host_out})
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()

    # ---- per-kernel-family timing (same conditions, right after the timed region) ----
    fam = {}
    if rank == 0:
        evs = []
        with torch.cuda.stream(ln.stream):
            for _ in range(args.steps):
                for layer, entry, params in ln.workloads:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    network.lib.call(entry, params, ln.stream.cuda_stream)
                    b.record()
                    evs.append((layer, entry, a, b))
        torch.cuda.synchronize()
        macs = {l[0]: l[4] for l in info["layers"]}
        for layer, entry, a, b in evs:
            f = fam.setdefault(entry, {"ms": 0.0, "launches": 0, "macs": 0})
            f["ms"] += a.elapsed_time(b)
            f["launches"] += 1
            f["macs"] += macs.get(layer.name, 0)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = _peaks()
    images = GLOBAL_BATCH * args.steps
    top = max(fam, key=lambda k: fam[k]["ms"])
    total_ms = sum(f["ms"] for f in fam.values())
    tensor_peak = 2.0 * peaks["bf16_tflops_sustained"]        # int8 runs at twice the bf16 rate on the same pipe
    if fam[top]["macs"] > 0:
        achieved = 2.0 * fam[top]["macs"] / (fam[top]["ms"] / 1e3) / 1e12
        roofline = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": tensor_peak, "unit": "TFLOP/s",
                    "frac": achieved / tensor_peak, "traffic": CONV_DRAM_BYTES_PER_LAUNCH if world == 1 else None,
                    "note": "int8 ops (2 x MAC) per launch / mean CUDA-event duration of the %d %s launches in one "
                            "instrumented pass; peak = 2 x %s sustained bf16 cuBLAS TFLOP/s (int8 is twice the bf16 rate); "
                            "share of step time %.2f" % (fam[top]["launches"], top, peaks["source"], fam[top]["ms"] / total_ms)}
    else:
        roofline = {"bound": "hbm", "kernel": top, "achieved": None, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": None,
                    "traffic": None}
    line = {"metric": "int8 ResNet-50 images/s", "value": images / dev_s, "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_s / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 (int32 accumulate, fp32 requantise)", "data": "synthetic",
            "config": _config(world),
            "e2e": {"value": images / e2e_s, "unit": "images/s", "h2d_bytes_per_step": host_in.numel(),
                    "d2h_bytes_per_step": host_out.numel(), "ms_per_step": e2e_s / args.steps * 1e3},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline,
            "kernel_families": {k: {"ms_per_step": v["ms"] / args.steps, "launches_per_step": v["launches"] // args.steps,
                                    "share": v["ms"] / total_ms} for k, v in fam.items()},
            "gmac_per_image": info["macs"] / per_gpu / 1e9}
    if world == 1 and not args.no_cpu_baseline:
        try:
            base = cpuref_images_per_s(1, 0)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as e:                                              # the number is reported, never required
            line["cpu_baseline"] = {"value": None, "unit": "images/s", "cores": 0, "kind": "reference",
                                    "sample": "failed: %s" % e}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
