#!/usr/bin/env python
"""Benchmark of the B200Acc hot path.  Headline: int8 ResNet-50 images/s at global batch 256, 224 x 224.

    python bench.py [--gpus N] [--steps K] [--warmup W]            the B200 arm, headline configuration
    python bench.py --impl reference [--steps K] [--warmup W]      the reference's own CpuRef on host cores
    python bench.py --config single_conv|fc_sweep|mobilenet_v2|qlstm   one JSON line for another configuration

One "step" = one pass of the whole ResNet-50 graph (batch 256 in total, sharded by batch rows over the N ranks,
no collective on the data path).  Prints ONE JSON line on rank 0:
  value      images/s with the input batch already resident in HBM: the workload queue replayed as one CUDA graph,
             CUDA events on the network's stream around exactly K steps, barrier + synchronize on both sides, max over
             ranks; the region is repeated `repeats` times and the median region is reported
  e2e        images/s through the Arm NN runtime API with HOST buffers: IRuntime::EnqueueWorkload on the B200Acc
             backend plugin inside the unmodified runtime, pre-imported pinned input / output buffers, every step's H2D
             copy of the image batch and D2H read of the class scores inside the timed region; two LoadedNetworks fed
             by two host threads, so that one network's copies run under the other one's kernels
  roofline   conv2d_q8 (the dominant kernel): int8 ops / CUDA-event time against the int8 tensor peak measured on
             this device by an MMA-only kernel, plus the step's time against its binding roof (per layer
             max(ops / tensor peak, bytes / HBM bandwidth), summed)
  cpu_baseline  the reference's CpuRef timed on this box's host cores on a bounded sample (N = 1 only)
"""
import argparse
import ctypes
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

GLOBAL_BATCH = 256
IMAGE = 224
NOMINAL_INT8_TOPS = 4500.0          # dense int8, per GPU (the doubled vendor figures are with 2:4 sparsity)


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"],
                "bf16_tflops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def _int8_peak():
    """TOP/s of the tcgen05 kind::i8 pipe of the current device, measured by libb200k's MMA-only kernel."""
    from armnn_b200 import lib
    tops = ctypes.c_double(0.0)
    lib.check(lib.load_library().b200k_int8_mma_peak(ctypes.byref(tops), None))
    return tops.value


class ClockSampler:
    """SM clock and throttle reasons sampled through NVML in this process (every 5 ms) while a timed region runs."""

    def __init__(self, index):
        self.index, self.rows, self.stop_flag, self.thread, self.h = index, [], threading.Event(), None, None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_sm = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.h = None

    def _loop(self):
        nv = self.nv
        while not self.stop_flag.is_set():
            try:
                self.rows.append((nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM),
                                  nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                                  if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons")
                                  else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)))
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        if self.h is None:
            return
        self.stop_flag.clear()
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def pause(self):
        if self.thread is not None:
            self.stop_flag.set()
            self.thread.join()
            self.thread = None

    def summary(self):
        if self.h is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"], "samples": 0}
        nv = self.nv
        names = {"hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                 "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                 "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                 "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
        reasons = sorted(n for n, bit in names.items() if any(r & bit for _, r in self.rows))
        sm = [c for c, _ in self.rows]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": self.max_sm, "reasons": reasons,
                "samples": len(sm)}


# ---------------------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's own CpuRef, one single-threaded instance per host core
# ---------------------------------------------------------------------------------------------------------------

def _cpuref_worker(args):
    """Child process: build the batch-1 ResNet-50 graph, load it on CpuRef, run `passes` timed inferences."""
    passes, warm = args
    import numpy as np
    from armnn_b200 import armnn_host, configs
    net, info = configs.resnet50(1, IMAGE)
    x = np.random.default_rng(0).integers(-128, 128, size=info["input_shape"]).astype(np.int8)
    if armnn_host.available():
        runner = armnn_host.ArmnnNetwork(net, "CpuRef")
        kind = "reference"
    else:
        # the plain-C restatement of CpuRef's arithmetic, single-threaded
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import hostnet
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
            "sample": "%d timed step(s) after %d warm-up of 1 image per core (batch-1 ResNet-50 224x224 graph, %d "
                      "single-threaded CpuRef instances in parallel)" % (steps, warmup, cores), "ms_per_step": mean * 1e3}


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

def _dist():
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the B200Acc kernels have no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(local)

    def max_over_ranks(seconds):
        if world == 1:
            return seconds
        t = torch.tensor([seconds], dtype=torch.float64, device=torch.device("cuda", local))
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    return torch, dist, world, rank, local, barrier, max_over_ranks


def _timed_regions(torch, ln, steps, repeats, barrier, max_over_ranks):
    """`repeats` regions of exactly `steps` graph replays each; per region the max over ranks of the CUDA-event time."""
    out, launches = [], 0
    for _ in range(repeats):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ln.stream):
            e0.record()
            for _ in range(steps):
                launches += ln.Execute()
            e1.record()
        barrier()
        out.append(max_over_ranks(e0.elapsed_time(e1) / 1e3))
    return out, launches // repeats


def _layer_pass(torch, network, ln, info, passes):
    """One instrumented eager pass per `passes`: CUDA events around every workload (graph replay cannot be timed per
    kernel).  Returns {layer name: (entry, best ms, macs, bytes)}."""
    meta = {l[0]: l for l in info["layers"]}
    import numpy as np
    width = {"Float32": 4, "Signed32": 4, "QSymmS16": 2}
    best = {}
    for _ in range(passes):
        evs = []
        with torch.cuda.stream(ln.stream):
            for layer, entry, params in ln.workloads:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                network.lib.call(entry, params, ln.stream.cuda_stream)
                b.record()
                evs.append((layer, entry, a, b))
        torch.cuda.synchronize()
        for layer, entry, a, b in evs:
            t = a.elapsed_time(b)
            if layer.name not in best or t < best[layer.name][1]:
                m = meta.get(layer.name)
                macs = m[4] if m else 0
                nbytes = sum(int(np.prod(i.shape)) * width.get(i.dtype.name, 1)
                             for i in [s.source.info for s in layer.inputs] + [o.info for o in layer.outputs])
                best[layer.name] = (entry, t, macs, nbytes)
    return best


def _plugin_e2e(torch, net, info, local, steps, warmup, barrier, max_over_ranks, rank, n_nets=2):
    """End to end through the Arm NN runtime + B200Acc plugin: two LoadedNetworks on this GPU, one host thread each,
    pre-imported pinned buffers; returns (seconds for `steps` requests, bytes in, bytes out, graph kernels per step)."""
    import numpy as np
    from armnn_b200 import armnn_host
    rt = armnn_host.Runtime(device_id=local)
    nets, bufs = [], []
    rng = np.random.default_rng(2000 + rank)
    for i in range(n_nets):
        n = armnn_host.ArmnnNetwork(net, "B200Acc", device_id=local, runtime=rt)
        x = torch.from_numpy(rng.integers(-128, 128, size=info["input_shape"]).astype(np.int8)).pin_memory()
        y = torch.empty(info["output_shape"], dtype=torch.int8).pin_memory()
        nets.append(n)
        bufs.append((x, y))
    errors = []

    def work(i, count):
        n, (x, y) = nets[i], bufs[i]
        for _ in range(count):
            if n.enqueue_ptrs([x.data_ptr()], [y.data_ptr()], preimported=True) != 0:
                errors.append(n.lib.armnnc_last_error().decode())
                return

    def run(total):
        counts = [total // n_nets + (1 if i < total % n_nets else 0) for i in range(n_nets)]
        threads = [threading.Thread(target=work, args=(i, c)) for i, c in enumerate(counts) if c > 0]
        for t in threads:
            t.start()
        for t in threads:
            t.join()

    run(max(n_nets * warmup, 4 * n_nets))         # warm-up: weight packing, graph recording (two warm inferences + one)
    g0 = armnn_host.graph_stats()
    barrier()
    t0 = time.perf_counter()
    run(steps)
    torch.cuda.synchronize(local)
    seconds = max_over_ranks(time.perf_counter() - t0)
    barrier()
    g1 = armnn_host.graph_stats()
    if errors:
        raise RuntimeError("EnqueueWorkload failed: " + errors[0])
    launches, kernels = g1[0] - g0[0], g1[1] - g0[1]
    for n in nets:
        n.close()
    return seconds, bufs[0][0].numel(), bufs[0][1].numel(), launches, kernels


def run_b200(args):
    import numpy as np
    torch, dist, world, rank, local, barrier, max_over_ranks = _dist()
    from armnn_b200 import armnn_host, configs, network
    if world != args.gpus and world == 1 and args.gpus > 1:
        raise SystemExit("--gpus %d needs torchrun with %d ranks" % (args.gpus, args.gpus))
    per_gpu = GLOBAL_BATCH // world
    net, info = configs.resnet50(per_gpu, IMAGE)

    # ---- device-resident throughput (the Python host mirror over the C ABI; one CUDA graph per step) ----
    rt = network.IRuntime.Create(local)
    ln = rt.GetLoadedNetwork(rt.LoadNetwork(network.Optimize(net, ["B200Acc"])))
    rng = np.random.default_rng(1000 + rank)
    host_in = torch.from_numpy(rng.integers(-128, 128, size=info["input_shape"]).astype(np.int8)).pin_memory()
    ln.input_tensor(0).copy_(host_in.cuda(), non_blocking=False)
    ln.Execute()
    torch.cuda.synchronize()
    ln.CaptureGraph()
    for _ in range(args.warmup):
        ln.Execute()
    sampler = ClockSampler(local)
    sampler.start()
    regions, launches = _timed_regions(torch, ln, args.steps, args.repeats, barrier, max_over_ranks)
    sampler.pause()
    dev_s = statistics.median(regions)

    # ---- per-layer times (eager, instrumented) for the roofline ----
    layers = _layer_pass(torch, network, ln, info, 3) if rank == 0 else {}
    int8_peak = _int8_peak() if rank == 0 else 0.0
    del ln, rt
    torch.cuda.empty_cache()

    # ---- the same graph at 256 images per GPU (N > 1): separates the per-GPU batch effect from the number of GPUs ----
    weak = None
    if world > 1:
        wnet, winfo = configs.resnet50(GLOBAL_BATCH, IMAGE)
        wrt = network.IRuntime.Create(local)
        wln = wrt.GetLoadedNetwork(wrt.LoadNetwork(network.Optimize(wnet, ["B200Acc"])))
        wln.input_tensor(0).copy_(torch.from_numpy(rng.integers(-128, 128, size=winfo["input_shape"]).astype(np.int8)).cuda())
        wln.Execute()
        torch.cuda.synchronize(local)
        wln.CaptureGraph()
        for _ in range(args.warmup):
            wln.Execute()
        wregions, _ = _timed_regions(torch, wln, args.steps, max(3, args.repeats // 2), barrier, max_over_ranks)
        wsec = statistics.median(wregions)
        weak = {"value": GLOBAL_BATCH * world * args.steps / wsec, "unit": "images/s", "per_gpu_batch": GLOBAL_BATCH,
                "global_batch": GLOBAL_BATCH * world, "ms_per_step": wsec / args.steps * 1e3,
                "note": "device-resident like `value`, every GPU at the N = 1 batch"}
        del wln, wrt
        torch.cuda.empty_cache()

    # ---- end to end with host buffers ----
    e2e = None
    if args.api == "plugin" and armnn_host.available() and os.path.exists(armnn_host.PLUGIN_PATH):
        sampler.start()
        # every LoadedNetwork has a host thread that spins in its stream synchronisation: with N ranks on one host no more
        # threads than half the cores (8 ranks x 4 threads on 32 cores gave 244 k images/s, 8 x 2 gave 302 k)
        cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 8)
        n_nets = max(1, min(args.e2e_nets, max(2, cores // (2 * world))))
        e2e_s, h2d, d2h, glaunches, gkernels = _plugin_e2e(torch, configs.resnet50(per_gpu, IMAGE)[0], info, local, args.steps,
                                                           args.warmup, barrier, max_over_ranks, rank, n_nets)
        sampler.pause()
        e2e = {"value": GLOBAL_BATCH * args.steps / e2e_s, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": e2e_s / args.steps * 1e3,
               "api": "IRuntime::EnqueueWorkload on the B200Acc plugin inside the unmodified Arm NN runtime, pre-imported "
                      "pinned host buffers, %d LoadedNetworks / host threads per GPU" % n_nets,
               "graph_launches": glaunches, "graph_kernels": gkernels}
    else:
        # the Python mirror's pipelined requests (the Arm NN runtime library is not present on this machine)
        net2, _ = configs.resnet50(per_gpu, IMAGE)
        rt2 = network.IRuntime.Create(local)
        ln2 = rt2.GetLoadedNetwork(rt2.LoadNetwork(network.Optimize(net2, ["B200Acc"])))
        host_out = torch.empty(info["output_shape"], dtype=torch.int8).pin_memory()
        ln2.Execute()
        torch.cuda.synchronize()
        ln2.CapturePipelined()
        for _ in range(min(args.warmup, 3)):
            ln2.WaitOutputs(ln2.EnqueueAsync({0: host_in}), {0: host_out})
        barrier()
        t0 = time.perf_counter()
        prev = None
        for _ in range(args.steps):
            ticket = ln2.EnqueueAsync({0: host_in})
            if prev is not None:
                ln2.WaitOutputs(prev, {0: host_out})
            prev = ticket
        ln2.WaitOutputs(prev, {0: host_out})
        torch.cuda.synchronize()
        e2e_s = max_over_ranks(time.perf_counter() - t0)
        barrier()
        e2e = {"value": GLOBAL_BATCH * args.steps / e2e_s, "unit": "images/s", "h2d_bytes_per_step": host_in.numel(),
               "d2h_bytes_per_step": host_out.numel(), "ms_per_step": e2e_s / args.steps * 1e3,
               "api": "armnn_b200.network.LoadedNetwork.EnqueueAsync / WaitOutputs (Python mirror of the runtime API; the Arm "
                      "NN runtime library or the plugin is not built here)"}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks = _peaks()
    fam, t_roof, t_meas = {}, 0.0, 0.0
    per_layer = []
    for name, (entry, ms, macs, nbytes) in layers.items():
        f = fam.setdefault(entry, {"ms": 0.0, "launches": 0, "macs": 0, "bytes": 0})
        f["ms"] += ms; f["launches"] += 1; f["macs"] += macs; f["bytes"] += nbytes
        roof_ms = max(2.0 * macs / (int8_peak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) * 1e3
        t_roof += roof_ms
        t_meas += ms
        per_layer.append({"layer": name, "kernel": entry, "ms": round(ms, 4), "roof_ms": round(roof_ms, 4),
                          "bound": "tensor" if 2.0 * macs / (int8_peak * 1e12) > nbytes / (peaks["hbm_gbs"] * 1e9) else "hbm"})
    top = max(fam, key=lambda k: fam[k]["ms"])
    total_ms = sum(f["ms"] for f in fam.values())
    achieved = 2.0 * fam[top]["macs"] / (fam[top]["ms"] / 1e3) / 1e12
    step_ms = dev_s / args.steps * 1e3
    roofline = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s",
                "frac": achieved / int8_peak, "traffic": None,
                "peak_source": "measured on this device: MMA-only tcgen05 kind::i8 kernel (b200k_int8_mma_peak)",
                "frac_of_nominal_4500": achieved / NOMINAL_INT8_TOPS,
                "frac_of_2x_measured_bf16_sustained": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                "binding_roof": {"step_roof_ms": t_roof, "layers_measured_ms": t_meas, "graph_step_ms": step_ms,
                                 "frac": t_roof / step_ms,
                                 "note": "per layer max(int8 ops / measured int8 peak, (inputs + weights + outputs) bytes / %s HBM "
                                         "GB/s), summed over the %d workloads; most layers of this network bind on HBM"
                                         % (peaks["source"], len(layers))},
                "note": "int8 ops (2 x MAC) of the %d %s launches / their summed CUDA-event durations in an instrumented eager "
                        "pass right after the timed region (event pairs defeat the programmatic-launch overlap of the graph, "
                        "so the sum of layers exceeds the graph's step time); share of step time %.2f; traffic: see "
                        "profiles/ (ncu), not measured live" % (fam[top]["launches"], top, fam[top]["ms"] / total_ms)}
    line = {"metric": "int8 ResNet-50 images/s", "value": GLOBAL_BATCH * args.steps / dev_s, "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "repeats": args.repeats, "ms_per_step": step_ms,
            "ms_per_step_regions": [round(r / args.steps * 1e3, 4) for r in regions], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "int8 (int32 accumulate, fp32 requantise)", "data": "synthetic",
            "config": _config(world), "e2e": e2e, "weak_scaling": weak, "gpu_launches": launches,
            "clocks": sampler.summary(), "roofline": roofline,
            "kernel_families": {k: {"ms_per_step": v["ms"], "launches_per_step": v["launches"], "share": v["ms"] / total_ms,
                                    "gb_per_s": v["bytes"] / (v["ms"] / 1e3) / 1e9} for k, v in fam.items()},
            "layers": per_layer, "gmac_per_image": info["macs"] / per_gpu / 1e9}
    if world == 1 and not args.no_cpu_baseline:
        try:
            base = cpuref_images_per_s(3, 1)
            line["cpu_baseline"] = {k: base[k] for k in ("value", "unit", "cores", "kind", "sample")}
        except Exception as e:                                              # the number is reported, never required
            line["cpu_baseline"] = {"value": None, "unit": "images/s", "cores": 0, "kind": "reference",
                                    "sample": "failed: %s" % e}
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------------------------
# the other configurations: one JSON line each (N = 1)
# ---------------------------------------------------------------------------------------------------------------

def _graph_ms(torch, ln, steps, repeats):
    """Median over `repeats` regions of `steps` graph replays; ms per replay."""
    ln.Execute()
    torch.cuda.synchronize()
    ln.CaptureGraph()
    for _ in range(5):
        ln.Execute()
    torch.cuda.synchronize()
    out = []
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ln.stream):
            e0.record()
            for _ in range(steps):
                ln.Execute()
            e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1) / steps)
    return statistics.median(out)


def run_config(args):
    import numpy as np
    torch, dist, world, rank, local, barrier, max_over_ranks = _dist()
    if rank != 0:
        return
    from armnn_b200 import configs, network
    peaks = _peaks()
    int8_peak = _int8_peak()
    sampler = ClockSampler(local)

    def load(net):
        rt = network.IRuntime.Create(local)
        ln = rt.GetLoadedNetwork(rt.LoadNetwork(network.Optimize(net, ["B200Acc"])))
        for bid in ln.inputs:
            t = ln.input_tensor(bid)
            lo, hi = (0, 256) if t.dtype == torch.uint8 else ((-2048, 2048) if t.dtype == torch.int16 else (-128, 128))
            t.copy_(torch.from_numpy(np.random.default_rng(7 + bid).integers(lo, hi, size=tuple(t.shape))).to(t.dtype).cuda())
        return ln

    base = {"n_gpus": 1, "steps": args.steps, "warmup": 5, "repeats": args.repeats, "data": "synthetic", "vs_baseline": None,
            "scaling": "weak", "dtype": "int8 (int32 accumulate, fp32 requantise)"}
    sampler.start()
    if args.config == "single_conv":
        net, info = configs.single_conv()
        ms = _graph_ms(torch, load(net), args.steps, args.repeats)
        nbytes = 2 * 56 * 56 * 64 + 64 * 9 * 64
        line = dict(base, metric="single quantized Conv2d latency", value=ms * 1e3, unit="us", higher_is_better=False,
                    ms_per_step=ms, config={"workload": "1x56x56x64 QAsymmS8, 3x3x64x64 per-axis weights, SAME, fused ReLU"},
                    roofline={"bound": "tensor", "achieved": 2 * info["macs"] / (ms * 1e-3) / 1e12, "peak": int8_peak, "unit": "TFLOP/s",
                              "frac": 2 * info["macs"] / (ms * 1e-3) / 1e12 / int8_peak, "traffic": None,
                              "note": "0.23 GOP and %d bytes: 51 ns at the tensor peak; a single launch is latency-bound, the "
                                      "fraction is not meaningful at batch 1" % nbytes})
    elif args.config == "fc_sweep":
        points = []
        for k in (1024, 4096):
            for m in (1, 16, 256, 4096):
                # a chain of layers with their own weights, replayed as one graph: per-layer time without one graph
                # launch per layer, and (K = 4096: 10 x 16.8 MB) every weight from HBM rather than from L2
                depth = max(2, min(64, -(-160 * 1024 * 1024 // (k * k))))
                net, info = configs.fc_stack(m, k, depth)
                ms = _graph_ms(torch, load(net), args.steps, args.repeats) / depth
                info = dict(info, macs=info["macs"] // depth)
                nbytes = m * k + k * k + m * k + 8 * k
                tops, gbs = 2.0 * info["macs"] / (ms * 1e-3) / 1e12, nbytes / (ms * 1e-3) / 1e9
                roof_ms = max(2.0 * info["macs"] / (int8_peak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) * 1e3
                points.append({"m": m, "k": k, "n": k, "us": ms * 1e3, "chain_depth": depth, "weights": "hbm" if depth * k * k > 126e6 else "l2",
                               "tops": tops, "gb_per_s": gbs,
                               "bound": "tensor" if 2.0 * info["macs"] / (int8_peak * 1e12) > nbytes / (peaks["hbm_gbs"] * 1e9) else "hbm",
                               "frac_of_binding_roof": roof_ms / ms})
        big = points[-1]
        line = dict(base, metric="quantized FullyConnected sweep, M=4096 K=N=4096 TOP/s", value=big["tops"], unit="TOP/s",
                    higher_is_better=True, ms_per_step=big["us"] / 1e3,
                    config={"workload": "FullyConnected QAsymmS8 x per-axis QSymmS8, M in {1,16,256,4096}, K=N in {1024,4096}; each point is the "
                                        "per-layer time of a chain of such layers with their own weights (one CUDA graph)"},
                    roofline={"bound": "tensor", "achieved": big["tops"], "peak": int8_peak, "unit": "TFLOP/s",
                              "frac": big["tops"] / int8_peak, "traffic": None, "frac_of_nominal_4500": big["tops"] / NOMINAL_INT8_TOPS},
                    points=points)
    elif args.config == "mobilenet_v2":
        net, info = configs.mobilenet_v2(64, 224)
        ms = _graph_ms(torch, load(net), args.steps, args.repeats)
        line = dict(base, metric="uint8 MobileNet-v2 images/s (batch 64)", value=64 / (ms * 1e-3), unit="images/s",
                    higher_is_better=True, ms_per_step=ms, config={"workload": "MobileNet-v2 1.0 224x224 QAsymmU8, batch 64"},
                    roofline={"bound": "hbm", "achieved": None, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": None, "traffic": None,
                              "note": "per-kernel GB/s: profiles/bandwidth_kernels_mobilenet_resnet_qlstm.md"})
    else:
        net, info = configs.qlstm_stack(batch=128)
        ms = _graph_ms(torch, load(net), args.steps, args.repeats)
        line = dict(base, metric="QLstm stack timesteps/s (3 layers, batch 128)", value=1.0 / (ms * 1e-3), unit="steps/s",
                    higher_is_better=True, ms_per_step=ms,
                    config={"workload": "3 stacked QLstm layers, 40 -> 512 units -> 256, projection + layer norm, batch 128; "
                                        "a 200-step sequence is 200 dependent steps"},
                    sequences_per_s=128 / (200 * ms * 1e-3), gmac_per_s=info["macs"] / (ms * 1e-3) / 1e9,
                    roofline={"bound": "hbm", "achieved": None, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": None, "traffic": None,
                              "note": "dependency / latency-bound: per-MAC re-quantisation chains, 3.1 MB of weights stay on chip"})
    sampler.pause()
    line["clocks"] = sampler.summary()
    line["gpu_launches"] = int(network.lib.load_library().b200k_kernel_launches())
    line["e2e"] = None
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--repeats", type=int, default=11, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--api", default="plugin", choices=["plugin", "mirror"],
                    help="what the end-to-end number goes through: the Arm NN runtime + B200Acc plugin, or the Python mirror")
    ap.add_argument("--config", default="resnet50", choices=["resnet50", "single_conv", "fc_sweep", "mobilenet_v2", "qlstm"])
    ap.add_argument("--e2e-nets", type=int, default=4, help="LoadedNetworks (one host thread each) per GPU in the end-to-end loop")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.impl == "reference":
        # one step = one image per core, ~15 s: keep the arm within minutes
        args.steps, args.warmup = min(args.steps, 3), min(args.warmup, 1)
        run_reference(args)
    elif args.config != "resnet50":
        run_config(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
