"""Device-time micro-benchmarks of single workloads and of whole graphs, layer by layer, through the public API
(INetwork -> Optimize -> IRuntime.LoadNetwork -> LoadedNetwork).  Inputs are seeded random bytes, resident in device
memory; times are CUDA-event durations on the network's stream (best of --reps after 3 warm-up passes); single
workloads are replayed as a CUDA graph so that the host's launch latency stays out of the interval.

    python -m armnn_b200.microbench conv --n 64 --h 56 --w 56 --c 64 --oc 256 --k 1 --relu --add
    python -m armnn_b200.microbench conv --n 32 --h 32 --w 32 --c 8192 --oc 2048 --k 1 --relu      # a large GEMM
    python -m armnn_b200.microbench fc --m 4096 --k 4096 --n 4096
    python -m armnn_b200.microbench fc-sweep
    python -m armnn_b200.microbench layers --net resnet50 --batch 256
    python -m armnn_b200.microbench layers --net mobilenet_v2 --batch 64
    python -m armnn_b200.microbench qlstm --batch 128 --steps 200
"""
import argparse
import sys

import numpy as np


def _fill_inputs(ln, torch, seed=1000):
    rng = np.random.default_rng(seed)
    for bid in ln.inputs:
        t = ln.input_tensor(bid)
        if t.dtype == torch.int16:
            host = rng.integers(-2048, 2048, size=tuple(t.shape)).astype(np.int16)
        elif t.dtype == torch.uint8:
            host = rng.integers(0, 256, size=tuple(t.shape)).astype(np.uint8)
        else:
            host = rng.integers(-128, 128, size=tuple(t.shape)).astype(np.int8)
        t.copy_(torch.from_numpy(host).cuda())


def _load(net, graph=False):
    """graph: replay the workload queue as one CUDA graph, which takes the host's launch latency (tens of
    microseconds per workload from Python) out of the measured interval."""
    import torch
    from armnn_b200 import network
    rt = network.IRuntime.Create(0)
    ln = rt.GetLoadedNetwork(rt.LoadNetwork(network.Optimize(net)))
    _fill_inputs(ln, torch)
    if graph:
        ln.Execute()
        torch.cuda.synchronize()
        ln.CaptureGraph()
    return ln, torch


def _time_whole(ln, torch, reps, inner=1):
    """Best of `reps` intervals of `inner` back-to-back passes each (per pass).  Several passes per interval keep the
    launch latency of the first one from dominating a short workload."""
    for _ in range(3):
        ln.Execute()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ln.stream):
            e0.record()
            for _ in range(inner):
                ln.Execute()
            e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / inner)
    return best


def _time_layers(ln, torch, reps):
    from armnn_b200 import network
    for _ in range(3):
        ln.Execute()
    torch.cuda.synchronize()
    acc = {}
    for _ in range(reps):
        evs = []
        with torch.cuda.stream(ln.stream):
            for layer, entry, params in ln.workloads:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                network.lib.call(entry, params, ln.stream.cuda_stream)
                b.record()
                evs.append((layer.name, entry, a, b))
        torch.cuda.synchronize()
        for name, entry, a, b in evs:
            t = a.elapsed_time(b)
            if name not in acc or t < acc[name][1]:
                acc[name] = (entry, t)
    return acc


def conv_graph(n, h, w, c, oc, k, stride=1, relu=False, add=False, seed="microbench_conv"):
    """One Convolution2d (SAME padding, per-channel QSymmS8 weights, int32 bias) with optional ReLU and an optional
    residual Add (+ ReLU) whose other operand is a second network input; Optimize fuses all of it into the
    convolution workload."""
    from armnn_b200 import configs
    from armnn_b200.network import DataType, TensorInfo
    b = configs._S8Builder(seed)
    x, rms = b.input((n, h, w, c), 0.02, -3)
    y, rms_y = b.conv(x, rms, oc, k, stride, relu and not add, 1.0, "conv")
    if add:
        il = b.net.AddInputLayer(1, "other")
        info = TensorInfo(y.info.shape, DataType.QAsymmS8, y.info.scale, -128)
        il.GetOutputSlot(0).SetTensorInfo(info)
        y, _ = b.add_relu(y, rms_y, il.GetOutputSlot(0), rms_y, "add")
    ol = b.net.AddOutputLayer(0, "output")
    y.Connect(ol.GetInputSlot(0))
    return b.net, b.macs


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    c = sub.add_parser("conv")
    for name, default in (("n", 64), ("h", 56), ("w", 56), ("c", 64), ("oc", 256), ("k", 1), ("stride", 1)):
        c.add_argument("--" + name, type=int, default=default)
    c.add_argument("--relu", action="store_true")
    c.add_argument("--add", action="store_true")
    f = sub.add_parser("fc")
    for name, default in (("m", 4096), ("k", 4096), ("n", 4096)):
        f.add_argument("--" + name, type=int, default=default)
    sub.add_parser("fc-sweep")
    l = sub.add_parser("layers")
    l.add_argument("--net", choices=("resnet50", "mobilenet_v2"), default="resnet50")
    l.add_argument("--batch", type=int, default=256)
    q = sub.add_parser("qlstm")
    q.add_argument("--batch", type=int, default=128)
    q.add_argument("--steps", type=int, default=200)
    for p in (c, f, l, q):
        p.add_argument("--reps", type=int, default=5)
    args = ap.parse_args(argv)
    from armnn_b200 import configs

    if args.cmd == "conv":
        net, macs = conv_graph(args.n, args.h, args.w, args.c, args.oc, args.k, args.stride, args.relu, args.add)
        ln, torch = _load(net, graph=True)
        ms = _time_whole(ln, torch, args.reps, inner=10)
        out = ln.output_tensor(0)
        nbytes = args.n * args.h * args.w * args.c + out.numel() * (2 if args.add else 1)
        print("conv %dx%d/%d  [%d,%d,%d,%d] -> %s%s  %.4f ms  %.1f TOP/s  %.0f GB/s (tensors once)" % (
            args.k, args.k, args.stride, args.n, args.h, args.w, args.c, tuple(out.shape), " +add" if args.add else "",
            ms, 2.0 * macs / ms / 1e9, nbytes / ms / 1e6))
    elif args.cmd in ("fc", "fc-sweep"):
        cases = [(args.m, args.k, args.n)] if args.cmd == "fc" else [(m, k, k) for k in (1024, 4096) for m in (1, 16, 256, 4096)]
        for m, k, n in cases:
            net, info = configs.fc_sweep_case(m, k, n)
            ln, torch = _load(net, graph=True)
            ms = _time_whole(ln, torch, getattr(args, "reps", 5), inner=10)
            nbytes = m * k + n * k + m * n
            print("fc  M=%-5d K=%-5d N=%-5d  %.4f ms  %8.1f TOP/s  %7.0f GB/s" % (m, k, n, ms, 2.0 * info["macs"] / ms / 1e9, nbytes / ms / 1e6))
            if k == n:
                # a chain of layers with their own weights in one graph: per-layer time without the launch of a graph per
                # layer, and (K = 4096: 10 x 16.8 MB) with every weight read from HBM
                depth = max(2, min(64, -(-160 * 1024 * 1024 // (k * k))))
                net, info = configs.fc_stack(m, k, depth)
                ln, torch = _load(net, graph=True)
                ms = _time_whole(ln, torch, getattr(args, "reps", 5), inner=10) / depth
                print("    chain of %2d: %.4f ms per layer  %8.1f TOP/s  %7.0f GB/s (weights %s)" % (
                    depth, ms, 2.0 * m * k * k / ms / 1e9, nbytes / ms / 1e6, "from HBM" if depth * k * k > 126e6 else "L2-resident"))
    elif args.cmd == "layers":
        net, info = (configs.resnet50 if args.net == "resnet50" else configs.mobilenet_v2)(args.batch, 224)
        ln, torch = _load(net)
        acc = _time_layers(ln, torch, args.reps)
        meta = {l[0]: l for l in info["layers"]}
        total = 0.0
        print("%-22s %-12s %-22s %-22s %8s %8s %8s" % ("layer", "kind", "in", "out", "ms", "TOP/s", "GB/s"))
        for layer, entry, params in ln.workloads:
            entry, t = acc[layer.name]
            total += t
            l = meta.get(layer.name)
            if l:
                inb, outb = int(np.prod(l[2])), int(np.prod(l[3]))
                print("%-22s %-12s %-22s %-22s %8.3f %8.1f %8.0f" % (layer.name, l[1], l[2], l[3], t, 2 * l[4] / t / 1e9 if l[4] else 0.0, (inb + outb) / t / 1e6))
            else:
                print("%-22s %-12s %-22s %-22s %8.3f" % (layer.name, entry, "", "", t))
        eager = _time_whole(ln, torch, args.reps)
        ln.CaptureGraph()
        print("sum of layers %.3f ms; whole queue back to back %.3f ms eager, %.3f ms as one CUDA graph" % (
            total, eager, _time_whole(ln, torch, args.reps)))
    elif args.cmd == "qlstm":
        net, info = configs.qlstm_stack(batch=args.batch)
        ln, torch = _load(net)
        ms = _time_whole(ln, torch, args.reps)
        ln.CaptureGraph()
        for _ in range(3):
            ln.Execute()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(ln.stream):
            e0.record()
            for _ in range(args.steps):
                ln.Execute()
            e1.record()
        torch.cuda.synchronize()
        seq = e0.elapsed_time(e1)
        print("qlstm stack  batch %d: one timestep (3 layers) %.4f ms; %d timesteps as graph replays %.3f ms (%.1f us/step, %.0f sequences/s)" % (
            args.batch, ms, args.steps, seq, seq / args.steps * 1e3, args.batch / (seq / 1e3)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
