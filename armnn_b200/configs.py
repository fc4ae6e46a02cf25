"""The benchmark configurations as seeded synthetic graphs built through the INetwork mirror.

There are no model files or datasets behind these: every graph is random-init, with one
numpy Generator per graph seeded from the config name, and the SAME bytes are fed to the reference
oracle and to the B200 kernels.  Quantisation scales are derived from the expected second moment of each
tensor (He-style weight variance), so that only a small fraction of outputs sits on a clamp and parity
checks are not vacuous.

  resnet50(batch, image)      ResNet-50 topology, QAsymmS8 activations, per-channel QSymmS8 weights
  mobilenet_v2(batch, image)  MobileNet-v2 1.0, all QAsymmU8, per-tensor uint8 weights with zero points
  single_conv()               1x56x56x64 3x3 conv + ReLU, the single-layer case
  fc_sweep_case(m, k)         FullyConnected M x K x K
  qlstm_stack(batch)          3 stacked QLstm layers (projection + layer norm), one timestep per run
"""
import zlib

import numpy as np

from .network import (ActivationFunction, BinaryOperation, DataType, INetwork, PaddingMethod, PoolingAlgorithm,
                      TensorInfo)

W_STD_S8 = 73.3      # std of uniform integers in [-127, 127]
W_STD_U8 = 73.9      # std of uniform integers in [0, 255]


def _rng(name):
    return np.random.default_rng(zlib.crc32(name.encode()))


def _f32(v):
    return float(np.float32(v))


def _out_hw(i, k, s, pb, pa, d=1):
    return (i + pb + pa - (d * (k - 1) + 1)) // s + 1


def same_pad(i, k, s):
    o = (i + s - 1) // s
    total = max((o - 1) * s + k - i, 0)
    return total // 2, total - total // 2


class _S8Builder:
    """Helper for QAsymmS8 CNN graphs; tracks the expected rms of every tensor."""

    def __init__(self, name):
        self.net = INetwork.Create()
        self.rng = _rng(name)
        self.macs = 0
        self.layer_list = []

    def input(self, shape, scale, zp):
        l = self.net.AddInputLayer(0, "input")
        info = TensorInfo(shape, DataType.QAsymmS8, scale, zp)
        l.GetOutputSlot(0).SetTensorInfo(info)
        return l.GetOutputSlot(0), 74.0 * scale

    def conv(self, x, rms_in, oc, k, stride, relu, gain, name):
        n, h, w, c = x.info.shape
        pt, pb = same_pad(h, k, stride)
        pl, pr = same_pad(w, k, stride)
        oh, ow = _out_hw(h, k, stride, pt, pb), _out_hw(w, k, stride, pl, pr)
        K = k * k * c
        # real weight std so that Var(pre-activation) = gain * E[x^2]
        sw_real = np.sqrt(gain / K)
        w_scales = (sw_real / W_STD_S8 * self.rng.uniform(0.7, 1.3, size=oc)).astype(np.float32)
        wq = self.rng.integers(-127, 128, size=(oc, k, k, c)).astype(np.int8)
        bq = self.rng.integers(-1000, 1001, size=oc).astype(np.int32)
        b_scales = (np.float32(x.info.scale) * w_scales).astype(np.float32)
        pre_std = rms_in * np.sqrt(gain)
        if relu:
            rms_out = pre_std / np.sqrt(2.0)
            y_info = TensorInfo((n, oh, ow, oc), DataType.QAsymmS8, _f32(4.0 * rms_out / 255.0), -128)
        else:
            rms_out = pre_std
            y_info = TensorInfo((n, oh, ow, oc), DataType.QAsymmS8, _f32(3.5 * rms_out / 127.0), 0)
        wl = self.net.AddConstantLayer(wq, TensorInfo(wq.shape, DataType.QSymmS8, scales=w_scales, quant_dim=0), name + "/w")
        bl = self.net.AddConstantLayer(bq, TensorInfo(bq.shape, DataType.Signed32, scales=b_scales, quant_dim=0), name + "/b")
        cl = self.net.AddConvolution2dLayer((stride, stride), (pt, pb, pl, pr), (1, 1), True, name)
        x.Connect(cl.GetInputSlot(0))
        wl.GetOutputSlot(0).Connect(cl.GetInputSlot(1))
        bl.GetOutputSlot(0).Connect(cl.GetInputSlot(2))
        cl.GetOutputSlot(0).SetTensorInfo(y_info)
        out = cl.GetOutputSlot(0)
        self.macs += n * oh * ow * oc * K
        self.layer_list.append((name, "conv%dx%d/%d" % (k, k, stride), (n, h, w, c), (n, oh, ow, oc), n * oh * ow * oc * K))
        if relu:
            al = self.net.AddActivationLayer(ActivationFunction.ReLu, name=name + "/relu")
            out.Connect(al.GetInputSlot(0))
            al.GetOutputSlot(0).SetTensorInfo(y_info)
            out = al.GetOutputSlot(0)
        return out, rms_out

    def add_relu(self, a, rms_a, b, rms_b, name):
        rms_pre = np.sqrt(rms_a ** 2 + rms_b ** 2)
        rms_out = rms_pre * 0.8
        info = TensorInfo(a.info.shape, DataType.QAsymmS8, _f32(4.0 * rms_out / 255.0), -128)
        l = self.net.AddElementwiseBinaryLayer(BinaryOperation.Add, name)
        a.Connect(l.GetInputSlot(0))
        b.Connect(l.GetInputSlot(1))
        l.GetOutputSlot(0).SetTensorInfo(info)
        al = self.net.AddActivationLayer(ActivationFunction.ReLu, name=name + "/relu")
        l.GetOutputSlot(0).Connect(al.GetInputSlot(0))
        al.GetOutputSlot(0).SetTensorInfo(info)
        self.layer_list.append((name, "add+relu", a.info.shape, a.info.shape, 0))
        return al.GetOutputSlot(0), rms_out

    def pool(self, x, ptype, k, stride, pad, name, scale_mul=1.0):
        n, h, w, c = x.info.shape
        oh, ow = _out_hw(h, k, stride, pad[0], pad[1]), _out_hw(w, k, stride, pad[2], pad[3])
        info = TensorInfo((n, oh, ow, c), x.info.dtype, _f32(x.info.scale * scale_mul), x.info.offset)
        l = self.net.AddPooling2dLayer(ptype, (k, k), (stride, stride), pad, PaddingMethod.Exclude, name)
        x.Connect(l.GetInputSlot(0))
        l.GetOutputSlot(0).SetTensorInfo(info)
        self.layer_list.append((name, "pool%d/%d" % (k, stride), x.info.shape, info.shape, 0))
        return l.GetOutputSlot(0)

    def fc_softmax(self, x, rms_in, n_out, name):
        n = x.info.shape[0]
        k = int(np.prod(x.info.shape[1:]))
        rl = self.net.AddReshapeLayer((n, k), name + "/flatten")
        x.Connect(rl.GetInputSlot(0))
        rl.GetOutputSlot(0).SetTensorInfo(TensorInfo((n, k), x.info.dtype, x.info.scale, x.info.offset))
        sw = _f32(np.sqrt(4.0 / k) / rms_in / W_STD_S8)        # logits with std ~ 2
        wq = self.rng.integers(-127, 128, size=(n_out, k)).astype(np.int8)
        bq = self.rng.integers(-1000, 1001, size=n_out).astype(np.int32)
        # per-tensor QAsymmS8 weights with zero point 0: the combination CpuRef's own layer-support accepts
        wl = self.net.AddConstantLayer(wq, TensorInfo(wq.shape, DataType.QAsymmS8, sw, 0), name + "/w")
        bl = self.net.AddConstantLayer(bq, TensorInfo(bq.shape, DataType.Signed32, _f32(np.float32(x.info.scale) * np.float32(sw)), 0), name + "/b")
        fl = self.net.AddFullyConnectedLayer(True, True, name)
        rl.GetOutputSlot(0).Connect(fl.GetInputSlot(0))
        wl.GetOutputSlot(0).Connect(fl.GetInputSlot(1))
        bl.GetOutputSlot(0).Connect(fl.GetInputSlot(2))
        fl.GetOutputSlot(0).SetTensorInfo(TensorInfo((n, n_out), DataType.QAsymmS8, _f32(8.0 / 127.0), 0))
        self.macs += n * k * n_out
        self.layer_list.append((name, "fc", (n, k), (n, n_out), n * k * n_out))
        sl = self.net.AddSoftmaxLayer(1.0, -1, name + "/softmax")
        fl.GetOutputSlot(0).Connect(sl.GetInputSlot(0))
        sl.GetOutputSlot(0).SetTensorInfo(TensorInfo((n, n_out), DataType.QAsymmS8, 1.0 / 256.0, -128))
        return sl.GetOutputSlot(0)


def resnet50(batch=256, image=224, classes=1001):
    """ResNet-50: 7x7/2 stem (+ReLU), 3x3/2 max pool, bottleneck stages [3,4,6,3] with output widths
    256/512/1024/2048 (1x1 reduce + ReLU, 3x3 + ReLU carrying the stride, 1x1 expand; projection shortcut in
    the first block of each stage), residual Add + ReLU, global average pool, FC, Softmax.  BatchNorm is
    folded (random-init weights).  Returns (network, info dict with the layer list and the exact MAC count)."""
    b = _S8Builder("resnet50")
    x, rms = b.input((batch, image, image, 3), 0.02, -3)
    x, rms = b.conv(x, rms, 64, 7, 2, True, 2.0, "stem")
    x = b.pool(x, PoolingAlgorithm.Max, 3, 2, (1, 1, 1, 1), "pool1")
    rms *= 1.7
    x_info = x.info
    # the max pool keeps its input's quantisation; widen it through the next convs' expectations only
    widths = (64, 128, 256, 512)
    blocks = (3, 4, 6, 3)
    for s, (wd, nb) in enumerate(zip(widths, blocks)):
        for i in range(nb):
            stride = 2 if (i == 0 and s > 0) else 1
            name = "s%d/b%d" % (s + 1, i + 1)
            y, r = b.conv(x, rms, wd, 1, 1, True, 2.0, name + "/reduce")
            y, r = b.conv(y, r, wd, 3, stride, True, 2.0, name + "/conv3")
            y, r = b.conv(y, r, wd * 4, 1, 1, False, 0.5, name + "/expand")
            if i == 0:
                sc, rs = b.conv(x, rms, wd * 4, 1, stride, False, 1.0, name + "/shortcut")
            else:
                sc, rs = x, rms
            x, rms = b.add_relu(y, r, sc, rs, name + "/add")
    n, h, w, c = x.info.shape
    x = b.pool(x, PoolingAlgorithm.Average, h, 1, (0, 0, 0, 0), "avgpool", scale_mul=0.8)
    rms *= 0.75
    out = b.fc_softmax(x, rms, classes, "fc")
    ol = b.net.AddOutputLayer(0, "output")
    out.Connect(ol.GetInputSlot(0))
    del x_info
    return b.net, {"macs": b.macs, "layers": b.layer_list, "batch": batch, "image": image,
                   "input_shape": (batch, image, image, 3), "output_shape": (batch, classes)}


class _U8Builder:
    """QAsymmU8 graphs with per-tensor uint8 weights carrying a zero point (MobileNet-v2 style)."""

    def __init__(self, name):
        self.net = INetwork.Create()
        self.rng = _rng(name)
        self.macs = 0
        self.layer_list = []

    def _scale(self):
        return _f32(self.rng.uniform(0.005, 0.05))

    def input(self, shape):
        l = self.net.AddInputLayer(0, "input")
        s = self._scale()
        l.GetOutputSlot(0).SetTensorInfo(TensorInfo(shape, DataType.QAsymmU8, s, 128))
        return l.GetOutputSlot(0), 74.0 * s

    def conv(self, x, rms_in, oc, k, stride, relu6, name, depthwise=False):
        n, h, w, c = x.info.shape
        pt, pb = same_pad(h, k, stride)
        pl, pr = same_pad(w, k, stride)
        oh, ow = _out_hw(h, k, stride, pt, pb), _out_hw(w, k, stride, pl, pr)
        K = k * k * (1 if depthwise else c)
        s_out = self._scale()
        if relu6:
            zp_out, target = 0, 2.0                                   # pre-activation std ~ 2 inside [0, 6]
            rms_out = 1.6
        else:
            zp_out = int(self.rng.integers(96, 161))
            target = 40.0 * s_out                                     # +-3 sigma ~ +-120 LSB
            rms_out = target
        sw = _f32(target / (rms_in * np.sqrt(K)) / W_STD_U8)
        zw = int(self.rng.integers(100, 156))
        if depthwise:
            oc = c
            wq = self.rng.integers(0, 256, size=(1, k, k, oc)).astype(np.uint8)
        else:
            wq = self.rng.integers(0, 256, size=(oc, k, k, c)).astype(np.uint8)
        bq = self.rng.integers(-1000, 1001, size=oc).astype(np.int32)
        y_info = TensorInfo((n, oh, ow, oc), DataType.QAsymmU8, s_out, zp_out)
        wl = self.net.AddConstantLayer(wq, TensorInfo(wq.shape, DataType.QAsymmU8, sw, zw), name + "/w")
        bl = self.net.AddConstantLayer(bq, TensorInfo(bq.shape, DataType.Signed32, _f32(np.float32(x.info.scale) * np.float32(sw)), 0), name + "/b")
        if depthwise:
            cl = self.net.AddDepthwiseConvolution2dLayer((stride, stride), (pt, pb, pl, pr), (1, 1), True, name)
        else:
            cl = self.net.AddConvolution2dLayer((stride, stride), (pt, pb, pl, pr), (1, 1), True, name)
        x.Connect(cl.GetInputSlot(0))
        wl.GetOutputSlot(0).Connect(cl.GetInputSlot(1))
        bl.GetOutputSlot(0).Connect(cl.GetInputSlot(2))
        cl.GetOutputSlot(0).SetTensorInfo(y_info)
        out = cl.GetOutputSlot(0)
        macs = n * oh * ow * oc * K
        self.macs += macs
        self.layer_list.append((name, ("dw" if depthwise else "conv") + "%dx%d/%d" % (k, k, stride), (n, h, w, c), (n, oh, ow, oc), macs))
        if relu6:
            al = self.net.AddActivationLayer(ActivationFunction.BoundedReLu, 6.0, 0.0, name + "/relu6")
            out.Connect(al.GetInputSlot(0))
            al.GetOutputSlot(0).SetTensorInfo(y_info)
            out = al.GetOutputSlot(0)
        return out, rms_out


def mobilenet_v2(batch=64, image=224, classes=1001):
    """MobileNet-v2 1.0: stem 3x3/2 -> 32, seventeen inverted-residual blocks
    (expansion, out, repeats, stride) = (1,16,1,1),(6,24,2,2),(6,32,3,2),(6,64,4,2),(6,96,3,1),(6,160,3,2),(6,320,1,1),
    1x1 -> 1280, global average pool, FC, Softmax; all QAsymmU8."""
    b = _U8Builder("mobilenet_v2")
    x, rms = b.input((batch, image, image, 3))
    x, rms = b.conv(x, rms, 32, 3, 2, True, "stem")
    cfg = ((1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1))
    blk = 0
    for t, oc, reps, stride in cfg:
        for i in range(reps):
            blk += 1
            name = "block%d" % blk
            s = stride if i == 0 else 1
            cin = x.info.shape[3]
            y, r = x, rms
            if t != 1:
                y, r = b.conv(y, r, cin * t, 1, 1, True, name + "/expand")
            y, r = b.conv(y, r, None, 3, s, True, name + "/dw", depthwise=True)
            y, r = b.conv(y, r, oc, 1, 1, False, name + "/project")
            if s == 1 and cin == oc:
                s_out = b._scale()
                info = TensorInfo(y.info.shape, DataType.QAsymmU8, s_out, int(b.rng.integers(96, 161)))
                al = b.net.AddElementwiseBinaryLayer(BinaryOperation.Add, name + "/add")
                x.Connect(al.GetInputSlot(0))
                y.Connect(al.GetInputSlot(1))
                al.GetOutputSlot(0).SetTensorInfo(info)
                b.layer_list.append((name + "/add", "add", y.info.shape, y.info.shape, 0))
                y, r = al.GetOutputSlot(0), float(np.sqrt(rms ** 2 + r ** 2))
            x, rms = y, r
    x, rms = b.conv(x, rms, 1280, 1, 1, True, "head")
    n, h, w, c = x.info.shape
    pl = b.net.AddPooling2dLayer(PoolingAlgorithm.Average, (h, w), (1, 1), (0, 0, 0, 0), PaddingMethod.Exclude, "avgpool")
    x.Connect(pl.GetInputSlot(0))
    pl.GetOutputSlot(0).SetTensorInfo(TensorInfo((n, 1, 1, c), DataType.QAsymmU8, x.info.scale, x.info.offset))
    rl = b.net.AddReshapeLayer((n, c), "flatten")
    pl.GetOutputSlot(0).Connect(rl.GetInputSlot(0))
    rl.GetOutputSlot(0).SetTensorInfo(TensorInfo((n, c), DataType.QAsymmU8, x.info.scale, x.info.offset))
    sw = _f32(2.0 / (1.2 * np.sqrt(c)) / W_STD_U8)
    wq = b.rng.integers(0, 256, size=(classes, c)).astype(np.uint8)
    bq = b.rng.integers(-1000, 1001, size=classes).astype(np.int32)
    wl = b.net.AddConstantLayer(wq, TensorInfo(wq.shape, DataType.QAsymmU8, sw, 128), "fc/w")
    bl = b.net.AddConstantLayer(bq, TensorInfo(bq.shape, DataType.Signed32, _f32(np.float32(x.info.scale) * np.float32(sw)), 0), "fc/b")
    fl = b.net.AddFullyConnectedLayer(True, True, "fc")
    rl.GetOutputSlot(0).Connect(fl.GetInputSlot(0))
    wl.GetOutputSlot(0).Connect(fl.GetInputSlot(1))
    bl.GetOutputSlot(0).Connect(fl.GetInputSlot(2))
    fl.GetOutputSlot(0).SetTensorInfo(TensorInfo((n, classes), DataType.QAsymmU8, _f32(8.0 / 127.0), 128))
    b.macs += n * c * classes
    b.layer_list.append(("fc", "fc", (n, c), (n, classes), n * c * classes))
    sl = b.net.AddSoftmaxLayer(1.0, -1, "softmax")
    fl.GetOutputSlot(0).Connect(sl.GetInputSlot(0))
    sl.GetOutputSlot(0).SetTensorInfo(TensorInfo((n, classes), DataType.QAsymmU8, 1.0 / 256.0, 0))   # Network.cpp:821-835
    ol = b.net.AddOutputLayer(0, "output")
    sl.GetOutputSlot(0).Connect(ol.GetInputSlot(0))
    return b.net, {"macs": b.macs, "layers": b.layer_list, "batch": batch, "image": image,
                   "input_shape": (batch, image, image, 3), "output_shape": (batch, classes)}


def single_conv(output_scale=0.05, output_zp=-128, seed_name="single_conv"):
    """NHWC 1x56x56x64 QAsymmS8 (0.02, -3); weights 64x3x3x64 QSymmS8 per-channel scales in [0.001, 0.01];
    int32 bias in [-1000, 1000]; stride 1, SAME padding; ReLU as a separate Activation layer;
    output QAsymmS8 (0.05, -128)."""
    rng = _rng(seed_name)
    net = INetwork.Create()
    il = net.AddInputLayer(0, "input")
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo((1, 56, 56, 64), DataType.QAsymmS8, 0.02, -3))
    w_scales = rng.uniform(0.001, 0.01, size=64).astype(np.float32)
    wq = rng.integers(-127, 128, size=(64, 3, 3, 64)).astype(np.int8)
    bq = rng.integers(-1000, 1001, size=64).astype(np.int32)
    wl = net.AddConstantLayer(wq, TensorInfo(wq.shape, DataType.QSymmS8, scales=w_scales, quant_dim=0), "w")
    bl = net.AddConstantLayer(bq, TensorInfo(bq.shape, DataType.Signed32, scales=(np.float32(0.02) * w_scales), quant_dim=0), "b")
    cl = net.AddConvolution2dLayer((1, 1), (1, 1, 1, 1), (1, 1), True, "conv")
    il.GetOutputSlot(0).Connect(cl.GetInputSlot(0))
    wl.GetOutputSlot(0).Connect(cl.GetInputSlot(1))
    bl.GetOutputSlot(0).Connect(cl.GetInputSlot(2))
    y_info = TensorInfo((1, 56, 56, 64), DataType.QAsymmS8, output_scale, output_zp)
    cl.GetOutputSlot(0).SetTensorInfo(y_info)
    al = net.AddActivationLayer(ActivationFunction.ReLu, name="relu")
    cl.GetOutputSlot(0).Connect(al.GetInputSlot(0))
    al.GetOutputSlot(0).SetTensorInfo(y_info)
    ol = net.AddOutputLayer(0, "output")
    al.GetOutputSlot(0).Connect(ol.GetInputSlot(0))
    return net, {"macs": 56 * 56 * 64 * 9 * 64, "input_shape": (1, 56, 56, 64), "output_shape": (1, 56, 56, 64)}


def fc_sweep_case(m, k, n=None, seed_name=None):
    """FullyConnected, activations QAsymmS8 (0.03, 5), weights [N, K] QSymmS8 per-output-channel scales in
    [0.001, 0.01], int32 bias, output QAsymmS8 with a scale that keeps saturation low."""
    n = n or k
    rng = _rng(seed_name or "fc_%d_%d_%d" % (m, k, n))
    net = INetwork.Create()
    il = net.AddInputLayer(0, "input")
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo((m, k), DataType.QAsymmS8, 0.03, 5))
    w_scales = rng.uniform(0.001, 0.01, size=n).astype(np.float32)
    wq = rng.integers(-127, 128, size=(n, k)).astype(np.int8)
    bq = rng.integers(-1000, 1001, size=n).astype(np.int32)
    wl = net.AddConstantLayer(wq, TensorInfo(wq.shape, DataType.QSymmS8, scales=w_scales, quant_dim=0), "w")
    bl = net.AddConstantLayer(bq, TensorInfo(bq.shape, DataType.Signed32, scales=(np.float32(0.03) * w_scales), quant_dim=0), "b")
    fl = net.AddFullyConnectedLayer(True, True, "fc")
    il.GetOutputSlot(0).Connect(fl.GetInputSlot(0))
    wl.GetOutputSlot(0).Connect(fl.GetInputSlot(1))
    bl.GetOutputSlot(0).Connect(fl.GetInputSlot(2))
    std = 0.03 * 0.0055 * 74.0 * 73.3 * np.sqrt(k)
    fl.GetOutputSlot(0).SetTensorInfo(TensorInfo((m, n), DataType.QAsymmS8, _f32(std * 4.0 / 127.0), 0))
    ol = net.AddOutputLayer(0, "output")
    fl.GetOutputSlot(0).Connect(ol.GetInputSlot(0))
    return net, {"macs": m * k * n, "input_shape": (m, k), "output_shape": (m, n)}


def fc_stack(m, k, depth, seed_name=None):
    """`depth` FullyConnected layers K -> K in a chain, each with its own weights (the quantisation of fc_sweep_case,
    every output feeding the next layer at scale 0.03, offset 5): with depth * K * K bytes above the L2 capacity a
    replay reads every weight from HBM, and the per-launch cost is spread over the chain."""
    rng = _rng(seed_name or "fc_stack_%d_%d_%d" % (m, k, depth))
    net = INetwork.Create()
    il = net.AddInputLayer(0, "input")
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo((m, k), DataType.QAsymmS8, 0.03, 5))
    cur = il.GetOutputSlot(0)
    for d in range(depth):
        w_scales = rng.uniform(0.001, 0.01, size=k).astype(np.float32)
        wq = rng.integers(-127, 128, size=(k, k)).astype(np.int8)
        bq = rng.integers(-1000, 1001, size=k).astype(np.int32)
        wl = net.AddConstantLayer(wq, TensorInfo(wq.shape, DataType.QSymmS8, scales=w_scales, quant_dim=0), "w%d" % d)
        bl = net.AddConstantLayer(bq, TensorInfo(bq.shape, DataType.Signed32, scales=(np.float32(0.03) * w_scales), quant_dim=0), "b%d" % d)
        fl = net.AddFullyConnectedLayer(True, True, "fc%d" % d)
        cur.Connect(fl.GetInputSlot(0))
        wl.GetOutputSlot(0).Connect(fl.GetInputSlot(1))
        bl.GetOutputSlot(0).Connect(fl.GetInputSlot(2))
        # the next layer reads this output as (0.03, 5) whatever its real spread: only the traffic matters here
        fl.GetOutputSlot(0).SetTensorInfo(TensorInfo((m, k), DataType.QAsymmS8, 0.03, 5))
        cur = fl.GetOutputSlot(0)
    ol = net.AddOutputLayer(0, "output")
    cur.Connect(ol.GetInputSlot(0))
    return net, {"macs": depth * m * k * k, "input_shape": (m, k), "output_shape": (m, k), "depth": depth}


QLSTM_SCALES = dict(input=2.0 ** -7, hidden=0.007, cell=2.0 ** -15, weights=0.00784314, layer_norm=3.05182e-05,
                    intermediate_i=0.007059, intermediate_f=0.007812, projection=0.00392157)


def qlstm_stack(batch=128, input_size=40, num_units=512, output_size=256, layers=3):
    """`layers` stacked QLstm cells (projection + layer norm, no CIFG / peephole), one timestep per
    EnqueueWorkload with the states fed back by the caller.  Quantisation parameters are those of the
    reference's projection + layer-norm QLstm layer test; every layer's output scale is the next layer's
    input scale (2^-7).  Bindings: input 0 = x [batch, input_size]; inputs 1+2l / 2+2l = outputStateIn /
    cellStateIn of layer l; outputs 0 = top layer output, 1+2l / 2+2l = outputStateOut / cellStateOut."""
    rng = _rng("qlstm_stack")
    q = QLSTM_SCALES
    net = INetwork.Create()
    il = net.AddInputLayer(0, "x")
    il.GetOutputSlot(0).SetTensorInfo(TensorInfo((batch, input_size), DataType.QAsymmS8, q["input"], 0))
    x = il.GetOutputSlot(0)
    macs = 0
    for l in range(layers):
        isz = input_size if l == 0 else output_size
        h_info = TensorInfo((batch, output_size), DataType.QAsymmS8, q["input"], 0)
        c_info = TensorInfo((batch, num_units), DataType.QSymmS16, q["cell"], 0)
        hl = net.AddInputLayer(1 + 2 * l, "h%d" % l)
        hl.GetOutputSlot(0).SetTensorInfo(h_info)
        cl = net.AddInputLayer(2 + 2 * l, "c%d" % l)
        cl.GetOutputSlot(0).SetTensorInfo(c_info)
        params = {}

        def wt(shape, dtype, scale, lo, hi):
            data = rng.integers(lo, hi, size=shape)
            return data, TensorInfo(shape, dtype, scale, 0, constant=True)
        for g in ("Input", "Forget", "Cell", "Output"):
            params["InputTo%sWeights" % g] = wt((num_units, isz), DataType.QSymmS8, q["weights"], -127, 128)
            params["RecurrentTo%sWeights" % g] = wt((num_units, output_size), DataType.QSymmS8, q["weights"], -127, 128)
            params["%sLayerNormWeights" % g] = wt((num_units,), DataType.QSymmS16, q["layer_norm"], 3000, 30000)
        for key in ("InputGateBias", "ForgetGateBias", "CellBias", "OutputGateBias"):
            params[key] = wt((num_units,), DataType.Signed32, _f32(np.float32(q["layer_norm"]) / np.float32(1024)), -8000000, 8000000)
        params["ProjectionWeights"] = wt((output_size, num_units), DataType.QSymmS8, q["projection"], -127, 128)
        desc = dict(CifgEnabled=False, PeepholeEnabled=False, ProjectionEnabled=True, LayerNormEnabled=True,
                    CellClip=0.0, ProjectionClip=0.0,
                    InputIntermediateScale=_f32(q["intermediate_i"]), ForgetIntermediateScale=_f32(q["intermediate_f"]),
                    CellIntermediateScale=_f32(q["intermediate_i"]), OutputIntermediateScale=_f32(q["intermediate_f"]),
                    HiddenStateScale=_f32(q["hidden"]), HiddenStateZeroPoint=0)
        ql = net.AddQLstmLayer(desc, params, "qlstm%d" % l)
        x.Connect(ql.GetInputSlot(0))
        hl.GetOutputSlot(0).Connect(ql.GetInputSlot(1))
        cl.GetOutputSlot(0).Connect(ql.GetInputSlot(2))
        ql.GetOutputSlot(0).SetTensorInfo(h_info)
        ql.GetOutputSlot(1).SetTensorInfo(c_info)
        ql.GetOutputSlot(2).SetTensorInfo(h_info)
        o1 = net.AddOutputLayer(1 + 2 * l, "h%d_out" % l)
        ql.GetOutputSlot(0).Connect(o1.GetInputSlot(0))
        o2 = net.AddOutputLayer(2 + 2 * l, "c%d_out" % l)
        ql.GetOutputSlot(1).Connect(o2.GetInputSlot(0))
        x = ql.GetOutputSlot(2)
        macs += batch * (4 * num_units * (isz + output_size) + output_size * num_units)
    ol = net.AddOutputLayer(0, "y")
    x.Connect(ol.GetInputSlot(0))
    return net, {"macs": macs, "batch": batch, "layers": layers, "input_shape": (batch, input_size),
                 "output_shape": (batch, output_size), "num_units": num_units, "output_size": output_size}
