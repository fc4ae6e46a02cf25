"""Shared helpers for the parity tests.

Three executors take the SAME parameter structs (include/b200k.h):
  * ORACLE  — oracle/libq8oracle.so, the plain-C restatement (host pointers)
  * CPUREF  — oracle/_ref/libarmnn_capi.so, the real CpuRef workloads of the reference (host pointers)
  * GPU     — armnn_b200/libb200k.so, the product (device pointers, via torch for memory only)
A test builds a case once (numpy arrays + geometry) and runs it on any of them.
"""
import ctypes as C
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from armnn_b200 import _abi  # noqa: E402

NP_OF = {_abi.U8: np.uint8, _abi.S8: np.int8, _abi.S16: np.int16, _abi.S32: np.int32, _abi.F32: np.float32}
RANGE = {_abi.U8: (0, 255), _abi.S8: (-128, 127), _abi.S16: (-32768, 32767)}

ORACLE_PATH = os.path.join(ROOT, "oracle", "libq8oracle.so")
CPUREF_PATH = os.path.join(ROOT, "oracle", "_ref", "libcpuref_capi.so")

_oracle = None
_cpuref = None


def oracle():
    global _oracle
    if _oracle is None:
        _oracle = C.CDLL(ORACLE_PATH)
    return _oracle


def have_cpuref():
    return os.path.exists(CPUREF_PATH)


def cpuref():
    global _cpuref
    if _cpuref is None:
        # libarmnn.so first and RTLD_GLOBAL: one copy of the Arm NN core for this binding, the runtime binding of
        # armnn_b200.armnn_host and the B200Acc plugin the runtime dlopen()s
        C.CDLL(os.path.join(os.path.dirname(CPUREF_PATH), "libarmnn.so"), mode=C.RTLD_GLOBAL)
        _cpuref = C.CDLL(CPUREF_PATH, mode=C.RTLD_GLOBAL)
        _cpuref.cpuref_last_error.restype = C.c_char_p
    return _cpuref


def have_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


class Host:
    """numpy memory"""
    name = "host"

    def __init__(self):
        self.keep = []

    def inp(self, arr):
        arr = np.ascontiguousarray(arr)
        self.keep.append(arr)
        return arr.ctypes.data

    def out(self, shape, np_dtype):
        a = np.zeros(shape, dtype=np_dtype)
        self.keep.append(a)
        return a, a.ctypes.data

    def fetch(self, handle):
        return handle


class Cuda:
    """torch CUDA memory (allocation and copies only)"""
    name = "cuda"

    def __init__(self):
        import torch
        self.torch = torch
        self.keep = []

    def inp(self, arr):
        t = self.torch.from_numpy(np.ascontiguousarray(arr)).cuda()
        self.keep.append(t)
        return t.data_ptr()

    def out(self, shape, np_dtype):
        t = self.torch.zeros(tuple(shape), dtype=getattr(self.torch, np.dtype(np_dtype).name), device="cuda")
        self.keep.append(t)
        return t, t.data_ptr()

    def fetch(self, handle):
        self.torch.cuda.synchronize()
        return handle.cpu().numpy()


def qt(mem, arr, dtype, scale=1.0, zp=0, scales=None):
    t = _abi.QTensor()
    t.data = mem.inp(arr.astype(NP_OF[dtype], copy=False)) if arr is not None else None
    t.dtype = dtype
    t.scale = float(scale)
    t.zero_point = int(zp)
    t.scales = mem.inp(np.asarray(scales, dtype=np.float32)) if scales is not None else None
    return t


def qt_out(mem, shape, dtype, scale=1.0, zp=0):
    handle, ptr = mem.out(shape, NP_OF[dtype])
    t = _abi.QTensor()
    t.data = ptr
    t.dtype = dtype
    t.scale = float(scale)
    t.zero_point = int(zp)
    t.scales = None
    return t, handle


def activation_clamp(kind, a, b, scale, zp, dtype):
    lo, hi = C.c_int32(), C.c_int32()
    rc = oracle().oracle_activation_clamp(C.c_int(kind), C.c_float(a), C.c_float(b), C.c_float(scale),
                                          C.c_int32(zp), C.c_int32(dtype), C.byref(lo), C.byref(hi))
    assert rc == 0
    return lo.value, hi.value


def gpu_pack(mem, conv_params):
    """b200k_conv2d_pack into a fresh device buffer; returns its pointer."""
    from armnn_b200 import lib
    l = lib.load_library()
    nbytes = l.b200k_conv2d_pack_bytes(conv_params.oc, conv_params.kh, conv_params.kw, conv_params.c)
    _, ptr = mem.out((nbytes // 4,), np.int32)
    lib.check(l.b200k_conv2d_pack(C.byref(conv_params), C.c_void_p(ptr), None))
    return ptr


def out_size(i, k, s, pb, pa, d=1):
    return (i + pb + pa - (d * (k - 1) + 1)) // s + 1


# --------------------------------------------------------------------------------------------------
# Cases.  Each case object knows how to fill the parameter struct for a memory space and how to call
# each executor.
# --------------------------------------------------------------------------------------------------

class ConvCase:
    """Convolution2d / DepthwiseConvolution2d (NHWC, weights OHWI or [1,H,W,O])."""

    def __init__(self, x, w, bias, x_q, w_q, y_q, stride=(1, 1), pad=(0, 0, 0, 0), dil=(1, 1), act=(0, 0.0, 0.0),
                 depthwise=False, w_scales=None, b_scale=None, b_scales=None, x_dtype=_abi.S8, w_dtype=_abi.S8,
                 y_dtype=_abi.S8, add=None):
        self.add = add                 # None, or (other operand array, (scale, zp), (out scale, out zp)): fused Add
        self.x, self.w, self.bias = x, w, bias
        self.x_q, self.w_q, self.y_q = x_q, w_q, y_q           # (scale, zp)
        self.w_scales, self.b_scale, self.b_scales = w_scales, b_scale, b_scales
        self.stride, self.pad, self.dil, self.act = stride, pad, dil, act   # pad = (top, bottom, left, right)
        self.depthwise = depthwise
        self.x_dtype, self.w_dtype, self.y_dtype = x_dtype, w_dtype, y_dtype
        n, h, wd, c = x.shape
        if depthwise:
            _, kh, kw, oc = w.shape
        else:
            oc, kh, kw, _ = w.shape
        self.geom = (n, h, wd, c, oc, kh, kw)
        self.oh = out_size(h, kh, stride[0], pad[0], pad[1], dil[0])
        self.ow = out_size(wd, kw, stride[1], pad[2], pad[3], dil[1])

    def params(self, mem, want_acc=False, algo=0):
        n, h, wd, c, oc, kh, kw = self.geom
        p = _abi.Conv2dParams()
        p.x = qt(mem, self.x, self.x_dtype, *self.x_q)
        p.w = qt(mem, self.w, self.w_dtype, self.w_q[0], self.w_q[1], self.w_scales)
        if self.bias is not None:
            p.bias = qt(mem, self.bias, _abi.S32, self.b_scale if self.b_scale is not None else 1.0, 0, self.b_scales)
        p.y, y = qt_out(mem, (n, self.oh, self.ow, oc), self.y_dtype, *self.y_q)
        p.n, p.h, p.wd, p.c, p.oh, p.ow, p.oc, p.kh, p.kw = n, h, wd, c, self.oh, self.ow, oc, kh, kw
        p.stride_h, p.stride_w = self.stride
        p.pad_top, p.pad_left = self.pad[0], self.pad[2]
        p.dil_h, p.dil_w = self.dil
        out_q = self.y_q
        if self.add is not None:
            other, other_q, out_q = self.add
            p.add_operand = qt(mem, other, self.y_dtype, *other_q)
            p.add_out, y = qt_out(mem, (n, self.oh, self.ow, oc), self.y_dtype, *out_q)
            p.y.data = None
        p.clamp_lo, p.clamp_hi = activation_clamp(self.act[0], self.act[1], self.act[2], out_q[0], out_q[1], self.y_dtype)
        acc = None
        if want_acc:
            acc, ptr = mem.out((n, self.oh, self.ow, oc), np.int32)
            p.acc_out = ptr
        p.algo = algo
        return p, y, acc

    def run_oracle(self, want_acc=True):
        mem = Host()
        p, y, acc = self.params(mem, want_acc)
        fn = oracle().oracle_dwconv2d_q8 if self.depthwise else oracle().oracle_conv2d_q8
        assert fn(C.byref(p)) == 0
        return y, acc

    def run_cpuref(self):
        mem = Host()
        if self.add is not None:
            # three separate CpuRef workloads: Convolution2d, ElementwiseBinary(Add), Activation
            plain = ConvCase(self.x, self.w, self.bias, self.x_q, self.w_q, self.y_q, self.stride, self.pad, self.dil,
                             (0, 0., 0.), self.depthwise, self.w_scales, self.b_scale, self.b_scales, self.x_dtype,
                             self.w_dtype, self.y_dtype)
            conv_out = plain.run_cpuref()
            other, other_q, out_q = self.add
            e = _abi.EltwiseParams()
            e.a = qt(mem, conv_out, self.y_dtype, *self.y_q)
            e.b = qt(mem, other, self.y_dtype, *other_q)
            e.out, out = qt_out(mem, conv_out.shape, self.y_dtype, *out_q)
            e.rank = 4
            for i in range(4):
                e.shape_a[i] = e.shape_b[i] = e.shape_out[i] = conv_out.shape[i]
            e.op = 0
            rc = cpuref().cpuref_eltwise_q8(C.byref(e), C.c_int(self.act[0]), C.c_float(self.act[1]), C.c_float(self.act[2]))
            assert rc == 0, cpuref().cpuref_last_error().decode()
            return out
        p, y, _ = self.params(mem)
        rc = cpuref().cpuref_conv2d_q8(C.byref(p), C.c_int(int(self.depthwise)), C.c_int(self.act[0]),
                                       C.c_float(self.act[1]), C.c_float(self.act[2]))
        assert rc == 0, cpuref().cpuref_last_error().decode()
        return y

    def run_gpu(self, want_acc=True, algo=0, pack=True):
        from armnn_b200 import lib
        mem = Cuda()
        p, y, acc = self.params(mem, want_acc, algo)
        if pack and not self.depthwise:
            p.packed = gpu_pack(mem, p)
            nbytes = lib.load_library().b200k_conv2d_scratch_bytes(C.byref(p))
            if nbytes:
                _, p.scratch = mem.out((nbytes,), np.uint8)
                p.scratch_bytes = nbytes
        lib.call("dwconv2d_q8" if self.depthwise else "conv2d_q8", p)
        return mem.fetch(y), (mem.fetch(acc) if acc is not None else None)


def random_conv_case(seed, n, h, wd, c, oc, kh, kw, stride=(1, 1), pad=(0, 0, 0, 0), dil=(1, 1), act=(0, 0., 0.),
                     depthwise=False, x_dtype=_abi.S8, w_dtype=_abi.S8, y_dtype=_abi.S8, per_axis=True,
                     x_q=(0.02, -3), y_scale=None, y_zp=None, bias=True, depth_multiplier=1, fused_add=False, w_zp=None):
    """Seeded synthetic conv in the style of the benchmark configs: uniform activations over the
    whole type range, weights uniform, per-output-channel scales uniform in [0.001, 0.01], int32 bias
    uniform in [-1000, 1000] with scale sx * sw[c].  The output scale defaults to one that leaves
    most outputs unsaturated so that the comparison is not vacuous."""
    rng = np.random.default_rng(seed)
    lo, hi = RANGE[x_dtype]
    x = rng.integers(lo, hi + 1, size=(n, h, wd, c)).astype(NP_OF[x_dtype])
    if depthwise:
        oc = c * depth_multiplier
        wshape = (1, kh, kw, oc)
    else:
        wshape = (oc, kh, kw, c)
    # w_zp: an explicit per-tensor weight zero point (QAsymmS8 / QAsymmU8 weights); default 0 for int8, random for uint8
    if w_dtype == _abi.S8:
        w = rng.integers(-128 if w_zp is not None else -127, 128, size=wshape).astype(np.int8)
        w_zp = 0 if w_zp is None else int(w_zp)
    else:
        w = rng.integers(0, 256, size=wshape).astype(np.uint8)
        w_zp = int(rng.integers(100, 156)) if w_zp is None else int(w_zp)
    if per_axis and w_dtype == _abi.S8:
        w_scales = rng.uniform(0.001, 0.01, size=oc).astype(np.float32)
        w_q = (1.0, 0)
        b_scales = (np.float32(x_q[0]) * w_scales).astype(np.float32)
        b_scale = None
    else:
        w_scales = None
        w_q = (float(np.float32(rng.uniform(0.001, 0.01))), w_zp)
        b_scales = None
        b_scale = float(np.float32(x_q[0]) * np.float32(w_q[0]))
    b = rng.integers(-1000, 1001, size=oc).astype(np.int32) if bias else None
    if y_scale is None:
        k = kh * kw * (1 if depthwise else c)
        mean_sw = float(np.mean(w_scales)) if w_scales is not None else w_q[0]
        std = x_q[0] * mean_sw * 74.0 * 74.0 * np.sqrt(k)       # uniform int8 std ~ 74
        y_scale = float(np.float32(std * 3.0 / 127.0))
    if y_zp is None:
        y_zp = 0 if y_dtype == _abi.S8 else 128
    case = ConvCase(x, w, b, x_q, w_q, (y_scale, y_zp), stride, pad, dil, act, depthwise, w_scales, b_scale, b_scales,
                    x_dtype, w_dtype, y_dtype)
    if fused_add:
        # residual operand at a different scale / offset, output wide enough for the sum
        lo, hi = RANGE[y_dtype]
        other = rng.integers(lo, hi + 1, size=(n, case.oh, case.ow, oc)).astype(NP_OF[y_dtype])
        other_q = (float(np.float32(y_scale * 0.8)), y_zp + 3)
        out_zp = lo if act[0] else y_zp - 2
        case.add = (other, other_q, (float(np.float32(y_scale * 1.3)), out_zp))
    return case


class FcCase:
    def __init__(self, x, w, bias, x_q, w_q, y_q, transpose_w=True, w_scales=None, b_scale=None, b_scales=None,
                 act=(0, 0., 0.), x_dtype=_abi.S8, w_dtype=_abi.S8, y_dtype=_abi.S8):
        self.__dict__.update(locals())
        self.m, self.k = x.shape
        self.n = w.shape[0] if transpose_w else w.shape[1]

    def params(self, mem, want_acc=False, algo=0):
        p = _abi.FcParams()
        p.x = qt(mem, self.x, self.x_dtype, *self.x_q)
        p.w = qt(mem, self.w, self.w_dtype, self.w_q[0], self.w_q[1], self.w_scales)
        if self.bias is not None:
            p.bias = qt(mem, self.bias, _abi.S32, self.b_scale if self.b_scale is not None else 1.0, 0, self.b_scales)
        p.y, y = qt_out(mem, (self.m, self.n), self.y_dtype, *self.y_q)
        p.m, p.k, p.n, p.transpose_w = self.m, self.k, self.n, int(self.transpose_w)
        p.clamp_lo, p.clamp_hi = activation_clamp(self.act[0], self.act[1], self.act[2], self.y_q[0], self.y_q[1], self.y_dtype)
        acc = None
        if want_acc:
            acc, ptr = mem.out((self.m, self.n), np.int32)
            p.acc_out = ptr
        p.algo = algo
        return p, y, acc

    def run_oracle(self, want_acc=True):
        mem = Host()
        p, y, acc = self.params(mem, want_acc)
        assert oracle().oracle_fully_connected_q8(C.byref(p)) == 0
        return y, acc

    def run_cpuref(self):
        mem = Host()
        p, y, _ = self.params(mem)
        rc = cpuref().cpuref_fully_connected_q8(C.byref(p), C.c_int(self.act[0]), C.c_float(self.act[1]), C.c_float(self.act[2]))
        assert rc == 0, cpuref().cpuref_last_error().decode()
        return y

    def run_gpu(self, want_acc=True, algo=0, pack=True):
        from armnn_b200 import lib
        mem = Cuda()
        p, y, acc = self.params(mem, want_acc, algo)
        if pack and self.transpose_w:
            c = _abi.Conv2dParams()
            c.w, c.oc, c.kh, c.kw, c.c = p.w, self.n, 1, 1, self.k
            p.packed = gpu_pack(mem, c)
        lib.call("fully_connected_q8", p)
        return mem.fetch(y), (mem.fetch(acc) if acc is not None else None)


def random_fc_case(seed, m, k, n, transpose_w=True, x_q=(0.03, 5), per_axis=True, x_dtype=_abi.S8, w_dtype=_abi.S8,
                   y_dtype=_abi.S8, act=(0, 0., 0.)):
    rng = np.random.default_rng(seed)
    lo, hi = RANGE[x_dtype]
    x = rng.integers(lo, hi + 1, size=(m, k)).astype(NP_OF[x_dtype])
    wshape = (n, k) if transpose_w else (k, n)
    if w_dtype == _abi.S8:
        w = rng.integers(-127, 128, size=wshape).astype(np.int8)
        w_zp = 0
    else:
        w = rng.integers(0, 256, size=wshape).astype(np.uint8)
        w_zp = int(rng.integers(100, 156))
    if per_axis and w_dtype == _abi.S8:
        w_scales = rng.uniform(0.001, 0.01, size=n).astype(np.float32)
        w_q = (1.0, 0)
        b_scales = (np.float32(x_q[0]) * w_scales).astype(np.float32)
        b_scale = None
        mean_sw = float(np.mean(w_scales))
    else:
        w_scales, b_scales = None, None
        w_q = (float(np.float32(rng.uniform(0.001, 0.01))), w_zp)
        b_scale = float(np.float32(x_q[0]) * np.float32(w_q[0]))
        mean_sw = w_q[0]
    b = rng.integers(-1000, 1001, size=n).astype(np.int32)
    std = x_q[0] * mean_sw * 74.0 * 74.0 * np.sqrt(k)
    y_q = (float(np.float32(std * 3.0 / 127.0)), 0 if y_dtype == _abi.S8 else 128)
    return FcCase(x, w, b, x_q, w_q, y_q, transpose_w, w_scales, b_scale, b_scales, act, x_dtype, w_dtype, y_dtype)


class SimpleCase:
    """A case defined by a function that fills a params struct from a memory space."""

    def __init__(self, entry, build, cpuref_extra=()):
        self.entry, self.build, self.cpuref_extra = entry, build, cpuref_extra

    def run_oracle(self):
        mem = Host()
        p, outs = self.build(mem)
        rc = getattr(oracle(), "oracle_" + self.entry)(C.byref(p))
        assert rc == 0, "oracle_%s returned %d" % (self.entry, rc)
        return outs

    def run_cpuref(self):
        mem = Host()
        p, outs = self.build(mem)
        rc = getattr(cpuref(), "cpuref_" + self.entry)(C.byref(p), *self.cpuref_extra)
        assert rc == 0, cpuref().cpuref_last_error().decode()
        return outs

    def run_gpu(self):
        from armnn_b200 import lib
        mem = Cuda()
        p, outs = self.build(mem)
        lib.call(self.entry, p)
        return [mem.fetch(o) for o in outs]


class OracleMoveParams(C.Structure):
    """oracle/move_desc.h"""
    _fields_ = [("kind", C.c_int32), ("rank", C.c_int32), ("whole", _abi.QTensor), ("whole_shape", C.c_int32 * 6),
                ("n_views", C.c_int32), ("view", _abi.QTensor * 8), ("view_rank", C.c_int32 * 8), ("view_shape", (C.c_int32 * 6) * 8),
                ("view_origin", (C.c_int32 * 6) * 8), ("perm", C.c_int32 * 6),
                ("begin", C.c_int32 * 6), ("end", C.c_int32 * 6), ("stride", C.c_int32 * 6),
                ("begin_mask", C.c_int32), ("end_mask", C.c_int32), ("shrink_axis_mask", C.c_int32)]


MOVE_KINDS = {"concat": 0, "split": 1, "permute": 2, "transpose": 3, "strided_slice": 4, "slice": 5,
              "depth_to_space": 6, "space_to_depth": 7, "channel_shuffle": 8, "stack": 9,
              "batch_to_space": 10, "space_to_batch": 11, "tile": 12, "broadcast_to": 13}


class MoveCase:
    """One data-movement layer stated as the reference's descriptor.  `whole` is the Concat output (then `parts` are the
    inputs) or the input of every other kind (then `parts` are the outputs).  Tensors are (shape, dtype, scale, zp)."""

    def __init__(self, kind, seed, whole, parts, origins=None, perm=None, begin=None, end=None, stride=None,
                 begin_mask=0, end_mask=0, shrink_axis_mask=0):
        self.kind, self.seed, self.whole, self.parts = kind, seed, whole, parts
        self.origins, self.perm, self.begin, self.end, self.stride = origins, perm, begin, end, stride
        self.masks = (begin_mask, end_mask, shrink_axis_mask)

    def _data(self, mem):
        """(whole tensor, part tensors, output handles) in `mem`, inputs filled with seeded values."""
        rng = np.random.default_rng(self.seed)

        def rand(shape, dtype):
            if dtype == _abi.F32:
                return rng.standard_normal(shape).astype(np.float32)
            if dtype == _abi.S32:
                return rng.integers(-100000, 100000, size=shape).astype(np.int32)
            lo, hi = RANGE[dtype]
            return rng.integers(lo, hi + 1, size=shape).astype(NP_OF[dtype])
        outs = []
        if self.kind in ("concat", "stack"):
            parts = [qt(mem, rand(sh, dt), dt, sc, zp) for sh, dt, sc, zp in self.parts]
            sh, dt, sc, zp = self.whole
            whole, h = qt_out(mem, sh, dt, sc, zp)
            outs.append(h)
        else:
            sh, dt, sc, zp = self.whole
            whole = qt(mem, rand(sh, dt), dt, sc, zp)
            parts = []
            for sh, dt, sc, zp in self.parts:
                t, h = qt_out(mem, sh, dt, sc, zp)
                parts.append(t)
                outs.append(h)
        return whole, parts, outs

    def _params(self, mem):
        whole, parts, outs = self._data(mem)
        p = OracleMoveParams()
        p.kind, p.rank = MOVE_KINDS[self.kind], len(self.whole[0])
        p.whole = whole
        for i, n in enumerate(self.whole[0]):
            p.whole_shape[i] = n
        p.n_views = len(parts)
        for v, t in enumerate(parts):
            p.view[v] = t
            p.view_rank[v] = len(self.parts[v][0])
            for i, n in enumerate(self.parts[v][0]):
                p.view_shape[v][i] = n
            if self.origins is not None:
                for i, o in enumerate(self.origins[v]):
                    p.view_origin[v][i] = o
        for name in ("perm", "begin", "end", "stride"):
            vals = getattr(self, name)
            if vals is not None:
                for i, x in enumerate(vals):
                    getattr(p, name)[i] = x
        p.begin_mask, p.end_mask, p.shrink_axis_mask = self.masks
        return p, outs

    def run_oracle(self):
        mem = Host()
        p, outs = self._params(mem)
        rc = oracle().oracle_move_q(C.byref(p))
        assert rc == 0, "oracle_move_q returned %d" % rc
        return outs

    def run_cpuref(self):
        mem = Host()
        p, outs = self._params(mem)
        rc = cpuref().cpuref_move_q(C.byref(p))
        assert rc == 0, cpuref().cpuref_last_error().decode()
        return outs

    def views(self):
        """[(view, source index, destination index)] with -1 for the whole tensor, -2 for one element holding the
        destination's encoding of 0.0, else the index of the part."""
        from armnn_b200 import views as V
        shapes = [pt[0] for pt in self.parts]
        if self.kind == "concat":
            vs = V.concat_views(self.whole[0], shapes, self.origins)
            order = list(reversed(range(len(shapes))))
            return [(v, i, -1) for v, i in zip(vs, order)]
        if self.kind == "split":
            return [(v, -1, i) for i, v in enumerate(V.splitter_views(self.whole[0], shapes, self.origins))]
        if self.kind == "stack":
            out_shape, vs = V.stack_views(shapes[0], len(shapes), self.perm[0])
            assert tuple(out_shape) == tuple(self.whole[0]), (out_shape, self.whole[0])
            return [(v, i, -1) for i, v in enumerate(vs)]
        if self.kind in ("depth_to_space", "space_to_depth"):
            fn = V.depth_to_space_view if self.kind == "depth_to_space" else V.space_to_depth_view
            out_shape, v = fn(self.whole[0], self.perm[0], bool(self.perm[1]))
            assert tuple(out_shape) == tuple(shapes[0]), (out_shape, shapes[0])
            return [(v, -1, 0)]
        if self.kind in ("batch_to_space", "space_to_batch"):
            sp = len(self.whole[0]) - 2
            block, edges = self.begin[:sp], list(zip(self.end[:sp], self.stride[:sp]))
            if self.kind == "batch_to_space":
                out_shape, vs = V.batch_to_space_views(self.whole[0], block, edges, bool(self.perm[0]))
                padded = False
            else:
                out_shape, vs, padded = V.space_to_batch_views(self.whole[0], block, edges, bool(self.perm[0]))
            assert tuple(out_shape) == tuple(shapes[0]), (out_shape, shapes[0])
            return ([(V.fill_view(out_shape), -2, 0)] if padded else []) + [(v, -1, 0) for v in vs]
        if self.kind == "tile":
            out_shape, v = V.tile_view(self.whole[0], self.perm)
            assert tuple(out_shape) == tuple(shapes[0]), (out_shape, shapes[0])
            return [(v, -1, 0)]
        if self.kind == "broadcast_to":
            return [(V.broadcast_to_view(self.whole[0], shapes[0]), -1, 0)]
        if self.kind == "channel_shuffle":
            return [(V.channel_shuffle_view(self.whole[0], self.perm[0], self.perm[1]), -1, 0)]
        if self.kind in ("permute", "transpose"):
            out_shape, v = V.permute_view(self.whole[0], self.perm, transpose=self.kind == "transpose")
            assert tuple(out_shape) == tuple(shapes[0]), (out_shape, shapes[0])
            return [(v, -1, 0)]
        if self.kind == "strided_slice":
            walk, out_shape, v = V.strided_slice_view(self.whole[0], self.begin, self.end, self.stride, *self.masks)
            assert int(np.prod(walk)) == int(np.prod(shapes[0])), (walk, shapes[0])
            return [(v, -1, 0)]
        out_shape, v = V.slice_view(self.whole[0], self.begin, self.end)
        assert tuple(out_shape) == tuple(shapes[0])
        return [(v, -1, 0)]

    def run_gpu(self):
        from armnn_b200 import lib
        from armnn_b200 import views as V
        mem = Cuda()
        whole, parts, outs = self._data(mem)
        for view, si, di in self.views():
            shape, so, ss, do, ds = V.merge_dims(view)
            p = _abi.ViewCopyParams()
            if si == -2:
                _, dt, sc, zp = self.parts[di]
                lo, hi = RANGE.get(dt, (0, 0))
                zero = np.zeros(1, np.float32) if dt == _abi.F32 else np.array([min(max(zp, lo), hi)], NP_OF[dt])
                p.x = qt(mem, zero, dt, sc, zp)
            else:
                p.x = whole if si < 0 else parts[si]
            p.y = whole if di < 0 else parts[di]
            p.rank = len(shape)
            for i in range(len(shape)):
                p.shape[i], p.src_strides[i], p.dst_strides[i] = shape[i], ss[i], ds[i]
            p.src_offset, p.dst_offset = so, do
            lib.call("view_copy_q", p)
        return [mem.fetch(o) for o in outs]


def diff_stats(a, b):
    d = a.astype(np.int64) - b.astype(np.int64)
    return {"max_abs": int(np.abs(d).max()) if d.size else 0,
            "mismatch_frac": float(np.mean(d != 0)) if d.size else 0.0}


def saturation(y, dtype):
    lo, hi = RANGE[dtype]
    return float(np.mean((y == lo) | (y == hi)))


class QLstmCase:
    """One QLstm step.  `w` maps ABI field names (w_i2f, ln_c, b_o, w_proj, ...) to numpy arrays;
    `s` maps scale / scalar field names to numbers.  Absent optional weights disable the option."""

    W_FIELDS = {"w_i2i": np.int8, "w_i2f": np.int8, "w_i2c": np.int8, "w_i2o": np.int8,
                "w_r2i": np.int8, "w_r2f": np.int8, "w_r2c": np.int8, "w_r2o": np.int8,
                "w_c2i": np.int16, "w_c2f": np.int16, "w_c2o": np.int16,
                "b_i": np.int32, "b_f": np.int32, "b_c": np.int32, "b_o": np.int32,
                "ln_i": np.int16, "ln_f": np.int16, "ln_c": np.int16, "ln_o": np.int16,
                "w_proj": np.int8, "b_proj": np.int32}

    def __init__(self, x, h, c, w, s):
        self.x, self.h, self.c, self.w, self.s = x, h, c, w, s
        self.batch, self.input_size = x.shape
        self.output_size = h.shape[1]
        self.num_units = c.shape[1]

    def params(self, mem):
        p = _abi.QLstmParams()
        p.batch, p.input_size, p.num_units, p.output_size = self.batch, self.input_size, self.num_units, self.output_size
        p.input = mem.inp(self.x.astype(np.int8))
        p.output_state_in = mem.inp(self.h.astype(np.int8))
        p.cell_state_in = mem.inp(self.c.astype(np.int16))
        hout, p.output_state_out = mem.out((self.batch, self.output_size), np.int8)
        cout, p.cell_state_out = mem.out((self.batch, self.num_units), np.int16)
        out, p.output = mem.out((self.batch, self.output_size), np.int8)
        for name, dt in self.W_FIELDS.items():
            if self.w.get(name) is not None:
                setattr(p, name, mem.inp(np.asarray(self.w[name]).astype(dt)))
        for name, v in self.s.items():
            setattr(p, name, v)
        return p, [hout, cout, out]

    def run_oracle(self):
        mem = Host()
        p, outs = self.params(mem)
        assert oracle().oracle_qlstm_step(C.byref(p)) == 0
        return outs

    def run_cpuref(self):
        mem = Host()
        p, outs = self.params(mem)
        rc = cpuref().cpuref_qlstm_step(C.byref(p))
        assert rc == 0, cpuref().cpuref_last_error().decode()
        return outs

    def run_gpu(self):
        from armnn_b200 import lib
        mem = Cuda()
        p, outs = self.params(mem)
        lib.call("qlstm_step", p)
        return [mem.fetch(o) for o in outs]


def qlstm_scales(input_scale=0.0078125, out_scale=0.007, ln_scale=3.05182e-05, w_scale=0.00784314,
                 proj_scale=0.00392157, cell_scale=3.05176e-05, layer_norm=True, projection=True):
    """Quantisation parameters of the reference's projection + layer-norm QLstm test
    (src/backends/backendsCommon/test/layerTests/LstmTestImpl.cpp:1937-1968)."""
    f32 = lambda v: float(np.float32(v))
    s = dict(input_scale=f32(input_scale), input_zp=0, output_state_scale=f32(out_scale), output_state_zp=0,
             cell_state_scale=f32(cell_scale), output_scale=f32(out_scale), output_zp=0,
             cell_clip=0.0, projection_clip=0.0,
             input_intermediate_scale=f32(0.007059), forget_intermediate_scale=f32(0.007812),
             cell_intermediate_scale=f32(0.007059), output_intermediate_scale=f32(0.007812),
             hidden_state_scale=f32(0.007), hidden_state_zp=0)
    for g in "ifco":
        s["s_i2" + g] = f32(w_scale)
        s["s_r2" + g] = f32(w_scale)
    for g in "ifco":
        s["s_b" + g] = float(np.float32(ln_scale) / np.float32(1024))
        if layer_norm:
            s["s_ln" + g] = f32(ln_scale)
    if projection:
        s["s_proj"] = f32(proj_scale)
    return s


def random_qlstm_case(seed, batch, input_size, num_units, output_size, layer_norm=True, projection=True, cifg=False,
                      peephole=False, state="random"):
    rng = np.random.default_rng(seed)
    x = rng.integers(-128, 128, size=(batch, input_size)).astype(np.int8)
    if state == "zero":
        h = np.zeros((batch, output_size), np.int8)
        c = np.zeros((batch, num_units), np.int16)
    else:
        h = rng.integers(-128, 128, size=(batch, output_size)).astype(np.int8)
        c = rng.integers(-20000, 20000, size=(batch, num_units)).astype(np.int16)
    w = {}
    gates = "fco" if cifg else "ifco"
    for g in gates:
        w["w_i2" + g] = rng.integers(-127, 128, size=(num_units, input_size)).astype(np.int8)
        w["w_r2" + g] = rng.integers(-127, 128, size=(num_units, output_size)).astype(np.int8)
        # gate biases are mandatory in the descriptor although CpuRef only reads them with layer norm
        w["b_" + g] = rng.integers(-8000000, 8000000, size=num_units).astype(np.int32)
        if layer_norm:
            w["ln_" + g] = rng.integers(3000, 30000, size=num_units).astype(np.int16)
    if peephole:
        for g in ("fo" if cifg else "ifo"):
            w["w_c2" + g] = rng.integers(-20000, 20000, size=num_units).astype(np.int16)
    if projection:
        w["w_proj"] = rng.integers(-127, 128, size=(output_size, num_units)).astype(np.int8)
    s = qlstm_scales(layer_norm=layer_norm, projection=projection)
    if peephole:
        for g in "ifo":
            s["s_c2" + g] = float(np.float32(2.0 ** -15))
    return QLstmCase(x, h, c, w, s)
