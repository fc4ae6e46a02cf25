"""Python binding of the Arm NN runtime API: the host side of the B200Acc backend as an Arm NN user sees it.

A graph built with armnn_b200.network.INetwork is replayed into the UNMODIFIED Arm NN runtime (libarmnn.so) through
the C binding armnn_b200/host/libarmnn_capi.so: INetwork -> Optimize(backends) -> IRuntime::LoadNetwork ->
IRuntime::EnqueueWorkload.  With backends="B200Acc" the runtime loads armnn_b200/backend/Nv_B200Acc_backend.so as a
dynamic backend (IRuntime::CreationOptions::m_DynamicBackendsPath) and every layer runs on the GPU; with "CpuRef"
the same graph runs on the reference's own CPU backend (the tests and the reference arm of bench.py use that).

The Arm NN runtime library itself is not part of this repository: $ARMNN_LIB_DIR names the directory that holds
libarmnn.so (default: oracle/_ref, where `make -C oracle ref` builds it from an Arm NN source tree).
"""
import ctypes as C
import os

import numpy as np

from . import _abi
from .network import _ABI_DTYPE as _KERNEL_DTYPE, _NP_DTYPE, DataType


class _BridgeDtype(dict):
    """Element type codes of the bridge to the Arm NN runtime: the C ABI's codes, plus 5 for Boolean (which the kernels see
    as bytes) and 6 for Float16 (which only the two conversion layers touch)."""
    def __missing__(self, key):
        return {DataType.Boolean: 5, DataType.Float16: 6}.get(key) or _KERNEL_DTYPE[key]


_ABI_DTYPE = _BridgeDtype()

_HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(_HERE)
PLUGIN_DIR = os.path.join(_HERE, "backend")
PLUGIN_PATH = os.path.join(PLUGIN_DIR, "Nv_B200Acc_backend.so")
CAPI_PATH = os.path.join(_HERE, "host", "libarmnn_capi.so")


def armnn_lib_dir():
    return os.environ.get("ARMNN_LIB_DIR") or os.path.join(ROOT, "oracle", "_ref")


def available():
    return os.path.exists(CAPI_PATH) and os.path.exists(os.path.join(armnn_lib_dir(), "libarmnn.so"))


_capi = None


def capi():
    """The loaded C binding.  libarmnn.so is loaded RTLD_GLOBAL first: the B200Acc plugin, dlopen()ed later by the
    runtime, resolves the Arm NN symbols it uses against it."""
    global _capi
    if _capi is None:
        if not available():
            raise ImportError("the Arm NN runtime binding is not built: %s and libarmnn.so in %s are needed "
                              "(python -m armnn_b200.build with ARMNN_ROOT set)" % (CAPI_PATH, armnn_lib_dir()))
        C.CDLL(os.path.join(armnn_lib_dir(), "libarmnn.so"), mode=C.RTLD_GLOBAL)
        lib = C.CDLL(CAPI_PATH, mode=C.RTLD_GLOBAL)
        lib.armnnc_last_error.restype = C.c_char_p
        for name in ("armnnc_runtime_create", "armnnc_runtime_create_ex", "armnnc_network_create", "armnnc_load"):
            getattr(lib, name).restype = C.c_void_p
        lib.armnnc_optimized_layers.restype = C.c_size_t
        lib.armnnc_profile_json.restype = C.c_size_t
        _capi = lib
    return _capi


def _shape_arr(shape):
    return (C.c_int32 * len(shape))(*shape)


class Runtime:
    """IRuntime with the B200Acc dynamic backend on its search path.  device_id / graph_replay / selftest_us become
    BackendOptions("B200Acc", {"DeviceId", "GraphReplay", "WaitSelfTestUs"}) of the runtime."""

    def __init__(self, device_id=-1, graph_replay=None, selftest_us=0):
        lib = capi()
        path = PLUGIN_DIR if os.path.exists(PLUGIN_PATH) else ""
        gr = -1 if graph_replay is None else int(bool(graph_replay))
        self.handle = C.c_void_p(lib.armnnc_runtime_create_ex(path.encode(), int(device_id), gr, int(selftest_us)))
        if not self.handle.value:
            raise RuntimeError("IRuntime::Create failed: " + lib.armnnc_last_error().decode())

    _default = None

    @classmethod
    def default(cls):
        if cls._default is None:
            cls._default = cls()
        return cls._default


def graph_stats():
    """(CUDA-graph launches, kernel nodes in them) of the B200Acc plugin in this process so far.  Creates no runtime:
    a second IRuntime would replace the process-wide default device of the first."""
    plugin = C.CDLL(PLUGIN_PATH)                  # the handle the runtime already holds, if one was created
    a, b = C.c_uint64(0), C.c_uint64(0)
    plugin.B200AccGraphStats(C.byref(a), C.byref(b))
    return a.value, b.value


def backend_available(name):
    Runtime.default()
    return bool(capi().armnnc_backend_available(Runtime.default().handle, name.encode()))


class ArmnnNetwork:
    """A graph of armnn_b200.network inside the real Arm NN runtime."""

    def __init__(self, network, backends="CpuRef", device_id=-1, profiling=False, optimize_only=False, import_io=False,
                 runtime=None):
        """device_id: ModelOption BackendOptions("B200Acc", {{"DeviceId", n}}) of this network (-1: the runtime's).
        optimize_only: no LoadNetwork (needs no device); `self.optimized_layers` lists the optimized graph as
        (layer type, name) in execution order.  import_io: load with INetworkProperties{Malloc, Malloc}, so that
        EnqueueWorkload imports the caller's buffers instead of copying them."""
        lib = capi()
        self.lib = lib
        self.rt = runtime or Runtime.default()
        rt = self.rt.handle
        net = C.c_void_p(lib.armnnc_network_create())
        ids = {}
        self.in_infos, self.out_infos = [], []

        def info_args(info):
            return (_ABI_DTYPE[info.dtype], len(info.shape), _shape_arr(info.shape), C.c_float(info.scale), info.offset)

        for layer in network.layers:
            t, d = layer.type, layer.desc
            if t == "Input":
                ids[id(layer)] = lib.armnnc_add_input(net, d["id"], *info_args(layer.outputs[0].info))
                self.in_infos.append((d["id"], layer.outputs[0].info))
                continue
            if t == "Constant" and layer.outputs[0].connections and all(
                    s.layer.type == "TransposeConvolution2d" and s.index > 0 for s in layer.outputs[0].connections):
                continue                              # travels inside the TransposeConvolution2d layer (ConstTensor arguments)
            if t == "Constant":
                info = layer.outputs[0].info
                sc = info.scales
                ids[id(layer)] = lib.armnnc_add_constant(
                    net, _ABI_DTYPE[info.dtype], len(info.shape), _shape_arr(info.shape), C.c_float(info.scale), info.offset,
                    sc.ctypes.data_as(C.c_void_p) if sc is not None else None, len(sc) if sc is not None else 0,
                    info.quant_dim or 0, layer.const_data.ctypes.data_as(C.c_void_p))
                continue
            if t == "Output":
                continue
            if t in ("Convolution2d", "DepthwiseConvolution2d"):
                lid = lib.armnnc_add_conv2d(net, int(t == "DepthwiseConvolution2d"), d["stride"][0], d["stride"][1],
                                            d["pad"][0], d["pad"][1], d["pad"][2], d["pad"][3], d["dilation"][0],
                                            d["dilation"][1], int(d["bias"]), int(d.get("nchw", False)))
            elif t == "FullyConnected":
                lid = lib.armnnc_add_fully_connected(net, int(d["transpose"]), int(d["bias"]))
            elif t == "Activation":
                lid = lib.armnnc_add_activation(net, int(d["function"]), C.c_float(d["a"]), C.c_float(d["b"]))
            elif t == "Pooling2d":
                lid = lib.armnnc_add_pool2d(net, int(d["type"]), int(d["method"]), d["pool"][0], d["pool"][1], d["stride"][0],
                                            d["stride"][1], d["pad"][0], d["pad"][1], d["pad"][2], d["pad"][3], int(d.get("nchw", False)))
            elif t == "Convolution3d":
                lid = lib.armnnc_add_conv3d(net, (C.c_int32 * 3)(*d["stride"]), (C.c_int32 * 6)(*d["pad"]), (C.c_int32 * 3)(*d["dilation"]),
                                            int(d["bias"]))
            elif t == "Pooling3d":
                lid = lib.armnnc_add_pool3d(net, int(d["type"]), int(d["method"]), (C.c_int32 * 3)(*d["pool"]), (C.c_int32 * 3)(*d["stride"]),
                                            (C.c_int32 * 6)(*d["pad"]))
            elif t == "ElementwiseBinary":
                lid = lib.armnnc_add_elementwise_binary(net, int(d["op"]))
            elif t == "Comparison":
                lid = lib.armnnc_add_comparison(net, d["op"])
            elif t == "LogicalBinary":
                lid = lib.armnnc_add_logical_binary(net, d["op"])
            elif t == "BatchMatMul":
                lid = lib.armnnc_add_batch_matmul(net, int(d["tx"]), int(d["ty"]), int(d.get("ax", False)), int(d.get("ay", False)))
            elif t == "Normalization":
                lid = lib.armnnc_add_normalization(net, d["channel_type"], C.c_uint(d["norm_size"]), C.c_float(d["alpha"]),
                                                   C.c_float(d["beta"]), C.c_float(d["k"]), int(d["nchw"]))
            elif t == "ScatterNd":
                lid = lib.armnnc_add_scatter_nd(net, d["function"], int(d["input_enabled"]))
            elif t == "ReverseV2":
                lid = lib.armnnc_add_reverse_v2(net)
            elif t == "GatherNd":
                lid = lib.armnnc_add_gather_nd(net)
            elif t == "Gather":
                lid = lib.armnnc_add_gather(net, d["axis"])
            elif t == "BatchNormalization":
                keys = ("mean", "variance", "beta", "gamma")
                arrs = [np.ascontiguousarray(np.asarray(layer.bn_params[k][0]).astype(_NP_DTYPE[layer.bn_params[k][1].dtype])) for k in keys]
                infos = [layer.bn_params[k][1] for k in keys]
                self._keep = getattr(self, "_keep", []) + arrs
                lid = lib.armnnc_add_batch_norm(
                    net, C.c_float(d["eps"]), int(d["nchw"]), int(arrs[0].size),
                    (C.c_int32 * 4)(*[_ABI_DTYPE[i.dtype] for i in infos]), (C.c_float * 4)(*[i.scale for i in infos]),
                    (C.c_int32 * 4)(*[i.offset for i in infos]), (C.c_void_p * 4)(*[a.ctypes.data for a in arrs]))
            elif t == "InstanceNormalization":
                lid = lib.armnnc_add_instance_norm(net, C.c_float(d["gamma"]), C.c_float(d["beta"]), C.c_float(d["eps"]), int(d["nchw"]))
            elif t == "LogSoftmax":
                lid = lib.armnnc_add_log_softmax(net, C.c_float(d["beta"]), d["axis"])
            elif t == "L2Normalization":
                lid = lib.armnnc_add_l2_normalization(net, C.c_float(d["eps"]), int(d["nchw"]))
            elif t == "ArgMinMax":
                lid = lib.armnnc_add_arg_min_max(net, d["function"], d["axis"])
            elif t == "Softmax":
                lid = lib.armnnc_add_softmax(net, C.c_float(d["beta"]), d["axis"])
            elif t == "Mean":
                axes = (C.c_int32 * len(d["axis"]))(*d["axis"])
                lid = lib.armnnc_add_mean(net, axes, len(d["axis"]), int(d["keep_dims"]))
            elif t == "Reshape":
                lid = lib.armnnc_add_reshape(net, len(d["shape"]), _shape_arr(d["shape"]))
            elif t == "Pad":
                flat = [v for pair in d["pads"] for v in pair]
                lid = lib.armnnc_add_pad(net, len(d["pads"]), (C.c_int32 * len(flat))(*flat), C.c_float(d["value"]), int(d.get("mode", 0)))
            elif t in ("Shape", "Rank"):
                lid = lib.armnnc_add_shape(net, int(t == "Rank"))
            elif t == "FakeQuantization":
                # armnn::INetwork has no AddFakeQuantizationLayer (the layer only enters a graph through the optimizer's
                # internals), so the bridge cannot state it
                raise NotImplementedError("ArmnnNetwork: FakeQuantization cannot be added through armnn::INetwork")
            elif t in ("ConvertFp16ToFp32", "ConvertFp32ToFp16"):
                # armnn::INetwork has no call for these: the optimizer inserts them around layers a backend only runs in Float32
                raise NotImplementedError("ArmnnNetwork: the fp16 conversion layers cannot be added through armnn::INetwork")
            elif t == "Cast":
                lid = lib.armnnc_add_cast(net)
            elif t == "Fill":
                lid = lib.armnnc_add_fill(net, C.c_float(d["value"]))
            elif t == "Floor":
                lid = lib.armnnc_add_floor(net)
            elif t == "TransposeConvolution2d":
                wl = layer.inputs[1].source.layer
                wi = wl.outputs[0].info
                wsc = wi.scales
                bdata = bsc = None
                bscale = 0.0
                if d["bias"]:
                    bl = layer.inputs[2].source.layer
                    bdata, bsc, bscale = bl.const_data, bl.outputs[0].info.scales, bl.outputs[0].info.scale
                lid = lib.armnnc_add_transpose_conv2d(
                    net, d["stride"][0], d["stride"][1], d["pad"][0], d["pad"][1], d["pad"][2], d["pad"][3],
                    _ABI_DTYPE[wi.dtype], _shape_arr(wi.shape), C.c_float(wi.scale), wi.offset,
                    wsc.ctypes.data_as(C.c_void_p) if wsc is not None else None, len(wsc) if wsc is not None else 0,
                    wl.const_data.ctypes.data_as(C.c_void_p),
                    bdata.ctypes.data_as(C.c_void_p) if bdata is not None else None, C.c_float(bscale),
                    bsc.ctypes.data_as(C.c_void_p) if bsc is not None else None, len(bsc) if bsc is not None else 0,
                    int(d.get("nchw", False)))
                assert lid >= 0, lib.armnnc_last_error().decode()
            elif t in ("DepthToSpace", "SpaceToDepth"):
                lid = lib.armnnc_add_depth_to_space(net, d["block"], int(d["nchw"]), int(t == "SpaceToDepth"))
            elif t in ("BatchToSpaceNd", "SpaceToBatchNd"):
                blk = (C.c_int32 * len(d["block"]))(*d["block"])
                flat = [v for pair in d["edges"] for v in pair]
                lid = lib.armnnc_add_batch_to_space(net, blk, (C.c_int32 * len(flat))(*flat), len(d["block"]), int(d["nchw"]),
                                                    int(t == "SpaceToBatchNd"))
            elif t == "Tile":
                lid = lib.armnnc_add_tile(net, (C.c_int32 * len(d["multiples"]))(*d["multiples"]), len(d["multiples"]))
            elif t == "BroadcastTo":
                lid = lib.armnnc_add_broadcast_to(net, _shape_arr(d["shape"]), len(d["shape"]))
            elif t == "ChannelShuffle":
                lid = lib.armnnc_add_channel_shuffle(net, d["axis"], d["groups"])
            elif t == "Stack":
                ish = layer.inputs[0].source.info.shape
                lid = lib.armnnc_add_stack(net, d["axis"], len(layer.inputs), len(ish), _shape_arr(ish))
            elif t == "Prelu":
                lid = lib.armnnc_add_prelu(net)
            elif t == "ElementwiseUnary":
                lid = lib.armnnc_add_elementwise_unary(net, d["op"])
            elif t == "Reduce":
                axes = (C.c_int32 * len(d["axis"]))(*d["axis"])
                lid = lib.armnnc_add_reduce(net, axes, len(d["axis"]), d["op"], int(d["keep_dims"]))
            elif t == "Resize":
                lid = lib.armnnc_add_resize(net, d["height"], d["width"], d["method"], int(d["align_corners"]),
                                            int(d["half_pixel_centers"]), int(d["nchw"]))
            elif t == "Concat":
                flat = [x for o in d["origins"] for x in o]
                lid = lib.armnnc_add_concat(net, len(d["origins"]), len(d["origins"][0]), (C.c_int32 * len(flat))(*flat))
            elif t == "Splitter":
                flat = [x for o in d["origins"] for x in o]
                sizes = [x for o in layer.outputs for x in o.info.shape]
                lid = lib.armnnc_add_splitter(net, len(d["origins"]), len(d["origins"][0]), (C.c_int32 * len(flat))(*flat),
                                              (C.c_int32 * len(sizes))(*sizes))
            elif t in ("Permute", "Transpose"):
                m = d["mappings"]
                lid = lib.armnnc_add_permute(net, len(m), (C.c_int32 * len(m))(*m), int(t == "Transpose"))
                assert lid >= 0, lib.armnnc_last_error().decode()
            elif t == "StridedSlice":
                r = len(d["begin"])
                arr = lambda v: (C.c_int32 * r)(*v)
                lid = lib.armnnc_add_strided_slice(net, r, arr(d["begin"]), arr(d["end"]), arr(d["stride"]), d["begin_mask"],
                                                   d["end_mask"], d["shrink_axis_mask"], d.get("ellipsis_mask", 0),
                                                   d.get("new_axis_mask", 0))
            elif t == "Slice":
                r = len(d["begin"])
                lid = lib.armnnc_add_slice(net, r, (C.c_int32 * r)(*d["begin"]), (C.c_int32 * r)(*d["size"]))
            elif t == "Quantize":
                lid = lib.armnnc_add_quantize(net)
            elif t == "Dequantize":
                lid = lib.armnnc_add_dequantize(net)
            elif t in ("Lstm", "UnidirectionalSequenceLstm"):
                lid = lib.armnnc_add_lstm(net, C.byref(self._lstm_params(layer)), int(t != "Lstm"), int(bool(d.get("TimeMajor", False))))
                assert lid >= 0, lib.armnnc_last_error().decode()
            elif t == "QLstm":
                lid = lib.armnnc_add_qlstm(net, C.byref(self._qlstm_params(layer)))
                assert lid >= 0, lib.armnnc_last_error().decode()
            else:
                raise NotImplementedError("ArmnnNetwork: layer type %s" % t)
            ids[id(layer)] = lid
            for i, o in enumerate(layer.outputs):
                lib.armnnc_set_output_info(net, lid, i, *info_args(o.info))
        for layer in network.layers:
            if layer.type == "Output":
                src = layer.inputs[0].source
                lib.armnnc_add_output(net, layer.desc["id"], ids[id(src.layer)], src.index)
                self.out_infos.append((layer.desc["id"], src.info))
                continue
            for s in layer.inputs:
                if layer.type == "TransposeConvolution2d" and s.index > 0:
                    continue
                lib.armnnc_connect(net, ids[id(s.source.layer)], s.source.index, ids[id(layer)], s.index)
        if optimize_only:
            need = lib.armnnc_optimized_layers(rt, net, backends.encode(), None, C.c_size_t(0))
            err = lib.armnnc_last_error().decode()
            buf = C.create_string_buffer(max(int(need), 1))
            lib.armnnc_optimized_layers(rt, net, backends.encode(), buf, C.c_size_t(len(buf)))
            lib.armnnc_network_destroy(net)
            if not need:
                raise RuntimeError("armnn optimize failed: " + err)
            self.optimized_layers = [tuple(line.split(" ", 1)) for line in buf.value.decode().splitlines()]
            self.handle = C.c_void_p(None)
            return
        self.handle = C.c_void_p(lib.armnnc_load(rt, net, backends.encode(), device_id, int(profiling) | (2 if import_io else 0)))
        err = lib.armnnc_last_error().decode()
        lib.armnnc_network_destroy(net)
        if not self.handle.value:
            raise RuntimeError("armnn load failed: " + err)

    _QLSTM_FIELDS = {"InputToInputWeights": ("w_i2i", "s_i2i"), "InputToForgetWeights": ("w_i2f", "s_i2f"),
                     "InputToCellWeights": ("w_i2c", "s_i2c"), "InputToOutputWeights": ("w_i2o", "s_i2o"),
                     "RecurrentToInputWeights": ("w_r2i", "s_r2i"), "RecurrentToForgetWeights": ("w_r2f", "s_r2f"),
                     "RecurrentToCellWeights": ("w_r2c", "s_r2c"), "RecurrentToOutputWeights": ("w_r2o", "s_r2o"),
                     "CellToInputWeights": ("w_c2i", "s_c2i"), "CellToForgetWeights": ("w_c2f", "s_c2f"),
                     "CellToOutputWeights": ("w_c2o", "s_c2o"), "InputGateBias": ("b_i", "s_bi"),
                     "ForgetGateBias": ("b_f", "s_bf"), "CellBias": ("b_c", "s_bc"), "OutputGateBias": ("b_o", "s_bo"),
                     "InputLayerNormWeights": ("ln_i", "s_lni"), "ForgetLayerNormWeights": ("ln_f", "s_lnf"),
                     "CellLayerNormWeights": ("ln_c", "s_lnc"), "OutputLayerNormWeights": ("ln_o", "s_lno"),
                     "ProjectionWeights": ("w_proj", "s_proj"), "ProjectionBias": ("b_proj", "s_bproj")}

    def _lstm_params(self, layer):
        """b200k_lstm_params with HOST weight pointers, as armnnc_add_lstm wants."""
        from .network import GraphProgram
        d = layer.desc
        p = _abi.LstmParams()
        x, h, c = (s.source.info for s in layer.inputs)
        p.input_size, p.output_size, p.num_units = x.shape[-1], h.shape[1], c.shape[1]
        self._keep = getattr(self, "_keep", [])
        for key, field in GraphProgram._LSTM_FIELDS.items():
            item = layer.qlstm_params.get(key)
            if item is None:
                continue
            arr = np.ascontiguousarray(np.asarray(item[0], np.float32))
            self._keep.append(arr)
            setattr(p, field, arr.ctypes.data)
        if d.get("CifgEnabled"):
            p.w_i2i = p.w_r2i = p.w_c2i = p.b_i = p.ln_i = None
        if not d.get("PeepholeEnabled"):
            p.w_c2i = p.w_c2f = p.w_c2o = None
        if not d.get("LayerNormEnabled"):
            p.ln_i = p.ln_f = p.ln_c = p.ln_o = None
        if not d.get("ProjectionEnabled"):
            p.w_proj = p.b_proj = None
        p.activation = int(d.get("ActivationFunc", 4))
        p.cell_clip, p.projection_clip = float(d.get("ClippingThresCell", 0.0)), float(d.get("ClippingThresProj", 0.0))
        return p

    def _qlstm_params(self, layer):
        """b200k_qlstm_params with HOST weight pointers, as armnnc_add_qlstm wants."""
        d = layer.desc
        p = _abi.QLstmParams()
        x, h, c = (s.source.info for s in layer.inputs)
        p.batch, p.input_size = x.shape
        p.output_size, p.num_units = h.shape[1], c.shape[1]
        self._keep = getattr(self, "_keep", [])
        for key, (wf, sf) in self._QLSTM_FIELDS.items():
            item = layer.qlstm_params.get(key)
            if item is None:
                continue
            data, info = item
            arr = np.ascontiguousarray(np.asarray(data).astype(_NP_DTYPE[info.dtype]))
            self._keep.append(arr)
            setattr(p, wf, arr.ctypes.data)
            setattr(p, sf, info.scale)
        if d.get("CifgEnabled"):
            p.w_i2i = p.w_r2i = None
        if not d.get("PeepholeEnabled"):
            p.w_c2i = p.w_c2f = p.w_c2o = None
        if not d.get("LayerNormEnabled"):
            p.ln_i = p.ln_f = p.ln_c = p.ln_o = None
        if not d.get("ProjectionEnabled"):
            p.w_proj = p.b_proj = None
        p.cell_clip, p.projection_clip = d.get("CellClip", 0.0), d.get("ProjectionClip", 0.0)
        p.input_intermediate_scale = d["InputIntermediateScale"]
        p.forget_intermediate_scale = d["ForgetIntermediateScale"]
        p.cell_intermediate_scale = d["CellIntermediateScale"]
        p.output_intermediate_scale = d["OutputIntermediateScale"]
        p.hidden_state_scale, p.hidden_state_zp = d["HiddenStateScale"], d["HiddenStateZeroPoint"]
        return p

    def run(self, inputs):
        ins = [np.ascontiguousarray(np.asarray(inputs[bid]).astype(_NP_DTYPE[info.dtype], copy=False)) for bid, info in self.in_infos]
        outs = [np.zeros(info.shape, dtype=_NP_DTYPE[info.dtype]) for _, info in self.out_infos]
        in_ptrs = (C.c_void_p * len(ins))(*[a.ctypes.data for a in ins])
        out_ptrs = (C.c_void_p * len(outs))(*[a.ctypes.data for a in outs])
        rc = self.lib.armnnc_enqueue(self.handle, in_ptrs, out_ptrs)
        assert rc == 0, self.lib.armnnc_last_error().decode()
        return {bid: o for (bid, _), o in zip(self.out_infos, outs)}

    def enqueue_ptrs(self, in_ptrs, out_ptrs, preimported=False):
        """EnqueueWorkload on raw host addresses (lists in binding order); returns the runtime's status (0 = Success)."""
        ip = (C.c_void_p * len(in_ptrs))(*in_ptrs)
        op = (C.c_void_p * len(out_ptrs))(*out_ptrs)
        fn = self.lib.armnnc_enqueue_preimported if preimported else self.lib.armnnc_enqueue
        return fn(self.handle, ip, op)

    def run_into(self, ins, outs, preimported=False):
        """EnqueueWorkload on caller-owned arrays ({binding id: ndarray}, used in place: no copies made here).
        preimported: through IRuntime::ImportInputs / ImportOutputs, importing the buffers on first use."""
        rc = self.enqueue_ptrs([ins[bid].ctypes.data for bid, _ in self.in_infos],
                               [outs[bid].ctypes.data for bid, _ in self.out_infos], preimported)
        assert rc == 0, self.lib.armnnc_last_error().decode()

    def profile_json(self):
        need = self.lib.armnnc_profile_json(self.handle, None, C.c_size_t(0))
        buf = C.create_string_buffer(max(int(need), 1))
        self.lib.armnnc_profile_json(self.handle, buf, C.c_size_t(len(buf)))
        return buf.value.decode()

    def close(self):
        if self.handle is not None and self.handle.value:
            self.lib.armnnc_unload(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
