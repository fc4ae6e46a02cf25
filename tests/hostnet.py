"""Test-only executors for graphs built with armnn_b200.network:

  OracleNetwork  — runs the optimized graph layer by layer on the plain-C oracle (numpy memory).  It reuses
                   GraphProgram, so the parameter structs are built by exactly the code the CUDA runtime uses;
                   only the memory space and the callee differ.
  ArmnnNetwork   — replays the same (un-optimized) INetwork into the real Arm NN runtime through the C binding
                   in oracle/_ref/libarmnn_capi.so and runs it on CpuRef or, when the plugin is built and a GPU
                   is present, on B200Acc.
"""
import ctypes as C
import os

import numpy as np

from q8util import ROOT, cpuref, oracle

from armnn_b200 import _abi
from armnn_b200.network import _ABI_DTYPE, _NP_DTYPE, DataType, GraphProgram


class OracleNetwork(GraphProgram):
    def __init__(self, optimized):
        super().__init__(optimized)
        self._build()

    def _alloc(self, info):
        return np.zeros(info.shape if info.shape else (1,), dtype=_NP_DTYPE[info.dtype])

    def _upload(self, array):
        return np.ascontiguousarray(array)

    def _ptr(self, tensor):
        return tensor.ctypes.data

    def _view(self, tensor, shape):
        return tensor.reshape(shape)

    def run(self, inputs, keep=None, force=None):
        """inputs: {binding id: ndarray}.  Returns {binding id: ndarray}; `keep`, when a dict, receives
        every intermediate tensor keyed by producing layer name (and output index).  `force`, when a dict
        {(workload index, input index): ndarray}, overwrites that workload's input tensor just before it runs
        (teacher forcing of single layers with another executor's intermediate results)."""
        for bid, arr in inputs.items():
            dst = self._dev(self.inputs[bid])
            dst[...] = np.asarray(arr).reshape(dst.shape).view(dst.dtype)
        for wi, (layer, entry, params) in enumerate(self.workloads):
            if force:
                for ii, s in enumerate(layer.inputs):
                    if (wi, ii) in force:
                        dst = self._dev(s.source)
                        dst[...] = np.asarray(force[(wi, ii)]).reshape(dst.shape).view(dst.dtype)
            rc = getattr(oracle(), "oracle_" + entry)(C.byref(params))
            assert rc == 0, "oracle_%s failed for %s" % (entry, layer.name)
            if keep is not None:
                for i, o in enumerate(layer.outputs):
                    keep[layer.name if i == 0 else "%s:%d" % (layer.name, i)] = self._dev(o).copy()
        return {bid: self._dev(slot).copy() for bid, slot in self.outputs.items()}


PLUGIN_DIR = os.path.join(ROOT, "armnn_b200", "backend")
PLUGIN_PATH = os.path.join(PLUGIN_DIR, "Nv_B200Acc_backend.so")


def _shape_arr(shape):
    return (C.c_int32 * len(shape))(*shape)


class ArmnnNetwork:
    """The same graph inside the real Arm NN runtime."""

    _runtime = None

    @classmethod
    def runtime(cls):
        if cls._runtime is None:
            lib = cpuref()
            lib.armnnc_runtime_create.restype = C.c_void_p
            lib.armnnc_network_create.restype = C.c_void_p
            lib.armnnc_load.restype = C.c_void_p
            path = PLUGIN_DIR if os.path.exists(PLUGIN_PATH) else ""
            cls._runtime = C.c_void_p(lib.armnnc_runtime_create(path.encode()))
            assert cls._runtime.value, lib.cpuref_last_error().decode()
        return cls._runtime

    @staticmethod
    def backend_available(name):
        return bool(cpuref().armnnc_backend_available(ArmnnNetwork.runtime(), name.encode()))

    def __init__(self, network, backends="CpuRef", device_id=-1, profiling=False, optimize_only=False, import_io=False):
        """optimize_only: no LoadNetwork (needs no device); `self.optimized_layers` lists the optimized graph as
        (layer type, name) in execution order.  import_io: load with INetworkProperties{Malloc, Malloc}, so that
        EnqueueWorkload imports the caller's buffers instead of copying them."""
        lib = cpuref()
        self.lib = lib
        rt = self.runtime()
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
                                            d["dilation"][1], int(d["bias"]))
            elif t == "FullyConnected":
                lid = lib.armnnc_add_fully_connected(net, int(d["transpose"]), int(d["bias"]))
            elif t == "Activation":
                lid = lib.armnnc_add_activation(net, int(d["function"]), C.c_float(d["a"]), C.c_float(d["b"]))
            elif t == "Pooling2d":
                lid = lib.armnnc_add_pool2d(net, int(d["type"]), int(d["method"]), d["pool"][0], d["pool"][1], d["stride"][0],
                                            d["stride"][1], d["pad"][0], d["pad"][1], d["pad"][2], d["pad"][3])
            elif t == "ElementwiseBinary":
                lid = lib.armnnc_add_elementwise_binary(net, int(d["op"]))
            elif t == "BatchMatMul":
                lid = lib.armnnc_add_batch_matmul(net, int(d["tx"]), int(d["ty"]), int(d.get("ax", False)), int(d.get("ay", False)))
            elif t == "Softmax":
                lid = lib.armnnc_add_softmax(net, C.c_float(d["beta"]), d["axis"])
            elif t == "Mean":
                axes = (C.c_int32 * len(d["axis"]))(*d["axis"])
                lid = lib.armnnc_add_mean(net, axes, len(d["axis"]), int(d["keep_dims"]))
            elif t == "Reshape":
                lid = lib.armnnc_add_reshape(net, len(d["shape"]), _shape_arr(d["shape"]))
            elif t == "Quantize":
                lid = lib.armnnc_add_quantize(net)
            elif t == "Dequantize":
                lid = lib.armnnc_add_dequantize(net)
            elif t == "QLstm":
                lid = lib.armnnc_add_qlstm(net, C.byref(self._qlstm_params(layer)))
                assert lid >= 0, lib.cpuref_last_error().decode()
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
                lib.armnnc_connect(net, ids[id(s.source.layer)], s.source.index, ids[id(layer)], s.index)
        if optimize_only:
            lib.armnnc_optimized_layers.restype = C.c_size_t
            need = lib.armnnc_optimized_layers(rt, net, backends.encode(), None, C.c_size_t(0))
            err = lib.cpuref_last_error().decode()
            buf = C.create_string_buffer(max(int(need), 1))
            lib.armnnc_optimized_layers(rt, net, backends.encode(), buf, C.c_size_t(len(buf)))
            lib.armnnc_network_destroy(net)
            if not need:
                raise RuntimeError("armnn optimize failed: " + err)
            self.optimized_layers = [tuple(line.split(" ", 1)) for line in buf.value.decode().splitlines()]
            self.handle = C.c_void_p(None)
            return
        self.handle = C.c_void_p(lib.armnnc_load(rt, net, backends.encode(), device_id, int(profiling) | (2 if import_io else 0)))
        err = lib.cpuref_last_error().decode()
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
        assert rc == 0, self.lib.cpuref_last_error().decode()
        return {bid: o for (bid, _), o in zip(self.out_infos, outs)}

    def run_into(self, ins, outs, preimported=False):
        """EnqueueWorkload on caller-owned arrays ({binding id: ndarray}, used in place: no copies made here).
        preimported: through IRuntime::ImportInputs / ImportOutputs, importing the buffers on first use."""
        in_ptrs = (C.c_void_p * len(self.in_infos))(*[ins[bid].ctypes.data for bid, _ in self.in_infos])
        out_ptrs = (C.c_void_p * len(self.out_infos))(*[outs[bid].ctypes.data for bid, _ in self.out_infos])
        fn = self.lib.armnnc_enqueue_preimported if preimported else self.lib.armnnc_enqueue
        rc = fn(self.handle, in_ptrs, out_ptrs)
        assert rc == 0, self.lib.cpuref_last_error().decode()

    def close(self):
        if self.handle is not None and self.handle.value:
            self.lib.armnnc_unload(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
