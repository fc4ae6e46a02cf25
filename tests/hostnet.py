"""Test-only executors for graphs built with armnn_b200.network:

  OracleNetwork  — runs the optimized graph layer by layer on the plain-C oracle (numpy memory).  It reuses
                   GraphProgram, so the parameter structs are built by exactly the code the CUDA runtime uses;
                   only the memory space and the callee differ.
  ArmnnNetwork   — (re-exported from armnn_b200.armnn_host) replays the same (un-optimized) INetwork into the real
                   Arm NN runtime and runs it on CpuRef or, when the plugin is built and a GPU is present, on B200Acc.
"""
import ctypes as C
import os

import numpy as np

from q8util import ROOT, oracle

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


# The graph-level executor on the real Arm NN runtime (CpuRef, or B200Acc through the plugin) lives in the package:
from armnn_b200.armnn_host import PLUGIN_DIR, PLUGIN_PATH, ArmnnNetwork, Runtime, backend_available  # noqa: E402,F401
