"""Pins the CPU oracle: every restated function against (a) the reference's own known-answer vectors and
(b) the real CpuRef workloads compiled from the reference sources (oracle/_ref), on the seeded cases that the
GPU tests later use.  No GPU needed."""
import json
import os

import numpy as np
import pytest

import cases
from q8util import (ConvCase, FcCase, QLstmCase, SimpleCase, _abi, diff_stats, have_cpuref, qlstm_scales, qt, qt_out)

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "ref_layer_tests.json")))
DT = {"u8": _abi.U8, "s8": _abi.S8}

needs_cpuref = pytest.mark.skipif(not have_cpuref(), reason="oracle/_ref not built (reference sources absent)")


def _q(real, scale, zp, lo, hi):
    """armnnUtils::QuantizedVector: Quantize() of each real value."""
    r = np.asarray(real, dtype=np.float32) / np.float32(scale)
    q = np.float32(zp) + np.where(r >= 0, np.floor(r + np.float32(0.5)), np.ceil(r - np.float32(0.5)))
    return np.clip(q, lo, hi).astype(np.int64)


def _golden_cases():
    g = GOLDEN["conv2d_per_axis_quant"]
    conv = ConvCase(np.array(g["x"], np.uint8).reshape(g["x_shape"]), np.array(g["w"], np.int8).reshape(g["w_shape"]),
                    np.array(g["bias"], np.int32), (g["x_scale"], g["x_zp"]), (1.0, 0), (g["y_scale"], g["y_zp"]),
                    w_scales=np.array(g["w_scales"], np.float32), b_scales=np.array(g["b_scales"], np.float32),
                    x_dtype=_abi.U8, w_dtype=_abi.S8, y_dtype=_abi.U8)
    yield "conv2d_per_axis_quant", conv, np.array(g["y"]), g["tolerance"], 0
    g = GOLDEN["dwconv2d_per_axis_quant"]
    dw = ConvCase(np.array(g["x"], np.uint8).reshape(g["x_shape"]), np.array(g["w"], np.int8).reshape(g["w_shape"]),
                  np.array(g["bias"], np.int32), (g["x_scale"], g["x_zp"]), (1.0, 0), (g["y_scale"], g["y_zp"]),
                  depthwise=True, w_scales=np.array(g["w_scales"], np.float32), b_scales=np.array(g["b_scales"], np.float32),
                  x_dtype=_abi.U8, w_dtype=_abi.S8, y_dtype=_abi.U8)
    yield "dwconv2d_per_axis_quant", dw, np.array(g["y"]), g["tolerance"], 0
    g = GOLDEN["fully_connected_u8_bias"]
    x = _q(g["x_real"], g["x_scale"], g["x_zp"], 0, 255).astype(np.uint8).reshape(1, 6)
    w = _q(g["w_real"], g["w_scale"], g["w_zp"], 0, 255).astype(np.uint8).reshape(g["w_shape"])
    fc = FcCase(x, w, np.array(g["bias"], np.int32), (g["x_scale"], g["x_zp"]), (g["w_scale"], g["w_zp"]),
                (g["y_scale"], g["y_zp"]), b_scale=float(np.float32(g["x_scale"]) * np.float32(g["w_scale"])),
                x_dtype=_abi.U8, w_dtype=_abi.U8, y_dtype=_abi.U8)
    yield "fully_connected_u8_bias", fc, _q(g["y_real"], g["y_scale"], g["y_zp"], 0, 255), g["tolerance"], 0
    g = GOLDEN["avg_pool_2x2_u8"]
    xq = _q(g["x_nchw_real"], g["scale"], g["zp"], 0, 255).astype(np.uint8).reshape(1, 2, 4, 4).transpose(0, 2, 3, 1)
    yq = _q(g["y_nchw_real"], g["scale"], g["zp"], 0, 255).reshape(1, 2, 2, 2).transpose(0, 2, 3, 1)

    def build(mem, g=g, xq=xq):
        p = _abi.Pool2dParams()
        p.x = qt(mem, np.ascontiguousarray(xq), _abi.U8, g["scale"], g["zp"])
        p.y, y = qt_out(mem, (1, 2, 2, 2), _abi.U8, g["scale"], g["zp"])
        p.n, p.h, p.wd, p.c, p.oh, p.ow = 1, 4, 4, 2, 2, 2
        p.pool_h = p.pool_w = p.stride_h = p.stride_w = 2
        p.pool_type, p.padding_method = 1, 1
        return p, [y]
    yield "avg_pool_2x2_u8", SimpleCase("pool2d_q8", build), yq, g["tolerance"], 0
    g = GOLDEN["qlstm_projection_layernorm"]
    sc = g["scales"]
    s = qlstm_scales(sc["input_scale"], sc["output_scale"], sc["layer_norm"], sc["weights"], sc["projection"], sc["cell_scale"])
    s.update(hidden_state_scale=float(np.float32(sc["hidden_scale"])),
             input_intermediate_scale=float(np.float32(sc["input_intermediate"])),
             forget_intermediate_scale=float(np.float32(sc["forget_intermediate"])),
             cell_intermediate_scale=float(np.float32(sc["cell_intermediate"])),
             output_intermediate_scale=float(np.float32(sc["output_intermediate"])))
    B, I, U, O = g["batch"], g["input_size"], g["num_units"], g["output_size"]
    w = {}
    for k in ("w_i2i", "w_i2f", "w_i2c", "w_i2o"):
        w[k] = np.array(g[k]).reshape(U, I)
    for k in ("w_r2i", "w_r2f", "w_r2c", "w_r2o"):
        w[k] = np.array(g[k]).reshape(U, O)
    for k in ("b_i", "b_f", "b_c", "b_o", "ln_i", "ln_f", "ln_c", "ln_o"):
        w[k] = np.array(g[k])
    w["w_proj"] = np.array(g["w_proj"]).reshape(O, U)
    ql = QLstmCase(np.array(g["input"]).reshape(B, I), np.zeros((B, O)), np.zeros((B, U)), w, s)
    yield "qlstm_projection_layernorm", ql, np.array(g["output"]).reshape(B, O), g["tolerance"], 2


def golden_bmm_cases():
    """BatchMatMul<QAsymmS8> known answers (tests/golden/transcribe_batch_matmul.py): (name, case, expected)."""
    for name, g in GOLDEN.items():
        if not name.startswith("batch_matmul_"):
            continue
        xs, ys = g["x_shape"], g["y_shape"]
        batch = int(np.prod(xs[:-2])) if len(xs) > 2 else 1
        ybatch = int(np.prod(ys[:-2])) if len(ys) > 2 else 1
        tx, ty = bool(g["transpose_x"]), bool(g["transpose_y"])
        m, k = (xs[-1], xs[-2]) if tx else (xs[-2], xs[-1])
        n = ys[-2] if ty else ys[-1]

        def build(mem, g=g, xs=xs, ys=ys, batch=batch, ybatch=ybatch, tx=tx, ty=ty, m=m, k=k, n=n):
            p = _abi.BmmParams()
            p.x = qt(mem, np.array(g["x"], np.int8).reshape(xs), _abi.S8, g["scale"], g["zp"])
            p.y = qt(mem, np.array(g["y"], np.int8).reshape(ys), _abi.S8, g["scale"], g["zp"])
            p.out, out = qt_out(mem, (batch, m, n), _abi.S8, g["scale"], g["zp"])
            p.batch, p.m, p.k, p.n = batch, m, k, n
            p.transpose_x, p.transpose_y = int(tx), int(ty)
            p.batch_stride_x = m * k
            p.batch_stride_y = k * n if ybatch == batch else 0
            return p, [out]
        # the lists hold the tests' real values; armnnUtils::QuantizedVector<int8_t> saturates them (3DBatch expects 267 -> 127)
        yield name, SimpleCase("batch_matmul_q8", build), np.clip(np.array(g["out"]), -128, 127)


def _all_golden():
    for c in _golden_cases():
        yield c
    for name, case, expected in golden_bmm_cases():
        yield name, case, expected, GOLDEN[name]["tolerance"], 0


GOLDEN_CASES = list(_all_golden())


@pytest.mark.parametrize("name,case,expected,tol,out_index", GOLDEN_CASES, ids=[c[0] for c in GOLDEN_CASES])
def test_oracle_matches_reference_known_answers(built, name, case, expected, tol, out_index):
    got = cases.run_case(case, "oracle")[out_index]
    assert np.abs(got.astype(np.int64).ravel() - expected.ravel()).max() <= tol


@needs_cpuref
@pytest.mark.parametrize("name,case,expected,tol,out_index", GOLDEN_CASES, ids=[c[0] for c in GOLDEN_CASES])
def test_real_cpuref_matches_its_own_known_answers(built, name, case, expected, tol, out_index):
    """Sanity of the harness around the compiled reference: CpuRef reproduces the vectors of its own tests."""
    got = cases.run_case(case, "cpuref")[out_index]
    assert np.abs(got.astype(np.int64).ravel() - expected.ravel()).max() <= tol


# group -> (max |delta| allowed vs real CpuRef, max fraction of differing elements)
# Contractions: the oracle accumulates exactly in int32, CpuRef in fp32, so they may differ on rounding ties.
# fp32-faithful restatements must be identical.
TOLERANCE = {"conv": (1, 2e-3), "dwconv": (1, 2e-3), "fc": (1, 2e-3), "bmm": (1, 2e-3),
             "pool": (0, 0.0), "mean": (0, 0.0), "eltwise": (0, 0.0), "activation": (0, 0.0), "softmax": (0, 0.0),
             "convert": (0, 0.0), "pad": (0, 0.0), "qlstm": (0, 0.0), "move": (0, 0.0), "resize": (0, 0.0), "reduce": (0, 0.0), "tconv": (1, 2e-3), "f32": (0, 0.0), "unary": (0, 0.0), "rows": (0, 0.0), "norm": (0, 0.0), "volume": (1, 2e-3), "lstm": (0, 0.0)}

ALL = [(g, n, f) for g, fn in cases.ALL_GROUPS.items() for n, f in fn().items()]


@needs_cpuref
@pytest.mark.parametrize("group,name,factory", ALL, ids=["%s-%s" % (g, n) for g, n, _ in ALL])
def test_oracle_equals_real_cpuref(built, group, name, factory):
    if (group, name) in cases.CPUREF_REFUSES:
        pytest.skip("the CpuRef workload refuses this input")
    case = factory()
    got = cases.run_case(case, "oracle")
    ref = cases.run_case(case, "cpuref")
    max_abs, max_frac = TOLERANCE[group]
    if group == "volume" and name.startswith("pool3d"):
        max_abs, max_frac = 0, 0.0                 # the contraction tolerance is for Convolution3d only
    if group == "bmm":                             # second output is the int32 accumulator, which CpuRef lacks
        got, ref = got[:1], ref[:1]
    for o, r in zip(got, ref):                     # zip: CpuRef has no accumulator output
        if o.dtype == np.float32:
            assert np.array_equal(o, r)
            continue
        st = diff_stats(o, r)
        assert st["max_abs"] <= max_abs and st["mismatch_frac"] <= max_frac, (group, name, st)
