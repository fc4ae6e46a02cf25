"""Parity tests proper: every libb200k entry point, called through the C ABI with device pointers, against
the CPU oracle on the same seeded inputs.

Bars:
  * contractions (conv / depthwise / fully-connected / batch-matmul): int32 accumulators AND quantised outputs
    bit-exact against the oracle (integer work);
  * fp32-faithful kernels (pooling, mean, elementwise, quantize/dequantize, non-transcendental activations):
    bit-exact against the oracle, which itself equals CpuRef bit for bit;
  * kernels that call exp / tanh / log (softmax, sigmoid, tanh, elu, soft-relu, QLstm gates): within +-1 LSB
    on at most 1 % of the elements — CUDA's and glibc's libm may differ in the last ulp of a transcendental,
    which can move a value across a rounding boundary.  +-1 LSB is the reference's own tolerance for
    quantised tensors (include/armnnTestUtils/TensorHelpers.hpp:25-31 of the Arm NN tree).
"""
import numpy as np
import pytest

import cases
from q8util import diff_stats

pytestmark = pytest.mark.gpu

EXACT_GROUPS = ("conv", "dwconv", "fc", "bmm", "pool", "mean", "eltwise", "convert", "pad", "move", "resize", "reduce", "tconv", "f32", "norm", "volume")
ALL = [(g, n, f) for g, fn in cases.ALL_GROUPS.items() for n, f in fn().items()]


@pytest.mark.parametrize("group,name,factory", ALL, ids=["%s-%s" % (g, n) for g, n, _ in ALL])
def test_cuda_matches_oracle(built, group, name, factory):
    case = factory()
    want = cases.run_case(case, "oracle")
    got = cases.run_case(case, "gpu")
    assert len(want) == len(got)
    exact = ((group in EXACT_GROUPS and not (group == "eltwise" and name in cases.TRANSCENDENTAL_ELTWISE) and
              not (group == "norm" and name in cases.TRANSCENDENTAL_NORM)) or
             (group == "activation" and name not in cases.TRANSCENDENTAL_ACTIVATIONS) or
             (group == "unary" and name not in cases.TRANSCENDENTAL_UNARY) or
             (group == "rows" and name not in cases.TRANSCENDENTAL_ROWS))
    for w, g in zip(want, got):
        assert w.shape == g.shape and w.dtype == g.dtype
        if exact:
            if w.dtype == np.float32:
                assert np.array_equal(w, g), (group, name)
            else:
                assert np.array_equal(w, g), (group, name, diff_stats(w, g))
        elif w.dtype == np.float32:
            # libm against the device's exp / log / sin: a few units in the last place; an LSTM step sums dozens of
            # such values (projection, layer norm), so its differences add up
            rtol, atol = (2e-5, 2e-6) if group == "lstm" else (1e-6, 1e-7)
            assert np.allclose(w, g, rtol=rtol, atol=atol), (group, name, float(np.abs(w - g).max()))
        else:
            st = diff_stats(w, g)
            # int16 cell state of the QLstm: +-2 (two chained transcendental roundings), everything else +-1
            tol = 2 if (group == "qlstm" and w.dtype == np.int16) else 1
            assert st["max_abs"] <= tol and st["mismatch_frac"] <= 0.01, (group, name, st)


def _golden_bmm():
    from test_oracle_vs_cpuref import golden_bmm_cases
    return list(golden_bmm_cases())


@pytest.mark.parametrize("name,case,expected", _golden_bmm(), ids=[c[0] for c in _golden_bmm()])
def test_batch_matmul_known_answers(built, name, case, expected):
    """The BatchMatMul<QAsymmS8> vectors of the reference's own layer tests, on the tensor-core kernel."""
    got = cases.run_case(case, "gpu")[0]
    assert np.array_equal(got.astype(np.int64).ravel(), expected.ravel()), name


def test_error_reporting_instead_of_aborting():
    """Bad arguments come back as negative codes with a message (never a crash)."""
    import ctypes
    from armnn_b200 import _abi, lib
    l = lib.load_library()
    p = _abi.Conv2dParams()
    assert l.b200k_conv2d_q8(ctypes.byref(p), None) == _abi.E_INVALID
    assert b"null" in l.b200k_last_error()
    q = _abi.SoftmaxParams()
    assert l.b200k_softmax_q8(ctypes.byref(q), None) == _abi.E_INVALID
    assert l.b200k_device_open(9999) == _abi.E_INVALID


def test_config2_fc_sweep_subset():
    """FullyConnected sweep rows that the oracle finishes quickly: accumulators and outputs bit-exact."""
    from q8util import random_fc_case
    for m, k in ((1, 4096), (16, 4096), (256, 1024)):
        c = random_fc_case(1000 + m + k, m, k, k)
        y, acc = c.run_oracle()
        gy, gacc = c.run_gpu()
        assert np.array_equal(acc, gacc) and np.array_equal(y, gy), (m, k)


def test_full_size_properties_conv_linearity_and_zero_point_shift():
    """Size-independent properties at a large shape (the oracle is too slow there):
    (1) the int32 accumulator is linear in the input: acc(x1 + x2) == acc(x1) + acc(x2) for zero points 0;
    (2) shifting input and zero point together leaves the accumulator unchanged."""
    import q8util
    from armnn_b200 import _abi
    rng = np.random.default_rng(7)
    n, h, w, c, oc = 8, 56, 56, 64, 64
    x1 = rng.integers(-60, 60, size=(n, h, w, c)).astype(np.int8)
    x2 = rng.integers(-60, 60, size=(n, h, w, c)).astype(np.int8)
    wt = rng.integers(-127, 128, size=(oc, 3, 3, c)).astype(np.int8)

    def acc_of(x, zx):
        case = q8util.ConvCase(x, wt, None, (0.02, zx), (0.005, 0), (0.5, 0), pad=(1, 1, 1, 1))
        return case.run_gpu()[1].astype(np.int64)
    a1, a2, a12 = acc_of(x1, 0), acc_of(x2, 0), acc_of((x1 + x2).astype(np.int8), 0)
    assert np.array_equal(a1 + a2, a12)
    assert np.array_equal(acc_of((x1 + 5).astype(np.int8), 5), a1)
