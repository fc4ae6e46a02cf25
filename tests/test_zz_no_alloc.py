"""b200k_conv2d_q8_static — the convolution entry point for hosts that cannot allocate device memory (for example
a workload living inside a server whose GPU memory pool is carved up once at start-up).  It keeps the weight table
and the re-packed input in a device array compiled into the library instead of in caller buffers.

The check: through the C ABI, its output equals the ordinary entry point's (which gets caller-allocated buffers)
and the CPU oracle's bit for bit — the tolerance every convolution test here uses — on calls in a row with
different inputs, shapes and table contents (a fused-add table, zero-padded channel copies), so that what one call
leaves in the shared array is shown not to matter to the next.  Collected last on purpose."""
import ctypes as C

import numpy as np
import pytest

from q8util import Cuda, _abi, gpu_pack, random_conv_case

pytestmark = pytest.mark.gpu


def _both(case):
    from armnn_b200 import lib
    l = lib.load_library()
    mem = Cuda()
    # ordinary entry point: weight table and input scratch allocated by the caller
    p, y_ref, _ = case.params(mem, False, 2)
    p.packed = gpu_pack(mem, p)
    nbytes = l.b200k_conv2d_scratch_bytes(C.byref(p))
    if nbytes:
        _, p.scratch = mem.out((nbytes,), np.uint8)
        p.scratch_bytes = nbytes
    lib.call("conv2d_q8", p)
    # allocation-free entry point: same tensors, no table, no scratch
    q, y_static, _ = case.params(mem, False, 2)
    lib.check(l.b200k_conv2d_q8_static(C.byref(q), None))
    lib.check(l.b200k_poll_status())
    a, b = mem.fetch(y_ref), mem.fetch(y_static)
    want, _ = case.run_oracle(want_acc=False)
    assert np.array_equal(want, b), "static entry point differs from the oracle"
    return a, b


def test_static_scratch_entry_point_matches_the_ordinary_one_twice(built):
    first = random_conv_case(301, 2, 64, 64, 3, 64, 7, 7, stride=(2, 2), pad=(2, 3, 2, 3), act=(1, 0, 0))
    a, b = _both(first)
    assert a.any() and np.array_equal(a, b)
    # a different, smaller problem right after: stale bytes of the first call stay in the shared array
    second = random_conv_case(302, 1, 40, 40, 3, 128, 3, 3, stride=(2, 2), pad=(0, 1, 0, 1))
    a, b = _both(second)
    assert a.any() and np.array_equal(a, b)
    # and a many-channel convolution, which only needs the weight-table part of the array
    third = random_conv_case(303, 1, 14, 14, 64, 64, 3, 3, pad=(1, 1, 1, 1))
    a, b = _both(third)
    assert np.array_equal(a, b)


def test_static_scratch_entry_point_rebuilds_tables_between_different_layers(built):
    """The shared array also holds the fused-add table and the zero-padded weight copies of channel counts that are
    multiples of 8 only; both are rebuilt by every call.  Two fused Adds with different quantisation around a
    24-channel convolution: a table or a padded copy left over from the previous call would change the result."""
    add1 = random_conv_case(305, 2, 14, 14, 64, 256, 1, 1, act=(1, 0, 0), fused_add=True)
    a, b = _both(add1)
    assert a.any() and np.array_equal(a, b)
    padded = random_conv_case(306, 2, 28, 28, 24, 144, 1, 1, x_dtype=_abi.U8, w_dtype=_abi.U8, y_dtype=_abi.U8,
                              x_q=(0.02, 128), act=(2, 6.0, 0.0), y_zp=0)
    a, b = _both(padded)
    assert a.any() and np.array_equal(a, b)
    add2 = random_conv_case(307, 1, 14, 14, 128, 256, 1, 1, fused_add=True, x_q=(0.03, 7))
    a, b = _both(add2)
    assert a.any() and np.array_equal(a, b)


def test_static_scratch_entry_point_rejects_oversized_problems(built):
    from armnn_b200 import lib
    l = lib.load_library()
    # 24 channels run on zero-padded copies of the input and the output, which live in the scratch
    big = random_conv_case(304, 1, 8, 8, 24, 24, 3, 3)
    mem = Cuda()
    p, _, _ = big.params(mem, False, 2)
    p.n, p.h, p.wd, p.oh, p.ow = 4096, 224, 224, 222, 222          # geometry only: needs far more than 15 MiB
    assert l.b200k_conv2d_q8_static(C.byref(p), None) == _abi.E_TOOBIG
    assert b"exceeds" in l.b200k_last_error()
