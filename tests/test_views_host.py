"""armnn_b200/views.py (descriptor -> rectangular view copies) against numpy's own indexing, on the CPU: the host logic
behind Concat, Splitter, Permute, Transpose, StridedSlice and Slice.  (The same descriptors run against the real CpuRef
workloads in test_oracle_vs_cpuref.py and on the GPU in test_kernels_gpu.py.)"""
import numpy as np
import pytest

from armnn_b200 import views as V


def apply_view(src, dst, view):
    """The copy `b200k_view_copy_q` performs, in numpy, through flat buffers."""
    shape, so, ss, do, ds = view
    s, d = src.reshape(-1), dst.reshape(-1)
    for idx in np.ndindex(*shape):
        d[do + sum(i * st for i, st in zip(idx, ds))] = s[so + sum(i * st for i, st in zip(idx, ss))]


def test_permute_and_transpose_views_match_numpy():
    rng = np.random.default_rng(1)
    x = rng.integers(-128, 128, size=(2, 3, 4, 5)).astype(np.int8)
    for perm in [(0, 2, 3, 1), (3, 2, 1, 0), (1, 0, 3, 2), (0, 1, 2, 3)]:
        # Transpose: destination dimension i is source dimension perm[i] (numpy's convention)
        out_shape, view = V.permute_view(x.shape, perm, transpose=True)
        want = np.transpose(x, perm)
        assert tuple(out_shape) == want.shape
        got = np.zeros(out_shape, np.int8)
        apply_view(x, got, view)
        assert np.array_equal(got, want)
        # Permute: source dimension i goes to destination dimension perm[i] (the inverse permutation for numpy)
        out_shape, view = V.permute_view(x.shape, perm, transpose=False)
        want = np.transpose(x, np.argsort(perm))
        assert tuple(out_shape) == want.shape
        got = np.zeros(out_shape, np.int8)
        apply_view(x, got, view)
        assert np.array_equal(got, want)
    with pytest.raises(ValueError):
        V.permute_view((2, 3), (0, 0))


def test_concat_and_splitter_views_match_numpy():
    rng = np.random.default_rng(2)
    a = rng.integers(0, 255, size=(2, 3, 4)).astype(np.uint8)
    b = rng.integers(0, 255, size=(2, 5, 4)).astype(np.uint8)
    want = np.concatenate([a, b], axis=1)
    got = np.zeros_like(want)
    vs = V.concat_views(want.shape, [a.shape, b.shape], [(0, 0, 0), (0, 3, 0)])
    for src, view in zip([b, a], vs):                      # (issued last view first)
        apply_view(src, got, view)
    assert np.array_equal(got, want)
    outs = [np.zeros_like(a), np.zeros_like(b)]
    for out, view in zip(outs, V.splitter_views(want.shape, [a.shape, b.shape], [(0, 0, 0), (0, 3, 0)])):
        apply_view(want, out, view)
    assert np.array_equal(outs[0], a) and np.array_equal(outs[1], b)
    with pytest.raises(ValueError):
        V.concat_views((2, 4), [(2, 3)], [(0, 2)])


@pytest.mark.parametrize("begin,end,stride,bm,em,sm,py", [
    ((1, 0, 2), (3, 5, 6), (1, 2, 1), 0, 0, 0, (slice(1, 3), slice(0, 5, 2), slice(2, 6))),
    ((0, -1, 0), (0, 0, 0), (1, -1, 2), 0b001, 0b111, 0, (slice(None), slice(None, None, -1), slice(None, None, 2))),
    ((2, 1, 0), (0, 4, 0), (1, 1, 1), 0, 0b100, 0b001, (2, slice(1, 4), slice(None))),
    ((-3, 0, -2), (-1, 5, 7), (1, 3, 1), 0, 0, 0, (slice(-3, -1), slice(0, 5, 3), slice(-2, 7))),
])
def test_strided_slice_views_match_numpy(begin, end, stride, bm, em, sm, py):
    x = np.arange(4 * 5 * 7, dtype=np.int16).reshape(4, 5, 7)
    walk, out_shape, view = V.strided_slice_view(x.shape, begin, end, stride, bm, em, sm)
    want = x[py]
    assert tuple(out_shape) == want.shape
    got = np.zeros(walk, np.int16)
    apply_view(x, got, view)
    assert np.array_equal(got.reshape(want.shape), want)


def test_slice_view_and_dimension_merging():
    x = np.arange(2 * 6 * 8 * 16, dtype=np.int32).reshape(2, 6, 8, 16)
    out_shape, view = V.slice_view(x.shape, (1, 2, 0, 0), (1, 3, 8, 16))
    got = np.zeros(out_shape, np.int32)
    apply_view(x, got, view)
    assert np.array_equal(got, x[1:2, 2:5])
    # whole rows and whole pixels are contiguous on both sides: one long row after merging
    merged = V.merge_dims(view)
    assert merged[0] == (3 * 8 * 16,) and merged[2] == [1] and merged[4] == [1]
    got2 = np.zeros(out_shape, np.int32)
    apply_view(x, got2, merged)
    assert np.array_equal(got2, got)
    # a channel slice keeps the pixel dimension apart
    _, view = V.slice_view(x.shape, (0, 0, 0, 4), (2, 6, 8, 8))
    merged = V.merge_dims(view)
    assert merged[0] == (2 * 6 * 8, 8)
    with pytest.raises(ValueError):
        V.slice_view(x.shape, (0, 0, 0, 10), (2, 6, 8, 8))


def _to_nhwc4(x, nchw):
    x4 = x if x.ndim == 4 else (x[:, :, :, None] if nchw else x[:, :, None, :])
    return x4.transpose(0, 2, 3, 1) if nchw else x4


def _from_nhwc4(y, rank, nchw):
    y = y.transpose(0, 3, 1, 2) if nchw else y
    if rank == 3:
        y = y[:, :, :, 0] if nchw else y[:, :, 0, :]
    return np.ascontiguousarray(y)


@pytest.mark.parametrize("nchw", [False, True])
@pytest.mark.parametrize("dims,block,edges", [
    ((8, 3, 4, 5), (2, 2), ((0, 0), (0, 0))), ((12, 3, 4, 5), (2, 3), ((1, 2), (3, 1))),
    ((6, 4, 2, 3), (3, 2), ((0, 5), (1, 0))), ((6, 4, None, 5), (3,), ((0, 0),)), ((4, 5, None, 3), (2,), ((1, 2),))])
def test_batch_to_space_views_follow_the_reference_loop(dims, block, edges, nchw):
    """`workloads/BatchToSpaceNd.cpp:86-116` restated with numpy indexing; uncropped cases are one six-dimensional walk."""
    ib, ih, iw, c = dims
    rank = 3 if iw is None else 4
    shape = ((ib, c, ih) if nchw else (ib, ih, c)) if rank == 3 else ((ib, c, ih, iw) if nchw else (ib, ih, iw, c))
    x = np.random.default_rng(3).integers(1, 255, size=shape).astype(np.uint8)
    x4 = _to_nhwc4(x, nchw)
    bh, bw = block[0], (block[1] if rank == 4 else 1)
    (ct, cb), (cl, cr) = edges[0], (edges[1] if rank == 4 else (0, 0))
    ob = ib // (bh * bw)
    want = np.zeros((ob, x4.shape[1] * bh - ct - cb, x4.shape[2] * bw - cl - cr, c), np.uint8)
    for b in range(ib):
        so = b // ob
        for h in range(x4.shape[1]):
            for w in range(x4.shape[2]):
                y, xx = h * bh + so // bw - ct, w * bw + so % bw - cl
                if 0 <= y < want.shape[1] and 0 <= xx < want.shape[2]:
                    want[b % ob, y, xx] = x4[b, h, w]
    want = _from_nhwc4(want, rank, nchw)
    out_shape, vs = V.batch_to_space_views(shape, block, edges, nchw)
    assert tuple(out_shape) == want.shape
    assert len(vs) == 1 or any(a or b for a, b in edges)
    got = np.zeros(out_shape, np.uint8)
    for v in vs:
        apply_view(x, got, V.merge_dims(v))
    assert np.array_equal(got, want)


@pytest.mark.parametrize("nchw", [False, True])
@pytest.mark.parametrize("dims,block,edges", [
    ((2, 4, 6, 5), (2, 2), ((0, 0), (0, 0))), ((2, 3, 5, 4), (2, 3), ((1, 2), (3, 1))),
    ((1, 2, 2, 3), (3, 2), ((4, 3), (1, 1))), ((2, 6, None, 5), (3,), ((0, 0),)), ((2, 5, None, 3), (2,), ((1, 2),))])
def test_space_to_batch_views_follow_the_reference_loop(dims, block, edges, nchw):
    """`workloads/SpaceToBatchNd.cpp:82-129` restated with numpy indexing; padding positions keep the fill value."""
    ib, ih, iw, c = dims
    rank = 3 if iw is None else 4
    shape = ((ib, c, ih) if nchw else (ib, ih, c)) if rank == 3 else ((ib, c, ih, iw) if nchw else (ib, ih, iw, c))
    x = np.random.default_rng(4).integers(1, 255, size=shape).astype(np.uint8)
    x4 = _to_nhwc4(x, nchw)
    bh, bw = block[0], (block[1] if rank == 4 else 1)
    (pt, pb), (pl, pr) = edges[0], (edges[1] if rank == 4 else (0, 0))
    oh, ow = (x4.shape[1] + pt + pb) // bh, (x4.shape[2] + pl + pr) // bw
    want = np.zeros((ib * bh * bw, oh, ow, c), np.uint8)
    for b in range(ib * bh * bw):
        sh, sw = (b // ib) // bw, (b // ib) % bw
        for y in range(oh):
            for xx in range(ow):
                h, w = y * bh + sh - pt, xx * bw + sw - pl
                if 0 <= h < x4.shape[1] and 0 <= w < x4.shape[2]:
                    want[b, y, xx] = x4[b % ib, h, w]
    want = _from_nhwc4(want, rank, nchw)
    out_shape, vs, padded = V.space_to_batch_views(shape, block, edges, nchw)
    assert tuple(out_shape) == want.shape and padded == any(a or b for a, b in edges)
    got = np.full(out_shape, 77, np.uint8)
    apply_view(np.zeros(1, np.uint8), got, V.fill_view(out_shape))
    for v in vs:
        apply_view(x, got, V.merge_dims(v))
    assert np.array_equal(got, want)


def test_batch_and_space_views_refuse_shapes_that_do_not_divide():
    with pytest.raises(ValueError):
        V.space_to_batch_views((1, 5, 4, 3), (2, 2), ((0, 0), (0, 0)))          # height 5 is not a multiple of 2
    with pytest.raises(ValueError):
        V.batch_to_space_views((6, 2, 2, 3), (2, 2), ((0, 0), (0, 0)))          # batch 6 is not a multiple of 4
    with pytest.raises(ValueError):
        V.batch_to_space_views((4, 1, 1, 3), (2, 2), ((1, 1), (0, 0)))          # crops leave nothing
    with pytest.raises(ValueError):
        V.batch_to_space_views((4, 2), (2,), ((0, 0),))                         # rank 2


def _move_cases():
    import cases
    return sorted(cases.move_cases().items())


@pytest.mark.parametrize("name,factory", _move_cases(), ids=[n for n, _ in _move_cases()])
def test_views_of_every_data_movement_case_reproduce_the_oracle(built, name, factory):
    """The views the product derives from each descriptor, applied with numpy, against the CPU restatement of the
    reference's loops (cases that re-quantise are covered on the GPU only: the views carry no arithmetic)."""
    case = factory()
    tensors = [case.whole] + list(case.parts)
    if any(t[1:] != tensors[0][1:] for t in tensors):
        pytest.skip("re-quantising case")
    from q8util import Host
    mem = Host()
    whole, parts, outs = case._data(mem)
    want = [o.copy() for o in case.run_oracle()]

    def array(t, spec):
        import ctypes
        from q8util import NP_OF
        n = int(np.prod(spec[0]))
        return np.ctypeslib.as_array(ctypes.cast(t.data, ctypes.POINTER(np.ctypeslib.as_ctypes_type(NP_OF[spec[1]]))), shape=(n,))
    whole_a = array(whole, case.whole)
    part_a = [array(t, spec) for t, spec in zip(parts, case.parts)]
    for view, si, di in case.views():
        src = np.zeros(1, whole_a.dtype) if si == -2 else (whole_a if si < 0 else part_a[si])
        if si == -2:
            src[0] = case.parts[di][3]                  # the zero point: the encoding of 0.0
        dst = whole_a if di < 0 else part_a[di]
        apply_view(src, dst, V.merge_dims(view))
    for w, o in zip(want, outs):
        assert np.array_equal(w, o)
