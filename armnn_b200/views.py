"""Layer descriptors of the data-movement layers -> the rectangular view copies that `b200k_view_copy_q` executes.

Every function returns a list of views `(shape, src_offset, src_strides, dst_offset, dst_strides)` (elements, outermost
dimension first) plus, where the layer defines it, the output shape.  The same arithmetic lives in the plugin
(`backend/B200Workloads.cpp`, the view workloads); this module serves the Python mirror of the runtime API and states the
rules once in a form that is easy to test against CpuRef:

* Concat (`src/backends/reference/workloads/Concatenate.cpp:14-85`) and Splitter (`workloads/Splitter.cpp:18-93`):
  view v of the whole tensor starts at `origin[v]` and has the shape of input / output v.  Where views overlap the
  reference lets the first one win: the copies are issued last view first.
* Permute (`src/armnnUtils/Permute.cpp:22-119`): `mappings[i]` is the destination dimension of source dimension i;
  Transpose (`src/armnnUtils/Transpose.cpp:22-117`): `mappings[i]` is the source dimension of destination dimension i.
* StridedSlice (`src/armnn/Descriptors.cpp:393-453`, `workloads/StridedSlice.cpp:188-222`) with begin / end / shrink-axis
  masks (ellipsis and new-axis masks are refused by layer support); Slice (`workloads/Slice.cpp:14-147`).
* DepthToSpace, SpaceToDepth, ChannelShuffle and Stack: six- or four-dimensional walks over the same bytes.
"""

INT_MIN, INT_MAX = -(1 << 31), (1 << 31) - 1


def dense_strides(shape):
    strides, st = [0] * len(shape), 1
    for d in range(len(shape) - 1, -1, -1):
        strides[d] = st
        st *= int(shape[d])
    return strides


def concat_views(out_shape, in_shapes, origins):
    """One view per input: input v (dense) -> the block of the output at origins[v]."""
    ds = dense_strides(out_shape)
    views = []
    for shape, origin in zip(in_shapes, origins):
        if len(shape) != len(out_shape) or any(o < 0 or o + s > t for o, s, t in zip(origin, shape, out_shape)):
            raise ValueError("Concat: view %s at %s does not fit the output %s" % (shape, origin, out_shape))
        views.append((tuple(shape), 0, dense_strides(shape), sum(o * s for o, s in zip(origin, ds)), ds))
    return list(reversed(views))


def splitter_views(in_shape, out_shapes, origins):
    """One view per output: the block of the input at origins[v] -> output v (dense)."""
    ss = dense_strides(in_shape)
    views = []
    for shape, origin in zip(out_shapes, origins):
        if len(shape) != len(in_shape) or any(o < 0 or o + s > t for o, s, t in zip(origin, shape, in_shape)):
            raise ValueError("Splitter: view %s at %s does not fit the input %s" % (shape, origin, in_shape))
        views.append((tuple(shape), sum(o * s for o, s in zip(origin, ss)), ss, 0, dense_strides(shape)))
    return views


def permute_view(in_shape, mappings, transpose=False):
    """(out_shape, view) of Permute (transpose=False) or Transpose."""
    rank = len(in_shape)
    if sorted(mappings) != list(range(rank)):
        raise ValueError("not a permutation of %d dimensions: %s" % (rank, list(mappings)))
    src_of_dst = list(mappings) if transpose else [0] * rank
    if not transpose:
        for i, m in enumerate(mappings):
            src_of_dst[m] = i
    out_shape = tuple(int(in_shape[src_of_dst[j]]) for j in range(rank))
    ss = dense_strides(in_shape)
    return out_shape, (out_shape, 0, [ss[src_of_dst[j]] for j in range(rank)], 0, dense_strides(out_shape))


def strided_slice_view(in_shape, begin, end, stride, begin_mask=0, end_mask=0, shrink_axis_mask=0):
    """(walk_shape, out_shape, view): walk_shape has one extent per input dimension; out_shape drops the shrunk axes."""
    rank = len(in_shape)
    if not (len(begin) == len(end) == len(stride) == rank):
        raise ValueError("StridedSlice: begin / end / stride must have one entry per input dimension")
    ss = dense_strides(in_shape)
    counts, offset, strides = [], 0, []
    for d in range(rank):
        size, st = int(in_shape[d]), int(stride[d])
        if st == 0:
            raise ValueError("StridedSlice: stride 0")
        b = int(begin[d])
        if begin_mask & (1 << d):
            b = INT_MIN if st > 0 else INT_MAX
        if b < 0:
            b += size
        start = max(0, min(b, size - 1))
        if shrink_axis_mask & (1 << d):
            stop = start + 1
        else:
            e = int(end[d])
            if end_mask & (1 << d):
                e = INT_MAX if st > 0 else INT_MIN
            if e < 0:
                e += size
            stop = max(0, min(e, size)) if st > 0 else max(-1, min(e, size - 1))
        n = max(0, -(-(stop - start) // st)) if st > 0 else max(0, -(-(start - stop) // -st))
        counts.append(n)
        offset += start * ss[d]
        strides.append(ss[d] * st)
    walk = tuple(counts)
    out_shape = tuple(c for d, c in enumerate(counts) if not (shrink_axis_mask & (1 << d))) or (1,)
    return walk, out_shape, (walk, offset, strides, 0, dense_strides(walk))


def slice_view(in_shape, begin, size):
    rank = len(in_shape)
    if not (len(begin) == len(size) == rank) or any(b < 0 or s < 0 or b + s > t for b, s, t in zip(begin, size, in_shape)):
        raise ValueError("Slice: block %s at %s does not fit %s" % (list(size), list(begin), list(in_shape)))
    ss = dense_strides(in_shape)
    out_shape = tuple(int(s) for s in size)
    return out_shape, (out_shape, sum(b * s for b, s in zip(begin, ss)), ss, 0, dense_strides(out_shape))


def depth_to_space_view(in_shape, block, nchw=False):
    """(out_shape, view) of DepthToSpace (`workloads/DepthToSpace.cpp:15-100`): the input read as
    [N, H, W, block, block, C'] (NHWC) or [N, block, block, C', H, W] (NCHW) and permuted to
    [N, H, block, W, block, C'] / [N, C', H, block, W, block]."""
    b = int(block)
    ss = dense_strides(in_shape)
    if nchw:
        n, c, h, w = in_shape
        if b < 1 or c % (b * b):
            raise ValueError("DepthToSpace: %d channels are not a multiple of block size %d squared" % (c, b))
        co = c // (b * b)
        out_shape = (n, co, h * b, w * b)
        # destination order n, c', h, i, w, j; source index ((i * b + j) * co + c') in the channel dimension
        walk = (n, co, h, b, w, b)
        src = [ss[0], ss[1], ss[2], b * co * ss[1], ss[3], co * ss[1]]
    else:
        n, h, w, c = in_shape
        if b < 1 or c % (b * b):
            raise ValueError("DepthToSpace: %d channels are not a multiple of block size %d squared" % (c, b))
        co = c // (b * b)
        out_shape = (n, h * b, w * b, co)
        walk = (n, h, b, w, b, co)
        src = [ss[0], ss[1], b * co, ss[2], co, 1]
    return out_shape, (walk, 0, src, 0, dense_strides(walk))


def space_to_depth_view(in_shape, block, nchw=False):
    """(out_shape, view) of SpaceToDepth (`workloads/SpaceToDepth.cpp:42-104`): output channel oc reads input channel
    oc % C at the spatial offset (oc / C) / block, (oc / C) % block inside the block."""
    b = int(block)
    ss = dense_strides(in_shape)
    if nchw:
        n, c, h, w = in_shape
        if b < 1 or h % b or w % b:
            raise ValueError("SpaceToDepth: %dx%d is not a multiple of block size %d" % (h, w, b))
        out_shape = (n, c * b * b, h // b, w // b)
        walk = (n, b, b, c, h // b, w // b)
        src = [ss[0], ss[2], ss[3], ss[1], b * ss[2], b * ss[3]]
    else:
        n, h, w, c = in_shape
        if b < 1 or h % b or w % b:
            raise ValueError("SpaceToDepth: %dx%d is not a multiple of block size %d" % (h, w, b))
        out_shape = (n, h // b, w // b, c * b * b)
        walk = (n, h // b, w // b, b, b, c)
        src = [ss[0], b * ss[1], b * ss[2], ss[1], ss[2], 1]
    return out_shape, (walk, 0, src, 0, dense_strides(walk))


def channel_shuffle_view(shape, axis, groups):
    """View of ChannelShuffle (`workloads/RefChannelShuffleWorkload.cpp:28-76`): with g groups of s channels, output
    channel i * g + j is input channel i + j * s."""
    rank = len(shape)
    if not (0 <= axis < rank) or groups < 1 or shape[axis] % groups:
        raise ValueError("ChannelShuffle: %d channels cannot be split into %d groups" % (shape[axis], groups))
    size = shape[axis] // groups
    outer = 1
    for d in shape[:axis]:
        outer *= int(d)
    inner = 1
    for d in shape[axis + 1:]:
        inner *= int(d)
    walk = (outer, size, groups, inner)
    return (walk, 0, [shape[axis] * inner, inner, size * inner, 1], 0, dense_strides(walk))


def stack_views(in_shape, num_inputs, axis):
    """(out_shape, views) of Stack (`workloads/Stack.cpp:14-120`): input i becomes index i of a new dimension `axis`."""
    rank = len(in_shape)
    if not (0 <= axis <= rank) or num_inputs < 1:
        raise ValueError("Stack: axis %d outside [0, %d]" % (axis, rank))
    out_shape = tuple(in_shape[:axis]) + (num_inputs,) + tuple(in_shape[axis:])
    os_ = dense_strides(out_shape)
    ds = os_[:axis] + os_[axis + 1:]
    return out_shape, [(tuple(in_shape), 0, dense_strides(in_shape), i * os_[axis], ds) for i in range(num_inputs)]


def merge_dims(view, max_rank=6):
    """Folds neighbouring dimensions that are contiguous on both sides (and drops extents of 1), so that views of any
    rank the layers allow fit the kernel's six dimensions and copies of whole rows become long rows."""
    shape, so, ss, do, ds = view
    dims = [(int(n), int(a), int(b)) for n, a, b in zip(shape, ss, ds) if n != 1]
    merged = []
    for n, a, b in dims:
        if merged and merged[-1][1] == a * n and merged[-1][2] == b * n:
            pn, _, _ = merged[-1]
            merged[-1] = (pn * n, a, b)
        else:
            merged.append((n, a, b))
    if not merged:
        merged = [(1, 1, 1)]
    if len(merged) > max_rank:
        raise ValueError("view of rank %d after merging" % len(merged))
    return (tuple(m[0] for m in merged), so, [m[1] for m in merged], do, [m[2] for m in merged])
