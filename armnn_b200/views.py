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
* BatchToSpaceNd (`workloads/BatchToSpaceNd.cpp:50-117`) and SpaceToBatchNd (`workloads/SpaceToBatchNd.cpp:49-131`): one
  strided block per position inside the spatial block; one six-dimensional walk when nothing is cropped or padded.
* Tile and BroadcastTo: repeated dimensions read with source stride 0.
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


def _spatial(shape, nchw):
    """(batch, height, width, channels) and the index of each in `shape` (rank 3: no width; rank 4)."""
    rank = len(shape)
    if rank == 4:
        idx = (0, 2, 3, 1) if nchw else (0, 1, 2, 3)
    elif rank == 3:
        idx = (0, 2, None, 1) if nchw else (0, 1, None, 2)
    else:
        raise ValueError("rank %d: BatchToSpaceNd / SpaceToBatchNd take 3 or 4 dimensions" % rank)
    dims = tuple(1 if i is None else int(shape[i]) for i in idx)
    return dims, idx


def _shape_from(idx, rank, b, h, w, c):
    out = [0] * rank
    for i, v in zip(idx, (b, h, w, c)):
        if i is not None:
            out[i] = v
    return tuple(out)


def _span(lo_num, hi_num, block, limit):
    """Indices n in [0, limit) with lo_num <= n * block <= hi_num: (first, count)."""
    first = max(0, -(-lo_num // block))
    last = min(limit - 1, hi_num // block)
    return first, max(0, last - first + 1)


def batch_to_space_views(in_shape, block, crops, nchw=False):
    """(out_shape, views) of BatchToSpaceNd: input batch (i * block_w + j) * out_batch + b holds, for output batch b,
    the pixels (y * block_h + i - crop_top, x * block_w + j - crop_left).  block: one entry per spatial dimension;
    crops: (before, after) per spatial dimension."""
    (ib, ih, iw, c), idx = _spatial(in_shape, nchw)
    rank = len(in_shape)
    block, crops = [int(v) for v in block], [(int(a), int(b)) for a, b in crops]
    if len(block) != rank - 2 or len(crops) != rank - 2 or any(v < 1 for v in block) or any(a < 0 or b < 0 for a, b in crops):
        raise ValueError("BatchToSpaceNd: block shape / crops do not match a tensor of rank %d" % rank)
    bh, (ct, cb) = block[0], crops[0]
    bw, (cl, cr) = (block[1], crops[1]) if rank == 4 else (1, (0, 0))
    if ib % (bh * bw):
        raise ValueError("BatchToSpaceNd: batch %d is not a multiple of the block size %d" % (ib, bh * bw))
    ob, oh, ow = ib // (bh * bw), ih * bh - ct - cb, iw * bw - cl - cr
    if oh < 1 or ow < 1:
        raise ValueError("BatchToSpaceNd: the crops leave nothing")
    out_shape = _shape_from(idx, rank, ob, oh, ow, c)
    ss4, ds4 = dense_strides(in_shape), dense_strides(out_shape)
    pick = lambda st: [0 if i is None else st[i] for i in idx]          # strides as (batch, height, width, channel)
    (sb, sh, sw, sc), (db, dh, dw, dc) = pick(ss4), pick(ds4)
    order = (0, 3, 1, 2) if nchw else (0, 1, 2, 3)                      # walk in the destination's memory order
    def arrange(vals):
        return [vals[k] for k in order]
    if not (ct or cb or cl or cr):
        # [ob, ih, bh, iw, bw, c] (NHWC) / [ob, c, ih, bh, iw, bw] (NCHW) over the dense output
        walk = {"b": (ob, sb, db), "h": (ih, sh, dh * bh), "i": (bh, bw * ob * sb, dh), "w": (iw, sw, dw * bw),
                "j": (bw, ob * sb, dw), "c": (c, sc, dc)}
        keys = "bchiwj" if nchw else "bhiwjc"
        return out_shape, [(tuple(walk[k][0] for k in keys), 0, [walk[k][1] for k in keys], 0, [walk[k][2] for k in keys])]
    out = []
    for i in range(bh):
        h0, nh = _span(ct - i, oh - 1 + ct - i, bh, ih)
        for j in range(bw):
            w0, nw = _span(cl - j, ow - 1 + cl - j, bw, iw)
            if nh == 0 or nw == 0:
                continue
            out.append((tuple(arrange([ob, nh, nw, c])), (i * bw + j) * ob * sb + h0 * sh + w0 * sw, arrange([sb, sh, sw, sc]),
                        (h0 * bh + i - ct) * dh + (w0 * bw + j - cl) * dw, arrange([db, dh * bh, dw * bw, dc])))
    return out_shape, out


def space_to_batch_views(in_shape, block, pads, nchw=False):
    """(out_shape, views, padded) of SpaceToBatchNd: output batch (i * block_w + j) * in_batch + b holds, for input
    batch b, the pixels (y * block_h + i - pad_top, x * block_w + j - pad_left); positions outside the input hold
    Q(0), which the caller writes first when `padded` is set."""
    (ib, ih, iw, c), idx = _spatial(in_shape, nchw)
    rank = len(in_shape)
    block, pads = [int(v) for v in block], [(int(a), int(b)) for a, b in pads]
    if len(block) != rank - 2 or len(pads) != rank - 2 or any(v < 1 for v in block) or any(a < 0 or b < 0 for a, b in pads):
        raise ValueError("SpaceToBatchNd: block shape / padding do not match a tensor of rank %d" % rank)
    bh, (pt, pb) = block[0], pads[0]
    bw, (pl, pr) = (block[1], pads[1]) if rank == 4 else (1, (0, 0))
    if (ih + pt + pb) % bh or (iw + pl + pr) % bw:
        raise ValueError("SpaceToBatchNd: the padded size %dx%d is not a multiple of the block %dx%d"
                         % (ih + pt + pb, iw + pl + pr, bh, bw))
    oh, ow = (ih + pt + pb) // bh, (iw + pl + pr) // bw
    out_shape = _shape_from(idx, rank, ib * bh * bw, oh, ow, c)
    ss4, ds4 = dense_strides(in_shape), dense_strides(out_shape)
    pick = lambda st: [0 if i is None else st[i] for i in idx]
    (sb, sh, sw, sc), (db, dh, dw, dc) = pick(ss4), pick(ds4)
    order = (0, 3, 1, 2) if nchw else (0, 1, 2, 3)
    def arrange(vals):
        return [vals[k] for k in order]
    out = []
    for i in range(bh):
        h0, nh = _span(pt - i, ih - 1 + pt - i, bh, oh)
        for j in range(bw):
            w0, nw = _span(pl - j, iw - 1 + pl - j, bw, ow)
            if nh == 0 or nw == 0:
                continue
            out.append((tuple(arrange([ib, nh, nw, c])), (h0 * bh + i - pt) * sh + (w0 * bw + j - pl) * sw,
                        arrange([sb, sh * bh, sw * bw, sc]),
                        (i * bw + j) * ib * db + h0 * dh + w0 * dw, arrange([db, dh, dw, dc])))
    return out_shape, out, bool(pt or pb or pl or pr)


def tile_view(in_shape, multiples):
    """(out_shape, view) of Tile (`workloads/Tile.cpp:47-103`): output coordinate o reads input coordinate o % size in
    every dimension: each dimension becomes a (repeat, size) pair whose repeat part has source stride 0."""
    if len(multiples) != len(in_shape) or any(int(m) < 1 for m in multiples):
        raise ValueError("Tile: one positive multiple per dimension")
    out_shape = tuple(int(n) * int(m) for n, m in zip(in_shape, multiples))
    ss, ds = dense_strides(in_shape), dense_strides(out_shape)
    shape, src, dst = [], [], []
    for n, m, a, b in zip(in_shape, multiples, ss, ds):
        shape += [int(m), int(n)]
        src += [0, a]
        dst += [int(n) * b, b]
    return out_shape, (tuple(shape), 0, src, 0, dst)


def broadcast_to_view(in_shape, out_shape):
    """View of BroadcastTo (`workloads/RefBroadcastToWorkload.cpp:29-44`): the input aligned to the innermost dimensions
    of the output, dimensions of extent 1 (or absent) repeated with source stride 0."""
    if len(in_shape) > len(out_shape):
        raise ValueError("BroadcastTo: the input has more dimensions than the output")
    padded = (1,) * (len(out_shape) - len(in_shape)) + tuple(int(n) for n in in_shape)
    if any(a != b and a != 1 for a, b in zip(padded, out_shape)):
        raise ValueError("BroadcastTo: %s cannot be broadcast to %s" % (list(in_shape), list(out_shape)))
    ss = dense_strides(padded)
    return (tuple(int(n) for n in out_shape), 0, [0 if a == 1 else st for a, st in zip(padded, ss)], 0, dense_strides(out_shape))


def fill_view(shape):
    """The whole dense tensor read from one element (all source strides 0): a constant fill."""
    return (tuple(int(n) for n in shape), 0, [0] * len(shape), 0, dense_strides(shape))


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
