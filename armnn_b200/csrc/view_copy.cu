// View copies: Concat, Splitter, Permute, Transpose, StridedSlice and Slice are all "a rectangular view of one tensor
// onto a rectangular view of another", element by element through Q_y(deq_x(.)) as the reference's Decoder / Encoder
// pair does it (src/backends/reference/workloads/Concatenate.cpp:14-85, Splitter.cpp:18-93) or byte for byte
// (src/armnnUtils/Permute.cpp, Transpose.cpp; workloads/StridedSlice.cpp, Slice.cpp).  Bandwidth kernels:
//   * rows: both views contiguous along the innermost dimension, equal quantisation, everything 16-byte aligned
//     (channel-wise Concat / Splitter of NHWC tensors, Slice of whole pixels): 128-bit loads and stores;
//   * generic: one element per thread, destination-major order (coalesced stores; loads as the source strides allow).
#include "common.cuh"

namespace b200k {

struct ViewArgs {
    QView x, y;
    int rank;
    int shape[6];
    long long ss[6], ds[6];
    long long soff, doff;
    long long count;
    int same;                       // equal type and quantisation: bytes move as they are
    int esize;
};

__global__ void __launch_bounds__(256) view_copy_kernel(const ViewArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.count) return;
    long long rest = i, s = a.soff, d = a.doff;
    #pragma unroll
    for (int k = 5; k >= 0; --k) {
        if (k >= a.rank) continue;
        const long long c = rest % a.shape[k];
        rest /= a.shape[k];
        s += c * a.ss[k];
        d += c * a.ds[k];
    }
    if (a.same) {
        if (a.esize == 1)      ((uint8_t*)a.y.data)[d] = ((const uint8_t*)a.x.data)[s];
        else if (a.esize == 2) ((uint16_t*)a.y.data)[d] = ((const uint16_t*)a.x.data)[s];
        else                   ((uint32_t*)a.y.data)[d] = ((const uint32_t*)a.x.data)[s];
    } else {
        a.y.set(d, a.x.get(s));
    }
}

// rows of `row16` 16-byte words: row r of the view starts at byte offsets sb / db (from the outer coordinates)
struct ViewRowArgs {
    const uint8_t* x; uint8_t* y;
    int rank;                       // outer dimensions
    int shape[6];
    long long ssb[6], dsb[6];       // strides in bytes
    long long rows;
    int row16;
};

__global__ void __launch_bounds__(256) view_rows_kernel(const ViewRowArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.rows * a.row16) return;
    long long rest = i / a.row16;
    const int w = (int)(i - rest * a.row16);
    long long s = 0, d = 0;
    #pragma unroll
    for (int k = 5; k >= 0; --k) {
        if (k >= a.rank) continue;
        const long long c = rest % a.shape[k];
        rest /= a.shape[k];
        s += c * a.ssb[k];
        d += c * a.dsb[k];
    }
    ((uint4*)(a.y + d))[w] = ((const uint4*)(a.x + s))[w];
}

// Gather (src/backends/reference/workloads/Gather.cpp:16-94): y[o, j, k] = Q_y(deq_x(x[o, indices[j], k])); a negative
// index counts from the end of the axis.  The reference throws on an index outside the axis; here such an index reads
// nothing and stores the encoding of 0.0.
struct GatherArgs {
    QView x, y;
    const int* indices;
    long long axis, inner, n_idx, count;
    int same, esize;
    int nd;                         // 0: one index per row (Gather); else index tuples of nd entries (GatherNd)
    long long coeff[8];             // GatherNd: the row number is sum_d tuple[d] * coeff[d]
};

__global__ void __launch_bounds__(256) gather_kernel(const GatherArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.count) return;
    const long long k = i % a.inner, oj = i / a.inner;
    const long long j = oj % a.n_idx, o = oj / a.n_idx;
    long long idx;
    if (a.nd == 0) {
        idx = a.indices[j];
        if (idx < 0) idx += a.axis;
    } else {
        idx = 0;
        bool ok = true;
        for (int d = 0; d < a.nd; ++d) {
            const long long t = a.indices[j * a.nd + d];
            ok = ok && t >= 0;
            idx += t * a.coeff[d];
        }
        if (!ok) idx = -1;
    }
    if (idx < 0 || idx >= a.axis) { a.y.set(i, 0.0f); return; }
    const long long s = (o * a.axis + idx) * a.inner + k;
    if (a.same) {
        if (a.esize == 1)      ((uint8_t*)a.y.data)[i] = ((const uint8_t*)a.x.data)[s];
        else if (a.esize == 2) ((uint16_t*)a.y.data)[i] = ((const uint16_t*)a.x.data)[s];
        else                   ((uint32_t*)a.y.data)[i] = ((const uint32_t*)a.x.data)[s];
    } else {
        a.y.set(i, a.x.get(s));
    }
}

// rows of whole 16-byte words (an embedding table with equal quantisation on both sides)
struct GatherRowArgs { const uint8_t* x; uint8_t* y; const int* indices; long long axis, n_idx, rows; int row16; };

__global__ void __launch_bounds__(256) gather_rows_kernel(const GatherRowArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.rows * a.row16) return;
    const long long r = i / a.row16;
    const int w = (int)(i - r * a.row16);
    const long long j = r % a.n_idx, o = r / a.n_idx;
    long long idx = a.indices[j];
    if (idx < 0) idx += a.axis;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (idx >= 0 && idx < a.axis) v = ((const uint4*)a.x)[((o * a.axis + idx) * a.row16) + w];
    ((uint4*)a.y)[i] = v;
}

// ReverseV2 (src/backends/reference/workloads/ReverseV2Impl.cpp:14-133): the axes are a run-time tensor, so the flip flags
// are read on the device; element i of the input goes to the position with the flagged coordinates mirrored.
struct ReverseArgs { QView x, y; const int* axes; int n_axes, rank; int shape[6]; long long count; int same, esize; };

__global__ void __launch_bounds__(256) reverse_kernel(const ReverseArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.count) return;
    unsigned flags = 0;
    for (int k = 0; k < a.n_axes; ++k) {
        int ax = a.axes[k];
        if (ax < 0) ax += a.rank;
        if (ax >= 0 && ax < a.rank) flags |= 1u << ax;
    }
    long long rest = i, dst = 0, stride = 1;
    #pragma unroll
    for (int d = 5; d >= 0; --d) {
        if (d >= a.rank) continue;
        long long c = rest % a.shape[d];
        rest /= a.shape[d];
        if (flags & (1u << d)) c = a.shape[d] - 1 - c;
        dst += c * stride;
        stride *= a.shape[d];
    }
    if (a.same) {
        if (a.esize == 1)      ((uint8_t*)a.y.data)[dst] = ((const uint8_t*)a.x.data)[i];
        else if (a.esize == 2) ((uint16_t*)a.y.data)[dst] = ((const uint16_t*)a.x.data)[i];
        else                   ((uint32_t*)a.y.data)[dst] = ((const uint32_t*)a.x.data)[i];
    } else {
        a.y.set(dst, a.x.get(i));
    }
}

// ScatterNd (src/backends/reference/workloads/ScatterNd.cpp:37-333): the output starts as the input (or as zeros when the
// layer is given a shape instead), then every index tuple j replaces its slice by op(base slice, updates[j]) where the
// base is the INPUT (not the running output): with tuples that address one slice the last one wins.  The reference works
// through the tuples in order; here a tuple that a later one repeats does nothing, which is the same result.
struct ScatterArgs {
    QView x, upd, y;
    const int* indices;
    int has_x, nd, fn;
    long long n_idx, inner, total;
    long long coeff[8], dims[8];
};

__global__ void __launch_bounds__(256) scatter_init_kernel(const ScatterArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    a.y.set(i, a.has_x ? a.x.get(i) : 0.0f);
}

__device__ __forceinline__ long long scatter_row(const ScatterArgs& a, long long j)
{
    long long flat = 0;
    for (int d = 0; d < a.nd; ++d) {
        const long long t = a.indices[j * a.nd + d];
        if (t < 0 || t >= a.dims[d]) return -1;              // the reference throws; here the tuple is skipped
        flat += t * a.coeff[d];
    }
    return flat;
}

__global__ void __launch_bounds__(256) scatter_kernel(const ScatterArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.n_idx * a.inner) return;
    const long long j = i / a.inner, k = i - j * a.inner;
    const long long row = scatter_row(a, j);
    if (row < 0) return;
    for (long long j2 = j + 1; j2 < a.n_idx; ++j2)
        if (scatter_row(a, j2) == row) return;               // a later tuple addresses the same slice: it wins
    const long long at = row * a.inner + k;
    const float base = a.has_x ? a.x.get(at) : 0.0f;
    const float u = a.upd.get(i);
    float r;
    switch (a.fn) {
        case 0:  r = u; break;
        case 1:  r = __fadd_rn(base, u); break;
        case 2:  r = __fsub_rn(base, u); break;
        case 3:  r = base < u ? u : base; break;             // std::max(input, update)
        case 4:  r = u < base ? u : base; break;             // std::min(input, update)
        default: r = __fmul_rn(base, u); break;
    }
    a.y.set(at, r);
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_scatter_nd_q(const b200k_scatter_nd_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "scatter_nd_q: null params");
    B200K_REQUIRE(p->updates.data && p->y.data && p->indices, B200K_E_INVALID, "scatter_nd_q: null tensor pointer");
    B200K_REQUIRE(p->nd >= 1 && p->nd <= 8 && p->n_indices > 0 && p->inner > 0, B200K_E_INVALID, "scatter_nd_q: bad shape");
    B200K_REQUIRE(p->function >= 0 && p->function <= 5, B200K_E_INVALID, "scatter_nd_q: unknown function %d", p->function);
    auto ok = [](int t) { return t == B200K_U8 || t == B200K_S8 || t == B200K_S16 || t == B200K_F32; };
    B200K_REQUIRE(ok(p->updates.dtype) && ok(p->y.dtype) && (!p->x.data || ok(p->x.dtype)), B200K_E_UNSUPPORTED, "scatter_nd_q: unsupported data type");
    ScatterArgs a;
    memset(&a, 0, sizeof(a));
    a.has_x = p->x.data != nullptr;
    if (a.has_x) a.x = make_view(p->x);
    a.upd = make_view(p->updates); a.y = make_view(p->y); a.indices = p->indices;
    a.nd = p->nd; a.fn = p->function; a.n_idx = p->n_indices; a.inner = p->inner;
    long long rows = 1;
    for (int d = p->nd - 1; d >= 0; --d) {
        B200K_REQUIRE(p->dims[d] > 0, B200K_E_INVALID, "scatter_nd_q: non-positive dimension");
        a.dims[d] = p->dims[d]; a.coeff[d] = rows; rows *= p->dims[d];
    }
    a.total = rows * p->inner;
    cudaStream_t s = (cudaStream_t)stream;
    launch_pdl(scatter_init_kernel, dim3(div_up(a.total, 256)), dim3(256), 0, s, a);
    int rc = check_launch("scatter_init_kernel");
    if (rc != B200K_OK) return rc;
    launch_pdl(scatter_kernel, dim3(div_up(a.n_idx * a.inner, 256)), dim3(256), 0, s, a);
    return check_launch("scatter_kernel");
}

extern "C" int b200k_reverse_q(const b200k_reverse_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "reverse_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data && (p->axes || p->n_axes == 0), B200K_E_INVALID, "reverse_q: null tensor pointer");
    B200K_REQUIRE(p->rank >= 1 && p->rank <= 6 && p->n_axes >= 0, B200K_E_UNSUPPORTED, "reverse_q: rank %d not in [1, 6]", p->rank);
    B200K_REQUIRE(p->x.dtype >= B200K_U8 && p->x.dtype <= B200K_F32 && p->x.dtype == p->y.dtype, B200K_E_UNSUPPORTED,
                  "reverse_q: one supported element type for input and output");
    ReverseArgs a;
    memset(&a, 0, sizeof(a));
    a.x = make_view(p->x); a.y = make_view(p->y); a.axes = p->axes; a.n_axes = p->n_axes; a.rank = p->rank;
    a.count = 1;
    for (int d = 0; d < p->rank; ++d) {
        B200K_REQUIRE(p->shape[d] >= 0, B200K_E_INVALID, "reverse_q: negative extent");
        a.shape[d] = p->shape[d];
        a.count *= p->shape[d];
    }
    if (a.count == 0) return B200K_OK;
    const bool quantised = p->x.dtype == B200K_U8 || p->x.dtype == B200K_S8 || p->x.dtype == B200K_S16;
    a.same = (!quantised || (p->x.scale == p->y.scale && p->x.zero_point == p->y.zero_point)) ? 1 : 0;
    a.esize = elem_size(p->x.dtype);
    launch_pdl(reverse_kernel, dim3(div_up(a.count, 256)), dim3(256), 0, (cudaStream_t)stream, a);
    return check_launch("reverse_kernel");
}

extern "C" int b200k_gather_q(const b200k_gather_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "gather_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data && p->indices, B200K_E_INVALID, "gather_q: null tensor pointer");
    B200K_REQUIRE(p->outer > 0 && p->axis_size > 0 && p->inner > 0 && p->n_indices >= 0, B200K_E_INVALID, "gather_q: bad shape");
    B200K_REQUIRE(p->x.dtype >= B200K_U8 && p->x.dtype <= B200K_F32, B200K_E_INVALID, "gather_q: unknown element type");
    B200K_REQUIRE(p->x.dtype == p->y.dtype, B200K_E_UNSUPPORTED, "gather_q: input and output types differ (%d, %d)", p->x.dtype, p->y.dtype);
    const long long count = (long long)p->outer * p->n_indices * p->inner;
    if (count == 0) return B200K_OK;
    const bool quantised = p->x.dtype == B200K_U8 || p->x.dtype == B200K_S8 || p->x.dtype == B200K_S16;
    const bool same = !quantised || (p->x.scale == p->y.scale && p->x.zero_point == p->y.zero_point);
    const int es = elem_size(p->x.dtype);
    cudaStream_t s = (cudaStream_t)stream;
    const long long row_bytes = (long long)p->inner * es;
    // the zero fill of an out-of-range index is only the encoding of 0.0 when the zero point is 0
    if (same && row_bytes % 16 == 0 && (uintptr_t)p->x.data % 16 == 0 && (uintptr_t)p->y.data % 16 == 0 &&
        (!quantised || p->y.zero_point == 0) && row_bytes / 16 <= 0x7fffffff) {
        GatherRowArgs a;
        a.x = (const uint8_t*)p->x.data; a.y = (uint8_t*)p->y.data; a.indices = p->indices;
        a.axis = p->axis_size; a.n_idx = p->n_indices; a.rows = (long long)p->outer * p->n_indices;
        a.row16 = (int)(row_bytes / 16);
        launch_pdl(gather_rows_kernel, dim3(div_up(a.rows * a.row16, 256)), dim3(256), 0, s, a);
        return check_launch("gather_rows_kernel");
    }
    GatherArgs a;
    memset(&a, 0, sizeof(a));
    a.x = make_view(p->x); a.y = make_view(p->y); a.indices = p->indices;
    a.axis = p->axis_size; a.inner = p->inner; a.n_idx = p->n_indices; a.count = count;
    a.same = same ? 1 : 0; a.esize = es;
    launch_pdl(gather_kernel, dim3(div_up(count, 256)), dim3(256), 0, s, a);
    return check_launch("gather_kernel");
}

extern "C" int b200k_view_copy_q(const b200k_view_copy_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "view_copy_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "view_copy_q: null tensor pointer");
    B200K_REQUIRE(p->rank >= 1 && p->rank <= 6, B200K_E_UNSUPPORTED, "view_copy_q: rank %d not in [1, 6]", p->rank);
    B200K_REQUIRE(p->x.dtype >= B200K_U8 && p->x.dtype <= B200K_F32 && p->y.dtype >= B200K_U8 && p->y.dtype <= B200K_F32,
                  B200K_E_INVALID, "view_copy_q: unknown element type");
    B200K_REQUIRE(p->x.dtype == p->y.dtype, B200K_E_UNSUPPORTED, "view_copy_q: input and output types differ (%d, %d)",
                  p->x.dtype, p->y.dtype);
    B200K_REQUIRE(p->src_offset >= 0 && p->dst_offset >= 0, B200K_E_INVALID, "view_copy_q: negative offset");
    long long count = 1;
    for (int d = 0; d < p->rank; ++d) {
        B200K_REQUIRE(p->shape[d] >= 0, B200K_E_INVALID, "view_copy_q: negative extent");
        count *= p->shape[d];
    }
    if (count == 0) return B200K_OK;                       // an empty view: nothing to copy
    const bool quantised = p->x.dtype == B200K_U8 || p->x.dtype == B200K_S8 || p->x.dtype == B200K_S16;
    const bool same = !quantised || (p->x.scale == p->y.scale && p->x.zero_point == p->y.zero_point);
    const int es = elem_size(p->x.dtype);
    cudaStream_t s = (cudaStream_t)stream;

    // rows: innermost dimension contiguous on both sides and a whole number of aligned 16-byte words
    const int in = p->rank - 1;
    const long long row_bytes = (long long)p->shape[in] * es;
    bool rows = same && p->src_strides[in] == 1 && p->dst_strides[in] == 1 && row_bytes % 16 == 0 &&
                ((uintptr_t)p->x.data + (uintptr_t)(p->src_offset * es)) % 16 == 0 &&
                ((uintptr_t)p->y.data + (uintptr_t)(p->dst_offset * es)) % 16 == 0 && row_bytes / 16 <= 0x7fffffff;
    for (int d = 0; d < in && rows; ++d)
        rows = (p->src_strides[d] * es) % 16 == 0 && (p->dst_strides[d] * es) % 16 == 0;
    if (rows) {
        ViewRowArgs a;
        memset(&a, 0, sizeof(a));
        a.x = (const uint8_t*)p->x.data + p->src_offset * es;
        a.y = (uint8_t*)p->y.data + p->dst_offset * es;
        a.rank = in;
        a.rows = 1;
        for (int d = 0; d < in; ++d) {
            a.shape[d] = p->shape[d]; a.ssb[d] = p->src_strides[d] * es; a.dsb[d] = p->dst_strides[d] * es;
            a.rows *= p->shape[d];
        }
        a.row16 = (int)(row_bytes / 16);
        launch_pdl(view_rows_kernel, dim3(div_up(a.rows * a.row16, 256)), dim3(256), 0, s, a);
        return check_launch("view_rows_kernel");
    }
    ViewArgs a;
    memset(&a, 0, sizeof(a));
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.rank = p->rank; a.count = count; a.same = same ? 1 : 0; a.esize = es;
    a.soff = p->src_offset; a.doff = p->dst_offset;
    for (int d = 0; d < p->rank; ++d) { a.shape[d] = p->shape[d]; a.ss[d] = p->src_strides[d]; a.ds[d] = p->dst_strides[d]; }
    launch_pdl(view_copy_kernel, dim3(div_up(count, 256)), dim3(256), 0, s, a);
    return check_launch("view_copy_kernel");
}

// GatherNd (src/backends/reference/workloads/RefGatherNdWorkload.cpp:20-92): the index tuples are flattened to row numbers
// of the tensor seen as [rows, inner] and the rows gathered.
extern "C" int b200k_gather_nd_q(const b200k_gather_nd_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "gather_nd_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data && p->indices, B200K_E_INVALID, "gather_nd_q: null tensor pointer");
    B200K_REQUIRE(p->nd >= 1 && p->nd <= 8 && p->n_indices >= 0 && p->inner > 0, B200K_E_INVALID, "gather_nd_q: bad shape");
    B200K_REQUIRE(p->x.dtype >= B200K_U8 && p->x.dtype <= B200K_F32, B200K_E_INVALID, "gather_nd_q: unknown element type");
    B200K_REQUIRE(p->x.dtype == p->y.dtype, B200K_E_UNSUPPORTED, "gather_nd_q: input and output types differ (%d, %d)", p->x.dtype, p->y.dtype);
    const long long count = (long long)p->n_indices * p->inner;
    if (count == 0) return B200K_OK;
    GatherArgs a;
    memset(&a, 0, sizeof(a));
    a.x = make_view(p->x); a.y = make_view(p->y); a.indices = p->indices;
    a.inner = p->inner; a.n_idx = p->n_indices; a.count = count; a.nd = p->nd;
    a.axis = 1;
    for (int d = 0; d < p->nd; ++d) {
        B200K_REQUIRE(p->dims[d] > 0, B200K_E_INVALID, "gather_nd_q: non-positive dimension");
        a.axis *= p->dims[d];
    }
    long long c = 1;
    for (int d = p->nd - 1; d >= 0; --d) { a.coeff[d] = c; c *= p->dims[d]; }
    const bool quantised = p->x.dtype == B200K_U8 || p->x.dtype == B200K_S8 || p->x.dtype == B200K_S16;
    a.same = (!quantised || (p->x.scale == p->y.scale && p->x.zero_point == p->y.zero_point)) ? 1 : 0;
    a.esize = elem_size(p->x.dtype);
    launch_pdl(gather_kernel, dim3(div_up(count, 256)), dim3(256), 0, (cudaStream_t)stream, a);
    return check_launch("gather_kernel");
}
