// Layout-agnostic quantised matrix product on CUDA cores: the fallback of BatchMatMul (whose default is the
// tensor-core kernel of bmm_mma.cu) and FullyConnected with non-transposed ([K, N]) weights.  16 x 16 output tile per
// CTA, operands staged through shared memory as zero-point-corrected ints.
#include <string.h>
#include <atomic>
#include "common.cuh"

namespace b200k {

int launch_conv_dp4a(const b200k_conv2d_params* p, cudaStream_t stream);
int conv2d_dispatch(const b200k_conv2d_params* p, cudaStream_t stream);
bool conv_tc_eligible(const b200k_conv2d_params* p);
bool fc_stream_eligible(const b200k_fc_params* p);
bool bmm_mma_eligible(const b200k_bmm_params* p);
int launch_bmm_mma(const b200k_bmm_params* p, cudaStream_t stream);
int launch_fc_stream(const b200k_fc_params* p, cudaStream_t stream);

struct BmmArgs {
    const void* x; const void* y; void* out; int32_t* acc_out;
    const int32_t* bias; const float* w_scales; const float* b_scales;
    float w_scale, b_scale;
    int x_dtype, y_dtype, out_dtype;
    int zx, zy;
    int B, M, K, N;
    long long xs_m, xs_k, ys_k, ys_n;      // element strides
    long long bsx, bsy;
    Requant rq;
};

__global__ void __launch_bounds__(256) bmm_generic_kernel(const BmmArgs a)
{
    __shared__ int xs[16][17];
    __shared__ int ys[16][17];
    const int b = blockIdx.z;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m = blockIdx.y * 16 + ty, n = blockIdx.x * 16 + tx;
    const long long xo = b * a.bsx, yo = b * a.bsy;
    int acc = 0;
    for (int k0 = 0; k0 < a.K; k0 += 16) {
        // xs[ty][tx] = x[m, k0 + tx];  ys[ty][tx] = y[k0 + ty, n]
        int kx = k0 + tx, ky = k0 + ty;
        xs[ty][tx] = (m < a.M && kx < a.K) ? load_q_dev(a.x, a.x_dtype, xo + m * a.xs_m + kx * a.xs_k) - a.zx : 0;
        ys[ty][tx] = (n < a.N && ky < a.K) ? load_q_dev(a.y, a.y_dtype, yo + ky * a.ys_k + n * a.ys_n) - a.zy : 0;
        __syncthreads();
        #pragma unroll
        for (int k = 0; k < 16; ++k) acc += xs[ty][k] * ys[k][tx];
        __syncthreads();
    }
    if (m < a.M && n < a.N) {
        const long long oi = ((long long)b * a.M + m) * a.N + n;
        if (a.acc_out) a.acc_out[oi] = acc;
        const float swc = a.w_scales ? a.w_scales[n] : a.w_scale;
        const float sbc = a.b_scales ? a.b_scales[n] : a.b_scale;
        const int bq = a.bias ? a.bias[n] : 0;
        store_q_dev(a.out, a.out_dtype, oi, a.rq(acc, swc, a.bias != nullptr, bq, sbc));
    }
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_batch_matmul_q8(const b200k_bmm_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "batch_matmul_q8: null params");
    B200K_REQUIRE(p->x.data && p->y.data && p->out.data, B200K_E_INVALID, "batch_matmul_q8: null tensor pointer");
    B200K_REQUIRE(is_q8(p->x.dtype) && is_q8(p->y.dtype) && is_q8(p->out.dtype), B200K_E_UNSUPPORTED,
                  "batch_matmul_q8: only 8-bit quantised tensors are supported");
    B200K_REQUIRE(p->batch > 0 && p->m > 0 && p->k > 0 && p->n > 0, B200K_E_INVALID, "batch_matmul_q8: bad shape");
    B200K_REQUIRE(p->batch <= 65535, B200K_E_TOOBIG, "batch_matmul_q8: batch %d > 65535", p->batch);
    B200K_REQUIRE(p->algo == 0 || p->algo == 1, B200K_E_INVALID, "batch_matmul_q8: algo %d not in {0,1}", p->algo);
    if (p->algo == 0 && bmm_mma_eligible(p)) return launch_bmm_mma(p, (cudaStream_t)stream);
    BmmArgs a;
    a.x = p->x.data; a.y = p->y.data; a.out = (void*)p->out.data; a.acc_out = p->acc_out;
    a.bias = nullptr; a.w_scales = nullptr; a.b_scales = nullptr; a.w_scale = p->y.scale; a.b_scale = 0.f;
    a.x_dtype = p->x.dtype; a.y_dtype = p->y.dtype; a.out_dtype = p->out.dtype;
    a.zx = p->x.zero_point; a.zy = p->y.zero_point;
    a.B = p->batch; a.M = p->m; a.K = p->k; a.N = p->n;
    a.xs_m = p->transpose_x ? 1 : p->k;  a.xs_k = p->transpose_x ? p->m : 1;
    a.ys_k = p->transpose_y ? 1 : p->n;  a.ys_n = p->transpose_y ? p->k : 1;
    a.bsx = p->batch_stride_x; a.bsy = p->batch_stride_y;
    int lo, hi;
    type_range(p->out.dtype, lo, hi);
    a.rq = make_requant(p->x.scale, p->out, lo, hi);
    dim3 grid(div_up(p->n, 16), div_up(p->m, 16), p->batch);
    bmm_generic_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    return check_launch("bmm_generic_kernel");
}

// ---- FullyConnected with [N, K] weights that the tcgen05 kernel cannot take (N not a multiple of 16: classifier heads)
//
// A block owns FC_COLS output columns (one per warp) and FC_ROWS (4, 16 or 32: the smallest that covers M) rows of x, which it stages in shared memory once.
// A warp streams its weight row through registers 16 bytes per lane at a time and multiplies it with every staged row
// (dp4a); the per-lane partial sums of the FC_ROWS rows are then reduced across the warp so that lane r ends up with
// row r, applies the zero-point terms  sum (x - zx)(w - zw) = sum x w - zw sum x - zx sum w + K zx zw  and the
// requantisation, and stores one byte.
constexpr int FC_COLS = 8, FC_KT = 2048;              // rows per block: 4, 16 or 32 (template parameter)

struct FcRowsArgs {
    const uint8_t* x; const uint8_t* w; const int32_t* bias; uint8_t* y; int32_t* acc_out;
    const float* w_scales; const float* b_scales;
    float w_scale, b_scale;
    int zx, zw, M, K, N;
    Requant rq;
    float inv_sy, lo, hi;
};

template <bool XU, bool WU, int FC_ROWS>
__global__ void __launch_bounds__(32 * FC_COLS) fc_rows_kernel(const FcRowsArgs a)
{
    pdl_enter();
    extern __shared__ uint4 s_x[];                           // [FC_ROWS][kt / 16]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * FC_COLS + warp;
    const int m0 = blockIdx.y * FC_ROWS;
    const int rows = min(FC_ROWS, a.M - m0);
    int acc[FC_ROWS], xs[FC_ROWS];
    #pragma unroll
    for (int r = 0; r < FC_ROWS; ++r) { acc[r] = 0; xs[r] = 0; }
    int wsum = 0;
    for (int k0 = 0; k0 < a.K; k0 += FC_KT) {
        const int kt = min(FC_KT, a.K - k0), kv = kt / 16;
        __syncthreads();
        for (int i = threadIdx.x; i < FC_ROWS * kv; i += 32 * FC_COLS) {
            const int r = i / kv, c = i - r * kv;
            s_x[i] = r < rows ? *(const uint4*)(a.x + (long long)(m0 + r) * a.K + k0 + c * 16) : make_uint4(0, 0, 0, 0);
        }
        __syncthreads();
        if (n < a.N) {
            for (int c = lane; c < kv; c += 32) {
                const uint4 wv = *(const uint4*)(a.w + (long long)n * a.K + k0 + c * 16);
                wsum = dp4a_mixed<WU, true>(wv.x, 0x01010101u, wsum);
                wsum = dp4a_mixed<WU, true>(wv.y, 0x01010101u, wsum);
                wsum = dp4a_mixed<WU, true>(wv.z, 0x01010101u, wsum);
                wsum = dp4a_mixed<WU, true>(wv.w, 0x01010101u, wsum);
                #pragma unroll
                for (int r = 0; r < FC_ROWS; ++r) {
                    const uint4 xv = s_x[r * kv + c];
                    int t = acc[r];
                    t = dp4a_mixed<XU, WU>(xv.x, wv.x, t);
                    t = dp4a_mixed<XU, WU>(xv.y, wv.y, t);
                    t = dp4a_mixed<XU, WU>(xv.z, wv.z, t);
                    t = dp4a_mixed<XU, WU>(xv.w, wv.w, t);
                    acc[r] = t;
                    if (a.zw != 0) {
                        int u = xs[r];
                        u = dp4a_mixed<XU, true>(xv.x, 0x01010101u, u);
                        u = dp4a_mixed<XU, true>(xv.y, 0x01010101u, u);
                        u = dp4a_mixed<XU, true>(xv.z, 0x01010101u, u);
                        u = dp4a_mixed<XU, true>(xv.w, 0x01010101u, u);
                        xs[r] = u;
                    }
                }
            }
        }
    }
    if (n >= a.N) return;
    // warp reduction that leaves row r's total in lane r: halve the row set five times
    #pragma unroll
    for (int r = 0; r < FC_ROWS; ++r) acc[r] -= a.zw * xs[r];
    // first fold the lanes that will share a row (FC_ROWS < 32), then halve the row set once per remaining lane bit
    #pragma unroll
    for (int off = 16; off >= FC_ROWS; off >>= 1) {
        #pragma unroll
        for (int r = 0; r < FC_ROWS; ++r) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
    }
    #pragma unroll
    for (int off = FC_ROWS / 2, cnt = FC_ROWS; off >= 1; off >>= 1, cnt >>= 1) {
        const bool upper = (lane & off) != 0;
        #pragma unroll
        for (int r = 0; r < cnt / 2; ++r) {
            const int keep = upper ? acc[r + cnt / 2] : acc[r];
            const int send = upper ? acc[r] : acc[r + cnt / 2];
            acc[r] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    #pragma unroll
    for (int off = 16; off >= 1; off >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, off);
    // step "off" sends the half of the remaining rows whose bit "off" differs from the lane's: lane l ends with row
    // l mod FC_ROWS (lanes FC_ROWS.. hold copies)
    const int r = lane;
    if (r >= FC_ROWS || r >= rows) return;
    const int total = acc[0] - a.zx * wsum + a.K * a.zx * a.zw;
    const long long o = (long long)(m0 + r) * a.N + n;
    if (a.acc_out) a.acc_out[o] = total;
    const float m = __fmul_rn(a.rq.sx, a.w_scales ? a.w_scales[n] : a.w_scale);
    const float b = a.bias ? __fmul_rn(__int2float_rn(a.bias[n]), a.b_scales ? a.b_scales[n] : a.b_scale) : 0.f;
    a.y[o] = (uint8_t)requant_fast(total, m, b, a.bias != nullptr, a.rq.sy, a.inv_sy, (float)a.rq.zy, a.lo, a.hi);
}

static bool fc_rows_eligible(const b200k_fc_params* p)
{
    if (!p->x.data || !p->w.data || !p->y.data) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->w.dtype) || !is_q8(p->y.dtype)) return false;
    if (p->bias.data && p->bias.dtype != B200K_S32) return false;
    if (p->k % 16 != 0 || ((((uintptr_t)p->x.data) | ((uintptr_t)p->w.data)) & 15) != 0) return false;
    if (p->w.scales && p->w.zero_point != 0) return false;
    return true;
}

static int launch_fc_rows(const b200k_fc_params* p, cudaStream_t stream)
{
    FcRowsArgs a;
    a.x = (const uint8_t*)p->x.data; a.w = (const uint8_t*)p->w.data; a.bias = (const int32_t*)p->bias.data;
    a.y = (uint8_t*)p->y.data; a.acc_out = p->acc_out;
    a.w_scales = p->w.scales; a.b_scales = p->bias.scales; a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.zx = p->x.zero_point; a.zw = p->w.scales ? 0 : p->w.zero_point;
    a.M = p->m; a.K = p->k; a.N = p->n;
    a.rq = make_requant(p->x.scale, p->y, p->clamp_lo, p->clamp_hi);
    a.inv_sy = rn_reciprocal(p->y.scale);
    a.lo = fmaxf(a.rq.tlo, (float)a.rq.clo);
    a.hi = fminf(a.rq.thi, (float)a.rq.chi);
    const int kt = p->k < FC_KT ? p->k : FC_KT;
    const bool xu = p->x.dtype == B200K_U8, wu = p->w.dtype == B200K_U8;
    #define B200K_FC_ROWS(XU, WU, RB)                                                                                  \
        do {                                                                                                           \
            /* the opt-in is per device: one flag per device index */                                                  \
            static std::atomic<bool> configured[64];                                                                   \
            int dev_ = 0;                                                                                              \
            if (cudaGetDevice(&dev_) != cudaSuccess || dev_ < 0 || dev_ >= 64) dev_ = 0;                               \
            if (!configured[dev_].load(std::memory_order_acquire)) {                                                   \
                B200K_CUDA(cudaFuncSetAttribute(fc_rows_kernel<XU, WU, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                                RB * FC_KT));                                                          \
                configured[dev_].store(true, std::memory_order_release);                                               \
            }                                                                                                          \
            const dim3 grid(div_up(p->n, FC_COLS), div_up(p->m, RB), 1);                                               \
            launch_pdl(fc_rows_kernel<XU, WU, RB>, grid, dim3(32 * FC_COLS), (size_t)RB * kt, stream, a);              \
        } while (0)
    #define B200K_FC_TYPES(RB)                                                                                         \
        do {                                                                                                           \
            if (xu) { if (wu) B200K_FC_ROWS(true, true, RB); else B200K_FC_ROWS(true, false, RB); }                    \
            else    { if (wu) B200K_FC_ROWS(false, true, RB); else B200K_FC_ROWS(false, false, RB); }                  \
        } while (0)
    if (p->m <= 4)       B200K_FC_TYPES(4);
    else if (p->m <= 16) B200K_FC_TYPES(16);
    else                 B200K_FC_TYPES(32);
    #undef B200K_FC_TYPES
    #undef B200K_FC_ROWS
    return check_launch("fc_rows_kernel");
}

extern "C" int b200k_fully_connected_q8(const b200k_fc_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "fully_connected_q8: null params");
    B200K_REQUIRE(p->m > 0 && p->k > 0 && p->n > 0, B200K_E_INVALID, "fully_connected_q8: bad shape");
    if (p->transpose_w) {
        // x [m, k] is an NHWC tensor [m, 1, 1, k]; w [n, k] is [O, 1, 1, I]: a 1x1 convolution.
        b200k_conv2d_params c;
        memset(&c, 0, sizeof(c));
        c.x = p->x; c.w = p->w; c.bias = p->bias; c.y = p->y;
        c.n = p->m; c.h = 1; c.wd = 1; c.c = p->k; c.oh = 1; c.ow = 1; c.oc = p->n;
        c.kh = c.kw = 1; c.stride_h = c.stride_w = 1; c.dil_h = c.dil_w = 1;
        c.clamp_lo = p->clamp_lo; c.clamp_hi = p->clamp_hi; c.acc_out = p->acc_out; c.algo = p->algo;
        c.packed = p->packed;
        // the tcgen05 kernel when it can take the shape; otherwise the row kernel; the CUDA-core convolution for the rest
        // (a few rows are a weight-streaming problem: the row kernel spreads the columns over every SM, whereas the
        // tensor-core kernel would give each 64-column tile's whole K loop to one CTA)
        // at most 16 rows: nothing but a read of the weights, which the streaming kernel spreads over every SM
        if (p->algo == 0 && fc_stream_eligible(p)) return launch_fc_stream(p, (cudaStream_t)stream);
        if (p->algo == 0 && fc_rows_eligible(p) && (p->m <= 4 || !conv_tc_eligible(&c))) return launch_fc_rows(p, (cudaStream_t)stream);
        return conv2d_dispatch(&c, (cudaStream_t)stream);
    }
    B200K_REQUIRE(p->x.data && p->w.data && p->y.data, B200K_E_INVALID, "fully_connected_q8: null tensor pointer");
    B200K_REQUIRE(is_q8(p->x.dtype) && is_q8(p->w.dtype) && is_q8(p->y.dtype), B200K_E_UNSUPPORTED,
                  "fully_connected_q8: only 8-bit quantised tensors are supported");
    B200K_REQUIRE(!p->bias.data || p->bias.dtype == B200K_S32, B200K_E_INVALID, "fully_connected_q8: bias must be Signed32");
    BmmArgs a;
    a.x = p->x.data; a.y = p->w.data; a.out = (void*)p->y.data; a.acc_out = p->acc_out;
    a.bias = (const int32_t*)p->bias.data; a.w_scales = p->w.scales; a.b_scales = p->bias.scales;
    a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.x_dtype = p->x.dtype; a.y_dtype = p->w.dtype; a.out_dtype = p->y.dtype;
    a.zx = p->x.zero_point; a.zy = p->w.zero_point;
    a.B = 1; a.M = p->m; a.K = p->k; a.N = p->n;
    a.xs_m = p->k; a.xs_k = 1; a.ys_k = p->n; a.ys_n = 1; a.bsx = a.bsy = 0;
    a.rq = make_requant(p->x.scale, p->y, p->clamp_lo, p->clamp_hi);
    dim3 grid(div_up(p->n, 16), div_up(p->m, 16), 1);
    bmm_generic_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(a);
    return check_launch("bmm_generic_kernel");
}
