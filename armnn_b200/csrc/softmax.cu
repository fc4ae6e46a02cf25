// Softmax, LogSoftmax, L2Normalization and ArgMinMax: independent rows along one axis of a quantised (or fp32) tensor.
//
// Softmax:
// One CTA per (outer, inner) row.  The row maximum is a warp-shuffle reduction (order does not matter
// for a maximum); the exponentials — the expensive part — are computed by all threads in parallel and
// parked in shared memory; the denominator is then summed by one thread in the row's index order,
// because CpuRef's fp32 sum is sequential (Softmax.cpp:40-46 of the Arm NN tree) and a tree reduction
// would round differently.  The final divide + re-quantise is parallel again.
#include "common.cuh"

namespace b200k {

struct SoftmaxArgs { QView x, y; int outer, axis, inner; float beta; };

constexpr int SM_THREADS = 128;
constexpr int SM_MAX_AXIS = (48 * 1024 - 64) / 4;        // dynamic floats + the static words below stay within 48 KiB

enum { ROW_SOFTMAX = 0, ROW_LOG_SOFTMAX = 1, ROW_L2_NORM = 2 };

// MODE ROW_SOFTMAX / ROW_LOG_SOFTMAX: beta as in the descriptor.  ROW_L2_NORM: beta is eps; the parked values are the
// squares, summed in index order like the reference's `reduction += value * value`
// (RefL2NormalizationWorkload.cpp:73-80), and every element is multiplied by 1 / sqrt(max(sum, eps)).
template <int MODE>
__global__ void __launch_bounds__(SM_THREADS) softmax_kernel(const SoftmaxArgs a)
{
    pdl_enter();
    extern __shared__ float ex[];            // [axis]
    __shared__ float red[SM_THREADS / 32];
    __shared__ float s_max, s_sum;
    const int row = blockIdx.x;
    const int o = row / a.inner, in = row - o * a.inner;
    const long long base = (long long)o * a.axis * a.inner + in;
    const int tid = threadIdx.x;

    float mx = 0.f;
    if (MODE != ROW_L2_NORM) {
        mx = -3.402823466e+38f;
        for (int i = tid; i < a.axis; i += SM_THREADS) mx = fmaxf(mx, a.x.get(base + (long long)i * a.inner));
        #pragma unroll
        for (int s = 16; s > 0; s >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, s));
        if ((tid & 31) == 0) red[tid >> 5] = mx;
        __syncthreads();
        if (tid == 0) {
            float m = red[0];
            for (int w = 1; w < SM_THREADS / 32; ++w) m = fmaxf(m, red[w]);
            s_max = m;
        }
        __syncthreads();
        mx = s_max;
    }

    for (int i = tid; i < a.axis; i += SM_THREADS) {
        const float v = a.x.get(base + (long long)i * a.inner);
        ex[i] = MODE == ROW_L2_NORM ? __fmul_rn(v, v) : expf(__fmul_rn(__fsub_rn(v, mx), a.beta));
    }
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;
        for (int i = 0; i < a.axis; ++i) sum = __fadd_rn(sum, ex[i]);
        s_sum = sum;
    }
    __syncthreads();
    const float sum = s_sum;
    if (MODE == ROW_SOFTMAX) {
        for (int i = tid; i < a.axis; i += SM_THREADS)
            a.y.set(base + (long long)i * a.inner, __fdiv_rn(ex[i], sum));
    } else if (MODE == ROW_LOG_SOFTMAX) {
        const float log_sum = logf(sum);
        for (int i = tid; i < a.axis; i += SM_THREADS) {
            const long long at = base + (long long)i * a.inner;
            a.y.set(at, __fsub_rn(__fmul_rn(__fsub_rn(a.x.get(at), mx), a.beta), log_sum));
        }
    } else {
        const float scale = __fdiv_rn(1.0f, __fsqrt_rn(sum < a.beta ? a.beta : sum));
        for (int i = tid; i < a.axis; i += SM_THREADS) {
            const long long at = base + (long long)i * a.inner;
            a.y.set(at, __fmul_rn(a.x.get(at), scale));
        }
    }
}

struct ArgArgs { QView x; void* y; int outer, axis, inner, want_max, out64; long long rows; };

// One row per warp when the axis is contiguous (inner == 1: lanes stride the axis, then a shuffle reduction that keeps
// the lower index among equals), else one row per thread (neighbouring threads read neighbouring `inner` positions).
template <bool WARP>
__global__ void __launch_bounds__(256) arg_min_max_kernel(const ArgArgs a)
{
    pdl_enter();
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long row = WARP ? t >> 5 : t;
    if (row >= a.rows) return;
    const int lane = WARP ? (int)(t & 31) : 0, step = WARP ? 32 : 1;
    const long long o = row / a.inner, in = row - o * a.inner;
    const long long base = o * a.axis * a.inner + in;
    // the reference starts from element 0 and replaces on a strict comparison: the first of equal elements wins
    float best = 0.f;
    int idx = 0x7fffffff;
    for (int i = lane; i < a.axis; i += step) {
        const float v = a.x.get(base + (long long)i * a.inner);
        if (idx == 0x7fffffff || (a.want_max ? v > best : v < best)) { best = v; idx = i; }
    }
    if (WARP) {
        #pragma unroll
        for (int s = 16; s > 0; s >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, s);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, s);
            const bool better = oi != 0x7fffffff && (idx == 0x7fffffff || (a.want_max ? ov > best : ov < best) || (ov == best && oi < idx));
            if (better) { best = ov; idx = oi; }
        }
        if (lane != 0) return;
    }
    if (a.out64) ((long long*)a.y)[row] = idx; else ((int*)a.y)[row] = idx;
}

}  // namespace b200k

using namespace b200k;

static int launch_rows(const b200k_softmax_params* p, void* stream, int mode, const char* what)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "%s: null params", what);
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "%s: null tensor pointer", what);
    B200K_REQUIRE(p->outer > 0 && p->axis_size > 0 && p->inner > 0, B200K_E_INVALID, "%s: bad shape", what);
    B200K_REQUIRE(p->x.dtype != B200K_S32 && p->y.dtype != B200K_S32, B200K_E_UNSUPPORTED, "%s: Signed32 not supported", what);
    // one float per element of the axis in dynamic shared memory, next to the kernel's few static words, within the
    // 48 KiB every launch may use without opting in
    B200K_REQUIRE(p->axis_size <= SM_MAX_AXIS, B200K_E_TOOBIG, "%s: axis length %d exceeds the %d this kernel stages in shared memory",
                  what, p->axis_size, SM_MAX_AXIS);
    SoftmaxArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.outer = p->outer; a.axis = p->axis_size; a.inner = p->inner; a.beta = p->beta;
    const long long rows = (long long)p->outer * p->inner;
    B200K_REQUIRE(rows < (1ll << 31), B200K_E_TOOBIG, "%s: too many rows", what);
    const size_t smem = p->axis_size * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (mode == ROW_SOFTMAX)          launch_pdl(softmax_kernel<ROW_SOFTMAX>, dim3((unsigned)rows), dim3(SM_THREADS), smem, s, a);
    else if (mode == ROW_LOG_SOFTMAX) launch_pdl(softmax_kernel<ROW_LOG_SOFTMAX>, dim3((unsigned)rows), dim3(SM_THREADS), smem, s, a);
    else                              launch_pdl(softmax_kernel<ROW_L2_NORM>, dim3((unsigned)rows), dim3(SM_THREADS), smem, s, a);
    return check_launch("softmax_kernel");
}

extern "C" int b200k_softmax_q8(const b200k_softmax_params* p, void* stream)
{
    return launch_rows(p, stream, ROW_SOFTMAX, "softmax_q8");
}

extern "C" int b200k_log_softmax_q(const b200k_softmax_params* p, void* stream)
{
    return launch_rows(p, stream, ROW_LOG_SOFTMAX, "log_softmax_q");
}

extern "C" int b200k_l2_normalization_q(const b200k_softmax_params* p, void* stream)
{
    return launch_rows(p, stream, ROW_L2_NORM, "l2_normalization_q");
}

extern "C" int b200k_arg_min_max_q(const b200k_arg_min_max_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "arg_min_max_q: null params");
    B200K_REQUIRE(p->x.data && p->y, B200K_E_INVALID, "arg_min_max_q: null tensor pointer");
    B200K_REQUIRE(p->outer > 0 && p->axis_size > 0 && p->inner > 0, B200K_E_INVALID, "arg_min_max_q: bad shape");
    B200K_REQUIRE(p->x.dtype == B200K_U8 || p->x.dtype == B200K_S8 || p->x.dtype == B200K_S16 || p->x.dtype == B200K_F32,
                  B200K_E_UNSUPPORTED, "arg_min_max_q: unsupported element type %d", p->x.dtype);
    B200K_REQUIRE(p->function == 0 || p->function == 1, B200K_E_INVALID, "arg_min_max_q: function %d is neither Min (0) nor Max (1)", p->function);
    ArgArgs a;
    a.x = make_view(p->x); a.y = p->y;
    a.outer = p->outer; a.axis = p->axis_size; a.inner = p->inner; a.want_max = p->function; a.out64 = p->out_int64 ? 1 : 0;
    a.rows = (long long)p->outer * p->inner;
    cudaStream_t s = (cudaStream_t)stream;
    if (p->inner == 1 && p->axis_size >= 64) {
        B200K_REQUIRE(a.rows < (1ll << 34), B200K_E_TOOBIG, "arg_min_max_q: too many rows");
        launch_pdl(arg_min_max_kernel<true>, dim3((unsigned)div_up(a.rows * 32, 256)), dim3(256), 0, s, a);
    } else {
        B200K_REQUIRE(a.rows < (1ll << 38), B200K_E_TOOBIG, "arg_min_max_q: too many rows");
        launch_pdl(arg_min_max_kernel<false>, dim3((unsigned)div_up(a.rows, 256)), dim3(256), 0, s, a);
    }
    return check_launch("arg_min_max_kernel");
}
