// Softmax over one axis of a quantised (or fp32) tensor.
//
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

    float mx = -3.402823466e+38f;
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

    for (int i = tid; i < a.axis; i += SM_THREADS)
        ex[i] = expf(__fmul_rn(__fsub_rn(a.x.get(base + (long long)i * a.inner), mx), a.beta));
    __syncthreads();
    if (tid == 0) {
        float sum = 0.0f;
        for (int i = 0; i < a.axis; ++i) sum = __fadd_rn(sum, ex[i]);
        s_sum = sum;
    }
    __syncthreads();
    const float sum = s_sum;
    for (int i = tid; i < a.axis; i += SM_THREADS)
        a.y.set(base + (long long)i * a.inner, __fdiv_rn(ex[i], sum));
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_softmax_q8(const b200k_softmax_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "softmax_q8: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "softmax_q8: null tensor pointer");
    B200K_REQUIRE(p->outer > 0 && p->axis_size > 0 && p->inner > 0, B200K_E_INVALID, "softmax_q8: bad shape");
    B200K_REQUIRE(p->x.dtype != B200K_S32 && p->y.dtype != B200K_S32, B200K_E_UNSUPPORTED, "softmax_q8: Signed32 not supported");
    // one float per element of the axis in dynamic shared memory, next to the kernel's few static words, within the
    // 48 KiB every launch may use without opting in
    B200K_REQUIRE(p->axis_size <= SM_MAX_AXIS, B200K_E_TOOBIG, "softmax_q8: axis length %d exceeds the %d this kernel stages in shared memory",
                  p->axis_size, SM_MAX_AXIS);
    SoftmaxArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.outer = p->outer; a.axis = p->axis_size; a.inner = p->inner; a.beta = p->beta;
    const long long rows = (long long)p->outer * p->inner;
    B200K_REQUIRE(rows < (1ll << 31), B200K_E_TOOBIG, "softmax_q8: too many rows");
    launch_pdl(softmax_kernel, dim3((unsigned)rows), dim3(SM_THREADS), p->axis_size * sizeof(float), (cudaStream_t)stream, a);
    return check_launch("softmax_kernel");
}
