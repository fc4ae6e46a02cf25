// BatchNormalization and InstanceNormalization of a 4-D tensor in either layout, with CpuRef's fp32 arithmetic
// (src/backends/reference/workloads/BatchNormImpl.cpp:16-63, InstanceNorm.cpp:16-84 of the Arm NN tree).
//   * BatchNormalization is elementwise with two per-channel constants, mult = gamma / sqrt(var + eps) and
//     add = beta - mult * mean, which a first small kernel derives from the four (possibly quantised) parameter tensors.
//   * InstanceNormalization needs the mean and the variance of every (batch, channel) plane, summed in the reference's
//     order (row-major over H, W), so one thread walks one plane: neighbouring threads take neighbouring channels (NHWC,
//     coalesced) or neighbouring planes (NCHW).  A coverage kernel, not a bandwidth one.
#include "common.cuh"

namespace b200k {

struct BnArgs { QView x, y, mean, var, beta, gamma; int c, nchw; long long hw, count; float eps; float* mult_add; };

__global__ void __launch_bounds__(256) batch_norm_constants_kernel(const BnArgs a)
{
    pdl_enter();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= a.c) return;
    const float mult = __fdiv_rn(a.gamma.get(c), __fsqrt_rn(__fadd_rn(a.var.get(c), a.eps)));
    a.mult_add[c] = mult;
    a.mult_add[a.c + c] = __fsub_rn(a.beta.get(c), __fmul_rn(mult, a.mean.get(c)));
}

__global__ void __launch_bounds__(256) batch_norm_kernel(const BnArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.count) return;
    const int c = a.nchw ? (int)((i / a.hw) % a.c) : (int)(i % a.c);
    a.y.set(i, __fadd_rn(__fmul_rn(a.mult_add[c], a.x.get(i)), a.mult_add[a.c + c]));
}

struct InArgs { QView x, y; int n, c, nchw; long long hw; float gamma, beta, eps; };

__global__ void __launch_bounds__(128) instance_norm_kernel(const InArgs a)
{
    pdl_enter();
    const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= (long long)a.n * a.c) return;
    const long long n = t / a.c, c = t - n * a.c;
    const long long base = a.nchw ? t * a.hw : n * a.hw * a.c + c;
    const long long step = a.nchw ? 1 : a.c;
    float mean = 0.f, var = 0.f;
    for (long long k = 0; k < a.hw; ++k) mean = __fadd_rn(mean, a.x.get(base + k * step));
    mean = __fdiv_rn(mean, (float)a.hw);
    for (long long k = 0; k < a.hw; ++k) {
        const float d = __fsub_rn(a.x.get(base + k * step), mean);
        var = __fadd_rn(var, __fmul_rn(d, d));
    }
    var = __fdiv_rn(var, (float)a.hw);
    const float root = __fsqrt_rn(__fadd_rn(var, a.eps));
    for (long long k = 0; k < a.hw; ++k) {
        const long long at = base + k * step;
        a.y.set(at, __fadd_rn(__fdiv_rn(__fmul_rn(__fsub_rn(a.x.get(at), mean), a.gamma), root), a.beta));
    }
}

}  // namespace b200k

using namespace b200k;

static bool act_type(int dtype) { return dtype == B200K_U8 || dtype == B200K_S8 || dtype == B200K_S16 || dtype == B200K_F32; }

extern "C" int b200k_batch_norm_q(const b200k_batch_norm_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "batch_norm_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data && p->mean.data && p->variance.data && p->beta.data && p->gamma.data && p->scratch,
                  B200K_E_INVALID, "batch_norm_q: null tensor or scratch pointer");
    B200K_REQUIRE(p->n > 0 && p->c > 0 && p->hw > 0, B200K_E_INVALID, "batch_norm_q: bad shape");
    B200K_REQUIRE(act_type(p->x.dtype) && act_type(p->y.dtype) && act_type(p->mean.dtype) && act_type(p->variance.dtype) &&
                  act_type(p->beta.dtype) && act_type(p->gamma.dtype), B200K_E_UNSUPPORTED, "batch_norm_q: unsupported data type");
    BnArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.mean = make_view(p->mean); a.var = make_view(p->variance); a.beta = make_view(p->beta); a.gamma = make_view(p->gamma);
    a.c = p->c; a.nchw = p->nchw ? 1 : 0; a.hw = p->hw; a.count = (long long)p->n * p->c * p->hw; a.eps = p->eps;
    a.mult_add = (float*)p->scratch;
    B200K_REQUIRE(a.count / 256 < (1ll << 31) - 1, B200K_E_TOOBIG, "batch_norm_q: tensor too large");
    cudaStream_t s = (cudaStream_t)stream;
    launch_pdl(batch_norm_constants_kernel, dim3(div_up(p->c, 256)), dim3(256), 0, s, a);
    int rc = check_launch("batch_norm_constants_kernel");
    if (rc != B200K_OK) return rc;
    launch_pdl(batch_norm_kernel, dim3(div_up(a.count, 256)), dim3(256), 0, s, a);
    return check_launch("batch_norm_kernel");
}

extern "C" int b200k_instance_norm_q(const b200k_instance_norm_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "instance_norm_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "instance_norm_q: null tensor pointer");
    B200K_REQUIRE(p->n > 0 && p->c > 0 && p->hw > 0, B200K_E_INVALID, "instance_norm_q: bad shape");
    // the reference supports Float32 (and Float16) only: InstanceNormalizationQueueDescriptor::Validate
    B200K_REQUIRE(p->x.dtype == B200K_F32 && p->y.dtype == B200K_F32, B200K_E_UNSUPPORTED, "instance_norm_q: Float32 tensors only");
    InArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.n = p->n; a.c = p->c; a.nchw = p->nchw ? 1 : 0; a.hw = p->hw;
    a.gamma = p->gamma; a.beta = p->beta; a.eps = p->eps;
    launch_pdl(instance_norm_kernel, dim3(div_up((long long)p->n * p->c, 128)), dim3(128), 0, (cudaStream_t)stream, a);
    return check_launch("instance_norm_kernel");
}
