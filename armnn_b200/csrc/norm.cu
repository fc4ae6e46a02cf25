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

// ---- Normalization (local response normalisation) --------------------------------------------------------------
// RefNormalizationWorkload.cpp:19-140 of the Arm NN tree, LocalBrightness only (the reference supports nothing else):
//   Across: s = sum of squares over the channels c - r .. c + r at the same pixel, y = x * powf(kappa + s * alpha, -beta);
//   Within: s = sum of squares over the (2 r + 1)^2 window around the pixel in the same channel, indexed as NCHW
//           whatever the layout says, y = x / powf(kappa + s * alpha, beta).
// r = norm_size / 2; positions outside the tensor are skipped; sums run in the reference's order.
namespace b200k {

struct LrnArgs { QView x, y; int n, c, h, w, nchw, within, radius; float alpha, beta, kappa; long long count; };

__global__ void __launch_bounds__(256) normalization_kernel(const LrnArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.count) return;
    float acc = 0.f;
    if (a.within) {
        const int w = (int)(i % a.w), h = (int)((i / a.w) % a.h);
        const long long plane = i - ((long long)h * a.w + w);
        for (int y = -a.radius; y <= a.radius; ++y)
            for (int x = -a.radius; x <= a.radius; ++x) {
                const int ix = w + x, iy = h + y;
                if (ix < 0 || ix >= a.w || iy < 0 || iy >= a.h) continue;
                const float v = a.x.get(plane + (long long)iy * a.w + ix);
                acc = __fadd_rn(acc, __fmul_rn(v, v));
            }
        a.y.set(i, __fdiv_rn(a.x.get(i), powf(__fadd_rn(a.kappa, __fmul_rn(acc, a.alpha)), a.beta)));
        return;
    }
    const long long hw = (long long)a.h * a.w;
    const int c = a.nchw ? (int)((i / hw) % a.c) : (int)(i % a.c);
    const long long cstride = a.nchw ? hw : 1;
    for (int z = -a.radius; z <= a.radius; ++z) {
        const int k = c + z;
        if (k < 0 || k >= a.c) continue;
        const float v = a.x.get(i + (long long)z * cstride);
        acc = __fadd_rn(acc, __fmul_rn(v, v));
    }
    const float scale = powf(__fadd_rn(a.kappa, __fmul_rn(acc, a.alpha)), -a.beta);
    a.y.set(i, __fmul_rn(scale, a.x.get(i)));
}

}  // namespace b200k

extern "C" int b200k_normalization_q(const b200k_normalization_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "normalization_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "normalization_q: null tensor pointer");
    B200K_REQUIRE(p->n > 0 && p->c > 0 && p->h > 0 && p->w > 0, B200K_E_INVALID, "normalization_q: bad shape");
    B200K_REQUIRE(act_type(p->x.dtype) && act_type(p->y.dtype), B200K_E_UNSUPPORTED, "normalization_q: unsupported data type");
    B200K_REQUIRE(p->channel_type == 0 || p->channel_type == 1, B200K_E_INVALID, "normalization_q: channel type %d is neither Across (0) nor Within (1)", p->channel_type);
    B200K_REQUIRE(p->channel_type == 0 || p->nchw, B200K_E_UNSUPPORTED, "normalization_q: Within indexes the tensor as NCHW (as the reference does): pass nchw = 1");
    B200K_REQUIRE(p->norm_size >= 1, B200K_E_INVALID, "normalization_q: norm_size must be positive");
    b200k::LrnArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.n = p->n; a.c = p->c; a.h = p->h; a.w = p->w; a.nchw = p->nchw ? 1 : 0; a.within = p->channel_type;
    a.radius = (int)(p->norm_size / 2);
    a.alpha = p->alpha; a.beta = p->beta; a.kappa = p->kappa;
    a.count = (long long)p->n * p->c * p->h * p->w;
    B200K_REQUIRE(a.count / 256 < (1ll << 31) - 1, B200K_E_TOOBIG, "normalization_q: tensor too large");
    launch_pdl(b200k::normalization_kernel, dim3(div_up(a.count, 256)), dim3(256), 0, (cudaStream_t)stream, a);
    return check_launch("normalization_kernel");
}
