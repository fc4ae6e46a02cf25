// Convolution3d (NDHWC input, weights [D, H, W, I, O]) and Pooling3d (NDHWC), as the reference computes them
// (src/backends/reference/workloads/Conv3dImpl.cpp:14-177, Pooling3d.cpp:138-328 of the Arm NN tree).  One thread per
// output element, the output channel fastest: weight reads of a warp are contiguous, input reads a broadcast.
//   * quantised convolution: exact int32 accumulation of (x - zx)(w - zw), then the contraction epilogue every
//     quantised contraction of this library uses (fp32 scale, bias, Quantize, clamp);
//   * Float32 convolution: the reference's term order (z, y, x, input channel) with separate multiply and add;
//   * pooling: the reference's fp32 accumulation over the window in (z, y, x) order.
// Coverage kernels on CUDA cores: volumetric layers are not on a benchmarked path.
#include "common.cuh"

namespace b200k {

struct Conv3dArgs {
    QView x, w;
    const void* bias; const float* w_scales; const float* b_scales; float b_scale;
    void* y; int y_dtype;
    Requant rq;
    int N, D, H, W, C, OD, OH, OW, OC, KD, KH, KW;
    int sd, sh, sw, pf, pt, pl, dd, dh, dw;
    long long total;
};

template <bool FLOAT>
__global__ void __launch_bounds__(256) conv3d_kernel(const Conv3dArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    const int co = (int)(i % a.OC);
    long long t = i / a.OC;
    const int ox = (int)(t % a.OW); t /= a.OW;
    const int oy = (int)(t % a.OH); t /= a.OH;
    const int oz = (int)(t % a.OD);
    const int n = (int)(t / a.OD);
    float sum = 0.0f;
    int acc = 0;
    for (int kz = 0; kz < a.KD; ++kz) {
        const int iz = oz * a.sd + kz * a.dd - a.pf;
        for (int ky = 0; ky < a.KH; ++ky) {
            const int iy = oy * a.sh + ky * a.dh - a.pt;
            for (int kx = 0; kx < a.KW; ++kx) {
                const int ix = ox * a.sw + kx * a.dw - a.pl;
                const bool inside = iz >= 0 && iz < a.D && iy >= 0 && iy < a.H && ix >= 0 && ix < a.W;
                if (!FLOAT && !inside) continue;                       // a padding tap adds 0
                const long long xb = ((((long long)n * a.D + iz) * a.H + iy) * a.W + ix) * a.C;
                const long long wb = ((((long long)kz * a.KH + ky) * a.KW + kx) * a.C) * a.OC + co;
                for (int c = 0; c < a.C; ++c) {
                    if (FLOAT) {
                        const float xv = inside ? ((const float*)a.x.data)[xb + c] : 0.0f;
                        sum = __fadd_rn(sum, __fmul_rn(((const float*)a.w.data)[wb + (long long)c * a.OC], xv));
                    } else {
                        acc += (load_q_dev(a.x.data, a.x.dtype, xb + c) - a.x.zp) *
                               (load_q_dev(a.w.data, a.w.dtype, wb + (long long)c * a.OC) - a.w.zp);
                    }
                }
            }
        }
    }
    if (FLOAT) {
        if (a.bias) sum = __fadd_rn(sum, ((const float*)a.bias)[co]);
        ((float*)a.y)[i] = sum;
        return;
    }
    const float swc = a.w_scales ? a.w_scales[co] : a.w.scale;
    const float sbc = a.b_scales ? a.b_scales[co] : a.b_scale;
    const int bq = a.bias ? ((const int*)a.bias)[co] : 0;
    store_q_dev(a.y, a.y_dtype, i, a.rq(acc, swc, a.bias != nullptr, bq, sbc));
}

struct Pool3dArgs {
    QView x, y;
    int N, D, H, W, C, OD, OH, OW;
    int pd, ph, pw, sd, sh, sw;
    int pad_front, pad_back, pad_top, pad_bottom, pad_left, pad_right;
    int type, exclude;          // armnn::PoolingAlgorithm (0 Max, 1 Average, 2 L2); PaddingMethod::Exclude
    long long total;
};

// Pooling3d.cpp:100-111: clamp a window to [0, extent]; true when anything was cut
__device__ __forceinline__ bool clamp_range(int& start, int& end, int extent)
{
    if (start < 0 || end > extent) {
        start = min(max(start, 0), extent);
        end = min(max(end, 0), extent);
        return true;
    }
    return false;
}

__global__ void __launch_bounds__(256) pool3d_kernel(const Pool3dArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    const int c = (int)(i % a.C);
    long long t = i / a.C;
    const int ox = (int)(t % a.OW); t /= a.OW;
    const int oy = (int)(t % a.OH); t /= a.OH;
    const int oz = (int)(t % a.OD);
    const int n = (int)(t / a.OD);
    // Pooling3d.cpp:196-265: the window in padded coordinates, cut at the far padding, its size, then clamped to the tensor
    int ds = oz * a.sd - a.pad_front, de = min(ds + a.pd, a.D + a.pad_back);
    int hs = oy * a.sh - a.pad_top,   he = min(hs + a.ph, a.H + a.pad_bottom);
    int ws = ox * a.sw - a.pad_left,  we = min(ws + a.pw, a.W + a.pad_right);
    float pool = (float)((de - ds) * (he - hs) * (we - ws));
    const bool dcl = clamp_range(ds, de, a.D), hcl = clamp_range(hs, he, a.H), wcl = clamp_range(ws, we, a.W);
    if (de <= 0 || ds > a.D || he <= 0 || hs > a.H || we <= 0 || ws > a.W) {       // OnPaddingOnly: lines 88-98, 232-243
        a.y.set(i, 0.0f);
        return;
    }
    if ((dcl || hcl || wcl) && a.exclude) pool = (float)((de - ds) * (he - hs) * (we - ws));
    float result = a.type == 0 ? -3.402823466e+38f : 0.0f;
    for (int z = ds; z < de; ++z)
        for (int y = hs; y < he; ++y)
            for (int x = ws; x < we; ++x) {
                const float v = a.x.get(((((long long)n * a.D + z) * a.H + y) * a.W + x) * a.C + c);
                if (a.type == 0)      { if (v > result) result = v; }
                else if (a.type == 1) result = __fadd_rn(result, v);
                else                  result = __fadd_rn(result, __fmul_rn(v, v));
            }
    if (a.type == 1)      result = __fdiv_rn(result, pool);
    else if (a.type == 2) result = __fsqrt_rn(__fdiv_rn(result, pool));
    a.y.set(i, result);
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_conv3d_q(const b200k_conv3d_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "conv3d_q: null params");
    B200K_REQUIRE(p->x.data && p->w.data && p->y.data, B200K_E_INVALID, "conv3d_q: null tensor pointer");
    B200K_REQUIRE(p->n > 0 && p->d > 0 && p->h > 0 && p->wd > 0 && p->c > 0 && p->od > 0 && p->oh > 0 && p->ow > 0 && p->oc > 0 &&
                  p->kd > 0 && p->kh > 0 && p->kw > 0, B200K_E_INVALID, "conv3d_q: bad shape");
    B200K_REQUIRE(p->stride_d > 0 && p->stride_h > 0 && p->stride_w > 0 && p->dil_d > 0 && p->dil_h > 0 && p->dil_w > 0 &&
                  p->pad_front >= 0 && p->pad_top >= 0 && p->pad_left >= 0, B200K_E_INVALID, "conv3d_q: bad stride / dilation / padding");
    const bool f32 = p->x.dtype == B200K_F32;
    if (f32) {
        B200K_REQUIRE(p->w.dtype == B200K_F32 && p->y.dtype == B200K_F32 && (!p->bias.data || p->bias.dtype == B200K_F32),
                      B200K_E_UNSUPPORTED, "conv3d_q: a Float32 input needs Float32 weights, bias and output");
    } else {
        B200K_REQUIRE(is_q8(p->x.dtype) && is_q8(p->w.dtype) && is_q8(p->y.dtype) && (!p->bias.data || p->bias.dtype == B200K_S32),
                      B200K_E_UNSUPPORTED, "conv3d_q: 8-bit tensors with a Signed32 bias, or Float32 throughout");
        B200K_REQUIRE(p->x.scale > 0.f && p->y.scale > 0.f, B200K_E_INVALID, "conv3d_q: non-positive scale");
    }
    Conv3dArgs a;
    memset(&a, 0, sizeof(a));
    a.x = make_view(p->x); a.w = make_view(p->w);
    a.bias = p->bias.data; a.w_scales = p->w.scales; a.b_scales = p->bias.scales; a.b_scale = p->bias.scale;
    a.y = (void*)p->y.data; a.y_dtype = p->y.dtype;
    if (!f32) a.rq = make_requant(p->x.scale, p->y, p->clamp_lo, p->clamp_hi);
    a.N = p->n; a.D = p->d; a.H = p->h; a.W = p->wd; a.C = p->c; a.OD = p->od; a.OH = p->oh; a.OW = p->ow; a.OC = p->oc;
    a.KD = p->kd; a.KH = p->kh; a.KW = p->kw;
    a.sd = p->stride_d; a.sh = p->stride_h; a.sw = p->stride_w; a.pf = p->pad_front; a.pt = p->pad_top; a.pl = p->pad_left;
    a.dd = p->dil_d; a.dh = p->dil_h; a.dw = p->dil_w;
    a.total = (long long)p->n * p->od * p->oh * p->ow * p->oc;
    B200K_REQUIRE(a.total / 256 < (1ll << 31) - 1, B200K_E_TOOBIG, "conv3d_q: tensor too large");
    cudaStream_t s = (cudaStream_t)stream;
    if (f32) launch_pdl(conv3d_kernel<true>, dim3(div_up(a.total, 256)), dim3(256), 0, s, a);
    else     launch_pdl(conv3d_kernel<false>, dim3(div_up(a.total, 256)), dim3(256), 0, s, a);
    return check_launch("conv3d_kernel");
}

extern "C" int b200k_pool3d_q(const b200k_pool3d_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "pool3d_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "pool3d_q: null tensor pointer");
    B200K_REQUIRE(p->n > 0 && p->d > 0 && p->h > 0 && p->wd > 0 && p->c > 0 && p->od > 0 && p->oh > 0 && p->ow > 0,
                  B200K_E_INVALID, "pool3d_q: bad shape");
    B200K_REQUIRE(p->pool_d > 0 && p->pool_h > 0 && p->pool_w > 0 && p->stride_d > 0 && p->stride_h > 0 && p->stride_w > 0,
                  B200K_E_INVALID, "pool3d_q: bad pool size / stride");
    B200K_REQUIRE(p->pool_type >= 0 && p->pool_type <= 2, B200K_E_INVALID, "pool3d_q: unknown pooling algorithm %d", p->pool_type);
    B200K_REQUIRE(p->padding_method == 0 || p->padding_method == 1, B200K_E_INVALID, "pool3d_q: unknown padding method %d", p->padding_method);
    B200K_REQUIRE(p->x.dtype != B200K_S32 && p->y.dtype != B200K_S32 && p->x.dtype >= B200K_U8 && p->x.dtype <= B200K_F32 &&
                  p->y.dtype >= B200K_U8 && p->y.dtype <= B200K_F32, B200K_E_UNSUPPORTED, "pool3d_q: unsupported data type");
    Pool3dArgs a;
    memset(&a, 0, sizeof(a));
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.N = p->n; a.D = p->d; a.H = p->h; a.W = p->wd; a.C = p->c; a.OD = p->od; a.OH = p->oh; a.OW = p->ow;
    a.pd = p->pool_d; a.ph = p->pool_h; a.pw = p->pool_w; a.sd = p->stride_d; a.sh = p->stride_h; a.sw = p->stride_w;
    a.pad_front = p->pad_front; a.pad_back = p->pad_back; a.pad_top = p->pad_top; a.pad_bottom = p->pad_bottom;
    a.pad_left = p->pad_left; a.pad_right = p->pad_right;
    a.type = p->pool_type; a.exclude = p->padding_method == 1;
    a.total = (long long)p->n * p->od * p->oh * p->ow * p->c;
    B200K_REQUIRE(a.total / 256 < (1ll << 31) - 1, B200K_E_TOOBIG, "pool3d_q: tensor too large");
    launch_pdl(pool3d_kernel, dim3(div_up(a.total, 256)), dim3(256), 0, (cudaStream_t)stream, a);
    return check_launch("pool3d_kernel");
}
