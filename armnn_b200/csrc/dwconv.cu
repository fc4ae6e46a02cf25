// DepthwiseConvolution2d for 8-bit quantised NHWC tensors: a bandwidth-bound kernel, no tensor cores.
//
// Each thread produces VEC consecutive output channels of one output pixel; consecutive threads walk
// the channel axis, so every tap is one coalesced vector load of the input row and of the
// [1, KH, KW, OC] weights (which stay in L1/L2: they are tiny).  Padding taps are skipped, exactly as
// CpuRef's zero contribution (ConvImpl.cpp:173-177 of the Arm NN tree).  VEC = 16 uses 128-bit loads.
#include "common.cuh"

namespace b200k {

struct DwArgs {
    const uint8_t* x; const uint8_t* w; const int32_t* bias; uint8_t* y; int32_t* acc_out;
    const float* w_scales; const float* b_scales;
    float w_scale, b_scale;
    int x_u8, w_u8;
    int zx, zw;                     // true zero points
    int N, H, W, C, OH, OW, OC, KH, KW, sh, sw, pt, pl, dh, dw, dm;
    long long total;                // number of thread work items
    Requant rq;
};

template <int VEC> struct VecT;
template <> struct VecT<16> { using type = uint4; };
template <> struct VecT<4>  { using type = unsigned; };
template <> struct VecT<1>  { using type = uint8_t; };

template <int VEC>
__device__ __forceinline__ void unpack(const typename VecT<VEC>::type& v, bool is_u8, int* out)
{
    const uint8_t* b = (const uint8_t*)&v;
    #pragma unroll
    for (int i = 0; i < VEC; ++i) out[i] = is_u8 ? (int)b[i] : (int)(int8_t)b[i];
}

// VEC > 1 requires depth multiplier 1 and C % VEC == 0 with matching pointer alignment.
template <int VEC>
__global__ void __launch_bounds__(256) dwconv_kernel(const DwArgs a)
{
    using V = typename VecT<VEC>::type;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int cg = a.OC / VEC;
    const int co = (int)(idx % cg) * VEC;
    long long t = idx / cg;
    const int ox = (int)(t % a.OW); t /= a.OW;
    const int oy = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    const int ci = co / a.dm;

    int acc[VEC];
    #pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0;

    for (int ky = 0; ky < a.KH; ++ky) {
        const int iy = oy * a.sh + ky * a.dh - a.pt;
        if (iy < 0 || iy >= a.H) continue;
        for (int kx = 0; kx < a.KW; ++kx) {
            const int ix = ox * a.sw + kx * a.dw - a.pl;
            if (ix < 0 || ix >= a.W) continue;
            const V xv = *(const V*)(a.x + (((long long)n * a.H + iy) * a.W + ix) * a.C + ci);
            const V wv = *(const V*)(a.w + ((long long)ky * a.KW + kx) * a.OC + co);
            int xi[VEC], wi[VEC];
            unpack<VEC>(xv, a.x_u8, xi);
            unpack<VEC>(wv, a.w_u8, wi);
            #pragma unroll
            for (int i = 0; i < VEC; ++i) acc[i] += (xi[i] - a.zx) * (wi[i] - a.zw);
        }
    }

    const long long ob = (((long long)n * a.OH + oy) * a.OW + ox) * a.OC + co;
    V outv;
    uint8_t* ob8 = (uint8_t*)&outv;
    #pragma unroll
    for (int i = 0; i < VEC; ++i) {
        const int ch = co + i;
        if (a.acc_out) a.acc_out[ob + i] = acc[i];
        const float swc = a.w_scales ? a.w_scales[ch] : a.w_scale;
        const float sbc = a.b_scales ? a.b_scales[ch] : a.b_scale;
        const int bq = a.bias ? a.bias[ch] : 0;
        ob8[i] = (uint8_t)a.rq(acc[i], swc, a.bias != nullptr, bq, sbc);
    }
    *(V*)(a.y + ob) = outv;
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_dwconv2d_q8(const b200k_conv2d_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "dwconv2d_q8: null params");
    B200K_REQUIRE(p->x.data && p->w.data && p->y.data, B200K_E_INVALID, "dwconv2d_q8: null tensor pointer");
    B200K_REQUIRE(is_q8(p->x.dtype) && is_q8(p->w.dtype) && is_q8(p->y.dtype), B200K_E_UNSUPPORTED,
                  "dwconv2d_q8: only 8-bit quantised tensors are supported");
    B200K_REQUIRE(!p->bias.data || p->bias.dtype == B200K_S32, B200K_E_INVALID, "dwconv2d_q8: bias must be Signed32");
    B200K_REQUIRE(!p->add_operand.data, B200K_E_UNSUPPORTED, "dwconv2d_q8: a fused Add is only available on Convolution2d");
    B200K_REQUIRE(p->n > 0 && p->h > 0 && p->wd > 0 && p->c > 0 && p->oh > 0 && p->ow > 0 && p->oc > 0 &&
                  p->kh > 0 && p->kw > 0 && p->stride_h > 0 && p->stride_w > 0 && p->dil_h > 0 && p->dil_w > 0,
                  B200K_E_INVALID, "dwconv2d_q8: bad geometry");
    B200K_REQUIRE(p->oc % p->c == 0, B200K_E_INVALID, "dwconv2d_q8: output channels %d not a multiple of input channels %d",
                  p->oc, p->c);
    DwArgs a;
    a.x = (const uint8_t*)p->x.data; a.w = (const uint8_t*)p->w.data; a.bias = (const int32_t*)p->bias.data;
    a.y = (uint8_t*)p->y.data; a.acc_out = p->acc_out;
    a.w_scales = p->w.scales; a.b_scales = p->bias.scales; a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.x_u8 = p->x.dtype == B200K_U8; a.w_u8 = p->w.dtype == B200K_U8;
    a.zx = p->x.zero_point; a.zw = p->w.zero_point;
    a.N = p->n; a.H = p->h; a.W = p->wd; a.C = p->c; a.OH = p->oh; a.OW = p->ow; a.OC = p->oc;
    a.KH = p->kh; a.KW = p->kw; a.sh = p->stride_h; a.sw = p->stride_w; a.pt = p->pad_top; a.pl = p->pad_left;
    a.dh = p->dil_h; a.dw = p->dil_w; a.dm = p->oc / p->c;
    a.rq = make_requant(p->x.scale, p->y, p->clamp_lo, p->clamp_hi);
    const long long pixels = (long long)p->n * p->oh * p->ow;
    const uintptr_t al = (uintptr_t)a.x | (uintptr_t)a.w | (uintptr_t)a.y;
    cudaStream_t s = (cudaStream_t)stream;
    if (a.dm == 1 && (a.C % 16) == 0 && (al & 15) == 0) {
        a.total = pixels * (a.OC / 16);
        dwconv_kernel<16><<<div_up(a.total, 256), 256, 0, s>>>(a);
    } else if (a.dm == 1 && (a.C % 4) == 0 && (al & 3) == 0) {
        a.total = pixels * (a.OC / 4);
        dwconv_kernel<4><<<div_up(a.total, 256), 256, 0, s>>>(a);
    } else {
        a.total = pixels * a.OC;
        dwconv_kernel<1><<<div_up(a.total, 256), 256, 0, s>>>(a);
    }
    return check_launch("dwconv_kernel");
}
