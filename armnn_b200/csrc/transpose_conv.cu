// TransposeConvolution2d (NHWC, weights [OC, KH, KW, C]) in gather form: an output element sums the taps (ky, kx) whose
// source pixel ((y + pad_top - ky) / stride_h, (x + pad_left - kx) / stride_w) exists, which visits exactly the products
// the reference's scatter loop adds to it (src/backends/reference/workloads/TransposeConvolution2d.cpp:57-128).  Exact
// int32 accumulation of (x - zx)(w - zw), then the contraction epilogue (Requant).  A CUDA-core kernel: one thread per
// output element, dp4a over the channel axis when it is a multiple of four; not on the benchmarked path.
#include "common.cuh"

namespace b200k {

struct TconvArgs {
    const uint8_t* x; const uint8_t* w; const int32_t* bias; uint8_t* y; int32_t* acc_out;
    const float* w_scales; const float* b_scales;
    float w_scale, b_scale;
    int x_u8, w_u8, zx, zw;
    int N, H, W, C, OH, OW, OC, KH, KW, sh, sw, pt, pl;
    long long total;
    Requant rq;
};

template <bool XU, bool WU>
__global__ void __launch_bounds__(256) transpose_conv_kernel(const TconvArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    const int co = (int)(i % a.OC);
    long long t = i / a.OC;
    const int ox = (int)(t % a.OW); t /= a.OW;
    const int oy = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    int acc = 0;
    const bool vec = (a.C & 3) == 0 && (((uintptr_t)a.x | (uintptr_t)a.w) & 3) == 0;
    for (int ky = 0; ky < a.KH; ++ky) {
        const int ty = oy + a.pt - ky;
        if (ty < 0 || ty % a.sh != 0) continue;
        const int iy = ty / a.sh;
        if (iy >= a.H) continue;
        for (int kx = 0; kx < a.KW; ++kx) {
            const int tx = ox + a.pl - kx;
            if (tx < 0 || tx % a.sw != 0) continue;
            const int ix = tx / a.sw;
            if (ix >= a.W) continue;
            const uint8_t* xp = a.x + (((long long)n * a.H + iy) * a.W + ix) * a.C;
            const uint8_t* wp = a.w + (((long long)co * a.KH + ky) * a.KW + kx) * a.C;
            if (vec) {
                // sum (x - zx)(w - zw) = sum x w - zw sum x - zx sum w + C zx zw
                int xw = 0, sx = 0, sw = 0;
                for (int c = 0; c < a.C; c += 4) {
                    const uint32_t xv = *(const uint32_t*)(xp + c), wv = *(const uint32_t*)(wp + c);
                    xw = dp4a_mixed<XU, WU>(xv, wv, xw);
                    sx = dp4a_mixed<XU, false>(xv, 0x01010101u, sx);
                    sw = dp4a_mixed<false, WU>(0x01010101u, wv, sw);
                }
                acc += xw - a.zw * sx - a.zx * sw + a.C * a.zx * a.zw;
            } else {
                for (int c = 0; c < a.C; ++c) {
                    const int xv = XU ? (int)xp[c] : (int)(int8_t)xp[c];
                    const int wv = WU ? (int)wp[c] : (int)(int8_t)wp[c];
                    acc += (xv - a.zx) * (wv - a.zw);
                }
            }
        }
    }
    if (a.acc_out) a.acc_out[i] = acc;
    const float swc = a.w_scales ? a.w_scales[co] : a.w_scale;
    const float sbc = a.b_scales ? a.b_scales[co] : a.b_scale;
    a.y[i] = (uint8_t)a.rq(acc, swc, a.bias != nullptr, a.bias ? a.bias[co] : 0, sbc);
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_transpose_conv2d_q8(const b200k_conv2d_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "transpose_conv2d_q8: null params");
    B200K_REQUIRE(p->x.data && p->w.data && p->y.data, B200K_E_INVALID, "transpose_conv2d_q8: null tensor pointer");
    B200K_REQUIRE(is_q8(p->x.dtype) && is_q8(p->w.dtype) && is_q8(p->y.dtype), B200K_E_UNSUPPORTED,
                  "transpose_conv2d_q8: only 8-bit quantised tensors are supported");
    B200K_REQUIRE(!p->bias.data || p->bias.dtype == B200K_S32, B200K_E_INVALID, "transpose_conv2d_q8: bias must be Signed32");
    B200K_REQUIRE(!p->add_operand.data, B200K_E_UNSUPPORTED, "transpose_conv2d_q8: a fused Add is only available on Convolution2d");
    B200K_REQUIRE(p->n > 0 && p->h > 0 && p->wd > 0 && p->c > 0 && p->oh > 0 && p->ow > 0 && p->oc > 0 && p->kh > 0 && p->kw > 0 &&
                  p->stride_h > 0 && p->stride_w > 0 && p->pad_top >= 0 && p->pad_left >= 0, B200K_E_INVALID,
                  "transpose_conv2d_q8: bad geometry");
    TconvArgs a;
    a.x = (const uint8_t*)p->x.data; a.w = (const uint8_t*)p->w.data; a.bias = (const int32_t*)p->bias.data;
    a.y = (uint8_t*)p->y.data; a.acc_out = p->acc_out;
    a.w_scales = p->w.scales; a.b_scales = p->bias.scales; a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.x_u8 = p->x.dtype == B200K_U8; a.w_u8 = p->w.dtype == B200K_U8;
    a.zx = p->x.zero_point; a.zw = p->w.scales ? 0 : p->w.zero_point;
    a.N = p->n; a.H = p->h; a.W = p->wd; a.C = p->c; a.OH = p->oh; a.OW = p->ow; a.OC = p->oc;
    a.KH = p->kh; a.KW = p->kw; a.sh = p->stride_h; a.sw = p->stride_w; a.pt = p->pad_top; a.pl = p->pad_left;
    a.total = (long long)p->n * p->oh * p->ow * p->oc;
    a.rq = make_requant(p->x.scale, p->y, p->clamp_lo, p->clamp_hi);
    const dim3 grid(div_up(a.total, 256)), block(256);
    cudaStream_t s = (cudaStream_t)stream;
    if (a.x_u8) { if (a.w_u8) launch_pdl(transpose_conv_kernel<true, true>, grid, block, 0, s, a); else launch_pdl(transpose_conv_kernel<true, false>, grid, block, 0, s, a); }
    else        { if (a.w_u8) launch_pdl(transpose_conv_kernel<false, true>, grid, block, 0, s, a); else launch_pdl(transpose_conv_kernel<false, false>, grid, block, 0, s, a); }
    return check_launch("transpose_conv_kernel");
}
