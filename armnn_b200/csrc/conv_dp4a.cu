// CUDA-core implicit-GEMM Convolution2d / FullyConnected for 8-bit quantised tensors (dp4a).
//
// This is the shape-agnostic kernel: any kernel size, stride, dilation, padding, channel count and
// alignment.  It is the bit-exact anchor the tcgen05 kernel is checked against and the path for
// shapes the tensor-core kernel does not take (tiny channel counts, unaligned tensors).
//
// GEMM view: rows = output pixels (n, oy, ox), columns = output channels, K = (ky, kx, c) in the
// order the NHWC input and the [O,H,W,I] weights already store it.  A 64 x 64 output tile per CTA,
// K consumed in 64-byte slices staged through shared memory (k-major, so that the 4 x 4 register
// tile of a thread is fed by two 128-bit shared loads per k-word).
//
// Zero points: operands are moved to the signed domain on load (u8 ^ 0x80, zero point - 128), taps
// that fall into the padding are filled with the input zero point and the K tail with both zero
// points, so every filled term contributes (x - zx)(w - zw) = 0.  The exact accumulator is then
//     sum x w  -  zx * sum w  -  zw * sum x  +  Kpad * zx * zw
// with the two plain sums produced by the same dp4a pipe (against 0x01010101) only when needed.
#include "common.cuh"

namespace b200k {

struct ConvArgs {
    const void* x; const void* w; const int32_t* bias; void* y; int32_t* acc_out;
    const float* w_scales; const float* b_scales;
    float w_scale, b_scale;
    int x_u8, w_u8, y_dtype;
    int zx, zw;                      // zero points in the signed domain
    int N, H, W, C, OH, OW, OC, KH, KW, sh, sw, pt, pl, dh, dw;
    int K;                           // KH*KW*C
    long long M;                     // N*OH*OW
    Requant rq;
    FusedAdd fa;
};

constexpr int BM = 64, BN = 64, BKW = 16;          // tile rows, cols, k-words (64 bytes) per slice

__device__ __forceinline__ unsigned rep4(int v) { return 0x01010101u * (unsigned)(v & 0xff); }

// MODE 2: C % 16 == 0 and 16-byte aligned tensors (128-bit loads); MODE 1: C % 4 == 0 and 4-byte
// aligned (32-bit loads); MODE 0: anything (byte gathers).
template <int MODE>
__global__ void __launch_bounds__(256) conv_dp4a_kernel(const ConvArgs a)
{
    __shared__ __align__(16) unsigned As[BKW][BM];
    __shared__ __align__(16) unsigned Bs[BKW][BN];

    const int tid = threadIdx.x;
    const int lrow = tid & 63;            // row (pixel / channel) this thread stages
    const int lg   = tid >> 6;            // which 16-byte group of the 64-byte slice
    const long long m0 = (long long)blockIdx.x * BM;
    const int n0 = blockIdx.y * BN;

    // geometry of the pixel this thread stages
    const long long pm = m0 + lrow;
    const bool pvalid = pm < a.M;
    int pn = 0, iy0 = 0, ix0 = 0;
    if (pvalid) {
        int ox = (int)(pm % a.OW);
        long long t = pm / a.OW;
        int oy = (int)(t % a.OH);
        pn = (int)(t / a.OH);
        iy0 = oy * a.sh - a.pt;
        ix0 = ox * a.sw - a.pl;
    }
    const int wch = n0 + lrow;            // output channel this thread stages
    const bool wvalid = wch < a.OC;
    const unsigned xfill = rep4(a.zx), wfill = rep4(a.zw);
    const unsigned xflip = a.x_u8 ? 0x80808080u : 0u, wflip = a.w_u8 ? 0x80808080u : 0u;
    const uint8_t* xb = (const uint8_t*)a.x;
    const uint8_t* wb = (const uint8_t*)a.w;

    unsigned ra[4], rb[4];

    auto x_byte = [&](int k) -> unsigned {       // one input byte of this thread's pixel, signed domain
        if (k >= a.K || !pvalid) return (unsigned)(a.zx & 0xff);
        int tap = k / a.C, c = k - tap * a.C;
        int ky = tap / a.KW, kx = tap - ky * a.KW;
        int iy = iy0 + ky * a.dh, ix = ix0 + kx * a.dw;
        if (iy < 0 || iy >= a.H || ix < 0 || ix >= a.W) return (unsigned)(a.zx & 0xff);
        unsigned v = xb[(((long long)pn * a.H + iy) * a.W + ix) * a.C + c];
        return (v ^ (xflip & 0xff)) & 0xff;
    };

    auto load_slice = [&](int k0) {
        const int kb = k0 + lg * 16;              // first byte of this thread's group
        // ---- A (input pixels) ----
        if (MODE == 2) {
            uint4 v = make_uint4(xfill, xfill, xfill, xfill);
            if (pvalid && kb < a.K) {
                int tap = kb / a.C, c = kb - tap * a.C;
                int ky = tap / a.KW, kx = tap - ky * a.KW;
                int iy = iy0 + ky * a.dh, ix = ix0 + kx * a.dw;
                if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W) {
                    v = *(const uint4*)(xb + (((long long)pn * a.H + iy) * a.W + ix) * a.C + c);
                    v.x ^= xflip; v.y ^= xflip; v.z ^= xflip; v.w ^= xflip;
                }
            }
            ra[0] = v.x; ra[1] = v.y; ra[2] = v.z; ra[3] = v.w;
        } else if (MODE == 1) {
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                int k = kb + j * 4;
                unsigned v = xfill;
                if (pvalid && k < a.K) {
                    int tap = k / a.C, c = k - tap * a.C;
                    int ky = tap / a.KW, kx = tap - ky * a.KW;
                    int iy = iy0 + ky * a.dh, ix = ix0 + kx * a.dw;
                    if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W)
                        v = *(const unsigned*)(xb + (((long long)pn * a.H + iy) * a.W + ix) * a.C + c) ^ xflip;
                }
                ra[j] = v;
            }
        } else {
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                int k = kb + j * 4;
                ra[j] = x_byte(k) | (x_byte(k + 1) << 8) | (x_byte(k + 2) << 16) | (x_byte(k + 3) << 24);
            }
        }
        // ---- B (weights, row = output channel, K contiguous) ----
        if (MODE == 2) {
            uint4 v = make_uint4(wfill, wfill, wfill, wfill);
            if (wvalid && kb < a.K) {
                v = *(const uint4*)(wb + (long long)wch * a.K + kb);
                v.x ^= wflip; v.y ^= wflip; v.z ^= wflip; v.w ^= wflip;
            }
            rb[0] = v.x; rb[1] = v.y; rb[2] = v.z; rb[3] = v.w;
        } else if (MODE == 1) {
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                int k = kb + j * 4;
                rb[j] = (wvalid && k < a.K) ? (*(const unsigned*)(wb + (long long)wch * a.K + k) ^ wflip) : wfill;
            }
        } else {
            #pragma unroll
            for (int j = 0; j < 4; ++j) {
                unsigned v = 0;
                #pragma unroll
                for (int b = 0; b < 4; ++b) {
                    int k = kb + j * 4 + b;
                    unsigned byte = (wvalid && k < a.K)
                                  ? ((wb[(long long)wch * a.K + k] ^ (wflip & 0xff)) & 0xff)
                                  : (unsigned)(a.zw & 0xff);
                    v |= byte << (8 * b);
                }
                rb[j] = v;
            }
        }
    };

    const int ty = tid >> 4, tx = tid & 15;
    int acc[4][4];
    int sa[4] = {0, 0, 0, 0}, sb[4] = {0, 0, 0, 0};
    #pragma unroll
    for (int i = 0; i < 4; ++i)
        #pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0;

    const bool need_sa = a.zw != 0, need_sb = a.zx != 0;
    const int nslices = (a.K + 63) / 64;
    load_slice(0);
    for (int s = 0; s < nslices; ++s) {
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            As[lg * 4 + j][lrow] = ra[j];
            Bs[lg * 4 + j][lrow] = rb[j];
        }
        __syncthreads();
        if (s + 1 < nslices) load_slice((s + 1) * 64);
        #pragma unroll
        for (int kw = 0; kw < BKW; ++kw) {
            const uint4 av = *(const uint4*)&As[kw][ty * 4];
            const uint4 bv = *(const uint4*)&Bs[kw][tx * 4];
            const int aa[4] = {(int)av.x, (int)av.y, (int)av.z, (int)av.w};
            const int bb[4] = {(int)bv.x, (int)bv.y, (int)bv.z, (int)bv.w};
            #pragma unroll
            for (int i = 0; i < 4; ++i)
                #pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __dp4a(aa[i], bb[j], acc[i][j]);
            if (need_sa) {
                #pragma unroll
                for (int i = 0; i < 4; ++i) sa[i] = __dp4a(aa[i], 0x01010101, sa[i]);
            }
            if (need_sb) {
                #pragma unroll
                for (int j = 0; j < 4; ++j) sb[j] = __dp4a(bb[j], 0x01010101, sb[j]);
            }
        }
        __syncthreads();
    }

    // ---- epilogue ----
    const int kpad = nslices * 64;
    const int kzz = kpad * a.zx * a.zw;
    int q[4];
    #pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long m = m0 + ty * 4 + i;
        if (m >= a.M) continue;
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int ch = n0 + tx * 4 + j;
            q[j] = 0;
            if (ch >= a.OC) continue;
            const int v = acc[i][j] - a.zx * sb[j] - a.zw * sa[i] + kzz;
            if (a.acc_out) a.acc_out[m * a.OC + ch] = v;
            const float swc = a.w_scales ? a.w_scales[ch] : a.w_scale;
            const float sbc = a.b_scales ? a.b_scales[ch] : a.b_scale;
            const int bq = a.bias ? a.bias[ch] : 0;
            q[j] = a.rq(v, swc, a.bias != nullptr, bq, sbc);
            if (a.fa.res) q[j] = a.fa(q[j], a.rq, m * a.OC + ch);
        }
        const int ch0 = n0 + tx * 4;
        uint8_t* yp = (uint8_t*)a.y + m * a.OC + ch0;
        if (ch0 + 3 < a.OC && ((a.OC & 3) == 0) && ((((uintptr_t)a.y) & 3) == 0)) {
            *(unsigned*)yp = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((unsigned)(q[3] & 0xff) << 24);
        } else {
            #pragma unroll
            for (int j = 0; j < 4; ++j)
                if (ch0 + j < a.OC) yp[j] = (uint8_t)q[j];
        }
    }
}

static int validate_common(const b200k_qtensor& x, const b200k_qtensor& w, const b200k_qtensor& bias,
                           const b200k_qtensor& y, bool y_stored, const char* what)
{
    B200K_REQUIRE(x.data && w.data && (y.data || !y_stored), B200K_E_INVALID, "%s: null tensor pointer", what);
    B200K_REQUIRE(is_q8(x.dtype) && is_q8(w.dtype) && is_q8(y.dtype), B200K_E_UNSUPPORTED,
                  "%s: only 8-bit quantised input/weights/output are supported (got %d/%d/%d)", what,
                  x.dtype, w.dtype, y.dtype);
    B200K_REQUIRE(!bias.data || bias.dtype == B200K_S32, B200K_E_INVALID, "%s: bias must be Signed32", what);
    B200K_REQUIRE(x.scale > 0.f && y.scale > 0.f, B200K_E_INVALID, "%s: non-positive scale", what);
    return B200K_OK;
}

int launch_conv_dp4a(const b200k_conv2d_params* p, cudaStream_t stream)
{
    int rc = validate_common(p->x, p->w, p->bias, p->y, p->add_operand.data == nullptr, "conv2d_q8");
    if (rc) return rc;
    B200K_REQUIRE(p->n > 0 && p->h > 0 && p->wd > 0 && p->c > 0 && p->oh > 0 && p->ow > 0 && p->oc > 0 &&
                  p->kh > 0 && p->kw > 0 && p->stride_h > 0 && p->stride_w > 0 && p->dil_h > 0 && p->dil_w > 0 &&
                  p->pad_top >= 0 && p->pad_left >= 0, B200K_E_INVALID, "conv2d_q8: bad geometry");
    const long long kk = (long long)p->kh * p->kw * p->c;
    B200K_REQUIRE(kk < (1ll << 30), B200K_E_TOOBIG, "conv2d_q8: K = %lld too large", kk);
    ConvArgs a;
    a.x = p->x.data; a.w = p->w.data; a.bias = (const int32_t*)p->bias.data; a.y = (void*)p->y.data;
    a.acc_out = p->acc_out;
    a.w_scales = p->w.scales; a.b_scales = p->bias.scales;
    a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.x_u8 = p->x.dtype == B200K_U8; a.w_u8 = p->w.dtype == B200K_U8; a.y_dtype = p->y.dtype;
    a.zx = p->x.zero_point - (a.x_u8 ? 128 : 0);
    a.zw = p->w.zero_point - (a.w_u8 ? 128 : 0);
    B200K_REQUIRE(a.zx >= -128 && a.zx <= 127 && a.zw >= -128 && a.zw <= 127, B200K_E_INVALID,
                  "conv2d_q8: zero point outside the element type's range");
    a.N = p->n; a.H = p->h; a.W = p->wd; a.C = p->c; a.OH = p->oh; a.OW = p->ow; a.OC = p->oc;
    a.KH = p->kh; a.KW = p->kw; a.sh = p->stride_h; a.sw = p->stride_w; a.pt = p->pad_top; a.pl = p->pad_left;
    a.dh = p->dil_h; a.dw = p->dil_w;
    a.K = (int)kk;
    a.M = (long long)p->n * p->oh * p->ow;
    B200K_REQUIRE(make_fused_add(p, a.rq, a.fa, a.y), B200K_E_INVALID, "conv2d_q8: malformed fused add operand / output");
    dim3 grid(div_up(a.M, BM), div_up(a.OC, BN));
    const uintptr_t al = (uintptr_t)a.x | (uintptr_t)a.w;
    if ((a.C % 16) == 0 && (al & 15) == 0)      conv_dp4a_kernel<2><<<grid, 256, 0, stream>>>(a);
    else if ((a.C % 4) == 0 && (al & 3) == 0)   conv_dp4a_kernel<1><<<grid, 256, 0, stream>>>(a);
    else                                         conv_dp4a_kernel<0><<<grid, 256, 0, stream>>>(a);
    return check_launch("conv_dp4a_kernel");
}

}  // namespace b200k
