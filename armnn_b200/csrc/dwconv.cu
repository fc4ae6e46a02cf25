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
    pdl_enter();
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

// ---- 3x3, depth multiplier 1, stride 1 or 2: the MobileNet shapes ------------------------------------------------
//
// A thread owns four channels (one 32-bit word of the NHWC pixel) and a strip of DW_STRIP output pixels of one output
// row; consecutive threads walk the channel axis, so loads and stores are coalesced.  The three input rows of a
// window column are transposed (two byte permutes per channel) into one word per channel [row0, row1, row2, -], so a
// window column costs one dp4a per channel against the equally transposed weights, and a column is loaded and
// transposed once however many windows it belongs to.  Zero points: out-of-image taps are replaced by the input zero
// point (their (x - zx) is 0, as in the reference, which skips them), and
//     sum (x - zx)(w - zw) = sum x w - zw sum x - (zx sum w - 9 zx zw)
// with the column sums of x from one more dp4a per column and channel and the bracket a per-channel constant.
constexpr int DW_STRIP = 8;

// bytes c of three words -> one word [a.c, b.c, c.c, a.0]
__device__ __forceinline__ uint32_t gather3(uint32_t r0, uint32_t r1, uint32_t r2, int c)
{
    const uint32_t t = __byte_perm(r0, r1, ((4 + c) << 4) | c);
    return __byte_perm(t, r2, ((4 + c) << 8) | 0x10);
}

struct Dw3Args {
    DwArgs d;
    float inv_sy, lo, hi;
    int strips;                     // strips per output row
};

template <int STRIDE, bool XU, bool WU>
__global__ void __launch_bounds__(256) dwconv3x3_kernel(const Dw3Args a3)
{
    pdl_enter();
    const DwArgs& a = a3.d;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int cw = a.C / 4;
    const int cq = (int)(idx % cw);                        // channel word
    long long t = idx / cw;
    const int strip = (int)(t % a3.strips); t /= a3.strips;
    const int oy = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    const int ch0 = cq * 4;
    const uint32_t zxw = 0x01010101u * (uint32_t)(a.zx & 0xff);

    // weights of the four channels, transposed per window column; per-channel constants
    uint32_t wcol[3][4];
    int kconst[4];
    float m[4], b[4];
    {
        uint32_t wr[3][3];
        #pragma unroll
        for (int ky = 0; ky < 3; ++ky)
            #pragma unroll
            for (int kx = 0; kx < 3; ++kx) wr[ky][kx] = *(const uint32_t*)(a.w + ((long long)ky * 3 + kx) * a.OC + ch0);
        #pragma unroll
        for (int c = 0; c < 4; ++c) {
            int wsum = 0;
            #pragma unroll
            for (int kx = 0; kx < 3; ++kx) {
                wcol[kx][c] = gather3(wr[0][kx], wr[1][kx], wr[2][kx], c) & 0x00ffffffu;
                wsum = WU ? (int)__dp4a(wcol[kx][c], 0x00010101u, (unsigned)wsum) : __dp4a((int)wcol[kx][c], 0x00010101, wsum);
            }
            kconst[c] = a.zx * wsum - 9 * a.zx * a.zw;
            const int ch = ch0 + c;
            m[c] = __fmul_rn(a.rq.sx, a.w_scales ? a.w_scales[ch] : a.w_scale);
            b[c] = a.bias ? __fmul_rn(__int2float_rn(a.bias[ch]), a.b_scales ? a.b_scales[ch] : a.b_scale) : 0.f;
        }
    }
    const f32x2 m01 = pack2(m[0], m[1]), m23 = pack2(m[2], m[3]), b01 = pack2(b[0], b[1]), b23 = pack2(b[2], b[3]);
    const f32x2 nsy2 = pack2(-a.rq.sy, -a.rq.sy), inv2 = pack2(a3.inv_sy, a3.inv_sy), zy2 = pack2((float)a.rq.zy, (float)a.rq.zy);
    const int iy0 = oy * STRIDE - a.pt;
    const bool rv0 = iy0 >= 0 && iy0 < a.H, rv1 = iy0 + 1 >= 0 && iy0 + 1 < a.H, rv2 = iy0 + 2 >= 0 && iy0 + 2 < a.H;
    const uint8_t* row0 = a.x + (((long long)n * a.H + iy0) * a.W) * a.C + ch0;
    const uint8_t* row1 = row0 + (long long)a.W * a.C;
    const uint8_t* row2 = row1 + (long long)a.W * a.C;

    // one window column: three rows of the channel word at input column ix, transposed; and its byte sums
    uint32_t xcol[3][4];
    int xsum[3][4];
    auto load_col = [&](int slot, int ix) {
        const bool cv = ix >= 0 && ix < a.W;
        const long long off = (long long)ix * a.C;
        const uint32_t r0 = (cv && rv0) ? *(const uint32_t*)(row0 + off) : zxw;
        const uint32_t r1 = (cv && rv1) ? *(const uint32_t*)(row1 + off) : zxw;
        const uint32_t r2 = (cv && rv2) ? *(const uint32_t*)(row2 + off) : zxw;
        #pragma unroll
        for (int c = 0; c < 4; ++c) {
            xcol[slot][c] = gather3(r0, r1, r2, c);
            xsum[slot][c] = a.zw != 0 ? dp4a_mixed<XU, true>(xcol[slot][c], 0x00010101u, 0) : 0;
        }
    };

    const int ox0 = strip * DW_STRIP;
    int ix = ox0 * STRIDE - a.pl;
    load_col(0, ix); load_col(1, ix + 1); load_col(2, ix + 2);
    #pragma unroll
    for (int s = 0; s < DW_STRIP; ++s) {
        const int ox = ox0 + s;
        if (ox >= a.OW) break;
        if (s > 0) {
            if (STRIDE == 1) {
                #pragma unroll
                for (int c = 0; c < 4; ++c) {
                    xcol[0][c] = xcol[1][c]; xsum[0][c] = xsum[1][c];
                    xcol[1][c] = xcol[2][c]; xsum[1][c] = xsum[2][c];
                }
                load_col(2, ix + 2);
            } else {
                #pragma unroll
                for (int c = 0; c < 4; ++c) { xcol[0][c] = xcol[2][c]; xsum[0][c] = xsum[2][c]; }
                load_col(1, ix + 1); load_col(2, ix + 2);
            }
        }
        const long long ob = (((long long)n * a.OH + oy) * a.OW + ox) * a.OC + ch0;
        int acc[4];
        #pragma unroll
        for (int c = 0; c < 4; ++c) {
            acc[c] = 0;
            #pragma unroll
            for (int j = 0; j < 3; ++j) acc[c] = dp4a_mixed<XU, WU>(xcol[j][c], wcol[j][c], acc[c]);
            acc[c] -= a.zw * (xsum[0][c] + xsum[1][c] + xsum[2][c]) + kconst[c];
            if (a.acc_out) a.acc_out[ob + c] = acc[c];
        }
        // exact requantisation, two channels per instruction (b is 0 without a bias: adding it changes nothing, as the
        // sum of a finite value and +0 is that value)
        float r[4];
        requant_fast2(acc[0], acc[1], m01, b01, nsy2, inv2, zy2, a3.lo, a3.hi, r[0], r[1]);
        requant_fast2(acc[2], acc[3], m23, b23, nsy2, inv2, zy2, a3.lo, a3.hi, r[2], r[3]);
        const uint32_t outw = ((uint32_t)__float2int_rn(r[0]) & 0xffu) | (((uint32_t)__float2int_rn(r[1]) & 0xffu) << 8) |
                              (((uint32_t)__float2int_rn(r[2]) & 0xffu) << 16) | (((uint32_t)__float2int_rn(r[3]) & 0xffu) << 24);
        *(uint32_t*)(a.y + ob) = outw;
        ix += STRIDE;
    }
}

template <int STRIDE>
static void launch_dw3(const Dw3Args& a, cudaStream_t s)
{
    const unsigned grid = (unsigned)div_up(a.d.total, 256);
    if (a.d.x_u8) {
        if (a.d.w_u8) launch_pdl(dwconv3x3_kernel<STRIDE, true, true>, dim3((unsigned)(grid)), dim3(256), 0, s, a);
        else          launch_pdl(dwconv3x3_kernel<STRIDE, true, false>, dim3((unsigned)(grid)), dim3(256), 0, s, a);
    } else {
        if (a.d.w_u8) launch_pdl(dwconv3x3_kernel<STRIDE, false, true>, dim3((unsigned)(grid)), dim3(256), 0, s, a);
        else          launch_pdl(dwconv3x3_kernel<STRIDE, false, false>, dim3((unsigned)(grid)), dim3(256), 0, s, a);
    }
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
    if (a.dm == 1 && a.KH == 3 && a.KW == 3 && a.dh == 1 && a.dw == 1 && a.sh == a.sw && (a.sh == 1 || a.sh == 2) &&
        (a.C % 4) == 0 && (al & 3) == 0) {
        Dw3Args a3;
        a3.d = a;
        a3.inv_sy = rn_reciprocal(p->y.scale);
        a3.lo = fmaxf(a.rq.tlo, (float)a.rq.clo);
        a3.hi = fminf(a.rq.thi, (float)a.rq.chi);
        a3.strips = (a.OW + DW_STRIP - 1) / DW_STRIP;
        a3.d.total = (long long)p->n * p->oh * a3.strips * (a.C / 4);
        if (a.sh == 1) launch_dw3<1>(a3, s);
        else           launch_dw3<2>(a3, s);
        return check_launch("dwconv3x3_kernel");
    }
    if (a.dm == 1 && (a.C % 16) == 0 && (al & 15) == 0) {
        a.total = pixels * (a.OC / 16);
        launch_pdl(dwconv_kernel<16>, dim3((unsigned)(div_up(a.total, 256))), dim3(256), 0, s, a);
    } else if (a.dm == 1 && (a.C % 4) == 0 && (al & 3) == 0) {
        a.total = pixels * (a.OC / 4);
        launch_pdl(dwconv_kernel<4>, dim3((unsigned)(div_up(a.total, 256))), dim3(256), 0, s, a);
    } else {
        a.total = pixels * a.OC;
        launch_pdl(dwconv_kernel<1>, dim3((unsigned)(div_up(a.total, 256))), dim3(256), 0, s, a);
    }
    return check_launch("dwconv_kernel");
}
