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

// ---- 3x3, depth multiplier 1: rows of windows along x, sliding down the image ---------------------------------------
//
// A thread owns four channels (one 32-bit word of the NHWC pixel), DWR_S consecutive output columns and a block of
// output rows.  It reads every input row of its block once (DWR_S + 2 pixel words at stride 1, 2 DWR_S + 1 at stride
// 2), transposes them with byte permutes into per-channel words of consecutive pixels, and a window row is one dp4a
// against [w0, w1, w2, 0] (the window one pixel further: the same word shifted down a byte).  At stride 1 an input row
// feeds the three output rows it belongs to, whose accumulators rotate through three register sets.
// Out-of-image taps are replaced by the input zero point (their (x - zx) is 0, as in the reference, which skips them),
// and sum (x - zx)(w - zw) = sum x (w - zw) - zx sum (w - zw) with the second term as the accumulators' start value.
// Unsigned weights are taken as signed bytes w - 128 (zero point zw - 128).  A non-zero weight zero point costs a
// second dp4a per window row, against [-zw, -zw, -zw, 0]: w - zw itself does not fit a signed byte.
//
// Requantisation: one fused multiply-add per value, q" = fma(float(acc), m / sy, b / sy + zy - lo), rounded with the
// magic constant; the bound E on |reference quotient + zy - lo - q"| is the one of the tensor-core epilogue
// (conv_tc.cu, epi_chunk_fast) with this thread's four channels' maxima in it.  rint(q") counts from the lower clamp
// bound: the saturating conversion to unsigned bytes is the lower clamp, one minimum the upper one, and adding the
// lower bound (as an offset from the type's minimum) to the four bytes at once cannot carry between them; signed
// outputs flip the top bit of every byte afterwards.  A word of four channels in which some value has
// |q" - rint(q")| >= 0.5 - E is redone with the reference chain (requant_fast2; its per-channel constants wait in
// shared memory, one private slot per thread).
constexpr int DWR_S = 4;
constexpr long long DWR_MIN_THREADS = 148 * 512;    // a heuristic only: two blocks of threads per SM of a B200

struct DwRowsArgs {
    DwArgs d;
    float inv_sy, lo, hi;           // reciprocal of the output scale; clamp bounds in the output domain (zero point included)
    float zoff;                     // output zero point - lower clamp bound
    float span;                     // upper - lower clamp bound
    float e_const;                  // 3 Rmax + 2 * 257 + |zoff| of the bound E
    uint32_t lo4, flip4;            // lower clamp bound - type minimum in every byte; 0x80 in every byte for signed outputs
    int strips, rowblocks, rows;    // strips per output row, row blocks per image, output rows per block
};

// 4 x 4 byte transpose: words p[k] = one pixel's four channels -> t[c] = channel c of the four pixels
__device__ __forceinline__ void transpose4(uint32_t p0, uint32_t p1, uint32_t p2, uint32_t p3, uint32_t* t)
{
    const uint32_t a = __byte_perm(p0, p1, 0x5140), b = __byte_perm(p0, p1, 0x7362);
    const uint32_t c = __byte_perm(p2, p3, 0x5140), d = __byte_perm(p2, p3, 0x7362);
    t[0] = __byte_perm(a, c, 0x5410); t[1] = __byte_perm(a, c, 0x7632);
    t[2] = __byte_perm(b, d, 0x5410); t[3] = __byte_perm(b, d, 0x7632);
}

// FULL: the clamp is the output type's own range (the saturating conversion does all of it)
template <int STRIDE, bool XU, bool FULL, bool ZW>
__global__ void __launch_bounds__(256, 2) dw3x3_rows_kernel(const __grid_constant__ DwRowsArgs a3)
{
    __shared__ float s_mb[8][256];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const DwArgs& a = a3.d;
    constexpr int NPIX = STRIDE == 1 ? DWR_S + 2 : 2 * DWR_S + 1;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int cw = a.C >> 2;
    const int cq = (int)(idx % cw);                        // channel word
    int t = (int)(idx / cw);
    const int strip = t % a3.strips; t /= a3.strips;
    const int rb = t % a3.rowblocks;
    const int n = t / a3.rowblocks;
    const int ch0 = cq * 4;
    const uint32_t zxw = 0x01010101u * (uint32_t)(a.zx & 0xff);

    // ---- per-channel constants: nothing here depends on the kernel before this one in the stream ----
    uint32_t wA[3][4];                                     // [ky][channel]: [w(ky,0), w(ky,1), w(ky,2), 0] as signed bytes
    int init[4];
    f32x2 mq01, mq23, bq01, bq23;
    float thr;
    const int zw_eff = a.zw - (a.w_u8 ? 128 : 0);          // zero point of the weights read as signed bytes
    const uint32_t kA = 0x00010101u * (uint32_t)(-zw_eff & 0xff);
    {
        int wsum[4] = {0, 0, 0, 0};
        const uint32_t flip = a.w_u8 ? 0x80808080u : 0u;
        #pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
            const uint32_t w0 = *(const uint32_t*)(a.w + ((long long)ky * 3 + 0) * a.OC + ch0) ^ flip;
            const uint32_t w1 = *(const uint32_t*)(a.w + ((long long)ky * 3 + 1) * a.OC + ch0) ^ flip;
            const uint32_t w2 = *(const uint32_t*)(a.w + ((long long)ky * 3 + 2) * a.OC + ch0) ^ flip;
            #pragma unroll
            for (int c = 0; c < 4; ++c) {
                wA[ky][c] = gather3(w0, w1, w2, c) & 0x00ffffffu;
                wsum[c] = __dp4a((int)wA[ky][c], 0x00010101, wsum[c]);
            }
        }
        float mq[4], bq[4], bqm = 0.f, bsy = 0.f;
        #pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int ch = ch0 + c;
            init[c] = -a.zx * (wsum[c] - 9 * zw_eff);
            const float m = __fmul_rn(a.rq.sx, a.w_scales ? a.w_scales[ch] : a.w_scale);
            const float b = a.bias ? __fmul_rn(__int2float_rn(a.bias[ch]), a.b_scales ? a.b_scales[ch] : a.b_scale) : 0.f;
            s_mb[c][threadIdx.x] = m;                      // the reference chain's own constants, for the rare second pass
            s_mb[4 + c][threadIdx.x] = b;
            mq[c] = __fdiv_rn(m, a.rq.sy);
            bq[c] = epi_make_bq(b, 0, m, a.rq.sy, a3.inv_sy, a3.zoff);
            bqm = fmaxf(bqm, fabsf(bq[c]));
            bsy = fmaxf(bsy, fabsf(__fmul_rn(b, a3.inv_sy)));
        }
        mq01 = pack2(mq[0], mq[1]); mq23 = pack2(mq[2], mq[3]);
        bq01 = pack2(bq[0], bq[1]); bq23 = pack2(bq[2], bq[3]);
        // (a 3 x 3 accumulator is below 2^24: its conversion to fp32 is exact.  NaN or infinity anywhere: no hot path.)
        const float e = 1.1f * 5.9604645e-8f * (a3.e_const + 1.0001f * bsy + 3.0f * bqm);
        thr = !(e < 0.0625f) ? 0.0f : 0.5f - e;
    }
    const f32x2 magic2 = pack2(12582912.0f, 12582912.0f), nmagic2 = pack2(-12582912.0f, -12582912.0f);
    const float span = a3.span;
    const uint32_t lo4 = a3.lo4, flip4 = a3.flip4;

    const bool dump = a.acc_out != nullptr;
    const int ox0 = strip * DWR_S;
    const int ix0 = ox0 * STRIDE - a.pl;
    const int nvalid = a.OW - ox0;                         // output columns of this strip inside the image (4 or more: all)
    uint32_t cmask = 0;                                    // bit k: pixel k of the strip's input span is inside the image
    #pragma unroll
    for (int k = 0; k < NPIX; ++k) cmask |= (ix0 + k >= 0 && ix0 + k < a.W) ? (1u << k) : 0u;
    const int oy0 = rb * a3.rows;
    const int nrows = min(a3.rows, a.OH - oy0);
    const int iy0 = oy0 * STRIDE - a.pt;
    // byte offsets fit 31 bits with room for the rows and columns around the image (the launcher checks the tensor
    // sizes); pixels outside the image are never read
    const int rowpitch = a.W * a.C;
    const int xoff = (n * a.H * a.W + ix0) * a.C + ch0;    // (row iy: + iy * rowpitch); negative left of / above the first image
    const uint32_t opitch = (uint32_t)(a.OW * a.OC);
    const uint32_t yoff = (uint32_t)(((n * a.OH + oy0) * a.OW + ox0) * a.OC + ch0);

    const bool allcols = cmask == (1u << NPIX) - 1u;
    auto load_row = [&](int iy, uint32_t* px) {
        const bool rv = iy >= 0 && iy < a.H;
        const uint8_t* rp = a.x + (ptrdiff_t)(xoff + iy * rowpitch);     // (signed: a pixel outside the image may lie before a.x)
        if (allcols) {
            // (all but the strips at the left and right image edge)
            #pragma unroll
            for (int k = 0; k < NPIX; ++k) px[k] = rv ? *(const uint32_t*)(rp + k * a.C) : zxw;
        } else {
            #pragma unroll
            for (int k = 0; k < NPIX; ++k) px[k] = (rv && ((cmask >> k) & 1u)) ? *(const uint32_t*)(rp + k * a.C) : zxw;
        }
    };
    // the DWR_S windows of one input row, per channel, bytes [p, p + 1, p + 2, -]
    auto windows = [&](const uint32_t* px, uint32_t (*win)[4]) {
        if (STRIDE == 1) {
            uint32_t tt[4];
            transpose4(px[0], px[1], px[2], px[3], tt);
            const uint32_t e = __byte_perm(px[4], px[5], 0x5140), f = __byte_perm(px[4], px[5], 0x7362);
            win[2][0] = __byte_perm(tt[0], e, 0x5432); win[2][1] = __byte_perm(tt[1], e, 0x7632);
            win[2][2] = __byte_perm(tt[2], f, 0x5432); win[2][3] = __byte_perm(tt[3], f, 0x7632);
            #pragma unroll
            for (int c = 0; c < 4; ++c) { win[0][c] = tt[c]; win[1][c] = tt[c] >> 8; win[3][c] = win[2][c] >> 8; }
        } else {
            uint32_t t0[4], t1[4];
            transpose4(px[0], px[1], px[2], px[3], t0);
            transpose4(px[4], px[5], px[6], px[7], t1);
            #pragma unroll
            for (int c = 0; c < 4; ++c) {
                win[0][c] = t0[c];
                win[1][c] = __byte_perm(t0[c], t1[c], 0x4432);                         // [p2, p3, p4, -]
                win[2][c] = t1[c];
                win[3][c] = __byte_perm(t1[c], px[8], 0x0032 | ((4 + c) << 8) | ((4 + c) << 12));   // [p6, p7, p8, -]
            }
        }
    };
    auto mac = [&](const uint32_t (*win)[4], int ky, int (*acc)[4], bool fresh) {
        #pragma unroll
        for (int s = 0; s < DWR_S; ++s)
            #pragma unroll
            for (int c = 0; c < 4; ++c) {
                acc[s][c] = dp4a_mixed<XU, false>(win[s][c], wA[ky][c], fresh ? init[c] : acc[s][c]);
                if (ZW) acc[s][c] = dp4a_mixed<XU, false>(win[s][c], kA, acc[s][c]);
            }
    };
    auto emit = [&](const int (*acc)[4], int j) {          // output row oy0 + j
        const uint32_t yo = yoff + (uint32_t)j * opitch;
        uint32_t outw[DWR_S];
        float dw[DWR_S];
        #pragma unroll
        for (int s = 0; s < DWR_S; ++s) {
            const f32x2 q01 = fma2(pack2(__int2float_rn(acc[s][0]), __int2float_rn(acc[s][1])), mq01, bq01);
            const f32x2 q23 = fma2(pack2(__int2float_rn(acc[s][2]), __int2float_rn(acc[s][3])), mq23, bq23);
            const f32x2 n01 = add2(add2(q01, magic2), nmagic2), n23 = add2(add2(q23, magic2), nmagic2);   // rint(q") (exact)
            const f32x2 d01 = sub2(q01, n01), d23 = sub2(q23, n23);                                      // q" - n (exact)
            float d0, d1, d2, d3, z0, z1, z2, z3;
            unpack2(d01, d0, d1); unpack2(d23, d2, d3);
            dw[s] = fmaxf(fmaxf(fabsf(d0), fabsf(d1)), fmaxf(fabsf(d2), fabsf(d3)));
            unpack2(n01, z0, z1); unpack2(n23, z2, z3);
            if (!FULL) { z0 = fminf(z0, span); z1 = fminf(z1, span); z2 = fminf(z2, span); z3 = fminf(z3, span); }
            int i0, i1, i2, i3;
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(i0) : "f"(z0));
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(i1) : "f"(z1));
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(i2) : "f"(z2));
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(i3) : "f"(z3));
            uint32_t hi16, w;
            asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi16) : "r"(i3), "r"(i2), "r"(0));
            asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(i1), "r"(i0), "r"(hi16));
            outw[s] = (w + lo4) ^ flip4;
        }
        if (fmaxf(fmaxf(dw[0], dw[1]), fmaxf(dw[2], dw[3])) >= thr || dump) {
            // (rare) some value is too close to a rounding boundary for the hot path to vouch for: the reference chain
            // for its word of four channels; and the accumulator dump of the tests
            #pragma unroll
            for (int s = 0; s < DWR_S; ++s) {
                if (dw[s] >= thr) {
                    const f32x2 nsy2 = pack2(-a.rq.sy, -a.rq.sy), inv2 = pack2(a3.inv_sy, a3.inv_sy), zy2 = pack2((float)a.rq.zy, (float)a.rq.zy);
                    const f32x2 m01 = pack2(s_mb[0][threadIdx.x], s_mb[1][threadIdx.x]), m23 = pack2(s_mb[2][threadIdx.x], s_mb[3][threadIdx.x]);
                    const f32x2 b01 = pack2(s_mb[4][threadIdx.x], s_mb[5][threadIdx.x]), b23 = pack2(s_mb[6][threadIdx.x], s_mb[7][threadIdx.x]);
                    float r0, r1, r2, r3;
                    requant_fast2(acc[s][0], acc[s][1], m01, b01, nsy2, inv2, zy2, a3.lo, a3.hi, r0, r1);
                    requant_fast2(acc[s][2], acc[s][3], m23, b23, nsy2, inv2, zy2, a3.lo, a3.hi, r2, r3);
                    outw[s] = ((uint32_t)__float2int_rn(r0) & 0xffu) | (((uint32_t)__float2int_rn(r1) & 0xffu) << 8) |
                              (((uint32_t)__float2int_rn(r2) & 0xffu) << 16) | (((uint32_t)__float2int_rn(r3) & 0xffu) << 24);
                }
                if (dump && s < nvalid) {
                    int32_t* ao = a.acc_out + (size_t)(yo + (uint32_t)(s * a.OC));
                    #pragma unroll
                    for (int c = 0; c < 4; ++c) ao[c] = acc[s][c];
                }
            }
        }
        #pragma unroll
        for (int s = 0; s < DWR_S; ++s)
            if (s < nvalid) *(uint32_t*)(a.y + (size_t)(yo + (uint32_t)(s * a.OC))) = outw[s];
    };

    asm volatile("griddepcontrol.wait;" ::: "memory");      // the input comes from the kernel before this one

    uint32_t cur[NPIX], nxt[NPIX];
    uint32_t win[DWR_S][4];
    if (STRIDE == 1) {
        // input row r of the block (iy0 + r) is tap row 2 of output row r - 2, tap row 1 of r - 1 and tap row 0 of r
        int accA[DWR_S][4] = {}, accB[DWR_S][4] = {}, accC[DWR_S][4] = {};
        const int last = nrows + 1;                        // last input row
        load_row(iy0, nxt);
        auto step = [&](int r, int (*A)[4], int (*B)[4], int (*C)[4]) {
            #pragma unroll
            for (int k = 0; k < NPIX; ++k) cur[k] = nxt[k];
            if (r < last) load_row(iy0 + r + 1, nxt);
            windows(cur, win);
            if (r >= 2) mac(win, 2, A, false);
            if (r >= 1 && r <= nrows) mac(win, 1, B, false);
            if (r < nrows) mac(win, 0, C, true);
            if (r >= 2) emit(A, r - 2);
        };
        for (int r = 0; r <= last; r += 3) {
            step(r, accA, accB, accC);
            if (r + 1 > last) break;
            step(r + 1, accB, accC, accA);
            if (r + 2 > last) break;
            step(r + 2, accC, accA, accB);
        }
    } else {
        // even input rows of the block (iy0 + 2 j) are tap row 0 of output row j and tap row 2 of row j - 1; odd rows
        // (iy0 + 2 j + 1) are tap row 1 of row j
        int accP[DWR_S][4] = {}, accQ[DWR_S][4] = {};
        load_row(iy0, nxt);
        auto step = [&](int j, int (*P)[4], int (*Q)[4]) {  // P: output row j - 1 (completed here), Q: output row j (started here)
            #pragma unroll
            for (int k = 0; k < NPIX; ++k) cur[k] = nxt[k];
            if (j < nrows) load_row(iy0 + 2 * j + 1, nxt);
            windows(cur, win);
            if (j >= 1) { mac(win, 2, P, false); emit(P, j - 1); }
            if (j >= nrows) return;
            mac(win, 0, Q, true);
            #pragma unroll
            for (int k = 0; k < NPIX; ++k) cur[k] = nxt[k];
            load_row(iy0 + 2 * j + 2, nxt);
            windows(cur, win);
            mac(win, 1, Q, false);
        };
        for (int j = 0; j <= nrows; j += 2) {
            step(j, accP, accQ);
            if (j + 1 > nrows) break;
            step(j + 1, accQ, accP);
        }
    }
}

template <int STRIDE, bool XU, bool ZW>
static void launch_dw_rows_k(const DwRowsArgs& a, bool full, cudaStream_t s)
{
    const unsigned grid = (unsigned)div_up(a.d.total, 256);
    if (full) launch_pdl(dw3x3_rows_kernel<STRIDE, XU, true, ZW>, dim3(grid), dim3(256), 0, s, a);
    else      launch_pdl(dw3x3_rows_kernel<STRIDE, XU, false, ZW>, dim3(grid), dim3(256), 0, s, a);
}
template <int STRIDE>
static void launch_dw_rows(const DwRowsArgs& a, bool full, bool zw, cudaStream_t s)
{
    if (a.d.x_u8) { if (zw) launch_dw_rows_k<STRIDE, true, true>(a, full, s); else launch_dw_rows_k<STRIDE, true, false>(a, full, s); }
    else          { if (zw) launch_dw_rows_k<STRIDE, false, true>(a, full, s); else launch_dw_rows_k<STRIDE, false, false>(a, full, s); }
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
        const int zw_eff = a.zw - (a.w_u8 ? 128 : 0);
        if (zw_eff >= -127 && zw_eff <= 127 && ((long long)p->n * p->h + 4) * (p->wd + 4) * p->c < (1ll << 31) &&
            (long long)p->n * p->oh * p->ow * p->oc < (1ll << 31)) {
            DwRowsArgs r;
            r.d = a;
            r.inv_sy = rn_reciprocal(p->y.scale);
            r.lo = fmaxf(a.rq.tlo, (float)a.rq.clo);
            r.hi = fminf(a.rq.thi, (float)a.rq.chi);
            r.zoff = (float)a.rq.zy - r.lo;
            r.span = r.hi - r.lo;
            // |R| of the values that can round into [lo - 1, hi + 1]: at most 257 + |zoff|
            r.e_const = 3.0f * (257.0f + fabsf(r.zoff)) + 2.0f * 257.0f + fabsf(r.zoff);
            r.lo4 = 0x01010101u * (uint32_t)(int)(r.lo - a.rq.tlo);
            r.flip4 = p->y.dtype == B200K_U8 ? 0u : 0x80808080u;
            r.strips = (a.OW + DWR_S - 1) / DWR_S;
            // output rows per thread: as many as leave every SM a few blocks of threads (an input row is then read
            // (rows + 2) / rows times at stride 1)
            const long long per_row_threads = (long long)p->n * r.strips * (a.C / 4);
            int rows = 8;
            while (rows > 1 && per_row_threads * ((a.OH + rows - 1) / rows) < DWR_MIN_THREADS) rows >>= 1;
            r.rows = rows;
            r.rowblocks = (a.OH + rows - 1) / rows;
            r.d.total = per_row_threads * r.rowblocks;
            const bool full = r.lo == a.rq.tlo && r.hi == a.rq.thi;
            if (a.sh == 1) launch_dw_rows<1>(r, full, zw_eff != 0, s);
            else           launch_dw_rows<2>(r, full, zw_eff != 0, s);
            return check_launch("dw3x3_rows_kernel");
        }
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
