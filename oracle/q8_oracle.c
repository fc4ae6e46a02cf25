/*
 * q8_oracle.c — TEST INFRASTRUCTURE ONLY.  A plain-C CPU restatement of the Arm NN CpuRef
 * arithmetic for the quantised operator hot path.  Nothing in the product (libb200k.so, the
 * B200Acc backend, armnn_b200/) links, loads or calls this file; only tests/, the smoke check
 * and the CPU-baseline leg of bench.py do, and only as the checker.
 *
 * Parity is pinned: tests/test_oracle_*.py check every function here against (i) known-answer
 * vectors transcribed from the reference's own layer tests (tests/golden/ref_layer_tests.json)
 * and (ii) outputs of the real CpuRef workloads compiled from the reference sources
 * (oracle/_ref/, driven by tests/test_oracle_vs_cpuref.py).
 *
 * Two kinds of restatement, because CpuRef computes everything in fp32:
 *  - contractions (conv / depthwise / fully-connected / batch-matmul): CpuRef sums
 *    deq(x)*deq(w) in a float.  Here the sum is an exact int32 accumulator over the same loop
 *    nest and index formulas, followed by ONE fp32 requantisation.  This is the function the
 *    GPU must match bit for bit (accumulator and output); it equals CpuRef except on rounding
 *    ties (+-1 LSB).
 *  - everything else (pooling, mean, elementwise, activation, softmax, quantize/dequantize):
 *    the same fp32 operations in the same order as CpuRef, so results equal CpuRef's exactly
 *    (up to libm exp/tanh differences where those are used).
 *
 * Parameter structs are the ones of include/b200k.h, with HOST pointers.
 * Build: gcc -O2 -fPIC -shared -ffp-contract=off -fopenmp (oracle/Makefile).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include "../include/b200k.h"
#include "move_desc.h"

/* ---- armnn::Quantize / armnn::Dequantize, src/armnn/TypesUtils.cpp:29-56 ------------------- */

static void type_range(int dtype, int32_t* lo, int32_t* hi)
{
    switch (dtype) {
        case B200K_U8:  *lo = 0;       *hi = 255;    break;
        case B200K_S8:  *lo = -128;    *hi = 127;    break;
        case B200K_S16: *lo = -32768;  *hi = 32767;  break;
        default:        *lo = INT32_MIN; *hi = INT32_MAX; break;
    }
}

/* q = clamp(float(zp) + round(v / scale), type_min, type_max), TypesUtils.cpp:38-41 */
static int32_t quantize_f(float v, float scale, int32_t zp, int dtype)
{
    int32_t lo, hi;
    type_range(dtype, &lo, &hi);
    volatile float d = v / scale;           /* volatile: keep the division in fp32, unfused */
    float r = roundf(d);
    float q = (float)zp + r;
    q = fminf(fmaxf(q, (float)lo), (float)hi);
    return (int32_t)q;
}

/* v = float(q - zp) * scale, TypesUtils.cpp:48-56 */
static float dequantize_i(int32_t q, float scale, int32_t zp)
{
    return (float)(q - zp) * scale;
}

static int32_t load_q(const void* p, int dtype, int64_t i)
{
    switch (dtype) {
        case B200K_U8:  return ((const uint8_t*)p)[i];
        case B200K_S8:  return ((const int8_t*)p)[i];
        case B200K_S16: return ((const int16_t*)p)[i];
        case B200K_S32: return ((const int32_t*)p)[i];
        default: return 0;
    }
}

static void store_q(void* p, int dtype, int64_t i, int32_t q)
{
    switch (dtype) {
        case B200K_U8:  ((uint8_t*)p)[i]  = (uint8_t)q;  break;
        case B200K_S8:  ((int8_t*)p)[i]   = (int8_t)q;   break;
        case B200K_S16: ((int16_t*)p)[i]  = (int16_t)q;  break;
        case B200K_S32: ((int32_t*)p)[i]  = q;           break;
        default: break;
    }
}

/* Decoder<float>::Get for any supported element type (Decoders.hpp:63-126) */
static float load_f(const b200k_qtensor* t, int64_t i)
{
    if (t->dtype == B200K_F32) return ((const float*)t->data)[i];
    return dequantize_i(load_q(t->data, t->dtype, i), t->scale, t->zero_point);
}

/* Encoder<float>::Set (Encoders.hpp:18-91) */
static void store_f(const b200k_qtensor* t, int64_t i, float v)
{
    if (t->dtype == B200K_F32) { ((float*)t->data)[i] = v; return; }
    store_q((void*)t->data, t->dtype, i, quantize_f(v, t->scale, t->zero_point, t->dtype));
}

static int32_t clampi(int32_t v, int32_t lo, int32_t hi) { return v < lo ? lo : (v > hi ? hi : v); }

int oracle_activation_clamp(int kind, float a, float b, float scale, int32_t zp, int32_t dtype,
                            int32_t* lo, int32_t* hi)
{
    type_range(dtype, lo, hi);
    if (kind == 1) {                       /* ReLu: max(0, x) */
        int32_t q0 = quantize_f(0.0f, scale, zp, dtype);
        if (q0 > *lo) *lo = q0;
    } else if (kind == 2) {                /* BoundedReLu: min(a, max(b, x)) */
        int32_t qb = quantize_f(b, scale, zp, dtype);
        int32_t qa = quantize_f(a, scale, zp, dtype);
        if (qb > *lo) *lo = qb;
        if (qa < *hi) *hi = qa;
    } else if (kind != 0) {
        return B200K_E_INVALID;
    }
    return 0;
}

/* The one requantisation shared by all contractions:
 *   v = float(acc) * (sx * sw) + float(bias) * sb ;  q = Quantize(v, sy, zy) ; clamp */
static int32_t requant(int32_t acc, float sx, float sw, int has_bias, int32_t bq, float sb,
                       float sy, int32_t zy, int dtype, int32_t clo, int32_t chi)
{
    volatile float m = sx * sw;
    volatile float v = (float)acc * m;
    if (has_bias) {
        volatile float bf = (float)bq * sb;
        v = v + bf;
    }
    return clampi(quantize_f(v, sy, zy, dtype), clo, chi);
}

/* ---- Convolve, ConvImpl.cpp:68-233 (NHWC; weights [O,H,W,I], depthwise [1,H,W,O]) ----------- */

static int conv_impl(const b200k_conv2d_params* p, int depthwise)
{
    const int N = p->n, H = p->h, W = p->wd, C = p->c, OH = p->oh, OW = p->ow, OC = p->oc;
    const int KH = p->kh, KW = p->kw;
    const int zx = p->x.zero_point, zw = p->w.zero_point;
    const int dm = depthwise ? OC / C : 1;          /* ConvImpl.cpp:100 */
    const int fused = !depthwise && p->add_operand.data != NULL;
    if (!p->x.data || !p->w.data || (!fused && !p->y.data) || (fused && !p->add_out.data)) return B200K_E_INVALID;
    int32_t ylo, yhi;
    type_range(p->y.dtype, &ylo, &yhi);
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < N; ++b)
    for (int oy = 0; oy < OH; ++oy)
    for (int ox = 0; ox < OW; ++ox)
    for (int co = 0; co < OC; ++co) {
        int32_t acc = 0;
        for (int ky = 0; ky < KH; ++ky) {
            int iy = oy * p->stride_h + ky * p->dil_h - p->pad_top;   /* :165, :170 */
            if (iy < 0 || iy >= H) continue;                          /* padding tap: adds 0.0 */
            for (int kx = 0; kx < KW; ++kx) {
                int ix = ox * p->stride_w + kx * p->dil_w - p->pad_left;
                if (ix < 0 || ix >= W) continue;
                if (depthwise) {
                    int ci = co / dm;                                         /* :138 */
                    int64_t wi = (int64_t)kx * OC + co + (int64_t)ky * KW * OC; /* :140-141 */
                    int64_t xi = (((int64_t)b * H + iy) * W + ix) * C + ci;
                    acc += (load_q(p->x.data, p->x.dtype, xi) - zx) *
                           (load_q(p->w.data, p->w.dtype, wi) - zw);
                } else {
                    int64_t wb = (((int64_t)co * KH + ky) * KW + kx) * C;      /* :149-152 */
                    int64_t xb = (((int64_t)b * H + iy) * W + ix) * C;         /* :185-188 */
                    if (p->x.dtype == B200K_S8 && p->w.dtype == B200K_S8) {
                        const int8_t* xp = (const int8_t*)p->x.data + xb;
                        const int8_t* wp = (const int8_t*)p->w.data + wb;
                        int32_t s = 0;
                        for (int ci = 0; ci < C; ++ci) s += ((int)xp[ci] - zx) * ((int)wp[ci] - zw);
                        acc += s;
                    } else if (p->x.dtype == B200K_U8 && p->w.dtype == B200K_U8) {
                        const uint8_t* xp = (const uint8_t*)p->x.data + xb;
                        const uint8_t* wp = (const uint8_t*)p->w.data + wb;
                        int32_t s = 0;
                        for (int ci = 0; ci < C; ++ci) s += ((int)xp[ci] - zx) * ((int)wp[ci] - zw);
                        acc += s;
                    } else {
                        for (int ci = 0; ci < C; ++ci)
                            acc += (load_q(p->x.data, p->x.dtype, xb + ci) - zx) *
                                   (load_q(p->w.data, p->w.dtype, wb + ci) - zw);
                    }
                }
            }
        }
        int64_t oi = (((int64_t)b * OH + oy) * OW + ox) * OC + co;             /* :214-217 */
        if (p->acc_out) p->acc_out[oi] = acc;
        float sw = p->w.scales ? p->w.scales[co] : p->w.scale;
        int has_bias = p->bias.data != NULL;
        int32_t bq = has_bias ? ((const int32_t*)p->bias.data)[co] : 0;
        float sb = p->bias.scales ? p->bias.scales[co] : p->bias.scale;
        if (fused) {
            /* RefConvolution2dWorkload, then RefElementwiseBinaryWorkload(Add) on its 8-bit output, then the clamp */
            int32_t q1 = requant(acc, p->x.scale, sw, has_bias, bq, sb, p->y.scale, p->y.zero_point, p->y.dtype, ylo, yhi);
            volatile float fa = dequantize_i(q1, p->y.scale, p->y.zero_point);
            volatile float fb = load_f(&p->add_operand, oi);
            volatile float r = fa + fb;
            store_q((void*)p->add_out.data, p->add_out.dtype, oi,
                    clampi(quantize_f(r, p->add_out.scale, p->add_out.zero_point, p->add_out.dtype), p->clamp_lo, p->clamp_hi));
            continue;
        }
        store_q((void*)p->y.data, p->y.dtype, oi,
                requant(acc, p->x.scale, sw, has_bias, bq, sb, p->y.scale, p->y.zero_point,
                        p->y.dtype, p->clamp_lo, p->clamp_hi));
    }
    return 0;
}

int oracle_conv2d_q8(const b200k_conv2d_params* p)   { return conv_impl(p, 0); }
int oracle_dwconv2d_q8(const b200k_conv2d_params* p) { return conv_impl(p, 1); }

/* ---- Float32 Convolve (ConvImpl.cpp:118-232) and FullyConnected (FullyConnected.cpp:32-62) -------
 * The reference's loops and its fp32 accumulation order (this file is built with -ffp-contract=off: a rounded
 * product and a rounded sum per term); padding taps add w * 0. */
static int conv_f32_impl(const b200k_conv2d_params* p, int depthwise)
{
    if (!p || !p->x.data || !p->w.data || !p->y.data || p->x.dtype != B200K_F32 || p->w.dtype != B200K_F32 || p->y.dtype != B200K_F32)
        return B200K_E_INVALID;
    const int N = p->n, H = p->h, W = p->wd, C = p->c, OH = p->oh, OW = p->ow, OC = p->oc, KH = p->kh, KW = p->kw;
    const float* x = (const float*)p->x.data; const float* w = (const float*)p->w.data;
    const float* bias = (const float*)p->bias.data; float* y = (float*)p->y.data;
    const int dm = depthwise ? OC / C : 1;
    for (int b = 0; b < N; ++b) for (int co = 0; co < OC; ++co) for (int oy = 0; oy < OH; ++oy) for (int ox = 0; ox < OW; ++ox) {
        float sum = 0.0f;
        for (int c = 0; c < (depthwise ? 1 : C); ++c) {
            const int ci = depthwise ? co / dm : c;
            for (int ky = 0; ky < KH; ++ky) for (int kx = 0; kx < KW; ++kx) {
                const int iy = oy * p->stride_h + ky * p->dil_h - p->pad_top, ix = ox * p->stride_w + kx * p->dil_w - p->pad_left;
                const float wv = depthwise ? w[((int64_t)ky * KW + kx) * OC + co] : w[(((int64_t)co * KH + ky) * KW + kx) * C + ci];
                const float xv = (iy < 0 || iy >= H || ix < 0 || ix >= W) ? 0.0f : x[(((int64_t)b * H + iy) * W + ix) * C + ci];
                sum += wv * xv;
            }
        }
        if (bias) sum += bias[co];
        y[(((int64_t)b * OH + oy) * OW + ox) * OC + co] = sum;
    }
    return 0;
}

int oracle_conv2d_f32(const b200k_conv2d_params* p)   { return conv_f32_impl(p, 0); }
int oracle_dwconv2d_f32(const b200k_conv2d_params* p) { return conv_f32_impl(p, 1); }

int oracle_fully_connected_f32(const b200k_fc_params* p)
{
    if (!p || !p->x.data || !p->w.data || !p->y.data || p->x.dtype != B200K_F32 || p->w.dtype != B200K_F32 || p->y.dtype != B200K_F32)
        return B200K_E_INVALID;
    const float* x = (const float*)p->x.data; const float* w = (const float*)p->w.data;
    const float* bias = (const float*)p->bias.data; float* y = (float*)p->y.data;
    for (int m = 0; m < p->m; ++m) for (int o = 0; o < p->n; ++o) {
        float out = 0.f;
        for (int k = 0; k < p->k; ++k) {
            const float wv = p->transpose_w ? w[(int64_t)o * p->k + k] : w[(int64_t)k * p->n + o];
            out += wv * x[(int64_t)m * p->k + k];
        }
        if (bias) out += bias[o];
        y[(int64_t)m * p->n + o] = out;
    }
    return 0;
}

/* ---- TransposeConvolution2dImpl, TransposeConvolution2d.cpp:14-160 (NHWC, weights [O,H,W,I]) ---
 * The reference's scatter loop nest with an exact int32 accumulator per output element instead of its float buffer,
 * then bias and quantisation through the contractions' one requantisation. */
int oracle_transpose_conv2d_q8(const b200k_conv2d_params* p)
{
    if (!p || !p->x.data || !p->w.data || !p->y.data) return B200K_E_INVALID;
    const int N = p->n, H = p->h, W = p->wd, C = p->c, OH = p->oh, OW = p->ow, OC = p->oc, KH = p->kh, KW = p->kw;
    const int zx = p->x.zero_point, zw = p->w.zero_point;
    const int64_t total = (int64_t)N * OH * OW * OC;
    int32_t* acc = (int32_t*)calloc((size_t)total, sizeof(int32_t));
    if (!acc) return B200K_E_INVALID;
    for (int b = 0; b < N; ++b)
    for (int yi = 0; yi < H; ++yi)
    for (int xi = 0; xi < W; ++xi) {
        const int xo0 = xi * p->stride_w - p->pad_left, yo0 = yi * p->stride_h - p->pad_top;      /* :61-62 */
        for (int co = 0; co < OC; ++co)
        for (int ky = 0; ky < KH; ++ky)
        for (int kx = 0; kx < KW; ++kx) {
            const int yo = yo0 + ky, xo = xo0 + kx;
            if (yo < 0 || yo >= OH || xo < 0 || xo >= OW) continue;                               /* :73 (unsigned compare) */
            const int64_t xb = (((int64_t)b * H + yi) * W + xi) * C;
            const int64_t wb = (((int64_t)co * KH + ky) * KW + kx) * C;
            int32_t s = 0;
            for (int ci = 0; ci < C; ++ci)
                s += (load_q(p->x.data, p->x.dtype, xb + ci) - zx) * (load_q(p->w.data, p->w.dtype, wb + ci) - zw);
            acc[(((int64_t)b * OH + yo) * OW + xo) * OC + co] += s;
        }
    }
    for (int64_t i = 0; i < total; ++i) {
        const int co = (int)(i % OC);
        if (p->acc_out) p->acc_out[i] = acc[i];
        const float sw = p->w.scales ? p->w.scales[co] : p->w.scale;
        const int has_bias = p->bias.data != NULL;
        const int32_t bq = has_bias ? ((const int32_t*)p->bias.data)[co] : 0;
        const float sb = p->bias.scales ? p->bias.scales[co] : p->bias.scale;
        store_q((void*)p->y.data, p->y.dtype, i,
                requant(acc[i], p->x.scale, sw, has_bias, bq, sb, p->y.scale, p->y.zero_point, p->y.dtype, p->clamp_lo, p->clamp_hi));
    }
    free(acc);
    return 0;
}

/* ---- FullyConnected, FullyConnected.cpp:13-65 --------------------------------------------- */

int oracle_fully_connected_q8(const b200k_fc_params* p)
{
    const int M = p->m, K = p->k, N = p->n;
    const int zx = p->x.zero_point, zw = p->w.zero_point;
    if (!p->x.data || !p->w.data || !p->y.data) return B200K_E_INVALID;
    #pragma omp parallel for schedule(static)
    for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
        int32_t acc = 0;
        for (int k = 0; k < K; ++k) {
            int64_t wi = p->transpose_w ? (int64_t)n * K + k : (int64_t)k * N + n;   /* :43-51 */
            acc += (load_q(p->x.data, p->x.dtype, (int64_t)m * K + k) - zx) *
                   (load_q(p->w.data, p->w.dtype, wi) - zw);
        }
        int64_t oi = (int64_t)m * N + n;
        if (p->acc_out) p->acc_out[oi] = acc;
        float sw = p->w.scales ? p->w.scales[n] : p->w.scale;
        int has_bias = p->bias.data != NULL;
        int32_t bq = has_bias ? ((const int32_t*)p->bias.data)[n] : 0;
        float sb = p->bias.scales ? p->bias.scales[n] : p->bias.scale;
        store_q((void*)p->y.data, p->y.dtype, oi,
                requant(acc, p->x.scale, sw, has_bias, bq, sb, p->y.scale, p->y.zero_point,
                        p->y.dtype, p->clamp_lo, p->clamp_hi));
    }
    return 0;
}

/* ---- BatchMatMul, BatchMatMulImpl.cpp:40-78 (sum over the shared axis, then Set) ------------- */

int oracle_batch_matmul_q8(const b200k_bmm_params* p)
{
    const int B = p->batch, M = p->m, K = p->k, N = p->n;
    if (!p->x.data || !p->y.data || !p->out.data) return B200K_E_INVALID;
    int32_t lo, hi;
    type_range(p->out.dtype, &lo, &hi);
    for (int b = 0; b < B; ++b)
    for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
        int32_t acc = 0;
        for (int k = 0; k < K; ++k) {
            int64_t xi = b * p->batch_stride_x + (p->transpose_x ? (int64_t)k * M + m : (int64_t)m * K + k);
            int64_t yi = b * p->batch_stride_y + (p->transpose_y ? (int64_t)n * K + k : (int64_t)k * N + n);
            acc += (load_q(p->x.data, p->x.dtype, xi) - p->x.zero_point) *
                   (load_q(p->y.data, p->y.dtype, yi) - p->y.zero_point);
        }
        int64_t oi = ((int64_t)b * M + m) * N + n;
        if (p->acc_out) p->acc_out[oi] = acc;
        store_q((void*)p->out.data, p->out.dtype, oi,
                requant(acc, p->x.scale, p->y.scale, 0, 0, 0.f, p->out.scale, p->out.zero_point,
                        p->out.dtype, lo, hi));
    }
    return 0;
}

int oracle_batch_matmul_f32(const b200k_bmm_params* p)
{
    const int B = p->batch, M = p->m, K = p->k, N = p->n;
    if (!p->x.data || !p->y.data || !p->out.data) return B200K_E_INVALID;
    for (int b = 0; b < B; ++b)
    for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
        volatile float sum = 0.0f;
        for (int k = 0; k < K; ++k) {
            const int64_t xi = b * p->batch_stride_x + (p->transpose_x ? (int64_t)k * M + m : (int64_t)m * K + k);
            const int64_t yi = b * p->batch_stride_y + (p->transpose_y ? (int64_t)n * K + k : (int64_t)k * N + n);
            volatile float prod = ((const float*)p->x.data)[xi] * ((const float*)p->y.data)[yi];
            sum = sum + prod;
        }
        ((float*)p->out.data)[((int64_t)b * M + m) * N + n] = sum;
    }
    return 0;
}

/* ---- Pooling2d, Pooling2d.cpp:142-303 ----------------------------------------------------- */

static int clamp_range(int* s, int* e, int maxr)       /* Pooling2d.cpp:121-134 */
{
    if (*s < 0 || *e > maxr) {
        int a = *s < 0 ? 0 : *s;  if (a > maxr) a = maxr;
        int b = *e < 0 ? 0 : *e;  if (b > maxr) b = maxr;
        *s = a; *e = b;
        return 1;
    }
    return 0;
}

int oracle_pool2d_q8(const b200k_pool2d_params* p)
{
    const int N = p->n, H = p->h, W = p->wd, C = p->c, OH = p->oh, OW = p->ow;
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    if (p->pool_type < 0 || p->pool_type > 2) return B200K_E_INVALID;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c)
    for (int oy = 0; oy < OH; ++oy) {
        int hstart = oy * p->stride_h - p->pad_top;
        int hend = hstart + p->pool_h;
        if (hend > H + p->pad_bottom) hend = H + p->pad_bottom;          /* :194 */
        int height = hend - hstart;
        int hclamped = clamp_range(&hstart, &hend, H);
        for (int ox = 0; ox < OW; ++ox) {
            int wstart = ox * p->stride_w - p->pad_left;
            int wend = wstart + p->pool_w;
            if (wend > W + p->pad_right) wend = W + p->pad_right;        /* :206 */
            float result = p->pool_type == 0 ? -3.402823466e+38f : 0.0f;
            float area = (float)(height * (wend - wstart));              /* :209 */
            int64_t oi = (((int64_t)n * OH + oy) * OW + ox) * C + c;
            /* window entirely inside the padding: 0 by convention, :216-241 (OnPaddingOnly) */
            if ((hend <= 0 || hstart > H) || (wend <= 0 || wstart > W)) {
                store_f(&p->y, oi, 0.0f);
                continue;
            }
            hclamped |= clamp_range(&wstart, &wend, W);                  /* :243 (sticky) */
            if (hclamped && p->padding_method == 1)                      /* Exclude, :245-250 */
                area = (float)((hend - hstart) * (wend - wstart));
            for (int iy = hstart; iy < hend; ++iy)
            for (int ix = wstart; ix < wend; ++ix) {
                float v = load_f(&p->x, (((int64_t)n * H + iy) * W + ix) * C + c);
                if (p->pool_type == 0) { if (v > result) result = v; }
                else if (p->pool_type == 1) { volatile float s = result + v; result = s; }
                else { volatile float sq = v * v; volatile float s = result + sq; result = s; }
            }
            if (p->pool_type == 1) { volatile float q = result / area; result = q; }
            else if (p->pool_type == 2) { volatile float q = result / area; result = sqrtf(q); }
            store_f(&p->y, oi, result);
        }
    }
    return 0;
}

/* ---- Mean over H,W, Reduce.cpp:68-173 --------------------------------------------------------- */

int oracle_mean_hw_q8(const b200k_mean_params* p)
{
    const int N = p->n, H = p->h, W = p->wd, C = p->c;
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    for (int n = 0; n < N; ++n)
    for (int c = 0; c < C; ++c) {
        float acc = 0.0f;
        for (int i = 0; i < H * W; ++i) {          /* row-major visit order == h, then w */
            volatile float s = acc + load_f(&p->x, ((int64_t)n * H * W + i) * C + c);
            acc = s;
        }
        volatile float m = acc / (float)(H * W);
        store_f(&p->y, (int64_t)n * C + c, m);
    }
    return 0;
}

/* ---- ElementwiseBinary, RefElementwiseBinaryWorkload.cpp:27-132 + Broadcast.hpp:13-104 ------- */

int oracle_eltwise_q8(const b200k_eltwise_params* p)
{
    int sa[4], sb[4], so[4], da[4] = {1,1,1,1}, db[4] = {1,1,1,1}, dout[4] = {1,1,1,1};
    if (p->rank < 1 || p->rank > 4) return B200K_E_INVALID;
    for (int i = 0; i < p->rank; ++i) {
        da[4 - p->rank + i] = p->shape_a[i];
        db[4 - p->rank + i] = p->shape_b[i];
        dout[4 - p->rank + i] = p->shape_out[i];
    }
    int64_t ta = 1, tb = 1, to = 1;
    for (int i = 3; i >= 0; --i) {
        sa[i] = da[i] == 1 ? 0 : (int)ta;  ta *= da[i];
        sb[i] = db[i] == 1 ? 0 : (int)tb;  tb *= db[i];
        so[i] = (int)to;                   to *= dout[i];
    }
    for (int i0 = 0; i0 < dout[0]; ++i0)
    for (int i1 = 0; i1 < dout[1]; ++i1)
    for (int i2 = 0; i2 < dout[2]; ++i2)
    for (int i3 = 0; i3 < dout[3]; ++i3) {
        int64_t ia = (int64_t)i0 * sa[0] + (int64_t)i1 * sa[1] + (int64_t)i2 * sa[2] + (int64_t)i3 * sa[3];
        int64_t ib = (int64_t)i0 * sb[0] + (int64_t)i1 * sb[1] + (int64_t)i2 * sb[2] + (int64_t)i3 * sb[3];
        int64_t io = (int64_t)i0 * so[0] + (int64_t)i1 * so[1] + (int64_t)i2 * so[2] + (int64_t)i3 * so[3];
        float a = load_f(&p->a, ia), b = load_f(&p->b, ib);
        volatile float r;
        switch (p->op) {
            case 0: r = a + b; break;
            case 1: r = a / b; break;
            case 2: r = a > b ? a : b; break;
            case 3: r = a < b ? a : b; break;
            case 4: r = a * b; break;
            case 5: r = a - b; break;
            case 6: { volatile float d = a - b; r = d * d; break; }
            case 7: r = powf(a, b); break;                                    /* Power.hpp:19-24 */
            case 8: r = (float)floor((double)a / (double)b); break;           /* FloorDiv.hpp:15-19 */
            case B200K_ELTWISE_PRELU: r = a < 0 ? b * a : a; break;           /* PreluImpl.cpp:25-28 */
            /* RefComparisonWorkload.cpp:60-104 and RefLogicalBinaryWorkload.cpp:33-56: a Boolean byte, 0 or 1 */
            case 200: r = a == b; break;
            case 201: r = a > b; break;
            case 202: r = a >= b; break;
            case 203: r = a < b; break;
            case 204: r = a <= b; break;
            case 205: r = a != b; break;
            case 210: r = (a != 0) && (b != 0); break;
            case 211: r = (a != 0) || (b != 0); break;
            default: return B200K_E_INVALID;
        }
        if (p->out.dtype == B200K_F32) { ((float*)p->out.data)[io] = r; continue; }
        int32_t q = quantize_f(r, p->out.scale, p->out.zero_point, p->out.dtype);
        store_q((void*)p->out.data, p->out.dtype, io, clampi(q, p->clamp_lo, p->clamp_hi));
    }
    return 0;
}

/* ---- Activation, Activation.cpp:13-119 ---------------------------------------------------------- */

static float activation_f(float in, int fn, float a, float b)
{
    switch (fn) {
        case 0:  return 1.f / (1.f + expf(-in));
        case 1:  return a * tanhf(b * in);
        case 2:  { volatile float t = a * in; return t + b; }
        case 3:  return in > 0.f ? in : 0.f;
        case 4:  { float t = in > b ? in : b; return t < a ? t : a; }
        case 5:  return logf(1.0f + expf(in));
        case 6:  return in > 0.0f ? in : (in * a);
        case 7:  return in < 0 ? -in : in;
        case 8:  return sqrtf(in);
        case 9:  return in * in;
        case 10: return (in >= 0) ? in : a * (expf(in) - 1);
        case 11: { volatile float t = in + 3; float r = t > 0.0f ? t : 0.0f; r = r < 6.0f ? r : 6.0f;
                   volatile float m = in * r; return m / 6; }
        case 12: return in * (0.5f * (1.0f + erff((float)(in / sqrt(2.0)))));          /* Activation.cpp:85-91 */
        case B200K_ACTIVATION_FAKE_QUANTIZATION: {                  /* RefFakeQuantizationFloat32Workload.cpp:15-27 */
            volatile float range = b - a;
            const float scale = range / 255.f;
            volatile float num = -a * 255.f;
            const int32_t offset = (int32_t)(num / range);
            return (float)quantize_f(in, scale, offset, B200K_U8);
        }
        default: return NAN;
    }
}

/* ElementwiseUnary, RefElementwiseUnaryWorkload.cpp:36-110: y = Q_y(f(deq_x(x))) with the std:: function of the operation */
int oracle_unary_q(const b200k_unary_params* p)
{
    if (!p || !p->x.data || !p->y.data || p->operation < 0 || p->operation > 9) return B200K_E_INVALID;
    for (int64_t i = 0; i < p->count; ++i) {
        const float in = load_f(&p->x, i);
        float r;
        switch (p->operation) {
            case 0: r = fabsf(in); break;
            case 1: r = expf(in); break;
            case 2: r = sqrtf(in); break;
            case 3: r = 1 / sqrtf(in); break;
            case 4: r = -in; break;
            case 5: r = in != 0 ? 0.f : 1.f; break;        /* RefLogicalUnaryWorkload.cpp: LogicalNot of a Boolean byte */
            case 6: r = logf(in); break;
            case 7: r = sinf(in); break;
            case 9: r = floorf(in); break;                 /* RefFloorWorkload.cpp */
            default: r = ceilf(in); break;
        }
        store_f(&p->y, i, r);
    }
    return 0;
}

int oracle_activation_q8(const b200k_activation_params* p)
{
    if (!p->x.data || !p->y.data || p->function < 0 || (p->function > 12 && p->function != B200K_ACTIVATION_FAKE_QUANTIZATION)) return B200K_E_INVALID;
    for (int64_t i = 0; i < p->count; ++i)
        store_f(&p->y, i, activation_f(load_f(&p->x, i), p->function, p->a, p->b));
    return 0;
}

/* ---- Softmax, Softmax.cpp:17-70 --------------------------------------------------------------- */

int oracle_softmax_q8(const b200k_softmax_params* p)
{
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    for (int o = 0; o < p->outer; ++o)
    for (int in = 0; in < p->inner; ++in) {
        int64_t base = (int64_t)o * p->axis_size * p->inner + in;
        float mx = -3.402823466e+38f;
        for (int i = 0; i < p->axis_size; ++i) {
            float v = load_f(&p->x, base + (int64_t)i * p->inner);
            if (v > mx) mx = v;
        }
        float sum = 0.0f;
        for (int i = 0; i < p->axis_size; ++i) {
            volatile float d = load_f(&p->x, base + (int64_t)i * p->inner) - mx;
            volatile float t = d * p->beta;
            volatile float s = sum + expf(t);
            sum = s;
        }
        for (int i = 0; i < p->axis_size; ++i) {
            volatile float d = load_f(&p->x, base + (int64_t)i * p->inner) - mx;
            volatile float t = d * p->beta;
            volatile float r = expf(t) / sum;
            store_f(&p->y, base + (int64_t)i * p->inner, r);
        }
    }
    return 0;
}

/* ---- LogSoftmax, LogSoftmax.cpp:30-88 ----------------------------------------------------------- */

int oracle_log_softmax_q(const b200k_softmax_params* p)
{
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    for (int o = 0; o < p->outer; ++o)
    for (int in = 0; in < p->inner; ++in) {
        int64_t base = (int64_t)o * p->axis_size * p->inner + in;
        float mx = load_f(&p->x, base);
        for (int i = 1; i < p->axis_size; ++i) {
            float v = load_f(&p->x, base + (int64_t)i * p->inner);
            if (v > mx) mx = v;
        }
        float sum = 0.0f;
        for (int i = 0; i < p->axis_size; ++i) {
            volatile float d = load_f(&p->x, base + (int64_t)i * p->inner) - mx;
            volatile float t = d * p->beta;
            volatile float s = sum + expf(t);
            sum = s;
        }
        const float log_sum = logf(sum);
        for (int i = 0; i < p->axis_size; ++i) {
            volatile float d = load_f(&p->x, base + (int64_t)i * p->inner) - mx;
            volatile float t = d * p->beta;
            volatile float r = t - log_sum;
            store_f(&p->y, base + (int64_t)i * p->inner, r);
        }
    }
    return 0;
}

/* ---- L2Normalization, RefL2NormalizationWorkload.cpp:29-93: beta carries eps --------------------- */

int oracle_l2_normalization_q(const b200k_softmax_params* p)
{
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    for (int o = 0; o < p->outer; ++o)
    for (int in = 0; in < p->inner; ++in) {
        int64_t base = (int64_t)o * p->axis_size * p->inner + in;
        float reduction = 0.0f;
        for (int i = 0; i < p->axis_size; ++i) {
            const float v = load_f(&p->x, base + (int64_t)i * p->inner);
            volatile float sq = v * v;
            volatile float s = reduction + sq;
            reduction = s;
        }
        const float maximum = reduction < p->beta ? p->beta : reduction;
        const float scale = 1.0f / sqrtf(maximum);
        for (int i = 0; i < p->axis_size; ++i) {
            volatile float r = load_f(&p->x, base + (int64_t)i * p->inner) * scale;
            store_f(&p->y, base + (int64_t)i * p->inner, r);
        }
    }
    return 0;
}

/* ---- ArgMinMax, ArgMinMax.cpp:16-48 ------------------------------------------------------------- */

int oracle_arg_min_max_q(const b200k_arg_min_max_params* p)
{
    if (!p->x.data || !p->y) return B200K_E_INVALID;
    for (int o = 0; o < p->outer; ++o)
    for (int in = 0; in < p->inner; ++in) {
        int64_t base = (int64_t)o * p->axis_size * p->inner + in;
        float best = load_f(&p->x, base);
        int idx = 0;
        for (int i = 1; i < p->axis_size; ++i) {
            const float v = load_f(&p->x, base + (int64_t)i * p->inner);
            if ((p->function == 0 && v < best) || (p->function == 1 && v > best)) { best = v; idx = i; }
        }
        const int64_t at = (int64_t)o * p->inner + in;
        if (p->out_int64) ((int64_t*)p->y)[at] = idx; else ((int32_t*)p->y)[at] = idx;
    }
    return 0;
}

/* ---- Gather, Gather.cpp:16-94 --------------------------------------------------------------------
 * An index outside the axis makes the reference throw; here it yields the encoding of 0.0 (what the CUDA path stores). */

int oracle_gather_q(const b200k_gather_params* p)
{
    if (!p->x.data || !p->y.data || !p->indices) return B200K_E_INVALID;
    int64_t out = 0;
    for (int o = 0; o < p->outer; ++o)
    for (int j = 0; j < p->n_indices; ++j) {
        int64_t idx = p->indices[j];
        if (idx < 0) idx += p->axis_size;
        for (int k = 0; k < p->inner; ++k, ++out) {
            if (idx < 0 || idx >= p->axis_size) { store_f(&p->y, out, 0.0f); continue; }
            store_f(&p->y, out, load_f(&p->x, ((int64_t)o * p->axis_size + idx) * p->inner + k));
        }
    }
    return 0;
}

/* ---- ReverseV2, ReverseV2Impl.cpp:14-133 --------------------------------------------------------------- */

int oracle_reverse_q(const b200k_reverse_params* p)
{
    if (!p->x.data || !p->y.data || p->rank < 1 || p->rank > 6) return B200K_E_INVALID;
    int flag[6] = {0, 0, 0, 0, 0, 0};
    for (int k = 0; k < p->n_axes; ++k) {
        int ax = p->axes[k];
        if (ax < 0) ax += p->rank;
        if (ax >= 0 && ax < p->rank) flag[ax] = 1;
    }
    int64_t count = 1;
    for (int d = 0; d < p->rank; ++d) count *= p->shape[d];
    for (int64_t i = 0; i < count; ++i) {
        int64_t rest = i, dst = 0, stride = 1;
        for (int d = p->rank - 1; d >= 0; --d) {
            int64_t c = rest % p->shape[d];
            rest /= p->shape[d];
            if (flag[d]) c = p->shape[d] - 1 - c;
            dst += c * stride;
            stride *= p->shape[d];
        }
        store_f(&p->y, dst, load_f(&p->x, i));
    }
    return 0;
}

/* ---- GatherNd without batch dimensions, RefGatherNdWorkload.cpp:20-92 ------------------------------ */

int oracle_gather_nd_q(const b200k_gather_nd_params* p)
{
    if (!p->x.data || !p->y.data || !p->indices || p->nd < 1 || p->nd > 8) return B200K_E_INVALID;
    int64_t rows = 1, coeff[8];
    for (int d = p->nd - 1; d >= 0; --d) { coeff[d] = rows; rows *= p->dims[d]; }
    for (int j = 0; j < p->n_indices; ++j) {
        int64_t flat = 0;
        int ok = 1;
        for (int d = 0; d < p->nd; ++d) {
            const int32_t t = p->indices[(int64_t)j * p->nd + d];
            if (t < 0) ok = 0;
            flat += (int64_t)t * coeff[d];
        }
        if (flat >= rows) ok = 0;
        for (int k = 0; k < p->inner; ++k) {
            const int64_t out = (int64_t)j * p->inner + k;
            if (!ok) { store_f(&p->y, out, 0.0f); continue; }
            store_f(&p->y, out, load_f(&p->x, flat * p->inner + k));
        }
    }
    return 0;
}

/* ---- BatchNormalization, BatchNormImpl.cpp:16-63 -------------------------------------------------- */

int oracle_batch_norm_q(const b200k_batch_norm_params* p)
{
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    for (int c = 0; c < p->c; ++c) {
        const float mean = load_f(&p->mean, c), var = load_f(&p->variance, c), beta = load_f(&p->beta, c), gamma = load_f(&p->gamma, c);
        volatile float ve = var + p->eps;
        const float mult = gamma / sqrtf(ve);
        volatile float mm = mult * mean;
        const float add = beta - mm;
        for (int n = 0; n < p->n; ++n)
        for (int64_t k = 0; k < p->hw; ++k) {
            const int64_t at = p->nchw ? ((int64_t)n * p->c + c) * p->hw + k : ((int64_t)n * p->hw + k) * p->c + c;
            volatile float m = mult * load_f(&p->x, at);
            volatile float r = m + add;
            store_f(&p->y, at, r);
        }
    }
    return 0;
}

/* ---- InstanceNormalization, InstanceNorm.cpp:16-84 ------------------------------------------------ */

int oracle_instance_norm_q(const b200k_instance_norm_params* p)
{
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    for (int n = 0; n < p->n; ++n)
    for (int c = 0; c < p->c; ++c) {
        const int64_t base = p->nchw ? ((int64_t)n * p->c + c) * p->hw : (int64_t)n * p->hw * p->c + c;
        const int64_t step = p->nchw ? 1 : p->c;
        volatile float mean = 0, var = 0;
        for (int64_t k = 0; k < p->hw; ++k) mean = mean + load_f(&p->x, base + k * step);
        mean = mean / (float)p->hw;
        for (int64_t k = 0; k < p->hw; ++k) {
            volatile float d = load_f(&p->x, base + k * step) - mean;
            volatile float sq = d * d;
            var = var + sq;
        }
        var = var / (float)p->hw;
        volatile float ve = var + p->eps;
        const float root = sqrtf(ve);
        for (int64_t k = 0; k < p->hw; ++k) {
            volatile float d = load_f(&p->x, base + k * step) - mean;
            volatile float g = d * p->gamma;
            volatile float q = g / root;
            volatile float r = q + p->beta;
            store_f(&p->y, base + k * step, r);
        }
    }
    return 0;
}

/* ---- Normalization (LocalBrightness), RefNormalizationWorkload.cpp:19-140 -------------------------- */

int oracle_normalization_q(const b200k_normalization_params* p)
{
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    const int radius = (int)(p->norm_size / 2);
    const int64_t hw = (int64_t)p->h * p->w;
    if (p->channel_type == 1) {
        if (!p->nchw) return B200K_E_UNSUPPORTED;
        for (int n = 0; n < p->n; ++n) for (int c = 0; c < p->c; ++c)
        for (int h = 0; h < p->h; ++h) for (int w = 0; w < p->w; ++w) {
            volatile float acc = 0.0f;
            for (int y = -radius; y <= radius; ++y) for (int x = -radius; x <= radius; ++x) {
                const int i = w + x, j = h + y;
                if (i < 0 || i >= p->w || j < 0 || j >= p->h) continue;
                const float v = load_f(&p->x, ((int64_t)n * p->c + c) * hw + (int64_t)j * p->w + i);
                volatile float sq = v * v;
                acc = acc + sq;
            }
            const int64_t at = ((int64_t)n * p->c + c) * hw + (int64_t)h * p->w + w;
            volatile float sa = acc * p->alpha;
            volatile float base = p->kappa + sa;
            volatile float r = load_f(&p->x, at) / powf(base, p->beta);
            store_f(&p->y, at, r);
        }
        return 0;
    }
    if (p->channel_type != 0) return B200K_E_INVALID;
    for (int n = 0; n < p->n; ++n) for (int c = 0; c < p->c; ++c)
    for (int64_t k = 0; k < hw; ++k) {
        volatile float acc = 0.0f;
        for (int z = -radius; z <= radius; ++z) {
            const int cc = c + z;
            if (cc < 0 || cc >= p->c) continue;
            const float v = load_f(&p->x, p->nchw ? ((int64_t)n * p->c + cc) * hw + k : ((int64_t)n * hw + k) * p->c + cc);
            volatile float sq = v * v;
            acc = acc + sq;
        }
        const int64_t at = p->nchw ? ((int64_t)n * p->c + c) * hw + k : ((int64_t)n * hw + k) * p->c + c;
        volatile float sa = acc * p->alpha;
        volatile float base = p->kappa + sa;
        volatile float r = powf(base, -p->beta) * load_f(&p->x, at);
        store_f(&p->y, at, r);
    }
    return 0;
}

/* ---- Convolution3d, Conv3dImpl.cpp:14-177 (NDHWC, weights [D, H, W, I, O]) ------------------------- */

int oracle_conv3d_q(const b200k_conv3d_params* p)
{
    if (!p->x.data || !p->w.data || !p->y.data) return B200K_E_INVALID;
    const int f32 = p->x.dtype == B200K_F32;
    const int zx = p->x.zero_point, zw = p->w.zero_point;
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < p->n; ++b)
    for (int oz = 0; oz < p->od; ++oz)
    for (int oy = 0; oy < p->oh; ++oy)
    for (int ox = 0; ox < p->ow; ++ox)
    for (int co = 0; co < p->oc; ++co) {
        int32_t acc = 0;
        volatile float sum = 0.0f;
        for (int kz = 0; kz < p->kd; ++kz) {
            const int iz = oz * p->stride_d + kz * p->dil_d - p->pad_front;
            for (int ky = 0; ky < p->kh; ++ky) {
                const int iy = oy * p->stride_h + ky * p->dil_h - p->pad_top;
                for (int kx = 0; kx < p->kw; ++kx) {
                    const int ix = ox * p->stride_w + kx * p->dil_w - p->pad_left;
                    const int inside = iz >= 0 && iz < p->d && iy >= 0 && iy < p->h && ix >= 0 && ix < p->wd;
                    const int64_t xb = ((((int64_t)b * p->d + iz) * p->h + iy) * p->wd + ix) * p->c;
                    const int64_t wb = ((((int64_t)kz * p->kh + ky) * p->kw + kx) * p->c) * p->oc + co;
                    for (int ci = 0; ci < p->c; ++ci) {
                        if (f32) {
                            const float xv = inside ? ((const float*)p->x.data)[xb + ci] : 0.0f;      /* :96-103 */
                            volatile float prod = ((const float*)p->w.data)[wb + (int64_t)ci * p->oc] * xv;
                            sum = sum + prod;
                        } else if (inside) {
                            acc += (load_q(p->x.data, p->x.dtype, xb + ci) - zx) *
                                   (load_q(p->w.data, p->w.dtype, wb + (int64_t)ci * p->oc) - zw);
                        }
                    }
                }
            }
        }
        const int64_t oi = ((((int64_t)b * p->od + oz) * p->oh + oy) * p->ow + ox) * p->oc + co;
        if (f32) {
            if (p->bias.data) sum = sum + ((const float*)p->bias.data)[co];
            ((float*)p->y.data)[oi] = sum;
            continue;
        }
        const float sw = p->w.scales ? p->w.scales[co] : p->w.scale;
        const int has_bias = p->bias.data != NULL;
        const int32_t bq = has_bias ? ((const int32_t*)p->bias.data)[co] : 0;
        const float sb = p->bias.scales ? p->bias.scales[co] : p->bias.scale;
        store_q((void*)p->y.data, p->y.dtype, oi,
                requant(acc, p->x.scale, sw, has_bias, bq, sb, p->y.scale, p->y.zero_point, p->y.dtype, p->clamp_lo, p->clamp_hi));
    }
    return 0;
}

/* ---- Pooling3d, Pooling3d.cpp:138-328 (NDHWC) -------------------------------------------------------- */

/* clamp_range above is Pooling3d.cpp:100-111 as well */
int oracle_pool3d_q(const b200k_pool3d_params* p)
{
    if (!p->x.data || !p->y.data || p->pool_type < 0 || p->pool_type > 2) return B200K_E_INVALID;
    for (int n = 0; n < p->n; ++n) for (int c = 0; c < p->c; ++c)
    for (int oz = 0; oz < p->od; ++oz) for (int oy = 0; oy < p->oh; ++oy) for (int ox = 0; ox < p->ow; ++ox) {
        int ds = oz * p->stride_d - p->pad_front, de = ds + p->pool_d;
        if (de > p->d + p->pad_back) de = p->d + p->pad_back;
        int hs = oy * p->stride_h - p->pad_top, he = hs + p->pool_h;
        if (he > p->h + p->pad_bottom) he = p->h + p->pad_bottom;
        int ws = ox * p->stride_w - p->pad_left, we = ws + p->pool_w;
        if (we > p->wd + p->pad_right) we = p->wd + p->pad_right;
        float pool = (float)((de - ds) * (he - hs) * (we - ws));
        const int dcl = clamp_range(&ds, &de, p->d), hcl = clamp_range(&hs, &he, p->h), wcl = clamp_range(&ws, &we, p->wd);
        const int64_t oi = ((((int64_t)n * p->od + oz) * p->oh + oy) * p->ow + ox) * p->c + c;
        if (de <= 0 || ds > p->d || he <= 0 || hs > p->h || we <= 0 || ws > p->wd) { store_f(&p->y, oi, 0.0f); continue; }
        if ((dcl || hcl || wcl) && p->padding_method == 1) pool = (float)((de - ds) * (he - hs) * (we - ws));
        volatile float result = p->pool_type == 0 ? -3.402823466e+38f : 0.0f;
        for (int z = ds; z < de; ++z) for (int y = hs; y < he; ++y) for (int x = ws; x < we; ++x) {
            const float v = load_f(&p->x, ((((int64_t)n * p->d + z) * p->h + y) * p->wd + x) * p->c + c);
            if (p->pool_type == 0) { if (v > result) result = v; }
            else if (p->pool_type == 1) result = result + v;
            else { volatile float sq = v * v; result = result + sq; }
        }
        if (p->pool_type == 1) result = result / pool;
        else if (p->pool_type == 2) { volatile float q = result / pool; result = sqrtf(q); }
        store_f(&p->y, oi, result);
    }
    return 0;
}

/* ---- Quantize / Dequantize / requantize, RefQuantizeWorkload.cpp:14-45, Dequantize.cpp:11-28 - */

int oracle_convert_q(const b200k_convert_params* p)
{
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    for (int64_t i = 0; i < p->count; ++i) store_f(&p->y, i, load_f(&p->x, i));
    return 0;
}

/* ---- Cast, RefCastWorkload.cpp:13-36, 95-106: scale 1 and offset 0 on both sides, floor before an integer output - */

int oracle_cast_q(const b200k_convert_params* p)
{
    if (!p->x.data || !p->y.data) return B200K_E_INVALID;
    b200k_qtensor x = p->x, y = p->y;
    x.scale = 1.0f; x.zero_point = 0; y.scale = 1.0f; y.zero_point = 0;
    for (int64_t i = 0; i < p->count; ++i) {
        const float v = load_f(&x, i);
        if (y.dtype == B200K_F32) ((float*)y.data)[i] = v;
        else if (y.dtype == B200K_S32) {
            const float f = floorf(v);
            ((int32_t*)y.data)[i] = f >= 2147483648.0f ? INT32_MAX : f <= -2147483648.0f ? INT32_MIN : (int32_t)f;
        }
        else store_f(&y, i, floorf(v));
    }
    return 0;
}

/* ---- Pad (constant), Pad.cpp:37-170 -----------------------------------------------------------
 * Every output element is the decoded input element at the shifted position encoded with the
 * output's quantisation, or the pad value; for a quantised output the pad value is encoded with
 * scale 1 and offset 0, i.e. it is a quantised number already (Pad.cpp:76-83). */
int oracle_pad_q(const b200k_pad_params* p)
{
    if (!p->x.data || !p->y.data || p->rank < 1 || p->rank > 4) return B200K_E_INVALID;
    int in_shape[4] = {1, 1, 1, 1}, out_shape[4] = {1, 1, 1, 1}, before[4] = {0, 0, 0, 0};
    int64_t count = 1;
    for (int d = 0; d < p->rank; ++d) {
        in_shape[d] = p->shape[d]; before[d] = p->pad_before[d];
        out_shape[d] = p->shape[d] + p->pad_before[d] + p->pad_after[d];
        count *= out_shape[d];
    }
    for (int64_t i = 0; i < count; ++i) {
        int64_t rest = i, src = 0, stride = 1;
        int coord[4] = {0, 0, 0, 0}, inside = 1;
        for (int d = p->rank - 1; d >= 0; --d) { coord[d] = (int)(rest % out_shape[d]); rest /= out_shape[d]; }
        for (int d = p->rank - 1; d >= 0; --d) {
            int c = coord[d] - before[d];
            if (p->mode != 0) {                            /* MirrorPad.cpp:95-125 */
                const int n = in_shape[d], edge = p->mode == 1 ? 0 : 1;
                if (c < 0) c = -c - edge;
                else if (c >= n) c = 2 * n - 2 + edge - c;
            }
            if (c < 0 || c >= in_shape[d]) inside = 0;
            src += (int64_t)c * stride;
            stride *= in_shape[d];
        }
        if (inside) { store_f(&p->y, i, load_f(&p->x, src)); continue; }
        b200k_qtensor raw = p->y;
        if (raw.dtype != B200K_F32) { raw.scale = 1.0f; raw.zero_point = 0; }
        store_f(&raw, i, p->pad_value);
    }
    return 0;
}

/* ---- Resize, Resize.cpp:17-216 ---------------------------------------------------------------------
 * The reference's fp32 operations in the reference's order (this file is built with -ffp-contract=off): scale,
 * PixelScaler, floor (or armnn::roundf for nearest neighbour with aligned corners), the four texels, three Lerps. */
static float lerp_ref(float a, float b, float w) { return w * b + (1.f - w) * a; }
static float round_ref(float v) { return v < 0.f ? floorf(v - 0.5f) : floorf(v + 0.5f); }      /* include/armnn/Utils.hpp:43-47 */
static float pixel_scaler(int pixel, float scale, int half, int method)
{
    if (half && method == 0) return ((float)pixel + 0.5f) * scale - 0.5f;
    if (half && method == 1) return ((float)pixel + 0.5f) * scale;
    return (float)pixel * scale;
}
static int mini(int a, int b) { return a < b ? a : b; }

int oracle_resize_q(const b200k_resize_params* p)
{
    if (!p || !p->x.data || !p->y.data || (p->method != 0 && p->method != 1) || (p->align_corners && p->half_pixel_centers))
        return B200K_E_INVALID;
    const int N = p->n, C = p->c, IH = p->in_h, IW = p->in_w, OH = p->out_h, OW = p->out_w;
    const float scale_y = (p->align_corners && OH > 1) ? (float)(IH - 1) / (float)(OH - 1) : (float)IH / (float)OH;
    const float scale_x = (p->align_corners && OW > 1) ? (float)(IW - 1) / (float)(OW - 1) : (float)IW / (float)OW;
    const int nn_round = p->method == 1 && p->align_corners;
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c)
            for (int y = 0; y < OH; ++y) {
                const float iy = pixel_scaler(y, scale_y, p->half_pixel_centers, p->method);
                const float fiy = nn_round ? round_ref(iy) : floorf(iy);
                const int y0 = mini((int)(fiy > 0.f ? fiy : 0.f), IH - 1);
                const float yw = iy - fiy;
                for (int x = 0; x < OW; ++x) {
                    const float ix = pixel_scaler(x, scale_x, p->half_pixel_centers, p->method);
                    const float fix = nn_round ? round_ref(ix) : floorf(ix);
                    const int x0 = mini((int)(fix > 0.f ? fix : 0.f), IW - 1);
                    const float xw = ix - fix;
                    int x1, y1;
                    if (p->half_pixel_centers) {
                        const float cx = ceilf(ix), cy = ceilf(iy);
                        x1 = mini((int)(cx > 0.f ? cx : 0.f), IW - 1);
                        y1 = mini((int)(cy > 0.f ? cy : 0.f), IH - 1);
                    } else {
                        x1 = mini(x0 + 1, IW - 1);
                        y1 = mini(y0 + 1, IH - 1);
                    }
#define RS_AT(t, yy, xx, HH, WW) (p->nchw ? (((int64_t)n * C + c) * (HH) + (yy)) * (WW) + (xx) : (((int64_t)n * (HH) + (yy)) * (WW) + (xx)) * C + c)
                    float v;
                    if (p->method == 0) {
                        const float ly0 = lerp_ref(load_f(&p->x, RS_AT(x, y0, x0, IH, IW)), load_f(&p->x, RS_AT(x, y0, x1, IH, IW)), xw);
                        const float ly1 = lerp_ref(load_f(&p->x, RS_AT(x, y1, x0, IH, IW)), load_f(&p->x, RS_AT(x, y1, x1, IH, IW)), xw);
                        v = lerp_ref(ly0, ly1, yw);
                    } else {
                        /* of the four neighbours the one at distance 0 from (fix, fiy) wins: (x0, y0), as the scaled
                         * coordinates are never negative (Resize.cpp:162-206) */
                        v = load_f(&p->x, RS_AT(x, y0, x0, IH, IW));
                    }
                    store_f(&p->y, RS_AT(y, y, x, OH, OW), v);
#undef RS_AT
                }
            }
    return 0;
}

/* ---- Concat, Splitter, Permute, Transpose, StridedSlice, Slice ----------------------------------
 * The reference's data-movement workloads, each walked the way the reference walks it. */

static int64_t elems(const int32_t* shape, int rank)
{
    int64_t n = 1;
    for (int d = 0; d < rank; ++d) n *= shape[d];
    return n;
}

static size_t esize(int dtype) { return dtype == B200K_U8 || dtype == B200K_S8 ? 1 : (dtype == B200K_S16 ? 2 : 4); }

/* flat index -> coordinates, outermost first */
static void coords_of(int64_t i, const int32_t* shape, int rank, int32_t* c)
{
    for (int d = rank - 1; d >= 0; --d) { c[d] = (int32_t)(i % shape[d]); i /= shape[d]; }
}

/* Concatenate.cpp:14-85: every output element takes the value of the first input view that contains it, decoded with
 * the input's quantisation and encoded with the output's; elements no view covers are left alone. */
static int move_concat(const oracle_move_params* p)
{
    const int64_t n = elems(p->whole_shape, p->rank);
    for (int64_t i = 0; i < n; ++i) {
        int32_t c[6];
        coords_of(i, p->whole_shape, p->rank, c);
        for (int v = 0; v < p->n_views; ++v) {
            int inside = 1;
            for (int d = 0; d < p->rank; ++d)
                if (c[d] < p->view_origin[v][d] || c[d] >= p->view_origin[v][d] + p->view_shape[v][d]) inside = 0;
            if (!inside) continue;
            int64_t idx = 0, stride = 1;
            for (int d = p->rank - 1; d >= 0; --d) { idx += stride * (c[d] - p->view_origin[v][d]); stride *= p->view_shape[v][d]; }
            store_f(&p->whole, i, load_f(&p->view[v], idx));
            break;
        }
    }
    return 0;
}

/* Splitter.cpp:18-93: every input element goes to the first output view that contains it. */
static int move_split(const oracle_move_params* p)
{
    const int64_t n = elems(p->whole_shape, p->rank);
    for (int64_t i = 0; i < n; ++i) {
        int32_t c[6];
        coords_of(i, p->whole_shape, p->rank, c);
        for (int v = 0; v < p->n_views; ++v) {
            int inside = 1;
            for (int d = 0; d < p->rank; ++d)
                if (c[d] < p->view_origin[v][d] || c[d] >= p->view_origin[v][d] + p->view_shape[v][d]) inside = 0;
            if (!inside) continue;
            int64_t idx = 0, stride = 1;
            for (int d = p->rank - 1; d >= 0; --d) { idx += stride * (c[d] - p->view_origin[v][d]); stride *= p->view_shape[v][d]; }
            store_f(&p->view[v], idx, load_f(&p->whole, i));
            break;
        }
    }
    return 0;
}

/* Permute.cpp:22-119 (mapping[i] is the destination dimension of source dimension i) and Transpose.cpp:22-117
 * (mapping[i] is the source dimension of destination dimension i): raw elements, no re-quantisation. */
static int move_permute(const oracle_move_params* p, int transpose)
{
    const size_t es = esize(p->whole.dtype);
    const int rank = p->rank;
    int32_t src_of_dst[6];                  /* source dimension that becomes destination dimension j */
    for (int i = 0; i < rank; ++i) {
        if (transpose) src_of_dst[i] = p->perm[i];
        else           src_of_dst[p->perm[i]] = i;
    }
    int32_t dst_shape[6];
    for (int j = 0; j < rank; ++j) dst_shape[j] = p->whole_shape[src_of_dst[j]];
    for (int j = 0; j < rank; ++j) if (dst_shape[j] != p->view_shape[0][j]) return B200K_E_INVALID;
    int64_t src_stride[6], st = 1;
    for (int d = rank - 1; d >= 0; --d) { src_stride[d] = st; st *= p->whole_shape[d]; }
    const int64_t n = elems(dst_shape, rank);
    for (int64_t i = 0; i < n; ++i) {
        int32_t c[6];
        coords_of(i, dst_shape, rank, c);
        int64_t src = 0;
        for (int j = 0; j < rank; ++j) src += (int64_t)c[j] * src_stride[src_of_dst[j]];
        memcpy((uint8_t*)p->view[0].data + (size_t)i * es, (const uint8_t*)p->whole.data + (size_t)src * es, es);
    }
    return 0;
}

/* StridedSliceDescriptor::GetStartForAxis / GetStopForAxis (src/armnn/Descriptors.cpp:393-453) and the loop nest of
 * StridedSlice.cpp:188-222 (without ellipsis and new-axis masks): raw elements in the order the strided walk visits. */
static int move_strided_slice(const oracle_move_params* p)
{
    const size_t es = esize(p->whole.dtype);
    const int rank = p->rank;
    int start[6], stop[6], count[6];
    for (int d = 0; d < rank; ++d) {
        const int size = p->whole_shape[d], stride = p->stride[d];
        if (stride == 0) return B200K_E_INVALID;
        long long b = p->begin[d];
        if (p->begin_mask & (1 << d)) b = stride > 0 ? -2147483648LL : 2147483647LL;
        if (b < 0) b += size;
        start[d] = (int)(b < 0 ? 0 : (b > size - 1 ? size - 1 : b));
        if (p->shrink_axis_mask & (1 << d)) {
            stop[d] = start[d] + 1;
        } else {
            long long e = p->end[d];
            if (p->end_mask & (1 << d)) e = stride > 0 ? 2147483647LL : -2147483648LL;
            if (e < 0) e += size;
            if (stride > 0) stop[d] = (int)(e < 0 ? 0 : (e > size ? size : e));
            else            stop[d] = (int)(e < -1 ? -1 : (e > size - 1 ? size - 1 : e));
        }
        count[d] = 0;
        for (int i = start[d]; stride > 0 ? i < stop[d] : i > stop[d]; i += stride) ++count[d];
    }
    int64_t src_stride[6], st = 1;
    for (int d = rank - 1; d >= 0; --d) { src_stride[d] = st; st *= p->whole_shape[d]; }
    const int64_t n = elems(count, rank);
    for (int64_t i = 0; i < n; ++i) {
        int32_t c[6];
        coords_of(i, count, rank, c);
        int64_t src = 0;
        for (int d = 0; d < rank; ++d) src += (int64_t)(start[d] + c[d] * p->stride[d]) * src_stride[d];
        memcpy((uint8_t*)p->view[0].data + (size_t)i * es, (const uint8_t*)p->whole.data + (size_t)src * es, es);
    }
    return 0;
}

/* Slice.cpp:14-147: the block of `size` elements per dimension that starts at `begin`, raw elements. */
static int move_slice(const oracle_move_params* p)
{
    const size_t es = esize(p->whole.dtype);
    const int rank = p->rank;
    int64_t src_stride[6], st = 1;
    for (int d = rank - 1; d >= 0; --d) {
        if (p->begin[d] < 0 || p->end[d] < 0 || p->begin[d] + p->end[d] > p->whole_shape[d]) return B200K_E_INVALID;
        src_stride[d] = st; st *= p->whole_shape[d];
    }
    const int64_t n = elems(p->end, rank);
    for (int64_t i = 0; i < n; ++i) {
        int32_t c[6];
        coords_of(i, p->end, rank, c);
        int64_t src = 0;
        for (int d = 0; d < rank; ++d) src += (int64_t)(p->begin[d] + c[d]) * src_stride[d];
        memcpy((uint8_t*)p->view[0].data + (size_t)i * es, (const uint8_t*)p->whole.data + (size_t)src * es, es);
    }
    return 0;
}

/* ---- Reduce, Reduce.cpp:63-175 -------------------------------------------------------------------
 * One fp32 accumulator per output element; the input is walked once in flat index order and every element is folded
 * into the accumulator of the output it belongs to (ReducedOutputOffset: the kept coordinates, in order). */
int oracle_reduce_q(const b200k_reduce_params* p)
{
    if (!p || !p->x.data || !p->y.data || p->rank < 1 || p->rank > 6 || p->op < 0 || p->op > 4) return B200K_E_INVALID;
    const int mask = p->axis_mask ? p->axis_mask : (1 << p->rank) - 1;
    int64_t outputs = 1, reduced = 1;
    for (int d = 0; d < p->rank; ++d) { if (mask & (1 << d)) reduced *= p->shape[d]; else outputs *= p->shape[d]; }
    float* tmp = (float*)malloc(sizeof(float) * (size_t)outputs);
    if (!tmp) return B200K_E_INVALID;
    const float init = (p->op == 0 || p->op == 2) ? 0.f : (p->op == 4 ? 1.f : (p->op == 1 ? -3.402823466e+38f : 3.402823466e+38f));
    for (int64_t o = 0; o < outputs; ++o) tmp[o] = init;
    const int64_t n = outputs * reduced;
    for (int64_t i = 0; i < n; ++i) {
        int32_t c[6];
        coords_of(i, p->shape, p->rank, c);
        int64_t o = 0;
        for (int d = 0; d < p->rank; ++d) if (!(mask & (1 << d))) o = o * p->shape[d] + c[d];
        const float v = load_f(&p->x, i);
        switch (p->op) {
            case 0: case 2: tmp[o] += v; break;
            case 4: tmp[o] *= v; break;
            case 1: if (v > tmp[o]) tmp[o] = v; break;
            default: if (v < tmp[o]) tmp[o] = v; break;
        }
    }
    for (int64_t o = 0; o < outputs; ++o) store_f(&p->y, o, p->op == 2 ? tmp[o] / (float)reduced : tmp[o]);
    free(tmp);
    return 0;
}

/* The view copy of include/b200k.h as the graph-level oracle executor calls it: element by element through
 * Decoder / Encoder when the quantisation differs, raw elements otherwise. */
int oracle_view_copy_q(const b200k_view_copy_params* p)
{
    if (!p || !p->x.data || !p->y.data || p->rank < 1 || p->rank > 6 || p->x.dtype != p->y.dtype) return B200K_E_INVALID;
    const int quantised = p->x.dtype == B200K_U8 || p->x.dtype == B200K_S8 || p->x.dtype == B200K_S16;
    const int same = !quantised || (p->x.scale == p->y.scale && p->x.zero_point == p->y.zero_point);
    const size_t es = esize(p->x.dtype);
    const int64_t n = elems(p->shape, p->rank);
    for (int64_t i = 0; i < n; ++i) {
        int32_t c[6];
        coords_of(i, p->shape, p->rank, c);
        int64_t s = p->src_offset, d = p->dst_offset;
        for (int k = 0; k < p->rank; ++k) { s += c[k] * p->src_strides[k]; d += c[k] * p->dst_strides[k]; }
        if (same) memcpy((uint8_t*)p->y.data + (size_t)d * es, (const uint8_t*)p->x.data + (size_t)s * es, es);
        else      store_f(&p->y, d, load_f(&p->x, s));
    }
    return 0;
}

/* DepthToSpace.cpp:15-100: per batch, the permutation [H, W, b, b, C'] -> [H, b, W, b, C'] (NHWC) or
 * [b, b, C', H, W] -> [C', H, b, W, b] (NCHW) of raw elements, i.e. out(n, h b + i, w b + j, c') = in(n, h, w, (i b + j) C' + c'). */
static int move_depth_to_space(const oracle_move_params* p)
{
    const size_t es = esize(p->whole.dtype);
    const int b = p->perm[0], nchw = p->perm[1];
    const int N = p->whole_shape[0];
    const int C = nchw ? p->whole_shape[1] : p->whole_shape[3], H = nchw ? p->whole_shape[2] : p->whole_shape[1],
              W = nchw ? p->whole_shape[3] : p->whole_shape[2];
    if (b < 1 || C % (b * b)) return B200K_E_INVALID;
    const int Co = C / (b * b), OH = H * b, OW = W * b;
    for (int n = 0; n < N; ++n) for (int h = 0; h < H; ++h) for (int w = 0; w < W; ++w)
    for (int i = 0; i < b; ++i) for (int j = 0; j < b; ++j) for (int c = 0; c < Co; ++c) {
        const int ci = (i * b + j) * Co + c, oh = h * b + i, ow = w * b + j;
        const int64_t src = nchw ? (((int64_t)n * C + ci) * H + h) * W + w : (((int64_t)n * H + h) * W + w) * C + ci;
        const int64_t dst = nchw ? (((int64_t)n * Co + c) * OH + oh) * OW + ow : (((int64_t)n * OH + oh) * OW + ow) * Co + c;
        memcpy((uint8_t*)p->view[0].data + (size_t)dst * es, (const uint8_t*)p->whole.data + (size_t)src * es, es);
    }
    return 0;
}

/* SpaceToDepth.cpp:42-104: output channel oc reads input channel oc % C at (oh b + (oc / C) / b, ow b + (oc / C) % b),
 * through Decoder / Encoder. */
static int move_space_to_depth(const oracle_move_params* p)
{
    const int b = p->perm[0], nchw = p->perm[1];
    const int N = p->whole_shape[0];
    const int C = nchw ? p->whole_shape[1] : p->whole_shape[3], H = nchw ? p->whole_shape[2] : p->whole_shape[1],
              W = nchw ? p->whole_shape[3] : p->whole_shape[2];
    if (b < 1 || H % b || W % b) return B200K_E_INVALID;
    const int OC = C * b * b, OH = H / b, OW = W / b;
    for (int oc = 0; oc < OC; ++oc) {
        const int ic = oc % C, sw = (oc / C) % b, sh = (oc / C) / b;
        for (int oh = 0; oh < OH; ++oh) for (int ow = 0; ow < OW; ++ow) for (int n = 0; n < N; ++n) {
            const int ih = oh * b + sh, iw = ow * b + sw;
            const int64_t src = nchw ? (((int64_t)n * C + ic) * H + ih) * W + iw : (((int64_t)n * H + ih) * W + iw) * C + ic;
            const int64_t dst = nchw ? (((int64_t)n * OC + oc) * OH + oh) * OW + ow : (((int64_t)n * OH + oh) * OW + ow) * OC + oc;
            store_f(&p->view[0], dst, load_f(&p->whole, src));
        }
    }
    return 0;
}

/* Offset of (batch, height, width, channel) in a tensor of rank 3 (no width) or 4, BatchToSpaceNd.cpp:14-46. */
static int64_t nd_offset(const int32_t* shape, int rank, int nchw, int b, int h, int w, int c)
{
    if (rank == 3) return nchw ? ((int64_t)b * shape[1] + c) * shape[2] + h : ((int64_t)b * shape[1] + h) * shape[2] + c;
    return nchw ? (((int64_t)b * shape[1] + c) * shape[2] + h) * shape[3] + w
                : (((int64_t)b * shape[1] + h) * shape[2] + w) * shape[3] + c;
}

static void nd_dims(const int32_t* shape, int rank, int nchw, int* h, int* w, int* c)
{
    if (rank == 3) { *h = nchw ? shape[2] : shape[1]; *w = 1; *c = nchw ? shape[1] : shape[2]; }
    else { *h = nchw ? shape[2] : shape[1]; *w = nchw ? shape[3] : shape[2]; *c = nchw ? shape[1] : shape[3]; }
}

/* BatchToSpaceNd.cpp:50-117: input batch ib = so * OB + ob carries the spatial offset so = i * BW + j; its pixel
 * (ih, iw) lands at (ih * BH + i - crop_top, iw * BW + j - crop_left) when that is inside the output. */
static int move_batch_to_space(const oracle_move_params* p)
{
    const int nchw = p->perm[0], rank = p->rank;
    if (rank != 3 && rank != 4) return B200K_E_INVALID;
    int IH, IW, C, OH, OW, OC;
    nd_dims(p->whole_shape, rank, nchw, &IH, &IW, &C);
    nd_dims(p->view_shape[0], rank, nchw, &OH, &OW, &OC);
    const int IB = p->whole_shape[0], OB = p->view_shape[0][0];
    const int BH = p->begin[0], BW = rank == 3 ? 1 : p->begin[1];
    const int ct = p->end[0], cl = rank == 3 ? 0 : p->end[1];
    if (BH < 1 || BW < 1 || OB < 1 || OC != C) return B200K_E_INVALID;
    for (int ib = 0; ib < IB; ++ib) {
        const int ob = ib % OB, so = ib / OB;
        for (int ih = 0; ih < IH; ++ih) {
            const int oh = ih * BH + so / BW - ct;
            if (oh < 0 || oh >= OH) continue;
            for (int iw = 0; iw < IW; ++iw) {
                const int ow = iw * BW + so % BW - cl;
                if (ow < 0 || ow >= OW) continue;
                for (int c = 0; c < C; ++c)
                    store_f(&p->view[0], nd_offset(p->view_shape[0], rank, nchw, ob, oh, ow, c),
                            load_f(&p->whole, nd_offset(p->whole_shape, rank, nchw, ib, ih, iw, c)));
            }
        }
    }
    return 0;
}

/* SpaceToBatchNd.cpp:49-131: output batch ob = (i * BW + j) * IB + ib reads pixel (oh * BH + i - pad_top,
 * ow * BW + j - pad_left) of input batch ib; outside the input the encoder stores 0.0. */
static int move_space_to_batch(const oracle_move_params* p)
{
    const int nchw = p->perm[0], rank = p->rank;
    if (rank != 3 && rank != 4) return B200K_E_INVALID;
    int IH, IW, C, OH, OW, OC;
    nd_dims(p->whole_shape, rank, nchw, &IH, &IW, &C);
    nd_dims(p->view_shape[0], rank, nchw, &OH, &OW, &OC);
    const int IB = p->whole_shape[0], OB = p->view_shape[0][0];
    const int BH = p->begin[0], BW = rank == 3 ? 1 : p->begin[1];
    const int pt = p->end[0], pl = rank == 3 ? 0 : p->end[1];
    if (BH < 1 || BW < 1 || IB < 1 || OC != C) return B200K_E_INVALID;
    for (int ob = 0; ob < OB; ++ob) {
        const int ib = ob % IB, sw = (ob / IB) % BW, sh = (ob / IB) / BW;
        for (int oh = 0; oh < OH; ++oh) for (int ow = 0; ow < OW; ++ow) {
            const int ih = oh * BH + sh - pt, iw = ow * BW + sw - pl;
            const int inside = ih >= 0 && ih < IH && iw >= 0 && iw < IW;
            for (int c = 0; c < C; ++c)
                store_f(&p->view[0], nd_offset(p->view_shape[0], rank, nchw, ob, oh, ow, c),
                        inside ? load_f(&p->whole, nd_offset(p->whole_shape, rank, nchw, ib, ih, iw, c)) : 0.0f);
        }
    }
    return 0;
}

/* Tile.cpp:47-103: output coordinate o reads input coordinate o % size in every dimension. */
static int move_tile(const oracle_move_params* p)
{
    int64_t total = 1;
    int32_t out_shape[6];
    for (int d = 0; d < p->rank; ++d) {
        if (p->perm[d] < 1) return B200K_E_INVALID;
        out_shape[d] = p->whole_shape[d] * p->perm[d];
        total *= out_shape[d];
    }
    for (int64_t o = 0; o < total; ++o) {
        int64_t rest = o, src = 0, stride = 1;
        for (int d = p->rank - 1; d >= 0; --d) {
            const int64_t c = rest % out_shape[d];
            rest /= out_shape[d];
            src += (c % p->whole_shape[d]) * stride;
            stride *= p->whole_shape[d];
        }
        store_f(&p->view[0], o, load_f(&p->whole, src));
    }
    return 0;
}

/* RefBroadcastToWorkload.cpp:29-44 with Broadcast.hpp: the input aligned to the innermost dimensions of the output. */
static int move_broadcast_to(const oracle_move_params* p)
{
    const int orank = p->view_rank[0] ? p->view_rank[0] : p->rank;
    if (orank < p->rank) return B200K_E_INVALID;
    int64_t total = 1;
    for (int d = 0; d < orank; ++d) total *= p->view_shape[0][d];
    for (int64_t o = 0; o < total; ++o) {
        int64_t rest = o, src = 0, stride = 1;
        for (int d = orank - 1; d >= 0; --d) {
            const int64_t c = rest % p->view_shape[0][d];
            rest /= p->view_shape[0][d];
            const int id = d - (orank - p->rank);
            if (id < 0) continue;
            if (p->whole_shape[id] != 1) src += c * stride;
            stride *= p->whole_shape[id];
        }
        store_f(&p->view[0], o, load_f(&p->whole, src));
    }
    return 0;
}

/* RefChannelShuffleWorkload.cpp:28-76: with g groups of s channels along `axis`, output channel i g + j takes input
 * channel i + j s, through Decoder / Encoder. */
static int move_channel_shuffle(const oracle_move_params* p)
{
    const int axis = p->perm[0], g = p->perm[1];
    if (axis < 0 || axis >= p->rank || g < 1 || p->whole_shape[axis] % g) return B200K_E_INVALID;
    const int ch = p->whole_shape[axis], s = ch / g;
    int64_t outer = 1, inner = 1;
    for (int d = 0; d < axis; ++d) outer *= p->whole_shape[d];
    for (int d = axis + 1; d < p->rank; ++d) inner *= p->whole_shape[d];
    for (int64_t o = 0; o < outer; ++o) for (int64_t in = 0; in < inner; ++in)
    for (int i = 0; i < s; ++i) for (int j = 0; j < g; ++j)
        store_f(&p->view[0], (o * ch + (i * g + j)) * inner + in, load_f(&p->whole, (o * ch + (i + j * s)) * inner + in));
    return 0;
}

/* Stack.cpp:14-120: input i becomes index i of the new dimension `axis` of the output, through Decoder / Encoder. */
static int move_stack(const oracle_move_params* p)
{
    const int axis = p->perm[0], in_rank = p->rank - 1;
    if (axis < 0 || axis > in_rank) return B200K_E_INVALID;
    int64_t os[6], st = 1;
    for (int d = p->rank - 1; d >= 0; --d) { os[d] = st; st *= p->whole_shape[d]; }
    for (int v = 0; v < p->n_views; ++v) {
        const int64_t n = elems(p->view_shape[v], in_rank);
        for (int64_t i = 0; i < n; ++i) {
            int32_t c[6];
            coords_of(i, p->view_shape[v], in_rank, c);
            int64_t dst = (int64_t)v * os[axis];
            for (int d = 0; d < in_rank; ++d) dst += (int64_t)c[d] * os[d < axis ? d : d + 1];
            store_f(&p->whole, dst, load_f(&p->view[v], i));
        }
    }
    return 0;
}

int oracle_move_q(const oracle_move_params* p)
{
    if (!p || p->rank < 1 || p->rank > 6 || !p->whole.data || p->n_views < 1 || p->n_views > 8) return B200K_E_INVALID;
    switch (p->kind) {
        case MOVE_CONCAT:        return move_concat(p);
        case MOVE_SPLIT:         return move_split(p);
        case MOVE_PERMUTE:       return move_permute(p, 0);
        case MOVE_TRANSPOSE:     return move_permute(p, 1);
        case MOVE_STRIDED_SLICE: return move_strided_slice(p);
        case MOVE_SLICE:         return move_slice(p);
        case MOVE_DEPTH_TO_SPACE:  return move_depth_to_space(p);
        case MOVE_SPACE_TO_DEPTH:  return move_space_to_depth(p);
        case MOVE_CHANNEL_SHUFFLE: return move_channel_shuffle(p);
        case MOVE_STACK:           return move_stack(p);
        case MOVE_TILE:            return move_tile(p);
        case MOVE_BROADCAST_TO:    return move_broadcast_to(p);
        case MOVE_BATCH_TO_SPACE:  return move_batch_to_space(p);
        case MOVE_SPACE_TO_BATCH:  return move_space_to_batch(p);
        default: return B200K_E_INVALID;
    }
}

/* ---- QLstm, RefQLstmWorkload.cpp:46-541 with LstmUtils.cpp:16-256 ------------------------------
 * A step-by-step restatement: every Encoder::Set / Decoder::Get of the reference is one
 * quantize_f / dequantize_i here, in the reference's order, including the re-quantisation of the
 * int16 gate accumulators after every multiply-accumulate (LstmUtils.cpp:87-111) and the scale
 * switches on the gate buffers around layer normalisation (RefQLstmWorkload.cpp:331-364). */

static int16_t q16(float v, float scale, int32_t zp) { return (int16_t)quantize_f(v, scale, zp, B200K_S16); }
static float   d16(int16_t q, float scale, int32_t zp) { return dequantize_i(q, scale, zp); }

/* MatrixBatchVectorMultiplyAccumulate, LstmUtils.cpp:87-111: out = Q(out + w * x) per element of K */
static void matvec_acc(const int8_t* w, float sw, int rows, int cols, const int8_t* x, float sx, int zx,
                       int batch, int16_t* out, float so, int zo)
{
    #pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < batch; ++b)
    for (int r = 0; r < rows; ++r) {
        int16_t acc = out[b * rows + r];
        for (int c = 0; c < cols; ++c) {
            volatile float wf = dequantize_i(w[r * cols + c], sw, 0);
            volatile float xf = dequantize_i(x[b * cols + c], sx, zx);
            volatile float p = wf * xf;
            volatile float s = d16(acc, so, zo) + p;
            acc = q16(s, so, zo);
        }
        out[b * rows + r] = acc;
    }
}

/* one gate after the mat-vecs: optional peephole, optional layer norm, activation
 * (RefQLstmWorkload.cpp:321-364 for the input gate; the other gates repeat the pattern) */
static void gate_post(const b200k_qlstm_params* p, int16_t* gate, float s_int,
                      const int16_t* peep, float s_peep, const int16_t* cell, float s_cell,
                      const int16_t* lnw, float s_lnw, const int32_t* bias, float s_bias, int tanh_act)
{
    const int B = p->batch, U = p->num_units;
    float s = s_int;
    if (peep) {                                    /* VectorBatchVectorCwiseProductAccumulate, :126-144 */
        for (int b = 0; b < B; ++b) for (int u = 0; u < U; ++u) {
            volatile float pr = d16(peep[u], s_peep, 0) * d16(cell[b * U + u], s_cell, 0);
            volatile float t = d16(gate[b * U + u], s, 0) + pr;
            gate[b * U + u] = q16(t, s, 0);
        }
    }
    if (lnw) {
        volatile float s_ln0 = p->input_scale * s_lnw;
        volatile float s_ln = s_ln0 * 1024;
        for (int b = 0; b < B; ++b) {             /* MeanStddevNormalization, :40-74 */
            int16_t* g = gate + b * U;
            float sum = 0.0f, sum_sq = 0.0f;
            for (int i = 0; i < U; ++i) {
                float v = d16(g[i], s, 0);
                volatile float a = sum + v; sum = a;
                volatile float sq = v * v;
                volatile float c = sum_sq + sq; sum_sq = c;
            }
            volatile float mean = sum / (float)U;
            volatile float ex2 = sum_sq / (float)U;
            volatile float mm = mean * mean;
            volatile float variance = ex2 - mm;
            float stddev_inv;
            if (variance == 0) stddev_inv = 1.0f / sqrtf(1e-8f);
            else               stddev_inv = 1.0f / sqrtf(variance);
            for (int i = 0; i < U; ++i) {
                volatile float d = d16(g[i], s, 0) - mean;
                volatile float n = d * stddev_inv;
                g[i] = q16(n, s_ln, 0);
            }
        }
        for (int b = 0; b < B; ++b) for (int u = 0; u < U; ++u) {   /* VectorBatchVectorCwiseProduct */
            volatile float t = d16(lnw[u], s_lnw, 0) * d16(gate[b * U + u], s_ln, 0);
            gate[b * U + u] = q16(t, s_ln, 0);
        }
        for (int b = 0; b < B; ++b) for (int u = 0; u < U; ++u) {   /* VectorBatchVectorAdd, bias */
            volatile float bf = (float)bias[u] * s_bias;
            volatile float t = d16(gate[b * U + u], s_ln, 0) + bf;
            gate[b * U + u] = q16(t, 1.f / 4096, 0);
        }
        s = 1.f / 4096;
    }
    for (int i = 0; i < B * U; ++i) {               /* Activation, Activation.cpp:103-119 */
        float v = d16(gate[i], s, 0);
        float r = tanh_act ? 1.0f * tanhf(1.0f * v) : 1.f / (1.f + expf(-v));
        gate[i] = q16(r, s_cell, 0);
    }
}

int oracle_qlstm_step(const b200k_qlstm_params* p)
{
    const int B = p->batch, I = p->input_size, U = p->num_units, O = p->output_size;
    const int cifg = p->w_i2i == NULL, peephole = p->w_c2f != NULL, ln = p->ln_f != NULL, proj = p->w_proj != NULL;
    const float sc = p->cell_state_scale;
    const size_t S = (size_t)B * U;
    int16_t* gi = (int16_t*)calloc(S, 2); int16_t* gf = (int16_t*)calloc(S, 2);
    int16_t* gc = (int16_t*)calloc(S, 2); int16_t* go = (int16_t*)calloc(S, 2);
    int8_t* hidden = (int8_t*)malloc(S);
    int16_t* out16 = (int16_t*)calloc((size_t)B * O, 2);
    const int8_t* x = (const int8_t*)p->input; const int8_t* h = (const int8_t*)p->output_state_in;
    const int16_t* cin = (const int16_t*)p->cell_state_in;
    int16_t* cout = (int16_t*)p->cell_state_out;
    int8_t* out = (int8_t*)p->output; int8_t* hout = (int8_t*)p->output_state_out;
    if (!gi || !gf || !gc || !go || !hidden || !out16) return B200K_E_INVALID;
    if (!proj && U != O) return B200K_E_INVALID;

    /* input and recurrent mat-vecs, :289-319 */
    if (!cifg) matvec_acc(p->w_i2i, p->s_i2i, U, I, x, p->input_scale, p->input_zp, B, gi, p->input_intermediate_scale, 0);
    matvec_acc(p->w_i2f, p->s_i2f, U, I, x, p->input_scale, p->input_zp, B, gf, p->forget_intermediate_scale, 0);
    matvec_acc(p->w_i2c, p->s_i2c, U, I, x, p->input_scale, p->input_zp, B, gc, p->cell_intermediate_scale, 0);
    matvec_acc(p->w_i2o, p->s_i2o, U, I, x, p->input_scale, p->input_zp, B, go, p->output_intermediate_scale, 0);
    if (!cifg) matvec_acc(p->w_r2i, p->s_r2i, U, O, h, p->output_state_scale, p->output_state_zp, B, gi, p->input_intermediate_scale, 0);
    matvec_acc(p->w_r2f, p->s_r2f, U, O, h, p->output_state_scale, p->output_state_zp, B, gf, p->forget_intermediate_scale, 0);
    matvec_acc(p->w_r2c, p->s_r2c, U, O, h, p->output_state_scale, p->output_state_zp, B, gc, p->cell_intermediate_scale, 0);
    matvec_acc(p->w_r2o, p->s_r2o, U, O, h, p->output_state_scale, p->output_state_zp, B, go, p->output_intermediate_scale, 0);

    if (!cifg)
        gate_post(p, gi, p->input_intermediate_scale, peephole ? p->w_c2i : NULL, p->s_c2i, cin, sc,
                  ln ? p->ln_i : NULL, p->s_lni, p->b_i, p->s_bi, 0);
    gate_post(p, gf, p->forget_intermediate_scale, peephole ? p->w_c2f : NULL, p->s_c2f, cin, sc,
              ln ? p->ln_f : NULL, p->s_lnf, p->b_f, p->s_bf, 0);
    gate_post(p, gc, p->cell_intermediate_scale, NULL, 0.f, cin, sc,
              ln ? p->ln_c : NULL, p->s_lnc, p->b_c, p->s_bc, 1);

    /* cell state, :443-462 */
    for (size_t i = 0; i < S; ++i) {
        volatile float t = d16(gf[i], sc, 0) * d16(cin[i], sc, 0);
        cout[i] = q16(t, sc, 0);
    }
    if (cifg) {
        for (size_t i = 0; i < S; ++i) { volatile float t = 1.0f - d16(gf[i], sc, 0); gf[i] = q16(t, sc, 0); }
    }
    for (size_t i = 0; i < S; ++i) {
        volatile float pr = d16(gc[i], sc, 0) * d16(cifg ? gf[i] : gi[i], sc, 0);
        volatile float t = d16(cout[i], sc, 0) + pr;
        cout[i] = q16(t, sc, 0);
    }
    if (p->cell_clip > 0.0f) {
        for (size_t i = 0; i < S; ++i) {
            float f = d16(cout[i], sc, 0);
            float r = (p->cell_clip < f) ? p->cell_clip : f;
            r = (-p->cell_clip > r) ? -p->cell_clip : r;
            cout[i] = q16(r, sc, 0);
        }
    }
    /* output gate (peephole reads the NEW cell state), :464-503 */
    gate_post(p, go, p->output_intermediate_scale, peephole ? p->w_c2o : NULL, p->s_c2o, cout, sc,
              ln ? p->ln_o : NULL, p->s_lno, p->b_o, p->s_bo, 0);
    /* hidden = o * tanh(c), :505-511 */
    for (size_t i = 0; i < S; ++i) {
        float v = d16(cout[i], sc, 0);
        gc[i] = q16(1.0f * tanhf(1.0f * v), sc, 0);
    }
    for (size_t i = 0; i < S; ++i) {
        volatile float t = d16(go[i], sc, 0) * d16(gc[i], sc, 0);
        hidden[i] = (int8_t)quantize_f(t, p->hidden_state_scale, p->hidden_state_zp, B200K_S8);
    }
    /* projection, :513-538 */
    if (proj) {
        if (p->b_proj)
            for (int b = 0; b < B; ++b) for (int j = 0; j < O; ++j) {
                volatile float bf = (float)p->b_proj[j] * p->s_bproj;
                out16[b * O + j] = q16(bf, p->output_scale, p->output_zp);
            }
        matvec_acc(p->w_proj, p->s_proj, O, U, hidden, p->hidden_state_scale, p->hidden_state_zp, B,
                   out16, p->output_scale, p->output_zp);
        for (int i = 0; i < B * O; ++i)
            out[i] = (int8_t)quantize_f(d16(out16[i], p->output_scale, p->output_zp), p->output_scale, p->output_zp, B200K_S8);
        if (p->projection_clip > 0.0f)
            for (int i = 0; i < B * O; ++i) {
                float f = dequantize_i(out[i], p->output_scale, p->output_zp);
                float r = (p->projection_clip < f) ? p->projection_clip : f;
                r = (-p->projection_clip > r) ? -p->projection_clip : r;
                out[i] = (int8_t)quantize_f(r, p->output_scale, p->output_zp, B200K_S8);
            }
    } else {
        for (int i = 0; i < B * O; ++i)
            out[i] = (int8_t)quantize_f(dequantize_i(hidden[i], p->hidden_state_scale, p->hidden_state_zp),
                                        p->output_scale, p->output_zp, B200K_S8);
    }
    for (int i = 0; i < B * O; ++i)
        hout[i] = (int8_t)quantize_f(dequantize_i(out[i], p->output_scale, p->output_zp),
                                     p->output_state_scale, p->output_state_zp, B200K_S8);
    free(gi); free(gf); free(gc); free(go); free(hidden); free(out16);
    return 0;
}

/* ---- Float32 LSTM step, Lstm.cpp:14-259 with LstmUtils.cpp (the Lstm layer and each time step of
 * UnidirectionalSequenceLstm).  Every sum is accumulated term by term in the reference's order. ---------------------- */

static float lstm_act(float in, int fn)                         /* LstmUtils.cpp:258-297 + Activation.cpp */
{
    switch (fn) {
        case 1: return in > 0.f ? in : 0.f;
        case 3: { float t = in > 0.f ? in : 0.f; return t < 6.f ? t : 6.f; }
        case 4: return tanhf(in);
        case 6: return 1.f / (1.f + expf(-in));
        default: return in;
    }
}

static void lstm_gate(const b200k_lstm_params* p, const float* x, const float* h, const float* wi, const float* wr,
                      const float* peephole, const float* cell, const float* bias, const float* ln, float* out)
{
    const int U = p->num_units;
    for (int u = 0; u < U; ++u) {
        volatile float acc = ln ? 0.0f : bias[u];               /* :59-82 */
        for (int k = 0; k < p->input_size; ++k) { volatile float t = wi[(int64_t)u * p->input_size + k] * x[k]; acc = acc + t; }
        for (int k = 0; k < p->output_size; ++k) { volatile float t = wr[(int64_t)u * p->output_size + k] * h[k]; acc = acc + t; }
        if (peephole) { volatile float t = peephole[u] * cell[u]; acc = acc + t; }
        out[u] = acc;
    }
    if (ln) {                                                   /* LstmUtils.cpp:40-74 */
        volatile float sum = 0.0f, sum_sq = 0.0f;
        for (int u = 0; u < U; ++u) { sum = sum + out[u]; volatile float sq = out[u] * out[u]; sum_sq = sum_sq + sq; }
        const float mean = sum / (float)U;
        volatile float m2 = mean * mean;
        volatile float ms = sum_sq / (float)U;
        const float variance = ms - m2;
        const float stddev_inv = variance == 0 ? 1.0f / sqrtf(p->layer_norm_eps) : 1.0f / sqrtf(variance);
        for (int u = 0; u < U; ++u) {
            volatile float d = out[u] - mean;
            volatile float n = d * stddev_inv;
            volatile float w = ln[u] * n;
            out[u] = w + bias[u];
        }
    }
}

int oracle_lstm_step_f32(const b200k_lstm_params* p)
{
    if (!p->input || !p->output_state_in || !p->cell_state_in || !p->output_state_out || !p->cell_state_out || !p->output) return B200K_E_INVALID;
    const int U = p->num_units, O = p->output_size;
    const int cifg = p->w_i2i == NULL, ln = p->ln_f != NULL;
    if (!p->w_proj && O != U) return B200K_E_INVALID;
    float* gi = (float*)malloc(sizeof(float) * U * 5);
    float *gf = gi + U, *gc = gf + U, *go = gc + U, *act = go + U;
    for (int b = 0; b < p->batch; ++b) {
        const float* x = p->input + b * p->input_stride;
        const float* h = p->output_state_in + (int64_t)b * O;
        const float* c_in = p->cell_state_in + (int64_t)b * U;
        float* c_out = p->cell_state_out + (int64_t)b * U;
        float* out = p->output + b * p->output_stride;
        if (!cifg) {
            lstm_gate(p, x, h, p->w_i2i, p->w_r2i, p->w_c2i, c_in, p->b_i, ln ? p->ln_i : NULL, gi);
            for (int u = 0; u < U; ++u) gi[u] = lstm_act(gi[u], 6);
        }
        lstm_gate(p, x, h, p->w_i2f, p->w_r2f, p->w_c2f, c_in, p->b_f, ln ? p->ln_f : NULL, gf);
        for (int u = 0; u < U; ++u) gf[u] = lstm_act(gf[u], 6);
        lstm_gate(p, x, h, p->w_i2c, p->w_r2c, NULL, NULL, p->b_c, ln ? p->ln_c : NULL, gc);
        for (int u = 0; u < U; ++u) {
            volatile float c = gf[u] * c_in[u];                                  /* :170 */
            if (p->activation > 0) gc[u] = lstm_act(gc[u], p->activation);       /* :176-181 */
            volatile float gate = cifg ? 1.0f - gf[u] : gi[u];                   /* :182-192 */
            volatile float t = gc[u] * gate;
            c = c + t;
            if (p->cell_clip > 0.0f) c = c > p->cell_clip ? p->cell_clip : (c < -p->cell_clip ? -p->cell_clip : c);
            c_out[u] = c;
        }
        /* the output gate's peephole reads the new cell state (:198-202); its matrix terms come first */
        lstm_gate(p, x, h, p->w_i2o, p->w_r2o, p->w_c2o, c_out, p->b_o, ln ? p->ln_o : NULL, go);
        for (int u = 0; u < U; ++u) {
            const float og = lstm_act(go[u], 6);
            /* without an activation function the cell scratch still holds the cell gate (:216-222) */
            const float cs = p->activation > 0 ? lstm_act(c_out[u], p->activation) : gc[u];
            volatile float r = og * cs;
            act[u] = r;
        }
        if (p->w_proj) {
            for (int o = 0; o < O; ++o) {
                volatile float acc = p->b_proj ? p->b_proj[o] : 0.0f;
                for (int k = 0; k < U; ++k) { volatile float t = p->w_proj[(int64_t)o * U + k] * act[k]; acc = acc + t; }
                if (p->projection_clip > 0.0f) acc = acc > p->projection_clip ? p->projection_clip : (acc < -p->projection_clip ? -p->projection_clip : acc);
                out[o] = acc;
            }
        } else {
            for (int o = 0; o < O; ++o) out[o] = act[o];
        }
        for (int o = 0; o < O; ++o) p->output_state_out[(int64_t)b * O + o] = out[o];
    }
    free(gi);
    return 0;
}

/* ---- ConvertFp16ToFp32 / ConvertFp32ToFp16, FloatingPointConverter.cpp:17-45 (half_float::half, nearest, ties to even) -- */

static float half_to_float(uint16_t h)
{
    const uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 31, man = h & 1023;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {                                          /* subnormal: man * 2^-24, exact in fp32 */
            float f = (float)man * 5.9604644775390625e-08f;
            memcpy(&bits, &f, 4);
            bits |= sign;
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

static uint16_t float_to_half(float f)
{
    uint32_t bits;
    memcpy(&bits, &f, 4);
    const uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    const uint32_t abs = bits & 0x7fffffffu;
    if (abs >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (abs > 0x7f800000u ? 0x200u | ((abs >> 13) & 0x3ffu) : 0));
    if (abs >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);            /* rounds to or beyond 65520: infinity */
    if (abs < 0x38800000u) {                                              /* below 2^-14: subnormal half or zero */
        /* |f| / 2^-24 rounded to nearest even is the mantissa; the magic-number addition does that rounding in fp32 */
        float a;
        memcpy(&a, &abs, 4);
        volatile float r = a * 16777216.0f;                               /* exact scaling */
        volatile float m = r + 8388608.0f;                                /* rounds to an integer, ties to even */
        uint32_t mb;
        float mf = m;
        memcpy(&mb, &mf, 4);
        return (uint16_t)(sign | (mb & 0x7ffu));                          /* up to 1024 = the smallest normal */
    }
    uint32_t rounded = abs + 0xfffu + ((abs >> 13) & 1u);                 /* nearest, ties to even on bit 13 */
    return (uint16_t)(sign | ((rounded - 0x38000000u) >> 13));
}

int oracle_convert_fp16(const b200k_convert_fp16_params* p)
{
    if (!p->x || !p->y || p->count < 0) return B200K_E_INVALID;
    for (int64_t i = 0; i < p->count; ++i) {
        if (p->to_half) {
            uint16_t hbits = float_to_half(((const float*)p->x)[i]);
            if ((hbits & 0x7fffu) == 0x7c00u) hbits = (uint16_t)((hbits & 0x8000u) | 0x7bffu);   /* :35-39: infinity becomes the largest finite half */
            ((uint16_t*)p->y)[i] = hbits;
        }
        else ((float*)p->y)[i] = half_to_float(((const uint16_t*)p->x)[i]);
    }
    return 0;
}

/* ---- ScatterNd, ScatterNd.cpp:37-333 (both variants; tuples outside the tensor, on which the reference throws, are skipped) -- */

int oracle_scatter_nd_q(const b200k_scatter_nd_params* p)
{
    if (!p->updates.data || !p->y.data || !p->indices || p->nd < 1 || p->nd > 8) return B200K_E_INVALID;
    int64_t rows = 1, coeff[8];
    for (int d = p->nd - 1; d >= 0; --d) { coeff[d] = rows; rows *= p->dims[d]; }
    const int64_t total = rows * p->inner;
    for (int64_t i = 0; i < total; ++i) store_f(&p->y, i, p->x.data ? load_f(&p->x, i) : 0.0f);
    for (int j = 0; j < p->n_indices; ++j) {
        int64_t row = 0;
        int ok = 1;
        for (int d = 0; d < p->nd; ++d) {
            const int32_t t = p->indices[(int64_t)j * p->nd + d];
            if (t < 0 || t >= p->dims[d]) ok = 0;
            row += (int64_t)t * coeff[d];
        }
        if (!ok) continue;
        for (int k = 0; k < p->inner; ++k) {
            const int64_t at = row * p->inner + k;
            const float base = p->x.data ? load_f(&p->x, at) : 0.0f;
            const float u = load_f(&p->updates, (int64_t)j * p->inner + k);
            volatile float r;
            switch (p->function) {
                case 0: r = u; break;
                case 1: r = base + u; break;
                case 2: r = base - u; break;
                case 3: r = base < u ? u : base; break;
                case 4: r = u < base ? u : base; break;
                default: r = base * u; break;
            }
            store_f(&p->y, at, r);
        }
    }
    return 0;
}
