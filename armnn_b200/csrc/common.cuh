// Shared device/host helpers of libb200k: error reporting, the fp32 requantisation that every
// epilogue uses, and typed element access.
//
// All fp32 arithmetic that has to reproduce CpuRef goes through explicit round-to-nearest
// intrinsics (no fused multiply-add, IEEE division), because the reference is built for baseline
// x86-64 without FMA contraction (cmake/GlobalConfig.cmake:107,126 of the Arm NN tree).
#pragma once
#include <cuda_runtime.h>
#include <math.h>
#include <string.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/b200k.h"

namespace b200k {

void set_error(const char* fmt, ...);

#define B200K_REQUIRE(cond, code, ...)                                   \
    do { if (!(cond)) { ::b200k::set_error(__VA_ARGS__); return (code); } } while (0)

#define B200K_CUDA(call)                                                               \
    do { cudaError_t e_ = (call);                                                      \
         if (e_ != cudaSuccess) {                                                      \
             ::b200k::set_error("%s failed: %s", #call, cudaGetErrorString(e_));      \
             return B200K_E_CUDA; } } while (0)

void count_launch();                       // one more kernel launched (api.cu)

inline int check_launch(const char* what)
{
    count_launch();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("launch of %s failed: %s", what, cudaGetErrorString(e)); return B200K_E_CUDA; }
    return B200K_OK;
}

inline bool is_q8(int dtype) { return dtype == B200K_U8 || dtype == B200K_S8; }

__host__ __device__ inline void type_range(int dtype, int& lo, int& hi)
{
    switch (dtype) {
        case B200K_U8:  lo = 0;      hi = 255;   break;
        case B200K_S8:  lo = -128;   hi = 127;   break;
        case B200K_S16: lo = -32768; hi = 32767; break;
        default:        lo = INT32_MIN; hi = INT32_MAX; break;
    }
}

// ---- armnn::Quantize / armnn::Dequantize (src/armnn/TypesUtils.cpp:29-56) on the device -------

// q = clamp(float(zp) + round(v / scale), type_min, type_max); ties away from zero.
__device__ __forceinline__ int quantize_dev(float v, float scale, int zp, float tlo, float thi)
{
    float r = roundf(__fdiv_rn(v, scale));
    float q = __fadd_rn(__int2float_rn(zp), r);
    q = fminf(fmaxf(q, tlo), thi);
    return __float2int_rz(q);
}

// RN(1 / b): the double quotient rounded to float is within one ulp; the exact residuals 1 - b * y (products of two
// 24-bit significands are exact in double) pick the nearest of the three candidates.
inline float rn_reciprocal(float b)
{
    const float y = (float)(1.0 / (double)b);
    const float cand[3] = {nextafterf(y, 0.f), y, nextafterf(y, INFINITY)};
    float best = y;
    double err = 1e300;
    for (int i = 0; i < 3; ++i) {
        const double e = fabs(1.0 - (double)b * (double)cand[i]);
        if (e < err) { err = e; best = cand[i]; }
    }
    return best;
}

// The contraction epilogue v = fl(fl(acc * m) + b); q = clamp(zy + round_half_away(fl(v / sy)), lo, hi) without the
// division unit: with y = RN(1 / sy) from the host, p = fl(v * y) and q = fma(fma(-p, sy, v), y, p) is the correctly
// rounded quotient (Markstein); it is rounded with the 1.5 * 2^23 constant (halves to even) and only exact halves, or
// values too large for the constant, go through roundf.  lo / hi: type range intersected with the activation clamp.
__device__ __forceinline__ int requant_fast(int acc, float m, float b, bool has_bias, float sy, float inv_sy, float zy, float lo, float hi)
{
    float v = __fmul_rn(__int2float_rn(acc), m);
    if (has_bias) v = __fadd_rn(v, b);
    const float p = __fmul_rn(v, inv_sy);
    const float q = __fmaf_rn(__fmaf_rn(-p, sy, v), inv_sy, p);
    float n = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
    if (fabsf(__fsub_rn(q, n)) == 0.5f || !(fabsf(q) < 4194304.0f)) n = roundf(q);
    return __float2int_rn(fminf(fmaxf(__fadd_rn(zy, n), lo), hi));
}

// four 8-bit products summed into acc, each operand signed or unsigned
template <bool XU, bool WU>
__device__ __forceinline__ int dp4a_mixed(uint32_t x, uint32_t w, int acc)
{
    int d;
    if (XU && WU)       asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(w), "r"(acc));
    else if (XU && !WU) asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(w), "r"(acc));
    else if (!XU && WU) asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(w), "r"(acc));
    else                asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(x), "r"(w), "r"(acc));
    return d;
}

// v = float(q - zp) * scale
__device__ __forceinline__ float dequantize_dev(int q, float scale, int zp)
{
    return __fmul_rn(__int2float_rn(q - zp), scale);
}

// Epilogue of every contraction:  v = float(acc) * (sx * sw) + float(bias) * sb ; Quantize ; clamp.
struct Requant {
    float sx;            // input scale
    float sy;            // output scale
    int   zy;            // output zero point
    float tlo, thi;      // output type range as float
    int   clo, chi;      // fused-activation clamp (already inside the type range)
    __device__ __forceinline__ int operator()(int acc, float sw, bool has_bias, int bq, float sb) const
    {
        float v = __fmul_rn(__int2float_rn(acc), __fmul_rn(sx, sw));
        if (has_bias) v = __fadd_rn(v, __fmul_rn(__int2float_rn(bq), sb));
        int q = quantize_dev(v, sy, zy, tlo, thi);
        return min(max(q, clo), chi);
    }
};

inline Requant make_requant(float sx, const b200k_qtensor& y, int clamp_lo, int clamp_hi)
{
    int lo, hi;
    type_range(y.dtype, lo, hi);
    Requant r;
    r.sx = sx; r.sy = y.scale; r.zy = y.zero_point;
    r.tlo = (float)lo; r.thi = (float)hi;
    r.clo = clamp_lo > lo ? clamp_lo : lo;
    r.chi = clamp_hi < hi ? clamp_hi : hi;
    return r;
}

// Fused ElementwiseBinary Add behind a convolution epilogue: q1 is the convolution's own 8-bit output (formed with
// `own`), the other operand is dequantised with its scale / offset, the fp32 sum is re-quantised with `out`.
struct FusedAdd {
    const uint8_t* res;          // null: no fusion
    float res_scale; int res_zp; int res_u8;
    Requant out;                 // quantisation and clamp of the Add's output
    __device__ __forceinline__ int operator()(int q1, const Requant& own, long long i) const
    {
        const int rq8 = res_u8 ? (int)res[i] : (int)(int8_t)res[i];
        const float fa = __fmul_rn(__int2float_rn(q1 - own.zy), own.sy);
        const float fb = __fmul_rn(__int2float_rn(rq8 - res_zp), res_scale);
        const int q = quantize_dev(__fadd_rn(fa, fb), out.sy, out.zy, out.tlo, out.thi);
        return min(max(q, out.clo), out.chi);
    }
};

// Fills the fused-add part of a launch from the C-ABI struct; returns false when the request is malformed.
inline bool make_fused_add(const b200k_conv2d_params* p, Requant& own, FusedAdd& fa, void*& out_ptr)
{
    fa.res = nullptr;
    out_ptr = (void*)p->y.data;
    own = make_requant(p->x.scale, p->y, p->clamp_lo, p->clamp_hi);
    if (!p->add_operand.data) return true;
    if (!is_q8(p->add_operand.dtype) || !is_q8(p->add_out.dtype) || !p->add_out.data) return false;
    if (!(p->add_operand.scale > 0.f) || !(p->add_out.scale > 0.f)) return false;
    int lo, hi;
    type_range(p->y.dtype, lo, hi);
    own = make_requant(p->x.scale, p->y, lo, hi);                      // the intermediate carries no activation
    fa.res = (const uint8_t*)p->add_operand.data;
    fa.res_scale = p->add_operand.scale; fa.res_zp = p->add_operand.zero_point;
    fa.res_u8 = p->add_operand.dtype == B200K_U8;
    fa.out = make_requant(0.f, p->add_out, p->clamp_lo, p->clamp_hi);
    out_ptr = (void*)p->add_out.data;
    return true;
}

// ---- typed element access ------------------------------------------------------------------

__device__ __forceinline__ int load_q_dev(const void* p, int dtype, long long i)
{
    switch (dtype) {
        case B200K_U8:  return ((const uint8_t*)p)[i];
        case B200K_S8:  return ((const int8_t*)p)[i];
        case B200K_S16: return ((const int16_t*)p)[i];
        default:        return ((const int32_t*)p)[i];
    }
}

__device__ __forceinline__ void store_q_dev(void* p, int dtype, long long i, int q)
{
    switch (dtype) {
        case B200K_U8:  ((uint8_t*)p)[i]  = (uint8_t)q;  break;
        case B200K_S8:  ((int8_t*)p)[i]   = (int8_t)q;   break;
        case B200K_S16: ((int16_t*)p)[i]  = (int16_t)q;  break;
        default:        ((int32_t*)p)[i]  = q;           break;
    }
}

// A tensor operand as the kernels see it (a trimmed b200k_qtensor plus the float type range).
struct QView {
    const void* data;
    int   dtype;
    float scale;
    int   zp;
    float tlo, thi;
    __device__ __forceinline__ float get(long long i) const      // Decoder<float>::Get
    {
        if (dtype == B200K_F32) return ((const float*)data)[i];
        return dequantize_dev(load_q_dev(data, dtype, i), scale, zp);
    }
    __device__ __forceinline__ int quant(float v) const { return quantize_dev(v, scale, zp, tlo, thi); }
    __device__ __forceinline__ void set(long long i, float v) const   // Encoder<float>::Set
    {
        if (dtype == B200K_F32) { ((float*)data)[i] = v; return; }
        store_q_dev((void*)data, dtype, i, quant(v));
    }
};

inline QView make_view(const b200k_qtensor& t)
{
    int lo, hi;
    type_range(t.dtype, lo, hi);
    QView v;
    v.data = t.data; v.dtype = t.dtype; v.scale = t.scale; v.zp = t.zero_point;
    v.tlo = (float)lo; v.thi = (float)hi;
    return v;
}

inline int elem_size(int dtype)
{
    switch (dtype) { case B200K_U8: case B200K_S8: return 1; case B200K_S16: return 2; default: return 4; }
}

inline unsigned div_up(long long a, long long b) { return (unsigned)((a + b - 1) / b); }

// Two-wide fp32 arithmetic (one instruction for two IEEE round-to-nearest operations) for code that is bound by
// instruction issue, not by the arithmetic pipes.  Pairs travel in 64-bit registers.  The assembler contracts a packed
// multiply feeding a packed add into one FMA even with explicit .rn; where the reference rounds the product, form it
// as fma2(a, b, zero).
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi)
{
    f32x2 d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c)
{
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b)
{
    f32x2 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b)
{
    f32x2 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b)
{
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}


// requant_fast for two values at once in two-wide fp32 instructions (m2, b2: the two channels' constants; the other
// constants the same value twice).  Returns the two results as integer-valued floats (already clamped).
__device__ __forceinline__ void requant_fast2(int acc0, int acc1, f32x2 m2, f32x2 b2, f32x2 sy2n, f32x2 inv2, f32x2 zy2, float lo, float hi,
                                              float& r0, float& r1)
{
    const f32x2 zero2 = pack2(0.f, 0.f), magic2 = pack2(12582912.0f, 12582912.0f);
    const f32x2 v2 = add2(fma2(pack2(__int2float_rn(acc0), __int2float_rn(acc1)), m2, zero2), b2);   // fl(fl(acc * m) + b)
    const f32x2 p2 = mul2(v2, inv2);
    const f32x2 q2 = fma2(fma2(p2, sy2n, v2), inv2, p2);
    const f32x2 n2 = sub2(add2(q2, magic2), magic2);
    float q0, q1, n0, n1;
    unpack2(q2, q0, q1); unpack2(n2, n0, n1);
    if (fabsf(__fsub_rn(q0, n0)) == 0.5f || !(fabsf(q0) < 4194304.0f)) n0 = roundf(q0);
    if (fabsf(__fsub_rn(q1, n1)) == 0.5f || !(fabsf(q1) < 4194304.0f)) n1 = roundf(q1);
    float z0, z1;
    unpack2(add2(pack2(n0, n1), zy2), z0, z1);
    r0 = fminf(fmaxf(z0, lo), hi);
    r1 = fminf(fmaxf(z1, lo), hi);
}


// Addend of the one-FMA requantisation q" = fma(float(acc), m / sy, bq): bq of one (class, column) to within one rounding
// of its last operation: X = (b - cc m) / sy from error-free
// products and sums (cc split into two exactly representable parts), one correction step on the quotient, + zoff.
__device__ __forceinline__ float epi_make_bq(float b, int cc, float m, float sy, float inv_sy, float zoff)
{
    const float ch = __int2float_rn(cc & ~0xfff), cl = __int2float_rn(cc & 0xfff);   // both exact
    const float p1 = __fmul_rn(ch, m), e1 = __fmaf_rn(ch, m, -p1);                   // ch m = p1 + e1
    const float p2 = __fmul_rn(cl, m), e2 = __fmaf_rn(cl, m, -p2);
    // s1 + r1 = b - p1, s2 + r2 = s1 - p2 (two-sum)
    const float s1 = __fsub_rn(b, p1);
    const float bb1 = __fsub_rn(s1, b);
    const float r1 = __fadd_rn(__fsub_rn(b, __fsub_rn(s1, bb1)), __fsub_rn(-p1, bb1));
    const float s2 = __fsub_rn(s1, p2);
    const float bb2 = __fsub_rn(s2, s1);
    const float r2 = __fadd_rn(__fsub_rn(s1, __fsub_rn(s2, bb2)), __fsub_rn(-p2, bb2));
    const float tail = __fsub_rn(__fsub_rn(__fadd_rn(r1, r2), e1), e2);
    const float hi = __fadd_rn(s2, tail);
    const float bb3 = __fsub_rn(hi, s2);
    const float lo = __fadd_rn(__fsub_rn(s2, __fsub_rn(hi, bb3)), __fsub_rn(tail, bb3));
    const float q0 = __fmul_rn(hi, inv_sy);
    const float rem = __fadd_rn(__fmaf_rn(-q0, sy, hi), lo);
    const float q = __fmaf_rn(rem, inv_sy, q0);
    return __fadd_rn(q, zoff);
}

// Programmatic dependent launch.  A grid launched with launch_pdl may be scheduled while its predecessor in the stream
// is still draining; its threads call pdl_enter() before they touch anything the predecessor may write (that is:
// first thing), which also lets the grid after it be scheduled early.  Kernels launched the plain way keep the full
// stream dependency.
__device__ __forceinline__ void pdl_enter()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
template <typename... KArgs, typename... Args>
static inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);      // errors surface in check_launch (cudaGetLastError)
}

}  // namespace b200k
