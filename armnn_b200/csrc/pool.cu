// Pooling2d (Max / Average / L2, both padding methods) and Mean over H,W for quantised NHWC tensors.
// Bandwidth-bound: each thread owns VEC consecutive channels of one output pixel, consecutive threads
// walk the channel axis, every tap is one coalesced vector load.  The arithmetic is CpuRef's own:
// dequantise to fp32, accumulate in CpuRef's (y, x) visiting order with unfused fp32 adds, divide,
// re-quantise — so the results equal CpuRef's bit for bit (Pooling2d.cpp:142-303, Reduce.cpp:68-173 of
// the Arm NN tree).
#include "common.cuh"

namespace b200k {

struct PoolArgs {
    QView x, y;
    int N, H, W, C, OH, OW;
    int ph, pw, sh, sw, pt, pb, pl, pr;
    int type, exclude;
    long long total;
};

__device__ __forceinline__ bool clamp_range(int& s, int& e, int maxr)
{
    if (s < 0 || e > maxr) {
        s = min(max(s, 0), maxr);
        e = min(max(e, 0), maxr);
        return true;
    }
    return false;
}

template <int VEC>
__device__ __forceinline__ void load_vec_f(const QView& t, long long i, float* out)
{
    if (VEC == 1) { out[0] = t.get(i); return; }
    // 8-bit only on the vector paths
    uint8_t raw[VEC];
    if (VEC == 16) *(uint4*)raw = *(const uint4*)((const uint8_t*)t.data + i);
    else           *(unsigned*)raw = *(const unsigned*)((const uint8_t*)t.data + i);
    #pragma unroll
    for (int k = 0; k < VEC; ++k) {
        int q = t.dtype == B200K_U8 ? (int)raw[k] : (int)(int8_t)raw[k];
        out[k] = dequantize_dev(q, t.scale, t.zp);
    }
}

template <int VEC>
__device__ __forceinline__ void store_vec_f(const QView& t, long long i, const float* v)
{
    if (VEC == 1) { t.set(i, v[0]); return; }
    uint8_t raw[VEC];
    #pragma unroll
    for (int k = 0; k < VEC; ++k) raw[k] = (uint8_t)t.quant(v[k]);
    if (VEC == 16) *(uint4*)((uint8_t*)t.data + i) = *(const uint4*)raw;
    else           *(unsigned*)((uint8_t*)t.data + i) = *(const unsigned*)raw;
}

template <int VEC>
__global__ void __launch_bounds__(256) pool2d_kernel(const PoolArgs a)
{
    pdl_enter();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int cg = a.C / VEC;
    const int c = (int)(idx % cg) * VEC;
    long long t = idx / cg;
    const int ox = (int)(t % a.OW); t /= a.OW;
    const int oy = (int)(t % a.OH);
    const int n = (int)(t / a.OH);

    int hstart = oy * a.sh - a.pt;
    int hend = min(hstart + a.ph, a.H + a.pb);
    const int height = hend - hstart;
    bool clamped = clamp_range(hstart, hend, a.H);
    int wstart = ox * a.sw - a.pl;
    int wend = min(wstart + a.pw, a.W + a.pr);
    float area = __int2float_rn(height * (wend - wstart));
    const long long oi = (((long long)n * a.OH + oy) * a.OW + ox) * a.C + c;

    float r[VEC];
    if ((hend <= 0 || hstart > a.H) || (wend <= 0 || wstart > a.W)) {
        // window lies entirely in the padding: 0 by convention (Pooling2d.cpp:216-241)
        #pragma unroll
        for (int k = 0; k < VEC; ++k) r[k] = 0.0f;
        store_vec_f<VEC>(a.y, oi, r);
        return;
    }
    clamped |= clamp_range(wstart, wend, a.W);
    if (clamped && a.exclude) area = __int2float_rn((hend - hstart) * (wend - wstart));

    #pragma unroll
    for (int k = 0; k < VEC; ++k) r[k] = a.type == 0 ? -3.402823466e+38f : 0.0f;
    for (int iy = hstart; iy < hend; ++iy)
        for (int ix = wstart; ix < wend; ++ix) {
            float v[VEC];
            load_vec_f<VEC>(a.x, (((long long)n * a.H + iy) * a.W + ix) * a.C + c, v);
            #pragma unroll
            for (int k = 0; k < VEC; ++k) {
                if (a.type == 0)      { if (v[k] > r[k]) r[k] = v[k]; }
                else if (a.type == 1) r[k] = __fadd_rn(r[k], v[k]);
                else                  r[k] = __fadd_rn(r[k], __fmul_rn(v[k], v[k]));
            }
        }
    #pragma unroll
    for (int k = 0; k < VEC; ++k) {
        if (a.type == 1)      r[k] = __fdiv_rn(r[k], area);
        else if (a.type == 2) r[k] = __fsqrt_rn(__fdiv_rn(r[k], area));
    }
    store_vec_f<VEC>(a.y, oi, r);
}

// Max pooling whose input and output share type, scale and offset: dequantisation is monotone (scale > 0) and
// Quantize(Dequantize(q)) == q, so the result is the maximum of the quantised bytes themselves — SIMD byte maxima, no
// floating point.  A window with no valid tap yields Quantize(lowest float) = the type minimum, a padding-only window
// Quantize(0) = the zero point, as in the general kernel.
__global__ void __launch_bounds__(256) maxpool_same_quant_kernel(const PoolArgs a)
{
    pdl_enter();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int cg = a.C / 16;
    const int c = (int)(idx % cg) * 16;
    long long t = idx / cg;
    const int ox = (int)(t % a.OW); t /= a.OW;
    const int oy = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    int hstart = oy * a.sh - a.pt;
    int hend = min(hstart + a.ph, a.H + a.pb);
    clamp_range(hstart, hend, a.H);
    int wstart = ox * a.sw - a.pl;
    int wend = min(wstart + a.pw, a.W + a.pr);
    const bool is_u8 = a.x.dtype == B200K_U8;
    uint4 r;
    if ((hend <= 0 || hstart > a.H) || (wend <= 0 || wstart > a.W)) {
        const unsigned z = 0x01010101u * (unsigned)(a.x.zp & 0xff);
        r = make_uint4(z, z, z, z);
    } else {
        clamp_range(wstart, wend, a.W);
        const unsigned lowest = is_u8 ? 0u : 0x80808080u;
        r = make_uint4(lowest, lowest, lowest, lowest);
        for (int iy = hstart; iy < hend; ++iy)
            for (int ix = wstart; ix < wend; ++ix) {
                const uint4 v = *(const uint4*)((const uint8_t*)a.x.data + (((long long)n * a.H + iy) * a.W + ix) * a.C + c);
                if (is_u8) { r.x = __vmaxu4(r.x, v.x); r.y = __vmaxu4(r.y, v.y); r.z = __vmaxu4(r.z, v.z); r.w = __vmaxu4(r.w, v.w); }
                else       { r.x = __vmaxs4(r.x, v.x); r.y = __vmaxs4(r.y, v.y); r.z = __vmaxs4(r.z, v.z); r.w = __vmaxs4(r.w, v.w); }
            }
    }
    *(uint4*)((uint8_t*)a.y.data + (((long long)n * a.OH + oy) * a.OW + ox) * a.C + c) = r;
}

struct MeanArgs { QView x, y; int N, HW, C; long long total; };

template <int VEC>
__global__ void __launch_bounds__(128) mean_hw_kernel(const MeanArgs a)
{
    pdl_enter();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= a.total) return;
    const int cg = a.C / VEC;
    const int c = (int)(idx % cg) * VEC;
    const int n = (int)(idx / cg);
    float r[VEC];
    #pragma unroll
    for (int k = 0; k < VEC; ++k) r[k] = 0.0f;
    for (int i = 0; i < a.HW; ++i) {
        float v[VEC];
        load_vec_f<VEC>(a.x, ((long long)n * a.HW + i) * a.C + c, v);
        #pragma unroll
        for (int k = 0; k < VEC; ++k) r[k] = __fadd_rn(r[k], v[k]);
    }
    const float cnt = __int2float_rn(a.HW);
    #pragma unroll
    for (int k = 0; k < VEC; ++k) r[k] = __fdiv_rn(r[k], cnt);
    store_vec_f<VEC>(a.y, (long long)n * a.C + c, r);
}

static int pick_vec(const b200k_qtensor& x, const b200k_qtensor& y, int C)
{
    if (!is_q8(x.dtype) || !is_q8(y.dtype)) return 1;
    const uintptr_t al = (uintptr_t)x.data | (uintptr_t)y.data;
    if ((C % 16) == 0 && (al & 15) == 0) return 16;
    if ((C % 4) == 0 && (al & 3) == 0) return 4;
    return 1;
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_pool2d_q8(const b200k_pool2d_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "pool2d_q8: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "pool2d_q8: null tensor pointer");
    B200K_REQUIRE(p->pool_type >= 0 && p->pool_type <= 2, B200K_E_INVALID, "pool2d_q8: unsupported pooling algorithm %d", p->pool_type);
    B200K_REQUIRE(p->padding_method == 0 || p->padding_method == 1, B200K_E_INVALID, "pool2d_q8: unsupported padding type %d", p->padding_method);
    B200K_REQUIRE(p->n > 0 && p->h > 0 && p->wd > 0 && p->c > 0 && p->oh > 0 && p->ow > 0 && p->pool_h > 0 &&
                  p->pool_w > 0 && p->stride_h > 0 && p->stride_w > 0, B200K_E_INVALID, "pool2d_q8: bad geometry");
    B200K_REQUIRE(p->x.dtype != B200K_S32 && p->y.dtype != B200K_S32, B200K_E_UNSUPPORTED, "pool2d_q8: Signed32 not supported");
    PoolArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.N = p->n; a.H = p->h; a.W = p->wd; a.C = p->c; a.OH = p->oh; a.OW = p->ow;
    a.ph = p->pool_h; a.pw = p->pool_w; a.sh = p->stride_h; a.sw = p->stride_w;
    a.pt = p->pad_top; a.pb = p->pad_bottom; a.pl = p->pad_left; a.pr = p->pad_right;
    a.type = p->pool_type; a.exclude = p->padding_method == 1;
    int vec = pick_vec(p->x, p->y, p->c);
    // few outputs with large windows (global average pooling): narrower vectors give more threads to hide the latency
    // of the window's loads
    if (vec == 16 && (long long)p->n * p->oh * p->ow * (p->c / 16) < 148 * 1024) vec = 4;
    a.total = (long long)p->n * p->oh * p->ow * (p->c / vec);
    cudaStream_t s = (cudaStream_t)stream;
    if (vec == 16 && p->pool_type == 0 && p->x.dtype == p->y.dtype && p->x.scale == p->y.scale &&
        p->x.zero_point == p->y.zero_point && p->x.scale > 0.f) {
        launch_pdl(maxpool_same_quant_kernel, dim3((unsigned)(div_up(a.total, 256))), dim3(256), 0, s, a);
        return check_launch("maxpool_same_quant_kernel");
    }
    if (vec == 16)     launch_pdl(pool2d_kernel<16>, dim3((unsigned)(div_up(a.total, 256))), dim3(256), 0, s, a);
    else if (vec == 4) launch_pdl(pool2d_kernel<4>, dim3((unsigned)(div_up(a.total, 256))), dim3(256), 0, s, a);
    else               launch_pdl(pool2d_kernel<1>, dim3((unsigned)(div_up(a.total, 256))), dim3(256), 0, s, a);
    return check_launch("pool2d_kernel");
}

extern "C" int b200k_mean_hw_q8(const b200k_mean_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "mean_hw_q8: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "mean_hw_q8: null tensor pointer");
    B200K_REQUIRE(p->n > 0 && p->h > 0 && p->wd > 0 && p->c > 0, B200K_E_INVALID, "mean_hw_q8: bad shape");
    B200K_REQUIRE(p->x.dtype != B200K_S32 && p->y.dtype != B200K_S32, B200K_E_UNSUPPORTED, "mean_hw_q8: Signed32 not supported");
    MeanArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.N = p->n; a.HW = p->h * p->wd; a.C = p->c;
    const int vec = pick_vec(p->x, p->y, p->c);
    a.total = (long long)p->n * (p->c / vec);
    cudaStream_t s = (cudaStream_t)stream;
    if (vec == 16)     launch_pdl(mean_hw_kernel<16>, dim3((unsigned)(div_up(a.total, 128))), dim3(128), 0, s, a);
    else if (vec == 4) launch_pdl(mean_hw_kernel<4>, dim3((unsigned)(div_up(a.total, 128))), dim3(128), 0, s, a);
    else               launch_pdl(mean_hw_kernel<1>, dim3((unsigned)(div_up(a.total, 128))), dim3(128), 0, s, a);
    return check_launch("mean_hw_kernel");
}
