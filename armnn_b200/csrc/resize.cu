// Resize (bilinear / nearest neighbour) of the H and W axes, the reference's arithmetic operation for operation
// (src/backends/reference/workloads/Resize.cpp:25-216): coordinates and weights in fp32, Lerp as two rounded products
// and a rounded sum, samples through Decoder / Encoder.  One output element per thread, channel fastest for NHWC (the
// four samples of neighbouring threads are neighbouring bytes); a bandwidth kernel.
#include "common.cuh"

namespace b200k {

struct ResizeArgs {
    QView x, y;
    int N, C, IH, IW, OH, OW;
    int method, align, half, nchw;
    float scale_y, scale_x;
    long long count;
};

// Lerp(a, b, w) = w * b + (1 - w) * a with every operation rounded (Resize.cpp:17-20)
__device__ __forceinline__ float lerp_ref(float a, float b, float w)
{
    return __fadd_rn(__fmul_rn(w, b), __fmul_rn(__fsub_rn(1.f, w), a));
}

// armnn::roundf (include/armnn/Utils.hpp:43-47)
__device__ __forceinline__ float round_ref(float v)
{
    return v < 0.f ? floorf(__fsub_rn(v, 0.5f)) : floorf(__fadd_rn(v, 0.5f));
}

// PixelScaler (Resize.cpp:36-56)
__device__ __forceinline__ float pixel_scaler(int pixel, float scale, bool half, int method)
{
    if (half && method == 0) return __fsub_rn(__fmul_rn(__fadd_rn((float)pixel, 0.5f), scale), 0.5f);
    if (half && method == 1) return __fmul_rn(__fadd_rn((float)pixel, 0.5f), scale);
    return __fmul_rn((float)pixel, scale);
}

__global__ void __launch_bounds__(256) resize_kernel(const ResizeArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.count) return;
    int n, c, oy, ox;
    long long t = i;
    if (a.nchw) { ox = (int)(t % a.OW); t /= a.OW; oy = (int)(t % a.OH); t /= a.OH; c = (int)(t % a.C); n = (int)(t / a.C); }
    else        { c = (int)(t % a.C); t /= a.C; ox = (int)(t % a.OW); t /= a.OW; oy = (int)(t % a.OH); n = (int)(t / a.OH); }
    const bool half = a.half != 0, nn_round = a.method == 1 && a.align != 0;
    const float iy = pixel_scaler(oy, a.scale_y, half, a.method);
    const float fiy = nn_round ? round_ref(iy) : floorf(iy);
    int y0 = (int)fmaxf(fiy, 0.f);
    const float yw = __fsub_rn(iy, fiy);
    const float ix = pixel_scaler(ox, a.scale_x, half, a.method);
    const float fix = nn_round ? round_ref(ix) : floorf(ix);
    int x0 = (int)fmaxf(fix, 0.f);
    const float xw = __fsub_rn(ix, fix);
    // (the reference reads past the row for coordinates a rounded scale pushes to the input size; here they are clamped)
    y0 = min(y0, a.IH - 1); x0 = min(x0, a.IW - 1);
    int x1, y1;
    if (half) {
        x1 = min((int)fmaxf(ceilf(ix), 0.f), a.IW - 1);
        y1 = min((int)fmaxf(ceilf(iy), 0.f), a.IH - 1);
    } else {
        x1 = min(x0 + 1, a.IW - 1);
        y1 = min(y0 + 1, a.IH - 1);
    }
    auto at = [&](int yy, int xx) -> long long {
        return a.nchw ? (((long long)n * a.C + c) * a.IH + yy) * a.IW + xx : (((long long)n * a.IH + yy) * a.IW + xx) * a.C + c;
    };
    float v;
    if (a.method == 0) {
        const float ly0 = lerp_ref(a.x.get(at(y0, x0)), a.x.get(at(y0, x1)), xw);
        const float ly1 = lerp_ref(a.x.get(at(y1, x0)), a.x.get(at(y1, x1)), xw);
        v = lerp_ref(ly0, ly1, yw);
    } else {
        // the neighbour at distance 0 from (fix, fiy) is (x0, y0): the scaled coordinates are never negative
        v = a.x.get(at(y0, x0));
    }
    a.y.set(i, v);
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_resize_q(const b200k_resize_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "resize_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "resize_q: null tensor pointer");
    B200K_REQUIRE(p->n > 0 && p->c > 0 && p->in_h > 0 && p->in_w > 0 && p->out_h > 0 && p->out_w > 0, B200K_E_INVALID,
                  "resize_q: bad geometry");
    B200K_REQUIRE(p->method == 0 || p->method == 1, B200K_E_INVALID, "resize_q: method %d is neither Bilinear (0) nor NearestNeighbor (1)", p->method);
    B200K_REQUIRE(!(p->align_corners && p->half_pixel_centers), B200K_E_INVALID,
                  "resize_q: align_corners and half_pixel_centers cannot both be set");
    B200K_REQUIRE(p->x.dtype != B200K_S32 && p->y.dtype != B200K_S32, B200K_E_UNSUPPORTED, "resize_q: Signed32 not supported");
    ResizeArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.N = p->n; a.C = p->c; a.IH = p->in_h; a.IW = p->in_w; a.OH = p->out_h; a.OW = p->out_w;
    a.method = p->method; a.align = p->align_corners; a.half = p->half_pixel_centers; a.nchw = p->nchw;
    // CalculateResizeScale (Resize.cpp:27-34), in fp32 like the reference
    a.scale_y = (p->align_corners && p->out_h > 1) ? (float)(p->in_h - 1) / (float)(p->out_h - 1) : (float)p->in_h / (float)p->out_h;
    a.scale_x = (p->align_corners && p->out_w > 1) ? (float)(p->in_w - 1) / (float)(p->out_w - 1) : (float)p->in_w / (float)p->out_w;
    a.count = (long long)p->n * p->c * p->out_h * p->out_w;
    launch_pdl(resize_kernel, dim3(div_up(a.count, 256)), dim3(256), 0, (cudaStream_t)stream, a);
    return check_launch("resize_kernel");
}
