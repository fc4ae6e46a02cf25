// Float32 Convolution2d, DepthwiseConvolution2d and FullyConnected: the reference's loops with the reference's
// rounding (src/backends/reference/workloads/ConvImpl.cpp:118-232, FullyConnected.cpp:32-62) — a rounded product and
// a rounded sum per term, terms in the reference's order — so that the results are CpuRef's bit for bit.  One thread
// per output element on the CUDA cores: coverage for float graphs, not a fast path.
#include "common.cuh"

namespace b200k {

struct ConvF32Args {
    const float* x; const float* w; const float* bias; float* y;
    int N, H, W, C, OH, OW, OC, KH, KW, sh, sw, pt, pl, dh, dw, dm;
    long long total;
};

template <bool DEPTHWISE>
__global__ void __launch_bounds__(256) conv_f32_kernel(const ConvF32Args a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    const int co = (int)(i % a.OC);
    long long t = i / a.OC;
    const int ox = (int)(t % a.OW); t /= a.OW;
    const int oy = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    float sum = 0.0f;
    const int c_end = DEPTHWISE ? 1 : a.C;
    for (int c = 0; c < c_end; ++c) {
        const int ci = DEPTHWISE ? co / a.dm : c;
        for (int ky = 0; ky < a.KH; ++ky) {
            const int iy = oy * a.sh + ky * a.dh - a.pt;
            for (int kx = 0; kx < a.KW; ++kx) {
                const int ix = ox * a.sw + kx * a.dw - a.pl;
                const float wv = DEPTHWISE ? a.w[((long long)ky * a.KW + kx) * a.OC + co]
                                           : a.w[(((long long)co * a.KH + ky) * a.KW + kx) * a.C + ci];
                const bool inside = iy >= 0 && iy < a.H && ix >= 0 && ix < a.W;
                const float xv = inside ? a.x[(((long long)n * a.H + iy) * a.W + ix) * a.C + ci] : 0.0f;
                sum = __fadd_rn(sum, __fmul_rn(wv, xv));
            }
        }
    }
    if (a.bias) sum = __fadd_rn(sum, a.bias[co]);
    a.y[i] = sum;
}

struct FcF32Args { const float* x; const float* w; const float* bias; float* y; int M, K, N, transpose_w; };

__global__ void __launch_bounds__(256) fc_f32_kernel(const FcF32Args a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.M * a.N) return;
    const int o = (int)(i % a.N), m = (int)(i / a.N);
    float out = 0.f;
    for (int k = 0; k < a.K; ++k) {
        const float wv = a.transpose_w ? a.w[(long long)o * a.K + k] : a.w[(long long)k * a.N + o];
        out = __fadd_rn(out, __fmul_rn(wv, a.x[(long long)m * a.K + k]));
    }
    if (a.bias) out = __fadd_rn(out, a.bias[o]);
    a.y[i] = out;
}

struct BmmF32Args { const float* x; const float* y; float* out; int B, M, K, N, tx, ty; long long bsx, bsy; };

// BatchMatMulImpl.cpp:15-139: every output is the sum over k, in order, of separately rounded products
__global__ void __launch_bounds__(256) bmm_f32_kernel(const BmmF32Args a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)a.B * a.M * a.N) return;
    const int n = (int)(i % a.N);
    const long long t = i / a.N;
    const int m = (int)(t % a.M), b = (int)(t / a.M);
    const float* x = a.x + b * a.bsx;
    const float* y = a.y + b * a.bsy;
    float sum = 0.f;
    for (int k = 0; k < a.K; ++k) {
        const float xv = a.tx ? x[(long long)k * a.M + m] : x[(long long)m * a.K + k];
        const float yv = a.ty ? y[(long long)n * a.K + k] : y[(long long)k * a.N + n];
        sum = __fadd_rn(sum, __fmul_rn(xv, yv));
    }
    a.out[i] = sum;
}

static int launch_conv_f32(const b200k_conv2d_params* p, cudaStream_t s, bool depthwise, const char* who)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "%s: null params", who);
    B200K_REQUIRE(p->x.data && p->w.data && p->y.data, B200K_E_INVALID, "%s: null tensor pointer", who);
    B200K_REQUIRE(p->x.dtype == B200K_F32 && p->w.dtype == B200K_F32 && p->y.dtype == B200K_F32 &&
                  (!p->bias.data || p->bias.dtype == B200K_F32), B200K_E_UNSUPPORTED, "%s: every tensor must be Float32", who);
    B200K_REQUIRE(!p->add_operand.data, B200K_E_UNSUPPORTED, "%s: a fused Add is only available on quantised Convolution2d", who);
    B200K_REQUIRE(p->n > 0 && p->h > 0 && p->wd > 0 && p->c > 0 && p->oh > 0 && p->ow > 0 && p->oc > 0 && p->kh > 0 && p->kw > 0 &&
                  p->stride_h > 0 && p->stride_w > 0 && p->dil_h > 0 && p->dil_w > 0, B200K_E_INVALID, "%s: bad geometry", who);
    B200K_REQUIRE(!depthwise || p->oc % p->c == 0, B200K_E_INVALID, "%s: output channels %d not a multiple of input channels %d", who, p->oc, p->c);
    ConvF32Args a;
    a.x = (const float*)p->x.data; a.w = (const float*)p->w.data; a.bias = (const float*)p->bias.data; a.y = (float*)p->y.data;
    a.N = p->n; a.H = p->h; a.W = p->wd; a.C = p->c; a.OH = p->oh; a.OW = p->ow; a.OC = p->oc; a.KH = p->kh; a.KW = p->kw;
    a.sh = p->stride_h; a.sw = p->stride_w; a.pt = p->pad_top; a.pl = p->pad_left; a.dh = p->dil_h; a.dw = p->dil_w;
    a.dm = depthwise ? p->oc / p->c : 1;
    a.total = (long long)p->n * p->oh * p->ow * p->oc;
    if (depthwise) launch_pdl(conv_f32_kernel<true>, dim3(div_up(a.total, 256)), dim3(256), 0, s, a);
    else           launch_pdl(conv_f32_kernel<false>, dim3(div_up(a.total, 256)), dim3(256), 0, s, a);
    return check_launch("conv_f32_kernel");
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_conv2d_f32(const b200k_conv2d_params* p, void* stream)
{
    return launch_conv_f32(p, (cudaStream_t)stream, false, "conv2d_f32");
}

extern "C" int b200k_dwconv2d_f32(const b200k_conv2d_params* p, void* stream)
{
    return launch_conv_f32(p, (cudaStream_t)stream, true, "dwconv2d_f32");
}

extern "C" int b200k_fully_connected_f32(const b200k_fc_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "fully_connected_f32: null params");
    B200K_REQUIRE(p->x.data && p->w.data && p->y.data, B200K_E_INVALID, "fully_connected_f32: null tensor pointer");
    B200K_REQUIRE(p->x.dtype == B200K_F32 && p->w.dtype == B200K_F32 && p->y.dtype == B200K_F32 &&
                  (!p->bias.data || p->bias.dtype == B200K_F32), B200K_E_UNSUPPORTED, "fully_connected_f32: every tensor must be Float32");
    B200K_REQUIRE(p->m > 0 && p->k > 0 && p->n > 0, B200K_E_INVALID, "fully_connected_f32: bad shape");
    FcF32Args a;
    a.x = (const float*)p->x.data; a.w = (const float*)p->w.data; a.bias = (const float*)p->bias.data; a.y = (float*)p->y.data;
    a.M = p->m; a.K = p->k; a.N = p->n; a.transpose_w = p->transpose_w;
    launch_pdl(fc_f32_kernel, dim3(div_up((long long)p->m * p->n, 256)), dim3(256), 0, (cudaStream_t)stream, a);
    return check_launch("fc_f32_kernel");
}

extern "C" int b200k_batch_matmul_f32(const b200k_bmm_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "batch_matmul_f32: null params");
    B200K_REQUIRE(p->x.data && p->y.data && p->out.data, B200K_E_INVALID, "batch_matmul_f32: null tensor pointer");
    B200K_REQUIRE(p->x.dtype == B200K_F32 && p->y.dtype == B200K_F32 && p->out.dtype == B200K_F32, B200K_E_UNSUPPORTED,
                  "batch_matmul_f32: every tensor must be Float32");
    B200K_REQUIRE(p->batch > 0 && p->m > 0 && p->k > 0 && p->n > 0 && p->batch_stride_x >= 0 && p->batch_stride_y >= 0,
                  B200K_E_INVALID, "batch_matmul_f32: bad shape");
    BmmF32Args a;
    a.x = (const float*)p->x.data; a.y = (const float*)p->y.data; a.out = (float*)p->out.data;
    a.B = p->batch; a.M = p->m; a.K = p->k; a.N = p->n; a.tx = p->transpose_x; a.ty = p->transpose_y;
    a.bsx = p->batch_stride_x; a.bsy = p->batch_stride_y;
    launch_pdl(bmm_f32_kernel, dim3(div_up((long long)p->batch * p->m * p->n, 256)), dim3(256), 0, (cudaStream_t)stream, a);
    return check_launch("bmm_f32_kernel");
}
