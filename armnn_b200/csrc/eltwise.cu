// ElementwiseBinary (Add / Mul / Sub / Div / Maximum / Minimum / SqDiff / Power / FloorDiv) and Prelu with numpy-style broadcast,
// standalone Activation, and Quantize / Dequantize / requantize.  All bandwidth-bound: same-shape 8-bit
// operands take a 128-bit vector path (16 elements per thread), everything else a scalar path.
// Arithmetic is CpuRef's: dequantise each operand with its own scale/offset, apply the fp32 operation
// unfused, re-quantise (RefElementwiseBinaryWorkload.cpp:27-132, Activation.cpp:13-119,
// RefQuantizeWorkload.cpp:14-45, Dequantize.cpp:11-28 of the Arm NN tree).
#include "common.cuh"
#include <cuda_fp16.h>

namespace b200k {

__device__ __forceinline__ float binary_op(int op, float a, float b)
{
    switch (op) {
        case 0:  return __fadd_rn(a, b);
        case 1:  return __fdiv_rn(a, b);
        case 2:  return a > b ? a : b;
        case 3:  return a < b ? a : b;
        case 4:  return __fmul_rn(a, b);
        case 5:  return __fsub_rn(a, b);
        case 7:  return powf(a, b);
        case 8:  return (float)floor((double)a / (double)b);
        case 100: return a < 0.f ? __fmul_rn(b, a) : a;      // Prelu: b is alpha
        // armnn::ComparisonOperation + 200 and armnn::LogicalBinaryOperation + 210: 1.0 or 0.0, stored as a Boolean byte
        case 200: return a == b ? 1.f : 0.f;
        case 201: return a > b ? 1.f : 0.f;
        case 202: return a >= b ? 1.f : 0.f;
        case 203: return a < b ? 1.f : 0.f;
        case 204: return a <= b ? 1.f : 0.f;
        case 205: return a != b ? 1.f : 0.f;
        case 210: return (a != 0.f && b != 0.f) ? 1.f : 0.f;
        case 211: return (a != 0.f || b != 0.f) ? 1.f : 0.f;
        default: { float d = __fsub_rn(a, b); return __fmul_rn(d, d); }
    }
}

struct EltArgs {
    QView a, b, out;
    int op, clo, chi;
    int dout[4];
    long long sa[4], sb[4];
    long long total;
};

__global__ void __launch_bounds__(256) eltwise_vec16_kernel(const EltArgs e)
{
    pdl_enter();
    const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 16;
    if (idx >= e.total) return;
    uint8_t ra[16], rb[16], ro[16];
    *(uint4*)ra = *(const uint4*)((const uint8_t*)e.a.data + idx);
    *(uint4*)rb = *(const uint4*)((const uint8_t*)e.b.data + idx);
    #pragma unroll
    for (int k = 0; k < 16; ++k) {
        const int qa = e.a.dtype == B200K_U8 ? (int)ra[k] : (int)(int8_t)ra[k];
        const int qb = e.b.dtype == B200K_U8 ? (int)rb[k] : (int)(int8_t)rb[k];
        const float r = binary_op(e.op, dequantize_dev(qa, e.a.scale, e.a.zp), dequantize_dev(qb, e.b.scale, e.b.zp));
        ro[k] = (uint8_t)min(max(e.out.quant(r), e.clo), e.chi);
    }
    *(uint4*)((uint8_t*)e.out.data + idx) = *(const uint4*)ro;
}

__global__ void __launch_bounds__(256) eltwise_generic_kernel(const EltArgs e)
{
    pdl_enter();
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= e.total) return;
    long long t = idx;
    const int i3 = (int)(t % e.dout[3]); t /= e.dout[3];
    const int i2 = (int)(t % e.dout[2]); t /= e.dout[2];
    const int i1 = (int)(t % e.dout[1]);
    const int i0 = (int)(t / e.dout[1]);
    const long long ia = i0 * e.sa[0] + i1 * e.sa[1] + i2 * e.sa[2] + i3 * e.sa[3];
    const long long ib = i0 * e.sb[0] + i1 * e.sb[1] + i2 * e.sb[2] + i3 * e.sb[3];
    const float r = binary_op(e.op, e.a.get(ia), e.b.get(ib));
    if (e.out.dtype == B200K_F32) { ((float*)e.out.data)[idx] = r; return; }
    store_q_dev((void*)e.out.data, e.out.dtype, idx, min(max(e.out.quant(r), e.clo), e.chi));
}

__device__ __forceinline__ float activation_f(int fn, float in, float a, float b)
{
    switch (fn) {
        case 0:  return __fdiv_rn(1.f, __fadd_rn(1.f, expf(-in)));
        case 1:  return __fmul_rn(a, tanhf(__fmul_rn(b, in)));
        case 2:  return __fadd_rn(__fmul_rn(a, in), b);
        case 3:  return fmaxf(0.f, in);
        case 4:  return fminf(a, fmaxf(b, in));
        case 5:  return logf(__fadd_rn(1.0f, expf(in)));
        case 6:  return in > 0.0f ? in : __fmul_rn(in, a);
        case 7:  return in < 0 ? -in : in;
        case 8:  return __fsqrt_rn(in);
        case 9:  return __fmul_rn(in, in);
        case 10: return (in >= 0) ? in : __fmul_rn(a, __fsub_rn(expf(in), 1.f));
        case 12: return __fmul_rn(in, __fmul_rn(0.5f, __fadd_rn(1.0f, erff((float)((double)in / 1.4142135623730951)))));
        // FakeQuantization (RefFakeQuantizationFloat32Workload.cpp:15-27): a = min, b = max; the value as an 8-bit code
        case 50: {
            const float range = __fsub_rn(b, a);
            const float scale = __fdiv_rn(range, 255.f);
            const int offset = (int)__fdiv_rn(__fmul_rn(-a, 255.f), range);
            return (float)quantize_dev(in, scale, offset, 0.f, 255.f);
        }
        // armnn::UnaryOperation + 100 (ElementwiseUnary): Abs, Exp, Sqrt, Rsqrt, Neg, -, Log, Sin, Ceil; 109: the Floor layer
        case 100: return fabsf(in);
        case 101: return expf(in);
        case 102: return __fsqrt_rn(in);
        case 103: return __fdiv_rn(1.f, __fsqrt_rn(in));
        case 104: return -in;
        case 105: return in != 0.f ? 0.f : 1.f;           // LogicalNot of a Boolean byte
        case 106: return logf(in);
        case 107: return sinf(in);
        case 108: return ceilf(in);
        case 109: return floorf(in);
        default: return __fdiv_rn(__fmul_rn(in, fminf(fmaxf(__fadd_rn(in, 3.f), 0.0f), 6.0f)), 6.f);
    }
}

struct UnaryArgs { QView x, y; long long count; int fn; float a, b; };

// fn < 0: plain conversion (Quantize / Dequantize / requantize)
__global__ void __launch_bounds__(256) unary_kernel(const UnaryArgs u)
{
    pdl_enter();
    const long long base = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    #pragma unroll
    for (int k = 0; k < 4; ++k) {
        const long long i = base + k;
        if (i >= u.count) return;
        float v = u.x.get(i);
        if (u.fn >= 0) v = activation_f(u.fn, v, u.a, u.b);
        u.y.set(i, v);
    }
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_eltwise_q8(const b200k_eltwise_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "eltwise_q8: null params");
    B200K_REQUIRE(p->a.data && p->b.data && p->out.data, B200K_E_INVALID, "eltwise_q8: null tensor pointer");
    B200K_REQUIRE(p->rank >= 1 && p->rank <= 4, B200K_E_UNSUPPORTED, "eltwise_q8: rank %d not in [1,4]", p->rank);
    B200K_REQUIRE((p->op >= 0 && p->op <= 8) || p->op == B200K_ELTWISE_PRELU || (p->op >= 200 && p->op <= 205) || p->op == 210 || p->op == 211,
                  B200K_E_UNSUPPORTED, "eltwise_q8: unsupported binary operation %d", p->op);
    B200K_REQUIRE(p->a.dtype != B200K_S32 && p->b.dtype != B200K_S32 && p->out.dtype != B200K_S32, B200K_E_UNSUPPORTED,
                  "eltwise_q8: Signed32 not supported");
    EltArgs e;
    e.a = make_view(p->a); e.b = make_view(p->b); e.out = make_view(p->out);
    e.op = p->op;
    int lo, hi;
    type_range(p->out.dtype, lo, hi);
    e.clo = p->clamp_lo > lo ? p->clamp_lo : lo;
    e.chi = p->clamp_hi < hi ? p->clamp_hi : hi;
    int da[4] = {1, 1, 1, 1}, db[4] = {1, 1, 1, 1};
    for (int i = 0; i < 4; ++i) e.dout[i] = 1;
    bool same = true;
    for (int i = 0; i < p->rank; ++i) {
        const int d = 4 - p->rank + i;
        da[d] = p->shape_a[i]; db[d] = p->shape_b[i]; e.dout[d] = p->shape_out[i];
        B200K_REQUIRE(da[d] > 0 && db[d] > 0 && e.dout[d] > 0, B200K_E_INVALID, "eltwise_q8: non-positive dimension");
        B200K_REQUIRE((da[d] == e.dout[d] || da[d] == 1) && (db[d] == e.dout[d] || db[d] == 1), B200K_E_INVALID,
                      "eltwise_q8: shapes are not broadcast-compatible in dimension %d", i);
        same = same && da[d] == e.dout[d] && db[d] == e.dout[d];
    }
    long long ta = 1, tb = 1;
    e.total = 1;
    for (int i = 3; i >= 0; --i) {
        e.sa[i] = da[i] == 1 ? 0 : ta;  ta *= da[i];
        e.sb[i] = db[i] == 1 ? 0 : tb;  tb *= db[i];
        e.total *= e.dout[i];
    }
    cudaStream_t s = (cudaStream_t)stream;
    const uintptr_t al = (uintptr_t)p->a.data | (uintptr_t)p->b.data | (uintptr_t)p->out.data;
    if (same && is_q8(p->a.dtype) && is_q8(p->b.dtype) && is_q8(p->out.dtype) && (e.total % 16) == 0 && (al & 15) == 0) {
        launch_pdl(eltwise_vec16_kernel, dim3((unsigned)(div_up(e.total / 16, 256))), dim3(256), 0, s, e);
        return check_launch("eltwise_vec16_kernel");
    }
    launch_pdl(eltwise_generic_kernel, dim3((unsigned)(div_up(e.total, 256))), dim3(256), 0, s, e);
    return check_launch("eltwise_generic_kernel");
}

static int launch_unary(const b200k_qtensor& x, const b200k_qtensor& y, long long count, int fn, float a, float b,
                        void* stream, const char* what, bool s32_out = false)
{
    B200K_REQUIRE(x.data && y.data, B200K_E_INVALID, "%s: null tensor pointer", what);
    B200K_REQUIRE(count >= 0, B200K_E_INVALID, "%s: negative element count", what);
    B200K_REQUIRE(x.dtype >= B200K_U8 && x.dtype <= B200K_F32 && y.dtype >= B200K_U8 && y.dtype <= B200K_F32 &&
                  (y.dtype != B200K_S32 || s32_out), B200K_E_UNSUPPORTED, "%s: unsupported data type", what);
    if (count == 0) return B200K_OK;
    UnaryArgs u;
    u.x = make_view(x); u.y = make_view(y); u.count = count; u.fn = fn; u.a = a; u.b = b;
    launch_pdl(unary_kernel, dim3((unsigned)(div_up(div_up(count, 4), 256))), dim3(256), 0, (cudaStream_t)stream, u);
    return check_launch("unary_kernel");
}

extern "C" int b200k_activation_q8(const b200k_activation_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "activation_q8: null params");
    B200K_REQUIRE((p->function >= 0 && p->function <= 12) || p->function == B200K_ACTIVATION_FAKE_QUANTIZATION, B200K_E_UNSUPPORTED,
                  "activation_q8: unsupported activation function %d", p->function);
    B200K_REQUIRE(p->function != B200K_ACTIVATION_FAKE_QUANTIZATION || (p->x.dtype == B200K_F32 && p->y.dtype == B200K_F32 && p->b > p->a),
                  B200K_E_INVALID, "activation_q8: FakeQuantization takes Float32 tensors and min < max");
    return launch_unary(p->x, p->y, p->count, p->function, p->a, p->b, stream, "activation_q8");
}

extern "C" int b200k_unary_q(const b200k_unary_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "unary_q: null params");
    B200K_REQUIRE(p->operation >= 0 && p->operation <= 9, B200K_E_UNSUPPORTED,
                  "unary_q: unsupported unary operation %d", p->operation);
    return launch_unary(p->x, p->y, p->count, 100 + p->operation, 0.f, 0.f, stream, "unary_q");
}

// armnn::Cast (RefCastWorkload.cpp:13-36, 95-106): both tensors read with scale 1 and offset 0 whatever their TensorInfo
// says; floor before an integer output, the value itself for a float output.
extern "C" int b200k_cast_q(const b200k_convert_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "cast_q: null params");
    b200k_qtensor x = p->x, y = p->y;
    x.scale = 1.0f; x.zero_point = 0; x.scales = nullptr;
    y.scale = 1.0f; y.zero_point = 0; y.scales = nullptr;
    return launch_unary(x, y, p->count, y.dtype == B200K_F32 ? -1 : 109, 0.f, 0.f, stream, "cast_q", true);
}

extern "C" int b200k_convert_q(const b200k_convert_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "convert_q: null params");
    return launch_unary(p->x, p->y, p->count, -1, 0.f, 0.f, stream, "convert_q");
}

// ---- ConvertFp16ToFp32 / ConvertFp32ToFp16 ---------------------------------------------------------------------
// armnnUtils::FloatingPointConverter (src/armnnUtils/FloatingPointConverter.cpp:17-45) over half_float::half with
// round-to-nearest, ties to even (src/armnnUtils/Half.hpp:11-16): widening is exact, narrowing is cvt.rn.f16.f32 with
// infinities replaced by the largest finite half.

namespace b200k {

__global__ void __launch_bounds__(256) convert_fp16_kernel(const void* x, void* y, long long count, int to_half)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    if (to_half) {
        // FloatingPointConverter.cpp:32-40: a result of infinity (overflow, or an infinite input) becomes the largest finite half
        unsigned short h = __half_as_ushort(__float2half_rn(((const float*)x)[i]));
        if ((h & 0x7fffu) == 0x7c00u) h = (unsigned short)((h & 0x8000u) | 0x7bffu);
        ((unsigned short*)y)[i] = h;
    }
    else         ((float*)y)[i] = __half2float(((const __half*)x)[i]);
}

}  // namespace b200k

extern "C" int b200k_convert_fp16(const b200k_convert_fp16_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "convert_fp16: null params");
    B200K_REQUIRE(p->x && p->y, B200K_E_INVALID, "convert_fp16: null tensor pointer");
    B200K_REQUIRE(p->count >= 0, B200K_E_INVALID, "convert_fp16: negative element count");
    if (p->count == 0) return B200K_OK;
    B200K_REQUIRE(p->count / 256 < (1ll << 31) - 1, B200K_E_TOOBIG, "convert_fp16: tensor too large");
    launch_pdl(b200k::convert_fp16_kernel, dim3(div_up(p->count, 256)), dim3(256), 0, (cudaStream_t)stream, p->x, p->y,
               (long long)p->count, (int)p->to_half);
    return check_launch("convert_fp16_kernel");
}

// ---- Pad ------------------------------------------------------------------------------------------------------

namespace b200k {

struct PadArgs { QView x, y; int rank; int in_shape[4], out_shape[4], before[4]; float pad_value; long long count; int mode; };

// armnn::Pad (src/backends/reference/workloads/Pad.cpp:37-170): every output element is either the input element at
// the shifted position, re-encoded with the output's quantisation, or the pad value.  For a quantised output the
// pad value is already a quantised number: the reference encodes it with scale 1 and offset 0 (Pad.cpp:76-83).
__global__ void __launch_bounds__(256) pad_kernel(const PadArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.count) return;
    long long rest = i, src = 0, stride = 1;
    bool inside = true;
    // innermost dimension first: build the source index while peeling coordinates off the flat output index
    int coord[4];
    for (int d = a.rank - 1; d >= 0; --d) { coord[d] = (int)(rest % a.out_shape[d]); rest /= a.out_shape[d]; }
    for (int d = a.rank - 1; d >= 0; --d) {
        int c = coord[d] - a.before[d];
        if (a.mode != 0) {
            // armnn::MirrorPad (MirrorPad.cpp:95-125): Reflect (1) mirrors about the edge element, Symmetric (2) repeats it
            const int n = a.in_shape[d], edge = a.mode == 1 ? 0 : 1;
            if (c < 0) c = -c - edge;
            else if (c >= n) c = 2 * n - 2 + edge - c;
        }
        inside = inside && c >= 0 && c < a.in_shape[d];
        src += (long long)c * stride;
        stride *= a.in_shape[d];
    }
    if (inside) { a.y.set(i, a.x.get(src)); return; }
    if (a.y.dtype == B200K_F32) { ((float*)a.y.data)[i] = a.pad_value; return; }
    store_q_dev((void*)a.y.data, a.y.dtype, i, quantize_dev(a.pad_value, 1.0f, 0, a.y.tlo, a.y.thi));
}

}  // namespace b200k

extern "C" int b200k_pad_q(const b200k_pad_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "pad_q: null params");
    B200K_REQUIRE(p->x.data && p->y.data, B200K_E_INVALID, "pad_q: null tensor pointer");
    B200K_REQUIRE(p->rank >= 1 && p->rank <= 4, B200K_E_UNSUPPORTED, "pad_q: rank %d not in [1, 4]", p->rank);
    B200K_REQUIRE(p->x.dtype != B200K_S32 && p->y.dtype != B200K_S32, B200K_E_UNSUPPORTED, "pad_q: Signed32 not supported");
    PadArgs a;
    a.x = make_view(p->x); a.y = make_view(p->y);
    a.rank = p->rank; a.pad_value = p->pad_value; a.mode = p->mode;
    B200K_REQUIRE(p->mode >= 0 && p->mode <= 2, B200K_E_INVALID, "pad_q: padding mode %d is not Constant (0), Reflect (1) or Symmetric (2)", p->mode);
    a.count = 1;
    for (int d = 0; d < 4; ++d) { a.in_shape[d] = a.out_shape[d] = 1; a.before[d] = 0; }
    for (int d = 0; d < p->rank; ++d) {
        B200K_REQUIRE(p->shape[d] > 0 && p->pad_before[d] >= 0 && p->pad_after[d] >= 0, B200K_E_INVALID, "pad_q: bad shape / padding");
        // MirrorPad.cpp:66-74: a mirrored border cannot be wider than the tensor (less its edge element for Reflect)
        B200K_REQUIRE(p->mode == 0 || (p->pad_before[d] <= p->shape[d] - (p->mode == 1) && p->pad_after[d] <= p->shape[d] - (p->mode == 1)),
                      B200K_E_INVALID, "pad_q: mirrored padding wider than dimension %d", d);
        a.in_shape[d] = p->shape[d]; a.before[d] = p->pad_before[d];
        a.out_shape[d] = p->shape[d] + p->pad_before[d] + p->pad_after[d];
        a.count *= a.out_shape[d];
    }
    launch_pdl(pad_kernel, dim3(div_up(a.count, 256)), dim3(256), 0, (cudaStream_t)stream, a);
    return check_launch("pad_kernel");
}
