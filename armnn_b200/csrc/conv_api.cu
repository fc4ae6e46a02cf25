// Convolution2d entry points: argument checks, the choice between the tcgen05 implicit-GEMM kernel and the
// shape-agnostic CUDA-core kernel, and the channel-padding layer that lets channel counts which are not multiples of
// 16 (MobileNet's 24-channel bottlenecks) use the tcgen05 kernel.
//
// TMA needs 16-byte pixel and row strides.  For other channel counts the weights are zero-padded once at load time
// (b200k_conv2d_pack), the input is copied into caller-provided scratch with zero-filled extra channels before the
// launch, and / or the output is computed into scratch with the padded width and compacted afterwards.  Zero weights
// and zero inputs contribute nothing to any of the sums the kernel forms; the one place that counts taps (the
// K zx zw term of the zero-point correction) is told the real channel count.
#include <string.h>
#include "common.cuh"

namespace b200k {

int launch_conv_dp4a(const b200k_conv2d_params* p, cudaStream_t stream);
int launch_conv_tc(const b200k_conv2d_params* p, cudaStream_t stream, int kvalid_c);   // B200K_E_UNSUPPORTED if not eligible
bool conv_tc_eligible(const b200k_conv2d_params* p);
size_t tc_pack_bytes(int oc, int kh, int kw, int c);
size_t tc_scratch_bytes(const b200k_conv2d_params* p);
int tc_pack(const b200k_conv2d_params* p, void* packed, cudaStream_t stream);
int tc_pack_host_tables(const b200k_conv2d_params* p, void* packed, cudaStream_t stream);

static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
static int up16(int v) { return (v + 15) & ~15; }

static bool wants_padding(int oc, int c) { return c > 16 && (c % 16 != 0 || oc % 16 != 0) && c % 8 == 0 && oc % 8 == 0; }

// Where the padded copies live: behind the regular tables in `packed`, and in `scratch`.
struct PadPlan {
    bool ok;
    int cpad, ocpad;
    size_t w_off, bias_off, ws_off, bs_off, inner_off, pack_total;       // relative to the start of the pad region
    size_t x_off, y_off, acc_off, scratch_total;
};

static PadPlan pad_plan(const b200k_conv2d_params* p)
{
    PadPlan r;
    memset(&r, 0, sizeof(r));
    if (!wants_padding(p->oc, p->c) || p->kh <= 0 || p->kw <= 0) return r;
    r.cpad = up16(p->c); r.ocpad = up16(p->oc);
    size_t o = 0;
    r.w_off = o;     o += up256((size_t)r.ocpad * p->kh * p->kw * r.cpad);
    r.bias_off = o;  o += up256((size_t)r.ocpad * 4);
    r.ws_off = o;    o += up256((size_t)r.ocpad * 4);
    r.bs_off = o;    o += up256((size_t)r.ocpad * 4);
    r.inner_off = o; o += up256(tc_pack_bytes(r.ocpad, p->kh, p->kw, r.cpad));
    r.pack_total = o;
    const size_t pixels_in = (size_t)(p->n > 0 ? p->n : 0) * (p->h > 0 ? p->h : 0) * (p->wd > 0 ? p->wd : 0);
    const size_t pixels_out = (size_t)(p->n > 0 ? p->n : 0) * (p->oh > 0 ? p->oh : 0) * (p->ow > 0 ? p->ow : 0);
    size_t s = 0;
    r.x_off = s;   if (p->c % 16 != 0) s += up256(pixels_in * r.cpad);
    r.y_off = s;   if (p->oc % 16 != 0) s += up256(pixels_out * r.ocpad);
    r.acc_off = s; if (p->oc % 16 != 0 && p->acc_out) s += up256(pixels_out * r.ocpad * 4);
    r.scratch_total = s;
    r.ok = true;
    return r;
}

// The same convolution on the padded tensors.
static b200k_conv2d_params padded_params(const b200k_conv2d_params* p, const PadPlan& pl)
{
    b200k_conv2d_params q = *p;
    uint8_t* region = (uint8_t*)p->packed + up256(tc_pack_bytes(p->oc, p->kh, p->kw, p->c));
    q.c = pl.cpad; q.oc = pl.ocpad;
    q.w.data = region + pl.w_off;
    if (p->w.scales) q.w.scales = (const float*)(region + pl.ws_off);
    if (p->bias.data) {
        q.bias.data = region + pl.bias_off;
        if (p->bias.scales) q.bias.scales = (const float*)(region + pl.bs_off);
    }
    q.packed = region + pl.inner_off;
    q.scratch = nullptr; q.scratch_bytes = 0;
    if (p->c % 16 != 0) q.x.data = (uint8_t*)p->scratch + pl.x_off;
    if (p->oc % 16 != 0) {
        q.y.data = (uint8_t*)p->scratch + pl.y_off;
        if (p->acc_out) q.acc_out = (int32_t*)((uint8_t*)p->scratch + pl.acc_off);
    }
    return q;
}

// dst[row][0..wd) = src[row][0..ws) followed by zeros (wd > ws) or cut (wd < ws); widths in units of 8 bytes
__global__ void __launch_bounds__(256) repitch_rows_kernel(const uint2* src, uint2* dst, long long rows, int ws, int wd)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= rows * wd) return;
    const long long row = i / wd;
    const int g = (int)(i - row * wd);
    dst[i] = g < ws ? src[row * ws + g] : make_uint2(0, 0);
}

// wp[o][tap][0..cpad) = w[o][tap][0..c) for o < oc, zeros elsewhere
__global__ void pad_weights_kernel(const uint8_t* w, uint8_t* wp, int oc, int taps, int c, int ocpad, int cpad)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)ocpad * taps * cpad) return;
    const int ch = (int)(i % cpad);
    const long long t = i / cpad;
    const int tap = (int)(t % taps), o = (int)(t / taps);
    wp[i] = (o < oc && ch < c) ? w[((long long)o * taps + tap) * c + ch] : (uint8_t)0;
}

__global__ void pad_vec_kernel(const uint32_t* src, uint32_t* dst, int n, int npad, uint32_t fill)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < npad) dst[i] = i < n ? src[i] : fill;
}

static bool padded_path_eligible(const b200k_conv2d_params* p, PadPlan& pl, b200k_conv2d_params& q)
{
    if (p->add_operand.data || !p->packed || !p->scratch) return false;
    if (!p->x.data || !p->w.data || !p->y.data) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->w.dtype) || !is_q8(p->y.dtype)) return false;
    if ((((uintptr_t)p->x.data | (uintptr_t)p->y.data | (uintptr_t)p->scratch | (uintptr_t)p->packed) & 15) != 0) return false;
    if (p->acc_out && (((uintptr_t)p->acc_out) & 7) != 0) return false;
    pl = pad_plan(p);
    if (!pl.ok || p->scratch_bytes < pl.scratch_total) return false;
    q = padded_params(p, pl);
    return conv_tc_eligible(&q);
}

static int launch_padded(const b200k_conv2d_params* p, const PadPlan& pl, const b200k_conv2d_params& q, cudaStream_t stream)
{
    const long long pixels_in = (long long)p->n * p->h * p->wd, pixels_out = (long long)p->n * p->oh * p->ow;
    if (p->c % 16 != 0) {
        launch_pdl(repitch_rows_kernel, dim3((unsigned)div_up(pixels_in * (pl.cpad / 8), 256)), dim3(256), 0, stream,
                   (const uint2*)p->x.data, (uint2*)q.x.data, pixels_in, p->c / 8, pl.cpad / 8);
        int rc = check_launch("repitch_rows_kernel");
        if (rc) return rc;
    }
    int rc = launch_conv_tc(&q, stream, p->c);
    if (rc) return rc;
    if (p->oc % 16 != 0) {
        launch_pdl(repitch_rows_kernel, dim3((unsigned)div_up(pixels_out * (p->oc / 8), 256)), dim3(256), 0, stream,
                   (const uint2*)q.y.data, (uint2*)p->y.data, pixels_out, pl.ocpad / 8, p->oc / 8);
        rc = check_launch("repitch_rows_kernel");
        if (rc) return rc;
        if (p->acc_out) {
            repitch_rows_kernel<<<div_up(pixels_out * (p->oc / 2), 256), 256, 0, stream>>>(
                (const uint2*)q.acc_out, (uint2*)p->acc_out, pixels_out, pl.ocpad / 2, p->oc / 2);
            rc = check_launch("repitch_rows_kernel");
        }
    }
    return rc;
}

// ---- 1x1 convolutions whose channel counts the tensor-core kernel cannot take as they are ---------------------------
//
// A 1x1, stride-1 convolution is the GEMM [M, C] x [C, OC].  Taking g consecutive pixels as one row turns it into
// [M / g, g C] x [g C, g OC] with a block-diagonal weight matrix (g copies of the weights; every other entry the weight
// zero point, i.e. a real zero), on the very same input and output bytes: no copy of either tensor.  g is the smallest
// power of two that makes g C and g OC multiples of 16 (and g C at least 32: the few-channel kernels are built for
// stems with wide filters, not for this; and g OC at least 64, the narrowest tile of the kernel).  The g-fold redundant multiplications are free on a layer that is bound by
// its memory traffic.  Needs M % g == 0; the channel-padded path below takes what is left.
struct GroupPlan {
    bool ok;
    int g, cg, ocg;
    size_t w_off, bias_off, ws_off, bs_off, inner_off, pack_total;      // relative to the start of the group region
};

static GroupPlan group_plan(int oc, int kh, int kw, int c)
{
    GroupPlan r;
    memset(&r, 0, sizeof(r));
    if (kh != 1 || kw != 1 || oc <= 0 || c <= 0) return r;
    if (c % 16 == 0 && oc % 16 == 0 && c > 16 && oc >= 64) return r;   // the kernel takes these directly
    // only the input channels are odd: a zero-padded copy of the (small) input is cheaper than the n-tiles that g OC
    // output columns would take
    if (c > 16 && oc % 16 == 0 && wants_padding(oc, c)) return r;
    int g = 1;
    while (g <= 16 && ((g * c) % 16 != 0 || (g * oc) % 16 != 0 || g * c < 32 || g * oc < 64)) g *= 2;
    if (g < 2 || g > 16 || (long long)g * oc > 4096 || (long long)g * c > 4096) return r;
    r.g = g; r.cg = g * c; r.ocg = g * oc;
    size_t o = 0;
    r.w_off = o;     o += up256((size_t)r.ocg * r.cg);
    r.bias_off = o;  o += up256((size_t)r.ocg * 4);
    r.ws_off = o;    o += up256((size_t)r.ocg * 4);
    r.bs_off = o;    o += up256((size_t)r.ocg * 4);
    r.inner_off = o; o += up256(tc_pack_bytes(r.ocg, 1, 1, r.cg));
    r.pack_total = o;
    r.ok = true;
    return r;
}

// start of the group region in `packed`: behind the regular tables and the channel-padded copies
static size_t group_region_offset(int oc, int kh, int kw, int c)
{
    size_t n = up256(tc_pack_bytes(oc, kh, kw, c));
    if (wants_padding(oc, c)) {
        b200k_conv2d_params t;
        memset(&t, 0, sizeof(t));
        t.oc = oc; t.kh = kh; t.kw = kw; t.c = c;
        n += pad_plan(&t).pack_total;
    }
    return n;
}

static b200k_conv2d_params grouped_params(const b200k_conv2d_params* p, const GroupPlan& pl)
{
    b200k_conv2d_params q = *p;
    uint8_t* region = (uint8_t*)p->packed + group_region_offset(p->oc, p->kh, p->kw, p->c);
    const long long M = (long long)p->n * p->h * p->wd;
    q.n = 1; q.h = 1; q.oh = 1; q.wd = (int)(M / pl.g); q.ow = q.wd;
    q.c = pl.cg; q.oc = pl.ocg;
    q.w.data = region + pl.w_off;
    if (p->w.scales) q.w.scales = (const float*)(region + pl.ws_off);
    if (p->bias.data) {
        q.bias.data = region + pl.bias_off;
        if (p->bias.scales) q.bias.scales = (const float*)(region + pl.bs_off);
    }
    q.packed = region + pl.inner_off;
    q.scratch = nullptr; q.scratch_bytes = 0;
    return q;
}

static bool grouped_path_eligible(const b200k_conv2d_params* p, b200k_conv2d_params& q)
{
    if (p->add_operand.data || !p->packed || !p->x.data || !p->w.data || !p->y.data) return false;
    if (p->kh != 1 || p->kw != 1 || p->stride_h != 1 || p->stride_w != 1 || p->dil_h != 1 || p->dil_w != 1) return false;
    if (p->pad_top != 0 || p->pad_left != 0 || p->oh != p->h || p->ow != p->wd) return false;
    if (p->n <= 0 || p->h <= 0 || p->wd <= 0) return false;
    const GroupPlan pl = group_plan(p->oc, p->kh, p->kw, p->c);
    const long long M = (long long)p->n * p->h * p->wd;
    if (!pl.ok || M % pl.g != 0 || M / pl.g > 0x7fffffff) return false;
    q = grouped_params(p, pl);
    return q.c > 16 && conv_tc_eligible(&q);
}

// wp[j oc + o][i c + ch] = w[o][ch] on the diagonal blocks (i == j), the weight zero point elsewhere
__global__ void group_weights_kernel(const uint8_t* w, uint8_t* wp, int oc, int c, int g, int fill)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int cg = g * c;
    if (i >= (long long)g * oc * cg) return;
    const int col = (int)(i % cg), row = (int)(i / cg);
    const int bj = row / oc, o = row - bj * oc, bi = col / c, ch = col - bi * c;
    wp[i] = bi == bj ? w[(long long)o * c + ch] : (uint8_t)fill;
}

__global__ void group_vec_kernel(const uint32_t* src, uint32_t* dst, int n, int g)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n * g) dst[i] = src[i % n];
}

int conv2d_dispatch(const b200k_conv2d_params* p, cudaStream_t stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "conv2d_q8: null params");
    B200K_REQUIRE(p->algo >= 0 && p->algo <= 2, B200K_E_INVALID, "conv2d_q8: algo %d not in {0,1,2}", p->algo);
    if (p->algo != 1) {
        b200k_conv2d_params q;
        // (group_plan only has a plan where groups of pixels beat what the kernel would do with the tensors as they are)
        if (grouped_path_eligible(p, q)) return launch_conv_tc(&q, stream, 0);
        if (conv_tc_eligible(p)) return launch_conv_tc(p, stream, 0);
        PadPlan pl;
        if (wants_padding(p->oc, p->c) && padded_path_eligible(p, pl, q)) return launch_padded(p, pl, q, stream);
        B200K_REQUIRE(p->algo != 2, B200K_E_UNSUPPORTED, "conv2d_q8: shape/alignment not eligible for the tcgen05 kernel");
    }
    return launch_conv_dp4a(p, stream);
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_conv2d_q8(const b200k_conv2d_params* p, void* stream)
{
    return conv2d_dispatch(p, (cudaStream_t)stream);
}

extern "C" size_t b200k_conv2d_pack_bytes(int32_t oc, int32_t kh, int32_t kw, int32_t c)
{
    if (oc <= 0 || kh <= 0 || kw <= 0) return 0;
    size_t n = group_region_offset(oc, kh, kw, c);
    const GroupPlan gp = group_plan(oc, kh, kw, c);
    if (gp.ok) n += gp.pack_total;
    return n;
}

extern "C" size_t b200k_conv2d_scratch_bytes(const b200k_conv2d_params* p)
{
    if (!p) return 0;
    if (p->c <= 16) return tc_scratch_bytes(p);
    if (wants_padding(p->oc, p->c) && !p->add_operand.data) return pad_plan(p).scratch_total;
    return 0;
}

namespace b200k {
// host_tables: also read a fused-Add layer's per-channel constants back (a stream synchronisation: load time only)
int conv2d_pack_impl(const b200k_conv2d_params* p, void* packed, cudaStream_t s, bool host_tables)
{
    B200K_REQUIRE(p && packed, B200K_E_INVALID, "conv2d_pack: null argument");
    int rc = tc_pack(p, packed, s);
    if (rc) return rc;
    if (host_tables) rc = tc_pack_host_tables(p, packed, s);
    if (rc) return rc;
    const GroupPlan gp = group_plan(p->oc, p->kh, p->kw, p->c);
    if (gp.ok) {
        // block-diagonal weights, g-fold bias and per-channel scales, and the tables of the grouped problem
        uint8_t* region = (uint8_t*)packed + group_region_offset(p->oc, p->kh, p->kw, p->c);
        group_weights_kernel<<<div_up((long long)gp.ocg * gp.cg, 256), 256, 0, s>>>(
            (const uint8_t*)p->w.data, region + gp.w_off, p->oc, p->c, gp.g, p->w.scales ? 0 : (p->w.zero_point & 0xff));
        rc = check_launch("group_weights_kernel");
        if (rc) return rc;
        if (p->bias.data)   group_vec_kernel<<<div_up(gp.ocg, 128), 128, 0, s>>>((const uint32_t*)p->bias.data, (uint32_t*)(region + gp.bias_off), p->oc, gp.g);
        if (p->w.scales)    group_vec_kernel<<<div_up(gp.ocg, 128), 128, 0, s>>>((const uint32_t*)p->w.scales, (uint32_t*)(region + gp.ws_off), p->oc, gp.g);
        if (p->bias.scales) group_vec_kernel<<<div_up(gp.ocg, 128), 128, 0, s>>>((const uint32_t*)p->bias.scales, (uint32_t*)(region + gp.bs_off), p->oc, gp.g);
        rc = check_launch("group_vec_kernel");
        if (rc) return rc;
        b200k_conv2d_params q = *p;
        q.c = gp.cg; q.oc = gp.ocg;
        q.w.data = region + gp.w_off;
        q.add_operand.data = nullptr; q.add_out.data = nullptr;
        rc = tc_pack(&q, region + gp.inner_off, s);
        if (rc) return rc;
    }
    if (!wants_padding(p->oc, p->c)) return rc;
    // zero-padded copies of the weights, the bias and the per-channel scales, and the tables of the padded problem
    const PadPlan pl = pad_plan(p);
    uint8_t* region = (uint8_t*)packed + up256(tc_pack_bytes(p->oc, p->kh, p->kw, p->c));
    const int taps = p->kh * p->kw;
    pad_weights_kernel<<<div_up((long long)pl.ocpad * taps * pl.cpad, 256), 256, 0, s>>>(
        (const uint8_t*)p->w.data, region + pl.w_off, p->oc, taps, p->c, pl.ocpad, pl.cpad);
    rc = check_launch("pad_weights_kernel");
    if (rc) return rc;
    const unsigned one = 0x3f800000u;                         // 1.0f: padded channels get a harmless scale
    if (p->bias.data)   pad_vec_kernel<<<div_up(pl.ocpad, 128), 128, 0, s>>>((const uint32_t*)p->bias.data, (uint32_t*)(region + pl.bias_off), p->oc, pl.ocpad, 0u);
    if (p->w.scales)    pad_vec_kernel<<<div_up(pl.ocpad, 128), 128, 0, s>>>((const uint32_t*)p->w.scales, (uint32_t*)(region + pl.ws_off), p->oc, pl.ocpad, one);
    if (p->bias.scales) pad_vec_kernel<<<div_up(pl.ocpad, 128), 128, 0, s>>>((const uint32_t*)p->bias.scales, (uint32_t*)(region + pl.bs_off), p->oc, pl.ocpad, one);
    rc = check_launch("pad_vec_kernel");
    if (rc) return rc;
    b200k_conv2d_params q = *p;
    q.c = pl.cpad; q.oc = pl.ocpad;
    q.w.data = region + pl.w_off;
    return tc_pack(&q, region + pl.inner_off, s);
}
}  // namespace b200k

extern "C" int b200k_conv2d_pack(const b200k_conv2d_params* p, void* packed, void* stream)
{
    return conv2d_pack_impl(p, packed, (cudaStream_t)stream, true);
}
