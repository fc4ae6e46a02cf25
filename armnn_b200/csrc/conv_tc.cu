// tcgen05 implicit-GEMM Convolution2d / FullyConnected for 8-bit quantised NHWC tensors (sm_100a).
//
// GEMM view: D[M, N] = A[M, K] * B[N, K]^T with M = output pixels (n, oy, ox), N = output channels and
// K = (ky, kx, c).  One CTA computes a 128 x BN tile of D:
//   * a producer thread feeds a multi-stage shared-memory ring with TMA.  The weight tile is a plain 2-D box of
//     the [OC, KH*KW*C] matrix.  The activation tile is fetched either as a 2-D box of [M, C] (1x1 stride-1
//     convolutions and FullyConnected) or with TMA's im2col mode straight from the NHWC tensor: one copy
//     delivers, for 128 consecutive output pixels, the channel slice of one filter tap, zero-filling taps that
//     fall outside the image.  Both land in the 128-byte (or 64-byte) swizzled K-major layout tcgen05 reads.
//   * one thread issues tcgen05.mma.kind::i8 (M = 128, N = BN, K = 32 per instruction); the int32 accumulator
//     lives in tensor memory (BN columns x 128 lanes); tcgen05.commit releases ring slots and finally signals
//     the epilogue.
//   * eight epilogue warps read the accumulator with tcgen05.ld, apply the zero-point correction, bias and the
//     fp32 requantisation, and store 8-bit outputs.
//
// Convolutions with very few input channels (the 3-channel network stems) cannot feed TMA directly: a pixel is
// not a 16-byte unit.  For those a pre-pass re-packs the input into caller-provided scratch as
// [N][Hp][Wp][8 or 16] with the spatial padding materialised (filled with the input zero point) and the channels
// padded, and the kernel runs in "row-window" mode: a tile is one output row, and the A operand of filter row ky is
// a tiled TMA box over an overlapping-window view of the packed rows (window = KW pixels = one 64- or 128-byte
// K-slice, window stride = stride_w pixels), so K = KH slices.  The weights are re-packed to match at load time.
//
// Zero points.  TMA fills out-of-image taps with raw zeros, whereas the reference pads with the real value 0,
// i.e. with the quantised value zx.  With symmetric weights (zw = 0)
//     sum_valid (x - zx) w = sum_all x_filled w - zx * sum_valid w
// and sum_valid w for an output pixel is the sum of per-tap channel sums over the rectangle of in-image taps,
// read from a 2-D prefix table over (ky, kx) that b200k_conv2d_pack builds once per weight tensor.
//
// Requantisation is the same function as in the CUDA-core kernel and the CPU oracle (IEEE fp32, unfused).  The
// division v / scale is evaluated as a multiplication by the reciprocal whenever the product is provably not
// within reach of a rounding tie, and falls back to the exact division otherwise, so results are bit-identical.
//
// Every wait on an mbarrier is bounded; when a bound is hit the kernel raises a status word (read with
// b200k_poll_status), drains and returns, so a logic error cannot hang the device.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>
#include <cudaTypedefs.h>
#include "common.cuh"

namespace b200k {

constexpr int TC_BM = 128;
constexpr int TC_EPI_WARPS = 16;
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS;   // warp 0 producer, warp 1 MMA issuer, then the epilogue warps
constexpr unsigned TC_SPIN_LIMIT = 1u << 22;

__device__ int g_tc_status = 0;                 // 0 ok, otherwise the code of the wait that gave up

struct TcArgs {
    const int32_t* bias; void* y; int32_t* acc_out;
    const float* w_scales; const float* b_scales;
    const int32_t* prefix;                      // [(KH+1)*(KW+1)][OC] or null
    float w_scale, b_scale;
    int zx;                                     // true input zero point
    int N, H, W, C, OH, OW, OC, KH, KW, sh, sw, pt, pl, dh, dw;
    long long M;
    int im2col;                                 // 0: A is a 2-D [M, C] matrix; 1: TMA im2col from NHWC; 2: row-window
    int tile_rows;                              // valid rows of an M-tile: 128, or OW in row-window mode
    int ntm;                                    // number of M-tiles
    int kstride;                                // bytes between consecutive taps in a weight row (C, or the window)
    uint32_t stage_tx;                          // bytes one ring stage receives
    int cchunks;                                // C / BK
    int nslices;                                // KH*KW*cchunks
    int need_corr;                              // zx != 0
    int need_rect;                              // need_corr and some tap can fall outside the image
    int a_signed, b_signed;                     // operand element types: 1 = int8, 0 = uint8
    Requant rq;                                 // the convolution's own output quantisation
    float inv_sy;
    // fused ElementwiseBinary Add (res != null): y = Q2(deq(Q(conv)) + deq(res)), clamp in rq2
    const uint8_t* res; float res_scale; int res_zp; int res_u8;
    Requant rq2;
    float inv_sy2;
    int stages;                                 // ring depth chosen by the launcher (<= 8)
    int prefix_ints;                            // ints of shared memory reserved for the prefix slice
    const uint8_t* add_lut;                     // [256][256] table of the fused Add (or null: evaluate arithmetically)
    int debug;                                  // 0 normal; 1: main loop without MMAs; 2: main loop without TMA loads
};

// ---- PTX wrappers --------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: returns false when the limit is hit.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity)
{
    const uint32_t addr = smem_u32(bar);
    for (unsigned i = 0; i < TC_SPIN_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.b32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_im2col(void* dst, const CUtensorMap* map, uint64_t* bar, int c, int w, int h,
                                                int n, uint16_t off_w, uint16_t off_h)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
                 ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n),
                   "h"(off_w), "h"(off_h) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32"
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32"
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
                 " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are one swizzle span (SWZ bytes) long:
// 8-row groups are 8 * SWZ bytes apart (stride byte offset); the leading byte offset is unused for swizzled
// K-major layouts; descriptor version 1; layout type 2 = 128-byte swizzle, 4 = 64-byte swizzle.
template <int SWZ>
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)((8 * SWZ) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(SWZ == 128 ? 2 : 4) << 61;
    return d;
}

// The epilogue arithmetic is written to stay off the conversion/transcendental (XU) pipe, which issues only 16 lanes
// per clock per SM and throttled the first version of this kernel: float <-> int conversions and rounding are done
// with the 1.5 * 2^23 magic constant on the FP32 pipe, and the only conversion instruction left is the int32 -> fp32
// of the accumulator.
constexpr float TC_MAGIC = 12582912.0f;          // 1.5 * 2^23: x + MAGIC - MAGIC == rint(x) for |x| < 2^22

struct QuantF {                                  // one quantisation target, everything as fp32
    float sy, inv_sy, zy, lo, hi;                // lo / hi: type range intersected with the activation clamp
};

// Quantize(v, sy, zy) then clamp, returned as an integer-valued float.  The division v / sy is evaluated as a
// multiplication by the reciprocal whenever that provably cannot change the rounded result: |v * inv - v / sy| is
// below 2^-12 for |v / sy| < 512 (beyond which every 8-bit output saturates whatever the rounding), so unless the
// product lies within 2^-11 of a rounding tie its nearest integer is round(v / sy).  Otherwise the exact division
// and round-half-away are evaluated, as armnn::Quantize does.
__device__ __forceinline__ float quantize_f32(float v, const QuantF& q)
{
    const float y = __fmul_rn(v, q.inv_sy);
    float n = __fsub_rn(__fadd_rn(y, TC_MAGIC), TC_MAGIC);
    const float e = fabsf(__fsub_rn(y, n)) - 0.5f;
    if (fabsf(e) <= 0.00048828125f) n = roundf(__fdiv_rn(v, q.sy));
    return fminf(fmaxf(__fadd_rn(q.zy, n), q.lo), q.hi);
}

// integer-valued float in [-128, 255] -> its low byte (two's complement)
__device__ __forceinline__ uint32_t f32_to_byte_bits(float qf) { return __float_as_uint(__fadd_rn(qf, TC_MAGIC)); }

// bytes of a packed word as integer-valued floats (signed or unsigned 8-bit)
__device__ __forceinline__ float byte_to_f32(uint32_t word, int idx, bool is_u8)
{
    // place the byte in the mantissa of 2^23 + 2^22: value = MAGIC + byte (after flipping the sign bit for int8)
    const uint32_t b = __byte_perm(word ^ (is_u8 ? 0u : 0x80808080u), 0x4B400000u, 0x7650 + idx);
    return __fsub_rn(__uint_as_float(b), is_u8 ? TC_MAGIC : TC_MAGIC + 128.0f);
}

struct EpiConsts {
    QuantF q1, q2;                               // the convolution's own quantisation; the fused Add's output
    float res_zp, res_scale; bool res_u8; int zx;
    const int32_t *p11, *p01, *p10, *p00;        // prefix-table rows of this thread's tap rectangle
    const uint8_t* lut;                          // shared-memory copy of the fused-add table, or null
};

// 16 accumulator columns of one output pixel -> 16 output bytes.  FUSED: add the residual operand (16 bytes in rv).
// INTERIOR: every tap of every pixel of the warp is inside the image, so the zero-point correction is the
// per-channel constant in s_corr; otherwise it comes from the pixel's tap rectangle in the prefix table.
template <bool FUSED, bool INTERIOR>
__device__ __forceinline__ uint4 epi_chunk(const uint32_t* r, const uint4 rv, const float* s_m, const float* s_bterm,
                                           const int32_t* s_corr, int col0, const EpiConsts& ec)
{
    const uint32_t resw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t packed[4];
    #pragma unroll
    for (int g = 0; g < 4; ++g) {                              // 4 columns at a time: 128-bit shared loads
        const float4 mv = *(const float4*)&s_m[g * 4];
        const float4 bv = *(const float4*)&s_bterm[g * 4];
        int4 cv;
        if (INTERIOR) {
            cv = *(const int4*)&s_corr[g * 4];
        } else {
            const int col = col0 + g * 4;
            const int4 c11 = *(const int4*)&ec.p11[col], c01 = *(const int4*)&ec.p01[col];
            const int4 c10 = *(const int4*)&ec.p10[col], c00 = *(const int4*)&ec.p00[col];
            cv.x = ec.zx * (c11.x - c01.x - c10.x + c00.x);
            cv.y = ec.zx * (c11.y - c01.y - c10.y + c00.y);
            cv.z = ec.zx * (c11.z - c01.z - c10.z + c00.z);
            cv.w = ec.zx * (c11.w - c01.w - c10.w + c00.w);
        }
        const float mm[4] = {mv.x, mv.y, mv.z, mv.w};
        const float bb[4] = {bv.x, bv.y, bv.z, bv.w};
        const int cc[4] = {cv.x, cv.y, cv.z, cv.w};
        uint32_t bits[4];
        #pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int acc = (int)r[g * 4 + e] - cc[e];
            // v = float(acc) * (sx * sw) + float(bias) * sb   (bterm is +0.0 without a bias)
            const float v = __fadd_rn(__fmul_rn(__int2float_rn(acc), mm[e]), bb[e]);
            float qf = quantize_f32(v, ec.q1);
            if (FUSED && ec.lut) {
                // The fused Add maps (convolution output byte, other operand byte) to the output byte; both operands
                // are per-tensor quantised, so the whole second quantisation is a 64 K-entry table built at load time
                // with the exact arithmetic of the branch below.
                const uint32_t idx = __byte_perm(f32_to_byte_bits(qf), resw[g], 0x0004 + e) & 0xffffu;   // (conv byte << 8) | other byte
                bits[e] = ec.lut[idx];
                continue;
            }
            if (FUSED) {
                // fused ElementwiseBinary Add: the convolution's own 8-bit output is formed first, then both operands
                // are dequantised, added in fp32 and re-quantised, as the two separate workloads do
                const float fa = __fmul_rn(__fsub_rn(qf, ec.q1.zy), ec.q1.sy);
                const float fb = __fmul_rn(__fsub_rn(byte_to_f32(resw[g], e, ec.res_u8), ec.res_zp), ec.res_scale);
                qf = quantize_f32(__fadd_rn(fa, fb), ec.q2);
            }
            bits[e] = f32_to_byte_bits(qf);
        }
        packed[g] = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
    }
    return make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

template <int BN, int SWZ>
struct TcSmem {
    static constexpr int A_BYTES = TC_BM * SWZ;
    static constexpr int B_BYTES = BN * SWZ;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int MAX_STAGES = 8;
    // after the ring (a.stages x STAGE_BYTES): float m[BN], float bterm[BN], int corr[BN], barriers (full[8], empty[8],
    // acc_full[2], acc_empty[2]), tmem slot; then the prefix slice and the fused-add table (dynamic sizes)
    static constexpr int CONST_BYTES = 3 * BN * 4 + (2 * MAX_STAGES + 4) * 8 + 16;
};

__device__ __forceinline__ void epi_barrier()       // the epilogue warps only (named barrier 1)
{
    asm volatile("bar.sync 1, %0;" ::"n"(32 * TC_EPI_WARPS) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Persistent kernel: one CTA per SM walks the tile list (n-tile fastest, so CTAs running at the same time share
// activation tiles in L2).  The shared-memory ring and its barriers run continuously across tiles, and the
// accumulator is double-buffered in tensor memory, so the TMA producer, the MMA issuer and the epilogue warps of
// consecutive tiles overlap.
template <int BN, int SWZ>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const TcArgs a)
{
    using L = TcSmem<BN, SWZ>;
    constexpr int MAX_STAGES = L::MAX_STAGES;
    const int STAGES = a.stages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float* s_m = (float*)(smem + (size_t)STAGES * L::STAGE_BYTES);
    float* s_bterm = s_m + BN;
    int32_t* s_corr = (int32_t*)(s_bterm + BN);             // zx * (sum of all taps) per channel
    uint64_t* full = (uint64_t*)(s_corr + BN);
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* acc_full = empty + MAX_STAGES;                // [2]
    uint64_t* acc_empty = acc_full + 2;                     // [2]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    int32_t* s_prefix = (int32_t*)(tmem_slot + 4);          // [(KH+1)*(KW+1)][BN] when need_rect
    uint8_t* s_lut = (uint8_t*)(s_prefix + a.prefix_ints);  // [256][256] fused-add table when a.add_lut

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ntn = a.OC / BN;                              // n-tiles (OC is a multiple of BN)
    const int ntiles = ntn * a.ntm;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], TC_EPI_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (a.add_lut) {
        const uint4* src = (const uint4*)a.add_lut;
        uint4* dst = (uint4*)s_lut;
        for (int i = threadIdx.x; i < 65536 / 16; i += TC_THREADS) dst[i] = src[i];
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (lane == 0) {
            uint32_t g = 0;                                  // slices issued so far (ring position)
            bool alive = true;
            for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
                const int n0 = (t % ntn) * BN;
                const long long m0 = (long long)(t / ntn) * a.tile_rows;
                int w0 = 0, h0 = 0, nimg = 0;
                if (a.im2col == 2) {
                    nimg = (int)((t / ntn) / a.OH);
                    h0 = (int)((t / ntn) % a.OH) * a.sh;          // first packed row of this output row
                } else if (a.im2col) {
                    const int ox = (int)(m0 % a.OW);
                    const long long q = m0 / a.OW;
                    const int oy = (int)(q % a.OH);
                    nimg = (int)(q / a.OH);
                    w0 = ox * a.sw - a.pl;
                    h0 = oy * a.sh - a.pt;
                }
                for (int s = 0; s < a.nslices; ++s, ++g) {
                    const int st = g % STAGES;
                    const uint32_t ph = (g / STAGES) & 1u;
                    if (!mbar_wait(&empty[st], ph ^ 1u)) { atomicExch(&g_tc_status, 1); alive = false; break; }
                    const int tap = s / a.cchunks;
                    const int c0 = (s - tap * a.cchunks) * SWZ;
                    uint8_t* sa = smem + st * L::STAGE_BYTES;
                    uint8_t* sb = sa + L::A_BYTES;
                    if (a.debug == 2) { mbar_arrive(&full[st]); continue; }
                    mbar_expect_tx(&full[st], a.stage_tx);
                    if (a.im2col == 2) {
                        tma_load_4d(sa, &tmA, &full[st], 0, 0, h0 + tap * a.dh, nimg);   // tap = filter row
                    } else if (a.im2col) {
                        const int ky = tap / a.KW, kx = tap - ky * a.KW;
                        tma_load_im2col(sa, &tmA, &full[st], c0, w0, h0, nimg, (uint16_t)(kx * a.dw), (uint16_t)(ky * a.dh));
                    } else {
                        tma_load_2d(sa, &tmA, &full[st], c0, (int)m0);
                    }
                    tma_load_2d(sb, &tmB, &full[st], tap * a.kstride + c0, n0);
                }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            // instruction descriptor: D = S32 (bits 4-5 = 2); A / B format at bits 7 / 10 (1 = signed 8-bit,
            // 0 = unsigned 8-bit); both operands K-major (bits 15, 16 = 0); N >> 3 at bit 17; M >> 4 at bit 24
            const uint32_t id = (2u << 4) | ((uint32_t)a.a_signed << 7) | ((uint32_t)a.b_signed << 10) |
                                ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            uint32_t g = 0;
            bool alive = true;
            int it = 0;
            for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x, ++it) {
                const int buf = it & 1;
                // the epilogue must have drained this accumulator buffer (two tiles ago)
                if (!mbar_wait(&acc_empty[buf], (((uint32_t)it >> 1) & 1u) ^ 1u)) { atomicExch(&g_tc_status, 4); break; }
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
                for (int s = 0; s < a.nslices; ++s, ++g) {
                    const int st = g % STAGES;
                    const uint32_t ph = (g / STAGES) & 1u;
                    if (!mbar_wait(&full[st], ph)) { atomicExch(&g_tc_status, 2); alive = false; break; }
                    tc_fence_after();
                    if (a.debug == 1) { mbar_arrive(&empty[st]); continue; }
                    const uint32_t sa = smem_u32(smem + st * L::STAGE_BYTES);
                    const uint64_t da = make_smem_desc<SWZ>(sa);
                    const uint64_t db = make_smem_desc<SWZ>(sa + L::A_BYTES);
                    #pragma unroll
                    for (int k = 0; k < SWZ / 32; ++k)
                        tc_mma_i8(tacc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), id, (s > 0 || k > 0) ? 1u : 0u);
                    tc_commit(&empty[st]);             // slot reusable once these MMAs have read it
                }
                if (alive) tc_commit(&acc_full[buf]);  // accumulator of this tile complete
            }
        }
    } else {
        // ===================== epilogue =====================
        // 16 warps: warp & 3 selects the TMEM lane quadrant (a hardware restriction), the other two bits select a
        // quarter of the tile's columns; each warp walks its columns in chunks of 16.
        const int ew = warp - 2;
        const int quad = warp & 3;
        const int part = ew >> 2;
        const int etid = threadIdx.x - 64;
        const int pw = a.KW + 1;
        const int cells = (a.KH + 1) * pw;
        constexpr int COLS_PER_PART = BN / 4;
        EpiConsts ec;
        ec.q1.sy = a.rq.sy; ec.q1.inv_sy = a.inv_sy; ec.q1.zy = (float)a.rq.zy;
        ec.q1.lo = fmaxf(a.rq.tlo, (float)a.rq.clo); ec.q1.hi = fminf(a.rq.thi, (float)a.rq.chi);
        ec.q2.sy = a.rq2.sy; ec.q2.inv_sy = a.inv_sy2; ec.q2.zy = (float)a.rq2.zy;
        ec.q2.lo = fmaxf(a.rq2.tlo, (float)a.rq2.clo); ec.q2.hi = fminf(a.rq2.thi, (float)a.rq2.chi);
        ec.res_zp = (float)a.res_zp; ec.res_scale = a.res_scale; ec.res_u8 = a.res_u8 != 0; ec.zx = a.zx;
        ec.lut = a.add_lut ? s_lut : nullptr;
        int cur_n0 = -1;
        int it = 0;
        for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
            const int n0 = (t % ntn) * BN;
            const long long m0 = (long long)(t / ntn) * a.tile_rows;
            const int buf = it & 1;
            if (n0 != cur_n0) {
                // per-channel constants of this n-tile (all epilogue warps are between tiles here)
                epi_barrier();
                for (int j = etid; j < BN; j += 32 * TC_EPI_WARPS) {
                    const int ch = n0 + j;
                    s_m[j] = __fmul_rn(a.rq.sx, a.w_scales ? a.w_scales[ch] : a.w_scale);
                    s_bterm[j] = a.bias ? __fmul_rn(__int2float_rn(a.bias[ch]), a.b_scales ? a.b_scales[ch] : a.b_scale) : 0.f;
                    s_corr[j] = a.need_corr ? a.zx * a.prefix[(long long)(cells - 1) * a.OC + ch] : 0;
                }
                if (a.need_rect) {
                    for (int i = etid; i < cells * BN; i += 32 * TC_EPI_WARPS) {
                        const int cell = i / BN, j = i - cell * BN;
                        s_prefix[i] = a.prefix[(long long)cell * a.OC + n0 + j];
                    }
                }
                epi_barrier();
                cur_n0 = n0;
            }
            const bool ok = mbar_wait(&acc_full[buf], ((uint32_t)it >> 1) & 1u);
            if (!ok) { atomicExch(&g_tc_status, 3); break; }
            tc_fence_after();
            const int row = quad * 32 + lane;
            const long long m = m0 + row;
            const bool mvalid = row < a.tile_rows && m < a.M;
            // rectangle of in-image taps of this pixel
            int ky0 = 0, ky1 = a.KH, kx0 = 0, kx1 = a.KW;
            if (a.need_rect) {
                const unsigned mu = (unsigned)m;               // M < 2^31
                const unsigned qd = mu / (unsigned)a.OW;
                const int ox = (int)(mu - qd * (unsigned)a.OW);
                const int oy = (int)(qd % (unsigned)a.OH);
                const int iy = oy * a.sh - a.pt, ix = ox * a.sw - a.pl;
                // first in-image tap, one past the last in-image tap
                ky0 = iy < 0 ? (-iy + a.dh - 1) / a.dh : 0;
                ky1 = iy >= a.H ? 0 : min(a.KH, (a.H - 1 - iy) / a.dh + 1);
                kx0 = ix < 0 ? (-ix + a.dw - 1) / a.dw : 0;
                kx1 = ix >= a.W ? 0 : min(a.KW, (a.W - 1 - ix) / a.dw + 1);
                ky0 = min(ky0, a.KH); kx0 = min(kx0, a.KW);
                ky1 = max(ky1, ky0);  kx1 = max(kx1, kx0);
            }
            const bool interior = ky0 == 0 && kx0 == 0 && ky1 == a.KH && kx1 == a.KW;
            const bool warp_interior = __all_sync(0xffffffffu, interior || !mvalid);
            ec.p11 = s_prefix + (ky1 * pw + kx1) * BN;
            ec.p01 = s_prefix + (ky0 * pw + kx1) * BN;
            ec.p10 = s_prefix + (ky1 * pw + kx0) * BN;
            ec.p00 = s_prefix + (ky0 * pw + kx0) * BN;
            const uint32_t tacc = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(quad * 32) << 16);
            #pragma unroll 1
            for (int cb = 0; cb < COLS_PER_PART; cb += 16) {
                const int col0 = part * COLS_PER_PART + cb;
                uint32_t r[16];
                tc_ld16(tacc + (uint32_t)col0, r);
                if (!mvalid) continue;
                const long long obase = m * a.OC + n0 + col0;
                if (a.acc_out) {                               // raw accumulators for the bit-exactness tests
                    for (int j = 0; j < 16; ++j) {
                        const int col = col0 + j;
                        const int c = warp_interior ? s_corr[col]
                                                    : ec.zx * (ec.p11[col] - ec.p01[col] - ec.p10[col] + ec.p00[col]);
                        a.acc_out[obase + j] = (int)r[j] - c;
                    }
                }
                uint4 outv;
                if (a.res) {
                    const uint4 rv = *(const uint4*)(a.res + obase);
                    if (warp_interior) outv = epi_chunk<true, true>(r, rv, s_m + col0, s_bterm + col0, s_corr + col0, col0, ec);
                    else               outv = epi_chunk<true, false>(r, rv, s_m + col0, s_bterm + col0, s_corr + col0, col0, ec);
                } else {
                    const uint4 rv = make_uint4(0, 0, 0, 0);
                    if (warp_interior) outv = epi_chunk<false, true>(r, rv, s_m + col0, s_bterm + col0, s_corr + col0, col0, ec);
                    else               outv = epi_chunk<false, false>(r, rv, s_m + col0, s_bterm + col0, s_corr + col0, col0, ec);
                }
                *(uint4*)((uint8_t*)a.y + obase) = outv;
            }
            // this warp has finished reading the accumulator buffer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2 * BN) : "memory");
    }
}

// ---- weight preparation: per-tap channel sums as a 2-D prefix table --------------------------------------------

struct PackArgs { const uint8_t* w; int32_t* prefix; int w_u8, OC, KH, KW, C; };

// prefix[(ky, kx)][oc] = sum over taps (y < ky, x < kx) and all channels of the raw weight value
__global__ void conv_prefix_kernel(const PackArgs a)
{
    const int oc = blockIdx.x * blockDim.x + threadIdx.x;
    if (oc >= a.OC) return;
    const int pw = a.KW + 1;
    for (int kx = 0; kx <= a.KW; ++kx) a.prefix[(long long)kx * a.OC + oc] = 0;
    for (int ky = 1; ky <= a.KH; ++ky) {
        a.prefix[(long long)(ky * pw) * a.OC + oc] = 0;
        int rowsum = 0;
        for (int kx = 1; kx <= a.KW; ++kx) {
            const uint8_t* wp = a.w + (((long long)oc * a.KH + (ky - 1)) * a.KW + (kx - 1)) * a.C;
            int s = 0;
            for (int c = 0; c < a.C; ++c) s += a.w_u8 ? (int)wp[c] : (int)(int8_t)wp[c];
            rowsum += s;
            a.prefix[(long long)(ky * pw + kx) * a.OC + oc] = a.prefix[(long long)((ky - 1) * pw + kx) * a.OC + oc] + rowsum;
        }
    }
}

// ---- row-window mode: plan, weight re-pack (load time) and input re-pack (every call) -------------------------

struct RowPlan {
    bool ok;
    int cpad;                 // channels per packed pixel (8 or 16 bytes)
    int swz;                  // window bytes = K-slice = swizzle span (64 or 128)
    int hp, wp;               // packed rows / pixels per row (spatial padding materialised)
    size_t scratch_bytes;     // packed input
    size_t wpack_offset;      // offset of the re-packed weights inside `packed`
};

static RowPlan row_window_plan(const b200k_conv2d_params* p)
{
    RowPlan r;
    memset(&r, 0, sizeof(r));
    if (p->c > 16 || p->c < 1 || p->dil_w != 1 || p->ow > TC_BM || p->oc % 64 != 0 || p->kh > 15 || p->kw > 15) return r;
    if (p->w.zero_point != 0 || p->stride_w > 8 || p->stride_h > 8) return r;
    r.cpad = (p->c <= 8 && (p->stride_w * 8) % 16 == 0) ? 8 : 16;
    const int window = p->kw * r.cpad;
    if (window > 128) return r;
    r.swz = window <= 64 ? 64 : 128;
    r.hp = (p->oh - 1) * p->stride_h + (p->kh - 1) * p->dil_h + 1;
    r.wp = (p->ow - 1) * p->stride_w + r.swz / r.cpad;
    if ((r.wp * r.cpad) % 16 != 0) r.wp += 1;
    r.scratch_bytes = (size_t)p->n * r.hp * r.wp * r.cpad;
    r.wpack_offset = (size_t)(p->kh + 1) * (p->kw + 1) * p->oc * sizeof(int32_t);
    r.ok = true;
    return r;
}

struct RowWeightArgs { const uint8_t* w; uint8_t* wp; int OC, KH, KW, C, cpad, swz; };

// wp[oc][ky][kx * cpad + c] = w[oc][ky][kx][c]; every other byte of the swz-wide window is 0
__global__ void row_weight_pack_kernel(const RowWeightArgs a)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.OC * a.KH * a.swz) return;
    const int b = i % a.swz;
    const int ky = (i / a.swz) % a.KH;
    const int oc = i / (a.swz * a.KH);
    const int kx = b / a.cpad, c = b - kx * a.cpad;
    uint8_t v = 0;
    if (kx < a.KW && c < a.C) v = a.w[(((long long)oc * a.KH + ky) * a.KW + kx) * a.C + c];
    a.wp[i] = v;
}

struct RowInputArgs { const uint8_t* x; uint8_t* xp; int N, H, W, C, hp, wp, cpad, pt, pl; unsigned fill; long long total; };

// xp[n][yp][xq][0..cpad) = x[n][yp - pt][xq - pl][0..C) inside the image, the input zero point everywhere else
template <int CPAD>
__global__ void __launch_bounds__(256) row_input_pack_kernel(const RowInputArgs a)
{
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    const int xq = (int)(i % a.wp);
    const long long t = i / a.wp;
    const int yp = (int)(t % a.hp);
    const int n = (int)(t / a.hp);
    const int iy = yp - a.pt, ix = xq - a.pl;
    uint8_t v[CPAD];
    #pragma unroll
    for (int c = 0; c < CPAD; ++c) v[c] = (uint8_t)a.fill;
    if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W) {
        const uint8_t* src = a.x + (((long long)n * a.H + iy) * a.W + ix) * a.C;
        #pragma unroll
        for (int c = 0; c < CPAD; ++c)
            if (c < a.C) v[c] = src[c];
    }
    if (CPAD == 8) *(uint2*)(a.xp + i * 8) = *(const uint2*)v;
    else           *(uint4*)(a.xp + i * 16) = *(const uint4*)v;
}

// ---- fused-add table ---------------------------------------------------------------------------------------------

struct AddLutArgs { uint8_t* lut; int y_u8, res_u8; float sy; int zy; float sr; int zr; Requant out; };

// lut[(conv byte << 8) | other byte] = clamp(Q_out(deq_y(conv) + deq(other))): RefElementwiseBinaryWorkload(Add)
// followed by the fused activation, evaluated once per pair of 8-bit values with the exact fp32 arithmetic
__global__ void add_lut_kernel(const AddLutArgs a)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;       // 65536 threads
    const int b1 = i >> 8, b2 = i & 255;
    const int q1 = a.y_u8 ? b1 : (int)(int8_t)b1;
    const int q2 = a.res_u8 ? b2 : (int)(int8_t)b2;
    const float fa = __fmul_rn(__int2float_rn(q1 - a.zy), a.sy);
    const float fb = __fmul_rn(__int2float_rn(q2 - a.zr), a.sr);
    const int q = quantize_dev(__fadd_rn(fa, fb), a.out.sy, a.out.zy, a.out.tlo, a.out.thi);
    a.lut[i] = (uint8_t)min(max(q, a.out.clo), a.out.chi);
}

static size_t add_lut_offset(int oc, int kh, int kw, int c)
{
    size_t n = (size_t)(kh + 1) * (kw + 1) * oc * sizeof(int32_t);
    if (c <= 16) n += (size_t)oc * kh * 128;
    return (n + 255) & ~(size_t)255;
}

// ---- host side ---------------------------------------------------------------------------------------------------

static PFN_cuTensorMapEncodeTiled_v12000 g_encode_tiled = nullptr;
static PFN_cuTensorMapEncodeIm2col_v12000 g_encode_im2col = nullptr;

static bool load_driver_entry_points()
{
    if (g_encode_tiled && g_encode_im2col) return true;
    cudaDriverEntryPointQueryResult q;
    void* f = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || !f) return false;
    g_encode_tiled = (PFN_cuTensorMapEncodeTiled_v12000)f;
    f = nullptr;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeIm2col", &f, cudaEnableDefault, &q) != cudaSuccess || !f) return false;
    g_encode_im2col = (PFN_cuTensorMapEncodeIm2col_v12000)f;
    return true;
}

static int pick_bn(int oc) { return (oc % 256 == 0) ? 256 : (oc % 128 == 0) ? 128 : 64; }

static bool row_window_eligible(const b200k_conv2d_params* p)
{
    const RowPlan r = row_window_plan(p);
    if (!r.ok || !p->packed || !p->scratch || p->scratch_bytes < r.scratch_bytes) return false;
    const void* outp = p->add_operand.data ? p->add_out.data : p->y.data;
    if (!p->x.data || !p->w.data || !outp) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->w.dtype) || !is_q8(p->y.dtype)) return false;
    if ((((uintptr_t)p->scratch | (uintptr_t)p->packed | (uintptr_t)outp) & 15) != 0) return false;
    if (p->add_operand.data && ((((uintptr_t)p->add_operand.data) & 15) != 0)) return false;
    if ((long long)p->n * p->oh > (1ll << 30) || (long long)p->n * p->oh * p->ow > (1ll << 31) - TC_BM) return false;
    return true;
}

bool conv_tc_eligible(const b200k_conv2d_params* p)
{
    if (p->c <= 16) return row_window_eligible(p);
    const void* outp = p->add_operand.data ? p->add_out.data : p->y.data;
    if (!p->x.data || !p->w.data || !outp) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->w.dtype) || !is_q8(p->y.dtype)) return false;
    if (p->add_operand.data && ((((uintptr_t)p->add_operand.data | (uintptr_t)p->add_out.data) & 15) != 0)) return false;
    if (p->c % 64 != 0 || p->oc % 64 != 0) return false;
    if (p->w.zero_point != 0) return false;                              // symmetric weights only on this path
    if ((((uintptr_t)p->x.data | (uintptr_t)p->w.data | (uintptr_t)outp) & 15) != 0) return false;
    if (p->x.zero_point != 0 && !p->packed) return false;              // needs the prefix table
    if (p->kh > 15 || p->kw > 15) return false;
    if (p->kh * p->dil_h > 255 || p->kw * p->dil_w > 255) return false;
    if (p->stride_h > 8 || p->stride_w > 8) return false;
    const long long M = (long long)p->n * p->oh * p->ow;
    if (M > (1ll << 31) - TC_BM) return false;
    const bool gemm = p->kh == 1 && p->kw == 1 && p->stride_h == 1 && p->stride_w == 1 && p->pad_top == 0 &&
                      p->pad_left == 0 && p->oh == p->h && p->ow == p->wd;
    if (!gemm) {
        // im2col corners must fit the descriptor's signed 8-bit fields
        const int up_w = (p->ow - 1) * p->stride_w + 1 - p->pad_left - p->wd;
        const int up_h = (p->oh - 1) * p->stride_h + 1 - p->pad_top - p->h;
        if (p->pad_left > 127 || p->pad_top > 127 || up_w < -128 || up_w > 127 || up_h < -128 || up_h > 127) return false;
    }
    const int bn = pick_bn(p->oc);
    const size_t prefix_bytes = p->x.zero_point != 0 ? (size_t)(p->kh + 1) * (p->kw + 1) * bn * 4 : 0;
    if (prefix_bytes > 48 * 1024) return false;
    return true;
}

static int sm_count()
{
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int SWZ>
static int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, const TcArgs& a, size_t prefix_bytes, cudaStream_t stream)
{
    using L = TcSmem<BN, SWZ>;
    const size_t lut_bytes = a.add_lut ? 65536 : 0;
    const size_t budget = 227 * 1024;                                   // opt-in shared memory per CTA on sm_100
    const size_t rest = 1024 + L::CONST_BYTES + prefix_bytes + lut_bytes;
    int stages = (int)((budget - rest) / L::STAGE_BYTES);
    if (stages > L::MAX_STAGES) stages = L::MAX_STAGES;
    B200K_REQUIRE(stages >= 2, B200K_E_TOOBIG, "conv2d_q8: shared memory exhausted (%zu bytes of tables)", rest);
    TcArgs a2 = a;
    a2.stages = stages;
    a2.prefix_ints = (int)(prefix_bytes / 4);
    const size_t smem = rest + (size_t)stages * L::STAGE_BYTES;
    auto kern = conv_tc_kernel<BN, SWZ>;
    static size_t configured = 0;                      // per instantiation: largest dynamic smem size set so far
    if (smem > configured) {
        B200K_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        configured = smem;
    }
    const long long tiles = (long long)(a.OC / BN) * a.ntm;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kern<<<grid, TC_THREADS, smem, stream>>>(tmA, tmB, a2);
    return check_launch("conv_tc_kernel");
}

int launch_conv_tc(const b200k_conv2d_params* p, cudaStream_t stream)
{
    B200K_REQUIRE(conv_tc_eligible(p), B200K_E_UNSUPPORTED, "conv2d_q8: not eligible for the tcgen05 kernel");
    B200K_REQUIRE(load_driver_entry_points(), B200K_E_CUDA, "conv2d_q8: cuTensorMapEncode* not available from the driver");
    TcArgs a;
    a.bias = (const int32_t*)p->bias.data; a.acc_out = p->acc_out;
    a.w_scales = p->w.scales; a.b_scales = p->bias.scales; a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.prefix = (const int32_t*)p->packed;
    a.zx = p->x.zero_point;
    a.N = p->n; a.H = p->h; a.W = p->wd; a.C = p->c; a.OH = p->oh; a.OW = p->ow; a.OC = p->oc;
    a.KH = p->kh; a.KW = p->kw; a.sh = p->stride_h; a.sw = p->stride_w; a.pt = p->pad_top; a.pl = p->pad_left;
    a.dh = p->dil_h; a.dw = p->dil_w;
    a.M = (long long)p->n * p->oh * p->ow;
    const RowPlan rowp = p->c <= 16 ? row_window_plan(p) : RowPlan{};
    const bool row_mode = rowp.ok;
    const bool gemm = !row_mode && p->kh == 1 && p->kw == 1 && p->stride_h == 1 && p->stride_w == 1 && p->pad_top == 0 &&
                      p->pad_left == 0 && p->oh == p->h && p->ow == p->wd;
    a.im2col = row_mode ? 2 : gemm ? 0 : 1;
    const int swz = row_mode ? rowp.swz : (p->c % 128 == 0) ? 128 : 64;
    a.cchunks = row_mode ? 1 : p->c / swz;
    a.nslices = row_mode ? p->kh : p->kh * p->kw * a.cchunks;
    a.tile_rows = row_mode ? p->ow : TC_BM;
    a.ntm = row_mode ? p->n * p->oh : (int)((a.M + TC_BM - 1) / TC_BM);
    a.kstride = row_mode ? swz : p->c;
    a.need_corr = a.zx != 0;
    // can any tap of any output pixel leave the image?
    const int last_y = (p->oh - 1) * p->stride_h - p->pad_top + (p->kh - 1) * p->dil_h;
    const int last_x = (p->ow - 1) * p->stride_w - p->pad_left + (p->kw - 1) * p->dil_w;
    // (row-window mode materialises the padding with the zero point itself: no tap is ever "outside")
    const int rect = (!row_mode && a.need_corr && (p->pad_top > 0 || p->pad_left > 0 || last_y >= p->h || last_x >= p->wd)) ? 1 : 0;
    a.need_rect = rect;
    a.a_signed = p->x.dtype == B200K_S8;
    a.b_signed = p->w.dtype == B200K_S8;
    FusedAdd fa;
    B200K_REQUIRE(make_fused_add(p, a.rq, fa, a.y), B200K_E_INVALID, "conv2d_q8: malformed fused add operand / output");
    a.inv_sy = 1.0f / p->y.scale;
    a.res = fa.res; a.res_scale = fa.res_scale; a.res_zp = fa.res_zp; a.res_u8 = fa.res_u8;
    a.rq2 = fa.out;
    a.inv_sy2 = fa.res ? 1.0f / p->add_out.scale : 0.f;
    // b200k_conv2d_pack builds the fused-add table when it is given the add operand: callers pass the same struct
    a.add_lut = (fa.res && p->packed) ? (const uint8_t*)p->packed + add_lut_offset(p->oc, p->kh, p->kw, p->c) : nullptr;
    // Measurement aid (results are wrong in modes 1 and 2): isolates the TMA side or the MMA side of the main loop.
    static const int debug_mode = getenv("B200K_TC_DEBUG") ? atoi(getenv("B200K_TC_DEBUG")) : 0;
    a.debug = debug_mode;

    const int bn = pick_bn(p->oc);
    CUtensorMap tmA, tmB;
    const CUtensorMapSwizzle swizzle = swz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
    a.stage_tx = (uint32_t)((a.tile_rows + bn) * swz);
    {   // weights: 2-D [OC][K] matrix, box = swz bytes x bn rows (row-window mode: the re-packed [OC][KH * swz] copy)
        const cuuint64_t K = row_mode ? (cuuint64_t)p->kh * swz : (cuuint64_t)p->kh * p->kw * p->c;
        const void* wptr = row_mode ? (const void*)((const uint8_t*)p->packed + rowp.wpack_offset) : p->w.data;
        cuuint64_t dims[2] = {K, (cuuint64_t)p->oc};
        cuuint64_t strides[1] = {K};
        cuuint32_t box[2] = {(cuuint32_t)swz, (cuuint32_t)bn};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = g_encode_tiled(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)wptr, dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        B200K_REQUIRE(r == CUDA_SUCCESS, B200K_E_CUDA, "conv2d_q8: cuTensorMapEncodeTiled(weights) failed with %d", (int)r);
    }
    if (row_mode) {
        // re-pack the input into the caller's scratch, then view it as overlapping windows: dim0 = the window's bytes,
        // dim1 = output column (stride = stride_w pixels), dim2 = packed row, dim3 = image
        RowInputArgs ra;
        ra.x = (const uint8_t*)p->x.data; ra.xp = (uint8_t*)p->scratch;
        ra.N = p->n; ra.H = p->h; ra.W = p->wd; ra.C = p->c; ra.hp = rowp.hp; ra.wp = rowp.wp; ra.cpad = rowp.cpad;
        ra.pt = p->pad_top; ra.pl = p->pad_left; ra.fill = (unsigned)(p->x.zero_point & 0xff);
        ra.total = (long long)p->n * rowp.hp * rowp.wp;
        if (rowp.cpad == 8) row_input_pack_kernel<8><<<div_up(ra.total, 256), 256, 0, stream>>>(ra);
        else                row_input_pack_kernel<16><<<div_up(ra.total, 256), 256, 0, stream>>>(ra);
        int rc = check_launch("row_input_pack_kernel");
        if (rc) return rc;
        const cuuint64_t rowb = (cuuint64_t)rowp.wp * rowp.cpad;
        cuuint64_t dims[4] = {(cuuint64_t)swz, (cuuint64_t)p->ow, (cuuint64_t)rowp.hp, (cuuint64_t)p->n};
        cuuint64_t strides[3] = {(cuuint64_t)p->stride_w * rowp.cpad, rowb, rowb * rowp.hp};
        cuuint32_t box[4] = {(cuuint32_t)swz, (cuuint32_t)p->ow, 1, 1};
        cuuint32_t estr[4] = {1, 1, 1, 1};
        CUresult r = g_encode_tiled(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, p->scratch, dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        B200K_REQUIRE(r == CUDA_SUCCESS, B200K_E_CUDA, "conv2d_q8: cuTensorMapEncodeTiled(row windows) failed with %d", (int)r);
    } else if (gemm) {
        cuuint64_t dims[2] = {(cuuint64_t)p->c, (cuuint64_t)a.M};
        cuuint64_t strides[1] = {(cuuint64_t)p->c};
        cuuint32_t box[2] = {(cuuint32_t)swz, (cuuint32_t)TC_BM};
        cuuint32_t estr[2] = {1, 1};
        CUresult r = g_encode_tiled(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void*)p->x.data, dims, strides, box, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        B200K_REQUIRE(r == CUDA_SUCCESS, B200K_E_CUDA, "conv2d_q8: cuTensorMapEncodeTiled(input) failed with %d", (int)r);
    } else {
        cuuint64_t dims[4] = {(cuuint64_t)p->c, (cuuint64_t)p->wd, (cuuint64_t)p->h, (cuuint64_t)p->n};
        cuuint64_t strides[3] = {(cuuint64_t)p->c, (cuuint64_t)p->wd * p->c, (cuuint64_t)p->h * p->wd * p->c};
        int lower[2] = {-p->pad_left, -p->pad_top};
        int upper[2] = {(p->ow - 1) * p->stride_w + 1 - p->pad_left - p->wd, (p->oh - 1) * p->stride_h + 1 - p->pad_top - p->h};
        cuuint32_t estr[4] = {1, (cuuint32_t)p->stride_w, (cuuint32_t)p->stride_h, 1};
        CUresult r = g_encode_im2col(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, (void*)p->x.data, dims, strides, lower, upper,
                                     (cuuint32_t)swz, (cuuint32_t)TC_BM, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                                     CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        B200K_REQUIRE(r == CUDA_SUCCESS, B200K_E_CUDA, "conv2d_q8: cuTensorMapEncodeIm2col failed with %d", (int)r);
        // Drivers up to 13.1 mis-encode im2col maps of tensors smaller than 128 KiB; the open-source CUTLASS
        // im2col copy traits clear bit 21 of the second descriptor word in that case, and so does this.
        int drv = 0;
        if (cudaDriverGetVersion(&drv) == cudaSuccess && drv <= 13010 &&
            (size_t)p->n * p->h * p->wd * p->c < 131072)
            reinterpret_cast<uint64_t*>(&tmA)[1] &= ~(1ull << 21);
    }
    const size_t prefix_bytes = a.need_rect ? (size_t)(p->kh + 1) * (p->kw + 1) * bn * 4 : 0;
    if (swz == 128) {
        if (bn == 256) return launch_tc<256, 128>(tmA, tmB, a, prefix_bytes, stream);
        if (bn == 128) return launch_tc<128, 128>(tmA, tmB, a, prefix_bytes, stream);
        return launch_tc<64, 128>(tmA, tmB, a, prefix_bytes, stream);
    }
    if (bn == 256) return launch_tc<256, 64>(tmA, tmB, a, prefix_bytes, stream);
    if (bn == 128) return launch_tc<128, 64>(tmA, tmB, a, prefix_bytes, stream);
    return launch_tc<64, 64>(tmA, tmB, a, prefix_bytes, stream);
}

}  // namespace b200k

using namespace b200k;

extern "C" size_t b200k_conv2d_pack_bytes(int32_t oc, int32_t kh, int32_t kw, int32_t c)
{
    if (oc <= 0 || kh <= 0 || kw <= 0) return 0;
    // prefix table, row-window weights for few-channel convolutions (widest window), fused-add table
    return add_lut_offset(oc, kh, kw, c) + 65536;
}

extern "C" size_t b200k_conv2d_scratch_bytes(const b200k_conv2d_params* p)
{
    if (!p || p->c > 16) return 0;
    const RowPlan r = row_window_plan(p);
    return r.ok ? r.scratch_bytes : 0;
}

extern "C" int b200k_conv2d_pack(const b200k_conv2d_params* p, void* packed, void* stream)
{
    B200K_REQUIRE(p && packed, B200K_E_INVALID, "conv2d_pack: null argument");
    B200K_REQUIRE(p->w.data && is_q8(p->w.dtype), B200K_E_INVALID, "conv2d_pack: weights must be an 8-bit device tensor");
    B200K_REQUIRE(p->oc > 0 && p->kh > 0 && p->kw > 0 && p->c > 0, B200K_E_INVALID, "conv2d_pack: bad geometry");
    PackArgs a;
    a.w = (const uint8_t*)p->w.data; a.prefix = (int32_t*)packed; a.w_u8 = p->w.dtype == B200K_U8;
    a.OC = p->oc; a.KH = p->kh; a.KW = p->kw; a.C = p->c;
    conv_prefix_kernel<<<div_up(p->oc, 128), 128, 0, (cudaStream_t)stream>>>(a);
    int rc = check_launch("conv_prefix_kernel");
    if (rc) return rc;
    if (p->add_operand.data && is_q8(p->add_operand.dtype) && is_q8(p->add_out.dtype) && is_q8(p->y.dtype)) {
        // table of the fused Add for exactly these quantisation parameters and this clamp
        AddLutArgs la;
        la.lut = (uint8_t*)packed + add_lut_offset(p->oc, p->kh, p->kw, p->c);
        la.y_u8 = p->y.dtype == B200K_U8; la.res_u8 = p->add_operand.dtype == B200K_U8;
        la.sy = p->y.scale; la.zy = p->y.zero_point; la.sr = p->add_operand.scale; la.zr = p->add_operand.zero_point;
        la.out = make_requant(0.f, p->add_out, p->clamp_lo, p->clamp_hi);
        add_lut_kernel<<<256, 256, 0, (cudaStream_t)stream>>>(la);
        rc = check_launch("add_lut_kernel");
        if (rc) return rc;
    }
    if (p->c > 16) return rc;
    // weights of a few-channel convolution, re-packed for the row-window mode (needs kw, c and stride_w)
    b200k_conv2d_params q = *p;
    if (q.stride_w <= 0) q.stride_w = 1;
    if (q.stride_h <= 0) q.stride_h = 1;
    if (q.dil_w <= 0) q.dil_w = 1;
    if (q.dil_h <= 0) q.dil_h = 1;
    if (q.ow <= 0) q.ow = 1;
    if (q.oh <= 0) q.oh = 1;
    if (q.n <= 0) q.n = 1;
    const RowPlan r = row_window_plan(&q);
    if (!r.ok) return B200K_OK;
    RowWeightArgs wa;
    wa.w = (const uint8_t*)p->w.data; wa.wp = (uint8_t*)packed + r.wpack_offset;
    wa.OC = p->oc; wa.KH = p->kh; wa.KW = p->kw; wa.C = p->c; wa.cpad = r.cpad; wa.swz = r.swz;
    row_weight_pack_kernel<<<div_up((long long)p->oc * p->kh * r.swz, 256), 256, 0, (cudaStream_t)stream>>>(wa);
    return check_launch("row_weight_pack_kernel");
}

extern "C" int b200k_poll_status(void)
{
    int s = 0;
    B200K_CUDA(cudaMemcpyFromSymbol(&s, g_tc_status, sizeof(int)));
    if (s != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
        set_error("a bounded device-side wait gave up (code %d: 1 producer, 2 MMA issuer, 3 epilogue)", s);
        return B200K_E_TIMEOUT;
    }
    return B200K_OK;
}
