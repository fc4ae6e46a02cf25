// tcgen05 implicit-GEMM Convolution2d / FullyConnected for 8-bit quantised NHWC tensors (sm_100a).
//
// GEMM view: D[M, N] = A[M, K] * B[N, K]^T with M = output pixels (n, oy, ox), N = output channels and
// K = (ky, kx, c).  One CTA computes a 128 x BN tile of D:
//   * two producer warps (one elected lane each, taking turns by stage) feed a shared-memory ring with TMA; a ring
//     stage holds one to eight K-slices behind one pair of barriers.  The weight tile is a plain 2-D box of
//     the [OC, KH*KW*C] matrix.  The activation tile is fetched either as a 2-D box of [M, C] (1x1 stride-1
//     convolutions and FullyConnected) or with TMA's im2col mode straight from the NHWC tensor: one copy
//     delivers, for 128 consecutive output pixels, the channel slice of one filter tap, zero-filling taps that
//     fall outside the image.  Both land in the 128-byte (or 64-byte) swizzled K-major layout tcgen05 reads.
//   * one elected lane of the issuer warp issues tcgen05.mma.kind::i8 (M = 128, N = BN, K = 32 per instruction);
//     the int32 accumulators live in tensor memory (2 to 8 buffers of BN columns x 128 lanes); tcgen05.commit
//     releases ring stages and finally signals the epilogue.
//   * sixteen epilogue warps, in one, two or four groups that work on different tiles, read an accumulator with
//     tcgen05.ld, apply the zero-point correction, bias and the fp32 requantisation (and a fused residual Add), and
//     send their 8-bit outputs with their own TMA stores.
//   The producer and issuer roles are warp-uniform code (every lane runs the loops, elect.sync guards the issuing
//   instructions), because TMA, MMA and mbarrier instructions take uniform-register operands.
//
// Convolutions with very few input channels (the 3-channel network stems) cannot feed TMA directly: a pixel is
// not a 16-byte unit.  For those a pre-pass re-packs the input into caller-provided scratch as
// [N][Hp][Wp][8 or 16] with the spatial padding materialised (filled with the input zero point) and the channels
// padded, and the kernel runs in "row-window" mode: a tile is one output row, and the A operand of filter row ky is
// a tiled TMA box over an overlapping-window view of the packed rows (window = KW pixels = one 64- or 128-byte
// K-slice, window stride = stride_w pixels), so K = KH slices.  The weights are re-packed to match at load time.
//
// Zero points.  TMA fills out-of-image taps with raw zeros, whereas the reference pads with the real value 0,
// i.e. with the quantised value zx:
//     sum_valid (x - zx)(w - zw) = sum_all x_filled w - zw sum_all x_filled - zx sum_valid w + K_valid zx zw.
// sum_valid w of an output pixel is the sum of per-tap channel sums over the rectangle of in-image taps, read from a
// 2-D prefix table over (ky, kx) that b200k_conv2d_pack builds once per weight tensor; pixels with the same rectangle
// form a class, and the last two terms are a per-class, per-channel constant kept in shared memory.  The second term
// (per-tensor asymmetric weights) is accumulated by the tensor core itself from constant B tiles holding -zw.
//
// Requantisation is the same function as in the CUDA-core kernel and the CPU oracle (IEEE fp32, unfused), evaluated
// without the division unit and bit-identically (see epi_chunk_fast and epi_fix_group).
//
// Every wait on an mbarrier is bounded; when a bound is hit the kernel raises a status word (read with
// b200k_poll_status), drains and returns, so a logic error cannot hang the device.
#include <cuda.h>
#include <stdlib.h>
#include <atomic>
#include <string.h>
#include <cudaTypedefs.h>
#include <type_traits>
#include <memory>
#include <mutex>
#include <unordered_map>
#include <vector>
#include "common.cuh"

namespace b200k {

constexpr int TC_BM = 128;
constexpr int TC_EPI_WARPS = 16;
constexpr int TC_LUT_TAG_WORDS = 12;
// Fused-add table: 256 rows (convolution value) of 256 entries (other operand's byte), rows 260 bytes apart so that
// the shared-memory bank of an entry depends on both indices: the other operand of a residual block is full of
// repeated values (half of a ReLU output is the zero point), and with a 256-byte pitch lanes that share it would all
// hit one bank.
constexpr int TC_LUT_PITCH = 260;
constexpr int TC_LUT_BYTES = 256 * TC_LUT_PITCH;
// The K-slices are dealt round-robin to TC_PRODUCERS producer warps.  Issuing a load (wait for the slot, arm its
// barrier, issue) is a chain of dependent shared-memory operations in one thread; for narrow tiles, whose MMAs are short,
// one producer cannot keep up (stem and 3 x 3 layers with 64 channels ran 25 % slower with one producer than with
// two), while four cost the epilogue-bound layers more issue slots than they gain elsewhere.
#ifndef B200K_TC_PRODUCERS
#define B200K_TC_PRODUCERS 2
#endif
constexpr int TC_PRODUCERS = B200K_TC_PRODUCERS;     // 1, 2 or 4
// warp 0: producer 0; warp 1: MMA issuer; then the epilogue warps; then producers 1 .. TC_PRODUCERS - 1
constexpr int TC_THREADS = 64 + 32 * TC_EPI_WARPS + 32 * (TC_PRODUCERS - 1);

constexpr long long TC_WAIT_LIMIT_CYCLES = 4000000000ll;  // about two seconds: no wait of a healthy launch comes near

__device__ int g_tc_status = 0;                 // 0 ok, otherwise the code of the wait that gave up

// Phase time stamps of CTA 0 (nanoseconds, %globaltimer), compiled in only with -DB200K_TRACE, which the build never sets.
#ifdef B200K_TRACE
__device__ unsigned long long g_tc_trace[64];
__device__ __forceinline__ void tc_trace(int i)
{
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        g_tc_trace[i] = t;
    }
}
#define TC_TRACE(i) tc_trace(i)
#else
#define TC_TRACE(i) do { } while (0)
#endif

// Constants of the hot path, filled in by the host: they sit in the kernel's parameter space, so the packed
// instructions read them as constant-bank operands and they take no registers.  Each is the same value twice.
struct EpiConsts {
    float2 inv2, nsy2, magic2, zero2, neg2;      // RN(1 / sy), -sy, MAGIC, 0, -1
    float2 nmagic2;                              // -MAGIC
    float2 zoff_lut2, zoff_sat2, zoff_clamp2;    // what is added to t = MAGIC + n (see epi_fix_group), per way of ending
    float lo, hi;                                // EPI_CLAMP: clamp bounds in the biased domain (MAGIC + ...)
};

struct TcArgs {
    const int32_t* bias; void* y; int32_t* acc_out;
    const float* w_scales; const float* b_scales;
    const int32_t* prefix;                      // [(KH+1)*(KW+1)][OC] or null
    float w_scale, b_scale;
    int zx;                                     // true input zero point
    int zw;                                     // weight zero point (per-tensor asymmetric weights), 0 otherwise
    int nzw;                                    // zw != 0: constant B tiles (1 or 2) that add -zw x (row sum of A) to every column
    int zw_val[2];                              // their int8 values, which add up to -zw
    int mask_cpad, mask_kw;                     // row-window mode: which bytes of a K-slice are real taps (for the row sums)
    int ntn;                                    // n-tiles: ceil(OC / BN); columns beyond OC are padding
    int kvalid_c;                               // real input channels per tap (C, or fewer when the caller zero-padded them)
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
    // fused ElementwiseBinary Add (res != null): y = Q2(deq(Q(conv)) + deq(res)), clamp in rq2
    const uint8_t* res; float res_scale; int res_zp; int res_u8;
    Requant rq2;
    float inv_sy;                               // RN(1 / rq.sy), correctly rounded (see epi_fix_group)
    EpiConsts ep;                               // the hot path's constants
    const uint8_t* add_lut;                     // fused-add table built by b200k_conv2d_pack (+ its tag), or null
    uint32_t lut_tag[TC_LUT_TAG_WORDS];         // the tag a table made for exactly this launch carries
    int stages;                                 // ring depth chosen by the launcher (<= 16)
    int nprod;                                  // producer threads that take turns: 1, 2 or 4, never more than stages
    int group;                                  // K-slices per ring stage: they share the stage's pair of barriers
    int eg;                                     // epilogue groups (1, 2 or 4): group g takes the tiles with index = g mod eg
    int bstat;                                  // weights stay in shared memory for the whole launch (one n-tile, small K)
    int nio;                                    // shared buffers for units of the fused Add's other operand: 0, 2 or 3
    int nstg;                                   // staging buffers per epilogue warp: 1 or 2
    // zero-point correction classes: pixels whose in-image tap rectangle [ky0, ky1) x [kx0, kx1) is the same share
    // one row of per-channel corrections.  ypair / xpair list the distinct (k0 << 4 | k1) of the geometry, ycls / xcls
    // map such a code back to its position in the list.
    int ncy, ncx, ncls;
    int acc_big;                                // |accumulator| or |accumulator - correction| can reach 2^24 (see epi_chunk_fast)
    float thr_host;                             // parameter-space tables: 0.5 - E as the host computed it
    uint8_t ypair[16], xpair[16];
    uint8_t ycls[256], xcls[256];
    long long wait_limit;                       // clock64 ticks after which a device-side wait gives up
    int skip_loads;                             // fault-injection self-test: the producers issue no loads (see b200k_conv2d_params.selftest_us)
};

// ---- PTX wrappers --------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// One lane of a converged warp.  The single-thread roles are written as warp-uniform code, in which only the issuing
// instructions themselves are restricted to the elected lane: TMA, MMA and mbarrier instructions take their operands from
// uniform registers, and inside a branch on the lane index every operand would have to be moved there one by one, which
// made each issue cost 100 - 170 cycles.
__device__ __forceinline__ bool elect_one()
{
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "elect.sync _|p, 0xffffffff;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait: returns false when the time limit is hit.  try_wait suspends the thread until the phase completes or
// a hardware time limit expires, so a waiting thread polls rarely; the clock is read once per 32 polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, long long limit)
{
    const uint32_t addr = smem_u32(bar);
    long long t0 = 0;
    for (;;) {
        #pragma unroll 1
        for (int i = 0; i < 32; ++i) {
            uint32_t ok;
            asm volatile("{\n\t.reg .pred p;\n\t"
                         "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                         "selp.b32 %0, 1, 0, p;\n\t}"
                         : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
            if (ok) return true;
        }
        const long long now = clock64();
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit) return false;
    }
}
// The single-thread roles (TMA producer, MMA issuer) run one dependent instruction chain per K-slice; everything in
// that chain is latency.  They test a barrier once inline by shared address and only fall into the bounded polling
// loop when it is not ready yet.
__device__ __forceinline__ bool mbar_test(uint32_t bar_saddr, uint32_t parity)
{
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.b32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar_saddr), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar_saddr, uint32_t parity, long long limit)
{
    long long t0 = 0;
    for (;;) {
        #pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (mbar_test(bar_saddr, parity)) return true;
        const long long now = clock64();
        if (t0 == 0) t0 = now;
        else if (now - t0 > limit) return false;
    }
}
__device__ __forceinline__ bool mbar_wait_fast(uint32_t bar_saddr, uint32_t parity, long long limit)
{
    return mbar_test(bar_saddr, parity) || mbar_wait_slow(bar_saddr, parity, limit);
}
// For waits whose owner is ahead of the work by construction (a producer that finds the ring full, the MMA issuer
// that finds no free accumulator buffer: the epilogue is the bottleneck then): sleep between polls, so that the
// waiting warp leaves its scheduler's issue slots to the epilogue warps it shares the scheduler with.
__device__ __forceinline__ bool mbar_wait_idle(uint32_t bar_saddr, uint32_t parity, long long limit)
{
    if (mbar_test(bar_saddr, parity) || mbar_test(bar_saddr, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        __nanosleep(200);
        if (mbar_test(bar_saddr, parity)) return true;
        if (clock64() - t0 > limit) return false;
    }
}
__device__ __forceinline__ void tma_load_2d_s(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_4d_s(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_im2col_s(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c, int w, int h,
                                                  int n, uint16_t off_w, uint16_t off_h)
{
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};"
                 ::"r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c), "r"(w), "r"(h), "r"(n), "h"(off_w), "h"(off_h) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_s(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_s(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_commit_s(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_i8_acc(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc)   // D += A B
{
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.eq.b32 p, 0, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
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
// The same load split in two, so that several can be in flight: the registers must not be touched between issue and
// wait, which the wait enforces by claiming to modify them.
__device__ __forceinline__ void tc_ld16_issue(uint32_t taddr, uint32_t* r)
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32"
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr));
}
__device__ __forceinline__ void tc_ld16_wait(uint32_t* r)
{
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                   "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
                 :: "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src_saddr, int c0, int c1, int c2)
{
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"((uint64_t)map), "r"(src_saddr), "r"(c0), "r"(c1), "r"(c2) : "memory");
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
// with the 1.5 * 2^23 magic constant on the FP32 pipe, and the only conversion instructions left are the int32 -> fp32
// of the accumulator and one saturating float -> byte conversion.
constexpr float TC_MAGIC = 12582912.0f;          // 1.5 * 2^23: x + MAGIC - MAGIC == rint(x) for |x| < 2^22

// Reference arithmetic of one output value (unfused IEEE fp32), used by the rare fix-up pass:
// v = fl(fl(acc * m) + b); q = clamp(zy + round_half_away(fl(v / sy))), then for a fused Add both operands are
// dequantised, added and re-quantised (RefElementwiseBinaryWorkload), followed by the activation clamp.
struct EpiExact {
    float sy1, zy1, lo1, hi1;                    // the convolution's own quantisation (plain clamp bounds)
    int fused, res_u8;
    float zr, sr, sy2, zy2, lo2, hi2;
    int always;                                  // no usable fused-add table: every value takes this arithmetic
};

__device__ __forceinline__ int exact_value(int acc, float m, float b, uint32_t res_byte, const EpiExact& x)
{
    const float v = __fadd_rn(__fmul_rn(__int2float_rn(acc), m), b);
    float n = __fadd_rn(x.zy1, roundf(__fdiv_rn(v, x.sy1)));
    n = fminf(fmaxf(n, x.lo1), x.hi1);
    if (x.fused) {
        const int rq = x.res_u8 ? (int)res_byte : (int)(int8_t)res_byte;
        const float fa = __fmul_rn(__fsub_rn(n, x.zy1), x.sy1);
        const float fb = __fmul_rn(__fsub_rn(__int2float_rn(rq), x.zr), x.sr);
        n = __fadd_rn(x.zy2, roundf(__fdiv_rn(__fadd_rn(fa, fb), x.sy2)));
        n = fminf(fmaxf(n, x.lo2), x.hi2);
    }
    return __float2int_rn(n);
}

// shared-memory accesses by 32-bit shared address (keeps them out of the generic address space)
__device__ __forceinline__ uint4 lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t addr)
{
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ int lds_s32(uint32_t addr)
{
    int v;
    asm volatile("ld.shared.s32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u8(uint32_t addr)
{
    uint32_t v;
    asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}

// What the last step of the hot path is: look the fused Add up in its table, convert with the output type's own
// saturation (the clamp is exactly the type's range), or clamp to a narrower activation range.
enum { EPI_LUT = 0, EPI_SAT_U8 = 1, EPI_SAT_S8 = 2, EPI_CLAMP = 3 };

__device__ __forceinline__ void lds_f2x2(uint32_t addr, float2& a, float2& b)   // four consecutive floats as two pairs
{
    asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(a.x), "=f"(a.y), "=f"(b.x), "=f"(b.y) : "r"(addr));
}

// The reference chain of one output value is
//     v = fl(fl(acc * m) + b);  q = fl(v / sy);  n = round_half_away(q);  out = clamp(zy + n)
// with m = sx * sw, b = bias * sb per channel and acc the accumulator minus the zero-point correction cc (followed, for a
// fused Add, by the re-quantisation that the table holds).  The fp32 arithmetic below runs two values per instruction
// (__ffma2_rn and friends: one issue slot for two IEEE round-to-nearest operations).

// ---- the hot path: one fused multiply-add per value, and a proof that its rounding is the reference's -----------
//
// The reference chain (above) is three roundings away from the real number R = ((acc - cc) m + b) / sy.  The hot path
// evaluates q" = fma(float(acc), mq, bq) with mq = RN(m / sy) and bq = (b - cc m) / sy + zoff (zoff = the output zero
// point, for the table also minus the type minimum) prepared per n-tile to within one rounding, so that
//     |reference q + zoff - q"| <= E = 1.5 * 2^-24 * (4 Rmax + 3 RZmax + 2 max|b / sy| + 4 max|bq| + |zoff|)
// for every value that can round to something inside the output range (Rmax, RZmax: the largest |R| and |R + zoff| that
// do).  t = q" + MAGIC rounds q" to an integer n; whenever |q" - n| < 0.5 - E the reference's q lies on the same side of
// every rounding boundary, so n is the reference's result and the halves-away-from-zero rule cannot matter.  A group of
// four values in which some lane sees |q" - n| >= 0.5 - E (about one group in twenty) is re-evaluated with the
// reference arithmetic itself (epi_fix_group).  Values whose q" is huge lose the integer grid of the magic constant:
// either they are flagged like the others or they saturate, as the reference's do.
// Where mq and bq come from.  TabFast: tables in shared memory, read with 128-bit loads that every lane of the warp
// repeats (all lanes work on the same columns; bq: this lane's class row): four wavefronts of the shared-memory pipe per
// four outputs and table.  TabFastP: tables in the kernel's parameter space (constant bank): the column index is the
// same for the whole warp, so the loads are uniform loads that do not touch the shared-memory pipe at all, which is
// what bounds the fused-Add epilogue (its table lookups live there too).  Only launches whose tables the host can
// compute (see HostPack) and that have a single class of pixels take that form.
struct TabFast {
    uint32_t mq, bq;
    __device__ __forceinline__ void load(int g, float2& m01, float2& m23, float2& b01, float2& b23) const
    {
        lds_f2x2(mq + g * 16, m01, m23);
        lds_f2x2(bq + g * 16, b01, b23);
    }
};
struct TabFastP {
    const float* mq; const float* bq;
    __device__ __forceinline__ void load(int g, float2& m01, float2& m23, float2& b01, float2& b23) const
    {
        m01 = make_float2(mq[g * 4 + 0], mq[g * 4 + 1]); m23 = make_float2(mq[g * 4 + 2], mq[g * 4 + 3]);
        b01 = make_float2(bq[g * 4 + 0], bq[g * 4 + 1]); b23 = make_float2(bq[g * 4 + 2], bq[g * 4 + 3]);
    }
};
constexpr int TC_PTAB_MAX = 2048;               // output channels whose tables fit the parameter space (16 KiB of the 32 KiB)
struct TcTabs { float mq[TC_PTAB_MAX]; float bq[TC_PTAB_MAX]; };
struct TcNoTabs { int unused; };

template <int KIND, class Tab>
__device__ __forceinline__ uint4 epi_chunk_fast(const uint32_t* r, const uint4 rv, const Tab& ad, const EpiConsts& ec, const uint32_t lut,
                                                float* dmg)
{
    const uint32_t resw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t packed[4];
    #pragma unroll
    for (int g = 0; g < 4; ++g) {
        float2 m01, m23, b01, b23;
        ad.load(g, m01, m23, b01, b23);
        const float2 a01 = make_float2(__int2float_rn((int)r[g * 4 + 0]), __int2float_rn((int)r[g * 4 + 1]));
        const float2 a23 = make_float2(__int2float_rn((int)r[g * 4 + 2]), __int2float_rn((int)r[g * 4 + 3]));
        const float2 q01 = __ffma2_rn(a01, m01, b01), q23 = __ffma2_rn(a23, m23, b23);
        const float2 t01 = __fadd2_rn(q01, ec.magic2), t23 = __fadd2_rn(q23, ec.magic2);
        const float2 n01 = __fadd2_rn(t01, ec.nmagic2), n23 = __fadd2_rn(t23, ec.nmagic2);       // rint(q") (exact)
        const float2 d01 = __ffma2_rn(n01, ec.neg2, q01), d23 = __ffma2_rn(n23, ec.neg2, q23);   // q" - n (exact)
        dmg[g] = fmaxf(fmaxf(fabsf(d01.x), fabsf(d01.y)), fmaxf(fabsf(d23.x), fabsf(d23.y)));
        const float z[4] = {n01.x, n01.y, n23.x, n23.y};
        if (KIND == EPI_CLAMP) {
            // clamp in the biased domain: the low byte of the bit pattern is the output byte
            const float tt[4] = {t01.x, t01.y, t23.x, t23.y};
            uint32_t bits[4];
            #pragma unroll
            for (int e = 0; e < 4; ++e) bits[e] = __float_as_uint(fminf(fmaxf(tt[e], ec.lo), ec.hi));
            packed[g] = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
        } else if (KIND == EPI_LUT) {
            uint32_t bits[4];
            #pragma unroll
            for (int e = 0; e < 4; ++e) {
                asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(bits[e]) : "f"(z[e]));
                // entry (conv output - type minimum) * pitch + other byte; lut holds the table's address, a multiple of
                // 256, and the other operand's byte goes into its low 8 bits
                bits[e] = lds_u8(bits[e] * (uint32_t)TC_LUT_PITCH + __byte_perm(resw[g], lut, 0x7650 + e));
            }
            packed[g] = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
        } else {
            // the clamp is the 8-bit type's own range: integer conversion, then two saturating packs
            int i0, i1, i2, i3;
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(i0) : "f"(z[0]));
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(i1) : "f"(z[1]));
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(i2) : "f"(z[2]));
            asm("cvt.rni.s32.f32 %0, %1;" : "=r"(i3) : "f"(z[3]));
            uint32_t hi16;
            if (KIND == EPI_SAT_S8) {
                asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi16) : "r"(i3), "r"(i2), "r"(0));
                asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(packed[g]) : "r"(i1), "r"(i0), "r"(hi16));
            } else {
                asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi16) : "r"(i3), "r"(i2), "r"(0));
                asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(packed[g]) : "r"(i1), "r"(i0), "r"(hi16));
            }
        }
    }
    return make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

// Four values the hot path could not vouch for: the reference chain itself.  The division is evaluated exactly without
// the division unit: with y = RN(1 / sy) (prepared on the host), p = fl(v * y), r = fma(-p, sy, v) (exact) and
// q = fma(r, y, p), q is the correctly rounded quotient (Markstein's theorem; it needs a correctly rounded y and a
// normal-range quotient; for tiny or huge quotients the last bit does not matter, they round to 0 or saturate).
// t = q + MAGIC rounds to an integer, halves to even where the reference rounds them away from zero: |q - n| = 0.5
// exactly marks those values (and any value too large for the constant), and only they go on to the plain reference
// arithmetic (exact_value).  Kept out of line: it runs for a few per cent of the groups and would otherwise be inlined
// sixteen times into every tile loop.
template <int KIND>
__device__ __noinline__ uint32_t epi_fix_group(int a0, int a1, int a2, int a3, uint32_t a_m, uint32_t a_b, uint32_t a_cc, uint32_t resw,
                                               const EpiConsts* ecp, uint32_t lut, const EpiExact* x)
{
    const EpiConsts& ec = *ecp;
    const float2 zoff2 = KIND == EPI_LUT ? ec.zoff_lut2 : (KIND == EPI_CLAMP ? ec.zoff_clamp2 : ec.zoff_sat2);
    float2 m01, m23, b01, b23;
    lds_f2x2(a_m, m01, m23);
    lds_f2x2(a_b, b01, b23);
    const uint4 cv = lds128(a_cc);
    const int acc[4] = {a0 - (int)cv.x, a1 - (int)cv.y, a2 - (int)cv.z, a3 - (int)cv.w};
    const float2 a01 = make_float2(__int2float_rn(acc[0]), __int2float_rn(acc[1]));
    const float2 a23 = make_float2(__int2float_rn(acc[2]), __int2float_rn(acc[3]));
    const float2 v01 = __fadd2_rn(__ffma2_rn(a01, m01, ec.zero2), b01), v23 = __fadd2_rn(__ffma2_rn(a23, m23, ec.zero2), b23);
    const float2 p01 = __ffma2_rn(v01, ec.inv2, ec.zero2), p23 = __ffma2_rn(v23, ec.inv2, ec.zero2);
    const float2 q01 = __ffma2_rn(__ffma2_rn(p01, ec.nsy2, v01), ec.inv2, p01), q23 = __ffma2_rn(__ffma2_rn(p23, ec.nsy2, v23), ec.inv2, p23);
    const float2 t01 = __fadd2_rn(q01, ec.magic2), t23 = __fadd2_rn(q23, ec.magic2);
    const float2 n01 = __fadd2_rn(t01, ec.nmagic2), n23 = __fadd2_rn(t23, ec.nmagic2);
    const float2 d01 = __ffma2_rn(n01, ec.neg2, q01), d23 = __ffma2_rn(n23, ec.neg2, q23);
    const float dmax = fmaxf(fmaxf(fabsf(d01.x), fabsf(d01.y)), fmaxf(fabsf(d23.x), fabsf(d23.y)));
    const float2 z01 = __fadd2_rn(t01, zoff2), z23 = __fadd2_rn(t23, zoff2);
    const float z[4] = {z01.x, z01.y, z23.x, z23.y};
    uint32_t bits[4];
    #pragma unroll
    for (int e = 0; e < 4; ++e) {
        if (KIND == EPI_CLAMP) {
            bits[e] = __float_as_uint(fminf(fmaxf(z[e], ec.lo), ec.hi));
        } else {
            if (KIND == EPI_SAT_S8) asm("cvt.rni.sat.s8.f32 %0, %1;" : "=r"(bits[e]) : "f"(z[e]));
            else                    asm("cvt.rni.sat.u8.f32 %0, %1;" : "=r"(bits[e]) : "f"(z[e]));
            if (KIND == EPI_LUT) bits[e] = lds_u8(bits[e] * (uint32_t)TC_LUT_PITCH + __byte_perm(resw, lut, 0x7650 + e));
        }
    }
    uint32_t out = __byte_perm(__byte_perm(bits[0], bits[1], 0x0040), __byte_perm(bits[2], bits[3], 0x0040), 0x5410);
    if (!(dmax < 0.5f) || x->always) {
        // (no usable table, an exact half, or a value too large for the constant)
        out = 0;
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int q = exact_value(acc[j], lds_f32(a_m + j * 4), lds_f32(a_b + j * 4), (resw >> (8 * j)) & 0xffu, *x);
            out |= ((uint32_t)q & 0xffu) << (8 * j);
        }
    }
    return out;
}

// The cold pass of one chunk (rare, or the accumulator dump of the tests): from the 16 accumulators still in
// registers, (fix) evaluate them with the reference arithmetic (other operand's bytes at res_slot, result to out_slot)
// and / or (acc_row) write the raw accumulators of a valid row out for the bit-exactness tests.
__device__ __forceinline__ void epi_cold(const uint32_t* r, uint32_t res_slot, uint32_t out_slot, uint32_t a_m, uint32_t a_b,
                                         uint32_t a_cc, const EpiExact& x, bool fix, int32_t* acc_row)
{
    if (acc_row) {
        #pragma unroll
        for (int j = 0; j < 16; ++j) acc_row[j] = (int)r[j] - lds_s32(a_cc + j * 4);
    }
    if (!fix) return;
    const uint4 rv = x.fused ? lds128(res_slot) : make_uint4(0, 0, 0, 0);
    const uint32_t resw[4] = {rv.x, rv.y, rv.z, rv.w};
    uint32_t out[4] = {0, 0, 0, 0};
    #pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int q = exact_value((int)r[j] - lds_s32(a_cc + j * 4), lds_f32(a_m + j * 4), lds_f32(a_b + j * 4),
                                  (resw[j >> 2] >> (8 * (j & 3))) & 0xffu, x);
        out[j >> 2] |= ((uint32_t)q & 0xffu) << (8 * (j & 3));
    }
    sts128(out_slot, make_uint4(out[0], out[1], out[2], out[3]));
}

template <int BN, int SWZ>
struct TcSmem {
    static constexpr int A_BYTES = TC_BM * SWZ;
    static constexpr int B_BYTES = BN * SWZ;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int MAX_STAGES = 16;
    static constexpr int UW = BN < 128 ? BN : 128;          // width of one output unit: bytes = columns
    static constexpr int UNITS = BN / UW;                   // units per tile
    static constexpr int IO_BYTES = TC_BM * UW;             // one unit buffer: [128 rows][UW], TMA-swizzled
    static constexpr int MAX_IO = 3;
    // after the ring (stages x group x STAGE_BYTES), the staging buffers (EG x IO_BYTES) and the unit buffers
    // (nio x IO_BYTES): per-channel m, bterm [BN each], barriers (full[16], empty[16], acc_full[8], acc_empty[8],
    // io_full[3], io_empty[3], w_full, lut_full), tmem slot + table-valid slot; then the zero-point correction table
    // [classes][BN], the fused-add table and the K-slice coordinate table (dynamic sizes)
    static constexpr int MAX_ACC = 8;
    static constexpr int CONST_BYTES = 2 * BN * 4 + (2 * MAX_STAGES + 2 * MAX_ACC + 2 * MAX_IO + 2) * 8 + 16;
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
// activation tiles in L2).  The shared-memory ring and its barriers run continuously across tiles, and there are
// 2 * EG accumulator buffers in tensor memory, so the TMA producers, the MMA issuer and the epilogue warps of
// consecutive tiles overlap.
//
// Output path.  A tile leaves in units of 128 rows x UW (<= 128) columns; each epilogue warp owns 32 rows x
// EG * UW / 4 columns of a unit of its group's tile (EG = 1: all sixteen warps on one tile).  It writes its bytes into a private shared-memory buffer laid out as the TMA swizzle expects
// (conflict-free 16-byte stores, one row per lane) and one of its lanes sends the buffer with a TMA store, which clips
// rows beyond the tensor; before the buffer is written again that lane has waited for the store to have read it.  No
// epilogue warp waits for another one.  With a fused Add the producer TMA-loads the other operand's unit into one of
// two shared buffers; every epilogue warp releases it after reading its part.
template <int BN, int SWZ, int EG, bool PTAB>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmY, const __grid_constant__ CUtensorMap tmR,
               const __grid_constant__ TcArgs a, const __grid_constant__ std::conditional_t<PTAB, TcTabs, TcNoTabs> tabs)
{
    using L = TcSmem<BN, SWZ>;
    constexpr int MAX_STAGES = L::MAX_STAGES;
    constexpr int UW = L::UW, UNITS = L::UNITS, IO_BYTES = L::IO_BYTES;
    constexpr int NACC_LOG2 = EG == 1 ? 1 : (EG == 2 ? 2 : 3);          // 2, 4 or 8 accumulator buffers in TMEM
    static_assert(EG == 1 || EG * BN <= 256, "epilogue groups: at most 256 / BN tiles at once");
    const int STAGES = a.stages;
    const int NIO = a.nio;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // Asymmetric weights: sum x (w - zw) = sum x w + sum x (-zw).  The second sum comes from one or two more MMAs per
    // K-slice against constant B tiles (every entry -zw, split in two int8 values when zw > 128) at the very start of
    // shared memory, so the accumulator already holds it and the epilogue is unchanged.
    uint8_t* s_zw = smem;
    uint8_t* s_wst = smem + (size_t)a.nzw * L::B_BYTES;
    // weight-stationary launches: all K-slices of the (only) weight tile first, then a ring of activation tiles only
    const int stage_stride = a.bstat ? L::A_BYTES : L::STAGE_BYTES;
    uint8_t* ring = s_wst + (a.bstat ? (size_t)a.nslices * L::B_BYTES : 0);
    uint8_t* s_io = ring + (size_t)STAGES * a.group * stage_stride;
    float* s_m = (float*)(s_io + (size_t)(a.nstg * EG + NIO) * IO_BYTES);   // first the warps' staging buffers (nstg * eg units' worth), then NIO operand units
    float* s_bterm = s_m + BN;
    uint64_t* full = (uint64_t*)(s_bterm + BN);
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* acc_full = empty + MAX_STAGES;                // [8]
    uint64_t* acc_empty = acc_full + L::MAX_ACC;            // [8]
    uint64_t* io_full = acc_empty + L::MAX_ACC;             // [3] other operand's unit has landed
    uint64_t* io_empty = io_full + L::MAX_IO;               // [3] the unit buffer's last store has been read out
    uint64_t* w_full = io_empty + L::MAX_IO;                // the stationary weight tile has landed
    uint64_t* lut_full = w_full + 1;                        // the fused-add table has landed
    uint32_t* tmem_slot = (uint32_t*)(w_full + 2);
    uint32_t* s_lut_ok = tmem_slot + 1;                     // the fused-add table in global memory carries our tag
    int32_t* s_cc = (int32_t*)(tmem_slot + 4);              // [classes][BN] zero-point corrections
    float* s_mq = (float*)(s_cc + a.ncls * BN);             // [BN] hot-path multiplier m / sy
    float* s_bq = s_mq + BN;                                // [classes][BN] hot-path addend (see epi_chunk_fast)
    uint32_t* s_emax = (uint32_t*)(s_bq + a.ncls * BN);     // [2][2] max |bq|, max |b / sy| of a staging (bit patterns), double-buffered
    EpiExact* s_ex = (EpiExact*)(s_emax + 4);               // the reference arithmetic's constants (epi_fix_group)
    uint8_t* s_lut = (uint8_t*)(((uintptr_t)(s_emax + 4 + 16) + 255) & ~(uintptr_t)255);   // fused-add table, 256-byte aligned
    // per K-slice: {channel offset, im2col offsets (x | y << 16), weight column, packed-row offset}: the producers read
    // their coordinates from here instead of carrying tap counters through every slice
    uint4* s_tab = (uint4*)(s_lut + (a.add_lut ? TC_LUT_BYTES : 0));

    if (threadIdx.x == 0) TC_TRACE(0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");     // the next kernel of the stream may begin its set-up
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;   // warp: provably uniform
    const int ntn = a.ntn;                                  // n-tiles; the last one may reach beyond OC (zero weights, clipped stores)
    const int ntiles = ntn * a.ntm;

    {
        // the barriers lie in one array (full, empty, acc_full, acc_empty, io_full, io_empty, w_full, lut_full): one
        // thread each, instead of one thread for all 58 of them
        constexpr int NBAR = 2 * MAX_STAGES + 2 * L::MAX_ACC + 2 * L::MAX_IO + 2;
        const int i = threadIdx.x;
        if (i < NBAR) {
            const bool acc_e = i >= 2 * MAX_STAGES + L::MAX_ACC && i < 2 * MAX_STAGES + 2 * L::MAX_ACC;
            const bool io_e = i >= 2 * MAX_STAGES + 2 * L::MAX_ACC + L::MAX_IO && i < 2 * MAX_STAGES + 2 * L::MAX_ACC + 2 * L::MAX_IO;
            mbar_init(&full[i], acc_e ? TC_EPI_WARPS / EG : (io_e ? TC_EPI_WARPS : 1));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BN << NACC_LOG2) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (a.nzw) {
        // BN identical logical rows (in row-window mode: zero on the bytes of a slice that are no real taps), each stored
        // with the swizzle of its own row index
        for (int i = threadIdx.x; i < a.nzw * BN * SWZ; i += TC_THREADS) {
            const int z = i / (BN * SWZ), j = i - z * (BN * SWZ);
            const int row = j / SWZ, k = j - row * SWZ;
            const bool real = a.mask_cpad == 0 || ((k / a.mask_cpad) < a.mask_kw && (k % a.mask_cpad) < a.C);
            const int sw = SWZ == 128 ? (row & 7) : ((row >> 1) & 3);
            s_zw[z * L::B_BYTES + row * SWZ + ((((k >> 4) ^ sw) << 4) | (k & 15))] = real ? (uint8_t)(int8_t)a.zw_val[z] : (uint8_t)0;
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x < 4) s_emax[threadIdx.x] = 0u;
    for (int i = threadIdx.x; i < a.nslices; i += TC_THREADS) {
        const int tap = i / a.cchunks, c0 = (i - tap * a.cchunks) * SWZ;
        const int ky = a.im2col == 2 ? tap : tap / a.KW, kx = a.im2col == 2 ? 0 : tap - ky * a.KW;
        s_tab[i] = make_uint4((uint32_t)c0, (uint32_t)(kx * a.dw) | ((uint32_t)(ky * a.dh) << 16), (uint32_t)(tap * a.kstride + c0),
                              (uint32_t)(ky * a.dh));
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) TC_TRACE(1);

    const int prod = warp == 0 ? 0 : (warp >= 2 + TC_EPI_WARPS ? warp - (1 + TC_EPI_WARPS) : -1);
    if (prod >= 0) {
        // ===================== TMA producers =====================
        // The ring is filled stage by stage (a stage = `group` consecutive K-slices of one tile); the stages are dealt
        // round-robin to the active producers, which all walk the same sequence of tiles and stages.  Producer 0 also
        // loads the stationary weights and the fused Add's operand.  Producers beyond nprod (short rings) never get a
        // turn.  Everything a producer does per stage that is not its own is a handful of uniform instructions: these
        // are single chains of dependent instructions, whose latency (not throughput) is what a stage costs.
        {
            uint32_t turn = 0;                               // global stage counter modulo the number of active producers
            const uint32_t turn_mask = (uint32_t)a.nprod - 1u;
            const int group = a.group, gpt = a.nslices / a.group;          // slices per stage, stages per tile
            int st = 0; uint32_t ph = 0;                     // ring position: stage and its phase bit
            int ub = 0; uint32_t uph = 0;                    // unit-buffer position (kept without divisions)
            bool alive = true;
            const uint32_t ring_addr = smem_u32(ring), full_addr = smem_u32(full), empty_addr = smem_u32(empty);
            const uint32_t tab_addr = smem_u32(s_tab);
            const int mode = a.im2col;
            const bool bstat = a.bstat != 0, skip_loads = a.skip_loads != 0;
            const long long wait_limit = a.wait_limit;
            const uint32_t group_tx = a.stage_tx * (uint32_t)a.group;
            const uint32_t group_stride = (uint32_t)stage_stride * (uint32_t)a.group;
            // weights, scales, bias and tables do not depend on the previous kernel of the stream; activations do
            if (a.bstat && !skip_loads && prod == 0 && elect_one()) {
                mbar_expect_tx(w_full, (uint32_t)a.nslices * L::B_BYTES);
                for (int s = 0; s < a.nslices; ++s)
                    tma_load_2d(s_wst + (size_t)s * L::B_BYTES, &tmB, w_full, (int)s_tab[s].z, 0);
            }
            if (a.add_lut && prod == 0 && elect_one()) {
                // the fused-add table: one bulk copy (the epilogue checks its tag before using it)
                mbar_expect_tx(lut_full, (uint32_t)TC_LUT_BYTES);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(smem_u32(s_lut)), "l"(a.add_lut), "r"((uint32_t)TC_LUT_BYTES), "r"(smem_u32(lut_full)) : "memory");
            }
            asm volatile("griddepcontrol.wait;" ::: "memory");
            for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x) {
                if (prod == 0 && t == blockIdx.x) TC_TRACE(2);
                // tile coordinates: only worked out by a producer that loads something of this tile
                int n0 = 0, tm = 0, w0 = 0, h0 = 0, nimg = 0;
                long long m0 = 0;
                bool have = false;
                auto locate = [&]() {
                    n0 = (t % ntn) * BN;
                    tm = t / ntn;
                    m0 = (long long)tm * a.tile_rows;
                    if (a.im2col == 2) {
                        nimg = tm / a.OH;
                        h0 = (tm % a.OH) * a.sh;                  // first packed row of this output row
                    } else if (a.im2col) {
                        const int ox = (int)(m0 % a.OW);
                        const long long q = m0 / a.OW;
                        const int oy = (int)(q % a.OH);
                        nimg = (int)(q / a.OH);
                        w0 = ox * a.sw - a.pl;
                        h0 = oy * a.sh - a.pt;
                    }
                    have = true;
                };
                uint32_t te = tab_addr;                           // table entry of the stage's first slice
                for (int g = 0; g < gpt && alive; ++g, te += 16u * (uint32_t)group) {
                    if (turn == (uint32_t)prod) {
                        if (!have) locate();
                        if (!__all_sync(0xffffffffu, mbar_wait_idle(empty_addr + st * 8, ph ^ 1u, wait_limit))) { atomicExch(&g_tc_status, 1); alive = false; }
                        const uint32_t fb = full_addr + st * 8;
                        // (self-test: no loads are issued, so the stage never fills and every waiter runs into its limit)
                        if (alive && !skip_loads && elect_one()) {
                            mbar_expect_tx_s(fb, group_tx);
                            uint32_t sa = ring_addr + (uint32_t)st * group_stride;
                            for (int gs = 0; gs < group; ++gs, sa += (uint32_t)stage_stride) {
                                const uint4 e = lds128(te + 16u * (uint32_t)gs);
                                if (mode == 2)      tma_load_4d_s(sa, &tmA, fb, 0, 0, h0 + (int)e.w, nimg);      // slice = filter row
                                else if (mode == 1) tma_load_im2col_s(sa, &tmA, fb, (int)e.x, w0, h0, nimg, (uint16_t)(e.y & 0xffffu), (uint16_t)(e.y >> 16));
                                else                tma_load_2d_s(sa, &tmA, fb, (int)e.x, (int)m0);
                                if (!bstat) tma_load_2d_s(sa + L::A_BYTES, &tmB, fb, (int)e.z, n0);
                            }
                        }
                    }
                    turn = (turn + 1) & turn_mask;
                    if (++st == STAGES) { st = 0; ph ^= 1u; }
                }
                if (prod == 0 && (t - (int)blockIdx.x) / (int)gridDim.x < 8) TC_TRACE(16 + (t - (int)blockIdx.x) / (int)gridDim.x);
                if (a.res && alive && !skip_loads && prod == 0) {
                    // the fused Add's other operand, one unit at a time, into the buffer the epilogue will overwrite
                    if (!have) locate();
                    for (int us = 0; us < UNITS; ++us) {
                        if (!__all_sync(0xffffffffu, mbar_wait(&io_empty[ub], uph ^ 1u, wait_limit))) { atomicExch(&g_tc_status, 6); alive = false; break; }
                        if (elect_one()) {
                            mbar_expect_tx(&io_full[ub], IO_BYTES);
                            tma_load_3d(s_io + (size_t)(a.nstg * EG + ub) * IO_BYTES, &tmR, &io_full[ub], n0 + us * UW,
                                        a.im2col == 2 ? 0 : (int)m0, a.im2col == 2 ? tm : 0);
                        }
                        if (++ub == NIO) { ub = 0; uph ^= 1u; }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        {
            // instruction descriptor: D = S32 (bits 4-5 = 2); A / B format at bits 7 / 10 (1 = signed 8-bit,
            // 0 = unsigned 8-bit); both operands K-major (bits 15, 16 = 0); N >> 3 at bit 17; M >> 4 at bit 24
            const uint32_t id = (2u << 4) | ((uint32_t)a.a_signed << 7) | ((uint32_t)a.b_signed << 10) |
                                ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            // the zero-point MMAs: same A, B = a constant int8 tile
            const uint32_t id_zw = (2u << 4) | ((uint32_t)a.a_signed << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
            const int group = a.group, gpt = a.nslices / a.group;          // slices per stage, stages per tile
            int st = 0; uint32_t ph = 0;                     // ring position: stage and its phase bit
            bool alive = true;
            int it = 0;
            const uint32_t full_addr = smem_u32(full), empty_addr = smem_u32(empty);
            const int nzw = a.nzw;
            const bool bstat = a.bstat != 0;
            const long long wait_limit = a.wait_limit;
            // descriptors differ from slot to slot only in the 14-bit start-address field: one add per slice
            const uint64_t da0 = make_smem_desc<SWZ>(smem_u32(ring));
            const uint64_t db0 = make_smem_desc<SWZ>(bstat ? smem_u32(s_wst) : smem_u32(ring) + L::A_BYTES);
            const uint64_t dstage = (uint64_t)(stage_stride >> 4);
            const uint64_t dgroup = dstage * (uint64_t)a.group;
            const uint64_t dwslice = (uint64_t)(L::B_BYTES >> 4);
            const uint64_t dbstep = bstat ? dwslice : dstage;            // from one slice's weight tile to the next
            const uint64_t dz0 = make_smem_desc<SWZ>(smem_u32(s_zw));
            if (bstat && !__all_sync(0xffffffffu, mbar_wait(w_full, 0, wait_limit))) { atomicExch(&g_tc_status, 7); alive = false; }
            TC_TRACE(3);
            tc_fence_after();
            for (int t = blockIdx.x; t < ntiles && alive; t += gridDim.x, ++it) {
                const int buf = it & ((1 << NACC_LOG2) - 1);
                // the epilogue must have drained this accumulator buffer (one round of the buffers ago)
                if (!__all_sync(0xffffffffu, mbar_wait_idle(smem_u32(&acc_empty[buf]), (((uint32_t)it >> NACC_LOG2) & 1u) ^ 1u, wait_limit))) { atomicExch(&g_tc_status, 4); break; }
                tc_fence_after();
                const uint32_t tacc = tmem_base + (uint32_t)(buf * BN);
                uint64_t dbs = db0;                              // stationary weights: the stage's first tile
                for (int g = 0; g < gpt; ++g, dbs += dwslice * (uint64_t)group) {
                    if (!__all_sync(0xffffffffu, mbar_wait_fast(full_addr + st * 8, ph, wait_limit))) { atomicExch(&g_tc_status, 2); alive = false; break; }
                    tc_fence_after();
                    const uint32_t eb = empty_addr + st * 8;
                    if (elect_one()) {                 // the same lane every time: a commit covers the MMAs of its own thread
                        uint64_t da = da0 + dgroup * (uint64_t)st;
                        uint64_t db = bstat ? dbs : db0 + dgroup * (uint64_t)st;
                        for (int gs = 0; gs < group; ++gs, da += dstage, db += dbstep) {
                            tc_mma_i8(tacc, da, db, id, (uint32_t)(g | gs));        // the tile's first MMA overwrites
                            #pragma unroll
                            for (int k = 1; k < SWZ / 32; ++k) tc_mma_i8_acc(tacc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), id);
                            for (int z = 0; z < nzw; ++z) {
                                const uint64_t dz = dz0 + dwslice * (uint64_t)z;
                                #pragma unroll
                                for (int k = 0; k < SWZ / 32; ++k) tc_mma_i8_acc(tacc, da + (uint64_t)(k * 2), dz + (uint64_t)(k * 2), id_zw);
                            }
                        }
                        tc_commit_s(eb);           // stage reusable once these MMAs have read it
                    }
                    if (++st == STAGES) { st = 0; ph ^= 1u; }
                }
                if (alive && elect_one()) tc_commit(&acc_full[buf]);  // accumulator of this tile complete
                if (it == 0) TC_TRACE(4);
                if (it < 8) TC_TRACE(24 + it);
            }
        }
    } else {
        // ===================== epilogue =====================
        // 16 warps: warp & 3 selects the TMEM lane quadrant (a hardware restriction), the other two bits select a
        // quarter of each unit's columns.  A warp that gives up on a wait keeps walking the tiles (without waiting
        // again) so that the named barriers it shares stay balanced; the host sees the status word.
        const int ew = warp - 2;
        const int quad = warp & 3;
        // With eg epilogue groups the 4 / eg warps of a quadrant that share a group split a unit's columns; group g works
        // on the tiles whose index is g modulo eg, so that up to eg tiles are in the epilogue at once and a warp's waits
        // (accumulator, TMEM load, store) overlap with the arithmetic of the other groups' warps on its scheduler.
        constexpr int eg = EG, ppg = 4 / EG;
        const int grp = (ew >> 2) / ppg;
        const int part = (ew >> 2) - grp * ppg;
        const int etid = threadIdx.x - 64;
        constexpr int NCH = EG * UW / 64;                     // 16-column chunks per warp and unit: 1, 2 or 4
        const int NSTG_UNITS = a.nstg * EG;                   // unit-sized buffers the staging area takes
        const int row = quad * 32 + lane;
        const uint32_t sw_x = UW == 128 ? (uint32_t)(row & 7) : (uint32_t)((row >> 1) & 3);   // TMA swizzle of this row
        const int pw = a.KW + 1;
        const bool fused = a.res != nullptr;
        // The fused-add table arrives by a bulk copy the producer has issued.  A table is used only if it was built
        // for exactly this launch's quantisation parameters.
        bool lut_ok = false;
        if (a.add_lut) {
            if (etid == 0) {
                uint32_t ok = 1;
                const uint32_t* tag = (const uint32_t*)(a.add_lut + TC_LUT_BYTES);
                for (int i = 0; i < TC_LUT_TAG_WORDS; ++i) ok &= (tag[i] == a.lut_tag[i]);
                *s_lut_ok = ok;
            }
            epi_barrier();
            lut_ok = *s_lut_ok != 0;
            // the producer's bulk copy of the table
            if (!mbar_wait(lut_full, 0, a.wait_limit)) { atomicExch(&g_tc_status, 8); lut_ok = false; }
        }
        const bool use_lut = fused && lut_ok;
        if (ew == 0) TC_TRACE(5);
        const bool always_fix = fused && !lut_ok;            // no table: every chunk takes the reference arithmetic
        const bool dump_acc = a.acc_out != nullptr;
        // the reference arithmetic's constants: only the cold pass uses them, which rebuilds them from the launch
        // arguments instead of keeping them in registers through the hot loop
        auto make_exact = [&]() {
            EpiExact ex;
            ex.sy1 = a.rq.sy; ex.zy1 = (float)a.rq.zy;
            ex.lo1 = fmaxf(a.rq.tlo, (float)a.rq.clo); ex.hi1 = fminf(a.rq.thi, (float)a.rq.chi);
            ex.fused = fused; ex.res_u8 = a.res_u8; ex.zr = (float)a.res_zp; ex.sr = a.res_scale;
            ex.sy2 = a.rq2.sy; ex.zy2 = (float)a.rq2.zy;
            ex.lo2 = fmaxf(a.rq2.tlo, (float)a.rq2.clo); ex.hi2 = fminf(a.rq2.thi, (float)a.rq2.chi);
            ex.always = always_fix;
            return ex;
        };
        static_assert(sizeof(EpiExact) <= 64, "EpiExact outgrew its shared-memory slot");
        if (etid == 0) *s_ex = make_exact();                  // (published by the first staging's barriers)
        const float lo1 = fmaxf(a.rq.tlo, (float)a.rq.clo), hi1 = fminf(a.rq.thi, (float)a.rq.chi), zy1 = (float)a.rq.zy;
        // how the hot path ends (warp-uniform, fixed for the launch)
        const int kind = use_lut ? EPI_LUT
                       : (lo1 == a.rq.tlo && hi1 == a.rq.thi) ? (a.rq.tlo == 0.f ? EPI_SAT_U8 : EPI_SAT_S8) : EPI_CLAMP;
        const uint32_t lut_addr = smem_u32(s_lut);
        int cur_n0 = -1;
        // this warp's staging buffers: [32 rows][W = eg * UW / 4 bytes] each, laid out as the TMA store's swizzle of that
        // width.  With two of them (a.nstg == 2) a unit's store is still reading one buffer while the next unit is
        // written into the other, so the warp never waits for a store it has only just issued.
        constexpr uint32_t W = (uint32_t)EG * (UW / 4);
        const uint32_t st_base0 = smem_u32(s_io) + (uint32_t)ew * (32u * W);
        const uint32_t st_flip = a.nstg == 2 ? (uint32_t)EG * (uint32_t)IO_BYTES : 0u;     // distance to the second buffer
        const uint32_t st_sw = W == 64 ? (uint32_t)((lane >> 1) & 3) : (W == 32 ? (uint32_t)((lane >> 2) & 1) : 0u);
        bool dead = false;
        // what the hot path adds to the requantised value: the output zero point; with the table also minus the type minimum
        const float zoff = use_lut ? zy1 - a.rq.tlo : zy1;
        float thr = 0.0f;                                    // 0.5 - E of the staged n-tile (see epi_chunk_fast); 0: no hot path
        int stagings = 0;
        auto stage_constants = [&](int n0) {
            {
                // per-channel constants of this n-tile (all epilogue warps are between tiles here)
                epi_barrier();
                uint32_t* emax = s_emax + 2 * (stagings & 1);
                float bq_max = 0.f, bsy_max = 0.f;
                for (int j = etid; j < BN; j += 32 * TC_EPI_WARPS) {
                    const int ch = min(n0 + j, a.OC - 1);           // columns beyond OC are padding: any finite constants do
                    const float m = __fmul_rn(a.rq.sx, a.w_scales ? a.w_scales[ch] : a.w_scale);
                    s_m[j] = m;
                    s_mq[j] = __fdiv_rn(m, a.rq.sy);
                    s_bterm[j] = a.bias ? __fmul_rn(__int2float_rn(a.bias[ch]), a.b_scales ? a.b_scales[ch] : a.b_scale) : 0.f;
                }
                for (int i = etid; i < a.ncls * BN; i += 32 * TC_EPI_WARPS) {
                    const int cls = i / BN, j = i - cls * BN;
                    const int ch = min(n0 + j, a.OC - 1);
                    int v = 0;
                    if (a.need_corr && n0 + j < a.OC) {
                        // sum over the in-image taps of (x - zx)(w - zw) - x w + zw x = -zx w + zx zw
                        const int yp = a.ypair[cls / a.ncx], xp = a.xpair[cls % a.ncx];
                        const int y0 = yp >> 4, y1 = yp & 15, x0 = xp >> 4, x1 = xp & 15;
                        const int32_t* P = a.prefix + n0 + j;
                        v = a.zx * (P[(long long)(y1 * pw + x1) * a.OC] - P[(long long)(y0 * pw + x1) * a.OC] -
                                    P[(long long)(y1 * pw + x0) * a.OC] + P[(long long)(y0 * pw + x0) * a.OC]) -
                            (y1 - y0) * (x1 - x0) * a.kvalid_c * a.zx * a.zw;
                    }
                    s_cc[i] = v;
                    // (recomputed rather than read back: another thread wrote s_m[j] and s_bterm[j])
                    const float m = __fmul_rn(a.rq.sx, a.w_scales ? a.w_scales[ch] : a.w_scale);
                    const float b = a.bias ? __fmul_rn(__int2float_rn(a.bias[ch]), a.b_scales ? a.b_scales[ch] : a.b_scale) : 0.f;
                    const float bq = epi_make_bq(b, v, m, a.rq.sy, a.inv_sy, zoff);
                    s_bq[i] = bq;
                    bq_max = fmaxf(bq_max, fabsf(bq));
                    bsy_max = fmaxf(bsy_max, fabsf(__fmul_rn(b, a.inv_sy)));
                }
                // (NaN or infinity anywhere turns into a huge bound: no hot path for this n-tile)
                const uint32_t w0 = __reduce_max_sync(0xffffffffu, __float_as_uint(bq_max <= 3.0e38f ? bq_max : 3.0e38f));
                const uint32_t w1 = __reduce_max_sync(0xffffffffu, __float_as_uint(bsy_max <= 3.0e38f ? bsy_max : 3.0e38f));
                if (lane == 0) { atomicMax(&emax[0], w0); atomicMax(&emax[1], w1); }
                epi_barrier();
                {
                    const float rz = 257.0f;                                                                 // |R + zoff| of interest
                    const float rmax = fmaxf(fabsf(a.rq.tlo - 1.0f - zy1), fabsf(a.rq.thi + 1.0f - zy1));    // |R| of interest
                    // big: an accumulator (or accumulator minus correction) of this launch can exceed 2^24, where the
                    // conversions to fp32 round as well
                    const float big = a.acc_big ? 1.0f : 0.0f;
                    const float bsy = 1.0001f * __uint_as_float(emax[1]), bqm = __uint_as_float(emax[0]);
                    const float e = 1.1f * 5.9604645e-8f *
                                    ((3.0f + big) * rmax + (1.0f + big) * bsy + (1.0f + big) * (rz + bqm) + 2.0f * bqm + fabsf(zoff) + rz);
                    // a bound this large means unusual scales: everything takes the reference arithmetic
                    thr = (always_fix || !(e < 0.0625f)) ? 0.0f : 0.5f - e;
                    // (parameter-space tables come with the host's own bound)
                    if (PTAB) thr = always_fix ? 0.0f : a.thr_host;
                }
                // the other slot: every thread has long finished reading it (it served the staging before this one)
                if (etid == 0) { s_emax[2 * ((stagings + 1) & 1)] = 0u; s_emax[2 * ((stagings + 1) & 1) + 1] = 0u; }
                ++stagings;
                cur_n0 = n0;
            }
        };
        // groups only exist with a single n-tile: its constants are staged once, by all warps, before any warp could
        // find itself without a tile
        if (eg > 1) stage_constants(0);
        if (ew == 0) TC_TRACE(6);
        // The tile loop exists once per way the hot path ends (KIND, fixed for the launch), chosen by one switch below, so
        // that the per-chunk code is straight-line.
        auto run_tiles = [&](auto kind_tag) {
            constexpr int KIND = decltype(kind_tag)::value;
            int it = 0;
            int ub = 0; uint32_t uph = 0;                    // operand-buffer position (kept without divisions)
            uint32_t st_base = st_base0;
            for (int t = blockIdx.x; t < ntiles; t += gridDim.x, ++it) {
                if ((it & (eg - 1)) != grp) continue;
                // (a single n-tile is the common case of the epilogue-bound layers: no divisions then)
                const int tm = ntn == 1 ? t : t / ntn;
                const int n0 = ntn == 1 ? 0 : (t - tm * ntn) * BN;
                const long long m0 = (long long)tm * a.tile_rows;
                const int buf = it & ((1 << NACC_LOG2) - 1);
                if (n0 != cur_n0) stage_constants(n0);
                if (ew == 0 && it < 8) TC_TRACE(56 + it);
                if (!dead && !mbar_wait(&acc_full[buf], ((uint32_t)it >> NACC_LOG2) & 1u, a.wait_limit)) { atomicExch(&g_tc_status, 3); dead = true; }
                if (ew == 0 && t == blockIdx.x) TC_TRACE(7);
                if (ew == 0 && it < 8) TC_TRACE(32 + it);
                tc_fence_after();
                const long long m = m0 + row;
                const bool mvalid = row < a.tile_rows && m < a.M;
                // class of this pixel's rectangle of in-image taps
                int cls = 0;
                if (a.need_rect) {
                    const unsigned mu = (unsigned)m;               // M < 2^31
                    const unsigned qd = mu / (unsigned)a.OW;
                    const int ox = (int)(mu - qd * (unsigned)a.OW);
                    const int oy = (int)(qd % (unsigned)a.OH);
                    const int iy = oy * a.sh - a.pt, ix = ox * a.sw - a.pl;
                    // first in-image tap, one past the last in-image tap
                    int ky0 = iy < 0 ? (-iy + a.dh - 1) / a.dh : 0;
                    int ky1 = iy >= a.H ? 0 : min(a.KH, (a.H - 1 - iy) / a.dh + 1);
                    int kx0 = ix < 0 ? (-ix + a.dw - 1) / a.dw : 0;
                    int kx1 = ix >= a.W ? 0 : min(a.KW, (a.W - 1 - ix) / a.dw + 1);
                    ky0 = min(ky0, a.KH); kx0 = min(kx0, a.KW);
                    ky1 = max(ky1, ky0);  kx1 = max(kx1, kx0);
                    cls = mvalid ? a.ycls[ky0 * 16 + ky1] * a.ncx + a.xcls[kx0 * 16 + kx1] : 0;
                }
                const int32_t* corr_row = s_cc + cls * BN;
                const uint32_t a_m = smem_u32(s_m), a_b = smem_u32(s_bterm), a_cc = smem_u32(corr_row);
                const uint32_t a_mq = smem_u32(s_mq), a_bq = smem_u32(s_bq + cls * BN);
                const uint32_t tacc = tmem_base + (uint32_t)(buf * BN) + ((uint32_t)(quad * 32) << 16);
                // units in which this warp has real columns (a prefix: the last n-tile may reach beyond OC)
                const int nact = min(UNITS, max(0, (a.OC - n0 - part * (int)W + UW - 1) / UW));
                #pragma unroll 1
                for (int us = 0; us < nact; ++us) {
                    const int colw = us * UW + part * (int)W;      // first column of this warp in this unit
                    const uint32_t res_row = smem_u32(s_io + (size_t)(NSTG_UNITS + ub) * IO_BYTES + row * UW);    // (fused: eg == 1)
                    // The warp's NCH chunks of 16 columns go through two register sets that take turns: the loads of
                    // the first two are issued before the unit's waits; a set is reloaded (chunk + 2) as soon as its
                    // chunk has been computed.  (tcgen05.wait::ld waits for every load the thread has issued.)
                    uint32_t r[2][16];
                    tc_ld16_issue(tacc + (uint32_t)colw, r[0]);
                    if (NCH > 1) tc_ld16_issue(tacc + (uint32_t)(colw + 16), r[1]);
                    if (fused && !dead && !mbar_wait(&io_full[ub], uph, a.wait_limit)) { atomicExch(&g_tc_status, 5); dead = true; }
                    // the store that last used this staging buffer has read it out
                    if (lane == 0) {
                        if (st_flip) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        else         asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    }
                    __syncwarp();
                    const uint32_t st_row = st_base + (uint32_t)lane * W;
                    #pragma unroll
                    for (int j = 0; j < NCH; ++j) {
                        if ((j & 1) == 0) {
                            tc_ld16_wait(r[0]);
                            if (j + 1 < NCH) tc_ld16_wait(r[1]);
                        }
                        const int col0 = colw + j * 16;
                        const uint4 rv = KIND == EPI_LUT ? lds128(res_row + ((((uint32_t)(part * NCH + j)) ^ sw_x) << 4)) : make_uint4(0, 0, 0, 0);
                        float dmg[4];
                        uint4 outv;
                        if constexpr (PTAB) {
                            const TabFastP ad = {tabs.mq + n0 + col0, tabs.bq + n0 + col0};
                            outv = epi_chunk_fast<KIND>(r[j & 1], rv, ad, a.ep, lut_addr, dmg);
                        } else {
                            const TabFast ad = {a_mq + col0 * 4, a_bq + col0 * 4};
                            outv = epi_chunk_fast<KIND>(r[j & 1], rv, ad, a.ep, lut_addr, dmg);
                        }
                        // groups the hot path cannot vouch for (|q" - n| within E of a half, a huge value, or no usable
                        // table at all: thr = 0) take the reference arithmetic, from the accumulators still in registers
                        if (__any_sync(0xffffffffu, fmaxf(fmaxf(dmg[0], dmg[1]), fmaxf(dmg[2], dmg[3])) >= thr)) {
                            const uint32_t* rr = r[j & 1];
                            const uint32_t resw[4] = {rv.x, rv.y, rv.z, rv.w};
                            uint32_t w[4] = {outv.x, outv.y, outv.z, outv.w};
                            #pragma unroll
                            for (int g = 0; g < 4; ++g) {
                                if (__any_sync(0xffffffffu, dmg[g] >= thr))
                                    w[g] = epi_fix_group<KIND>((int)rr[g * 4], (int)rr[g * 4 + 1], (int)rr[g * 4 + 2], (int)rr[g * 4 + 3],
                                                               a_m + (col0 + g * 4) * 4, a_b + (col0 + g * 4) * 4, a_cc + (col0 + g * 4) * 4, resw[g],
                                                               &a.ep, lut_addr, s_ex);
                            }
                            outv = make_uint4(w[0], w[1], w[2], w[3]);
                        }
                        sts128(st_row + (((uint32_t)j ^ st_sw) << 4), outv);
                        if (j + 2 < NCH) tc_ld16_issue(tacc + (uint32_t)(colw + (j + 2) * 16), r[j & 1]);
                    }
                    // the accumulator dump of the tests: from a second read of the accumulators
                    if (dump_acc) {
                        const EpiExact ex = make_exact();
                        #pragma unroll 1
                        for (int j = 0; j < NCH; ++j) {
                            const int col0 = colw + j * 16;
                            uint32_t rr[16];
                            tc_ld16(tacc + (uint32_t)col0, rr);
                            epi_cold(rr, res_row + ((((uint32_t)(part * NCH + j)) ^ sw_x) << 4), st_row + (((uint32_t)j ^ st_sw) << 4),
                                     a_m + col0 * 4, a_b + col0 * 4, a_cc + col0 * 4, ex, false,
                                     (mvalid && n0 + col0 < a.OC) ? a.acc_out + m * a.OC + n0 + col0 : nullptr);
                        }
                    }
                    if (fused) {
                        // this warp has finished reading the other operand's unit
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&io_empty[ub]);
                        if (++ub == NIO) { ub = 0; uph ^= 1u; }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the TMA store
                    __syncwarp();
                    if (lane == 0) {
                        const int row0 = quad * 32;
                        if (row0 < a.tile_rows && m0 + row0 < a.M)
                            tma_store_3d(&tmY, st_base, n0 + colw, a.im2col == 2 ? row0 : (int)(m0 + row0), a.im2col == 2 ? tm : 0);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    st_base = st_base == st_base0 ? st_base0 + st_flip : st_base0;
                }
                if (fused) {
                    // padding-only units: nothing to read, but the operand buffers still want this warp's release.  The
                    // warp first waits for the unit's load like everybody else: an arrival that came before the buffer's
                    // previous use was complete would be counted towards that use and release the buffer under a slower
                    // warp.
                    for (int us = nact; us < UNITS; ++us) {
                        if (!dead && !mbar_wait(&io_full[ub], uph, a.wait_limit)) { atomicExch(&g_tc_status, 5); dead = true; }
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&io_empty[ub]);
                        if (++ub == NIO) { ub = 0; uph ^= 1u; }
                    }
                }
                // this warp has finished reading the accumulator buffer
                if (ew == 0 && it < 8) TC_TRACE(48 + it);
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&acc_empty[buf]);
                if (ew == 0 && t == blockIdx.x) TC_TRACE(8);
                if (ew == 0 && it < 8) TC_TRACE(40 + it);
                if (ew == 0) TC_TRACE(9);
            }
        };
        switch (kind) {
            case EPI_LUT:    run_tiles(std::integral_constant<int, EPI_LUT>{}); break;
            case EPI_SAT_U8: run_tiles(std::integral_constant<int, EPI_SAT_U8>{}); break;
            case EPI_SAT_S8: run_tiles(std::integral_constant<int, EPI_SAT_S8>{}); break;
            default:         run_tiles(std::integral_constant<int, EPI_CLAMP>{}); break;
        }
        // shared memory may go once the last store has read it; its global writes complete with the kernel
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        if (ew == 0) TC_TRACE(10);
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BN << NACC_LOG2) : "memory");
        TC_TRACE(11);
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
    if (p->c > 16 || p->c < 1 || p->dil_w != 1 || p->ow > TC_BM || p->oc % 16 != 0 || p->kh > 15 || p->kw > 15) return r;
    if (p->stride_w > 8 || p->stride_h > 8) return r;
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

// xp[n][yp][xq][0..C) = x[n][yp - pt][xq - pl][0..C) inside the image, the input zero point outside; [C..cpad) = 0
template <int CPAD>
__global__ void __launch_bounds__(256) row_input_pack_kernel(const RowInputArgs a)
{
    pdl_enter();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.total) return;
    const int xq = (int)(i % a.wp);
    const long long t = i / a.wp;
    const int yp = (int)(t % a.hp);
    const int n = (int)(t / a.hp);
    const int iy = yp - a.pt, ix = xq - a.pl;
    uint8_t v[CPAD];
    #pragma unroll
    for (int c = 0; c < CPAD; ++c) v[c] = c < a.C ? (uint8_t)a.fill : (uint8_t)0;
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

struct AddLutArgs { uint8_t* lut; int y_u8, res_u8; float sy; int zy; float sr; int zr; Requant out; uint32_t tag[TC_LUT_TAG_WORDS]; };

// lut[(conv value - type minimum) * pitch + other operand's byte] = output byte of RefElementwiseBinaryWorkload(Add)
// followed by the fused activation, evaluated once per pair of 8-bit values with the reference fp32 arithmetic.  The
// tag behind the table names the quantisation parameters it was built for.
__global__ void add_lut_kernel(const AddLutArgs a)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;       // 65536 threads
    const int b1 = i >> 8, b2 = i & 255;
    const int q1 = a.y_u8 ? b1 : b1 - 128;
    const int q2 = a.res_u8 ? b2 : (int)(int8_t)b2;
    const float fa = __fmul_rn(__int2float_rn(q1 - a.zy), a.sy);
    const float fb = __fmul_rn(__int2float_rn(q2 - a.zr), a.sr);
    const int q = quantize_dev(__fadd_rn(fa, fb), a.out.sy, a.out.zy, a.out.tlo, a.out.thi);
    a.lut[b1 * TC_LUT_PITCH + b2] = (uint8_t)min(max(q, a.out.clo), a.out.chi);
    if (i < TC_LUT_TAG_WORDS) ((uint32_t*)(a.lut + TC_LUT_BYTES))[i] = a.tag[i];
}

static size_t add_lut_offset(int oc, int kh, int kw, int c)
{
    size_t n = (size_t)(kh + 1) * (kw + 1) * oc * sizeof(int32_t);
    if (c <= 16) n += 3 * (size_t)oc * kh * 128;            // row-window weights, then the direct-stem weights in both pixel widths
    return (n + 255) & ~(size_t)255;
}

static uint32_t f32_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

// what identifies a fused-add table: both operands' and the output's quantisation, and the activation clamp
static void make_lut_tag(const b200k_conv2d_params* p, uint32_t* tag)
{
    const Requant out = make_requant(0.f, p->add_out, p->clamp_lo, p->clamp_hi);
    tag[0] = 0x4C555431u;
    tag[1] = f32_bits(p->y.scale);           tag[2] = (uint32_t)p->y.zero_point;           tag[3] = (uint32_t)p->y.dtype;
    tag[4] = f32_bits(p->add_operand.scale); tag[5] = (uint32_t)p->add_operand.zero_point; tag[6] = (uint32_t)p->add_operand.dtype;
    tag[7] = f32_bits(p->add_out.scale);     tag[8] = (uint32_t)p->add_out.zero_point;     tag[9] = (uint32_t)p->add_out.dtype;
    tag[10] = (uint32_t)out.clo;             tag[11] = (uint32_t)out.chi;
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

// State that CUDA keeps per device (SM count, the opt-in shared-memory size of a kernel) is cached per device: a
// process may drive several GPUs, one network and one host thread each.
constexpr int TC_MAX_DEVICES = 64;

static int current_device()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= TC_MAX_DEVICES) dev = 0;
    return dev;
}

static int sm_count()
{
    static std::atomic<int> cached[TC_MAX_DEVICES];
    const int dev = current_device();
    int n = cached[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

// Tile width.  The kernel is persistent with one CTA per SM, and on the network shapes a tile's cost is its epilogue
// (proportional to its columns) plus a fixed part, so the estimate of a launch is waves x (columns + fixed), with
// waves = ceil(tiles / SMs): narrow tiles fill the SMs when there are few rows, wide tiles win when there are many
// (fewer re-reads of the activation tile).  Ties go to the wider tile.
static int pick_bn(int oc, long long ntm)
{
    const long long sms = sm_count();
    int best = 64;
    long long best_cost = -1;
    for (int bn = 64; bn <= 256; bn *= 2) {
        const long long tiles = ntm * ((oc + bn - 1) / bn);
        const long long cost = ((tiles + sms - 1) / sms) * (bn + 96);
        if (best_cost < 0 || cost <= best_cost) { best = bn; best_cost = cost; }
    }
    return best;
}

// Distinct in-image tap ranges [k0, k1) along one axis, over all output positions of that axis.
struct TapClasses {
    bool ok;
    int ncy, ncx;
    uint8_t ypair[16], xpair[16];
    uint8_t ycls[256], xcls[256];
};

static bool axis_classes(int out, int in, int k, int stride, int pad, int dil, uint8_t* pairs, uint8_t* cls, int& n)
{
    n = 0;
    memset(cls, 0, 256);
    bool seen[256] = {false};
    // output positions o_lo .. o_hi have their whole window inside the image (one class): the walk skips from the first
    // of them to the last (a 1x1 convolution over a GEMM-shaped tensor has hundreds of thousands of them)
    const int o_lo = pad <= 0 ? 0 : (pad + stride - 1) / stride;
    const long long last_full = (long long)in - 1 - (long long)(k - 1) * dil + pad;
    const int o_hi = last_full < 0 ? -1 : (int)(last_full / stride < out - 1 ? last_full / stride : out - 1);
    for (int o = 0; o < out; ++o) {
        const int i0 = o * stride - pad;
        int k0 = i0 < 0 ? (-i0 + dil - 1) / dil : 0;
        int k1 = i0 >= in ? 0 : ((in - 1 - i0) / dil + 1 < k ? (in - 1 - i0) / dil + 1 : k);
        if (k0 > k) k0 = k;
        if (k1 < k0) k1 = k0;
        const int code = k0 * 16 + k1;
        if (!seen[code]) {
            if (n == 16) return false;
            seen[code] = true;
            pairs[n] = (uint8_t)code;
            cls[code] = (uint8_t)n;
            ++n;
        }
        if (o >= o_lo && o < o_hi) o = o_hi - 1;          // (the next one visited is o_hi)
    }
    return n > 0;
}

static TapClasses tap_classes(const b200k_conv2d_params* p)
{
    TapClasses t;
    memset(&t, 0, sizeof(t));
    if (p->kh > 15 || p->kw > 15) return t;
    t.ok = axis_classes(p->oh, p->h, p->kh, p->stride_h, p->pad_top, p->dil_h, t.ypair, t.ycls, t.ncy) &&
           axis_classes(p->ow, p->wd, p->kw, p->stride_w, p->pad_left, p->dil_w, t.xpair, t.xcls, t.ncx);
    return t;
}

// Zero points must lie in their element type's range (the constant -zw tiles and the padding fill are 8-bit values),
// and the output scale in a range where its reciprocal is an ordinary number.
static bool quantisation_in_range(const b200k_conv2d_params* p)
{
    int lo, hi;
    type_range(p->x.dtype, lo, hi);
    if (p->x.zero_point < lo || p->x.zero_point > hi) return false;
    type_range(p->w.dtype, lo, hi);
    if (!p->w.scales && (p->w.zero_point < lo || p->w.zero_point > hi)) return false;
    type_range(p->y.dtype, lo, hi);
    if (p->y.zero_point < lo || p->y.zero_point > hi) return false;
    if (!(p->y.scale > 1e-30f && p->y.scale < 1e30f)) return false;
    if (p->add_operand.data) {
        type_range(p->add_out.dtype, lo, hi);
        if (p->add_out.zero_point < lo || p->add_out.zero_point > hi) return false;
    }
    return true;
}

static bool row_window_eligible(const b200k_conv2d_params* p)
{
    const RowPlan r = row_window_plan(p);
    if (!r.ok || !p->packed || !p->scratch || p->scratch_bytes < r.scratch_bytes) return false;
    const void* outp = p->add_operand.data ? p->add_out.data : p->y.data;
    if (!p->x.data || !p->w.data || !outp) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->w.dtype) || !is_q8(p->y.dtype)) return false;
    if (!quantisation_in_range(p)) return false;
    if ((((uintptr_t)p->scratch | (uintptr_t)p->packed | (uintptr_t)outp) & 15) != 0) return false;
    if (p->add_operand.data && ((((uintptr_t)p->add_operand.data) & 15) != 0)) return false;
    if ((long long)p->n * p->oh > (1ll << 30) || (long long)p->n * p->oh * p->ow > (1ll << 31) - TC_BM) return false;
    return true;
}

static bool stem_direct_eligible(const b200k_conv2d_params* p);

bool conv_tc_eligible(const b200k_conv2d_params* p)
{
    if (p->c <= 16) return stem_direct_eligible(p) || row_window_eligible(p);
    const void* outp = p->add_operand.data ? p->add_out.data : p->y.data;
    if (!p->x.data || !p->w.data || !outp) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->w.dtype) || !is_q8(p->y.dtype)) return false;
    if (!quantisation_in_range(p)) return false;
    if (p->add_operand.data && ((((uintptr_t)p->add_operand.data | (uintptr_t)p->add_out.data) & 15) != 0)) return false;
    if (p->c % 16 != 0 || p->oc % 16 != 0) return false;               // TMA: 16-byte pixel and row strides
    if (p->w.zero_point != 0 && p->w.scales) return false;             // per-axis weights are symmetric
    if ((((uintptr_t)p->x.data | (uintptr_t)p->w.data | (uintptr_t)outp) & 15) != 0) return false;
    if (p->x.zero_point != 0 && !p->packed) return false;              // needs the prefix table
    if (p->kh > 15 || p->kw > 15) return false;
    if ((long long)p->kh * p->kw * ((p->c + 63) / 64) > 2048) return false;   // K-slice table in shared memory: at most 32 KiB
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
    if (p->x.zero_point != 0) {
        const TapClasses tc = tap_classes(p);
        if (!tc.ok || (size_t)tc.ncy * tc.ncx * pick_bn(p->oc, (M + TC_BM - 1) / TC_BM) * 4 > 32 * 1024) return false;
    }
    return true;
}


template <int BN, int SWZ, int EG, bool PTAB = false>
static int launch_tc(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmY, const CUtensorMap& tmR,
                     const TcArgs& a, cudaStream_t stream, const TcTabs* tabs = nullptr)
{
    if constexpr (EG == 1 && !PTAB) {
        if (tabs) return launch_tc<BN, SWZ, EG, true>(tmA, tmB, tmY, tmR, a, stream, tabs);
    }
    using L = TcSmem<BN, SWZ>;
    const size_t budget = 227 * 1024;                                   // opt-in shared memory per CTA on sm_100
    TcArgs a2 = a;
    size_t rest = 1024 + L::CONST_BYTES + ((size_t)a.ncls * 2 + 1) * BN * 4 + 16 + 64 + (size_t)(EG + a.nio) * L::IO_BYTES + (a.add_lut ? TC_LUT_BYTES : 0) + 256 +
                  (size_t)a.nslices * 16 +
                  (size_t)a.nzw * L::B_BYTES;
    // a second staging buffer per epilogue warp, then a third buffer for the fused Add's other operand (its loads then
    // run a whole unit ahead of the epilogue), each when the ring keeps at least three stages
    a2.nstg = 1;
    if (rest + (size_t)EG * L::IO_BYTES + 3 * L::STAGE_BYTES <= budget) { a2.nstg = 2; rest += (size_t)EG * L::IO_BYTES; }
    if (a.nio == 2 && rest + L::IO_BYTES + 3 * L::STAGE_BYTES <= budget) { a2.nio = 3; rest += L::IO_BYTES; }
    B200K_REQUIRE(rest + 2 * L::STAGE_BYTES <= budget, B200K_E_TOOBIG, "conv2d_q8: shared memory exhausted (%zu bytes of tables)", rest);
    // One n-tile and a weight tile of at most 64 KiB over all of K: keep it in shared memory for the whole launch, so
    // that the ring (and the L2 bandwidth behind it) carries activations only.
    const size_t wbytes = (size_t)a.nslices * L::B_BYTES;
    a2.bstat = (a.ntn == 1 && wbytes <= 64 * 1024 && rest + wbytes + 4 * L::A_BYTES <= budget) ? 1 : 0;
    const size_t stride = a2.bstat ? L::A_BYTES : L::STAGE_BYTES;
    const size_t fixed = rest + (a2.bstat ? wbytes : 0);
    // Ring: `stages` stages of `group` K-slices each.  Waiting for a stage, arming and releasing its barriers cost the
    // producer and the MMA issuer about as much as issuing two MMAs, so narrow tiles (short MMAs) want several slices per
    // stage: the largest divisor of the slice count, up to 8, that still leaves three stages.
    const int slots = (int)((budget - fixed) / stride);
    int group = 1, stages = slots < L::MAX_STAGES ? slots : L::MAX_STAGES;
    for (int g = 8; g >= 2; --g) {
        if (a.nslices % g != 0 || slots / g < 3) continue;
        group = g;
        stages = slots / g < L::MAX_STAGES ? slots / g : L::MAX_STAGES;
        break;
    }
    a2.group = group;
    a2.stages = stages;
    // A producer tells "slot consumed" from "slot consumed one ring pass earlier" by the barrier's phase parity alone,
    // which is only sound while it cannot run more than one pass ahead of the consumer: its previous turn (nprod
    // slices back) must lie within the same ring pass as the slot it waits for, i.e. nprod <= stages.
    a2.nprod = stages >= TC_PRODUCERS ? TC_PRODUCERS : (stages >= 2 ? 2 : 1);
    if (a2.bstat) a2.stage_tx = (uint32_t)(a.stage_tx - L::B_BYTES);
    const size_t smem = fixed + (size_t)stages * group * stride;
    auto kern = conv_tc_kernel<BN, SWZ, EG, PTAB>;
    // per instantiation and device: the largest dynamic shared-memory size opted into so far (a racing second thread
    // at worst repeats the call)
    static std::atomic<size_t> configured[TC_MAX_DEVICES];
    const int dev = current_device();
    if (smem > configured[dev].load(std::memory_order_acquire)) {
        B200K_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        size_t seen = configured[dev].load(std::memory_order_relaxed);
        while (seen < smem && !configured[dev].compare_exchange_weak(seen, smem, std::memory_order_release)) {}
    }
    const long long tiles = (long long)a.ntn * a.ntm;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    // Programmatic dependent launch: the grid may start while its predecessor in the stream drains (its set-up touches
    // nothing the predecessor writes); the producer threads wait for the predecessor before their first activation load.
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)grid, 1, 1);
    cfg.blockDim = dim3(TC_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if constexpr (PTAB) {
        B200K_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmY, tmR, a2, *tabs));
    } else {
        const TcNoTabs none = {0};
        B200K_CUDA(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, tmY, tmR, a2, none));
    }
    return check_launch("conv_tc_kernel");
}


// ---- few-channel convolutions (network stems) straight from the NHWC input -----------------------------------------
//
// A 3-channel pixel is not a TMA unit, and im2col rows of a 7 x 7 x 3 window overlap almost entirely.  This kernel
// keeps the rows themselves in shared memory and lets the tensor core read the overlapping windows where they lie:
//   * a loader thread brings the raw input rows in with bulk copies, well ahead; expander warps rewrite each into a ring
//     of "packed rows": the spatial
//     padding materialised with the input zero point, every pixel padded to cpad = 16 / stride_w bytes, so that the
//     window of output pixel ox starts exactly 16 * ox bytes into the row;
//   * the A operand of filter row ky is a K-major, non-swizzled matrix descriptor over one packed row with a row pitch of
//     16 bytes (8-row groups 128 bytes apart, K chunks 16 bytes apart): row ox of the matrix is bytes [16 ox, 16 ox + WB)
//     of the packed row, i.e. the window, and consecutive rows overlap.  Nothing is copied per window.
//   * the weights are re-packed at load time as [ky][OC / 8][WB / 16][8][16] (the same canonical layout) with zero in
//     the padded channel lanes, and stay in shared memory for the whole launch;
//   * a CTA walks a contiguous range of output rows (a tile is one output row), so every input row is expanded once per
//     CTA and serves KH / stride_h tiles; accumulators are double-buffered in tensor memory and sixteen epilogue warps
//     requantise them with the same code as the main kernel and store their bytes directly.
// Padding taps hold the zero point, so sum (x - zx) w = sum x w - zx sum_all w: one correction per channel, no border
// classes.  Symmetric weights only (zero point 0).  Every wait is bounded as in the main kernel.
constexpr int ST_SLOTS = 32;                    // packed-row ring (a power of two)
constexpr int ST_LOOKAHEAD = 4;                 // tiles the expanders may run ahead of the MMAs
constexpr int ST_DONE = 8;                      // ring of per-tile "MMAs complete" barriers (a power of two)
constexpr int ST_EXPANDERS = 4;
constexpr int ST_RAW = 16;                      // ring of raw input rows (bulk copies in flight ahead of the expanders)
constexpr int ST_THREADS = 32 * (2 + ST_EXPANDERS + TC_EPI_WARPS);     // MMA issuer, row loader, expanders, epilogue

struct StemArgs {
    const uint8_t* x; uint8_t* y; int32_t* acc_out;
    const uint8_t* wpk; const int32_t* wsum;
    const int32_t* bias; const float* w_scales; const float* b_scales;
    float w_scale, b_scale;
    int N, H, W, C, OH, OW, OC, KH, KW, sh, sw, pt, pl;
    int cpad, WB, slot_bytes, raw_bytes, Hp, Wp, tiles, tmem_cols;
    int split;                                  // 4-byte pixels, even / odd output pixels as the two 64-row halves of a tile
    int zx, a_signed, b_signed, acc_big;
    Requant rq;
    float inv_sy;
    EpiConsts ep;
    long long wait_limit;
};

__device__ __forceinline__ uint64_t make_smem_desc_plain(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;      // K chunk (16 bytes) to K chunk
    d |= (uint64_t)(sbo_bytes >> 4) << 32;      // 8-row group to 8-row group
    d |= (uint64_t)1 << 46;
    return d;                                   // layout type 0: no swizzle
}

__global__ void __launch_bounds__(ST_THREADS, 1) conv_stem_kernel(const __grid_constant__ StemArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* s_rows = smem;                                            // [ST_SLOTS][slot_bytes]
    uint8_t* s_w = s_rows + (size_t)ST_SLOTS * a.slot_bytes;           // [KH][OC * WB]
    float* s_m = (float*)(s_w + (size_t)a.KH * a.OC * a.WB);
    float* s_bterm = s_m + a.OC;
    int32_t* s_cc = (int32_t*)(s_bterm + a.OC);
    float* s_mq = (float*)(s_cc + a.OC);
    float* s_bq = s_mq + a.OC;
    uint32_t* s_emax = (uint32_t*)(s_bq + a.OC);                       // [2]
    EpiExact* s_ex = (EpiExact*)(s_emax + 4);
    uint64_t* row_full = (uint64_t*)(s_emax + 4 + 16);                 // [ST_SLOTS]
    uint64_t* mma_done = row_full + ST_SLOTS;                          // [ST_DONE]
    uint64_t* acc_full = mma_done + ST_DONE;                           // [2]
    uint64_t* acc_empty = acc_full + 2;                                // [2]
    uint64_t* w_full = acc_empty + 2;
    uint64_t* raw_full = w_full + 1;                                   // [ST_RAW] a raw row has landed
    uint64_t* raw_empty = raw_full + ST_RAW;                           // [ST_RAW] its expander has read it
    uint32_t* tmem_slot = (uint32_t*)(raw_empty + ST_RAW);
    uint8_t* s_raw = (uint8_t*)(((uintptr_t)(tmem_slot + 4) + 127) & ~(uintptr_t)127);   // [ST_RAW][raw_bytes]

    if (threadIdx.x == 0) TC_TRACE(0);
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    // this CTA's contiguous range of tiles (output rows)
    const int t_begin = (int)((long long)a.tiles * blockIdx.x / gridDim.x), t_end = (int)((long long)a.tiles * (blockIdx.x + 1) / gridDim.x);
    const int ntiles = t_end - t_begin;
    const long long v0 = (long long)(t_begin / a.OH) * a.Hp + (long long)(t_begin % a.OH) * a.sh;     // first virtual row
    const long long wait_limit = a.wait_limit;

    if (threadIdx.x < ST_SLOTS + ST_DONE + 5 + 2 * ST_RAW) {
        const int i = threadIdx.x;
        mbar_init(&row_full[i], (i >= ST_SLOTS + ST_DONE + 2 && i < ST_SLOTS + ST_DONE + 4) ? TC_EPI_WARPS : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 4) s_emax[threadIdx.x] = 0u;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ===================== weights, then the MMAs =====================
        if (elect_one()) {
            const uint32_t wbytes = (uint32_t)(a.KH * a.OC * a.WB);
            mbar_expect_tx(w_full, wbytes);
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                         ::"r"(smem_u32(s_w)), "l"(a.wpk), "r"(wbytes), "r"(smem_u32(w_full)) : "memory");
        }
        const uint32_t id = (2u << 4) | ((uint32_t)a.a_signed << 7) | ((uint32_t)a.b_signed << 10) |
                            ((uint32_t)(a.OC >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
        bool alive = __all_sync(0xffffffffu, mbar_wait(w_full, 0, wait_limit));
        if (!alive) atomicExch(&g_tc_status, 7);
        const uint32_t rows_addr = smem_u32(s_rows), w_addr = smem_u32(s_w);
        const uint32_t w_sbo = (uint32_t)(a.WB / 16) * 128u;
        // The issuing warp is one dependent chain per tile, and that chain is what the tile rate hangs on: relative row
        // indices in 32 bits, only the rows no earlier tile has waited for are waited for, descriptors advance by adds.
        const uint64_t da0 = make_smem_desc_plain(rows_addr, 16u, 128u);
        const uint64_t db0 = make_smem_desc_plain(w_addr, 128u, w_sbo);
        const uint64_t da_slot = (uint64_t)(a.slot_bytes >> 4), db_ky = (uint64_t)((a.OC * a.WB) >> 4);
        const int kks = a.WB / 32;
        int n = t_begin / a.OH, oy = t_begin - n * a.OH;
        const int base_n = n, base_oy = oy;                 // (v0 = base_n * Hp + base_oy * sh)
        int waited = 0;                                      // packed rows [0, waited) have been seen complete
        for (int i = 0; i < ntiles && alive; ++i) {
            const int lo = (n - base_n) * a.Hp + (oy - base_oy) * a.sh;                              // first packed row, relative
            const int buf = i & 1;
            for (int rv = lo > waited ? lo : waited; rv < lo + a.KH && alive; ++rv) {
                if (!__all_sync(0xffffffffu, mbar_wait(&row_full[rv & (ST_SLOTS - 1)], (uint32_t)(rv / ST_SLOTS) & 1u, wait_limit))) { atomicExch(&g_tc_status, 2); alive = false; }
            }
            waited = lo + a.KH;
            if (i < 8) TC_TRACE(16 + i);
            if (alive && !__all_sync(0xffffffffu, mbar_wait(&acc_empty[buf], (((uint32_t)i >> 1) & 1u) ^ 1u, wait_limit))) { atomicExch(&g_tc_status, 4); alive = false; }
            if (!alive) break;
            tc_fence_after();
            if (elect_one()) {
                const uint32_t tacc = tmem_base + (uint32_t)(buf * a.OC);
                uint64_t db = db0;
                int slot = lo & (ST_SLOTS - 1);
                for (int ky = 0; ky < a.KH; ++ky, db += db_ky) {
                    const uint64_t da = da0 + da_slot * (uint64_t)slot;
                    for (int kk = 0; kk < kks; ++kk)
                        tc_mma_i8(tacc, da + (uint64_t)(kk * 2), db + (uint64_t)(kk * 16), id, (ky | kk) != 0 ? 1u : 0u);
                    slot = (slot + 1) & (ST_SLOTS - 1);
                }
                tc_commit(&acc_full[buf]);
                tc_commit(&mma_done[i & (ST_DONE - 1)]);
            }
            __syncwarp();
            if (i < 8) TC_TRACE(24 + i);
            if (++oy == a.OH) { oy = 0; ++n; }
        }
    } else if (warp == 1) {
        // ===================== loader: raw input rows into the raw ring =====================
        asm volatile("griddepcontrol.wait;" ::: "memory");                 // the input comes from the kernel before this one
        if (lane == 0) {
            long long next = 0, loaded = 0;
            bool alive = true;
            for (int i = 0; i < ntiles && alive; ++i) {
                const int t = t_begin + i;
                const int n = t / a.OH, oy = t % a.OH;
                const long long lo = (long long)n * a.Hp + (long long)oy * a.sh - v0;
                for (long long rv = lo > next ? lo : next; rv < lo + a.KH && alive; ++rv) {
                    const int iy = (int)(rv - lo) + oy * a.sh - a.pt;
                    if (iy < 0 || iy >= a.H) continue;                       // a padding row: nothing to load
                    const int rs = (int)(loaded % ST_RAW);
                    if (!mbar_wait(&raw_empty[rs], ((uint32_t)(loaded / ST_RAW) & 1u) ^ 1u, wait_limit)) { atomicExch(&g_tc_status, 1); alive = false; break; }
                    const uint32_t bytes = (uint32_t)(a.W * a.C);
                    mbar_expect_tx(&raw_full[rs], bytes);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(smem_u32(s_raw + (size_t)rs * a.raw_bytes)), "l"(a.x + ((long long)n * a.H + iy) * bytes), "r"(bytes),
                                   "r"(smem_u32(&raw_full[rs])) : "memory");
                    ++loaded;
                }
                if (lo + a.KH > next) next = lo + a.KH;
                if (i < 8) TC_TRACE(56 + i);
            }
        }
    } else if (warp <= 1 + ST_EXPANDERS) {
        // ===================== expanders: raw rows -> packed rows =====================
        const int e = warp - 2;
        long long next = 0, loaded = 0;                                      // packed rows dealt out; raw rows consumed (all warps count alike)
        bool alive = true;
        const uint32_t zx4 = (uint32_t)(a.zx & 0xff) * 0x01010101u;
        for (int i = 0; i < ntiles && alive; ++i) {
            const int t = t_begin + i;
            const int n = t / a.OH, oy = t % a.OH;
            const long long lo = (long long)n * a.Hp + (long long)oy * a.sh - v0;
            if (e == 0 && i == 1) TC_TRACE(12);
            if (i >= ST_LOOKAHEAD) {
                const int j = i - ST_LOOKAHEAD;
                if (!mbar_wait(&mma_done[j % ST_DONE], (uint32_t)(j / ST_DONE) & 1u, wait_limit)) { atomicExch(&g_tc_status, 1); alive = false; break; }
            }
            for (long long rv = lo > next ? lo : next; rv < lo + a.KH && alive; ++rv) {
                const int iy = (int)(rv - lo) + oy * a.sh - a.pt;
                const bool inside_y = iy >= 0 && iy < a.H;
                const long long my_raw = loaded;
                if (inside_y) ++loaded;
                if ((int)(rv % ST_EXPANDERS) != e) continue;
                uint8_t* slot = s_rows + (size_t)(rv % ST_SLOTS) * a.slot_bytes;
                const int rs = (int)(my_raw % ST_RAW);
                const uint8_t* src = s_raw + (size_t)rs * a.raw_bytes;
                if (e == 0 && rv == 8) TC_TRACE(8);
                if (inside_y && !mbar_wait(&raw_full[rs], (uint32_t)(my_raw / ST_RAW) & 1u, wait_limit)) { atomicExch(&g_tc_status, 2); alive = false; break; }
                if (e == 0 && rv == 8) TC_TRACE(9);
                const uint32_t cmask = a.C >= 4 ? 0xffffffffu : (1u << (8 * a.C)) - 1u;
                const uint32_t slot_addr = smem_u32(slot), src_addr = smem_u32(src);
                if (a.C <= 4) {
                    // All of the row's loads first, then all of its stores: through generic pointers the compiler has to
                    // assume that a store may alias the next pixel's load, which serialises the row (1.8 us measured).
                    constexpr int MAXP = 9;                                  // pixels per lane: Wp * cpad <= slot_bytes
                    uint32_t pw[MAXP];
                    #pragma unroll
                    for (int k = 0; k < MAXP; ++k) {
                        const int px = lane + 32 * k, ix = px - a.pl;
                        uint32_t w0 = zx4;
                        if (px < a.Wp && inside_y && ix >= 0 && ix < a.W) {
                            // the pixel's bytes out of the two aligned words that hold them (the raw ring has slack behind every row)
                            const int off = ix * a.C;
                            const uint32_t qa = src_addr + (uint32_t)(off & ~3);
                            uint32_t lo32, hi32;
                            asm("ld.shared.b32 %0, [%1];" : "=r"(lo32) : "r"(qa));
                            asm("ld.shared.b32 %0, [%1 + 4];" : "=r"(hi32) : "r"(qa));
                            w0 = __funnelshift_r(lo32, hi32, 8 * (off & 3)) & cmask;
                        }
                        pw[k] = w0;
                    }
                    #pragma unroll
                    for (int k = 0; k < MAXP; ++k) {
                        const int px = lane + 32 * k, ix = px - a.pl;
                        if (px >= a.Wp) continue;
                        const bool real = inside_y && ix >= 0 && ix < a.W;
                        const uint32_t fill = real ? 0u : zx4;               // the pixel's bytes beyond the first word
                        if (a.cpad == 4) {
                            asm volatile("st.shared.b32 [%0], %1;" ::"r"(slot_addr + (uint32_t)(px * 4)), "r"(pw[k]) : "memory");
                            if (px >= 2) asm volatile("st.shared.b32 [%0], %1;" ::"r"(slot_addr + (uint32_t)(1024 + px * 4 - 8)), "r"(pw[k]) : "memory");   // the copy the odd pixels are read from
                        } else if (a.cpad == 8) {
                            asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(slot_addr + (uint32_t)(px * 8)), "r"(pw[k]), "r"(fill) : "memory");
                        } else {
                            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(slot_addr + (uint32_t)(px * 16)), "r"(pw[k]), "r"(fill), "r"(fill), "r"(fill) : "memory");
                        }
                    }
                } else {
                    for (int px = lane; px < a.Wp; px += 32) {
                        const int ix = px - a.pl;
                        uint32_t w0 = zx4, w1 = zx4, w2 = zx4, w3 = zx4;
                        if (inside_y && ix >= 0 && ix < a.W) {
                            const uint8_t* q = src + ix * a.C;
                            unsigned long long lo8 = 0, hi8 = 0;             // bytes 0..7 and 8..15 of the packed pixel
                            for (int c = 0; c < a.C; ++c) {
                                const unsigned long long b = q[c];
                                if (c < 8) lo8 |= b << (8 * c); else hi8 |= b << (8 * (c - 8));
                            }
                            w0 = (uint32_t)lo8; w1 = (uint32_t)(lo8 >> 32); w2 = (uint32_t)hi8; w3 = (uint32_t)(hi8 >> 32);
                        }
                        if (a.cpad == 8) *(uint2*)(slot + px * 8) = make_uint2(w0, w1);
                        else             *(uint4*)(slot + px * 16) = make_uint4(w0, w1, w2, w3);
                    }
                }
                if (e == 0 && rv == 8) TC_TRACE(10);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // generic-proxy writes -> visible to the MMA's reads
                __syncwarp();
                if (e == 0 && rv == 8) TC_TRACE(11);
                if (lane == 0) {
                    if (inside_y) mbar_arrive(&raw_empty[rs]);
                    mbar_arrive(&row_full[rv % ST_SLOTS]);
                }
            }
            if (lo + a.KH > next) next = lo + a.KH;
            if (e == 0 && i < 8) TC_TRACE(48 + i);
        }
    } else {
        // ===================== epilogue =====================
        const int ew = warp - (2 + ST_EXPANDERS);
        const int quad = warp & 3, part = ew >> 2;
        const int etid = threadIdx.x - 32 * (2 + ST_EXPANDERS);
        const int nchunks = a.OC / 16;
        const float lo1 = fmaxf(a.rq.tlo, (float)a.rq.clo), hi1 = fminf(a.rq.thi, (float)a.rq.chi), zy1 = (float)a.rq.zy;
        const int kind = (lo1 == a.rq.tlo && hi1 == a.rq.thi) ? (a.rq.tlo == 0.f ? EPI_SAT_U8 : EPI_SAT_S8) : EPI_CLAMP;
        if (etid == 0) {
            EpiExact ex;
            ex.sy1 = a.rq.sy; ex.zy1 = zy1; ex.lo1 = lo1; ex.hi1 = hi1;
            ex.fused = 0; ex.res_u8 = 0; ex.zr = 0.f; ex.sr = 0.f; ex.sy2 = 1.f; ex.zy2 = 0.f; ex.lo2 = 0.f; ex.hi2 = 0.f; ex.always = 0;
            *s_ex = ex;
        }
        // per-channel constants (one n-tile, one class)
        {
            float bq_max = 0.f, bsy_max = 0.f;
            for (int j = etid; j < a.OC; j += 32 * TC_EPI_WARPS) {
                const float m = __fmul_rn(a.rq.sx, a.w_scales ? a.w_scales[j] : a.w_scale);
                const float b = a.bias ? __fmul_rn(__int2float_rn(a.bias[j]), a.b_scales ? a.b_scales[j] : a.b_scale) : 0.f;
                const int cc = a.zx * a.wsum[j];
                s_m[j] = m; s_bterm[j] = b; s_cc[j] = cc;
                s_mq[j] = __fdiv_rn(m, a.rq.sy);
                const float bq = epi_make_bq(b, cc, m, a.rq.sy, a.inv_sy, zy1);
                s_bq[j] = bq;
                bq_max = fmaxf(bq_max, fabsf(bq));
                bsy_max = fmaxf(bsy_max, fabsf(__fmul_rn(b, a.inv_sy)));
            }
            const uint32_t w0 = __reduce_max_sync(0xffffffffu, __float_as_uint(bq_max <= 3.0e38f ? bq_max : 3.0e38f));
            const uint32_t w1 = __reduce_max_sync(0xffffffffu, __float_as_uint(bsy_max <= 3.0e38f ? bsy_max : 3.0e38f));
            if (lane == 0) { atomicMax(&s_emax[0], w0); atomicMax(&s_emax[1], w1); }
        }
        epi_barrier();
        float thr;
        {
            const float rz = 257.0f;
            const float rmax = fmaxf(fabsf(a.rq.tlo - 1.0f - zy1), fabsf(a.rq.thi + 1.0f - zy1));
            const float big = a.acc_big ? 1.0f : 0.0f;
            const float bsy = 1.0001f * __uint_as_float(s_emax[1]), bqm = __uint_as_float(s_emax[0]);
            const float e = 1.1f * 5.9604645e-8f * ((3.0f + big) * rmax + (1.0f + big) * bsy + (1.0f + big) * (rz + bqm) + 2.0f * bqm + fabsf(zy1) + rz);
            thr = !(e < 0.0625f) ? 0.0f : 0.5f - e;
        }
        const uint32_t a_m = smem_u32(s_m), a_b = smem_u32(s_bterm), a_cc = smem_u32(s_cc), a_mq = smem_u32(s_mq), a_bq = smem_u32(s_bq);
        const int trow = quad * 32 + lane;                  // row of the tile = lane of tensor memory
        const int px = a.split ? (trow & 63) * 2 + (trow >> 6) : trow;
        const bool valid = px < a.OW;
        bool dead = false;
        // A warp's share of a tile is nchunks / 4 chunks of 16 columns (one, for 64 channels): too little to hide the
        // tensor-memory load behind.  So the loads of the next (chunk, tile) are issued before the arithmetic of the
        // current one, and an accumulator buffer is released as soon as the warp has its last chunk in registers.
        auto run_tiles = [&](auto kind_tag) {
            constexpr int KIND = decltype(kind_tag)::value;
            const int cpw = part < nchunks ? (nchunks - part + 3) / 4 : 0;          // chunks per warp and tile
            uint32_t r0[16], r1[16];
            // chunk k of tile i (this warp's k-th: column chunk part + 4 k); the first chunk of a tile waits for its accumulator
            auto issue = [&](int i, int k, uint32_t* dst) {
                if (k == 0) {
                    if (!dead && !mbar_wait(&acc_full[i & 1], ((uint32_t)i >> 1) & 1u, wait_limit)) { atomicExch(&g_tc_status, 3); dead = true; }
                    tc_fence_after();
                }
                tc_ld16_issue(tmem_base + (uint32_t)((i & 1) * a.OC) + ((uint32_t)(quad * 32) << 16) + (uint32_t)((part + 4 * k) * 16), dst);
            };
            int i = 0, k = 0;                                 // the chunk whose load is in flight / being worked on
            if (cpw > 0 && ntiles > 0) issue(0, 0, r0);
            // (two register sets that take turns: the step is instantiated once for each, so both stay in registers)
            auto step = [&](uint32_t* rc, uint32_t* rn) {
                const int c = part + 4 * k;
                const int t = t_begin + i;
                tc_ld16_wait(rc);
                if (ew == 0 && k == 0 && i < 8) TC_TRACE(32 + i);
                int ni = i, nk = k + 1;
                if (nk == cpw) {
                    // the warp's last chunk of tile i is in registers
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[i & 1]);
                    nk = 0; ni = i + 1;
                }
                if (ni < ntiles) issue(ni, nk, rn);
                uint8_t* orow = a.y + ((long long)t * a.OW + px) * a.OC;
                const TabFast ad = {a_mq + c * 64, a_bq + c * 64};
                float dmg[4];
                uint4 outv = epi_chunk_fast<KIND>(rc, make_uint4(0, 0, 0, 0), ad, a.ep, 0u, dmg);
                if (__any_sync(0xffffffffu, fmaxf(fmaxf(dmg[0], dmg[1]), fmaxf(dmg[2], dmg[3])) >= thr)) {
                    uint32_t w[4] = {outv.x, outv.y, outv.z, outv.w};
                    #pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        if (__any_sync(0xffffffffu, dmg[g] >= thr))
                            w[g] = epi_fix_group<KIND>((int)rc[g * 4], (int)rc[g * 4 + 1], (int)rc[g * 4 + 2], (int)rc[g * 4 + 3],
                                                       a_m + (c * 16 + g * 4) * 4, a_b + (c * 16 + g * 4) * 4, a_cc + (c * 16 + g * 4) * 4, 0u,
                                                       &a.ep, 0u, s_ex);
                    }
                    outv = make_uint4(w[0], w[1], w[2], w[3]);
                }
                if (valid && !dead) {
                    *(uint4*)(orow + c * 16) = outv;
                    if (a.acc_out) {
                        int32_t* arow = a.acc_out + ((long long)t * a.OW + px) * a.OC + c * 16;
                        #pragma unroll
                        for (int j = 0; j < 16; ++j) arow[j] = (int)rc[j] - lds_s32(a_cc + (c * 16 + j) * 4);
                    }
                }
                if (ew == 0 && nk == 0 && i < 8) TC_TRACE(40 + i);
                i = ni; k = nk;
            };
            while (cpw > 0 && i < ntiles) {
                step(r0, r1);
                if (i < ntiles) step(r1, r0);
            }
            // warps without a chunk (fewer than four chunks per tile) still release every accumulator buffer
            if (cpw == 0) {
                for (int j = 0; j < ntiles; ++j) {
                    if (!dead && !mbar_wait(&acc_full[j & 1], ((uint32_t)j >> 1) & 1u, wait_limit)) { atomicExch(&g_tc_status, 3); dead = true; }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&acc_empty[j & 1]);
                }
            }
        };
        switch (kind) {
            case EPI_SAT_U8: run_tiles(std::integral_constant<int, EPI_SAT_U8>{}); break;
            case EPI_SAT_S8: run_tiles(std::integral_constant<int, EPI_SAT_S8>{}); break;
            default:         run_tiles(std::integral_constant<int, EPI_CLAMP>{}); break;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
    }
}

struct StemPlan { bool ok; int cpad, WB, slot_bytes, raw_bytes, Wp, Hp, split; size_t wbytes, smem; int tmem_cols; };

static StemPlan stem_plan(const b200k_conv2d_params* p)
{
    StemPlan r;
    memset(&r, 0, sizeof(r));
    if (p->c < 1 || p->c > 16 || p->dil_w != 1 || p->dil_h != 1 || p->ow > TC_BM || p->ow < 1) return r;
    if (p->stride_w != 1 && p->stride_w != 2) return r;
    if (p->stride_h < 1 || p->stride_h > 4 || p->kh < 1 || p->kh > 11 || p->kw < 1) return r;
    if (p->oc % 16 != 0 || p->oc < 16 || p->oc > 256) return r;
    r.cpad = 16 / p->stride_w;
    // Stride 2 with at most four channels: 4-byte pixels.  Windows of even output pixels then start 16 bytes apart, and
    // so do those of odd ones, 8 bytes later: the even pixels are rows 0..63 of the tile, the odd ones rows 64..127, read
    // from a second copy of the packed row that is shifted by 8 bytes and lies 1024 bytes (eight 8-row groups) behind the
    // first.  A 7-pixel window is 28 bytes: one K = 32 MMA per filter row instead of two.
    r.split = (p->stride_w == 2 && p->c <= 4 && p->ow <= 124 && ((p->ow - 1) * 2 + p->kw) * 4 <= 1024) ? 1 : 0;
    if (r.split) r.cpad = 4;
    if (p->c > r.cpad) return r;
    r.WB = (p->kw * r.cpad + 31) & ~31;
    if (r.WB > 128) return r;
    r.slot_bytes = ((TC_BM - 1) * 16 + r.WB + 127) & ~127;
    r.Wp = (p->ow - 1) * p->stride_w + p->kw;
    if ((long long)r.Wp * r.cpad > r.slot_bytes) return r;
    r.Hp = (p->oh - 1) * p->stride_h + p->kh;
    r.wbytes = (size_t)p->kh * p->oc * r.WB;
    if (r.wbytes > 64 * 1024) return r;
    r.tmem_cols = 32;
    while (r.tmem_cols < 2 * p->oc) r.tmem_cols <<= 1;
    // raw rows arrive by bulk copies: whole rows of a multiple of 16 bytes
    if (((long long)p->wd * p->c) % 16 != 0) return r;
    r.raw_bytes = (p->wd * p->c + 8 + 127) & ~127;         // (+8: the expanders read whole words around a pixel)
    r.smem = 1024 + (size_t)ST_SLOTS * r.slot_bytes + r.wbytes + (size_t)p->oc * 20 + 16 + 64 + (ST_SLOTS + ST_DONE + 5 + 2 * ST_RAW) * 8 + 16 +
             128 + (size_t)ST_RAW * r.raw_bytes;
    r.ok = r.smem <= 227 * 1024;
    return r;
}

// wpk[ky][oc / 8][chunk][oc % 8][16]: byte b of chunk = window byte chunk * 16 + b = (kx, c) with kx = byte / cpad, c = byte % cpad
struct StemWeightArgs { const uint8_t* w; uint8_t* wpk; int OC, KH, KW, C, cpad, WB; };
__global__ void stem_weight_pack_kernel(const StemWeightArgs a)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= a.KH * a.OC * a.WB) return;
    const int b = i & 15;
    const int r8 = (i >> 4) & 7;
    const int rest = i >> 7;
    const int chunks = a.WB / 16;
    const int chunk = rest % chunks;
    const int og = (rest / chunks) % (a.OC / 8);
    const int ky = rest / (chunks * (a.OC / 8));
    const int oc = og * 8 + r8, wb = chunk * 16 + b;
    const int kx = wb / a.cpad, c = wb - kx * a.cpad;
    uint8_t v = 0;
    if (kx < a.KW && c < a.C) v = a.w[(((long long)oc * a.KH + ky) * a.KW + kx) * a.C + c];
    a.wpk[i] = v;
}

// split: the 4-byte-pixel layout (packed next to the other one, so that the choice can be made per launch: it depends
// on the output width, which is not a property of the weights)
static size_t stem_wpack_offset(const b200k_conv2d_params* p, int split)
{
    return (size_t)(p->kh + 1) * (p->kw + 1) * p->oc * sizeof(int32_t) + (size_t)p->oc * p->kh * 128 * (split ? 2 : 1);
}

static bool stem_direct_eligible(const b200k_conv2d_params* p)
{
    if (p->add_operand.data || p->selftest_us > 0 || !p->packed) return false;
    if (!p->x.data || !p->w.data || !p->y.data) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->w.dtype) || !is_q8(p->y.dtype)) return false;
    if (!p->w.scales && p->w.zero_point != 0) return false;                   // symmetric weights only
    if (p->bias.data && p->bias.dtype != B200K_S32) return false;
    if (!quantisation_in_range(p)) return false;
    if ((((uintptr_t)p->packed | (uintptr_t)p->y.data | (uintptr_t)p->x.data) & 15) != 0) return false;
    if (p->acc_out && (((uintptr_t)p->acc_out) & 3) != 0) return false;
    if ((long long)p->n * p->oh > (1ll << 30)) return false;
    const StemPlan pl = stem_plan(p);
    return pl.ok && (long long)p->n * pl.Hp < (1ll << 30);        // (relative packed-row indices are 32-bit)
}

static int launch_conv_stem(const b200k_conv2d_params* p, cudaStream_t stream)
{
    const StemPlan pl = stem_plan(p);
    StemArgs a;
    a.x = (const uint8_t*)p->x.data; a.y = (uint8_t*)p->y.data; a.acc_out = p->acc_out;
    a.wpk = (const uint8_t*)p->packed + stem_wpack_offset(p, pl.split);
    a.wsum = (const int32_t*)p->packed + (long long)(p->kh * (p->kw + 1) + p->kw) * p->oc;       // prefix[(KH, KW)]: all taps
    a.bias = (const int32_t*)p->bias.data; a.w_scales = p->w.scales; a.b_scales = p->bias.scales;
    a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.N = p->n; a.H = p->h; a.W = p->wd; a.C = p->c; a.OH = p->oh; a.OW = p->ow; a.OC = p->oc;
    a.KH = p->kh; a.KW = p->kw; a.sh = p->stride_h; a.sw = p->stride_w; a.pt = p->pad_top; a.pl = p->pad_left;
    a.cpad = pl.cpad; a.WB = pl.WB; a.slot_bytes = pl.slot_bytes; a.raw_bytes = pl.raw_bytes; a.Hp = pl.Hp; a.Wp = pl.Wp;
    a.split = pl.split;
    a.tiles = p->n * p->oh; a.tmem_cols = pl.tmem_cols;
    a.zx = p->x.zero_point;
    a.a_signed = p->x.dtype == B200K_S8; a.b_signed = p->w.dtype == B200K_S8;
    {
        const long long taps = (long long)p->kh * p->kw * p->c;
        const long long xm = p->x.dtype == B200K_U8 ? 255 : 128, wm = p->w.dtype == B200K_U8 ? 255 : 128;
        const long long azx = a.zx < 0 ? -a.zx : a.zx;
        a.acc_big = taps * xm * wm + azx * taps * wm >= (1ll << 24) ? 1 : 0;
    }
    a.rq = make_requant(p->x.scale, p->y, p->clamp_lo, p->clamp_hi);
    a.inv_sy = rn_reciprocal(p->y.scale);
    {
        auto two = [](float v) { return make_float2(v, v); };
        const float lo1 = fmaxf(a.rq.tlo, (float)a.rq.clo), hi1 = fminf(a.rq.thi, (float)a.rq.chi), zy1 = (float)a.rq.zy;
        a.ep.inv2 = two(a.inv_sy); a.ep.nsy2 = two(-a.rq.sy); a.ep.magic2 = two(TC_MAGIC); a.ep.zero2 = two(0.f); a.ep.neg2 = two(-1.f);
        a.ep.nmagic2 = two(-TC_MAGIC);
        a.ep.zoff_lut2 = two((zy1 - a.rq.tlo) - TC_MAGIC);
        a.ep.zoff_sat2 = two(zy1 - TC_MAGIC);
        a.ep.zoff_clamp2 = two(zy1);
        a.ep.lo = TC_MAGIC + lo1;
        a.ep.hi = TC_MAGIC + hi1;
    }
    a.wait_limit = TC_WAIT_LIMIT_CYCLES;
    static std::atomic<bool> configured[TC_MAX_DEVICES];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= TC_MAX_DEVICES) dev = 0;
    if (!configured[dev].load(std::memory_order_acquire)) {
        B200K_CUDA(cudaFuncSetAttribute(conv_stem_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
        configured[dev].store(true, std::memory_order_release);
    }
    const int sms = sm_count();
    const int grid = a.tiles < sms ? a.tiles : sms;
    launch_pdl(conv_stem_kernel, dim3((unsigned)grid), dim3(ST_THREADS), pl.smem, stream, a);
    return check_launch("conv_stem_kernel");
}


// ---- host copies of a fused-Add convolution's per-channel constants ------------------------------------------------
//
// The fused-Add epilogue is bound by the shared-memory pipe (table lookups), so its mq / bq tables go through the
// kernel's parameter space instead (TabFastP), which means the host has to know them.  b200k_conv2d_pack therefore
// reads the per-channel weight sums, scales and bias of such a layer back once (a few KB, at load time) and keeps
// them keyed by the packed buffer's address; a launch uses them when the buffer and the four device arrays are the
// ones that were packed, and otherwise stages its tables on the device as every other launch does.
struct HostPack {
    const void* w; const void* w_scales; const void* bias; const void* b_scales;
    int oc, kh, kw, c;
    std::vector<float> ws, bs;
    std::vector<int32_t> bias_v, wsum;
    // the tables of the last launch and what they were computed from (a layer is launched with the same quantisation
    // parameters every time: the ~2 k table entries are then formed once, not per launch)
    std::mutex mu;
    bool have = false;
    float key[8];
    int ikey[6];
    float thr = 0.f;
    TcTabs tabs;
};
static std::mutex g_hp_mutex;
static std::unordered_map<const void*, std::shared_ptr<HostPack>> g_hp;

int tc_pack_host_tables(const b200k_conv2d_params* p, void* packed, cudaStream_t stream)
{
    {
        std::lock_guard<std::mutex> lock(g_hp_mutex);
        g_hp.erase(packed);
    }
    if (!p->add_operand.data || p->oc > TC_PTAB_MAX || p->oc % 16 != 0 || p->c <= 16) return B200K_OK;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) { cudaGetLastError(); return B200K_OK; }
    auto hp = std::make_shared<HostPack>();
    hp->w = p->w.data; hp->w_scales = p->w.scales; hp->bias = p->bias.data; hp->b_scales = p->bias.scales;
    hp->oc = p->oc; hp->kh = p->kh; hp->kw = p->kw; hp->c = p->c;
    const size_t n = (size_t)p->oc;
    hp->wsum.resize(n);
    B200K_CUDA(cudaMemcpyAsync(hp->wsum.data(), (const int32_t*)packed + (size_t)(p->kh * (p->kw + 1) + p->kw) * n, n * 4, cudaMemcpyDeviceToHost, stream));
    if (p->w.scales) { hp->ws.resize(n); B200K_CUDA(cudaMemcpyAsync(hp->ws.data(), p->w.scales, n * 4, cudaMemcpyDeviceToHost, stream)); }
    if (p->bias.data) { hp->bias_v.resize(n); B200K_CUDA(cudaMemcpyAsync(hp->bias_v.data(), p->bias.data, n * 4, cudaMemcpyDeviceToHost, stream)); }
    if (p->bias.data && p->bias.scales) { hp->bs.resize(n); B200K_CUDA(cudaMemcpyAsync(hp->bs.data(), p->bias.scales, n * 4, cudaMemcpyDeviceToHost, stream)); }
    B200K_CUDA(cudaStreamSynchronize(stream));
    std::lock_guard<std::mutex> lock(g_hp_mutex);
    g_hp[packed] = hp;
    return B200K_OK;
}

// epi_make_bq on the host (the same operations in the same order; fmaf is the IEEE fused multiply-add)
static float host_make_bq(float b, int cc, float m, float sy, float inv_sy, float zoff)
{
    const float ch = (float)(cc & ~0xfff), cl = (float)(cc & 0xfff);
    const float p1 = ch * m, e1 = fmaf(ch, m, -p1);
    const float p2 = cl * m, e2 = fmaf(cl, m, -p2);
    const float s1 = b - p1;
    const float bb1 = s1 - b;
    const float r1 = (b - (s1 - bb1)) + (-p1 - bb1);
    const float s2 = s1 - p2;
    const float bb2 = s2 - s1;
    const float r2 = (s1 - (s2 - bb2)) + (-p2 - bb2);
    const float tail = ((r1 + r2) - e1) - e2;
    const float hi = s2 + tail;
    const float bb3 = hi - s2;
    const float lo = (s2 - (hi - bb3)) + (tail - bb3);
    const float q0 = hi * inv_sy;
    const float rem = fmaf(-q0, sy, hi) + lo;
    const float q = fmaf(rem, inv_sy, q0);
    return q + zoff;
}

// Fills the parameter-space tables of a fused-Add launch from the host copies; false: not available for this launch.
static bool host_tables_for(const b200k_conv2d_params* p, const TcArgs& a, TcTabs* tabs, float* thr_out)
{
    if (!p->packed || a.ncls != 1 || a.im2col == 2 || p->oc > TC_PTAB_MAX) return false;
    std::shared_ptr<HostPack> hp;
    {
        std::lock_guard<std::mutex> lock(g_hp_mutex);
        auto it = g_hp.find(p->packed);
        if (it == g_hp.end()) return false;
        hp = it->second;
    }
    if (hp->w != p->w.data || hp->w_scales != p->w.scales || hp->bias != p->bias.data || hp->b_scales != p->bias.scales ||
        hp->oc != p->oc || hp->kh != p->kh || hp->kw != p->kw || hp->c != p->c) return false;
    const float sx = a.rq.sx, sy = a.rq.sy, inv_sy = a.inv_sy, zy1 = (float)a.rq.zy;
    const float zoff = zy1 - a.rq.tlo;                       // the table's index: minus the type minimum
    const float key[8] = {sx, sy, inv_sy, zy1, a.rq.tlo, a.rq.thi, p->w.scale, p->bias.scale};
    const int ikey[6] = {a.zx, a.zw, a.kvalid_c, a.need_corr, a.acc_big, p->bias.data ? 1 : 0};
    std::lock_guard<std::mutex> lock(hp->mu);
    if (hp->have && memcmp(key, hp->key, sizeof(key)) == 0 && memcmp(ikey, hp->ikey, sizeof(ikey)) == 0) {
        memcpy(tabs, &hp->tabs, sizeof(TcTabs));
        *thr_out = hp->thr;
        return true;
    }
    float bq_max = 0.f, bsy_max = 0.f;
    for (int ch = 0; ch < p->oc; ++ch) {
        const float m = sx * (p->w.scales ? hp->ws[ch] : p->w.scale);
        const float b = p->bias.data ? (float)hp->bias_v[ch] * (p->bias.scales ? hp->bs[ch] : p->bias.scale) : 0.f;
        const int cc = a.need_corr ? a.zx * hp->wsum[ch] - p->kh * p->kw * a.kvalid_c * a.zx * a.zw : 0;
        tabs->mq[ch] = m / sy;
        const float bq = host_make_bq(b, cc, m, sy, inv_sy, zoff);
        tabs->bq[ch] = bq;
        bq_max = fmaxf(bq_max, fabsf(bq));
        bsy_max = fmaxf(bsy_max, fabsf(b * inv_sy));
    }
    for (int ch = p->oc; ch < TC_PTAB_MAX; ++ch) { tabs->mq[ch] = 0.f; tabs->bq[ch] = 0.f; }
    if (!(bq_max <= 3.0e38f) || !(bsy_max <= 3.0e38f)) return false;
    const float rz = 257.0f;
    const float rmax = fmaxf(fabsf(a.rq.tlo - 1.0f - zy1), fabsf(a.rq.thi + 1.0f - zy1));
    const float big = a.acc_big ? 1.0f : 0.0f;
    const float bsy = 1.0001f * bsy_max;
    const float e = 1.1f * 5.9604645e-8f * ((3.0f + big) * rmax + (1.0f + big) * bsy + (1.0f + big) * (rz + bq_max) + 2.0f * bq_max + fabsf(zoff) + rz);
    *thr_out = !(e < 0.0625f) ? 0.0f : 0.5f - e;
    memcpy(hp->key, key, sizeof(key));
    memcpy(hp->ikey, ikey, sizeof(ikey));
    memcpy(&hp->tabs, tabs, sizeof(TcTabs));
    hp->thr = *thr_out;
    hp->have = true;
    return true;
}

int launch_conv_tc(const b200k_conv2d_params* p, cudaStream_t stream, int kvalid_c)
{
    // few-channel stems: straight from the NHWC input when the geometry allows it (no re-packed copy of the input)
    if (p->c <= 16 && kvalid_c == 0 && stem_direct_eligible(p)) return launch_conv_stem(p, stream);
    B200K_REQUIRE(conv_tc_eligible(p), B200K_E_UNSUPPORTED, "conv2d_q8: not eligible for the tcgen05 kernel");
    B200K_REQUIRE(load_driver_entry_points(), B200K_E_CUDA, "conv2d_q8: cuTensorMapEncode* not available from the driver");
    TcArgs a;
    a.bias = (const int32_t*)p->bias.data; a.acc_out = p->acc_out;
    a.w_scales = p->w.scales; a.b_scales = p->bias.scales; a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.prefix = (const int32_t*)p->packed;
    a.zx = p->x.zero_point;
    a.kvalid_c = kvalid_c > 0 ? kvalid_c : p->c;
    a.zw = p->w.scales ? 0 : p->w.zero_point;
    // -zw as one int8 tile value, or as the sum of two when it does not fit (zw > 128, or zw = -128 whose negative is +128)
    a.nzw = a.zw == 0 ? 0 : ((a.zw <= 128 && a.zw > -128) ? 1 : 2);
    a.zw_val[0] = a.nzw == 2 ? (a.zw > 0 ? -128 : 64) : -a.zw;
    a.zw_val[1] = a.nzw == 2 ? -a.zw - a.zw_val[0] : 0;
    a.N = p->n; a.H = p->h; a.W = p->wd; a.C = p->c; a.OH = p->oh; a.OW = p->ow; a.OC = p->oc;
    a.KH = p->kh; a.KW = p->kw; a.sh = p->stride_h; a.sw = p->stride_w; a.pt = p->pad_top; a.pl = p->pad_left;
    a.dh = p->dil_h; a.dw = p->dil_w;
    a.M = (long long)p->n * p->oh * p->ow;
    const RowPlan rowp = p->c <= 16 ? row_window_plan(p) : RowPlan{};
    const bool row_mode = rowp.ok;
    const bool gemm = !row_mode && p->kh == 1 && p->kw == 1 && p->stride_h == 1 && p->stride_w == 1 && p->pad_top == 0 &&
                      p->pad_left == 0 && p->oh == p->h && p->ow == p->wd;
    a.im2col = row_mode ? 2 : gemm ? 0 : 1;
    const int swz = row_mode ? rowp.swz : p->c >= 128 ? 128 : 64;
    a.cchunks = row_mode ? 1 : (p->c + swz - 1) / swz;     // the last chunk of a tap may reach beyond C: TMA fills A with zeros there
    a.mask_cpad = row_mode ? rowp.cpad : 0;
    a.mask_kw = p->kw;
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
    a.res = fa.res; a.res_scale = fa.res_scale; a.res_zp = fa.res_zp; a.res_u8 = fa.res_u8;
    a.rq2 = fa.out;
    a.inv_sy = rn_reciprocal(p->y.scale);
    {
        // t = MAGIC + n comes out of the rounding; adding zoff (an integer below 2^24, so exact) gives: with the
        // fused-add table the table's row index n + zy - type minimum, a byte in 0..255; with the type's own saturation
        // the result n + zy itself; with an explicit clamp the biased result MAGIC + n + zy, clamped in that domain
        const float zy1 = (float)a.rq.zy;
        const float lo1 = fmaxf(a.rq.tlo, (float)a.rq.clo), hi1 = fminf(a.rq.thi, (float)a.rq.chi);
        auto two = [](float v) { return make_float2(v, v); };
        a.ep.inv2 = two(a.inv_sy); a.ep.nsy2 = two(-a.rq.sy); a.ep.magic2 = two(TC_MAGIC); a.ep.zero2 = two(0.f); a.ep.neg2 = two(-1.f); a.ep.nmagic2 = two(-TC_MAGIC);
        a.ep.zoff_lut2 = two((zy1 - a.rq.tlo) - TC_MAGIC);
        a.ep.zoff_sat2 = two(zy1 - TC_MAGIC);
        a.ep.zoff_clamp2 = two(zy1);
        a.ep.lo = TC_MAGIC + lo1;
        a.ep.hi = TC_MAGIC + hi1;
    }
    // b200k_conv2d_pack builds the fused-add table when it is given the add operand; the kernel checks its tag and
    // falls back to the reference arithmetic (slow) when the table was made for other parameters
    a.add_lut = (fa.res && p->packed) ? (const uint8_t*)p->packed + add_lut_offset(p->oc, p->kh, p->kw, p->c) : nullptr;
    memset(a.lut_tag, 0, sizeof(a.lut_tag));
    if (fa.res) make_lut_tag(p, a.lut_tag);
    a.nio = fa.res ? 2 : 0;
    {
        // worst-case magnitudes: taps * max |x| * max |w| for the accumulator (with the -zw term), zx * taps * max |w| +
        // taps |zx zw| for the correction
        const long long taps = (long long)p->kh * p->kw * p->c;
        const long long xm = p->x.dtype == B200K_U8 ? 255 : 128, wm = p->w.dtype == B200K_U8 ? 255 : 128;
        const long long azx = a.zx < 0 ? -a.zx : a.zx, azw = a.zw < 0 ? -a.zw : a.zw;
        const long long amax = taps * xm * (wm + azw), cmax = azx * taps * (wm + azw);
        a.acc_big = amax + cmax >= (1ll << 24) ? 1 : 0;
    }
    a.ncy = a.ncx = a.ncls = 1;
    memset(a.ypair, 0, sizeof(a.ypair)); memset(a.xpair, 0, sizeof(a.xpair));
    memset(a.ycls, 0, sizeof(a.ycls));   memset(a.xcls, 0, sizeof(a.xcls));
    a.ypair[0] = (uint8_t)p->kh; a.xpair[0] = (uint8_t)p->kw;          // the full rectangle [0, KH) x [0, KW)
    if (rect) {
        const TapClasses tc = tap_classes(p);
        B200K_REQUIRE(tc.ok, B200K_E_UNSUPPORTED, "conv2d_q8: too many distinct border cases for the tcgen05 kernel");
        a.ncy = tc.ncy; a.ncx = tc.ncx; a.ncls = tc.ncy * tc.ncx;
        memcpy(a.ypair, tc.ypair, 16); memcpy(a.xpair, tc.xpair, 16);
        memcpy(a.ycls, tc.ycls, 256);  memcpy(a.xcls, tc.xcls, 256);
    }
    // bounded waits: about two seconds, or the caller's self-test limit (clock64 runs at no more than 2 GHz)
    a.skip_loads = p->selftest_us > 0 ? 1 : 0;
    a.wait_limit = p->selftest_us > 0 ? (long long)p->selftest_us * 2000ll : TC_WAIT_LIMIT_CYCLES;

    const int bn = pick_bn(p->oc, a.ntm);
    a.ntn = (p->oc + bn - 1) / bn;
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
        if (rowp.cpad == 8) launch_pdl(row_input_pack_kernel<8>, dim3((unsigned)div_up(ra.total, 256)), dim3(256), 0, stream, ra);
        else                launch_pdl(row_input_pack_kernel<16>, dim3((unsigned)div_up(ra.total, 256)), dim3(256), 0, stream, ra);
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
    // output (and the fused Add's other operand) as [groups][rows][OC]: one group of M rows, or in row-window mode
    // one group of OW rows per output row, so that a tile's surplus rows fall outside the tensor and are clipped
    CUtensorMap tmY, tmR;
    {
        const int uw = bn < 128 ? bn : 128;
        const cuuint64_t rows = row_mode ? (cuuint64_t)p->ow : (cuuint64_t)a.M;
        const cuuint64_t groups = row_mode ? (cuuint64_t)p->n * p->oh : 1;
        cuuint64_t dims[3] = {(cuuint64_t)p->oc, rows, groups};
        cuuint64_t strides[2] = {(cuuint64_t)p->oc, (cuuint64_t)p->oc * rows};
        cuuint32_t estr[3] = {1, 1, 1};
        const CUtensorMapSwizzle usw = uw == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
        // Epilogue groups: with one n-tile and no fused Add, 256 / bn (at most 4) tiles are in the epilogue at once, each
        // on its own accumulator buffer and a quarter (half) of the epilogue warps.  (Measured on ResNet-50's layers at
        // batch 256: 1x1 and 3x3 convolutions with 64 or 128 output channels run 10 - 30 % faster this way.)
        a.eg = (a.ntn == 1 && !fa.res && !row_mode) ? (bn == 64 ? 4 : (bn == 128 ? 2 : 1)) : 1;
        // row-window mode (network stems): two groups (0.41 -> 0.32 ms for ResNet-50's stem at batch 256; four were slower
        // than one there)
        if (row_mode && a.ntn == 1 && !fa.res && bn == 64) a.eg = 2;
        // stores: one epilogue warp's 32 rows x (eg * uw / 4) columns
        const int stw = a.eg * uw / 4;
        cuuint32_t box_st[3] = {(cuuint32_t)stw, 32, 1};
        CUresult r = g_encode_tiled(&tmY, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, a.y, dims, strides, box_st, estr,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE,
                                    stw == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : (stw == 32 ? CU_TENSOR_MAP_SWIZZLE_32B : CU_TENSOR_MAP_SWIZZLE_NONE),
                                    CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        B200K_REQUIRE(r == CUDA_SUCCESS, B200K_E_CUDA, "conv2d_q8: cuTensorMapEncodeTiled(output) failed with %d", (int)r);
        tmR = tmY;
        if (fa.res) {
            cuuint32_t box_ld[3] = {(cuuint32_t)uw, (cuuint32_t)TC_BM, 1};
            r = g_encode_tiled(&tmR, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, (void*)fa.res, dims, strides, box_ld, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, usw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            B200K_REQUIRE(r == CUDA_SUCCESS, B200K_E_CUDA, "conv2d_q8: cuTensorMapEncodeTiled(add operand) failed with %d", (int)r);
        }
    }
    const bool grouped = a.eg > 1;
    // a fused Add whose per-channel constants the host knows: tables through the parameter space
    TcTabs tabs_storage;
    const TcTabs* host_tabs = nullptr;
    a.thr_host = 0.f;
    if (fa.res && a.eg == 1 && kvalid_c == 0 && host_tables_for(p, a, &tabs_storage, &a.thr_host)) host_tabs = &tabs_storage;
    if (swz == 128) {
        if (bn == 256) return launch_tc<256, 128, 1>(tmA, tmB, tmY, tmR, a, stream, host_tabs);
        if (bn == 128) return grouped ? launch_tc<128, 128, 2>(tmA, tmB, tmY, tmR, a, stream) : launch_tc<128, 128, 1>(tmA, tmB, tmY, tmR, a, stream, host_tabs);
        if (a.eg == 2) return launch_tc<64, 128, 2>(tmA, tmB, tmY, tmR, a, stream);
        return grouped ? launch_tc<64, 128, 4>(tmA, tmB, tmY, tmR, a, stream) : launch_tc<64, 128, 1>(tmA, tmB, tmY, tmR, a, stream, host_tabs);
    }
    if (bn == 256) return launch_tc<256, 64, 1>(tmA, tmB, tmY, tmR, a, stream, host_tabs);
    if (bn == 128) return grouped ? launch_tc<128, 64, 2>(tmA, tmB, tmY, tmR, a, stream) : launch_tc<128, 64, 1>(tmA, tmB, tmY, tmR, a, stream, host_tabs);
    if (a.eg == 2) return launch_tc<64, 64, 2>(tmA, tmB, tmY, tmR, a, stream);
    return grouped ? launch_tc<64, 64, 4>(tmA, tmB, tmY, tmR, a, stream) : launch_tc<64, 64, 1>(tmA, tmB, tmY, tmR, a, stream, host_tabs);
}



size_t tc_pack_bytes(int oc, int kh, int kw, int c)
{
    if (oc <= 0 || kh <= 0 || kw <= 0) return 0;
    // prefix table, row-window weights of few-channel convolutions (widest window), fused-add table and its tag
    return add_lut_offset(oc, kh, kw, c) + TC_LUT_BYTES + 64;
}

size_t tc_scratch_bytes(const b200k_conv2d_params* p)
{
    if (!p || p->c > 16) return 0;
    // the direct stem kernel reads the input where it lies: no packed copy
    if (!p->add_operand.data && (p->w.scales || p->w.zero_point == 0) && p->selftest_us == 0 && stem_plan(p).ok) return 0;
    const RowPlan r = row_window_plan(p);
    return r.ok ? r.scratch_bytes : 0;
}

// The kernels below are launched the plain way (full stream dependency, no programmatic dependent launch) on purpose:
// conv_tc_kernel reads the prefix table, the re-packed weights and the fused-add table BEFORE its griddepcontrol.wait,
// which is only sound while whatever wrote them has completed when the convolution's grid starts.  A caller that
// packs and convolves back to back on one stream (b200k_conv2d_q8_static does) relies on that.
int tc_pack(const b200k_conv2d_params* p, void* packed, cudaStream_t stream)
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
    uint8_t* lut = (uint8_t*)packed + add_lut_offset(p->oc, p->kh, p->kw, p->c);
    if (p->add_operand.data && is_q8(p->add_operand.dtype) && is_q8(p->add_out.dtype) && is_q8(p->y.dtype)) {
        // table of the fused Add for exactly these quantisation parameters and this clamp
        AddLutArgs la;
        la.lut = lut;
        la.y_u8 = p->y.dtype == B200K_U8; la.res_u8 = p->add_operand.dtype == B200K_U8;
        la.sy = p->y.scale; la.zy = p->y.zero_point; la.sr = p->add_operand.scale; la.zr = p->add_operand.zero_point;
        la.out = make_requant(0.f, p->add_out, p->clamp_lo, p->clamp_hi);
        make_lut_tag(p, la.tag);
        add_lut_kernel<<<256, 256, 0, (cudaStream_t)stream>>>(la);
        rc = check_launch("add_lut_kernel");
        if (rc) return rc;
    } else {
        B200K_CUDA(cudaMemsetAsync(lut + TC_LUT_BYTES, 0, 64, (cudaStream_t)stream));      // no table: no tag
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
    rc = check_launch("row_weight_pack_kernel");
    if (rc) return rc;
    // the direct stem kernel's weights: pixels of 16 / stride_w bytes and, for stride 2 with at most four channels, of 4
    if (p->oc % 8 == 0 && (q.stride_w == 1 || q.stride_w == 2)) {
        for (int split = 0; split < 2 && rc == B200K_OK; ++split) {
            const int cpad = split ? 4 : 16 / q.stride_w;
            if (split && !(q.stride_w == 2 && p->c <= 4)) break;
            const int WB = (p->kw * cpad + 31) & ~31;
            if (p->c > cpad || WB > 128) continue;
            StemWeightArgs sa;
            sa.w = (const uint8_t*)p->w.data; sa.wpk = (uint8_t*)packed + stem_wpack_offset(p, split);
            sa.OC = p->oc; sa.KH = p->kh; sa.KW = p->kw; sa.C = p->c; sa.cpad = cpad; sa.WB = WB;
            stem_weight_pack_kernel<<<div_up((long long)p->kh * p->oc * WB, 256), 256, 0, (cudaStream_t)stream>>>(sa);
            rc = check_launch("stem_weight_pack_kernel");
        }
    }
    return rc;
}

// ---- int8 tensor-core ceiling ---------------------------------------------------------------------------------
//
// What the tcgen05 pipe can do when nothing else is in the way: every CTA (one per SM) issues kind::i8 MMAs of
// 128 x 256 x 32 back to back on one pair of shared-memory tiles (no loads, no epilogue), 64 per commit.  The result
// is the denominator for "fraction of the int8 tensor peak" figures measured on the same device and clocks.
struct PeakArgs { int rounds; long long wait_limit; int* status; };

__global__ void __launch_bounds__(128, 1) mma_peak_kernel(const PeakArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* s_a = smem;                                   // 128 rows x 128 bytes, 128-byte swizzle
    uint8_t* s_b = smem + 128 * 128;                       // 256 rows x 128 bytes
    uint64_t* bar = (uint64_t*)(s_b + 256 * 128);
    uint32_t* tmem_slot = (uint32_t*)(bar + 1);
    for (int i = threadIdx.x; i < (128 + 256) * 128 / 16; i += blockDim.x) ((uint4*)smem)[i] = make_uint4(0x01010101u, 0x02020202u, 0x01010101u, 0x02020202u);
    if (threadIdx.x == 0) { mbar_init(bar, 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const int warp = threadIdx.x >> 5;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    if (warp == 0) {
        const uint32_t id = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const uint64_t da = make_smem_desc<128>(smem_u32(s_a)), db = make_smem_desc<128>(smem_u32(s_b));
        bool alive = true;
        for (int r = 0; r < a.rounds && alive; ++r) {
            if (elect_one()) {
                #pragma unroll 1
                for (int i = 0; i < 16; ++i) {
                    #pragma unroll
                    for (int k = 0; k < 4; ++k) tc_mma_i8(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), id, (uint32_t)(r | i | k));
                }
                tc_commit(bar);
            }
            if (!__all_sync(0xffffffffu, mbar_wait(bar, (uint32_t)(r & 1), a.wait_limit))) { atomicExch(a.status, 1); alive = false; }
            tc_fence_after();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}

}  // namespace b200k

using namespace b200k;

extern "C" int b200k_int8_mma_peak(double* tops, void* stream_)
{
    B200K_REQUIRE(tops, B200K_E_INVALID, "int8_mma_peak: null output");
    cudaStream_t stream = (cudaStream_t)stream_;
    const int sms = sm_count(), rounds = 2000;
    const size_t smem = 1024 + (128 + 256) * 128 + 64;
    B200K_CUDA(cudaFuncSetAttribute(mma_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int* status = nullptr;
    B200K_CUDA(cudaMalloc(&status, sizeof(int)));
    B200K_CUDA(cudaMemsetAsync(status, 0, sizeof(int), stream));
    cudaEvent_t e0, e1;
    B200K_CUDA(cudaEventCreate(&e0));
    B200K_CUDA(cudaEventCreate(&e1));
    PeakArgs a;
    a.rounds = rounds; a.wait_limit = TC_WAIT_LIMIT_CYCLES; a.status = status;
    double best = 0.0;
    int rc = B200K_OK;
    for (int rep = 0; rep < 4 && rc == B200K_OK; ++rep) {          // the first repetition warms up
        cudaEventRecord(e0, stream);
        mma_peak_kernel<<<sms, 128, smem, stream>>>(a);
        cudaEventRecord(e1, stream);
        rc = check_launch("mma_peak_kernel");
        if (cudaEventSynchronize(e1) != cudaSuccess) { set_error("int8_mma_peak: %s", cudaGetErrorString(cudaGetLastError())); rc = B200K_E_CUDA; break; }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        const double ops = 2.0 * 128.0 * 256.0 * 32.0 * 64.0 * rounds * sms;
        if (rep > 0 && ms > 0.f && ops / (ms * 1e-3) / 1e12 > best) best = ops / (ms * 1e-3) / 1e12;
    }
    int st = 0;
    if (rc == B200K_OK) cudaMemcpy(&st, status, sizeof(int), cudaMemcpyDeviceToHost);
    cudaFree(status);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (rc != B200K_OK) return rc;
    B200K_REQUIRE(st == 0, B200K_E_TIMEOUT, "int8_mma_peak: a bounded wait gave up");
    *tops = best;
    return B200K_OK;
}

#ifdef B200K_TRACE
extern "C" int b200k_tc_trace(unsigned long long* out64)
{
    B200K_CUDA(cudaDeviceSynchronize());
    B200K_CUDA(cudaMemcpyFromSymbol(out64, g_tc_trace, sizeof(unsigned long long) * 64));
    return B200K_OK;
}
#endif

namespace b200k { int fc_stream_poll_status(); }

extern "C" int b200k_poll_status(void)
{
    int s = 0;
    const int fs = fc_stream_poll_status();
    if (fs != 0) {
        set_error("a bounded device-side wait of the weight-streaming FullyConnected kernel gave up (code %d: 1 producer/ring slot, "
                  "2 consumer/weights)", fs);
        return B200K_E_TIMEOUT;
    }
    B200K_CUDA(cudaMemcpyFromSymbol(&s, g_tc_status, sizeof(int)));
    if (s != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
        set_error("a bounded device-side wait gave up (code %d: 1 producer/ring, 2 MMA issuer/ring, 3 epilogue/accumulator, "
                  "4 MMA issuer/accumulator buffer, 5 epilogue/add operand, 6 producer/unit buffer, 7 MMA issuer/weights, 8 epilogue/add table)", s);
        return B200K_E_TIMEOUT;
    }
    return B200K_OK;
}
