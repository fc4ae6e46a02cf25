// FullyConnected with at most 16 input rows: a weight-streaming kernel.
//
// With so few rows the layer is a read of the weight matrix ([N, K], K contiguous) and nothing else, so the kernel is
// built around keeping every SM's share of that read in flight: one persistent CTA per SM, a producer thread that
// streams units of R consecutive weight rows into a shared-memory ring with bulk copies (cp.async.bulk, completion on
// an mbarrier), and eight consumer warps that multiply a landed unit with the input rows, which stay in shared memory
// for the whole launch.  The weights do not depend on the kernel before this one in the stream, so under programmatic
// dependent launch the producer starts streaming before griddepcontrol.wait; only the staging of the input waits.
//
// Arithmetic: mma.sync m16n8k32 on 8-bit operands (the 16 rows of A are the input rows, the 8 columns of B are the
// unit's weight rows); tensor memory and tcgen05 have nothing to offer a 16 x 8 tile, and the kernel is bound by the
// weight stream, not by the multiply.  Every lane reads 16 contiguous bytes of an input row and of a weight row per
// pair of MMAs: the contraction does not care in which order K is walked as long as A and B agree, so the fragment's
// k-groups are assigned to whatever bytes a 128-bit load brings.  Row pitches are K + 64 bytes (64 modulo 128), which
// makes those loads conflict-free.  The eight warps take the 64-byte blocks of K round-robin and their partial
// 16 x 8 sums are added through shared memory.
//
// Zero points: sum (x - zx)(w - zw) = sum x w - zw sum x - zx sum w + K zx zw; sum x per input row is formed once per
// launch, sum w per weight row from the bytes each lane has loaded anyway (only when zx != 0).  The requantisation
// is requant_fast, the same function as in the other FullyConnected kernels.
//
// Every wait on an mbarrier is bounded: a wait that gives up raises a status word (b200k_poll_status) and the CTA
// drains and returns.
#include <atomic>
#include "common.cuh"

namespace b200k {

constexpr int FS_WARPS = 8;                          // consumer warps
constexpr int FS_THREADS = 32 * (FS_WARPS + 1);      // + the producer warp
constexpr int FS_MAX_STAGES = 16;
constexpr int FS_BATCH = 4;                          // units whose partial sums are added behind one barrier
constexpr int FS_TAB_UNITS = 32;                     // units per CTA whose per-channel constants are staged ahead of the wait
constexpr long long FS_WAIT_LIMIT_CYCLES = 4000000000ll;

__device__ int g_fs_status = 0;

struct FsArgs {
    const uint8_t* x; const uint8_t* w; const int32_t* bias; uint8_t* y; int32_t* acc_out;
    const float* w_scales; const float* b_scales;
    float w_scale, b_scale;
    int zx, zw, M, K, N;
    int R, stages, pitch, mp;                        // weight rows per unit, ring depth, row pitch in bytes, staged input rows (= M)
    float sx, sy, inv_sy, zy, lo, hi;
    long long wait_limit;
};

__device__ __forceinline__ uint32_t fs_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool fs_wait(uint64_t* bar, uint32_t parity, long long limit)
{
    const uint32_t addr = fs_smem_u32(bar);
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

__device__ __forceinline__ uint4 fs_lds128(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

template <bool XU, bool WU>
__device__ __forceinline__ void fs_mma(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    if (XU && WU)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else if (XU && !WU)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else if (!XU && WU)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void fs_consumer_barrier()
{
    asm volatile("bar.sync 1, %0;" ::"n"(32 * FS_WARPS) : "memory");
}

template <bool XU, bool WU>
__global__ void __launch_bounds__(FS_THREADS, 2) fc_stream_kernel(const FsArgs a)
{
    extern __shared__ __align__(128) uint8_t fs_smem[];
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    // [mp input rows][pitch] | ring [stages][R][pitch] | partial sums [FS_BATCH][FS_WARPS][M * 8] | weight-row sums [FS_BATCH][FS_WARPS][8]
    // | input-row sums [16] | barriers full[16], empty[16] | per-channel multiplier and bias term of the CTA's first
    // FS_TAB_UNITS units [2][FS_TAB_UNITS][8]
    uint8_t* s_x = fs_smem;
    uint8_t* s_ring = s_x + (size_t)a.mp * a.pitch;
    int* s_part = (int*)(s_ring + (size_t)a.stages * a.R * a.pitch);
    int* s_wpart = s_part + FS_BATCH * FS_WARPS * a.M * 8;
    int* s_xsum = s_wpart + FS_BATCH * FS_WARPS * 8;
    uint64_t* full = (uint64_t*)(s_xsum + 16);
    uint64_t* empty = full + FS_MAX_STAGES;
    float* s_mm = (float*)(empty + FS_MAX_STAGES);
    float* s_bb = s_mm + FS_TAB_UNITS * 8;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = (a.N + a.R - 1) / a.R;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fs_smem_u32(&full[s])), "r"(1) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(fs_smem_u32(&empty[s])), "r"(FS_WARPS) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == FS_WARPS) {
        // ===================== producer =====================
        if (lane == 0) {
            int s = 0; uint32_t ph = 0;
            for (int u = blockIdx.x; u < units; u += gridDim.x) {
                if (!fs_wait(&empty[s], ph ^ 1u, a.wait_limit)) { atomicExch(&g_fs_status, 1); break; }
                const int n0 = u * a.R;
                const int rows = min(a.R, a.N - n0);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(fs_smem_u32(&full[s])), "r"(rows * a.K) : "memory");
                for (int r = 0; r < rows; ++r) {
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                                 ::"r"(fs_smem_u32(s_ring + ((size_t)s * a.R + r) * a.pitch)), "l"(a.w + (size_t)(n0 + r) * a.K), "r"(a.K),
                                   "r"(fs_smem_u32(&full[s])) : "memory");
                }
                if (++s == a.stages) { s = 0; ph ^= 1u; }
            }
        }
        return;
    }

    // ===================== consumers =====================
    const int ctid = threadIdx.x;                                         // 0 .. 255
    // Scales and bias do not depend on the kernel before this one either: the requantisation constants of this CTA's
    // units are formed now, so that no global load sits between a unit's sums and its stores later on.
    for (int i = ctid; i < FS_TAB_UNITS * 8; i += 32 * FS_WARPS) {
        const int n = (blockIdx.x + (i >> 3) * gridDim.x) * a.R + (i & 7);
        if ((i & 7) < a.R && n < a.N) {
            s_mm[i] = __fmul_rn(a.sx, a.w_scales ? a.w_scales[n] : a.w_scale);
            s_bb[i] = a.bias ? __fmul_rn(__int2float_rn(a.bias[n]), a.b_scales ? a.b_scales[n] : a.b_scale) : 0.f;
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");                 // the input rows come from the kernel before this one
    {
        const int kv = a.K / 16;
        for (int i = ctid; i < a.mp * kv; i += 32 * FS_WARPS) {
            const int r = i / kv, c = i - r * kv;
            const uint4 v = *(const uint4*)(a.x + (size_t)r * a.K + c * 16);
            *(uint4*)(s_x + (size_t)r * a.pitch + c * 16) = v;
        }
        fs_consumer_barrier();
        // sum x per input row (rows warp and warp + 8)
        for (int r = warp; r < 16; r += FS_WARPS) {
            int sum = 0;
            if (a.zw != 0 && r < a.M) {
                for (int c = lane; c < kv; c += 32) {
                    const uint4 v = *(const uint4*)(s_x + (size_t)r * a.pitch + c * 16);
                    sum = dp4a_mixed<XU, true>(v.x, 0x01010101u, sum);
                    sum = dp4a_mixed<XU, true>(v.y, 0x01010101u, sum);
                    sum = dp4a_mixed<XU, true>(v.z, 0x01010101u, sum);
                    sum = dp4a_mixed<XU, true>(v.w, 0x01010101u, sum);
                }
                #pragma unroll
                for (int off = 16; off >= 1; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            }
            if (lane == 0) s_xsum[r] = sum;
        }
        fs_consumer_barrier();
    }
    const int g = lane >> 2, t = lane & 3;
    const uint32_t xa_addr = fs_smem_u32(s_x) + (uint32_t)(g * a.pitch + t * 16);
    const uint32_t xb_addr = xa_addr + (uint32_t)(8 * a.pitch);
    const bool row_a = g < a.M, row_b = g + 8 < a.M;        // fragment rows without an input row are zero
    const int nblk = a.K / 64;
    int s = 0; uint32_t ph = 0;
    bool dead = false;
    // The CTA's units are worked off in batches of FS_BATCH: every warp runs through its share of K for all units of
    // the batch without meeting the other warps (it only waits for the weights), then the partial sums of the whole
    // batch are added and requantised behind one barrier.  [unit of the batch][warp][input row][8 weight rows]
    const int my_units = units > (int)blockIdx.x ? (units - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    for (int base = 0; base < my_units; base += FS_BATCH) {
        const int nb = min(FS_BATCH, my_units - base);
        #pragma unroll
        for (int j = 0; j < FS_BATCH; ++j) {
            if (j >= nb) break;
            const int u = (int)blockIdx.x + (base + j) * (int)gridDim.x;
            const int rows = min(a.R, a.N - u * a.R);
            if (!dead && !fs_wait(&full[s], ph, a.wait_limit)) { atomicExch(&g_fs_status, 2); dead = true; }
            // four independent accumulator sets: consecutive MMAs do not wait for one another (a dependent mma.sync
            // chain, not the weight stream, would otherwise set the time per unit)
            int acc[4][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}};
            int wl = 0;                                      // this lane's share of sum w of weight row g
            const uint32_t w_addr = fs_smem_u32(s_ring) + (uint32_t)((s * a.R + g) * a.pitch + t * 16);
            if (!dead) {
                const bool wrow = g < rows;
                #pragma unroll 2
                for (int b = warp; b < nblk; b += 2 * FS_WARPS) {
                    const int b2 = b + FS_WARPS;
                    const bool second = b2 < nblk;
                    const uint4 xa0 = row_a ? fs_lds128(xa_addr + b * 64) : make_uint4(0, 0, 0, 0);
                    const uint4 xb0 = row_b ? fs_lds128(xb_addr + b * 64) : make_uint4(0, 0, 0, 0);
                    const uint4 wv0 = wrow ? fs_lds128(w_addr + b * 64) : make_uint4(0, 0, 0, 0);
                    const uint4 xa1 = (second && row_a) ? fs_lds128(xa_addr + b2 * 64) : make_uint4(0, 0, 0, 0);
                    const uint4 xb1 = (second && row_b) ? fs_lds128(xb_addr + b2 * 64) : make_uint4(0, 0, 0, 0);
                    const uint4 wv1 = (second && wrow) ? fs_lds128(w_addr + b2 * 64) : make_uint4(0, 0, 0, 0);
                    fs_mma<XU, WU>(acc[0], xa0.x, xb0.x, xa0.y, xb0.y, wv0.x, wv0.y);
                    fs_mma<XU, WU>(acc[1], xa0.z, xb0.z, xa0.w, xb0.w, wv0.z, wv0.w);
                    fs_mma<XU, WU>(acc[2], xa1.x, xb1.x, xa1.y, xb1.y, wv1.x, wv1.y);
                    fs_mma<XU, WU>(acc[3], xa1.z, xb1.z, xa1.w, xb1.w, wv1.z, wv1.w);
                    if (a.zx != 0) {
                        wl = dp4a_mixed<WU, true>(wv0.x, 0x01010101u, wl); wl = dp4a_mixed<WU, true>(wv0.y, 0x01010101u, wl);
                        wl = dp4a_mixed<WU, true>(wv0.z, 0x01010101u, wl); wl = dp4a_mixed<WU, true>(wv0.w, 0x01010101u, wl);
                        wl = dp4a_mixed<WU, true>(wv1.x, 0x01010101u, wl); wl = dp4a_mixed<WU, true>(wv1.y, 0x01010101u, wl);
                        wl = dp4a_mixed<WU, true>(wv1.z, 0x01010101u, wl); wl = dp4a_mixed<WU, true>(wv1.w, 0x01010101u, wl);
                    }
                }
            }
            #pragma unroll
            for (int c = 0; c < 4; ++c) acc[0][c] += acc[1][c] + acc[2][c] + acc[3][c];
            // sum w of row g: the four lanes of a group hold the four 16-byte columns
            wl += __shfl_xor_sync(0xffffffffu, wl, 1);
            wl += __shfl_xor_sync(0xffffffffu, wl, 2);
            // this warp has read its part of the stage
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(fs_smem_u32(&empty[s])) : "memory");
            if (++s == a.stages) { s = 0; ph ^= 1u; }
            // partial sums of this warp: C fragment (row g: columns 2t, 2t + 1; row g + 8 likewise); rows without an
            // input row are not kept
            int* part = s_part + (j * FS_WARPS + warp) * (a.M * 8);
            if (row_a) { part[g * 8 + 2 * t] = acc[0][0]; part[g * 8 + 2 * t + 1] = acc[0][1]; }
            if (row_b) { part[(g + 8) * 8 + 2 * t] = acc[0][2]; part[(g + 8) * 8 + 2 * t + 1] = acc[0][3]; }
            if (t == 0) s_wpart[(j * FS_WARPS + warp) * 8 + g] = wl;
        }
        fs_consumer_barrier();
        for (int o = ctid; o < nb * a.M * 8; o += 32 * FS_WARPS) {
            const int j = o / (a.M * 8), r = o - j * (a.M * 8);
            const int m = r >> 3, nl = r & 7;
            const int it = base + j;
            const int n0 = ((int)blockIdx.x + it * (int)gridDim.x) * a.R;
            const int rows = min(a.R, a.N - n0);
            int total = 0, ws = 0;
            #pragma unroll
            for (int w8 = 0; w8 < FS_WARPS; ++w8) {
                total += s_part[(j * FS_WARPS + w8) * (a.M * 8) + r];
                ws += s_wpart[(j * FS_WARPS + w8) * 8 + nl];
            }
            if (nl < rows && !dead) {
                const int n = n0 + nl;
                total = total - a.zw * s_xsum[m] - a.zx * ws + a.K * a.zx * a.zw;
                const long long oi = (long long)m * a.N + n;
                if (a.acc_out) a.acc_out[oi] = total;
                float mm, bb;
                if (it < FS_TAB_UNITS) {
                    mm = s_mm[it * 8 + nl]; bb = s_bb[it * 8 + nl];
                } else {
                    mm = __fmul_rn(a.sx, a.w_scales ? a.w_scales[n] : a.w_scale);
                    bb = a.bias ? __fmul_rn(__int2float_rn(a.bias[n]), a.b_scales ? a.b_scales[n] : a.b_scale) : 0.f;
                }
                a.y[oi] = (uint8_t)requant_fast(total, mm, bb, a.bias != nullptr, a.sy, a.inv_sy, a.zy, a.lo, a.hi);
            }
        }
        // the partial sums are overwritten by the next batch
        if (base + FS_BATCH < my_units) fs_consumer_barrier();
    }
}

bool fc_stream_eligible(const b200k_fc_params* p)
{
    if (!p->transpose_w || p->m < 1 || p->m > 16 || p->k < 64 || p->k % 64 != 0 || p->n < 1) return false;
    if (!p->x.data || !p->w.data || !p->y.data) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->w.dtype) || !is_q8(p->y.dtype)) return false;
    if (p->bias.data && p->bias.dtype != B200K_S32) return false;
    if (((((uintptr_t)p->x.data) | ((uintptr_t)p->w.data)) & 15) != 0) return false;
    if (p->w.scales && p->w.zero_point != 0) return false;
    // the input rows and at least two one-row stages must fit
    const size_t pitch = (size_t)p->k + 64;
    return (size_t)(p->m + 2) * pitch + 16 * 1024 <= 227 * 1024 && (long long)p->k * 255 * 255 < (1ll << 31);
}

int launch_fc_stream(const b200k_fc_params* p, cudaStream_t stream)
{
    static std::atomic<int> sm_count[64];
    static std::atomic<bool> configured[64][4];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) dev = 0;
    int sms = sm_count[dev].load(std::memory_order_acquire);
    if (sms == 0) {
        B200K_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        sm_count[dev].store(sms, std::memory_order_release);
    }
    FsArgs a;
    a.x = (const uint8_t*)p->x.data; a.w = (const uint8_t*)p->w.data; a.bias = (const int32_t*)p->bias.data;
    a.y = (uint8_t*)p->y.data; a.acc_out = p->acc_out;
    a.w_scales = p->w.scales; a.b_scales = p->bias.scales; a.w_scale = p->w.scale; a.b_scale = p->bias.scale;
    a.zx = p->x.zero_point; a.zw = p->w.scales ? 0 : p->w.zero_point;
    a.M = p->m; a.K = p->k; a.N = p->n;
    a.pitch = p->k + 64;
    a.mp = p->m;
    // Two CTAs fit an SM when each takes at most half of its shared memory: under programmatic dependent launch the
    // next layer's CTAs then become resident while this layer's are still computing and their producers stream weights
    // in the meantime, which hides the launch and the first loads' latency.  That only pays while each CTA still keeps
    // about 90 KB of weights in flight (an SM's share of the HBM bandwidth times the latency under load): with one or
    // two input rows, say.  Otherwise one CTA per SM with all of the shared memory.
    // Rows per unit (at most 8, the MMA's width): the fewest rounds of units over the SMs, each round costing a fixed
    // quarter of a microsecond (barrier, reduction, requantisation) plus the unit's share of the SM's 43 GB/s of HBM.
    const size_t fixed = (size_t)a.mp * a.pitch + (size_t)(FS_BATCH * FS_WARPS * a.mp * 8 + FS_BATCH * FS_WARPS * 8 + 16) * 4 + 2 * FS_MAX_STAGES * 8 + 128 +
                         2 * FS_TAB_UNITS * 8 * 4;
    const size_t budget = fixed + 90 * 1024 <= 112 * 1024 ? 112 * 1024 : 227 * 1024;
    a.R = 0;
    {
        double best = 1e30;
        for (int r = 1; r <= 8; r <<= 1) {
            if (fixed + (size_t)3 * r * a.pitch > budget && r > 1) break;
            if (fixed + (size_t)2 * r * a.pitch > budget) break;
            const long long u = (p->n + r - 1) / r;
            const double cost = (double)((u + sms - 1) / sms) * (0.25 + (double)r * p->k / 43.0e3);
            if (cost < best * 0.999) { best = cost; a.R = r; }
        }
    }
    B200K_REQUIRE(a.R > 0, B200K_E_TOOBIG, "fully_connected_q8: K = %d does not fit the streaming kernel", p->k);
    long long stages = (long long)((budget - fixed) / ((size_t)a.R * a.pitch));
    if (stages > FS_MAX_STAGES) stages = FS_MAX_STAGES;
    a.stages = (int)stages;
    const Requant rq = make_requant(p->x.scale, p->y, p->clamp_lo, p->clamp_hi);
    a.sx = rq.sx; a.sy = rq.sy; a.inv_sy = rn_reciprocal(p->y.scale); a.zy = (float)rq.zy;
    a.lo = fmaxf(rq.tlo, (float)rq.clo); a.hi = fminf(rq.thi, (float)rq.chi);
    a.wait_limit = FS_WAIT_LIMIT_CYCLES;
    const size_t smem = fixed + (size_t)a.stages * a.R * a.pitch;
    const int units = (p->n + a.R - 1) / a.R;
    const dim3 grid((unsigned)(units < sms ? units : sms));
    const bool xu = p->x.dtype == B200K_U8, wu = p->w.dtype == B200K_U8;
    #define B200K_FS_LAUNCH(XU, WU, IDX)                                                                              \
        do {                                                                                                          \
            if (!configured[dev][IDX].load(std::memory_order_acquire)) {                                              \
                B200K_CUDA(cudaFuncSetAttribute(fc_stream_kernel<XU, WU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)); \
                configured[dev][IDX].store(true, std::memory_order_release);                                          \
            }                                                                                                         \
            launch_pdl(fc_stream_kernel<XU, WU>, grid, dim3(FS_THREADS), smem, stream, a);                            \
        } while (0)
    if (xu) { if (wu) B200K_FS_LAUNCH(true, true, 0); else B200K_FS_LAUNCH(true, false, 1); }
    else    { if (wu) B200K_FS_LAUNCH(false, true, 2); else B200K_FS_LAUNCH(false, false, 3); }
    #undef B200K_FS_LAUNCH
    return check_launch("fc_stream_kernel");
}

// 0, or the code of the wait that gave up (1 producer / ring slot, 2 consumer / weights); resets the word
int fc_stream_poll_status()
{
    int s = 0;
    if (cudaMemcpyFromSymbol(&s, g_fs_status, sizeof(int)) != cudaSuccess) return 0;
    if (s != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_fs_status, &zero, sizeof(int));
    }
    return s;
}

}  // namespace b200k
