// BatchMatMul on the tensor cores: out[b] = X[b] (M x K) * Y[b] (K x N), 8-bit operands, int32 accumulation, the fp32
// requantisation of the reference (src/backends/reference/workloads/BatchMatMulImpl.cpp:15-139 of the Arm NN tree).
//
// Both operands of a BatchMatMul are activations that arrive in whatever layout the graph has: [M, K] or (transpose_x)
// [K, M], [K, N] or (transpose_y) [N, K], with no load-time pass in which to re-pack them and no scratch memory in the
// entry point's contract.  The tensor-memory pipeline of the convolution kernel wants both operands K-contiguous; this
// kernel takes either layout as it is: a 128 x 128 tile per CTA, K in steps of 64 bytes, mma.sync m16n8k32 on int8.
//
// An operand that is K-contiguous in memory is staged as [row][k] (pitch 80 bytes) and a lane reads its fragment words
// directly.  An operand that is contiguous along M (or N) is staged as it lies, [k][m] (pitch 136 bytes): a lane reads
// the words that hold four consecutive m at four consecutive k and transposes the 4 x 4 bytes in registers, which gives
// it one fragment register for each of four m-tiles, provided the tiles' rows are assigned as row = 4 g + tile instead of
// 16 tile + g.  A matrix product does not care which rows an MMA tile holds as long as the epilogue writes each
// accumulator where its row belongs, so the assignment is simply different for that layout.  Both pitches make the
// fragment loads conflict-free.
//
// Zero points: sum (x - zx)(y - zy) = sum x y - zy sum_k x - zx sum_k y + K zx zy.  The row sums of X and column sums of
// Y come from MMAs against an all-ones operand (one per tile and step instead of sixteen), issued only for a non-zero
// zero point.
#include "common.cuh"

namespace b200k {

constexpr int BM_T = 128, BM_K = 64;                 // tile edge (both M and N), K step in bytes
constexpr int BM_THREADS = 256;
constexpr int BM_PITCH_K = 80;                       // [row][k] staging: 20 words, rows g = 0..7 land on distinct banks
constexpr int BM_PITCH_MN = 136;                     // [k][mn] staging: 34 words, k rows 4 apart land 8 banks apart

struct BmmTcArgs {
    const uint8_t* x; const uint8_t* y; uint8_t* out; int32_t* acc_out;
    int zx, zy, B, M, K, N;
    long long bsx, bsy;
    float m, sy, inv_sy, fzy, lo, hi;                // requant_fast: sx * sy(operand), output scale, RN(1 / scale), offset, clamp
};

template <bool AU, bool BU>
__device__ __forceinline__ void bm_mma(int* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    if (AU && BU)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else if (AU && !BU)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else if (!AU && BU)
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// w[j] = four consecutive rows' bytes at k + j  ->  o[i] = row i's bytes at k .. k + 3
__device__ __forceinline__ void bm_transpose4(const uint32_t* w, uint32_t* o)
{
    const uint32_t t0 = __byte_perm(w[0], w[1], 0x5140), t1 = __byte_perm(w[2], w[3], 0x5140);
    const uint32_t t2 = __byte_perm(w[0], w[1], 0x7362), t3 = __byte_perm(w[2], w[3], 0x7362);
    o[0] = __byte_perm(t0, t1, 0x5410); o[1] = __byte_perm(t0, t1, 0x7632);
    o[2] = __byte_perm(t2, t3, 0x5410); o[3] = __byte_perm(t2, t3, 0x7632);
}

// One operand's 128 x 64 tile from global memory into registers (two 16-byte pieces per thread), zero beyond the
// matrix.  KC: the operand is K-contiguous (element (r, k) at r * ld + k, ld = K); otherwise (k, r) at k * ld + r.
template <bool KC>
__device__ __forceinline__ void bm_fetch(const uint8_t* base, int ld, int r0, int rows, int k0, int K, bool vec_ok, uint4* v)
{
    #pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int idx = threadIdx.x + i * BM_THREADS;        // 512 pieces
        int r, k;
        if (KC) { r = r0 + (idx >> 2); k = k0 + (idx & 3) * 16; }          // 4 pieces per row
        else    { k = k0 + (idx >> 3); r = r0 + (idx & 7) * 16; }          // 8 pieces per k
        uint4 q = make_uint4(0, 0, 0, 0);
        const int rlim = KC ? rows : K, clim = KC ? K : rows;               // bound of the slow / the contiguous index
        const int slow = KC ? r : k, fast = KC ? k : r;
        if (slow < rlim && fast < clim) {
            const uint8_t* p = base + (long long)slow * ld + fast;
            if (vec_ok && fast + 16 <= clim) {
                q = *(const uint4*)p;
            } else {
                uint32_t w[4] = {0, 0, 0, 0};
                for (int e = 0; e < 16 && fast + e < clim; ++e) w[e >> 2] |= (uint32_t)p[e] << (8 * (e & 3));
                q = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        v[i] = q;
    }
}

template <bool KC>
__device__ __forceinline__ void bm_stage(uint8_t* s, const uint4* v)
{
    #pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int idx = threadIdx.x + i * BM_THREADS;
        if (KC) {
            *(uint4*)(s + (idx >> 2) * BM_PITCH_K + (idx & 3) * 16) = v[i];
        } else {
            uint8_t* d = s + (idx >> 3) * BM_PITCH_MN + (idx & 7) * 16;    // 8-byte aligned (136 = 17 * 8)
            *(uint2*)d = make_uint2(v[i].x, v[i].y);
            *(uint2*)(d + 8) = make_uint2(v[i].z, v[i].w);
        }
    }
}

// TX / TY: the operand is stored transposed with respect to the K-contiguous form the MMA wants, i.e. X as [K, M]
// (transpose_x) and Y as [K, N] (no transpose_y).
template <bool TX, bool TY, bool XU, bool YU>
__global__ void __launch_bounds__(BM_THREADS) bmm_mma_kernel(const BmmTcArgs a)
{
    __shared__ __align__(16) uint8_t s_a[TX ? BM_K * BM_PITCH_MN : BM_T * BM_PITCH_K];
    __shared__ __align__(16) uint8_t s_b[TY ? BM_K * BM_PITCH_MN : BM_T * BM_PITCH_K];
    pdl_enter();
    const int b = blockIdx.z, m0 = blockIdx.y * BM_T, n0 = blockIdx.x * BM_T;
    const uint8_t* xb = a.x + (long long)b * a.bsx;
    const uint8_t* yb = a.y + (long long)b * a.bsy;
    const int ldx = TX ? a.M : a.K, ldy = TY ? a.N : a.K;
    const bool vx = (((uintptr_t)xb | (uintptr_t)ldx) & 15) == 0, vy = (((uintptr_t)yb | (uintptr_t)ldy) & 15) == 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp >> 2, wn = warp & 3;                 // warp tile: rows wm * 64 .. + 64, columns wn * 32 .. + 32

    int acc[4][4][4];
    int rsum[4][4], csum[4][4];                              // ones-MMAs: [m-tile] rows g / g + 8 in c0 / c2; [n-tile] columns 2t, 2t + 1 in c0, c1
    #pragma unroll
    for (int i = 0; i < 4; ++i)
        #pragma unroll
        for (int j = 0; j < 4; ++j) {
            rsum[i][j] = 0; csum[i][j] = 0;
            #pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0;
        }

    uint4 va[2], vb[2];
    bm_fetch<!TX>(xb, ldx, m0, a.M, 0, a.K, vx, va);
    bm_fetch<!TY>(yb, ldy, n0, a.N, 0, a.K, vy, vb);
    for (int k0 = 0; k0 < a.K; k0 += BM_K) {
        __syncthreads();                                     // the previous step's fragment loads are done
        bm_stage<!TX>(s_a, va);
        bm_stage<!TY>(s_b, vb);
        __syncthreads();
        if (k0 + BM_K < a.K) {                               // the next step's global loads fly during this step's MMAs
            bm_fetch<!TX>(xb, ldx, m0, a.M, k0 + BM_K, a.K, vx, va);
            bm_fetch<!TY>(yb, ldy, n0, a.N, k0 + BM_K, a.K, vy, vb);
        }
        #pragma unroll
        for (int ks = 0; ks < 2; ++ks) {
            uint32_t fa[4][4], fb[4][2];                     // [tile][register]
            if (!TX) {
                #pragma unroll
                for (int mi = 0; mi < 4; ++mi) {
                    const uint8_t* p = s_a + (wm * 64 + mi * 16 + g) * BM_PITCH_K + ks * 32 + 4 * t;
                    fa[mi][0] = *(const uint32_t*)p;                       fa[mi][1] = *(const uint32_t*)(p + 8 * BM_PITCH_K);
                    fa[mi][2] = *(const uint32_t*)(p + 16);                fa[mi][3] = *(const uint32_t*)(p + 8 * BM_PITCH_K + 16);
                }
            } else {
                // rows of tile mi: 4 g + mi (fragment rows g) and 32 + 4 g + mi (fragment rows g + 8)
                #pragma unroll
                for (int half = 0; half < 2; ++half)
                    #pragma unroll
                    for (int kh = 0; kh < 2; ++kh) {
                        uint32_t w[4], o[4];
                        #pragma unroll
                        for (int j = 0; j < 4; ++j)
                            w[j] = *(const uint32_t*)(s_a + (ks * 32 + kh * 16 + 4 * t + j) * BM_PITCH_MN + wm * 64 + half * 32 + 4 * g);
                        bm_transpose4(w, o);
                        #pragma unroll
                        for (int mi = 0; mi < 4; ++mi) fa[mi][kh * 2 + half] = o[mi];
                    }
            }
            if (!TY) {
                #pragma unroll
                for (int ni = 0; ni < 4; ++ni) {
                    const uint8_t* p = s_b + (wn * 32 + ni * 8 + g) * BM_PITCH_K + ks * 32 + 4 * t;
                    fb[ni][0] = *(const uint32_t*)p; fb[ni][1] = *(const uint32_t*)(p + 16);
                }
            } else {
                // columns of tile ni: 4 g + ni
                #pragma unroll
                for (int kh = 0; kh < 2; ++kh) {
                    uint32_t w[4], o[4];
                    #pragma unroll
                    for (int j = 0; j < 4; ++j)
                        w[j] = *(const uint32_t*)(s_b + (ks * 32 + kh * 16 + 4 * t + j) * BM_PITCH_MN + wn * 32 + 4 * g);
                    bm_transpose4(w, o);
                    #pragma unroll
                    for (int ni = 0; ni < 4; ++ni) fb[ni][kh] = o[ni];
                }
            }
            #pragma unroll
            for (int mi = 0; mi < 4; ++mi)
                #pragma unroll
                for (int ni = 0; ni < 4; ++ni)
                    bm_mma<XU, YU>(acc[mi][ni], fa[mi][0], fa[mi][1], fa[mi][2], fa[mi][3], fb[ni][0], fb[ni][1]);
            if (a.zy != 0) {
                #pragma unroll
                for (int mi = 0; mi < 4; ++mi) bm_mma<XU, YU>(rsum[mi], fa[mi][0], fa[mi][1], fa[mi][2], fa[mi][3], 0x01010101u, 0x01010101u);
            }
            if (a.zx != 0) {
                #pragma unroll
                for (int ni = 0; ni < 4; ++ni) bm_mma<XU, YU>(csum[ni], 0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u, fb[ni][0], fb[ni][1]);
            }
        }
    }

    const int kzz = a.K * a.zx * a.zy;
    #pragma unroll
    for (int mi = 0; mi < 4; ++mi)
        #pragma unroll
        for (int ni = 0; ni < 4; ++ni)
            #pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int fr = g + (e >> 1) * 8, fc = 2 * t + (e & 1);        // fragment row (0..15) and column (0..7)
                const int row = TX ? (fr >> 3) * 32 + 4 * (fr & 7) + mi : mi * 16 + fr;
                const int col = TY ? 4 * fc + ni : ni * 8 + fc;
                const int m = m0 + wm * 64 + row, n = n0 + wn * 32 + col;
                if (m >= a.M || n >= a.N) continue;
                const int total = acc[mi][ni][e] - a.zy * rsum[mi][(e >> 1) * 2] - a.zx * csum[ni][e & 1] + kzz;
                const long long o = ((long long)b * a.M + m) * a.N + n;
                if (a.acc_out) a.acc_out[o] = total;
                a.out[o] = (uint8_t)requant_fast(total, a.m, 0.f, false, a.sy, a.inv_sy, a.fzy, a.lo, a.hi);
            }
}

bool bmm_mma_eligible(const b200k_bmm_params* p)
{
    if (!p->x.data || !p->y.data || !p->out.data) return false;
    if (!is_q8(p->x.dtype) || !is_q8(p->y.dtype) || !is_q8(p->out.dtype)) return false;
    if (p->batch < 1 || p->batch > 65535 || p->m < 1 || p->k < 1 || p->n < 1) return false;
    if ((p->m + BM_T - 1) / BM_T > 65535) return false;
    // (the int32 accumulator of the reference and of the generic kernel has the same range)
    return true;
}

int launch_bmm_mma(const b200k_bmm_params* p, cudaStream_t stream)
{
    BmmTcArgs a;
    a.x = (const uint8_t*)p->x.data; a.y = (const uint8_t*)p->y.data; a.out = (uint8_t*)p->out.data; a.acc_out = p->acc_out;
    a.zx = p->x.zero_point; a.zy = p->y.zero_point;
    a.B = p->batch; a.M = p->m; a.K = p->k; a.N = p->n;
    a.bsx = p->batch_stride_x; a.bsy = p->batch_stride_y;
    int lo, hi;
    type_range(p->out.dtype, lo, hi);
    // v = float(acc) * fl(sx * sy): the multiplier is formed once here with the same single rounding as on the device
    a.m = p->x.scale * p->y.scale;
    a.sy = p->out.scale; a.inv_sy = rn_reciprocal(p->out.scale); a.fzy = (float)p->out.zero_point;
    a.lo = (float)lo; a.hi = (float)hi;
    const dim3 grid((unsigned)((p->n + BM_T - 1) / BM_T), (unsigned)((p->m + BM_T - 1) / BM_T), (unsigned)p->batch);
    const bool tx = p->transpose_x != 0, ty = p->transpose_y == 0;       // "transposed" = not K-contiguous
    const bool xu = p->x.dtype == B200K_U8, yu = p->y.dtype == B200K_U8;
    #define B200K_BMM_TYPES(TX, TY)                                                                                    \
        do {                                                                                                           \
            if (xu) { if (yu) launch_pdl(bmm_mma_kernel<TX, TY, true, true>, grid, dim3(BM_THREADS), 0, stream, a);     \
                      else    launch_pdl(bmm_mma_kernel<TX, TY, true, false>, grid, dim3(BM_THREADS), 0, stream, a); }  \
            else    { if (yu) launch_pdl(bmm_mma_kernel<TX, TY, false, true>, grid, dim3(BM_THREADS), 0, stream, a);    \
                      else    launch_pdl(bmm_mma_kernel<TX, TY, false, false>, grid, dim3(BM_THREADS), 0, stream, a); } \
        } while (0)
    if (tx) { if (ty) B200K_BMM_TYPES(true, true); else B200K_BMM_TYPES(true, false); }
    else    { if (ty) B200K_BMM_TYPES(false, true); else B200K_BMM_TYPES(false, false); }
    #undef B200K_BMM_TYPES
    return check_launch("bmm_mma_kernel");
}

}  // namespace b200k
