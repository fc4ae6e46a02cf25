// Probe: what the single-thread roles of the tcgen05 convolution kernel pay per operation on this GPU.
//
//   issue_cost tma [MiB]   one thread per warp issues 2-D tiled TMA loads into a shared-memory ring (wait for the slot,
//                          arm its barrier, issue) under `if (lane == 0)`: ns per load and SM for several box sizes,
//                          ring depths and numbers of issuing warps
//   issue_cost mbar        cycles of mbarrier operations for one thread, and of a two-thread ring hand-over
//
// Every wait is bounded (a clock64 limit or an iteration count); nothing here can spin forever.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* b, int n)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(b)), "r"(n) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* b, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t a) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(a) : "memory"); }
__device__ __forceinline__ bool try_wait(uint32_t a, uint32_t ph)
{
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(a), "r"(ph) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool wait_bounded(uint32_t a, uint32_t ph)
{
    const long long t0 = clock64();
    while (!try_wait(a, ph)) { if (clock64() - t0 > 2000000000LL) return false; }
    return true;
}

// ---- TMA issue ------------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(128, 1) tma_kernel(const __grid_constant__ CUtensorMap map, int rows, int row_bytes, int stages,
                                                     int iters, int total_rows, int row_chunks, int* status)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const int warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const uint32_t box_bytes = (uint32_t)rows * row_bytes;
    uint64_t* bars = (uint64_t*)smem + warp * 16;
    uint8_t* ring = smem + 1024 + (size_t)warp * stages * box_bytes;
    if ((threadIdx.x & 31) == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(&bars[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if ((threadIdx.x & 31) == 0) {
        const int tiles = total_rows / rows;
        int t = blockIdx.x * nwarps + warp;
        iters /= nwarps;
        int st = 0; uint32_t ph = 0;
        for (int i = 0; i < iters + stages; ++i) {
            if (i >= stages && !wait_bounded(smem_u32(&bars[st]), ph)) { atomicExch(status, 1); break; }
            if (i < iters) {
                mbar_expect_tx(&bars[st], box_bytes);
                const int tile = t; t += gridDim.x * nwarps; if (t >= tiles) t -= tiles;
                const int xc = (i & (row_chunks - 1)) * row_bytes;
                asm volatile("cp.async.bulk.tensor.2d.shared::cta.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                             ::"r"(smem_u32(ring + (size_t)st * box_bytes)), "l"(&map), "r"(smem_u32(&bars[st])), "r"(xc), "r"(tile * rows) : "memory");
            }
            if (++st == stages) { st = 0; if (i >= stages) ph ^= 1u; }
        }
    }
}

static int run_tma(size_t mib)
{
    const size_t total_bytes = mib << 20;
    const int pitch = 256;
    const int total_rows = (int)(total_bytes / pitch);
    uint8_t* d; cudaMalloc(&d, total_bytes); cudaMemset(d, 1, total_bytes);
    int* status; cudaMalloc(&status, 4); cudaMemset(status, 0, 4);
    void* f = nullptr; cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || !f) { printf("no cuTensorMapEncodeTiled\n"); return 1; }
    auto encode = (PFN_cuTensorMapEncodeTiled_v12000)f;
    int sms = 0; cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
    cudaFuncSetAttribute(tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    printf("tensor %zu MiB, %d SMs; ns per TMA load per SM, aggregate GB/s\n", mib, sms);
    for (int nw = 1; nw <= 4; nw *= 2)
        for (int rb : {64, 128}) for (int rows : {32, 128, 256}) for (int stages : {1, 4, 8}) {
            const size_t smem = 1024 + (size_t)nw * stages * rows * rb;
            if (smem > 200 * 1024) continue;
            CUtensorMap map;
            cuuint64_t dims[2] = {(cuuint64_t)pitch, (cuuint64_t)total_rows};
            cuuint64_t strides[1] = {(cuuint64_t)pitch};
            cuuint32_t box[2] = {(cuuint32_t)rb, (cuuint32_t)rows};
            cuuint32_t estr[2] = {1, 1};
            if (encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, d, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                       rb == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) { printf("encode failed\n"); return 1; }
            const int iters = 4000;
            float best = 1e30f;
            for (int rep = 0; rep < 3; ++rep) {
                cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
                cudaEventRecord(e0);
                tma_kernel<<<sms, 32 * nw, smem>>>(map, rows, rb, stages, iters, total_rows, pitch / rb, status);
                cudaEventRecord(e1);
                if (cudaDeviceSynchronize() != cudaSuccess) { printf("kernel failed: %s\n", cudaGetErrorString(cudaGetLastError())); return 1; }
                float ms; cudaEventElapsedTime(&ms, e0, e1);
                if (ms < best) best = ms;
            }
            printf("issuing warps %d  box %3d B x %3d rows (%5d B)  in flight %d per warp : %7.1f ns per load  %7.0f GB/s\n",
                   nw, rb, rows, rows * rb, stages, best * 1e6 / iters, (double)sms * iters * rows * rb / (best * 1e-3) / 1e9);
        }
    int h = 0; cudaMemcpy(&h, status, 4, cudaMemcpyDeviceToHost);
    printf("timeouts: %d\n", h);
    return h;
}

// ---- mbarrier operations ----------------------------------------------------------------------------------------------

constexpr int N = 2000;

__global__ void __launch_bounds__(64) mbar_kernel(long long* results, int stages)
{
    __shared__ __align__(8) uint64_t full[16], empty[16], one;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int i = 0; i < 16; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(&one, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t a = smem_u32(&one);
        uint32_t acc = 0;
        long long t0 = clock64();
        for (int i = 0; i < N; ++i) acc += try_wait(a, 1);                 // a completed phase
        long long t1 = clock64(); results[0] = (t1 - t0) / N;
        t0 = clock64();
        for (int i = 0; i < N; ++i) mbar_arrive(a);                        // count 1: every arrive completes a phase
        t1 = clock64(); results[1] = (t1 - t0) / N;
        uint32_t ph = 0;
        t0 = clock64();
        for (int i = 0; i < N; ++i) { mbar_arrive(a); acc += wait_bounded(a, ph); ph ^= 1; }   // dependent pair
        t1 = clock64(); results[2] = (t1 - t0) / N;
        results[7] = acc;
    }
    __syncthreads();
    if (lane == 0) {                                                        // warp 0 produces, warp 1 consumes
        const uint32_t fa = smem_u32(full), ea = smem_u32(empty);
        int st = 0; uint32_t ph = 0; bool ok = true;
        const long long t0 = clock64();
        for (int i = 0; i < N * 4 && ok; ++i) {
            if (warp == 0) { ok = wait_bounded(ea + st * 8, ph ^ 1); mbar_arrive(fa + st * 8); }
            else           { ok = wait_bounded(fa + st * 8, ph);     mbar_arrive(ea + st * 8); }
            if (++st == stages) { st = 0; ph ^= 1; }
        }
        results[3 + warp] = ok ? (clock64() - t0) / (N * 4) : -1;
    }
}

static int run_mbar()
{
    long long* d; cudaMalloc(&d, 8 * sizeof(long long));
    for (int stages : {1, 4, 16}) {
        cudaMemset(d, 0, 8 * sizeof(long long));
        mbar_kernel<<<1, 64>>>(d, stages);
        if (cudaDeviceSynchronize() != cudaSuccess) { printf("failed: %s\n", cudaGetErrorString(cudaGetLastError())); return 1; }
        long long h[8]; cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost);
        printf("cycles: try_wait (complete) %lld, arrive %lld, arrive + wait on the same barrier %lld; "
               "two-thread ring of %2d stages: %lld per hand-over (producer), %lld (consumer)\n", h[0], h[1], h[2], stages, h[3], h[4]);
    }
    return 0;
}

int main(int argc, char** argv)
{
    if (argc >= 2 && !strcmp(argv[1], "tma")) return run_tma(argc >= 3 ? (size_t)atoll(argv[2]) : 64);
    if (argc >= 2 && !strcmp(argv[1], "mbar")) return run_mbar();
    printf("usage: issue_cost tma [MiB] | mbar\n");
    return 2;
}
