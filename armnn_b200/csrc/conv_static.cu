// b200k_conv2d_q8_static: Convolution2d for callers that cannot allocate device memory.
//
// The ordinary entry point wants two caller-provided device buffers besides the tensors: the load-time weight
// table (b200k_conv2d_pack) and, for few-channel convolutions, a per-call scratch for the re-packed input.  Some
// hosts of this library cannot supply them: a backend workload created inside an inference server whose memory
// pool is sized and frozen before any model is loaded, code running under a memory manager that forbids
// cudaMalloc after start-up, or a CUDA-graph replay path that must not touch the allocator.  For those this
// file keeps both buffers in one file-scope device array of fixed size.  The price is the size limit below and the
// fact that all calls share the array.
#include <mutex>
#include "common.cuh"

namespace b200k {
int conv2d_dispatch(const b200k_conv2d_params* p, cudaStream_t stream);
int conv2d_pack_impl(const b200k_conv2d_params* p, void* packed, cudaStream_t s, bool host_tables);
}

using namespace b200k;

// 16 MiB per process and GPU, resident from the moment the library is loaded on a device until the process exits:
// the first 1 MiB holds the weight table of the current call, the rest the re-packed input.
#define B200K_STATIC_TABLE_BYTES   (1u << 20)
#define B200K_STATIC_SCRATCH_BYTES (16u << 20)

static __device__ __align__(256) unsigned char g_static_scratch[B200K_STATIC_SCRATCH_BYTES];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address; the address a kernel can
// use comes from cudaGetSymbolAddress, asked once per device with that device current.
static int static_scratch_address(unsigned char** out)
{
    static std::mutex mu;
    static unsigned char* per_device[64] = {nullptr};
    int dev = -1;
    B200K_CUDA(cudaGetDevice(&dev));
    B200K_REQUIRE(dev >= 0 && dev < 64, B200K_E_INVALID, "conv2d_q8_static: device index %d not supported", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!per_device[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            set_error("conv2d_q8_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return B200K_E_CUDA;
        }
        per_device[dev] = (unsigned char*)ptr;
    }
    *out = per_device[dev];
    return B200K_OK;
}

extern "C" int b200k_conv2d_q8_static(const b200k_conv2d_params* p, void* stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "conv2d_q8_static: null params");
    B200K_REQUIRE(p->w.data && p->oc > 0 && p->kh > 0 && p->kw > 0 && p->c > 0, B200K_E_INVALID,
                  "conv2d_q8_static: weights / geometry missing");
    const size_t table = b200k_conv2d_pack_bytes(p->oc, p->kh, p->kw, p->c);
    const size_t scratch = b200k_conv2d_scratch_bytes(p);
    B200K_REQUIRE(table <= B200K_STATIC_TABLE_BYTES, B200K_E_TOOBIG,
                  "conv2d_q8_static: weight table of %zu bytes exceeds the built-in %u bytes", table, B200K_STATIC_TABLE_BYTES);
    B200K_REQUIRE(scratch <= B200K_STATIC_SCRATCH_BYTES - B200K_STATIC_TABLE_BYTES, B200K_E_TOOBIG,
                  "conv2d_q8_static: input scratch of %zu bytes exceeds the built-in %u bytes", scratch,
                  B200K_STATIC_SCRATCH_BYTES - B200K_STATIC_TABLE_BYTES);
    unsigned char* base = nullptr;
    int rc = static_scratch_address(&base);
    if (rc) return rc;
    b200k_conv2d_params q = *p;
    q.packed = base;
    q.scratch = scratch ? base + B200K_STATIC_TABLE_BYTES : nullptr;
    q.scratch_bytes = scratch;
    // Both regions are overwritten in full before they are read (the table by the pack kernels below, the input
    // region by the convolution's own re-pack), so nothing left over from an earlier call can leak into this one.
    // The pack kernels are ordinary launches: they have completed before the convolution's grid starts, which reads
    // the tables ahead of its programmatic-dependency wait (see tc_pack).
    // (device-side tables only: nothing here may wait for the stream)
    rc = conv2d_pack_impl(&q, base, (cudaStream_t)stream, false);
    if (rc) return rc;
    return conv2d_dispatch(&q, (cudaStream_t)stream);
}
