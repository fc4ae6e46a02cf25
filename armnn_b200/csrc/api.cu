// Device management and host-only helpers of the libb200k C ABI.
#include <math.h>
#include <stdarg.h>
#include <string.h>
#include <atomic>
#include "common.cuh"

namespace b200k {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

}  // namespace b200k

using namespace b200k;

extern "C" const char* b200k_last_error(void) { return g_err; }

extern "C" unsigned long long b200k_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" const char* b200k_version(void) { return "b200k 0.1 (sm_100a)"; }

extern "C" int b200k_device_count(void)
{
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

extern "C" int b200k_device_open(int device)
{
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        set_error("no CUDA device visible (%s)", e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
        return B200K_E_NODEVICE;
    }
    B200K_REQUIRE(device >= 0 && device < n, B200K_E_INVALID, "DeviceId %d out of range [0,%d)", device, n);
    cudaDeviceProp prop;
    B200K_CUDA(cudaGetDeviceProperties(&prop, device));
    B200K_REQUIRE(prop.major == 10, B200K_E_NODEVICE,
                  "device %d (%s) is sm_%d%d; libb200k is built for sm_100a only", device, prop.name,
                  prop.major, prop.minor);
    B200K_CUDA(cudaSetDevice(device));
    return B200K_OK;
}

// Quantize(0), Quantize(a), Quantize(b) on the host, same formula as the device epilogue.
static int quantize_host(float v, float scale, int zp, int lo, int hi)
{
    volatile float d = v / scale;
    float q = (float)zp + roundf(d);
    q = fminf(fmaxf(q, (float)lo), (float)hi);
    return (int)q;
}

extern "C" int b200k_activation_clamp(int kind, float a, float b, float scale, int32_t zero_point,
                                      int32_t dtype, int32_t* clamp_lo, int32_t* clamp_hi)
{
    B200K_REQUIRE(clamp_lo && clamp_hi, B200K_E_INVALID, "activation_clamp: null output");
    B200K_REQUIRE(dtype == B200K_U8 || dtype == B200K_S8 || dtype == B200K_S16, B200K_E_INVALID,
                  "activation_clamp: dtype %d is not quantised", dtype);
    int lo, hi;
    type_range(dtype, lo, hi);
    if (kind == 1) {
        int q0 = quantize_host(0.0f, scale, zero_point, lo, hi);
        if (q0 > lo) lo = q0;
    } else if (kind == 2) {
        int qb = quantize_host(b, scale, zero_point, lo, hi);
        int qa = quantize_host(a, scale, zero_point, lo, hi);
        if (qb > lo) lo = qb;
        if (qa < hi) hi = qa;
    } else {
        B200K_REQUIRE(kind == 0, B200K_E_INVALID, "activation_clamp: kind %d not in {0,1,2}", kind);
    }
    *clamp_lo = lo;
    *clamp_hi = hi;
    return B200K_OK;
}

// Size of each parameter struct as this library was compiled, so that a binding in another language can
// check its own declaration of the struct against the header it was written from.
extern "C" size_t b200k_sizeof_params(int which)
{
    switch (which) {
        case 0: return sizeof(b200k_conv2d_params);
        case 1: return sizeof(b200k_fc_params);
        case 2: return sizeof(b200k_bmm_params);
        case 3: return sizeof(b200k_pool2d_params);
        case 4: return sizeof(b200k_mean_params);
        case 5: return sizeof(b200k_eltwise_params);
        case 6: return sizeof(b200k_activation_params);
        case 7: return sizeof(b200k_softmax_params);
        case 8: return sizeof(b200k_convert_params);
        case 9: return sizeof(b200k_qlstm_params);
        case 10: return sizeof(b200k_pad_params);
        case 11: return sizeof(b200k_view_copy_params);
        case 12: return sizeof(b200k_resize_params);
        case 13: return sizeof(b200k_reduce_params);
        case 14: return sizeof(b200k_unary_params);
        case 15: return sizeof(b200k_arg_min_max_params);
        case 16: return sizeof(b200k_gather_params);
        case 17: return sizeof(b200k_batch_norm_params);
        case 18: return sizeof(b200k_instance_norm_params);
        case 19: return sizeof(b200k_normalization_params);
        case 20: return sizeof(b200k_conv3d_params);
        case 21: return sizeof(b200k_pool3d_params);
        case 22: return sizeof(b200k_gather_nd_params);
        case 23: return sizeof(b200k_lstm_params);
        case 24: return sizeof(b200k_reverse_params);
        case 25: return sizeof(b200k_convert_fp16_params);
        case 26: return sizeof(b200k_scatter_nd_params);
        default: return 0;
    }
}
