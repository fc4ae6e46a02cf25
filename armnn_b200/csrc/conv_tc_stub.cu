#include "common.cuh"
namespace b200k {
bool conv_tc_eligible(const b200k_conv2d_params*) { return false; }
int launch_conv_tc(const b200k_conv2d_params*, cudaStream_t) { set_error("tcgen05 path not built"); return B200K_E_UNSUPPORTED; }
}
extern "C" size_t b200k_conv2d_pack_bytes(int32_t, int32_t, int32_t, int32_t) { return 0; }
extern "C" int b200k_conv2d_pack(const b200k_conv2d_params*, void*, void*) { return B200K_E_UNSUPPORTED; }
