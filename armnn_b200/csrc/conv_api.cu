// Convolution2d entry point: argument checks and the choice between the tcgen05 implicit-GEMM kernel
// and the shape-agnostic CUDA-core kernel.
#include <string.h>
#include "common.cuh"

namespace b200k {

int launch_conv_dp4a(const b200k_conv2d_params* p, cudaStream_t stream);
int launch_conv_tc(const b200k_conv2d_params* p, cudaStream_t stream);      // B200K_E_UNSUPPORTED if not eligible
bool conv_tc_eligible(const b200k_conv2d_params* p);

int conv2d_dispatch(const b200k_conv2d_params* p, cudaStream_t stream)
{
    B200K_REQUIRE(p, B200K_E_INVALID, "conv2d_q8: null params");
    B200K_REQUIRE(p->algo >= 0 && p->algo <= 2, B200K_E_INVALID, "conv2d_q8: algo %d not in {0,1,2}", p->algo);
    if (p->algo == 2) {
        B200K_REQUIRE(conv_tc_eligible(p), B200K_E_UNSUPPORTED,
                      "conv2d_q8: shape/alignment not eligible for the tcgen05 kernel");
        return launch_conv_tc(p, stream);
    }
    if (p->algo == 0 && conv_tc_eligible(p)) return launch_conv_tc(p, stream);
    return launch_conv_dp4a(p, stream);
}

}  // namespace b200k

extern "C" int b200k_conv2d_q8(const b200k_conv2d_params* p, void* stream)
{
    return b200k::conv2d_dispatch(p, (cudaStream_t)stream);
}
