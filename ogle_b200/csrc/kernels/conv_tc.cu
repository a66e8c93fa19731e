// tcgen05 tensor-core path for dense conv2d and gemm (placeholder until the
// TMA/TMEM pipeline lands: reports "not supported" so callers use CUDA cores).
#include "conv_args.cuh"

namespace ogle {

bool conv_tc_supported(const ConvArgs&, int) { return false; }
int launch_conv_tc(const ConvArgs&, int, int, const float*, const float*, const float*, const float*,
                   float*, cudaStream_t) { return OGLE_ERR_UNSUPPORTED; }
bool gemm_tc_supported(const OgleGemmParams&, const float*, const float*) { return false; }
int launch_gemm_tc(const OgleGemmParams&, const float*, const float*, const float*, float*, cudaStream_t) {
    return OGLE_ERR_UNSUPPORTED;
}

}  // namespace ogle
