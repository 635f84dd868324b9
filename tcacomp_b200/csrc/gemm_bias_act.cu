// gemm_bias_act.cu -- placeholder until the tcgen05 contraction lands.
#include "common.cuh"
namespace tcab {
int launch_gemm_bias_act(const __nv_bfloat16*, const __nv_bfloat16*, const float*, int, __nv_bfloat16*, uint32_t,
                         uint32_t, uint32_t, cudaStream_t) {
  return fail(TCAB_ERR_UNSUPPORTED, "gemm_bias_act: not built yet");
}
}  // namespace tcab
