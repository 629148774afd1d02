// Grouped (MoE) NVFP4 GEMM entry points.
#include "common.cuh"

extern "C" {

int64_t frt_nvfp4_grouped_gemm_workspace_bytes(int rows, int num_experts) {
  (void)rows; (void)num_experts;
  return 0;
}

int frt_nvfp4_grouped_gemm_bf16(const void*, const void*, const void*, const void*, const void*, const void*,
                                const void*, int, void*, int, int, int, int, int64_t, int64_t, void*, void*) {
  return FRT_E_UNSUPPORTED;
}

}  // extern "C"
