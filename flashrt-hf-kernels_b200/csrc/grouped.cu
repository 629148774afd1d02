// Grouped (MoE) NVFP4 GEMM entry points: argument checks, then the CTA-pair
// kernel in its grouped form (gemm_pair.cuh) driven by a device-built work list.
#include "common.cuh"

namespace frt {
int64_t grouped_max_items(int rows, int experts);
int run_grouped(const void* a, const void* sfa, const void* b_stack, const void* sfb_stack, const void* alpha,
                const void* offsets, const void* tile_expert, int tile_rows, void* out, int rows, int N, int K,
                int experts, int64_t b_stride, int64_t sfb_stride, void* workspace, cudaStream_t st);
}  // namespace frt

using namespace frt;

extern "C" {

int64_t frt_nvfp4_grouped_gemm_workspace_bytes(int rows, int num_experts) {
  if (rows <= 0 || num_experts <= 0) return 0;
  return 16 + 32 * grouped_max_items(rows, num_experts);
}

int frt_nvfp4_grouped_gemm_bf16(const void* a_packed, const void* sfa, const void* b_stack, const void* sfb_stack,
                                const void* alpha, const void* expert_offsets, const void* tile_expert, int tile_rows,
                                void* out, int rows, int N, int K, int num_experts, int64_t b_stride,
                                int64_t sfb_stride, void* work, void* stream) {
  if (!a_packed || !sfa || !b_stack || !sfb_stack || !alpha || !out || !work) return FRT_E_NULL;
  if ((expert_offsets == nullptr) == (tile_expert == nullptr)) return FRT_E_NULL;   // exactly one description
  if (rows <= 0 || N <= 0 || K <= 0 || num_experts <= 0 || K % 64 != 0 || N % 8 != 0) return FRT_E_SHAPE;
  if (tile_expert && tile_rows != 16 && tile_rows != 64) return FRT_E_SHAPE;
  if (tile_expert && rows % tile_rows != 0) return FRT_E_SHAPE;
  if (b_stride < static_cast<int64_t>(N) * (K / 2) || b_stride % 16 != 0) return FRT_E_SHAPE;
  if (sfb_stride < frt_nvfp4_sf_swizzled_bytes(N, K) || sfb_stride % 16 != 0) return FRT_E_SHAPE;
  if (!aligned(a_packed, 16) || !aligned(b_stack, 16) || !aligned(sfa, 16) || !aligned(sfb_stack, 16) ||
      !aligned(work, 16) || !aligned(out, 2))
    return FRT_E_ALIGN;
  return run_grouped(a_packed, sfa, b_stack, sfb_stack, alpha, expert_offsets, tile_expert,
                     tile_expert ? tile_rows : 0, out, rows, N, K, num_experts, b_stride, sfb_stride, work,
                     as_stream(stream));
}

}  // extern "C"
