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

namespace {

// Work-list storage for the entry point that allocates nothing.  It is part of
// the library image: every GPU that loads the library carries these bytes until
// the process exits.  Sized for FRT_GROUPED_STATIC_MAX_ROWS rows and
// FRT_GROUPED_STATIC_MAX_EXPERTS experts (16 + 32 * (rows/16 + 2*experts + 8) = 393,488 bytes).
constexpr int64_t kStaticScratchBytes =
    16 + 32 * (FRT_GROUPED_STATIC_MAX_ROWS / 16 + 2ll * FRT_GROUPED_STATIC_MAX_EXPERTS + 8);
static __device__ __align__(256) unsigned char g_grouped_static_scratch[kStaticScratchBytes];

// In host code the array's name is only a handle for the runtime, not a device
// address; the address each device gave the array is looked up once per device.
void* g_static_scratch_ptr[64] = {};
std::atomic<bool> g_static_scratch_ready[64] = {};

int static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return FRT_E_DEVICE;
  if (!g_static_scratch_ready[dev].load(std::memory_order_acquire)) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_grouped_static_scratch) != cudaSuccess || ptr == nullptr) return FRT_E_LAUNCH;
    g_static_scratch_ptr[dev] = ptr;            // same value from every thread that races here
    g_static_scratch_ready[dev].store(true, std::memory_order_release);
  }
  *out = g_static_scratch_ptr[dev];
  return FRT_OK;
}

}  // namespace

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

int frt_nvfp4_grouped_gemm_bf16_noalloc(const void* a_packed, const void* sfa, const void* b_stack,
                                        const void* sfb_stack, const void* alpha, const void* expert_offsets,
                                        const void* tile_expert, int tile_rows, void* out, int rows, int N, int K,
                                        int num_experts, int64_t b_stride, int64_t sfb_stride, void* stream) {
  if (rows > FRT_GROUPED_STATIC_MAX_ROWS || num_experts > FRT_GROUPED_STATIC_MAX_EXPERTS) return FRT_E_TOO_LARGE;
  void* scratch = nullptr;
  if (int rc = static_scratch(&scratch)) return rc;
  // the plan kernel's item counter is the only part of the scratch that must start at
  // zero; the shared launch path clears it on `stream` before planning
  return frt_nvfp4_grouped_gemm_bf16(a_packed, sfa, b_stack, sfb_stack, alpha, expert_offsets, tile_expert,
                                     tile_rows, out, rows, N, K, num_experts, b_stride, sfb_stride, scratch, stream);
}

}  // extern "C"
