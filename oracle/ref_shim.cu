// extern "C" doors into the reference's own CUDA launchers, so that GPU tests
// can run the UNMODIFIED reference kernels beside ours (test infrastructure;
// built by oracle/Makefile into oracle/_ref/, never linked into the product).
// Only declarations are taken from the reference headers at build time.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "quantize_fp4_sfa.cuh"                 // fp4-gemm/csrc/quantize
#include "quantize_fp4_sfa_bf16.cuh"            // fp4-gemm/csrc/quantize
#include "dequantize_fp4_sfa.cuh"               // fp4-gemm/csrc
#include "nvfp4_sf_reshape_sm120.cuh"           // flashrt-nvfp4/csrc
#include "residual_norm_quant.cuh"              // flashrt-residual-norm-quant/csrc
#include "kernels/rms_norm_quantize_fp4_sfa_bf16.cuh"   // fp4-fused-ops/csrc
#include "kernels/silu_mul_quantize_fp4_sfa_bf16.cuh"   // fp4-fused-ops/csrc
#include "kernels/nexn2_router_topk.cuh"               // transformer-fused-ops/csrc
#include "kernels/moe_weighted_sum_sm120.cuh"          // transformer-fused-ops/csrc
#ifdef REF_HAVE_CUTLASS
#define FLASHRT_HAVE_COSMOS3_EDGE 1
#include "fused_fp4/cosmos3_edge_fp4.cuh"       // fp4-fused-ops/csrc
#include "fused_fp4/norm_silu_fp4_sfa.cuh"      // fp4-fused-ops/csrc
#include "cutlass_nvfp4_w4a16_gemm_sm100.cuh"   // fp4-gemm/csrc/gemm/fp4
#endif

#define S(x) reinterpret_cast<cudaStream_t>(x)

extern "C" {

int ref_has_cutlass() {
#ifdef REF_HAVE_CUTLASS
  return 1;
#else
  return 0;
#endif
}

// K4: the vectorised bf16 "reference quantizer"
int ref_quantize_bf16_vec(const void* src, void* packed, void* sfa, int rows, int dim, void* st) {
  return flash_rt::fp4::quantize_fp4_dynamic_sfa_bf16_vec(src, packed, sfa, rows, dim, false, S(st));
}
// K3: scalar bf16 / fp16 quantizers
int ref_quantize_bf16(const void* src, void* packed, void* sfa, int rows, int dim, void* st) {
  return flash_rt::fp4::quantize_fp4_dynamic_sfa_bf16(src, packed, sfa, rows, dim, false, S(st));
}
int ref_quantize_fp16(const void* src, void* packed, void* sfa, int rows, int dim, void* st) {
  return flash_rt::fp4::quantize_fp4_dynamic_sfa_fp16(src, packed, sfa, rows, dim, false, S(st));
}
// K6
int ref_quantize_mse_bf16(const void* src, void* packed, void* sfa, int rows, int dim, void* st) {
  return flash_rt::fp4::quantize_fp4_dynamic_sfa_mse_bf16(src, packed, sfa, rows, dim, true, S(st));
}
int ref_quantize_mse_fp16(const void* src, void* packed, void* sfa, int rows, int dim, void* st) {
  return flash_rt::fp4::quantize_fp4_dynamic_sfa_mse_fp16(src, packed, sfa, rows, dim, true, S(st));
}
int ref_dequantize_fp16(const void* packed, const void* sfa, void* out, int rows, int dim, void* st) {
  flash_rt::fused_fp4::dequantize_fp4_sfa_fp16(static_cast<const uint8_t*>(packed), static_cast<const uint8_t*>(sfa),
                                               static_cast<__half*>(out), rows, dim, false, S(st));
  return 0;
}
// K2
int ref_sf_linear_to_swizzled(const void* src, void* dst, int rows, int dim, void* st) {
  return flash_rt::fp4::nvfp4_sf_linear_to_swizzled(src, dst, rows, dim, false, S(st));
}
// K7 / K8
int ref_rms_norm_bf16(const void* x, const void* w, void* out, int rows, int dim, float eps, void* st) {
  flash_rt::residual_norm_quant::rms_norm_bf16(x, w, out, rows, dim, eps, S(st));
  return 0;
}
int ref_residual_add_rms_norm_bf16(void* res, const void* x, const void* w, void* out, int rows, int dim,
                                   float eps, void* st) {
  flash_rt::residual_norm_quant::residual_add_rms_norm_bf16(res, x, w, out, rows, dim, eps, S(st));
  return 0;
}
int ref_layer_norm_bf16(const void* x, const void* w, const void* b, void* out, int rows, int dim, float eps, void* st) {
  flash_rt::residual_norm_quant::layer_norm_bf16(x, w, b, out, rows, dim, eps, S(st));
  return 0;
}
int ref_rms_norm_quant_fp8(void* res, const void* x, const void* w, void* out, int rows, int dim, float eps,
                           const void* scale, void* st) {
  if (res)
    flash_rt::residual_norm_quant::residual_add_rms_norm_quant_fp8_static_bf16(
        res, x, w, out, rows, dim, eps, static_cast<const float*>(scale), S(st));
  else
    flash_rt::residual_norm_quant::rms_norm_quant_fp8_static_bf16(x, w, out, rows, dim, eps,
                                                                   static_cast<const float*>(scale), S(st));
  return 0;
}
// K13
int ref_rms_norm_quantize_bf16(const void* x, const void* w, float eps, void* normed, void* packed, void* sfa,
                               int rows, int dim, void* st) {
  return flash_rt::fp4::rms_norm_quantize_fp4_sfa_bf16(x, w, eps, normed, packed, sfa, rows, dim, S(st));
}

// SwiGLU -> NVFP4 producer ([gate | up] bf16 (rows, 2H) -> packed + swizzled scales)
int ref_silu_mul_quantize_bf16(const void* merged, void* packed, void* sfa, int rows, int hidden, void* st) {
  return flash_rt::fp4::silu_mul_quantize_fp4_sfa_bf16(merged, packed, sfa, rows, hidden, S(st));
}

// MoE routing glue of transformer-fused-ops: one-row top-k router, weighted un-permute
int ref_router_topk_bf16(const void* logits, void* idx, void* val, int n_experts, int k, void* st) {
  return flash_rt::kernels::nexn2_router_topk_bf16(logits, idx, val, n_experts, k, S(st));
}
int ref_moe_weighted_sum_bf16(const void* y, const void* rows, const void* w, void* out, int tokens, int topk,
                              int hidden, int stride, void* st) {
  return flash_rt::kernels::moe_weighted_sum_sm120_bf16(y, rows, w, out, tokens, topk, hidden, stride, S(st));
}

#ifdef REF_HAVE_CUTLASS
// K10: residual_add_rms_norm_quant_nvfp4_swizzled_bf16
int ref_res_rms_fp4_bf16(void* res, const void* x, const void* w, void* packed, void* sfa, int rows, int dim,
                         float eps, void* st) {
  flash_rt::fused_fp4::cosmos3_edge_res_rms_fp4_sfa_bf16(
      static_cast<__nv_bfloat16*>(res), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<uint8_t*>(packed), static_cast<uint8_t*>(sfa), rows, dim, eps, S(st));
  return 0;
}
// fp16 residual + RMSNorm -> NVFP4 (v2: one thread per 16-element block)
int ref_res_rms_fp4_v2_fp16(void* res, const void* x, void* packed, void* sfa, int rows, int dim, void* st) {
  flash_rt::fused_fp4::residual_add_rms_norm_fp4_sfa_v2_fp16(static_cast<__half*>(res), static_cast<const __half*>(x),
                                                             static_cast<uint8_t*>(packed), static_cast<uint8_t*>(sfa),
                                                             rows, dim, S(st));
  return 0;
}
// K15 / K16: the reference's CUTLASS sm100 GEMM (cluster 1x1x1), bf16 out
int ref_gemm_sm100_bf16(const void* a, const void* b, void* d, int M, int N, int K, const void* sfa,
                        const void* sfb, float alpha, int widen, void* st) {
  if (widen)
    flash_rt::gemm::fp4_w4a16_gemm_sm100_bf16out_widen(a, b, d, M, N, K, sfa, sfb, alpha, S(st));
  else
    flash_rt::gemm::fp4_w4a16_gemm_sm100_bf16out(a, b, d, M, N, K, sfa, sfb, alpha, S(st));
  return 0;
}
#endif

}  // extern "C"
