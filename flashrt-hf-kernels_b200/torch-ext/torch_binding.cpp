// Torch operator libraries of the B200 NVFP4 path.
//
// Tensor-level validation, device guard and current-stream lookup live here;
// every op then makes exactly one call into the C ABI (include/flashrt_b200.h).
// Operator names, argument order and defaults follow the reference's
// per-package bindings so its Python wrappers and fake registrations apply
// unchanged:
//   fp4_gemm               fp4-gemm/torch-ext/torch_binding.cpp:1357-1428
//   fp4_fused_ops          fp4-fused-ops/torch-ext/torch_binding.cpp:1373-1410
//   flashrt_nvfp4          flashrt-nvfp4/torch-ext/torch_binding.cpp:73-82
//   flashrt_residual_norm_quant  flashrt-residual-norm-quant/torch-ext/torch_binding.cpp:228-250
//   grouped_moe_gemm       grouped-moe-gemm/torch-ext/torch_binding.cpp:84-93
//   transformer_fused_ops  transformer-fused-ops/torch-ext/torch_binding.cpp:735-737 (router, weighted sum only)
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <map>
#include <mutex>
#include <torch/all.h>
#include <torch/library.h>

#include <limits>

#include "flashrt_b200.h"
#include "registration.h"

namespace {

using torch::Tensor;

void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
void check_dtype(const Tensor& t, c10::ScalarType dt, const char* name, const char* dt_name) {
  check_cuda(t, name);
  TORCH_CHECK(t.scalar_type() == dt, name, " must be ", dt_name);
}
void check_same_device(const Tensor& a, const Tensor& b, const char* an, const char* bn) {
  TORCH_CHECK(a.get_device() == b.get_device(), an, " and ", bn, " must be on the same device");
}
int as_int(int64_t v, const char* name) {
  TORCH_CHECK(v >= 0 && v <= std::numeric_limits<int>::max(), name, " does not fit in int");
  return static_cast<int>(v);
}
void* stream_of(const Tensor& t) { return at::cuda::getCurrentCUDAStream(t.get_device()).stream(); }
void check_rc(int rc, const char* op) {
  TORCH_CHECK(rc == 0, op, " failed with rc=", rc, " (", frt_error_string(rc), ")");
}

// packed [rows, dim/2] u8 + flat swizzled scales with enough bytes
void check_packed_scales(const Tensor& packed, const Tensor& sf, int64_t rows, int64_t dim, const char* pn,
                         const char* sn) {
  check_dtype(packed, torch::kUInt8, pn, "torch.uint8");
  check_dtype(sf, torch::kUInt8, sn, "torch.uint8");
  TORCH_CHECK(dim % 16 == 0, "dim must be divisible by 16");
  TORCH_CHECK(packed.dim() == 2 && packed.size(0) == rows && packed.size(1) * 2 == dim, pn,
              " must have shape (rows, dim / 2)");
  TORCH_CHECK(sf.numel() >= frt_nvfp4_sf_swizzled_bytes(as_int(rows, "rows"), as_int(dim, "dim")), sn,
              " is smaller than the swizzled scale-factor buffer for (rows, dim)");
}

// ------------------------------------------------------------------ flashrt_nvfp4
void nvfp4_sf_linear_to_swizzled(const Tensor& scales, Tensor& out, int64_t D, bool /*is_sfb*/) {
  check_dtype(scales, torch::kUInt8, "scales", "torch.uint8");
  check_dtype(out, torch::kUInt8, "out", "torch.uint8");
  TORCH_CHECK(scales.dim() == 2, "scales must have shape (rows, D / 16)");
  TORCH_CHECK(D > 0 && D % 16 == 0, "D must be positive and divisible by 16");
  TORCH_CHECK(scales.size(0) > 0, "rows must be positive");
  TORCH_CHECK(scales.size(1) * 16 == D, "scales must have shape (rows, D / 16)");
  const int rows = as_int(scales.size(0), "rows"), dim = as_int(D, "D");
  TORCH_CHECK(out.numel() >= frt_nvfp4_sf_swizzled_bytes(rows, dim), "out is smaller than nvfp4_sf_swizzled_bytes");
  check_same_device(scales, out, "scales", "out");
  c10::cuda::CUDAGuard guard(scales.device());
  check_rc(frt_nvfp4_sf_linear_to_swizzled(scales.data_ptr(), out.data_ptr(), rows, dim, stream_of(scales)),
           "nvfp4_sf_linear_to_swizzled");
}

// ------------------------------------------------------------------ quantise / dequantise
void quantize_common(const Tensor& x, Tensor& packed, Tensor& sfa, c10::ScalarType dt, int frt_dt, const char* dt_name,
                     const char* op) {
  check_dtype(x, dt, "x", dt_name);
  TORCH_CHECK(x.dim() == 2, "x must have shape (rows, dim)");
  TORCH_CHECK(x.size(1) % 16 == 0, "dim must be divisible by 16");
  check_packed_scales(packed, sfa, x.size(0), x.size(1), "packed", "sfa");
  check_same_device(x, packed, "x", "packed");
  check_same_device(x, sfa, "x", "sfa");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_nvfp4_quantize(x.data_ptr(), frt_dt, packed.data_ptr(), sfa.data_ptr(), as_int(x.size(0), "rows"),
                              as_int(x.size(1), "dim"), stream_of(x)), op);
}
void quantize_mse_common(const Tensor& x, Tensor& packed, Tensor& sfa, c10::ScalarType dt, int frt_dt,
                         const char* dt_name, const char* op) {
  check_dtype(x, dt, "x", dt_name);
  TORCH_CHECK(x.dim() == 2, "x must have shape (rows, dim)");
  TORCH_CHECK(x.size(1) % 16 == 0, "dim must be divisible by 16");
  check_packed_scales(packed, sfa, x.size(0), x.size(1), "packed", "sfa");
  check_same_device(x, packed, "x", "packed");
  check_same_device(x, sfa, "x", "sfa");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_nvfp4_quantize_mse(x.data_ptr(), frt_dt, packed.data_ptr(), sfa.data_ptr(), as_int(x.size(0), "rows"),
                                  as_int(x.size(1), "dim"), stream_of(x)), op);
}
void quantize_fp4_sfa_mse_bf16(const Tensor& x, Tensor& packed, Tensor& sfa, bool) {
  quantize_mse_common(x, packed, sfa, torch::kBFloat16, FRT_DTYPE_BF16, "torch.bfloat16", "quantize_fp4_sfa_mse_bf16");
}
void quantize_fp4_sfa_mse_fp16(const Tensor& x, Tensor& packed, Tensor& sfa, bool) {
  quantize_mse_common(x, packed, sfa, torch::kFloat16, FRT_DTYPE_FP16, "torch.float16", "quantize_fp4_sfa_mse_fp16");
}
void quantize_fp4_sfa_bf16(const Tensor& x, Tensor& packed, Tensor& sfa, bool) {
  quantize_common(x, packed, sfa, torch::kBFloat16, FRT_DTYPE_BF16, "torch.bfloat16", "quantize_fp4_sfa_bf16");
}
void quantize_fp4_sfa_fp16(const Tensor& x, Tensor& packed, Tensor& sfa, bool) {
  quantize_common(x, packed, sfa, torch::kFloat16, FRT_DTYPE_FP16, "torch.float16", "quantize_fp4_sfa_fp16");
}
void dequantize_fp4_sfa_fp16(const Tensor& packed, const Tensor& sfa, Tensor& out, bool) {
  check_dtype(out, torch::kFloat16, "out", "torch.float16");
  TORCH_CHECK(out.dim() == 2, "out must have shape (rows, dim)");
  check_packed_scales(packed, sfa, out.size(0), out.size(1), "packed", "sfa");
  check_same_device(packed, out, "packed", "out");
  c10::cuda::CUDAGuard guard(out.device());
  check_rc(frt_nvfp4_dequantize_fp16(packed.data_ptr(), sfa.data_ptr(), out.data_ptr(), as_int(out.size(0), "rows"),
                                     as_int(out.size(1), "dim"), stream_of(out)), "dequantize_fp4_sfa_fp16");
}
void dequantize_fp4_sfa_fp16_3(const Tensor& packed, const Tensor& sfa, Tensor& out) {
  dequantize_fp4_sfa_fp16(packed, sfa, out, false);
}

// ------------------------------------------------------------------ GEMM
struct GemmShape { int m, n, k; };
GemmShape check_gemm_inputs(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb, const Tensor& out) {
  check_dtype(a, torch::kUInt8, "a_packed", "torch.uint8");
  check_dtype(b, torch::kUInt8, "b_packed", "torch.uint8");
  check_dtype(sfa, torch::kUInt8, "sfa", "torch.uint8");
  check_dtype(sfb, torch::kUInt8, "sfb", "torch.uint8");
  check_dtype(out, torch::kBFloat16, "out", "torch.bfloat16");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2, "a_packed, b_packed and out must be matrices");
  TORCH_CHECK(a.size(1) == b.size(1), "a_packed and b_packed must have the same packed K");
  const int64_t m = a.size(0), n = b.size(0), k = a.size(1) * 2;
  TORCH_CHECK(m > 0 && n > 0 && k > 0, "empty GEMM operand");
  TORCH_CHECK(k % 16 == 0, "K must be divisible by 16");
  TORCH_CHECK(k % 32 == 0, "K must be divisible by 32 on this device (16-byte packed row pitch)");
  TORCH_CHECK(n % 8 == 0, "N must be divisible by 8");
  TORCH_CHECK(out.size(0) == m && out.size(1) == n, "out must have shape (M, N)");
  GemmShape s{as_int(m, "M"), as_int(n, "N"), as_int(k, "K")};
  TORCH_CHECK(sfa.numel() >= frt_nvfp4_sf_swizzled_bytes(s.m, s.k), "sfa is smaller than the swizzled buffer for (M, K)");
  TORCH_CHECK(sfb.numel() >= frt_nvfp4_sf_swizzled_bytes(s.n, s.k), "sfb is smaller than the swizzled buffer for (N, K)");
  check_same_device(a, b, "a_packed", "b_packed");
  check_same_device(a, sfa, "a_packed", "sfa");
  check_same_device(a, sfb, "a_packed", "sfb");
  check_same_device(a, out, "a_packed", "out");
  return s;
}
void gemm_call(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb, const Tensor* bias,
               const Tensor* residual, Tensor& out, double alpha, const char* op) {
  const GemmShape s = check_gemm_inputs(a, b, sfa, sfb, out);
  if (bias) {
    check_dtype(*bias, torch::kBFloat16, "bias", "torch.bfloat16");
    TORCH_CHECK(bias->numel() == s.n, "bias must have N elements");
    check_same_device(a, *bias, "a_packed", "bias");
  }
  if (residual) {
    check_dtype(*residual, torch::kBFloat16, "residual", "torch.bfloat16");
    TORCH_CHECK(residual->sizes() == out.sizes(), "residual must have shape (M, N)");
    check_same_device(a, *residual, "a_packed", "residual");
  }
  c10::cuda::CUDAGuard guard(a.device());
  check_rc(frt_nvfp4_gemm_bf16(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(),
                               bias ? bias->data_ptr() : nullptr, residual ? residual->data_ptr() : nullptr,
                               out.data_ptr(), s.m, s.n, s.k, static_cast<float>(alpha), residual ? 1.0f : 0.0f,
                               stream_of(a)), op);
}
// `variant` selected a CUTLASS tile in the reference; this build has one kernel
// family whose tile is chosen from the shape, so every value is accepted.
void nvfp4_gemm_bf16(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb, Tensor& out, double alpha,
                     int64_t /*variant*/) {
  gemm_call(a, b, sfa, sfb, nullptr, nullptr, out, alpha, "nvfp4_gemm_bf16");
}
void nvfp4_gemm_bias_bf16(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb, const Tensor& bias,
                          Tensor& out) {
  gemm_call(a, b, sfa, sfb, &bias, nullptr, out, 1.0, "nvfp4_gemm_bias_bf16");
}
void nvfp4_gemm_bias_residual_bf16(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb,
                                   const Tensor& bias, const Tensor& residual, Tensor& out) {
  gemm_call(a, b, sfa, sfb, &bias, &residual, out, 1.0, "nvfp4_gemm_bias_residual_bf16");
}
void nvfp4_gemm_residual_bf16(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb,
                              const Tensor& residual, Tensor& out, double alpha) {
  gemm_call(a, b, sfa, sfb, nullptr, &residual, out, alpha, "nvfp4_gemm_residual_bf16");
}
// gate/up GEMM with the SwiGLU -> NVFP4 producer as its epilogue (additive op): b_packed is the
// stacked [gate ; up] weight (2 * hidden rows); the outputs describe a (M, hidden) NVFP4 tensor.
void nvfp4_gemm_swiglu_nvfp4_bf16(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb,
                                  Tensor& out_packed, Tensor& out_sfa, double alpha) {
  check_dtype(a, torch::kUInt8, "a_packed", "torch.uint8");
  check_dtype(b, torch::kUInt8, "b_packed", "torch.uint8");
  check_dtype(sfa, torch::kUInt8, "sfa", "torch.uint8");
  check_dtype(sfb, torch::kUInt8, "sfb", "torch.uint8");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "a_packed and b_packed must be matrices");
  TORCH_CHECK(a.size(1) == b.size(1), "a_packed and b_packed must have the same packed K");
  const int64_t m = a.size(0), n2 = b.size(0), k = a.size(1) * 2;
  TORCH_CHECK(m > 0 && n2 > 0 && k > 0, "empty GEMM operand");
  TORCH_CHECK(k % 32 == 0, "K must be divisible by 32 on this device (16-byte packed row pitch)");
  TORCH_CHECK(n2 % 256 == 0, "stacked gate/up N must be divisible by 256 (hidden divisible by 128)");
  const int64_t hidden = n2 / 2;
  check_packed_scales(out_packed, out_sfa, m, hidden, "out_packed", "out_sfa");
  const int mi = as_int(m, "M"), ni = as_int(n2, "N"), ki = as_int(k, "K");
  TORCH_CHECK(sfa.numel() >= frt_nvfp4_sf_swizzled_bytes(mi, ki), "sfa is smaller than the swizzled buffer for (M, K)");
  TORCH_CHECK(sfb.numel() >= frt_nvfp4_sf_swizzled_bytes(ni, ki), "sfb is smaller than the swizzled buffer for (N, K)");
  check_same_device(a, b, "a_packed", "b_packed");
  check_same_device(a, sfa, "a_packed", "sfa");
  check_same_device(a, sfb, "a_packed", "sfb");
  check_same_device(a, out_packed, "a_packed", "out_packed");
  check_same_device(a, out_sfa, "a_packed", "out_sfa");
  c10::cuda::CUDAGuard guard(a.device());
  check_rc(frt_nvfp4_gemm_swiglu_nvfp4(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(),
                                       out_packed.data_ptr(), out_sfa.data_ptr(), mi, ni, ki,
                                       static_cast<float>(alpha), stream_of(a)), "nvfp4_gemm_swiglu_nvfp4_bf16");
}
// Small-M entry points of the reference (SM120 warp-split kernels): same
// contraction; `warps` / `stages` tuned those kernels and are accepted and ignored.
void fp4_w4a4_gemv_warpsplit_bf16(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb, Tensor& out,
                                  double alpha, int64_t, int64_t) {
  TORCH_CHECK(a.dim() == 2 && a.size(0) == 1, "a_packed must have exactly 1 row");
  gemm_call(a, b, sfa, sfb, nullptr, nullptr, out, alpha, "fp4_w4a4_gemv_warpsplit_bf16");
}
void fp4_w4a4_gemm_warpsplit_mrows_bf16(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb,
                                        Tensor& out, double alpha, int64_t, int64_t) {
  TORCH_CHECK(a.dim() == 2 && a.size(0) >= 1 && a.size(0) <= 16, "a_packed must have 1..16 rows");
  gemm_call(a, b, sfa, sfb, nullptr, nullptr, out, alpha, "fp4_w4a4_gemm_warpsplit_mrows_bf16");
}

// Bind-time interleaved weight layout of the M = 1 GEMV and the GEMV that reads it
// (fp4-gemm/torch-ext/torch_binding.cpp:317-387): same checks and messages; `warps` / `stages` accepted and ignored.
void fp4_repack_b_interleaved_sm120(const Tensor& b_packed, Tensor& b_interleaved) {
  check_dtype(b_packed, torch::kUInt8, "b_packed", "torch.uint8");
  check_dtype(b_interleaved, torch::kUInt8, "b_interleaved", "torch.uint8");
  TORCH_CHECK(b_packed.dim() == 2, "b_packed must have shape (N, K / 2)");
  TORCH_CHECK(b_interleaved.sizes() == b_packed.sizes(), "b_interleaved must have the same shape as b_packed");
  const int64_t n = b_packed.size(0), k = b_packed.size(1) * 2;
  TORCH_CHECK(n > 0 && n % 8 == 0, "N must be positive and divisible by 8");
  TORCH_CHECK(k > 0 && k % 64 == 0, "K must be positive and divisible by 64");
  check_same_device(b_packed, b_interleaved, "b_packed", "b_interleaved");
  c10::cuda::CUDAGuard guard(b_packed.device());
  check_rc(frt_nvfp4_repack_interleaved(b_packed.data_ptr(), b_interleaved.data_ptr(), as_int(n, "N"), as_int(k, "K"),
                                        stream_of(b_packed)), "fp4_repack_b_interleaved_sm120");
}
void fp4_w4a4_gemv_warpsplit_interleaved_bf16(const Tensor& a, const Tensor& b_interleaved, const Tensor& sfa,
                                              const Tensor& sfb, Tensor& out, double alpha, int64_t warps,
                                              int64_t stages) {
  const GemmShape s = check_gemm_inputs(a, b_interleaved, sfa, sfb, out);
  TORCH_CHECK(s.m == 1, "interleaved warp-split GEMV serves M=1 only");
  TORCH_CHECK(warps == 2 || warps == 4 || warps == 8, "warps must be 2, 4 or 8");
  TORCH_CHECK(stages == 3 || stages == 4 || stages == 6, "stages must be 3, 4 or 6");
  TORCH_CHECK(s.k % 64 == 0, "K/64 must be divisible by warps");
  c10::cuda::CUDAGuard guard(a.device());
  check_rc(frt_nvfp4_gemv_interleaved_bf16(a.data_ptr(), sfa.data_ptr(), b_interleaved.data_ptr(), sfb.data_ptr(),
                                           out.data_ptr(), s.n, s.k, static_cast<float>(alpha), stream_of(a)),
           "fp4_w4a4_gemv_warpsplit_interleaved_bf16");
}

// M = 1 decode matvec of the reference's small-M package (flashrt-smallm-gemm/torch-ext/torch_binding.cpp:55-108):
// a_packed (K/2,) or (1, K/2), out (N,).  Any K % 32 == 0 is accepted (the reference kernel takes 4096 and 12288).
void nvfp4_w4a4_decode_matvec_bf16out(const Tensor& a, const Tensor& b, const Tensor& sfa, const Tensor& sfb, Tensor& out,
                                      double alpha) {
  check_dtype(a, torch::kUInt8, "a_packed", "torch.uint8");
  check_dtype(b, torch::kUInt8, "b_packed", "torch.uint8");
  check_dtype(sfa, torch::kUInt8, "sfa", "torch.uint8");
  check_dtype(sfb, torch::kUInt8, "sfb", "torch.uint8");
  check_dtype(out, torch::kBFloat16, "out", "torch.bfloat16");
  TORCH_CHECK(b.dim() == 2, "b_packed must have shape (N, K / 2)");
  TORCH_CHECK(a.dim() == 1 || (a.dim() == 2 && a.size(0) == 1), "a_packed must have shape (K / 2,) or (1, K / 2)");
  const int64_t n = b.size(0), k = b.size(1) * 2;
  TORCH_CHECK(n > 0, "N must be positive");
  TORCH_CHECK(k > 0, "K must be positive");
  TORCH_CHECK(a.numel() * 2 == k, "a_packed must contain K / 2 bytes");
  TORCH_CHECK(k % 32 == 0, "K must be divisible by 32 on this device (16-byte packed row pitch)");
  TORCH_CHECK(n % 8 == 0, "N must be divisible by 8");
  TORCH_CHECK(out.numel() >= n, "out must contain at least N BF16 values");
  const int ni = as_int(n, "N"), ki = as_int(k, "K");
  TORCH_CHECK(sfa.numel() >= frt_nvfp4_sf_swizzled_bytes(1, ki), "sfa must contain the swizzled bytes for one activation row");
  TORCH_CHECK(sfb.numel() >= frt_nvfp4_sf_swizzled_bytes(ni, ki), "sfb must contain the swizzled bytes for N weight rows");
  check_same_device(a, b, "a_packed", "b_packed");
  check_same_device(a, sfa, "a_packed", "sfa");
  check_same_device(a, sfb, "a_packed", "sfb");
  check_same_device(a, out, "a_packed", "out");
  c10::cuda::CUDAGuard guard(a.device());
  check_rc(frt_nvfp4_gemm_bf16(a.data_ptr(), sfa.data_ptr(), b.data_ptr(), sfb.data_ptr(), nullptr, nullptr,
                               out.data_ptr(), 1, ni, ki, static_cast<float>(alpha), 0.0f, stream_of(a)),
           "nvfp4_w4a4_decode_matvec_bf16out");
}

// ------------------------------------------------------------------ norms
void check_norm_inputs(const Tensor& x, const Tensor* weight, const Tensor* other, const char* other_name) {
  check_dtype(x, torch::kBFloat16, "x", "torch.bfloat16");
  TORCH_CHECK(x.dim() == 2, "x must have shape (rows, dim)");
  TORCH_CHECK(x.size(0) > 0, "rows must be positive");
  TORCH_CHECK(x.size(1) % 16 == 0 && x.size(1) <= 16384, "dim must be a multiple of 16 and at most 16384");
  if (weight) {
    check_dtype(*weight, torch::kBFloat16, "weight", "torch.bfloat16");
    TORCH_CHECK(weight->dim() == 1 && weight->size(0) == x.size(1), "weight must have shape (dim,)");
    check_same_device(x, *weight, "x", "weight");
  }
  if (other) {
    check_dtype(*other, torch::kBFloat16, other_name, "torch.bfloat16");
    TORCH_CHECK(other->sizes() == x.sizes(), other_name, " and x must have the same 2D shape");
    check_same_device(x, *other, "x", other_name);
  }
}
void rms_norm_bf16(const Tensor& x, const Tensor& weight, double eps, Tensor& out) {
  check_norm_inputs(x, &weight, &out, "out");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_rms_norm_bf16(x.data_ptr(), weight.data_ptr(), out.data_ptr(), as_int(x.size(0), "rows"),
                             as_int(x.size(1), "dim"), static_cast<float>(eps), stream_of(x)), "rms_norm_bf16");
}
// x: bf16 [tokens, width], unit stride along width (a stacked q/k/v projection output); normalises heads
// [0, heads_a + heads_b) of every row in place (extension of this build: no reference schema)
void rms_norm_heads_bf16_(Tensor& x, const Tensor& weight_a, int64_t heads_a, const c10::optional<Tensor>& weight_b,
                          int64_t heads_b, int64_t head_dim, double eps) {
  check_dtype(x, torch::kBFloat16, "x", "torch.bfloat16");
  check_dtype(weight_a, torch::kBFloat16, "weight_a", "torch.bfloat16");
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.stride(1) == 1, "x must be a CUDA (tokens, width) tensor with unit inner stride");
  TORCH_CHECK(weight_a.is_contiguous() && weight_a.dim() == 1 && weight_a.size(0) == head_dim, "weight_a must have shape (head_dim,)");
  TORCH_CHECK((heads_a + heads_b) * head_dim <= x.size(1), "the heads do not fit the row");
  const void* wb = nullptr;
  if (heads_b > 0) {
    TORCH_CHECK(weight_b.has_value(), "weight_b is required when heads_b > 0");
    check_dtype(*weight_b, torch::kBFloat16, "weight_b", "torch.bfloat16");
    TORCH_CHECK(weight_b->is_contiguous() && weight_b->dim() == 1 && weight_b->size(0) == head_dim, "weight_b must have shape (head_dim,)");
    check_same_device(x, *weight_b, "x", "weight_b");
    wb = weight_b->data_ptr();
  }
  check_same_device(x, weight_a, "x", "weight_a");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_rms_norm_heads_bf16(x.data_ptr(), as_int(x.size(0), "tokens"), as_int(x.stride(0), "row pitch"),
                                   as_int(head_dim, "head_dim"), as_int(heads_a, "heads_a"), weight_a.data_ptr(),
                                   as_int(heads_b, "heads_b"), wb, static_cast<float>(eps), stream_of(x)),
           "rms_norm_heads_bf16_");
}
void layer_norm_bf16(const Tensor& x, const Tensor& weight, const Tensor& bias, double eps, Tensor& out) {
  check_norm_inputs(x, &weight, &out, "out");
  check_dtype(bias, torch::kBFloat16, "bias", "torch.bfloat16");
  TORCH_CHECK(bias.dim() == 1 && bias.size(0) == x.size(1), "bias must have shape (dim,)");
  check_same_device(x, bias, "x", "bias");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_layer_norm_bf16(x.data_ptr(), weight.data_ptr(), bias.data_ptr(), out.data_ptr(),
                               as_int(x.size(0), "rows"), as_int(x.size(1), "dim"), static_cast<float>(eps),
                               stream_of(x)), "layer_norm_bf16");
}
void fp8_norm_call(Tensor* residual, const Tensor& x, const Tensor& weight, const Tensor& scale, double eps, Tensor& out,
                   const char* op) {
  check_norm_inputs(x, &weight, residual, "residual");
  check_dtype(scale, torch::kFloat32, "scale", "torch.float32");
  TORCH_CHECK(scale.numel() == 1, "scale must hold one float32 value");
  check_cuda(out, "out");
  TORCH_CHECK(out.scalar_type() == torch::kFloat8_e4m3fn, "out must be torch.float8_e4m3fn");
  TORCH_CHECK(out.sizes() == x.sizes(), "out and x must have the same 2D shape");
  check_same_device(x, scale, "x", "scale");
  check_same_device(x, out, "x", "out");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_rms_norm_quant_fp8(residual ? residual->data_ptr() : nullptr, x.data_ptr(), weight.data_ptr(),
                                  scale.data_ptr(), out.data_ptr(), as_int(x.size(0), "rows"),
                                  as_int(x.size(1), "dim"), static_cast<float>(eps), stream_of(x)), op);
}
void rms_norm_quant_fp8_static_bf16(const Tensor& x, const Tensor& weight, const Tensor& scale, double eps, Tensor& out) {
  fp8_norm_call(nullptr, x, weight, scale, eps, out, "rms_norm_quant_fp8_static_bf16");
}
void residual_add_rms_norm_quant_fp8_static_bf16(Tensor& residual, const Tensor& x, const Tensor& weight,
                                                 const Tensor& scale, double eps, Tensor& out) {
  fp8_norm_call(&residual, x, weight, scale, eps, out, "residual_add_rms_norm_quant_fp8_static_bf16");
}
void residual_add_rms_norm_bf16(Tensor& residual, const Tensor& x, const Tensor& weight, double eps, Tensor& out) {
  check_norm_inputs(x, &weight, &out, "out");
  check_norm_inputs(x, nullptr, &residual, "residual");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_residual_add_rms_norm_bf16(residual.data_ptr(), x.data_ptr(), weight.data_ptr(), out.data_ptr(),
                                          as_int(x.size(0), "rows"), as_int(x.size(1), "dim"),
                                          static_cast<float>(eps), stream_of(x)), "residual_add_rms_norm_bf16");
}

// ------------------------------------------------------------------ fused producers
void producer_call(Tensor* residual, const Tensor& x, const Tensor* weight, double eps, double inv_global_scale,
                   Tensor* normed, Tensor& packed, Tensor& sfa, unsigned flags, const char* op) {
  check_norm_inputs(x, weight, residual, "residual");
  if (normed) check_norm_inputs(x, nullptr, normed, "normed");
  check_packed_scales(packed, sfa, x.size(0), x.size(1), "packed", "sfa");
  check_same_device(x, packed, "x", "packed");
  check_same_device(x, sfa, "x", "sfa");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_norm_quant_nvfp4(residual ? residual->data_ptr() : nullptr, x.data_ptr(),
                                weight ? weight->data_ptr() : nullptr, static_cast<float>(eps),
                                static_cast<float>(inv_global_scale), normed ? normed->data_ptr() : nullptr,
                                packed.data_ptr(), sfa.data_ptr(), as_int(x.size(0), "rows"), as_int(x.size(1), "dim"),
                                flags, stream_of(x)), op);
}
void residual_add_rms_norm_quant_nvfp4_swizzled_bf16(Tensor& residual, const Tensor& x, const Tensor& weight,
                                                     double eps, Tensor& packed, Tensor& sfa) {
  producer_call(&residual, x, &weight, eps, 1.0, nullptr, packed, sfa, 0u,
                "residual_add_rms_norm_quant_nvfp4_swizzled_bf16");
}
void rms_norm_quantize_fp4_sfa_bf16(const Tensor& x, const Tensor& weight, double eps, Tensor& normed, Tensor& packed,
                                    Tensor& sfa) {
  producer_call(nullptr, x, &weight, eps, 1.0, &normed, packed, sfa,
                FRT_PRODUCER_ONE_PLUS_W | FRT_PRODUCER_ROUND_BF16, "rms_norm_quantize_fp4_sfa_bf16");
}
void residual_add_rms_norm_nvfp4_bf16(Tensor& residual, const Tensor& x, const c10::optional<Tensor>& inv_s, double eps,
                                      Tensor& packed, Tensor& sfa) {
  const Tensor* w = inv_s.has_value() ? &inv_s.value() : nullptr;
  producer_call(&residual, x, w, eps, 1.0, nullptr, packed, sfa,
                FRT_PRODUCER_RNE_E2M1 | FRT_PRODUCER_ROUND_BF16 | FRT_PRODUCER_NORM_FROM_BF16_RESIDUAL,
                "residual_add_rms_norm_nvfp4_bf16");
}
void silu_mul_quantize_fp4_sfa_bf16(const Tensor& merged, Tensor& packed, Tensor& sfa) {
  check_dtype(merged, torch::kBFloat16, "merged", "torch.bfloat16");
  TORCH_CHECK(merged.dim() == 2, "merged must have shape (rows, 2 * hidden)");
  TORCH_CHECK(merged.size(0) > 0, "rows must be positive");
  TORCH_CHECK(merged.size(1) % 32 == 0, "merged.shape[1] must be divisible by 32");
  const int64_t rows = merged.size(0), hidden = merged.size(1) / 2;
  check_packed_scales(packed, sfa, rows, hidden, "packed", "sfa");
  check_same_device(merged, packed, "merged", "packed");
  check_same_device(merged, sfa, "merged", "sfa");
  c10::cuda::CUDAGuard guard(merged.device());
  check_rc(frt_silu_mul_quant_nvfp4(merged.data_ptr(), packed.data_ptr(), sfa.data_ptr(), as_int(rows, "rows"),
                                    as_int(hidden, "hidden"), stream_of(merged)), "silu_mul_quantize_fp4_sfa_bf16");
}
// Additive op: the reference recipe plus an optional second-level (per-tensor)
// scale and an optional bf16 copy of the quantiser input.
void residual_add_rms_norm_quant_nvfp4_ex(Tensor& residual, const Tensor& x, const Tensor& weight, double eps,
                                          double inv_global_scale, const c10::optional<Tensor>& normed, Tensor& packed,
                                          Tensor& sfa) {
  Tensor n = normed.has_value() ? normed.value() : Tensor();
  producer_call(&residual, x, &weight, eps, inv_global_scale, normed.has_value() ? &n : nullptr, packed, sfa, 0u,
                "residual_add_rms_norm_quant_nvfp4_ex");
}
// fp16 activations / residual, unweighted, eps = 1e-6 (fp4-fused-ops/torch-ext/torch_binding.cpp:269-296)
void residual_add_rms_norm_fp4_sfa_v2_fp16(Tensor& residual, const Tensor& x, Tensor& packed, Tensor& sfa) {
  check_dtype(residual, torch::kFloat16, "residual", "torch.float16");
  check_dtype(x, torch::kFloat16, "x", "torch.float16");
  TORCH_CHECK(x.dim() == 2 && residual.sizes() == x.sizes(), "residual and x must have the same shape");
  TORCH_CHECK(x.size(1) <= 16384, "v2 residual path supports dim <= 16384");
  TORCH_CHECK(x.size(1) % 16 == 0, "dim must be divisible by 16");
  check_same_device(residual, x, "residual", "x");
  check_packed_scales(packed, sfa, x.size(0), x.size(1), "packed", "sfa");
  check_same_device(x, packed, "x", "packed");
  check_same_device(x, sfa, "x", "sfa");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_residual_norm_quant_nvfp4_fp16(residual.data_ptr(), x.data_ptr(), 1e-6f, packed.data_ptr(), sfa.data_ptr(),
                                              as_int(x.size(0), "rows"), as_int(x.size(1), "dim"), stream_of(x)),
           "residual_add_rms_norm_fp4_sfa_v2_fp16");
}
// Additive op: RMSNorm (plain or 1 + weight) -> NVFP4 without a residual, optional bf16 copy of
// the normalised tensor (what transformers' decoder layers pass on to the projections).
void rms_norm_quant_nvfp4_ex(const Tensor& x, const Tensor& weight, double eps, const c10::optional<Tensor>& normed,
                             Tensor& packed, Tensor& sfa, bool one_plus_weight, bool round_bf16) {
  Tensor n = normed.has_value() ? normed.value() : Tensor();
  producer_call(nullptr, x, &weight, eps, 1.0, normed.has_value() ? &n : nullptr, packed, sfa,
                (one_plus_weight ? FRT_PRODUCER_ONE_PLUS_W : 0u) | (round_bf16 ? FRT_PRODUCER_ROUND_BF16 : 0u),
                "rms_norm_quant_nvfp4_ex");
}
int64_t sfa_size_bytes_for(const Tensor& /*anchor*/, int64_t rows, int64_t dim, bool /*is_sfb*/) {
  TORCH_CHECK(rows > 0 && dim > 0 && dim % 16 == 0, "rows must be positive and dim positive/divisible by 16");
  return frt_nvfp4_sf_swizzled_bytes(as_int(rows, "rows"), as_int(dim, "dim"));
}

// ------------------------------------------------------------------ grouped MoE
void grouped_common(const Tensor& input, const Tensor& weight, const Tensor& input_scale, const Tensor& weight_scale,
                    const Tensor& alpha, Tensor& output) {
  check_dtype(input, torch::kUInt8, "input", "torch.uint8");
  check_dtype(weight, torch::kUInt8, "weight", "torch.uint8");
  check_dtype(input_scale, torch::kUInt8, "input_scale", "torch.uint8");
  check_dtype(weight_scale, torch::kUInt8, "weight_scale", "torch.uint8");
  check_dtype(alpha, torch::kFloat32, "alpha", "torch.float32");
  check_dtype(output, torch::kBFloat16, "output", "torch.bfloat16");
  TORCH_CHECK(input.dim() == 2 && weight.dim() == 3 && output.dim() == 2,
              "input/output must be matrices and weight must be (experts,N,K/2)");
  const int64_t K = input.size(1) * 2, N = weight.size(1);
  TORCH_CHECK(weight.size(2) * 2 == K && K % 64 == 0, "packed K mismatch or K not divisible by 64");
  TORCH_CHECK(output.size(0) == input.size(0) && output.size(1) == N, "output shape mismatch");
  TORCH_CHECK(alpha.numel() >= weight.size(0), "alpha must cover all experts");
  TORCH_CHECK(N % 8 == 0, "N must be divisible by 8");
  TORCH_CHECK(input.get_device() == output.get_device(), "all tensors must share one device");
}
// Work-list scratch of the reference-schema op, which has no workspace argument: one buffer per (device,
// stream), allocated on the first call that needs it (or a larger one) and reused by every later call, so the
// hot call allocates nothing.  Calls on one stream are ordered, so they may share it; another stream gets its own.
Tensor grouped_workspace(const Tensor& like, int rows, int experts, void* stream) {
  static std::mutex mu;
  static std::map<std::pair<int, void*>, Tensor> cache;
  const int64_t need = frt_nvfp4_grouped_gemm_workspace_bytes(rows, experts);
  std::lock_guard<std::mutex> lock(mu);
  Tensor& slot = cache[{static_cast<int>(like.get_device()), stream}];
  if (!slot.defined() || slot.numel() < need)
    slot = torch::empty({need}, torch::TensorOptions().dtype(torch::kUInt8).device(like.device()));
  return slot;
}
void grouped_nvfp4_gemm_bf16_out(const Tensor& input, const Tensor& weight, const Tensor& input_scale,
                                 const Tensor& weight_scale, const Tensor& alpha, const Tensor& tile_expert,
                                 int64_t tile_rows, int64_t input_scale_stride, int64_t weight_stride,
                                 int64_t weight_scale_stride, Tensor& output, const c10::optional<Tensor>& workspace) {
  grouped_common(input, weight, input_scale, weight_scale, alpha, output);
  check_dtype(tile_expert, torch::kInt32, "tile_expert", "torch.int32");
  TORCH_CHECK(tile_rows == 16 || tile_rows == 64, "tile_rows must be 16 or 64");
  const int64_t num_tiles = tile_expert.numel();
  TORCH_CHECK(num_tiles > 0 && input.size(0) == num_tiles * tile_rows, "input rows must equal num_tiles * tile_rows");
  TORCH_CHECK(input_scale_stride >= 0 && weight_stride > 0 && weight_scale_stride > 0, "invalid byte strides");
  const int rows = as_int(input.size(0), "rows"), experts = as_int(weight.size(0), "experts");
  c10::cuda::CUDAGuard guard(input.device());
  Tensor work = workspace.has_value() ? workspace.value() : grouped_workspace(input, rows, experts, stream_of(input));
  TORCH_CHECK(work.is_cuda() && work.nbytes() >= static_cast<size_t>(frt_nvfp4_grouped_gemm_workspace_bytes(rows, experts)),
              "workspace is too small");
  check_rc(frt_nvfp4_grouped_gemm_bf16(input.data_ptr(), input_scale.data_ptr(), weight.data_ptr(),
                                       weight_scale.data_ptr(), alpha.data_ptr(), nullptr, tile_expert.data_ptr(),
                                       static_cast<int>(tile_rows), output.data_ptr(), rows, as_int(weight.size(1), "N"),
                                       as_int(input.size(1) * 2, "K"), experts, weight_stride, weight_scale_stride,
                                       work.data_ptr(), stream_of(input)), "grouped NVFP4 GEMM");
}
void grouped_nvfp4_gemm_bf16_legacy(const Tensor& input, const Tensor& weight, const Tensor& input_scale,
                                    const Tensor& weight_scale, const Tensor& alpha, const Tensor& tile_expert,
                                    int64_t tile_rows, int64_t input_scale_stride, int64_t weight_stride,
                                    int64_t weight_scale_stride, Tensor& output) {
  grouped_nvfp4_gemm_bf16_out(input, weight, input_scale, weight_scale, alpha, tile_expert, tile_rows,
                              input_scale_stride, weight_stride, weight_scale_stride, output, c10::nullopt);
}
// Additive op: expert-sorted rows described by an offsets array.
void grouped_nvfp4_gemm_bf16_offsets_out(const Tensor& input, const Tensor& weight, const Tensor& input_scale,
                                         const Tensor& weight_scale, const Tensor& alpha, const Tensor& expert_offsets,
                                         Tensor& workspace, Tensor& output) {
  grouped_common(input, weight, input_scale, weight_scale, alpha, output);
  check_dtype(expert_offsets, torch::kInt32, "expert_offsets", "torch.int32");
  const int rows = as_int(input.size(0), "rows"), experts = as_int(weight.size(0), "experts");
  TORCH_CHECK(expert_offsets.numel() == experts + 1, "expert_offsets must have num_experts + 1 entries");
  TORCH_CHECK(workspace.is_cuda() && workspace.nbytes() >=
                  static_cast<size_t>(frt_nvfp4_grouped_gemm_workspace_bytes(rows, experts)), "workspace is too small");
  c10::cuda::CUDAGuard guard(input.device());
  check_rc(frt_nvfp4_grouped_gemm_bf16(input.data_ptr(), input_scale.data_ptr(), weight.data_ptr(),
                                       weight_scale.data_ptr(), alpha.data_ptr(), expert_offsets.data_ptr(), nullptr, 0,
                                       output.data_ptr(), rows, as_int(weight.size(1), "N"),
                                       as_int(input.size(1) * 2, "K"), experts,
                                       weight.size(1) * weight.size(2), weight_scale.numel() / experts,
                                       workspace.data_ptr(), stream_of(input)), "grouped NVFP4 GEMM (offsets)");
}
int64_t grouped_nvfp4_gemm_workspace_size(int64_t rows, int64_t experts) {
  return frt_nvfp4_grouped_gemm_workspace_bytes(as_int(rows, "rows"), as_int(experts, "experts"));
}

// ------------------------------------------------------------------ MoE routing glue
// logits (n_experts,) as in the reference, or (tokens, n_experts); outputs (k,) / (tokens, k)
void router_topk_bf16(const Tensor& logits, Tensor& out_idx, Tensor& out_val, int64_t k) {
  check_dtype(logits, torch::kBFloat16, "logits", "torch.bfloat16");
  check_dtype(out_idx, torch::kInt32, "out_idx", "torch.int32");
  check_dtype(out_val, torch::kFloat32, "out_val", "torch.float32");
  TORCH_CHECK(logits.dim() == 1 || logits.dim() == 2, "logits must have shape (n_experts,) or (tokens, n_experts)");
  const int64_t tokens = logits.dim() == 1 ? 1 : logits.size(0), n = logits.size(-1);
  if (logits.dim() == 1) {
    TORCH_CHECK(out_idx.sizes() == torch::IntArrayRef({k}) && out_val.sizes() == torch::IntArrayRef({k}),
                "topk outputs must have shape (k,)");
  } else {
    TORCH_CHECK(out_idx.sizes() == torch::IntArrayRef({tokens, k}) && out_val.sizes() == torch::IntArrayRef({tokens, k}),
                "topk outputs must have shape (tokens, k)");
  }
  check_same_device(logits, out_idx, "logits", "out_idx");
  check_same_device(logits, out_val, "logits", "out_val");
  c10::cuda::CUDAGuard guard(logits.device());
  check_rc(frt_router_topk_bf16(logits.data_ptr(), out_idx.data_ptr(), out_val.data_ptr(), as_int(tokens, "tokens"),
                                as_int(n, "n_experts"), as_int(k, "k"), stream_of(logits)), "router_topk_bf16");
}
// additive: top-k with the softmax of the selected logits as routing weights, in the same kernel
void router_topk_softmax_bf16(const Tensor& logits, Tensor& out_idx, Tensor& out_val, Tensor& out_weight, int64_t k) {
  check_dtype(out_weight, torch::kFloat32, "out_weight", "torch.float32");
  TORCH_CHECK(out_weight.sizes() == out_val.sizes(), "out_weight must have the shape of out_val");
  check_dtype(logits, torch::kBFloat16, "logits", "torch.bfloat16");
  check_dtype(out_idx, torch::kInt32, "out_idx", "torch.int32");
  check_dtype(out_val, torch::kFloat32, "out_val", "torch.float32");
  TORCH_CHECK(logits.dim() == 2, "logits must have shape (tokens, n_experts)");
  const int64_t tokens = logits.size(0), n = logits.size(1);
  TORCH_CHECK(out_idx.sizes() == torch::IntArrayRef({tokens, k}) && out_val.sizes() == torch::IntArrayRef({tokens, k}),
              "topk outputs must have shape (tokens, k)");
  check_same_device(logits, out_idx, "logits", "out_idx");
  check_same_device(logits, out_val, "logits", "out_val");
  check_same_device(logits, out_weight, "logits", "out_weight");
  c10::cuda::CUDAGuard guard(logits.device());
  check_rc(frt_router_topk_softmax_bf16(logits.data_ptr(), out_idx.data_ptr(), out_val.data_ptr(), out_weight.data_ptr(),
                                        as_int(tokens, "tokens"), as_int(n, "n_experts"), as_int(k, "k"),
                                        stream_of(logits)), "router_topk_softmax_bf16");
}
void moe_weighted_sum_bf16_to_fp32(const Tensor& expert_output, const Tensor& row_indices, const Tensor& router_weight,
                                   Tensor& out) {
  check_dtype(expert_output, torch::kBFloat16, "expert_output", "torch.bfloat16");
  check_dtype(row_indices, torch::kInt32, "row_indices", "torch.int32");
  check_dtype(router_weight, torch::kFloat32, "router_weight", "torch.float32");
  check_dtype(out, torch::kFloat32, "out", "torch.float32");
  TORCH_CHECK(expert_output.dim() == 2, "expert_output must have shape (routed_rows, stride)");
  TORCH_CHECK(row_indices.dim() == 2 && router_weight.sizes() == row_indices.sizes(),
              "row_indices and router_weight must have shape (tokens, topk)");
  TORCH_CHECK(out.dim() == 2 && out.size(0) == row_indices.size(0), "out must have shape (tokens, hidden)");
  TORCH_CHECK(expert_output.size(1) >= out.size(1), "expert_output stride must cover out hidden size");
  check_same_device(expert_output, row_indices, "expert_output", "row_indices");
  check_same_device(expert_output, router_weight, "expert_output", "router_weight");
  check_same_device(expert_output, out, "expert_output", "out");
  c10::cuda::CUDAGuard guard(expert_output.device());
  check_rc(frt_moe_weighted_sum_bf16(expert_output.data_ptr(), row_indices.data_ptr(), router_weight.data_ptr(),
                                     out.data_ptr(), as_int(row_indices.size(0), "tokens"),
                                     as_int(row_indices.size(1), "topk"), as_int(out.size(1), "hidden"),
                                     as_int(expert_output.size(1), "expert_output stride"), stream_of(expert_output)),
           "moe_weighted_sum_bf16_to_fp32");
}
// additive: the routing sort and the gather into expert order that the reference leaves to the caller
void moe_route_plan(const Tensor& topk_idx, int64_t n_experts, Tensor& expert_offsets, Tensor& row_of_pair,
                    Tensor& token_of_row) {
  check_dtype(topk_idx, torch::kInt32, "topk_idx", "torch.int32");
  check_dtype(expert_offsets, torch::kInt32, "expert_offsets", "torch.int32");
  check_dtype(row_of_pair, torch::kInt32, "row_of_pair", "torch.int32");
  check_dtype(token_of_row, torch::kInt32, "token_of_row", "torch.int32");
  TORCH_CHECK(topk_idx.dim() == 2, "topk_idx must have shape (tokens, topk)");
  TORCH_CHECK(n_experts > 0 && expert_offsets.numel() == n_experts + 1, "expert_offsets must have n_experts + 1 elements");
  TORCH_CHECK(row_of_pair.numel() == topk_idx.numel() && token_of_row.numel() == topk_idx.numel(),
              "row_of_pair and token_of_row must have tokens * topk elements");
  check_same_device(topk_idx, expert_offsets, "topk_idx", "expert_offsets");
  check_same_device(topk_idx, row_of_pair, "topk_idx", "row_of_pair");
  check_same_device(topk_idx, token_of_row, "topk_idx", "token_of_row");
  c10::cuda::CUDAGuard guard(topk_idx.device());
  check_rc(frt_moe_route_plan(topk_idx.data_ptr(), as_int(topk_idx.size(0), "tokens"), as_int(topk_idx.size(1), "topk"),
                              as_int(n_experts, "n_experts"), expert_offsets.data_ptr(), row_of_pair.data_ptr(),
                              token_of_row.data_ptr(), stream_of(topk_idx)), "moe_route_plan");
}
void moe_quantize_scatter_nvfp4(const Tensor& x, const Tensor& row_of_pair, Tensor& out_packed, Tensor& out_sfa) {
  check_dtype(x, torch::kBFloat16, "x", "torch.bfloat16");
  check_dtype(row_of_pair, torch::kInt32, "row_of_pair", "torch.int32");
  TORCH_CHECK(x.dim() == 2 && row_of_pair.dim() == 2 && row_of_pair.size(0) == x.size(0),
              "x must be (tokens, K) and row_of_pair (tokens, topk)");
  TORCH_CHECK(x.size(1) % 16 == 0, "K must be divisible by 16");
  TORCH_CHECK(out_packed.dim() == 2 && out_packed.size(0) >= row_of_pair.numel(),
              "out_packed must have a row for every (token, slot) pair");
  check_packed_scales(out_packed, out_sfa, out_packed.size(0), x.size(1), "out_packed", "out_sfa");
  check_same_device(x, row_of_pair, "x", "row_of_pair");
  check_same_device(x, out_packed, "x", "out_packed");
  check_same_device(x, out_sfa, "x", "out_sfa");
  c10::cuda::CUDAGuard guard(x.device());
  check_rc(frt_moe_quantize_scatter_nvfp4(x.data_ptr(), row_of_pair.data_ptr(), out_packed.data_ptr(), out_sfa.data_ptr(),
                                          as_int(x.size(0), "tokens"), as_int(row_of_pair.size(1), "topk"),
                                          as_int(x.size(1), "K"), stream_of(x)), "moe_quantize_scatter_nvfp4");
}
void moe_gather_nvfp4(const Tensor& packed, const Tensor& sfa, const Tensor& token_of_row, Tensor& out_packed,
                      Tensor& out_sfa) {
  check_dtype(token_of_row, torch::kInt32, "token_of_row", "torch.int32");
  TORCH_CHECK(packed.dim() == 2 && out_packed.dim() == 2 && packed.size(1) == out_packed.size(1),
              "packed and out_packed must be matrices with the same packed K");
  const int64_t tokens = packed.size(0), rows = out_packed.size(0), K = packed.size(1) * 2;
  TORCH_CHECK(K % 64 == 0, "K must be divisible by 64");
  TORCH_CHECK(token_of_row.numel() >= rows, "token_of_row must have one entry per output row");
  check_packed_scales(packed, sfa, tokens, K, "packed", "sfa");
  check_packed_scales(out_packed, out_sfa, rows, K, "out_packed", "out_sfa");
  check_same_device(packed, sfa, "packed", "sfa");
  check_same_device(packed, token_of_row, "packed", "token_of_row");
  check_same_device(packed, out_packed, "packed", "out_packed");
  check_same_device(packed, out_sfa, "packed", "out_sfa");
  c10::cuda::CUDAGuard guard(packed.device());
  check_rc(frt_moe_gather_nvfp4(packed.data_ptr(), sfa.data_ptr(), token_of_row.data_ptr(), out_packed.data_ptr(),
                                out_sfa.data_ptr(), as_int(rows, "rows"), as_int(tokens, "tokens"), as_int(K, "K"),
                                stream_of(packed)), "moe_gather_nvfp4");
}

}  // namespace

TORCH_LIBRARY_EXPAND(flashrt_smallm_gemm_b200, ops) {
  ops.def("nvfp4_w4a4_decode_matvec_bf16out(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor! out, float alpha=1.0) -> ()");
  ops.impl("nvfp4_w4a4_decode_matvec_bf16out", torch::kCUDA, &nvfp4_w4a4_decode_matvec_bf16out);
}

TORCH_LIBRARY_EXPAND(transformer_fused_ops_b200, ops) {
  ops.def("nexn2_router_topk_bf16(Tensor logits, Tensor! out_idx, Tensor! out_val, int k) -> ()");
  ops.def("router_topk_bf16(Tensor logits, Tensor! out_idx, Tensor! out_val, int k) -> ()");
  ops.def("moe_weighted_sum_bf16_to_fp32(Tensor expert_output, Tensor row_indices, Tensor router_weight, Tensor! out) -> ()");
  ops.impl("nexn2_router_topk_bf16", torch::kCUDA, &router_topk_bf16);
  ops.impl("router_topk_bf16", torch::kCUDA, &router_topk_bf16);
  ops.impl("moe_weighted_sum_bf16_to_fp32", torch::kCUDA, &moe_weighted_sum_bf16_to_fp32);
  ops.def("router_topk_softmax_bf16(Tensor logits, Tensor! out_idx, Tensor! out_val, Tensor! out_weight, int k) -> ()");
  ops.impl("router_topk_softmax_bf16", torch::kCUDA, &router_topk_softmax_bf16);
}

TORCH_LIBRARY_EXPAND(flashrt_nvfp4_b200, ops) {
  ops.def("nvfp4_sf_linear_to_swizzled(Tensor scales, Tensor! out, int D, bool is_sfb=False) -> ()");
  ops.impl("nvfp4_sf_linear_to_swizzled", torch::kCUDA, &nvfp4_sf_linear_to_swizzled);
}

TORCH_LIBRARY_EXPAND(flashrt_residual_norm_quant_b200, ops) {
  ops.def("rms_norm_bf16(Tensor x, Tensor weight, float eps, Tensor! out) -> ()");
  ops.def("residual_add_rms_norm_bf16(Tensor! residual, Tensor x, Tensor weight, float eps, Tensor! out) -> ()");
  ops.impl("rms_norm_bf16", torch::kCUDA, &rms_norm_bf16);
  ops.impl("residual_add_rms_norm_bf16", torch::kCUDA, &residual_add_rms_norm_bf16);
  ops.def("rms_norm_heads_bf16_(Tensor! x, Tensor weight_a, int heads_a, Tensor? weight_b, int heads_b, int head_dim, float eps) -> ()");
  ops.impl("rms_norm_heads_bf16_", torch::kCUDA, &rms_norm_heads_bf16_);
  ops.def("layer_norm_bf16(Tensor x, Tensor weight, Tensor bias, float eps, Tensor! out) -> ()");
  ops.def("rms_norm_quant_fp8_static_bf16(Tensor x, Tensor weight, Tensor scale, float eps, Tensor! out) -> ()");
  ops.def("residual_add_rms_norm_quant_fp8_static_bf16(Tensor! residual, Tensor x, Tensor weight, Tensor scale, float eps, Tensor! out) -> ()");
  ops.impl("layer_norm_bf16", torch::kCUDA, &layer_norm_bf16);
  ops.impl("rms_norm_quant_fp8_static_bf16", torch::kCUDA, &rms_norm_quant_fp8_static_bf16);
  ops.impl("residual_add_rms_norm_quant_fp8_static_bf16", torch::kCUDA, &residual_add_rms_norm_quant_fp8_static_bf16);
}

TORCH_LIBRARY_EXPAND(fp4_gemm_b200, ops) {
  ops.def("nvfp4_gemm_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor! out, float alpha=1.0, int variant=-1) -> ()");
  ops.def("fp4_w4a16_linear_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor! out, float alpha=1.0, int variant=-1) -> ()");
  ops.def("nvfp4_gemm_bias_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor bias, Tensor! out) -> ()");
  ops.def("nvfp4_gemm_bias_residual_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor bias, Tensor residual, Tensor! out) -> ()");
  ops.def("nvfp4_gemm_residual_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor residual, Tensor! out, float alpha=1.0) -> ()");
  ops.def("fp4_w4a4_gemv_warpsplit_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor! out, float alpha=1.0, int warps=4, int stages=4) -> ()");
  ops.def("fp4_repack_b_interleaved_sm120(Tensor b_packed, Tensor! b_interleaved) -> ()");
  ops.def("fp4_w4a4_gemv_warpsplit_interleaved_bf16(Tensor a_packed, Tensor b_interleaved, Tensor sfa, Tensor sfb, Tensor! out, float alpha=1.0, int warps=4, int stages=4) -> ()");
  ops.def("fp4_w4a4_gemm_warpsplit_mrows_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor! out, float alpha=1.0, int warps=2, int stages=6) -> ()");
  ops.def("quantize_fp4_sfa_fp16(Tensor x, Tensor! packed, Tensor! sfa, bool is_sfb=False) -> ()");
  ops.def("quantize_fp4_sfa_bf16(Tensor x, Tensor! packed, Tensor! sfa, bool is_sfb=False) -> ()");
  ops.def("dequantize_fp4_sfa_fp16(Tensor packed, Tensor sfa, Tensor! out, bool is_sfb=False) -> ()");
  // "_pdl" twins of the reference: every launch of this library is a programmatic dependent launch already
  ops.def("quantize_fp4_sfa_bf16_pdl(Tensor x, Tensor! packed, Tensor! sfa, bool is_sfb=False) -> ()");
  ops.def("fp4_w4a4_gemm_warpsplit_mrows_pdl_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor! out, float alpha=1.0, int warps=2, int stages=6) -> ()");
  ops.impl("quantize_fp4_sfa_bf16_pdl", torch::kCUDA, &quantize_fp4_sfa_bf16);
  ops.impl("fp4_w4a4_gemm_warpsplit_mrows_pdl_bf16", torch::kCUDA, &fp4_w4a4_gemm_warpsplit_mrows_bf16);
  ops.def("quantize_fp4_sfa_mse_fp16(Tensor x, Tensor! packed, Tensor! sfa, bool is_sfb=False) -> ()");
  ops.def("quantize_fp4_sfa_mse_bf16(Tensor x, Tensor! packed, Tensor! sfa, bool is_sfb=False) -> ()");
  ops.impl("quantize_fp4_sfa_mse_fp16", torch::kCUDA, &quantize_fp4_sfa_mse_fp16);
  ops.impl("quantize_fp4_sfa_mse_bf16", torch::kCUDA, &quantize_fp4_sfa_mse_bf16);
  ops.def("nvfp4_gemm_swiglu_nvfp4_bf16(Tensor a_packed, Tensor b_packed, Tensor sfa, Tensor sfb, Tensor! out_packed, Tensor! out_sfa, float alpha=1.0) -> ()");
  ops.impl("nvfp4_gemm_swiglu_nvfp4_bf16", torch::kCUDA, &nvfp4_gemm_swiglu_nvfp4_bf16);
  ops.impl("nvfp4_gemm_bf16", torch::kCUDA, &nvfp4_gemm_bf16);
  ops.impl("fp4_w4a16_linear_bf16", torch::kCUDA, &nvfp4_gemm_bf16);
  ops.impl("nvfp4_gemm_bias_bf16", torch::kCUDA, &nvfp4_gemm_bias_bf16);
  ops.impl("nvfp4_gemm_bias_residual_bf16", torch::kCUDA, &nvfp4_gemm_bias_residual_bf16);
  ops.impl("nvfp4_gemm_residual_bf16", torch::kCUDA, &nvfp4_gemm_residual_bf16);
  ops.impl("fp4_w4a4_gemv_warpsplit_bf16", torch::kCUDA, &fp4_w4a4_gemv_warpsplit_bf16);
  ops.impl("fp4_repack_b_interleaved_sm120", torch::kCUDA, &fp4_repack_b_interleaved_sm120);
  ops.impl("fp4_w4a4_gemv_warpsplit_interleaved_bf16", torch::kCUDA, &fp4_w4a4_gemv_warpsplit_interleaved_bf16);
  ops.impl("fp4_w4a4_gemm_warpsplit_mrows_bf16", torch::kCUDA, &fp4_w4a4_gemm_warpsplit_mrows_bf16);
  ops.impl("quantize_fp4_sfa_fp16", torch::kCUDA, &quantize_fp4_sfa_fp16);
  ops.impl("quantize_fp4_sfa_bf16", torch::kCUDA, &quantize_fp4_sfa_bf16);
  ops.impl("dequantize_fp4_sfa_fp16", torch::kCUDA, &dequantize_fp4_sfa_fp16);
}

TORCH_LIBRARY_EXPAND(fp4_fused_ops_b200, ops) {
  ops.def("sfa_size_bytes_for(Tensor anchor, int rows, int dim, bool is_sfb=False) -> int");
  ops.def("rms_norm_quantize_fp4_sfa_bf16(Tensor x, Tensor weight, float eps, Tensor! normed, Tensor! packed, Tensor! sfa) -> ()");
  ops.def("residual_add_rms_norm_nvfp4_bf16(Tensor! residual, Tensor x, Tensor? inv_s, float eps, Tensor! packed, Tensor! sfa) -> ()");
  ops.def("residual_add_rms_norm_quant_nvfp4_swizzled_bf16(Tensor! residual, Tensor x, Tensor weight, float eps, Tensor! packed, Tensor! sfa) -> ()");
  ops.def("residual_add_rms_norm_quant_nvfp4_ex(Tensor! residual, Tensor x, Tensor weight, float eps, float inv_global_scale, Tensor!? normed, Tensor! packed, Tensor! sfa) -> ()");
  ops.def("dequantize_fp4_sfa_fp16(Tensor packed, Tensor sfa, Tensor! out) -> ()");
  ops.def("silu_mul_quantize_fp4_sfa_bf16(Tensor merged, Tensor! packed, Tensor! sfa) -> ()");
  ops.def("residual_add_rms_norm_fp4_sfa_v2_fp16(Tensor! residual, Tensor x, Tensor! packed, Tensor! sfa) -> ()");
  ops.impl("residual_add_rms_norm_fp4_sfa_v2_fp16", torch::kCUDA, &residual_add_rms_norm_fp4_sfa_v2_fp16);
  ops.def("rms_norm_quant_nvfp4_ex(Tensor x, Tensor weight, float eps, Tensor!? normed, Tensor! packed, Tensor! sfa, bool one_plus_weight=False, bool round_bf16=True) -> ()");
  ops.impl("rms_norm_quant_nvfp4_ex", torch::kCUDA, &rms_norm_quant_nvfp4_ex);
  ops.impl("silu_mul_quantize_fp4_sfa_bf16", torch::kCUDA, &silu_mul_quantize_fp4_sfa_bf16);
  ops.impl("sfa_size_bytes_for", torch::kCUDA, &sfa_size_bytes_for);
  ops.impl("rms_norm_quantize_fp4_sfa_bf16", torch::kCUDA, &rms_norm_quantize_fp4_sfa_bf16);
  ops.impl("residual_add_rms_norm_nvfp4_bf16", torch::kCUDA, &residual_add_rms_norm_nvfp4_bf16);
  ops.impl("residual_add_rms_norm_quant_nvfp4_swizzled_bf16", torch::kCUDA,
           &residual_add_rms_norm_quant_nvfp4_swizzled_bf16);
  ops.impl("residual_add_rms_norm_quant_nvfp4_ex", torch::kCUDA, &residual_add_rms_norm_quant_nvfp4_ex);
  ops.impl("dequantize_fp4_sfa_fp16", torch::kCUDA, &dequantize_fp4_sfa_fp16_3);
}

TORCH_LIBRARY_EXPAND(grouped_moe_gemm_b200, ops) {
  ops.def("grouped_nvfp4_gemm_bf16_out(Tensor input, Tensor weight, Tensor input_scale, Tensor weight_scale, Tensor alpha, Tensor tile_expert, int tile_rows, int input_scale_stride, int weight_stride, int weight_scale_stride, Tensor! output) -> ()");
  ops.def("grouped_nvfp4_gemm_bf16_offsets_out(Tensor input, Tensor weight, Tensor input_scale, Tensor weight_scale, Tensor alpha, Tensor expert_offsets, Tensor! workspace, Tensor! output) -> ()");
  ops.def("grouped_nvfp4_gemm_workspace_size(int rows, int experts) -> int");
  ops.impl("grouped_nvfp4_gemm_bf16_out", torch::kCUDA, &grouped_nvfp4_gemm_bf16_legacy);
  ops.impl("grouped_nvfp4_gemm_bf16_offsets_out", torch::kCUDA, &grouped_nvfp4_gemm_bf16_offsets_out);
  ops.impl("grouped_nvfp4_gemm_workspace_size", &grouped_nvfp4_gemm_workspace_size);
  ops.def("moe_route_plan(Tensor topk_idx, int n_experts, Tensor! expert_offsets, Tensor! row_of_pair, Tensor! token_of_row) -> ()");
  ops.def("moe_gather_nvfp4(Tensor packed, Tensor sfa, Tensor token_of_row, Tensor! out_packed, Tensor! out_sfa) -> ()");
  ops.impl("moe_route_plan", torch::kCUDA, &moe_route_plan);
  ops.impl("moe_gather_nvfp4", torch::kCUDA, &moe_gather_nvfp4);
  ops.def("moe_quantize_scatter_nvfp4(Tensor x, Tensor row_of_pair, Tensor! out_packed, Tensor! out_sfa) -> ()");
  ops.impl("moe_quantize_scatter_nvfp4", torch::kCUDA, &moe_quantize_scatter_nvfp4);
}

REGISTER_EXTENSION(TORCH_EXTENSION_NAME)
