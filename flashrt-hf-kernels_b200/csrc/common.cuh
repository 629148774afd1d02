// Shared host/device helpers of the B200 NVFP4 path.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>

#include "flashrt_b200.h"

namespace frt {

extern std::atomic<int64_t> g_launches;     // kernels launched by this library
extern int g_opt_quant_encoder;             // FRT_OPT_QUANT_ENCODER
extern int g_opt_gemm_config;               // FRT_OPT_GEMM_CONFIG
extern int g_opt_pdl;                       // FRT_OPT_PDL: programmatic dependent launch (default on)
extern int g_opt_norm_form;                 // FRT_OPT_NORM_FORM: 0 automatic, 1 per-row-group, 2 streamed
extern int g_opt_tail_split;                // FRT_OPT_GEMM_TAIL_SPLIT: slice the last wave of the dense pair GEMM
extern int g_opt_split_k;                   // FRT_OPT_GEMM_SPLIT_K: cluster split-K of the small-M GEMM
extern int g_opt_wait_limit_log2;            // FRT_OPT_WAIT_LIMIT_LOG2: log2 of the SM-clock budget of device-side waits
extern int g_opt_grouped_form;               // FRT_OPT_GROUPED_FORM: 0 automatic, 1 weight-major, 2 token-major
extern int g_opt_smallm_stages;             // FRT_OPT_SMALLM_STAGES: ring depth of the small-M GEMM (0 = default)
#ifdef FRT_DEBUG
extern int g_opt_gemm_debug;                // experiment switches of the GEMM kernel (debug builds only)
#endif

// Status word written by kernels whose bounded waits ran out (one per device
// context, lives in device global memory of this library).
unsigned* device_status_word();

// SM clocks a device-side wait (mbarrier, peer flag) may spin before it gives up and reports through the status word
inline long long wait_limit_clocks() { return 1ll << g_opt_wait_limit_log2; }

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

inline int launch_result() {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return cudaGetLastError() == cudaSuccess ? FRT_OK : FRT_E_LAUNCH;
}

// Launch with the "programmatic stream serialization" attribute: the grid may start while the
// previous kernel of the stream is still running (its CTAs become resident as resources free up and
// run their prologue), and every kernel launched this way executes griddepcontrol.wait before it
// touches global memory, which blocks until the previous grid has completed and its writes are
// visible.  Hides launch latency and kernel prologues behind the predecessor's tail; capturable in
// CUDA graphs (programmatic edges).
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  if (g_opt_pdl) {
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned(const void* p, uintptr_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Byte offset of the UE4M3 scale of (row, 16-element block kb) in the swizzled
// buffer of a tensor with `sf_cols` = ceil(dim/64) 512-byte tiles per 128 rows.
__host__ __device__ __forceinline__ int64_t sf_offset(int row, int kb, int sf_cols) {
  return (static_cast<int64_t>(row >> 7) * sf_cols + (kb >> 2)) * 512 +
         (row & 31) * 16 + ((row >> 5) & 3) * 4 + (kb & 3);
}

#ifdef __CUDACC__
// Device side of launch_pdl (no-ops for a kernel launched without the attribute).
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- NVFP4 block quantiser -------------------------------------------------

// UE4M3 byte -> fp32 (exact).
__device__ __forceinline__ float ue4m3_to_float(uint8_t b) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}

// max(amax/6, 1e-12) -> UE4M3 byte (round to nearest even, saturating).
__device__ __forceinline__ uint8_t block_scale_byte(float amax) {
  float d = __fdiv_rn(amax, 6.f);
  if (d < 1e-12f) d = 1e-12f;
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(d, __NV_SATFINITE, __NV_E4M3));
}

// Rule A (thresholds, ties toward the smaller magnitude) by a compare chain.
// `!(a <= t)` keeps the NaN behaviour of an if/else-if chain of `<=`.
__device__ __forceinline__ uint32_t e2m1_rule_a_chain(float q) {
  const float a = fabsf(q);
  uint32_t m = 0;
  m += !(a <= 0.25f);
  m += !(a <= 0.75f);
  m += !(a <= 1.25f);
  m += !(a <= 1.75f);
  m += !(a <= 2.5f);
  m += !(a <= 3.5f);
  m += !(a <= 5.0f);
  return m | (q < 0.f ? 8u : 0u);
}

// Rule A through the hardware e2m1 conversion.  The conversion rounds to
// nearest even; replacing |q| by the float just below it with its lowest
// mantissa bit set puts the value strictly on the rule-A side of every
// threshold (thresholds have a clear low bit), so no tie is ever seen and the
// hardware result equals the compare chain.  The caller produces q as
// fma(v, inv, +0): the rounding of v*inv is unchanged and a -0 product becomes
// +0, whose sign bit the chain would not set.
//
// Two forms of the same map m -> (m - 1) | 1 on the magnitude bits m:
//  * integer form: correct for every input, infinities included;
//  * float form: q * (1 - 2^-24) rounded toward zero IS the float just below q
//    in magnitude (the exact product lies in (m-1, m-1/2] units of the last
//    place, and for m = 2^23 it is the largest float of the binade below), a
//    zero stays a zero, and the sign is untouched; `| 1` finishes the map.
//    One multiply on the FMA pipe and one logic op instead of five integer
//    ops.  It must not see an infinity (inf | 1 is a NaN); q is infinite only
//    in blocks whose scale byte is 0, which take the integer form.
__device__ __forceinline__ float rule_a_nudge(float q) {
  const uint32_t u = __float_as_uint(q);
  const uint32_t mag = u & 0x7fffffffu;
  const uint32_t nudged = (max(mag, 1u) - 1u) | 1u;
  return __uint_as_float((u & 0x80000000u) | nudged);
}
__device__ __forceinline__ float rule_a_nudge_finite(float q) {
  return __uint_as_float(__float_as_uint(__fmul_rz(q, 0x1.fffffep-1f)) | 1u);
}

__device__ __forceinline__ uint32_t e2m1x2_rule_a_hw(float q_lo, float q_hi) {
  return __nv_cvt_float2_to_fp4x2(make_float2(rule_a_nudge(q_lo), rule_a_nudge(q_hi)),
                                  __NV_E2M1, cudaRoundNearest);
}
__device__ __forceinline__ uint32_t e2m1x2_rule_a_hw_finite(float q_lo, float q_hi) {
  return __nv_cvt_float2_to_fp4x2(make_float2(rule_a_nudge_finite(q_lo), rule_a_nudge_finite(q_hi)),
                                  __NV_E2M1, cudaRoundNearest);
}

// Hardware round-to-nearest-even e2m1 pair ("rule B").
__device__ __forceinline__ uint32_t e2m1x2_rne_hw(float q_lo, float q_hi) {
  return __nv_cvt_float2_to_fp4x2(make_float2(q_lo, q_hi), __NV_E2M1, cudaRoundNearest);
}

enum : int { kEncHw = 0, kEncChain = 1, kEncRne = 2 };

// 1 / float(b) for every UE4M3 scale byte b (bit patterns of the fp32 results of the IEEE
// round-to-nearest division; b = 0 gives +inf).  One cached 4-byte load replaces the
// byte -> half -> float conversion and the division in the quantiser.
static __device__ __align__(16) const uint32_t kInvScaleBits[128] = {
    0x7f800000u, 0x44000000u, 0x43800000u, 0x432aaaabu, 0x43000000u, 0x42cccccdu, 0x42aaaaabu, 0x42924925u,
    0x42800000u, 0x42638e39u, 0x424ccccdu, 0x423a2e8cu, 0x422aaaabu, 0x421d89d9u, 0x42124925u, 0x42088889u,
    0x42000000u, 0x41e38e39u, 0x41cccccdu, 0x41ba2e8cu, 0x41aaaaabu, 0x419d89d9u, 0x41924925u, 0x41888889u,
    0x41800000u, 0x41638e39u, 0x414ccccdu, 0x413a2e8cu, 0x412aaaabu, 0x411d89d9u, 0x41124925u, 0x41088889u,
    0x41000000u, 0x40e38e39u, 0x40cccccdu, 0x40ba2e8cu, 0x40aaaaabu, 0x409d89d9u, 0x40924925u, 0x40888889u,
    0x40800000u, 0x40638e39u, 0x404ccccdu, 0x403a2e8cu, 0x402aaaabu, 0x401d89d9u, 0x40124925u, 0x40088889u,
    0x40000000u, 0x3fe38e39u, 0x3fcccccdu, 0x3fba2e8cu, 0x3faaaaabu, 0x3f9d89d9u, 0x3f924925u, 0x3f888889u,
    0x3f800000u, 0x3f638e39u, 0x3f4ccccdu, 0x3f3a2e8cu, 0x3f2aaaabu, 0x3f1d89d9u, 0x3f124925u, 0x3f088889u,
    0x3f000000u, 0x3ee38e39u, 0x3ecccccdu, 0x3eba2e8cu, 0x3eaaaaabu, 0x3e9d89d9u, 0x3e924925u, 0x3e888889u,
    0x3e800000u, 0x3e638e39u, 0x3e4ccccdu, 0x3e3a2e8cu, 0x3e2aaaabu, 0x3e1d89d9u, 0x3e124925u, 0x3e088889u,
    0x3e000000u, 0x3de38e39u, 0x3dcccccdu, 0x3dba2e8cu, 0x3daaaaabu, 0x3d9d89d9u, 0x3d924925u, 0x3d888889u,
    0x3d800000u, 0x3d638e39u, 0x3d4ccccdu, 0x3d3a2e8cu, 0x3d2aaaabu, 0x3d1d89d9u, 0x3d124925u, 0x3d088889u,
    0x3d000000u, 0x3ce38e39u, 0x3ccccccdu, 0x3cba2e8cu, 0x3caaaaabu, 0x3c9d89d9u, 0x3c924925u, 0x3c888889u,
    0x3c800000u, 0x3c638e39u, 0x3c4ccccdu, 0x3c3a2e8cu, 0x3c2aaaabu, 0x3c1d89d9u, 0x3c124925u, 0x3c088889u,
    0x3c000000u, 0x3be38e39u, 0x3bcccccdu, 0x3bba2e8cu, 0x3baaaaabu, 0x3b9d89d9u, 0x3b924925u, 0x3b888889u,
    0x3b800000u, 0x3b638e39u, 0x3b4ccccdu, 0x3b3a2e8cu, 0x3b2aaaabu, 0x3b1d89d9u, 0x3b124925u, 0x3b088889u
};

__device__ __forceinline__ const float* inv_scale_table() {
  return reinterpret_cast<const float*>(kInvScaleBits);
}

// max |v_i| over 16 values with the three-input max of sm_100 (max is exact, so the
// grouping does not matter; a NaN operand is ignored like fmaxf does).
__device__ __forceinline__ float max3_abs(float a, float b, float c) {
  float r;
  asm("max.abs.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float amax16(const float (&v)[16]) {
  const float a = max3_abs(v[0], v[1], v[2]), b = max3_abs(v[3], v[4], v[5]);
  const float c = max3_abs(v[6], v[7], v[8]), d = max3_abs(v[9], v[10], v[11]);
  const float e = max3_abs(v[12], v[13], v[14]);
  return max3_abs(max3_abs(a, b, c), max3_abs(d, e, v[15]), 0.f);
}

// Encode 16 fp32 values with the reciprocal `inv` of the block scale: 8 packed bytes.
// FINITE selects the float form of the nudge (the caller guarantees a non-zero scale).
template <int ENC, bool FINITE>
__device__ __forceinline__ uint2 encode_block16(const float (&v)[16], float inv) {
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int p = 0; p < 8; ++p) {
    float q0, q1;
    if (ENC == kEncHw) {
      q0 = __fmaf_rn(v[2 * p], inv, 0.f);
      q1 = __fmaf_rn(v[2 * p + 1], inv, 0.f);
    } else {
      q0 = __fmul_rn(v[2 * p], inv);
      q1 = __fmul_rn(v[2 * p + 1], inv);
    }
    uint32_t byte;
    if (ENC == kEncHw) byte = FINITE ? e2m1x2_rule_a_hw_finite(q0, q1) : e2m1x2_rule_a_hw(q0, q1);
    else if (ENC == kEncRne) byte = e2m1x2_rne_hw(q0, q1);
    else byte = e2m1_rule_a_chain(q0) | (e2m1_rule_a_chain(q1) << 4);
    w[p >> 2] |= (byte & 0xffu) << (8 * (p & 3));
  }
  return make_uint2(w[0], w[1]);
}

// Quantise 16 fp32 values: returns 8 packed bytes in a uint2 and the scale byte.
// `inv_lut`, when given, is a 128-entry table of 1/float(scale byte) (the results of the
// same IEEE division), replacing the conversion and the division.
template <int ENC>
__device__ __forceinline__ uint2 quantize_block16(const float (&v)[16], uint8_t& sf_byte,
                                                  const float* inv_lut = nullptr) {
  sf_byte = block_scale_byte(amax16(v));
  const float inv = inv_lut ? __ldg(inv_lut + (sf_byte & 0x7f)) : __fdiv_rn(1.f, ue4m3_to_float(sf_byte));
  if (ENC == kEncHw && sf_byte != 0) return encode_block16<ENC, true>(v, inv);
  return encode_block16<ENC, false>(v, inv);
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& raw, float* out) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// SwiGLU stage of the NVFP4 producer: bf16((g / (1 + exp(-g))) * u) as fp32, every step a
// separately rounded fp32 operation (accurate expf, IEEE division), which is what the
// reference's kernel evaluates.
__device__ __forceinline__ float swiglu_bf16(float g, float u) {
  const float s = __fdiv_rn(g, __fadd_rn(1.f, expf(-g)));
  return __bfloat162float(__float2bfloat16_rn(__fmul_rn(s, u)));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
#endif  // __CUDACC__

}  // namespace frt
