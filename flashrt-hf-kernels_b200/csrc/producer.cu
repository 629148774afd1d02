// HBM-bound kernels of the NVFP4 path: scale-factor layout, stand-alone
// quantiser / dequantiser, and the fused (residual-add +) RMSNorm -> NVFP4
// producer.  Hand-written for sm_100a; every kernel touches each byte of its
// operands exactly once, with 128-bit loads.
#include "common.cuh"
#include "ptx.cuh"

namespace frt {

std::atomic<int64_t> g_launches{0};
int g_opt_quant_encoder = 0;
int g_opt_gemm_config = 0;
int g_opt_pdl = 1;
int g_opt_norm_form = 0;
int g_opt_tail_split = 1;
int g_opt_split_k = 1;
int g_opt_smallm_stages = 0;
int g_opt_wait_limit_log2 = 31;
int g_opt_grouped_form = 0;
#ifdef FRT_DEBUG
int g_opt_gemm_debug = 0;
#endif

namespace {

// Stores the scale byte of block kb of `row`; the thread that owns the row's last block also zeroes the
// (up to three) padding bytes that complete the row's last 64-element group when dim % 64 != 0: the tensor
// cores read whole groups, and a NaN pattern left there would poison the (zero) padding products.
__device__ __forceinline__ void store_scale(uint8_t* sf, int row, int kb, int nb, int sf_cols, uint8_t value) {
  sf[sf_offset(row, kb, sf_cols)] = value;
  if (kb == nb - 1)
    for (int j = nb; j < 4 * sf_cols; ++j) sf[sf_offset(row, j, sf_cols)] = 0;
}

// ---------------------------------------------------------------------------
// linear [rows, nb] -> swizzled.  One thread moves the 4 scale bytes of one
// (row, 64-element group): a 4-byte read (or byte reads at a ragged edge) and
// one aligned 4-byte write.
// ---------------------------------------------------------------------------
__global__ void sf_linear_to_swizzled_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                             int rows, int nb, int sf_cols, bool vec_ok) {
  const int g = blockIdx.x * blockDim.x + threadIdx.x;   // 4-block group in the row
  const int row = blockIdx.y;
  if (g >= sf_cols) return;
  const uint8_t* s = src + static_cast<int64_t>(row) * nb + 4 * g;
  uint8_t* d = dst + sf_offset(row, 4 * g, sf_cols);
  if (vec_ok && 4 * g + 4 <= nb) {
    *reinterpret_cast<uint32_t*>(d) = *reinterpret_cast<const uint32_t*>(s);
  } else {
    for (int j = 0; j < 4; ++j) d[j] = 4 * g + j < nb ? s[j] : 0;   // padding of the last group: zero
  }
}

// ---------------------------------------------------------------------------
// Stand-alone quantiser: one thread per 16-element block (two 16-byte loads,
// one 8-byte store); a warp covers 1 KiB of one row.
// ---------------------------------------------------------------------------
template <int ENC, bool FP16>
__global__ void __launch_bounds__(256)
quantize_kernel(const uint4* __restrict__ src, uint2* __restrict__ packed, uint8_t* __restrict__ sf,
                int rows, int nb, int sf_cols) {
  // No early griddepcontrol.launch_dependents here: this kernel also packs WEIGHTS, and the small-M GEMM
  // loads its weight operand before it waits on the previous grid.  Without the trigger a dependent grid
  // starts only when this one has completed, so a GEMM enqueued right after a weight pack sees whole weights.
  pdl_wait();
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(rows) * nb) return;
  const int row = static_cast<int>(idx / nb);
  const int kb = static_cast<int>(idx - static_cast<int64_t>(row) * nb);
  const uint4 r0 = __ldcs(src + 2 * idx);
  const uint4 r1 = __ldcs(src + 2 * idx + 1);
  float v[16];
  if (FP16) {
    const __half2* h0 = reinterpret_cast<const __half2*>(&r0);
    const __half2* h1 = reinterpret_cast<const __half2*>(&r1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __half22float2(h0[i]);
      const float2 b = __half22float2(h1[i]);
      v[2 * i] = a.x; v[2 * i + 1] = a.y;
      v[8 + 2 * i] = b.x; v[8 + 2 * i + 1] = b.y;
    }
  } else {
    unpack_bf16x8(r0, v);
    unpack_bf16x8(r1, v + 8);
  }
  uint8_t sfb;
  const uint2 out = quantize_block16<ENC>(v, sfb, inv_scale_table());
  packed[idx] = out;
  store_scale(sf, row, kb, nb, sf_cols, sfb);
}

// ---------------------------------------------------------------------------
// Bind-time weight packer with a per-block scale search: of nine candidate scales
// e4m3(max(amax * (1/6) * m, 1e-12)), m in {.375 ... 1.5}, keep the first with the lowest
// squared reconstruction error (fp32, fused multiply-adds as the reference's compiled
// kernel evaluates them), then encode with it.  Not a hot-path kernel.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float e2m1_code_value(uint32_t c) {
  const uint32_t m = c & 7u;
  const float mag = m < 2 ? 0.5f * m : (m & 1 ? 1.5f : 1.0f) * static_cast<float>(1 << ((m >> 1) - 1));
  return (c & 8u) ? -mag : mag;
}

template <bool FP16>
__global__ void __launch_bounds__(256)
quantize_mse_kernel(const uint4* __restrict__ src, uint2* __restrict__ packed, uint8_t* __restrict__ sf,
                    int rows, int nb, int sf_cols) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(rows) * nb) return;
  const int row = static_cast<int>(idx / nb);
  const int kb = static_cast<int>(idx - static_cast<int64_t>(row) * nb);
  const uint4 r0 = __ldcs(src + 2 * idx);
  const uint4 r1 = __ldcs(src + 2 * idx + 1);
  float v[16];
  if (FP16) {
    const __half2* h0 = reinterpret_cast<const __half2*>(&r0);
    const __half2* h1 = reinterpret_cast<const __half2*>(&r1);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __half22float2(h0[i]);
      const float2 b = __half22float2(h1[i]);
      v[2 * i] = a.x; v[2 * i + 1] = a.y;
      v[8 + 2 * i] = b.x; v[8 + 2 * i + 1] = b.y;
    }
  } else {
    unpack_bf16x8(r0, v);
    unpack_bf16x8(r1, v + 8);
  }
  const float amax = amax16(v);
  const float base = __fmul_rn(amax, 1.f / 6.f);
  const float mult[9] = {.375f, .5f, .625f, .75f, .875f, 1.f, 1.125f, 1.25f, 1.5f};
  float best_err = INFINITY;
  uint8_t best = static_cast<uint8_t>(__nv_cvt_float_to_fp8(1e-12f, __NV_SATFINITE, __NV_E4M3));
#pragma unroll 1
  for (int c = 0; c < 9; ++c) {
    const float want = fmaxf(fmaxf(__fmul_rn(base, mult[c]), 1e-12f), 0.f);
    const uint8_t sq = static_cast<uint8_t>(__nv_cvt_float_to_fp8(want, __NV_SATFINITE, __NV_E4M3));
    const float scale = ue4m3_to_float(sq);
    const float inv = __fdiv_rn(1.f, scale);
    float err = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t q = e2m1_rule_a_chain(__fmul_rn(v[i], inv));
      const float delta = __fmaf_rn(e2m1_code_value(q), scale, -v[i]);
      err = __fmaf_rn(delta, delta, err);
    }
    if (err < best_err) { best_err = err; best = sq; }
  }
  const float inv = __fdiv_rn(1.f, ue4m3_to_float(best));
  packed[idx] = encode_block16<kEncChain, false>(v, inv);
  store_scale(sf, row, kb, nb, sf_cols, best);
}

// ---------------------------------------------------------------------------
// SwiGLU -> NVFP4: merged = [gate | up] bf16 (rows, 2H); one thread per 16 outputs
// (two 16-byte loads from each half, one 8-byte store).  Instruction-bound (an
// exponential and a division per element): the GEMM epilogue form of the same
// arithmetic (gemm_pair.cuh) is the fast path, this kernel the stand-alone op.
// ---------------------------------------------------------------------------
template <int ENC>
__global__ void __launch_bounds__(256)
silu_mul_quant_kernel(const uint4* __restrict__ merged, uint2* __restrict__ packed, uint8_t* __restrict__ sf,
                      int rows, int nb, int sf_cols) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(rows) * nb) return;
  const int row = static_cast<int>(idx / nb);
  const int kb = static_cast<int>(idx - static_cast<int64_t>(row) * nb);
  const uint4* g_src = merged + static_cast<int64_t>(row) * (4 * nb) + 2 * kb;
  const uint4* u_src = g_src + 2 * nb;
  float g[16], u[16], v[16];
  unpack_bf16x8(__ldcs(g_src), g);
  unpack_bf16x8(__ldcs(g_src + 1), g + 8);
  unpack_bf16x8(__ldcs(u_src), u);
  unpack_bf16x8(__ldcs(u_src + 1), u + 8);
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = swiglu_bf16(g[j], u[j]);
  uint8_t sfb;
  const uint2 out = quantize_block16<ENC>(v, sfb, inv_scale_table());
  packed[idx] = out;
  store_scale(sf, row, kb, nb, sf_cols, sfb);
}

// ---------------------------------------------------------------------------
// Dequantiser (validation helper): one thread per block, fp16 out.
// ---------------------------------------------------------------------------
__global__ void dequantize_kernel(const uint2* __restrict__ packed, const uint8_t* __restrict__ sf,
                                  uint4* __restrict__ out, int rows, int nb, int sf_cols) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(rows) * nb) return;
  const int row = static_cast<int>(idx / nb);
  const int kb = static_cast<int>(idx - static_cast<int64_t>(row) * nb);
  const float s = ue4m3_to_float(sf[sf_offset(row, kb, sf_cols)]);
  const uint2 p = packed[idx];
  const uint32_t w[2] = {p.x, p.y};
  __align__(16) __half h[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const uint32_t c = (w[i >> 3] >> (4 * (i & 7))) & 0xfu;
    const uint32_t m = c & 7u;
    // e2m1 magnitudes 0,.5,1,1.5,2,3,4,6
    const float mag = m < 2 ? 0.5f * m : (m & 1 ? 1.5f : 1.0f) * static_cast<float>(1 << ((m >> 1) - 1));
    h[i] = __float2half_rn((c & 8u) ? -mag * s : mag * s);
  }
  out[2 * idx] = *reinterpret_cast<uint4*>(h);
  out[2 * idx + 1] = *reinterpret_cast<uint4*>(h + 8);
}

// ---------------------------------------------------------------------------
// Fused (residual-add +) RMSNorm (-> NVFP4).
//
// One thread owns one 16-element block of a row for the whole kernel: two
// 16-byte loads per input tensor, the values stay in registers through the
// row reduction, then scale / quantise / store.  A row of nb = dim/16 blocks
// is covered by TPR threads (a power of two >= nb, 32..1024); a CTA is
// max(TPR, 256) threads and holds 256/TPR rows when TPR < 256.  Consecutive
// threads read consecutive 32-byte pieces, so every warp access is one
// contiguous 1 KiB segment, and global memory is read once and written once.
// Small per-thread state (about 50 registers) keeps all 64 warps of an SM
// resident, which is what hides the HBM latency.
//
// The summation order is fixed so that a CPU restatement reproduces rstd bit
// for bit: each thread sums v*v over its 16 elements in order (separately
// rounded multiply and add), a warp combines its 32 threads with an xor
// butterfly (offsets 16,8,4,2,1), and the row total adds the warp totals in
// warp order.
// ---------------------------------------------------------------------------
struct NormParams {
  uint4* residual;        // bf16 [rows, dim] or null (in/out)
  const uint4* x;         // bf16 [rows, dim]
  const uint4* weight;    // bf16 [dim] or null
  uint4* normed;          // bf16 [rows, dim] or null
  uint2* packed;          // u8   [rows, dim/2] or null when QUANT is false
  uint8_t* sf;            // swizzled scales
  uint4* out_fp8;         // e4m3 [rows, dim] or null: static-scale FP8 output of the normalised values
  const float* fp8_scale; // device scalar: out_fp8 = e4m3(clamp(v / scale, +-448))
  int rows, nb, sf_cols;
  float eps, inv_global_scale;
  float dim_f;
  unsigned flags;
};

// 16 fp32 values -> 16 e4m3 bytes with a static scale: e4m3_rn(clamp(v * inv_scale, +-448))
// (flashrt-residual-norm-quant/csrc/residual_norm_quant.cu:54-57).
__device__ __forceinline__ uint4 fp8_static16(const float (&v)[16], float inv_scale) {
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t word = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float q = fminf(fmaxf(__fmul_rn(v[4 * i + j], inv_scale), -448.f), 448.f);
      word |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(q, __NV_SATFINITE, __NV_E4M3)) << (8 * j);
    }
    w[i] = word;
  }
  return make_uint4(w[0], w[1], w[2], w[3]);
}

__device__ __forceinline__ void pack16_bf16(const float (&v)[16], uint4& o0, uint4& o1) {
  o0.x = pack_bf16x2(v[0], v[1]);   o0.y = pack_bf16x2(v[2], v[3]);
  o0.z = pack_bf16x2(v[4], v[5]);   o0.w = pack_bf16x2(v[6], v[7]);
  o1.x = pack_bf16x2(v[8], v[9]);   o1.y = pack_bf16x2(v[10], v[11]);
  o1.z = pack_bf16x2(v[12], v[13]); o1.w = pack_bf16x2(v[14], v[15]);
}

// 8 packed 16-bit values <-> fp32, bf16 or (FP16) IEEE half
template <bool FP16>
__device__ __forceinline__ void unpack8(const uint4& raw, float* out) {
  if (FP16) {
    const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __half22float2(h[i]);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  } else {
    unpack_bf16x8(raw, out);
  }
}
template <bool FP16>
__device__ __forceinline__ void pack16(const float (&v)[16], uint4& o0, uint4& o1) {
  if (FP16) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __half2 h = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    o0 = make_uint4(w[0], w[1], w[2], w[3]);
    o1 = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    pack16_bf16(v, o0, o1);
  }
}

// FP16: activations and residual are IEEE half instead of bf16 (the weight, when given, stays bf16).
template <int TPR, bool HAS_RES, bool QUANT, int ENC, bool FP16 = false>
__global__ void __launch_bounds__(TPR > 256 ? TPR : 256)
norm_quant_kernel(const NormParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CTA = TPR > 256 ? TPR : 256;
  constexpr int ROWS_PER_CTA = CTA / TPR;
  constexpr int WPR = TPR >= 32 ? TPR / 32 : 1;       // warps per row (TPR = 8, 16: several rows per warp)
  __shared__ float warp_sums[CTA / 32];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row = blockIdx.x * ROWS_PER_CTA + threadIdx.x / TPR;
  const int s = threadIdx.x % TPR;                    // block index inside the row
  const bool ok = row < p.rows && s < p.nb;
  const int64_t idx = static_cast<int64_t>(row) * p.nb + s;

  float v[16];
  uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0, r0 = x0, r1 = x0, g0 = x0, g1 = x0;
  // A few rows (decode): the kernel is a chain of dependent trips to L2, so the norm weight travels with the
  // activations instead of after the row reduction, and the quantiser divides instead of looking its
  // reciprocal scale up in a table in global memory (the same IEEE division: identical bytes).
  const bool few_rows = p.rows <= 16;
  if (ok) {
    x0 = __ldcs(p.x + 2 * idx);
    x1 = __ldcs(p.x + 2 * idx + 1);
    if (HAS_RES) {
      r0 = __ldcs(p.residual + 2 * idx);
      r1 = __ldcs(p.residual + 2 * idx + 1);
    }
    if (few_rows && p.weight != nullptr) {
      g0 = __ldg(p.weight + 2 * s);
      g1 = __ldg(p.weight + 2 * s + 1);
    }
  }
  unpack8<FP16>(x0, v);
  unpack8<FP16>(x1, v + 8);
  float part = 0.f;
  if (HAS_RES) {
    float r[16];
    unpack8<FP16>(r0, r);
    unpack8<FP16>(r1, r + 8);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __fadd_rn(r[j], v[j]);
    uint4 o0, o1;
    pack16<FP16>(v, o0, o1);
    if (ok) {
      __stcs(p.residual + 2 * idx, o0);
      __stcs(p.residual + 2 * idx + 1, o1);
    }
    // the sum of squares always comes from the fp32 sums
#pragma unroll
    for (int j = 0; j < 16; ++j) part = __fadd_rn(part, __fmul_rn(v[j], v[j]));
    if (p.flags & FRT_PRODUCER_NORM_FROM_BF16_RESIDUAL) {   // norm input = the rounded residual
      unpack8<FP16>(o0, v);
      unpack8<FP16>(o1, v + 8);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) part = __fadd_rn(part, __fmul_rn(v[j], v[j]));
  }

  // ---- row reduction -------------------------------------------------------
  // (rows of at most 8 / 16 blocks share a warp: the butterfly stays inside the row's aligned group of lanes;
  // the offsets it skips would only add the zeros of lanes that own no block, so the sum is the same bits)
#pragma unroll
  for (int o = TPR >= 32 ? 16 : TPR / 2; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
  float ssq = part;
  if (WPR > 1) {
    if (lane == 0) warp_sums[warp] = part;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    ssq = warp_sums[first];
#pragma unroll
    for (int w = 1; w < WPR; ++w) ssq = __fadd_rn(ssq, warp_sums[first + w]);
  }
  if (!ok) return;
  const float rstd = __frsqrt_rn(__fadd_rn(__fdiv_rn(ssq, p.dim_f), p.eps));

  // ---- scale, (round,) quantise, store -------------------------------------
  if (p.weight != nullptr) {
    float g[16];
    if (!few_rows) {
      g0 = __ldg(p.weight + 2 * s);
      g1 = __ldg(p.weight + 2 * s + 1);
    }
    unpack_bf16x8(g0, g);
    unpack_bf16x8(g1, g + 8);
    if (p.flags & FRT_PRODUCER_ONE_PLUS_W) {
#pragma unroll
      for (int j = 0; j < 16; ++j) g[j] = __fadd_rn(1.f, g[j]);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], rstd), g[j]);
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(v[j], rstd);
  }
  if (p.inv_global_scale != 1.0f) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(v[j], p.inv_global_scale);
  }
  const bool round_bf16 = p.flags & FRT_PRODUCER_ROUND_BF16;
  if (p.normed != nullptr || round_bf16) {
    uint4 o0, o1;
    pack16_bf16(v, o0, o1);
    if (p.normed != nullptr) {
      p.normed[2 * idx] = o0;
      p.normed[2 * idx + 1] = o1;
    }
    if (round_bf16) {
      unpack_bf16x8(o0, v);
      unpack_bf16x8(o1, v + 8);
    }
  }
  if (!QUANT && p.out_fp8 != nullptr) p.out_fp8[idx] = fp8_static16(v, __fdiv_rn(1.f, __ldg(p.fp8_scale)));
  if (QUANT) {
    uint8_t sfb;
    uint2 out;
    const float* lut = few_rows ? nullptr : inv_scale_table();
    if (p.flags & FRT_PRODUCER_RNE_E2M1) out = quantize_block16<kEncRne>(v, sfb, lut);
    else out = quantize_block16<ENC>(v, sfb, lut);
    p.packed[idx] = out;
    store_scale(p.sf, row, s, p.nb, p.sf_cols, sfb);
  }
}

// ---------------------------------------------------------------------------
// LayerNorm (bf16, affine weight and bias): the same one-thread-per-block cover as the RMSNorm
// kernel with two row reductions (mean, then the squared deviations), fp32 throughout:
//   y = bf16(((x - mean) * inv_std) * w + b).
// Summation order of each reduction: thread over its 16 elements in order, warp butterfly,
// warps in order.
// ---------------------------------------------------------------------------
template <int TPR>
__global__ void __launch_bounds__(TPR > 256 ? TPR : 256)
layer_norm_kernel(const uint4* __restrict__ x, const uint4* __restrict__ weight, const uint4* __restrict__ bias,
                  uint4* __restrict__ out, int rows, int nb, float dim_f, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CTA = TPR > 256 ? TPR : 256;
  constexpr int ROWS_PER_CTA = CTA / TPR;
  constexpr int WPR = TPR / 32;
  __shared__ float warp_sums[2][CTA / 32];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row = blockIdx.x * ROWS_PER_CTA + threadIdx.x / TPR;
  const int s = threadIdx.x % TPR;
  const bool ok = row < rows && s < nb;
  const int64_t idx = static_cast<int64_t>(row) * nb + s;
  float v[16];
  uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
  if (ok) {
    x0 = __ldcs(x + 2 * idx);
    x1 = __ldcs(x + 2 * idx + 1);
  }
  unpack_bf16x8(x0, v);
  unpack_bf16x8(x1, v + 8);
  auto row_total = [&](float part, int buf) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
    float total = part;
    if (WPR > 1) {
      if (lane == 0) warp_sums[buf][warp] = part;
      __syncthreads();
      const int first = (warp / WPR) * WPR;
      total = warp_sums[buf][first];
#pragma unroll
      for (int w = 1; w < WPR; ++w) total = __fadd_rn(total, warp_sums[buf][first + w]);
    }
    return total;
  };
  float part = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) part = __fadd_rn(part, v[j]);
  const float mean = __fdiv_rn(row_total(part, 0), dim_f);
  part = 0.f;
  if (ok) {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float d = __fsub_rn(v[j], mean);
      part = __fadd_rn(part, __fmul_rn(d, d));
    }
  }
  const float inv_std = __frsqrt_rn(__fadd_rn(__fdiv_rn(row_total(part, 1), dim_f), eps));
  if (!ok) return;
  float g[16], b[16];
  unpack_bf16x8(__ldg(weight + 2 * s), g);
  unpack_bf16x8(__ldg(weight + 2 * s + 1), g + 8);
  unpack_bf16x8(__ldg(bias + 2 * s), b);
  unpack_bf16x8(__ldg(bias + 2 * s + 1), b + 8);
#pragma unroll
  for (int j = 0; j < 16; ++j)
    v[j] = __fadd_rn(__fmul_rn(__fmul_rn(__fsub_rn(v[j], mean), inv_std), g[j]), b[j]);
  uint4 o0, o1;
  pack16_bf16(v, o0, o1);
  out[2 * idx] = o0;
  out[2 * idx + 1] = o1;
}

template <int TPR>
int launch_layer_norm(const uint4* x, const uint4* w, const uint4* b, uint4* out, int rows, int nb, float dim_f,
                      float eps, cudaStream_t st) {
  constexpr int CTA = TPR > 256 ? TPR : 256;
  constexpr int rows_per_cta = CTA / TPR;
  launch_pdl(layer_norm_kernel<TPR>, dim3((rows + rows_per_cta - 1) / rows_per_cta), dim3(CTA), 0, st, x, w, b, out,
             rows, nb, dim_f, eps);
  return launch_result();
}

// ---------------------------------------------------------------------------
// Streaming form of the same kernel: persistent CTAs, inputs staged through
// shared memory by bulk copies (TMA engine), three row groups deep.
//
// A "group" is the rows one CTA pass covers (CTA / TPR rows, contiguous in
// memory).  Thread 0 keeps bulk copies of the next groups in flight, so HBM
// latency is covered by whole groups of bytes per CTA rather than by the few
// loads a warp can issue before it starts computing; the threads read their 32
// bytes per tensor from shared memory.  The row-sum barrier doubles as the
// "stage is free" signal: once every thread is past it, the stage's data is in
// registers and thread 0 refills it.  Per-thread state that does not change
// from row to row (the weight in fp32) is set up once per CTA.  Arithmetic, operation order and results are those of
// norm_quant_kernel.
// ---------------------------------------------------------------------------
constexpr int kStreamStages = 3;

__device__ __forceinline__ void st_global_v8(void* dst, const uint4& a, const uint4& b) {
  asm volatile("st.global.cs.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
               ::"l"(dst), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}

template <int TPR, bool HAS_RES, bool QUANT, int ENC>
__global__ void __launch_bounds__(TPR > 256 ? TPR : 256, TPR > 256 ? 1024 / TPR : 4)
norm_quant_stream_kernel(const NormParams p, unsigned* status, long long wait_limit) {
  constexpr int CTA = TPR > 256 ? TPR : 256;
  constexpr int RPC = CTA / TPR;                      // rows per group
  constexpr int WPR = TPR / 32;                       // warps per row
  constexpr int TENSORS = HAS_RES ? 2 : 1;
  constexpr int STAGE_STRIDE = CTA * 32;              // bytes per tensor per stage
  extern __shared__ __align__(128) unsigned char stage_mem[];
  __shared__ uint64_t full[kStreamStages];
  __shared__ float warp_sums[2][CTA / 32];

  const int tid = threadIdx.x;
  const int lane = tid & 31, warp = tid >> 5;
  const int local_row = tid / TPR;
  const int s = tid % TPR;                            // block index inside the row
  const int n_groups = (p.rows + RPC - 1) / RPC;
  const uint32_t row_bytes = static_cast<uint32_t>(p.nb) * 32u;
  pdl_launch_dependents();
  pdl_wait();

  auto issue = [&](int group, int stage) {            // thread 0 only
    const int row0 = group * RPC;
    const int nrows = min(RPC, p.rows - row0);
    const uint32_t bytes = static_cast<uint32_t>(nrows) * row_bytes;
    unsigned char* dst = stage_mem + static_cast<size_t>(stage) * TENSORS * STAGE_STRIDE;
    const size_t src_off = static_cast<size_t>(row0) * row_bytes;
    ptx::mbar_expect_tx(&full[stage], bytes * TENSORS);
    ptx::bulk_load(dst, reinterpret_cast<const unsigned char*>(p.x) + src_off, bytes, &full[stage]);
    if (HAS_RES)
      ptx::bulk_load(dst + STAGE_STRIDE, reinterpret_cast<const unsigned char*>(p.residual) + src_off, bytes,
                     &full[stage]);
  };

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < kStreamStages; ++i) ptx::mbar_init(&full[i], 1);
    ptx::fence_barrier_init();
#pragma unroll
    for (int i = 0; i < kStreamStages; ++i) {
      const int g = blockIdx.x + i * gridDim.x;
      if (g < n_groups) issue(g, i);
    }
  }

  // per-thread weight (fp32), fixed for the kernel
  float g[16];
  const bool has_w = p.weight != nullptr;
  if (has_w && s < p.nb) {
    unpack_bf16x8(__ldg(p.weight + 2 * s), g);
    unpack_bf16x8(__ldg(p.weight + 2 * s + 1), g + 8);
    if (p.flags & FRT_PRODUCER_ONE_PLUS_W) {
#pragma unroll
      for (int j = 0; j < 16; ++j) g[j] = __fadd_rn(1.f, g[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) g[j] = 1.f;
  }
  __syncthreads();                                    // barriers initialised

  int it = 0;
  for (int group = blockIdx.x; group < n_groups; group += gridDim.x, ++it) {
    const int stage = it % kStreamStages;
    const uint32_t parity = (it / kStreamStages) & 1;
    if (!ptx::mbar_wait_bounded(&full[stage], parity, wait_limit)) atomicOr(status, 0x100u);
    const int row = group * RPC + local_row;
    const bool ok = row < p.rows && s < p.nb;
    const int64_t idx = static_cast<int64_t>(row) * p.nb + s;

    float v[16];
    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0, r0 = x0, r1 = x0;
    if (ok) {
      const uint4* sx = reinterpret_cast<const uint4*>(
          stage_mem + static_cast<size_t>(stage) * TENSORS * STAGE_STRIDE + static_cast<size_t>(local_row) * row_bytes) + 2 * s;
      x0 = sx[0];
      x1 = sx[1];
      if (HAS_RES) {
        const uint4* sr = reinterpret_cast<const uint4*>(reinterpret_cast<const unsigned char*>(sx) + STAGE_STRIDE);
        r0 = sr[0];
        r1 = sr[1];
      }
    }
    unpack_bf16x8(x0, v);
    unpack_bf16x8(x1, v + 8);
    float part = 0.f;
    if (HAS_RES) {
      float r[16];
      unpack_bf16x8(r0, r);
      unpack_bf16x8(r1, r + 8);
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = __fadd_rn(r[j], v[j]);
      uint4 o0, o1;
      pack16_bf16(v, o0, o1);
      if (ok) st_global_v8(p.residual + 2 * idx, o0, o1);
#pragma unroll
      for (int j = 0; j < 16; ++j) part = __fadd_rn(part, __fmul_rn(v[j], v[j]));
      if (p.flags & FRT_PRODUCER_NORM_FROM_BF16_RESIDUAL) {
        unpack_bf16x8(o0, v);
        unpack_bf16x8(o1, v + 8);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j) part = __fadd_rn(part, __fmul_rn(v[j], v[j]));
    }

#pragma unroll
    for (int o = 16; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
    float ssq = part;
    if (WPR > 1 && lane == 0) warp_sums[it & 1][warp] = part;
    __syncthreads();                                  // warp sums visible; stage data is in registers
    if (tid == 0) {
      const int next = group + kStreamStages * gridDim.x;
      if (next < n_groups) issue(next, stage);
    }
    if (WPR > 1) {
      const int first = (warp / WPR) * WPR;
      ssq = warp_sums[it & 1][first];
#pragma unroll
      for (int w = 1; w < WPR; ++w) ssq = __fadd_rn(ssq, warp_sums[it & 1][first + w]);
    }
    if (ok) {
      const float rstd = __frsqrt_rn(__fadd_rn(__fdiv_rn(ssq, p.dim_f), p.eps));
      if (has_w) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], rstd), g[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(v[j], rstd);
      }
      if (p.inv_global_scale != 1.0f) {
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(v[j], p.inv_global_scale);
      }
      const bool round_bf16 = p.flags & FRT_PRODUCER_ROUND_BF16;
      if (p.normed != nullptr || round_bf16) {
        uint4 o0, o1;
        pack16_bf16(v, o0, o1);
        if (p.normed != nullptr) {
          p.normed[2 * idx] = o0;
          p.normed[2 * idx + 1] = o1;
        }
        if (round_bf16) {
          unpack_bf16x8(o0, v);
          unpack_bf16x8(o1, v + 8);
        }
      }
      if (QUANT) {
        uint8_t sfb;
        uint2 out;
        if (p.flags & FRT_PRODUCER_RNE_E2M1) out = quantize_block16<kEncRne>(v, sfb, inv_scale_table());
        else out = quantize_block16<ENC>(v, sfb, inv_scale_table());
        p.packed[idx] = out;
        store_scale(p.sf, row, s, p.nb, p.sf_cols, sfb);
      }
    }
  }
}

template <int TPR, bool HAS_RES, bool QUANT, int ENC>
int launch_norm_stream(const NormParams& p, cudaStream_t st) {
  constexpr int CTA = TPR > 256 ? TPR : 256;
  constexpr int RPC = CTA / TPR;
  constexpr int smem = kStreamStages * (HAS_RES ? 2 : 1) * CTA * 32;
  auto kernel = norm_quant_stream_kernel<TPR, HAS_RES, QUANT, ENC>;
  static int ctas_per_sm[16] = {0};                   // per device, filled on first use
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return FRT_E_DEVICE;
  if (ctas_per_sm[dev] == 0) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return FRT_E_LAUNCH;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, CTA, smem) != cudaSuccess || n < 1)
      return FRT_E_LAUNCH;
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return FRT_E_DEVICE;
    ctas_per_sm[dev] = n * sms;
  }
  const int n_groups = (p.rows + RPC - 1) / RPC;
  const int grid = n_groups < ctas_per_sm[dev] ? n_groups : ctas_per_sm[dev];
  launch_pdl(kernel, dim3(grid), dim3(CTA), smem, st, p, device_status_word(), wait_limit_clocks());
  return launch_result();
}

template <int TPR>
int launch_norm(const NormParams& p, bool has_res, bool quant, cudaStream_t st) {
  const bool chain = g_opt_quant_encoder == 1;
  // Measured on B200: one CTA per row group wins while a row fits 256 threads (64 resident
  // warps per SM hide the latency by themselves); for wider rows the CTA-wide barrier of a
  // 512/1024-thread CTA stalls the SM and the staged persistent form is 15-35 % faster.
  // FRT_OPT_NORM_FORM forces one form or the other (tests run every case on both).
  const bool stream = p.out_fp8 == nullptr && TPR >= 32 &&       // (rows that share a warp: the one-CTA form only)
                      (g_opt_norm_form == 2 || (g_opt_norm_form != 1 && TPR > (quant ? 256 : 512)));
  if (!stream) {
    constexpr int CTA = TPR > 256 ? TPR : 256;
    constexpr int rows_per_cta = CTA / TPR;
    const dim3 grid((p.rows + rows_per_cta - 1) / rows_per_cta), block(CTA);
#define FRT_LAUNCH(HR, Q, E) launch_pdl(norm_quant_kernel<TPR, HR, Q, E>, grid, block, 0, st, p)
    if (!quant) {
      if (has_res) FRT_LAUNCH(true, false, kEncHw); else FRT_LAUNCH(false, false, kEncHw);
    } else if (chain) {
      if (has_res) FRT_LAUNCH(true, true, kEncChain); else FRT_LAUNCH(false, true, kEncChain);
    } else {
      if (has_res) FRT_LAUNCH(true, true, kEncHw); else FRT_LAUNCH(false, true, kEncHw);
    }
#undef FRT_LAUNCH
    return launch_result();
  }
  if (!quant) {
    return has_res ? launch_norm_stream<TPR, true, false, kEncHw>(p, st)
                   : launch_norm_stream<TPR, false, false, kEncHw>(p, st);
  }
  if (chain) {
    return has_res ? launch_norm_stream<TPR, true, true, kEncChain>(p, st)
                   : launch_norm_stream<TPR, false, true, kEncChain>(p, st);
  }
  return has_res ? launch_norm_stream<TPR, true, true, kEncHw>(p, st)
                 : launch_norm_stream<TPR, false, true, kEncHw>(p, st);
}

// Per-head RMSNorm in place over the heads of a stacked projection output (the q and k heads of a fused q/k/v
// GEMM): row (token, head) is head_dim contiguous elements at token * row_pitch + head * head_dim; heads
// [0, heads_a) take weight_a, the next heads_b take weight_b.  Arithmetic and summation order of the plain
// rms_norm path above (a thread per 16-element block, butterfly inside the row's LPR lanes), so each head equals
// frt_rms_norm_bf16 of its contiguous copy bit for bit; one launch instead of two copies and two norms.
template <int LPR>
__global__ void __launch_bounds__(256)
head_norm_kernel(uint4* __restrict__ x, int tokens, int pitch_blocks, int heads_a, int heads_b,
                 const uint4* __restrict__ wa, const uint4* __restrict__ wb, float eps, float dim_f) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int ROWS = 256 / LPR;
  const int heads = heads_a + heads_b;
  const int64_t r = static_cast<int64_t>(blockIdx.x) * ROWS + threadIdx.x / LPR;
  const int s = threadIdx.x % LPR;
  const bool ok = r < static_cast<int64_t>(tokens) * heads;
  const int token = ok ? static_cast<int>(r / heads) : 0, head = ok ? static_cast<int>(r % heads) : 0;
  uint4* px = x + 2 * (static_cast<int64_t>(token) * pitch_blocks + head * LPR + s);
  float v[16];
  uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
  if (ok) { x0 = px[0]; x1 = px[1]; }
  unpack_bf16x8(x0, v);
  unpack_bf16x8(x1, v + 8);
  float part = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) part = __fadd_rn(part, __fmul_rn(v[j], v[j]));
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, o));
  if (!ok) return;
  const float rstd = __frsqrt_rn(__fadd_rn(__fdiv_rn(part, dim_f), eps));
  const uint4* w = head < heads_a ? wa : wb;
  float g[16];
  unpack_bf16x8(__ldg(w + 2 * s), g);
  unpack_bf16x8(__ldg(w + 2 * s + 1), g + 8);
#pragma unroll
  for (int j = 0; j < 16; ++j) v[j] = __fmul_rn(__fmul_rn(v[j], rstd), g[j]);
  uint4 o0, o1;
  pack16_bf16(v, o0, o1);
  px[0] = o0;
  px[1] = o1;
}

int dispatch_norm(NormParams& p, bool has_res, bool quant, cudaStream_t st) {
  const int nb = p.nb;
  if (nb <= 8) return launch_norm<8>(p, has_res, quant, st);       // per-head norms (dim 128): four rows per warp
  if (nb <= 16) return launch_norm<16>(p, has_res, quant, st);
  if (nb <= 32) return launch_norm<32>(p, has_res, quant, st);
  if (nb <= 64) return launch_norm<64>(p, has_res, quant, st);
  if (nb <= 128) return launch_norm<128>(p, has_res, quant, st);
  if (nb <= 256) return launch_norm<256>(p, has_res, quant, st);
  if (nb <= 512) return launch_norm<512>(p, has_res, quant, st);
  return launch_norm<1024>(p, has_res, quant, st);
}

// fp16 activations / residual, no weight: residual_add_rms_norm_fp4_sfa_v2_fp16 of the reference
template <int TPR>
int launch_norm_fp16(const NormParams& p, cudaStream_t st) {
  constexpr int CTA = TPR > 256 ? TPR : 256;
  constexpr int rows_per_cta = CTA / TPR;
  const dim3 grid((p.rows + rows_per_cta - 1) / rows_per_cta), block(CTA);
  if (g_opt_quant_encoder == 1) launch_pdl(norm_quant_kernel<TPR, true, true, kEncChain, true>, grid, block, 0, st, p);
  else launch_pdl(norm_quant_kernel<TPR, true, true, kEncHw, true>, grid, block, 0, st, p);
  return launch_result();
}

int check_norm_args(const void* x, int rows, int dim) {
  if (!x) return FRT_E_NULL;
  if (rows <= 0 || dim <= 0 || dim % 16 != 0) return FRT_E_SHAPE;
  if (dim > 16384) return FRT_E_UNSUPPORTED;
  return FRT_OK;
}

}  // namespace
}  // namespace frt

using namespace frt;

extern "C" {

const char* frt_error_string(int rc) {
  switch (rc) {
    case FRT_OK: return "ok";
    case FRT_E_NULL: return "a required pointer is null";
    case FRT_E_SHAPE: return "invalid shape (non-positive or not divisible as required)";
    case FRT_E_ALIGN: return "pointer alignment violated";
    case FRT_E_UNSUPPORTED: return "shape outside the supported range";
    case FRT_E_LAUNCH: return "CUDA launch failed";
    case FRT_E_DEVICE: return "device is not compute capability 10.x (B200)";
    case FRT_E_DRIVER: return "tensor-map encode failed";
    case FRT_E_TOO_LARGE: return "size beyond the fixed maximum of this entry point";
    default: return "unknown error";
  }
}

int64_t frt_nvfp4_sf_swizzled_bytes(int rows, int dim) {
  if (rows <= 0 || dim <= 0) return 0;
  return static_cast<int64_t>((rows + 127) / 128) * ((dim + 63) / 64) * 512;
}

int64_t frt_nvfp4_sf_offset(int row, int k, int dim) { return sf_offset(row, k >> 4, (dim + 63) >> 6); }

int64_t frt_launch_count(void) { return g_launches.load(); }

int frt_set_option(int key, int value) {
  int prev = -1;
  if (key == FRT_OPT_QUANT_ENCODER) { prev = g_opt_quant_encoder; g_opt_quant_encoder = value; }
  if (key == FRT_OPT_GEMM_CONFIG) { prev = g_opt_gemm_config; g_opt_gemm_config = value; }
  if (key == FRT_OPT_PDL) { prev = g_opt_pdl; g_opt_pdl = value; }
  if (key == FRT_OPT_NORM_FORM) { prev = g_opt_norm_form; g_opt_norm_form = value; }
  if (key == FRT_OPT_GEMM_TAIL_SPLIT) { prev = g_opt_tail_split; g_opt_tail_split = value; }
  if (key == FRT_OPT_GEMM_SPLIT_K) { prev = g_opt_split_k; g_opt_split_k = value; }
  if (key == FRT_OPT_SMALLM_STAGES) { prev = g_opt_smallm_stages; g_opt_smallm_stages = value; }
  if (key == FRT_OPT_GROUPED_FORM) { prev = g_opt_grouped_form; g_opt_grouped_form = value; }
  if (key == FRT_OPT_WAIT_LIMIT_LOG2) {
    prev = g_opt_wait_limit_log2;
    g_opt_wait_limit_log2 = value < 20 ? 20 : value > 40 ? 40 : value;
  }
#ifdef FRT_DEBUG
  if (key == 3) { prev = g_opt_gemm_debug; g_opt_gemm_debug = value; }
#endif
  return prev;
}

int frt_nvfp4_sf_linear_to_swizzled(const void* src, void* dst, int rows, int dim, void* stream) {
  if (!src || !dst) return FRT_E_NULL;
  if (rows <= 0 || dim <= 0 || dim % 16 != 0) return FRT_E_SHAPE;
  if (!aligned(dst, 4)) return FRT_E_ALIGN;
  const int nb = dim / 16, sf_cols = (dim + 63) / 64;
  const bool vec_ok = aligned(src, 4) && (nb & 3) == 0;   // else byte moves
  const dim3 block(128), grid((sf_cols + 127) / 128, rows);
  sf_linear_to_swizzled_kernel<<<grid, block, 0, as_stream(stream)>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), rows, nb, sf_cols, vec_ok);
  return launch_result();
}

int frt_nvfp4_quantize(const void* src, int src_dtype, void* packed, void* sf, int rows, int dim, void* stream) {
  if (!src || !packed || !sf) return FRT_E_NULL;
  if (rows <= 0 || dim <= 0 || dim % 16 != 0) return FRT_E_SHAPE;
  if (src_dtype != FRT_DTYPE_BF16 && src_dtype != FRT_DTYPE_FP16) return FRT_E_UNSUPPORTED;
  if (!aligned(src, 16) || !aligned(packed, 8)) return FRT_E_ALIGN;
  const int nb = dim / 16, sf_cols = (dim + 63) / 64;
  const int64_t total = static_cast<int64_t>(rows) * nb;
  const dim3 block(256), grid(static_cast<unsigned>((total + 255) / 256));
  auto s = static_cast<const uint4*>(src);
  auto pk = static_cast<uint2*>(packed);
  auto sfp = static_cast<uint8_t*>(sf);
  cudaStream_t st = as_stream(stream);
  const bool chain = g_opt_quant_encoder == 1;
  if (src_dtype == FRT_DTYPE_FP16) {
    if (chain) launch_pdl(quantize_kernel<kEncChain, true>, grid, block, 0, st, s, pk, sfp, rows, nb, sf_cols);
    else launch_pdl(quantize_kernel<kEncHw, true>, grid, block, 0, st, s, pk, sfp, rows, nb, sf_cols);
  } else {
    if (chain) launch_pdl(quantize_kernel<kEncChain, false>, grid, block, 0, st, s, pk, sfp, rows, nb, sf_cols);
    else launch_pdl(quantize_kernel<kEncHw, false>, grid, block, 0, st, s, pk, sfp, rows, nb, sf_cols);
  }
  return launch_result();
}

int frt_nvfp4_quantize_mse(const void* src, int src_dtype, void* packed, void* sf, int rows, int dim, void* stream) {
  if (!src || !packed || !sf) return FRT_E_NULL;
  if (rows <= 0 || dim <= 0 || dim % 16 != 0) return FRT_E_SHAPE;
  if (src_dtype != FRT_DTYPE_BF16 && src_dtype != FRT_DTYPE_FP16) return FRT_E_UNSUPPORTED;
  if (!aligned(src, 16) || !aligned(packed, 8)) return FRT_E_ALIGN;
  const int nb = dim / 16, sf_cols = (dim + 63) / 64;
  const int64_t total = static_cast<int64_t>(rows) * nb;
  const dim3 block(256), grid(static_cast<unsigned>((total + 255) / 256));
  auto s = static_cast<const uint4*>(src);
  auto pk = static_cast<uint2*>(packed);
  auto sfp = static_cast<uint8_t*>(sf);
  if (src_dtype == FRT_DTYPE_FP16)
    quantize_mse_kernel<true><<<grid, block, 0, as_stream(stream)>>>(s, pk, sfp, rows, nb, sf_cols);
  else
    quantize_mse_kernel<false><<<grid, block, 0, as_stream(stream)>>>(s, pk, sfp, rows, nb, sf_cols);
  return launch_result();
}

int frt_silu_mul_quant_nvfp4(const void* merged, void* packed, void* sf, int rows, int hidden, void* stream) {
  if (!merged || !packed || !sf) return FRT_E_NULL;
  if (rows <= 0 || hidden <= 0 || hidden % 16 != 0) return FRT_E_SHAPE;
  if (!aligned(merged, 16) || !aligned(packed, 8)) return FRT_E_ALIGN;
  const int nb = hidden / 16, sf_cols = (hidden + 63) / 64;
  const int64_t total = static_cast<int64_t>(rows) * nb;
  const dim3 block(256), grid(static_cast<unsigned>((total + 255) / 256));
  auto m = static_cast<const uint4*>(merged);
  auto pk = static_cast<uint2*>(packed);
  auto sfp = static_cast<uint8_t*>(sf);
  if (g_opt_quant_encoder == 1)
    launch_pdl(silu_mul_quant_kernel<kEncChain>, grid, block, 0, as_stream(stream), m, pk, sfp, rows, nb, sf_cols);
  else
    launch_pdl(silu_mul_quant_kernel<kEncHw>, grid, block, 0, as_stream(stream), m, pk, sfp, rows, nb, sf_cols);
  return launch_result();
}

int frt_nvfp4_dequantize_fp16(const void* packed, const void* sf, void* out, int rows, int dim, void* stream) {
  if (!packed || !sf || !out) return FRT_E_NULL;
  if (rows <= 0 || dim <= 0 || dim % 16 != 0) return FRT_E_SHAPE;
  if (!aligned(out, 16) || !aligned(packed, 8)) return FRT_E_ALIGN;
  const int nb = dim / 16, sf_cols = (dim + 63) / 64;
  const int64_t total = static_cast<int64_t>(rows) * nb;
  dequantize_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(
      static_cast<const uint2*>(packed), static_cast<const uint8_t*>(sf), static_cast<uint4*>(out), rows, nb, sf_cols);
  return launch_result();
}

int frt_norm_quant_nvfp4(void* residual, const void* x, const void* weight, float eps, float inv_global_scale,
                         void* normed, void* packed, void* sf, int rows, int dim, unsigned flags, void* stream) {
  if (int rc = check_norm_args(x, rows, dim)) return rc;
  if (!packed || !sf) return FRT_E_NULL;
  if (!aligned(x, 16) || !aligned(residual, 16) || !aligned(weight, 16) || !aligned(normed, 16) ||
      !aligned(packed, 8))
    return FRT_E_ALIGN;
  NormParams p{};
  p.residual = static_cast<uint4*>(residual);
  p.x = static_cast<const uint4*>(x);
  p.weight = static_cast<const uint4*>(weight);
  p.normed = static_cast<uint4*>(normed);
  p.packed = static_cast<uint2*>(packed);
  p.sf = static_cast<uint8_t*>(sf);
  p.rows = rows; p.nb = dim / 16; p.sf_cols = (dim + 63) / 64;
  p.eps = eps; p.inv_global_scale = inv_global_scale; p.dim_f = static_cast<float>(dim);
  p.flags = flags;
  return dispatch_norm(p, residual != nullptr, true, as_stream(stream));
}

int frt_residual_norm_quant_nvfp4_fp16(void* residual, const void* x, float eps, void* packed, void* sf, int rows,
                                       int dim, void* stream) {
  if (int rc = check_norm_args(x, rows, dim)) return rc;
  if (!residual || !packed || !sf) return FRT_E_NULL;
  if (!aligned(x, 16) || !aligned(residual, 16) || !aligned(packed, 8)) return FRT_E_ALIGN;
  NormParams p{};
  p.residual = static_cast<uint4*>(residual);
  p.x = static_cast<const uint4*>(x);
  p.packed = static_cast<uint2*>(packed);
  p.sf = static_cast<uint8_t*>(sf);
  p.rows = rows; p.nb = dim / 16; p.sf_cols = (dim + 63) / 64;
  p.eps = eps; p.inv_global_scale = 1.0f; p.dim_f = static_cast<float>(dim);
  cudaStream_t st = as_stream(stream);
  const int nb = p.nb;
  if (nb <= 32) return launch_norm_fp16<32>(p, st);
  if (nb <= 64) return launch_norm_fp16<64>(p, st);
  if (nb <= 128) return launch_norm_fp16<128>(p, st);
  if (nb <= 256) return launch_norm_fp16<256>(p, st);
  if (nb <= 512) return launch_norm_fp16<512>(p, st);
  return launch_norm_fp16<1024>(p, st);
}

int frt_rms_norm_bf16(const void* x, const void* weight, void* out, int rows, int dim, float eps, void* stream) {
  if (int rc = check_norm_args(x, rows, dim)) return rc;
  if (!weight || !out) return FRT_E_NULL;
  if (!aligned(x, 16) || !aligned(weight, 16) || !aligned(out, 16)) return FRT_E_ALIGN;
  NormParams p{};
  p.x = static_cast<const uint4*>(x);
  p.weight = static_cast<const uint4*>(weight);
  p.normed = static_cast<uint4*>(out);
  p.rows = rows; p.nb = dim / 16; p.sf_cols = (dim + 63) / 64;
  p.eps = eps; p.inv_global_scale = 1.0f; p.dim_f = static_cast<float>(dim);
  return dispatch_norm(p, false, false, as_stream(stream));
}

int frt_rms_norm_heads_bf16(void* x, int tokens, int row_pitch, int head_dim, int heads_a, const void* weight_a,
                            int heads_b, const void* weight_b, float eps, void* stream) {
  if (!x || !weight_a || (heads_b > 0 && !weight_b)) return FRT_E_NULL;
  if (tokens <= 0 || heads_a <= 0 || heads_b < 0 || row_pitch <= 0 || row_pitch % 8 != 0 ||
      static_cast<int64_t>(heads_a + heads_b) * head_dim > row_pitch)
    return FRT_E_SHAPE;
  if (head_dim != 64 && head_dim != 128 && head_dim != 256 && head_dim != 512) return FRT_E_UNSUPPORTED;
  if (row_pitch % 16 != 0) return FRT_E_SHAPE;
  if (!aligned(x, 16) || !aligned(weight_a, 16) || !aligned(weight_b, 16)) return FRT_E_ALIGN;
  const int lpr = head_dim / 16;
  const int64_t rows = static_cast<int64_t>(tokens) * (heads_a + heads_b);
  const dim3 grid(static_cast<unsigned>((rows + 256 / lpr - 1) / (256 / lpr))), block(256);
  auto xs = static_cast<uint4*>(x);
  auto wa = static_cast<const uint4*>(weight_a);
  auto wb = static_cast<const uint4*>(weight_b ? weight_b : weight_a);
  const cudaStream_t st = as_stream(stream);
  const float dim_f = static_cast<float>(head_dim);
  switch (lpr) {
    case 4: launch_pdl(head_norm_kernel<4>, grid, block, 0, st, xs, tokens, row_pitch / 16, heads_a, heads_b, wa, wb, eps, dim_f); break;
    case 8: launch_pdl(head_norm_kernel<8>, grid, block, 0, st, xs, tokens, row_pitch / 16, heads_a, heads_b, wa, wb, eps, dim_f); break;
    case 16: launch_pdl(head_norm_kernel<16>, grid, block, 0, st, xs, tokens, row_pitch / 16, heads_a, heads_b, wa, wb, eps, dim_f); break;
    default: launch_pdl(head_norm_kernel<32>, grid, block, 0, st, xs, tokens, row_pitch / 16, heads_a, heads_b, wa, wb, eps, dim_f); break;
  }
  return launch_result();
}

int frt_layer_norm_bf16(const void* x, const void* weight, const void* bias, void* out, int rows, int dim, float eps,
                        void* stream) {
  if (int rc = check_norm_args(x, rows, dim)) return rc;
  if (!weight || !bias || !out) return FRT_E_NULL;
  if (!aligned(x, 16) || !aligned(weight, 16) || !aligned(bias, 16) || !aligned(out, 16)) return FRT_E_ALIGN;
  const int nb = dim / 16;
  auto xs = static_cast<const uint4*>(x);
  auto w = static_cast<const uint4*>(weight);
  auto b = static_cast<const uint4*>(bias);
  auto o = static_cast<uint4*>(out);
  const float dim_f = static_cast<float>(dim);
  cudaStream_t st = as_stream(stream);
  if (nb <= 32) return launch_layer_norm<32>(xs, w, b, o, rows, nb, dim_f, eps, st);
  if (nb <= 64) return launch_layer_norm<64>(xs, w, b, o, rows, nb, dim_f, eps, st);
  if (nb <= 128) return launch_layer_norm<128>(xs, w, b, o, rows, nb, dim_f, eps, st);
  if (nb <= 256) return launch_layer_norm<256>(xs, w, b, o, rows, nb, dim_f, eps, st);
  if (nb <= 512) return launch_layer_norm<512>(xs, w, b, o, rows, nb, dim_f, eps, st);
  return launch_layer_norm<1024>(xs, w, b, o, rows, nb, dim_f, eps, st);
}

int frt_rms_norm_quant_fp8(void* residual, const void* x, const void* weight, const void* scale, void* out_fp8,
                           int rows, int dim, float eps, void* stream) {
  if (int rc = check_norm_args(x, rows, dim)) return rc;
  if (!weight || !scale || !out_fp8) return FRT_E_NULL;
  if (!aligned(x, 16) || !aligned(weight, 16) || !aligned(out_fp8, 16) || !aligned(residual, 16) || !aligned(scale, 4))
    return FRT_E_ALIGN;
  NormParams p{};
  p.residual = static_cast<uint4*>(residual);
  p.x = static_cast<const uint4*>(x);
  p.weight = static_cast<const uint4*>(weight);
  p.out_fp8 = static_cast<uint4*>(out_fp8);
  p.fp8_scale = static_cast<const float*>(scale);
  p.rows = rows; p.nb = dim / 16; p.sf_cols = (dim + 63) / 64;
  p.eps = eps; p.inv_global_scale = 1.0f; p.dim_f = static_cast<float>(dim);
  p.flags = residual ? FRT_PRODUCER_NORM_FROM_BF16_RESIDUAL : 0u;
  return dispatch_norm(p, residual != nullptr, false, as_stream(stream));
}

int frt_residual_add_rms_norm_bf16(void* residual, const void* x, const void* weight, void* out,
                                   int rows, int dim, float eps, void* stream) {
  if (int rc = check_norm_args(x, rows, dim)) return rc;
  if (!residual || !weight || !out) return FRT_E_NULL;
  if (!aligned(x, 16) || !aligned(weight, 16) || !aligned(out, 16) || !aligned(residual, 16)) return FRT_E_ALIGN;
  NormParams p{};
  p.residual = static_cast<uint4*>(residual);
  p.x = static_cast<const uint4*>(x);
  p.weight = static_cast<const uint4*>(weight);
  p.normed = static_cast<uint4*>(out);
  p.rows = rows; p.nb = dim / 16; p.sf_cols = (dim + 63) / 64;
  p.eps = eps; p.inv_global_scale = 1.0f; p.dim_f = static_cast<float>(dim);
  p.flags = FRT_PRODUCER_NORM_FROM_BF16_RESIDUAL;
  return dispatch_norm(p, true, false, as_stream(stream));
}

}  // extern "C"
