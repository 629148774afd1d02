// Routing glue around the grouped (MoE) NVFP4 GEMM: exact top-k router, stable expert sort
// (routing plan), gather of quantised activation rows into expert order, and the weighted
// un-permute.  Small latency- or HBM-bound kernels; every result is deterministic (no
// floating-point atomics, fixed summation order).
#include "common.cuh"

#include <cfloat>

namespace frt {
namespace {

// ---------------------------------------------------------------------------
// Router top-k: one warp per token.  k rounds of a warp-wide arg-max over the token's
// logits (staged as fp32 in shared memory), masking the winner each round.  Logits are
// returned in descending order.  Equal logits are ordered the way the reference's kernel
// orders them (256 threads own the indices congruent to their id, then fold pairwise with
// strides 128 ... 1 keeping the lower slot on a tie): by the bit-reversed low 8 bits of
// the index, then by the index.
// ---------------------------------------------------------------------------
constexpr int kRouterWarps = 8;

__device__ __forceinline__ int tie_key(int i) {
  return static_cast<int>((__brev(static_cast<unsigned>(i) & 255u) >> 24) << 8) | (i >> 8);
}

__global__ void __launch_bounds__(kRouterWarps * 32)
router_topk_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ out_idx,
                   float* __restrict__ out_val, float* __restrict__ out_weight, int tokens, int n, int k) {
  extern __shared__ float s_logits[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x * kRouterWarps + warp;
  if (token >= tokens) return;
  float* mine = s_logits + warp * n;
  const __nv_bfloat16* src = logits + static_cast<int64_t>(token) * n;
  for (int i = lane; i < n; i += 32) mine[i] = __bfloat162float(src[i]);
  __syncwarp();
  for (int r = 0; r < k; ++r) {
    float best = -FLT_MAX;
    int bidx = -1;
    for (int i = lane; i < n; i += 32) {
      const float v = mine[i];
      if (v > best || (v == best && bidx >= 0 && tie_key(i) < tie_key(bidx))) { best = v; bidx = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bidx, o);
      const bool take = oi >= 0 && (bidx < 0 || ov > best || (ov == best && tie_key(oi) < tie_key(bidx)));
      if (take) { best = ov; bidx = oi; }
    }
    if (lane == 0) {
      out_idx[static_cast<int64_t>(token) * k + r] = bidx;
      out_val[static_cast<int64_t>(token) * k + r] = best;
      if (bidx >= 0) mine[bidx] = -FLT_MAX;
    }
    __syncwarp();
  }
  // optional: softmax over the k selected logits (equal to re-normalising the top-k of the full softmax);
  // lane j owns slot j, the maximum is slot 0
  if (out_weight != nullptr) {
    const float v0 = out_val[static_cast<int64_t>(token) * k];
    const float e = lane < k ? expf(out_val[static_cast<int64_t>(token) * k + lane] - v0) : 0.f;
    float sum = e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane < k) out_weight[static_cast<int64_t>(token) * k + lane] = __fdiv_rn(e, sum);
  }
}

// ---------------------------------------------------------------------------
// Routing plan: stable counting sort of the (token, slot) pairs by expert.
//   count: CTA e counts the pairs routed to expert e          -> offsets[e + 1]
//   scan : one CTA turns the counts into exclusive offsets     -> offsets[0 .. E]
//   place: CTA e walks the pairs in order and numbers its own  -> row_of_pair, token_of_row
// ---------------------------------------------------------------------------
constexpr int kPlanThreads = 256;

__global__ void __launch_bounds__(kPlanThreads)
plan_count_kernel(const int* __restrict__ idx, int n_pairs, int* __restrict__ offsets) {
  __shared__ int warp_counts[kPlanThreads / 32];
  const int e = blockIdx.x;
  int c = 0;
#pragma unroll 4
  for (int i = threadIdx.x; i < n_pairs; i += kPlanThreads) c += idx[i] == e;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xffffffffu, c, o);
  if ((threadIdx.x & 31) == 0) warp_counts[threadIdx.x >> 5] = c;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < kPlanThreads / 32; ++w) t += warp_counts[w];
    offsets[e + 1] = t;
    if (e == 0) offsets[0] = 0;
  }
}

__global__ void __launch_bounds__(1024) plan_scan_kernel(int* __restrict__ offsets, int n_experts) {
  // inclusive scan of offsets[1 .. E] in place; each thread owns a contiguous run
  __shared__ int partial[1024];
  const int per = (n_experts + 1023) / 1024;
  const int lo = 1 + threadIdx.x * per, hi = min(lo + per, n_experts + 1);
  int s = 0;
  for (int i = lo; i < hi; ++i) s += offsets[i];
  partial[threadIdx.x] = s;
  __syncthreads();
  for (int d = 1; d < 1024; d <<= 1) {
    const int v = threadIdx.x >= d ? partial[threadIdx.x - d] : 0;
    __syncthreads();
    partial[threadIdx.x] += v;
    __syncthreads();
  }
  int run = threadIdx.x ? partial[threadIdx.x - 1] : 0;
  for (int i = lo; i < hi; ++i) { run += offsets[i]; offsets[i] = run; }
}

// 1024 threads, four consecutive pairs per thread and pass: a pass numbers 4096 pairs with one
// warp scan, one scan over the 32 warp totals and two barriers.
constexpr int kPlaceThreads = 1024;

__global__ void __launch_bounds__(kPlaceThreads)
plan_place_kernel(const int* __restrict__ idx, int n_pairs, int k, int n_experts, const int* __restrict__ offsets,
                  int* __restrict__ row_of_pair, int* __restrict__ token_of_row) {
  __shared__ int warp_totals[kPlaceThreads / 32];
  const int e = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool vec = (n_pairs & 3) == 0 && (reinterpret_cast<uintptr_t>(idx) & 15) == 0;
  int running = offsets[e];
  for (int base = 0; base < n_pairs; base += 4 * kPlaceThreads) {
    const int i0 = base + 4 * threadIdx.x;
    int v[4] = {-2, -2, -2, -2};
    if (vec && i0 < n_pairs) {
      const int4 q = *reinterpret_cast<const int4*>(idx + i0);
      v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) if (i0 + j < n_pairs) v[j] = idx[i0 + j];
    }
    int mine = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) mine += v[j] == e;
    int incl = mine;                                   // inclusive scan over the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_totals[warp] = incl;
    __syncthreads();
    const int wt = warp_totals[lane];                  // every warp scans the 32 warp totals
    int wincl = wt;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, wincl, o);
      if (lane >= o) wincl += up;
    }
    const int before_warp = __shfl_sync(0xffffffffu, wincl - wt, warp);
    const int total = __shfl_sync(0xffffffffu, wincl, 31);
    int row = running + before_warp + incl - mine;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (v[j] == e) {
        row_of_pair[i0 + j] = row;
        token_of_row[row] = (i0 + j) / k;
        ++row;
      } else if (e == 0 && i0 + j < n_pairs && (v[j] < 0 || v[j] >= n_experts)) {
        row_of_pair[i0 + j] = -1;                      // not routed anywhere
      }
    }
    running += total;
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Gather NVFP4 rows into expert order: output row r = input row token_of_row[r], packed
// bytes and the row's scale bytes (4 consecutive k-blocks are 4 contiguous bytes in the
// swizzled layout).  One warp per output row.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
gather_nvfp4_kernel(const uint4* __restrict__ packed_in, const uint8_t* __restrict__ sf_in,
                    const int* __restrict__ token_of_row, uint4* __restrict__ packed_out,
                    uint8_t* __restrict__ sf_out, int rows, int tokens, int row_vec /* K/32 */, int sf_cols) {
  const int r = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const int t = token_of_row[r];
  if (t < 0 || t >= tokens) return;
  const uint4* src = packed_in + static_cast<int64_t>(t) * row_vec;
  uint4* dst = packed_out + static_cast<int64_t>(r) * row_vec;
  for (int i = lane; i < row_vec; i += 32) dst[i] = __ldg(src + i);
  for (int g = lane; g < sf_cols; g += 32)
    *reinterpret_cast<uint32_t*>(sf_out + sf_offset(r, 4 * g, sf_cols)) =
        *reinterpret_cast<const uint32_t*>(sf_in + sf_offset(t, 4 * g, sf_cols));
}

// ---------------------------------------------------------------------------
// Quantise bf16 token rows to NVFP4 straight into expert order: every 16-element block is quantised once
// and its 8 packed bytes + scale byte are stored to each of the token's k expert-sorted rows (pairs with a
// negative row are skipped).  Replaces quantise + gather (and their intermediate) in the routed layer.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quantize_scatter_kernel(const uint4* __restrict__ x, const int* __restrict__ row_of_pair, uint2* __restrict__ packed,
                        uint8_t* __restrict__ sf, int tokens, int k, int nb, int sf_cols) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(tokens) * nb) return;
  const int t = static_cast<int>(idx / nb);
  const int kb = static_cast<int>(idx - static_cast<int64_t>(t) * nb);
  float v[16];
  unpack_bf16x8(__ldcs(x + 2 * idx), v);
  unpack_bf16x8(__ldcs(x + 2 * idx + 1), v + 8);
  uint8_t sfb;
  const uint2 out = quantize_block16<kEncHw>(v, sfb, inv_scale_table());
  for (int j = 0; j < k; ++j) {
    const int r = __ldg(row_of_pair + static_cast<int64_t>(t) * k + j);
    if (r < 0) continue;
    packed[static_cast<int64_t>(r) * nb + kb] = out;
    sf[sf_offset(r, kb, sf_cols)] = sfb;
    if (kb == nb - 1)
      for (int q = nb; q < 4 * sf_cols; ++q) sf[sf_offset(r, q, sf_cols)] = 0;
  }
}

// ---------------------------------------------------------------------------
// Weighted un-permute: out[t, :] = sum_j w[t, j] * y[row[t, j], :] in fp32, slots in order
// (one fused multiply-add per slot), pairs with a negative row skipped.  One CTA per token.
// ---------------------------------------------------------------------------
template <bool VEC>
__global__ void __launch_bounds__(256)
weighted_sum_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ rows, const float* __restrict__ w,
                    float* __restrict__ out, int k, int hid, int stride) {
  extern __shared__ unsigned char ws_smem[];
  int* s_rows = reinterpret_cast<int*>(ws_smem);
  float* s_w = reinterpret_cast<float*>(s_rows + k);
  const int t = blockIdx.x;
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    s_rows[j] = rows[static_cast<int64_t>(t) * k + j];
    s_w[j] = w[static_cast<int64_t>(t) * k + j];
  }
  __syncthreads();
  float* o = out + static_cast<int64_t>(t) * hid;
  if (VEC) {
    for (int c = threadIdx.x * 8; c < hid; c += blockDim.x * 8) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int j = 0; j < k; ++j) {
        const int r = s_rows[j];
        if (r < 0) continue;
        float v[8];
        unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(y + static_cast<int64_t>(r) * stride + c)), v);
        const float wj = s_w[j];
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = __fmaf_rn(v[q], wj, acc[q]);
      }
      *reinterpret_cast<float4*>(o + c) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(o + c + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  } else {
    for (int c = threadIdx.x; c < hid; c += blockDim.x) {
      float acc = 0.f;
      for (int j = 0; j < k; ++j) {
        const int r = s_rows[j];
        if (r < 0) continue;
        acc = __fmaf_rn(__bfloat162float(y[static_cast<int64_t>(r) * stride + c]), s_w[j], acc);
      }
      o[c] = acc;
    }
  }
}

}  // namespace
}  // namespace frt

using namespace frt;

extern "C" {

int frt_router_topk_softmax_bf16(const void* logits, void* out_idx, void* out_val, void* out_weight, int tokens,
                                 int n_experts, int k, void* stream) {
  if (!logits || !out_idx || !out_val) return FRT_E_NULL;
  if (tokens <= 0 || n_experts <= 0 || k <= 0) return FRT_E_SHAPE;
  if (k > 32 || n_experts > 1024) return FRT_E_UNSUPPORTED;
  const int grid = (tokens + kRouterWarps - 1) / kRouterWarps;
  const size_t smem = static_cast<size_t>(kRouterWarps) * n_experts * sizeof(float);
  router_topk_kernel<<<grid, kRouterWarps * 32, smem, as_stream(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), static_cast<int*>(out_idx), static_cast<float*>(out_val),
      static_cast<float*>(out_weight), tokens, n_experts, k);
  return launch_result();
}

int frt_router_topk_bf16(const void* logits, void* out_idx, void* out_val, int tokens, int n_experts, int k,
                         void* stream) {
  return frt_router_topk_softmax_bf16(logits, out_idx, out_val, nullptr, tokens, n_experts, k, stream);
}

int frt_moe_quantize_scatter_nvfp4(const void* x, const void* row_of_pair, void* packed_out, void* sf_out, int tokens,
                                   int k, int K, void* stream) {
  if (!x || !row_of_pair || !packed_out || !sf_out) return FRT_E_NULL;
  if (tokens <= 0 || k <= 0 || K <= 0 || K % 16 != 0) return FRT_E_SHAPE;
  if (!aligned(x, 16) || !aligned(packed_out, 8)) return FRT_E_ALIGN;
  const int nb = K / 16;
  const int64_t total = static_cast<int64_t>(tokens) * nb;
  quantize_scatter_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, as_stream(stream)>>>(
      static_cast<const uint4*>(x), static_cast<const int*>(row_of_pair), static_cast<uint2*>(packed_out),
      static_cast<uint8_t*>(sf_out), tokens, k, nb, (K + 63) / 64);
  return launch_result();
}

int frt_moe_route_plan(const void* topk_idx, int tokens, int k, int n_experts, void* expert_offsets,
                       void* row_of_pair, void* token_of_row, void* stream) {
  if (!topk_idx || !expert_offsets || !row_of_pair || !token_of_row) return FRT_E_NULL;
  if (tokens <= 0 || k <= 0 || n_experts <= 0) return FRT_E_SHAPE;
  if (static_cast<int64_t>(tokens) * k > (1ll << 30)) return FRT_E_TOO_LARGE;
  const int n_pairs = tokens * k;
  cudaStream_t st = as_stream(stream);
  auto idx = static_cast<const int*>(topk_idx);
  auto off = static_cast<int*>(expert_offsets);
  plan_count_kernel<<<n_experts, kPlanThreads, 0, st>>>(idx, n_pairs, off);
  if (int rc = launch_result()) return rc;
  plan_scan_kernel<<<1, 1024, 0, st>>>(off, n_experts);
  if (int rc = launch_result()) return rc;
  plan_place_kernel<<<n_experts, kPlaceThreads, 0, st>>>(idx, n_pairs, k, n_experts, off,
                                                         static_cast<int*>(row_of_pair),
                                                         static_cast<int*>(token_of_row));
  return launch_result();
}

int frt_moe_gather_nvfp4(const void* packed_in, const void* sf_in, const void* token_of_row, void* packed_out,
                         void* sf_out, int rows, int tokens, int K, void* stream) {
  if (!packed_in || !sf_in || !token_of_row || !packed_out || !sf_out) return FRT_E_NULL;
  if (rows <= 0 || tokens <= 0 || K <= 0 || K % 64 != 0) return FRT_E_SHAPE;
  if (!aligned(packed_in, 16) || !aligned(packed_out, 16) || !aligned(sf_in, 4) || !aligned(sf_out, 4))
    return FRT_E_ALIGN;
  gather_nvfp4_kernel<<<(rows + 7) / 8, 256, 0, as_stream(stream)>>>(
      static_cast<const uint4*>(packed_in), static_cast<const uint8_t*>(sf_in), static_cast<const int*>(token_of_row),
      static_cast<uint4*>(packed_out), static_cast<uint8_t*>(sf_out), rows, tokens, K / 32, K / 64);
  return launch_result();
}

int frt_moe_weighted_sum_bf16(const void* expert_out, const void* row_of_pair, const void* weights, void* out,
                              int tokens, int k, int hidden, int stride, void* stream) {
  if (!expert_out || !row_of_pair || !weights || !out) return FRT_E_NULL;
  if (tokens <= 0 || k <= 0 || hidden <= 0 || stride < hidden) return FRT_E_SHAPE;
  if (k > 1024) return FRT_E_UNSUPPORTED;
  const size_t smem = static_cast<size_t>(k) * (sizeof(int) + sizeof(float));
  const bool vec = hidden % 8 == 0 && stride % 8 == 0 && aligned(expert_out, 16) && aligned(out, 16);
  auto y = static_cast<const __nv_bfloat16*>(expert_out);
  auto r = static_cast<const int*>(row_of_pair);
  auto w = static_cast<const float*>(weights);
  auto o = static_cast<float*>(out);
  if (vec) weighted_sum_kernel<true><<<tokens, 256, smem, as_stream(stream)>>>(y, r, w, o, k, hidden, stride);
  else weighted_sum_kernel<false><<<tokens, 256, smem, as_stream(stream)>>>(y, r, w, o, k, hidden, stride);
  return launch_result();
}

}  // extern "C"
