// Row-sharded activation producer fused with its exchange, for column-parallel GEMMs on the GPUs of one node.
//
// Column-parallel GEMMs need the NVFP4 activations of ALL token rows on every GPU.  Instead of every GPU running
// the whole producer (or each running its rows and a library all-gather afterwards), each GPU runs the fused
// residual-add + RMSNorm -> NVFP4 producer on ITS row shard and stores the packed codes and scale bytes straight
// into every GPU's copy of the activation buffer, in the same kernel:
//   * through one NVSwitch multicast address (`multimem.st`: the switch replicates each store to all GPUs), or
//   * with plain stores to each GPU's mapped address (peer stores over NVLink), when no multicast mapping exists.
// The producer kernel itself sends only the packed codes (8 contiguous bytes per thread, merged to 16-byte
// multicast stores) and writes the scale bytes into this GPU's own copy; a second, small kernel then copies the
// shard's scale bytes - one contiguous range of the swizzled layout, since shards are whole 128-row groups - to
// the other GPUs with 16-byte stores (one row's scale bytes are scattered over 64 tiles, and 4-byte remote stores
// cost an NVLink request each) and publishes this rank's epoch number in every GPU's flag array (release stores at
// system scope; the kernel boundary orders them after all of the producer's stores, so no CTA of the producer
// has to wait for its remote stores).  `peer_wait_kernel`, enqueued before the consumer GEMM, polls the local
// flag array until every rank's flag has reached the epoch; the wait is bounded and reports through the status word.
//
// Arithmetic, summation order and bytes are those of norm_quant_kernel (producer.cu) on the same rows.
// The buffers are owned by the caller (symmetric allocations mapped into every process); nothing here allocates.
#include "common.cuh"

namespace frt {
namespace {

constexpr int kMaxRanks = 8;

struct BcastParams {
  uint4* residual;            // this rank's rows, bf16 [rows, dim], in/out (or null)
  const uint4* x;             // this rank's rows, bf16 [rows, dim]
  const uint4* weight;        // bf16 [dim] or null
  uint8_t* mc_packed;         // multicast address of the whole [M, dim/2] packed buffer, or null
  uint8_t* mc_sf;             // multicast address of the whole swizzled scale buffer, or null
  uint8_t* dst_packed[kMaxRanks];   // per-destination addresses of the same buffers (used when mc_* is null)
  uint8_t* dst_sf[kMaxRanks];
  int n_dst;
  int row0;                   // index of this rank's first row in the whole tensor
  int rows, nb, sf_cols;
  float eps, inv_global_scale, dim_f;
  unsigned flags;
  uint8_t* local_sf;          // this GPU's own copy of the scale buffer (the producer kernel writes scales only here)
  int64_t sf_lo, sf_bytes;    // byte range of this rank's rows in the swizzled scale buffer
  unsigned* counter;          // CTAs of the finishing grid that are done (local scratch word, zero between calls)
  unsigned* peer_flags[kMaxRanks];  // every rank's flag array, as mapped into this process
  int n_ranks, rank;
  unsigned epoch;
};

__device__ __forceinline__ void multimem_st_b64(void* addr, uint2 v) {
  const unsigned long long w = (static_cast<unsigned long long>(v.y) << 32) | v.x;
  asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(addr), "l"(w) : "memory");
}
__device__ __forceinline__ void multimem_st_v4(void* addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(addr), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)), "f"(__uint_as_float(c)),
                 "f"(__uint_as_float(d)) : "memory");
}
__device__ __forceinline__ void st_release_sys(unsigned* addr, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* addr) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// One thread per 16-element block, TPR threads per row, as norm_quant_kernel.
template <int TPR, bool HAS_RES>
__global__ void __launch_bounds__(TPR > 256 ? TPR : 256)
norm_quant_bcast_kernel(const BcastParams p) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CTA = TPR > 256 ? TPR : 256;
  constexpr int ROWS_PER_CTA = CTA / TPR;
  constexpr int WPR = TPR / 32;
  __shared__ float warp_sums[CTA / 32];
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int row = blockIdx.x * ROWS_PER_CTA + threadIdx.x / TPR;
  const int s = threadIdx.x % TPR;
  const bool ok = row < p.rows && s < p.nb;
  const int64_t idx = static_cast<int64_t>(row) * p.nb + s;

  float v[16];
  uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0, r0 = x0, r1 = x0;
  if (ok) {
    x0 = __ldcs(p.x + 2 * idx);
    x1 = __ldcs(p.x + 2 * idx + 1);
    if (HAS_RES) {
      r0 = __ldcs(p.residual + 2 * idx);
      r1 = __ldcs(p.residual + 2 * idx + 1);
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
    o0.x = pack_bf16x2(v[0], v[1]);   o0.y = pack_bf16x2(v[2], v[3]);
    o0.z = pack_bf16x2(v[4], v[5]);   o0.w = pack_bf16x2(v[6], v[7]);
    o1.x = pack_bf16x2(v[8], v[9]);   o1.y = pack_bf16x2(v[10], v[11]);
    o1.z = pack_bf16x2(v[12], v[13]); o1.w = pack_bf16x2(v[14], v[15]);
    if (ok) {
      __stcs(p.residual + 2 * idx, o0);
      __stcs(p.residual + 2 * idx + 1, o1);
    }
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
  if (WPR > 1) {
    if (lane == 0) warp_sums[warp] = part;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    ssq = warp_sums[first];
#pragma unroll
    for (int w = 1; w < WPR; ++w) ssq = __fadd_rn(ssq, warp_sums[first + w]);
  }
  uint2 packed = make_uint2(0, 0);
  uint32_t sf_byte = 0;
  if (ok) {
    const float rstd = __frsqrt_rn(__fadd_rn(__fdiv_rn(ssq, p.dim_f), p.eps));
    if (p.weight != nullptr) {
      float g[16];
      unpack_bf16x8(__ldg(p.weight + 2 * s), g);
      unpack_bf16x8(__ldg(p.weight + 2 * s + 1), g + 8);
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
    if (p.flags & FRT_PRODUCER_ROUND_BF16) {
#pragma unroll
      for (int j = 0; j < 16; j += 2) {
        const uint32_t w = pack_bf16x2(v[j], v[j + 1]);
        v[j] = __uint_as_float(w << 16);
        v[j + 1] = __uint_as_float(w & 0xffff0000u);
      }
    }
    uint8_t sfb;
    if (p.flags & FRT_PRODUCER_RNE_E2M1) packed = quantize_block16<kEncRne>(v, sfb, inv_scale_table());
    else packed = quantize_block16<kEncHw>(v, sfb, inv_scale_table());
    sf_byte = sfb;
  }
  // multicast stores travel as separate requests: even lanes send their own 8 packed bytes and their odd
  // neighbour's as one 16-byte store (rows of an odd number of blocks keep 8-byte stores)
  const uint32_t nx = __shfl_down_sync(0xffffffffu, packed.x, 1), ny = __shfl_down_sync(0xffffffffu, packed.y, 1);
  if (ok) {
    const int grow = p.row0 + row;
    const int64_t packed_off = (static_cast<int64_t>(grow) * p.nb + s) * 8;
    // scale byte into this GPU's copy (the padding of a row's last 64-element group is zeroed by the owner of
    // the row's last block); the finishing kernel forwards the whole range
    p.local_sf[sf_offset(grow, s, p.sf_cols)] = static_cast<uint8_t>(sf_byte);
    if (s == p.nb - 1)
      for (int j = p.nb; j < 4 * p.sf_cols; ++j) p.local_sf[sf_offset(grow, j, p.sf_cols)] = 0;
    if (p.mc_packed != nullptr) {
      if (p.nb & 1) {                        // rows of an odd number of blocks start 8-byte aligned only
        multimem_st_b64(p.mc_packed + packed_off, packed);
      } else if ((s & 1) == 0) {
        multimem_st_v4(p.mc_packed + packed_off, packed.x, packed.y, nx, ny);
      }
    } else {
      for (int d = 0; d < p.n_dst; ++d) *reinterpret_cast<uint2*>(p.dst_packed[d] + packed_off) = packed;
    }
  }
}

// Forwards this rank's scale bytes (a contiguous range) to the other GPUs and publishes the epoch.  Runs after the
// producer grid has completed (programmatic dependency + griddepcontrol.wait), so its flag stores are ordered after
// every store of that grid.
__global__ void __launch_bounds__(256)
exchange_finish_kernel(const BcastParams p, unsigned* status, long long wait_limit) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t n16 = p.sf_bytes >> 4;
  const uint4* src = reinterpret_cast<const uint4*>(p.local_sf + p.sf_lo);
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint4 v = src[i];
    if (p.mc_sf != nullptr) {
      multimem_st_v4(p.mc_sf + p.sf_lo + i * 16, v.x, v.y, v.z, v.w);
    } else {
      for (int d = 0; d < p.n_dst; ++d)
        if (d != p.rank) *reinterpret_cast<uint4*>(p.dst_sf[d] + p.sf_lo + i * 16) = v;
    }
  }
  __shared__ int is_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned done = atomicAdd(p.counter, 1u) + 1u;
    is_last = done == gridDim.x;
    if (is_last) {
      *p.counter = 0;                                   // ready for the next call on this stream
      __threadfence_system();
      for (int r = 0; r < p.n_ranks; ++r) st_release_sys(p.peer_flags[r] + p.rank, p.epoch);
    }
  }
  __syncthreads();
  // FRT_PRODUCER_WAIT_PEERS: the CTA that published also waits (bounded) until every rank's rows of this epoch
  // have landed here, so the next kernel of the stream may consume the buffer without a separate wait kernel.
  if ((p.flags & FRT_PRODUCER_WAIT_PEERS) && is_last && threadIdx.x < p.n_ranks) {
    const unsigned* mine = p.peer_flags[p.rank] + threadIdx.x;
    const long long t0 = clock64();
    while (static_cast<int>(ld_acquire_sys(mine) - p.epoch) < 0) {
      if (clock64() - t0 > wait_limit) {
        atomicOr(status, 0x400u);
        break;
      }
      __nanosleep(64);
    }
  }
}

// Polls this GPU's flag array until every rank has published `epoch` (flags only grow).  One warp; bounded.
__global__ void peer_wait_kernel(const unsigned* flags, int n_ranks, unsigned epoch, unsigned* status,
                                 long long wait_limit) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = threadIdx.x;
  if (r >= n_ranks) return;
  const long long t0 = clock64();
  while (static_cast<int>(ld_acquire_sys(flags + r) - epoch) < 0) {
    if (clock64() - t0 > wait_limit) {
      atomicOr(status, 0x400u);
      return;
    }
    __nanosleep(64);
  }
}

template <int TPR>
int launch_bcast(const BcastParams& p, bool has_res, cudaStream_t st) {
  constexpr int CTA = TPR > 256 ? TPR : 256;
  constexpr int rows_per_cta = CTA / TPR;
  const dim3 grid((p.rows + rows_per_cta - 1) / rows_per_cta), block(CTA);
  if (has_res) launch_pdl(norm_quant_bcast_kernel<TPR, true>, grid, block, 0, st, p);
  else launch_pdl(norm_quant_bcast_kernel<TPR, false>, grid, block, 0, st, p);
  if (int rc = launch_result()) return rc;
  const int64_t n16 = p.sf_bytes >> 4;
  const int blocks = static_cast<int>(n16 / 256 < 1 ? 1 : n16 / 256 > 64 ? 64 : n16 / 256);
  launch_pdl(exchange_finish_kernel, dim3(blocks), dim3(256), 0, st, p, device_status_word(), wait_limit_clocks());
  return launch_result();
}

}  // namespace
}  // namespace frt

using namespace frt;

extern "C" {

int frt_norm_quant_nvfp4_bcast(void* residual, const void* x, const void* weight, float eps, float inv_global_scale,
                               void* mc_packed, void* mc_sf, void* const* dst_packed, void* const* dst_sf, int n_dst,
                               int row0, int rows, int dim, unsigned flags, void* counter, void* const* peer_flags,
                               int n_ranks, int rank, unsigned epoch, void* stream) {
  if (!x || !counter || !peer_flags) return FRT_E_NULL;
  if ((mc_packed == nullptr) != (mc_sf == nullptr)) return FRT_E_NULL;
  if (rows <= 0 || dim <= 0 || dim % 16 != 0 || row0 < 0) return FRT_E_SHAPE;
  if (row0 % 128 != 0 || rows % 128 != 0) return FRT_E_SHAPE;       // a shard is whole 128-row scale groups
  if (dim > 16384 || n_ranks < 1 || n_ranks > kMaxRanks || rank < 0 || rank >= n_ranks || n_dst > kMaxRanks)
    return FRT_E_UNSUPPORTED;
  if (!dst_sf || n_dst <= rank || !dst_sf[rank]) return FRT_E_NULL;   // this GPU's own copy of the scale buffer
  if (mc_packed == nullptr && (!dst_packed || n_dst != n_ranks)) return FRT_E_NULL;
  if (!aligned(x, 16) || !aligned(residual, 16) || !aligned(weight, 16) || !aligned(mc_packed, 16) ||
      !aligned(counter, 4))
    return FRT_E_ALIGN;
  BcastParams p{};
  p.residual = static_cast<uint4*>(residual);
  p.x = static_cast<const uint4*>(x);
  p.weight = static_cast<const uint4*>(weight);
  p.mc_packed = static_cast<uint8_t*>(mc_packed);
  p.mc_sf = static_cast<uint8_t*>(mc_sf);
  if (mc_packed == nullptr) {
    for (int d = 0; d < n_dst; ++d) {
      if (!dst_packed[d] || !dst_sf[d]) return FRT_E_NULL;
      if (!aligned(dst_packed[d], 8) || !aligned(dst_sf[d], 16)) return FRT_E_ALIGN;
      p.dst_packed[d] = static_cast<uint8_t*>(dst_packed[d]);
      p.dst_sf[d] = static_cast<uint8_t*>(dst_sf[d]);
    }
    p.n_dst = n_dst;
  }
  if (!aligned(dst_sf[rank], 16) || !aligned(mc_sf, 16)) return FRT_E_ALIGN;
  p.local_sf = static_cast<uint8_t*>(dst_sf[rank]);
  for (int r = 0; r < n_ranks; ++r) {
    if (!peer_flags[r]) return FRT_E_NULL;
    p.peer_flags[r] = static_cast<unsigned*>(peer_flags[r]);
  }
  p.row0 = row0;
  p.rows = rows; p.nb = dim / 16; p.sf_cols = (dim + 63) / 64;
  p.sf_lo = static_cast<int64_t>(row0 / 128) * p.sf_cols * 512;
  p.sf_bytes = static_cast<int64_t>(rows / 128) * p.sf_cols * 512;
  p.eps = eps; p.inv_global_scale = inv_global_scale; p.dim_f = static_cast<float>(dim);
  p.flags = flags;
  p.counter = static_cast<unsigned*>(counter);
  p.n_ranks = n_ranks; p.rank = rank; p.epoch = epoch;
  cudaStream_t st = as_stream(stream);
  const bool has_res = residual != nullptr;
  const int nb = p.nb;
  if (nb <= 32) return launch_bcast<32>(p, has_res, st);
  if (nb <= 64) return launch_bcast<64>(p, has_res, st);
  if (nb <= 128) return launch_bcast<128>(p, has_res, st);
  if (nb <= 256) return launch_bcast<256>(p, has_res, st);
  if (nb <= 512) return launch_bcast<512>(p, has_res, st);
  return launch_bcast<1024>(p, has_res, st);
}

int frt_peer_wait(const void* flags, int n_ranks, unsigned epoch, void* stream) {
  if (!flags) return FRT_E_NULL;
  if (n_ranks < 1 || n_ranks > kMaxRanks) return FRT_E_UNSUPPORTED;
  unsigned* status = device_status_word();
  if (!status) return FRT_E_LAUNCH;
  launch_pdl(peer_wait_kernel, dim3(1), dim3(32), 0, as_stream(stream), static_cast<const unsigned*>(flags), n_ranks,
             epoch, status, wait_limit_clocks());
  return launch_result();
}

}  // extern "C"
