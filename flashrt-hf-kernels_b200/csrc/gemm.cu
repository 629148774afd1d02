// NVFP4 A4W4 block-scaled GEMM with bf16 output for sm_100a.
//
//   D[p, q] = alpha * sum_k P[p,k] * SFP[p,k/16] * Q[q,k] * SFQ[q,k/16]  (+ bias) (+ beta*C)
//
// P is the operand on the 128-lane (UMMA M) axis, Q the operand on the UMMA N
// axis.  For prefill shapes P = activations and Q = weights; for small token
// counts the host swaps them (P = weights, so every CTA streams 128 distinct
// weight rows and the tokens sit on a narrow N axis) and the epilogue writes
// the transposed tile.
//
// One persistent CTA per SM, 6 warps:
//   warp 0      TMA producer: 128B-swizzled operand tiles (cp.async.bulk.tensor)
//               and the swizzled scale-factor chunks (cp.async.bulk) into a
//               STAGES-deep shared-memory ring, mbarrier complete_tx.
//   warp 1      MMA issuer: tcgen05.cp of the scale chunks shared -> TMEM, then
//               tcgen05.mma kind::mxf4nvf4 (K = 64 per instruction, 4 per stage)
//               into one of ACC accumulator stages in TMEM; tcgen05.commit frees
//               the smem stage / publishes the accumulator.
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one 32-lane TMEM quarter
//               per warp), alpha / bias / residual in fp32, bf16 pack, 16-byte
//               global stores; overlaps the next tile's mainloop when ACC == 2.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets a bit in the
// device status word and the CTA drains and returns.
#include <cuda.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "common.cuh"
#include "ptx.cuh"

namespace frt {

namespace {

__device__ unsigned g_status_word = 0;

// Experiment hooks (skip the output stores, skip the scale copies, a clock64 timeline of one CTA
// pair) exist only in a build with -DFRT_DEBUG; the shipped library has none of them.
#ifdef FRT_DEBUG
long long* g_trace = nullptr;   // set by frt_debug_set_trace
#define FRT_DBG(p, bit) (((p).dbg & (bit)) != 0)
#define FRT_TRACING(p) ((p).trace != nullptr)
#define FRT_TRACE(p, slot) ((p).trace[slot] = clock64())
// wall-clock (globaltimer, ns) phase stamps of the small-M kernel: one 16-word record per CTA, slots handed out
// by an atomic counter in word 0 of the trace buffer
__device__ __forceinline__ long long frt_globaltimer() { long long v; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(v)); return v; }
#define FRT_GT_DECL __shared__ long long gt_ts[12]
#define FRT_GT_ZERO do { for (int i_ = 0; i_ < 12; ++i_) gt_ts[i_] = 0; } while (0)
#define FRT_GT(p, slot) do { if ((p).trace) gt_ts[slot] = frt_globaltimer(); } while (0)
#else
#define FRT_DBG(p, bit) false
#define FRT_TRACING(p) false
#define FRT_TRACE(p, slot) ((void)0)
#define FRT_GT_DECL
#define FRT_GT_ZERO ((void)0)
#define FRT_GT(p, slot) ((void)0)
#endif

constexpr int BM = 128;            // UMMA M, rows of P per tile
constexpr int BK = 256;            // elements of K per smem stage (128 bytes per row)
constexpr int KT_PER_STAGE = 4;    // UMMA K = 64 elements
constexpr int SF_TILE = 512;       // bytes of scales for 128 rows x 64 elements
#define WAIT_LIMIT p.wait_limit   // SM clocks before a wait gives up (GemmParams::wait_limit, about a second by default)

struct GemmParams {
  int P, Q, K;              // extents on the M axis, N axis, reduction
  int p_tiles, q_tiles;     // tile counts
  int k_tiles;              // ceil(K / 64)
  int sf_cols;              // ceil(K / 64): 512-byte scale tiles per 128-row group
  const uint8_t* sfp;       // swizzled scales of P
  const uint8_t* sfq;       // swizzled scales of Q
  int sfq_row_blocks;       // 128-row groups present in sfq
  __nv_bfloat16* d;
  const __nv_bfloat16* c;       // or null
  const __nv_bfloat16* bias;    // or null
  int ldd;                  // row stride of d and c, in elements
  float alpha, beta;
  int group_m;              // raster: tiles walk GROUP_M p-tiles before the next q-tile
  const float* alpha_stack; // grouped: per-expert alpha
  int max_items;            // grouped: capacity of the work list (items beyond it were dropped by the plan)
  const int* inline_offsets;  // grouped, weight-major: expert offsets [num_experts + 1] when every CTA plans for itself
  int num_experts;
  int splits;               // split-K cluster size (small-M form), 1 otherwise
  long long wait_limit;     // SM clocks a wait on an mbarrier may take before the CTA gives up
  int p_interleaved;        // P is stored in the interleaved GEMV layout [rows/8][K/64][8][32 B] (4-D tensor map)
#ifdef FRT_DEBUG
  int dbg;                  // experiment switches
  long long* trace;         // clock64 timeline of pair 0, 8 slots per tile
#endif
  // SwiGLU -> NVFP4 epilogue: Q holds [gate ; up] (2 * hidden rows); outputs are hidden wide
  // dense 256-wide pair form: work units = tiles, those of the last partial wave cut in column slices
  int units, tail_first, tail_split;
  int hidden;
  uint8_t* out_packed;      // [P, hidden / 2]
  uint8_t* out_sf;          // swizzled scales of a [P, hidden] tensor
};

template <int BN, int STAGES>
struct SmemLayout {
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SFQ_BLOCKS = BN <= 128 ? 1 : 2;   // 128-row scale groups a Q tile can touch
  static constexpr int SFP_BYTES = KT_PER_STAGE * SF_TILE;
  static constexpr int SFQ_BYTES = SFQ_BLOCKS * KT_PER_STAGE * SF_TILE;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFP_BYTES + SFQ_BYTES;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 /*align slack*/ + 256 /*barriers*/;
  // split-K form: fp32 partials received from the cluster, [token slot][source rank][128 rows]
  static constexpr int RECV_BYTES = BN <= 16 ? (BN + 8) * BM * 4 : 0;   // (wider tiles reduce by remote loads)
  static constexpr int TOTAL_SPLITK = TOTAL + RECV_BYTES;
};

__device__ __forceinline__ void tile_coords(int t, const GemmParams& p, int& pt, int& qt) {
  const int per_group = p.group_m * p.q_tiles;
  const int group = t / per_group;
  const int first = group * p.group_m;
  const int gsize = min(p.p_tiles - first, p.group_m);
  const int r = t - group * per_group;
  pt = first + r % gsize;
  qt = r / gsize;
}

// One stage of P: 128 rows x 128 bytes.  Plain layout: one 2-D box, 128B swizzle.  Interleaved GEMV layout
// ([rows/8][K/64][8 rows][32 B], a dense 4-D tensor): a box of 16 row groups x 4 k-tiles x 8 rows x 32 B, stored
// in that order with the 32-byte swizzle, so that every (row group, k-tile) is one 8-row x 32-byte swizzle atom
// of 256 bytes; the MMA reads it with a SWIZZLE_32B descriptor whose 8-row-group pitch is 1024 bytes and which
// advances 256 bytes per k-tile.
__device__ __forceinline__ void load_p_stage(void* dst, const CUtensorMap* map, uint64_t* bar, int ks, int pt,
                                             bool interleaved) {
  if (interleaved) ptx::tma_load_4d(dst, map, bar, 0, 0, ks * KT_PER_STAGE, pt * (BM / 8));
  else ptx::tma_load_2d(dst, map, bar, ks * 128, pt * BM);
}

// SPLITK (small token counts, SWAP form only): `p.splits` CTAs form a cluster on one tile of 128
// weight rows; CTA r contracts its share of K and PUSHES its fp32 partials into the shared memory of
// the CTA that owns the token column (token j belongs to rank j % splits): one asynchronous store through
// distributed shared memory per value (st.async), which credits its bytes to the owner's mbarrier as it lands.  The owner expects splits x 128 x 4 bytes per column it owns, sums the partials in rank order
// (deterministic) and writes the column out; a CTA that owns no live token exits right after its pushes,
// and nobody reads another CTA's memory, so no barrier holds the cluster together at the end.  That is
// the form for up to 16 token columns (-1.2 us per launch at one token against the pull form).  Wider
// tiles keep the pull form: partials stay in place, and between two cluster barriers every rank reads its
// columns from all ranks' shared memory (pushing 64 columns, by remote stores or by bulk copies from a
// staging area, measured 3 us slower per launch).
// This is what lets a layer with few 128-row tiles pull weights through every SM.
//
// Small token counts (SWAP, BN <= 32): two CTAs fit an SM (4 stages of ~22 KB, 256 TMEM columns
// each), and the kernel is launched as a programmatic dependent: its CTAs become resident beside
// the previous kernel's, and the TMA thread loads the WEIGHT halves of its first stages (weights
// are not written by any kernel of the stream) before it waits for the previous grid; only the
// activation halves wait.  The weight stream of kernel n+1 thus overlaps kernel n, which is what a
// chain of latency-bound decode GEMMs needs.
// TMEM columns a CTA allocates: accumulators + two scale buffers, rounded up to a power of two (>= 32).
template <int BN, int ACC>
__host__ __device__ constexpr int tmem_cols() {
  const int need = ACC * BN + 2 * KT_PER_STAGE * (4 + (BN <= 128 ? 1 : 2) * 4);
  int c = 32;
  while (c < need) c *= 2;
  return c;
}
// CTAs of the small-M (swapped) form that share an SM: as many as fit its shared memory (228 KB, 1 KB reserved
// per CTA) and TMEM (512 columns), at most 4.  Several small CTAs per SM let the CTAs of the NEXT kernel of the
// stream become resident, and prefetch their weights, while this kernel still runs.
template <int BN, int STAGES, int ACC, bool SWAP, bool SPLITK = false>
__host__ __device__ constexpr int ctas_per_sm() {
  if (!SWAP || BN > 64) return 1;
  int n = (228 * 1024) / ((SPLITK ? SmemLayout<BN, STAGES>::TOTAL_SPLITK : SmemLayout<BN, STAGES>::TOTAL) + 1024);
  if (512 / tmem_cols<BN, ACC>() < n) n = 512 / tmem_cols<BN, ACC>();
  return n > 4 ? 4 : (n < 1 ? 1 : n);
}

template <int BN, int STAGES, int ACC, bool SWAP, bool SPLITK = false>
__global__ void __launch_bounds__(192, ctas_per_sm<BN, STAGES, ACC, SWAP, SPLITK>())
nvfp4_gemm_kernel(const __grid_constant__ CUtensorMap map_p, const __grid_constant__ CUtensorMap map_q,
                  const GemmParams p) {
  using L = SmemLayout<BN, STAGES>;
  constexpr int SFQ_COLS_PER_KT = L::SFQ_BLOCKS * 4;               // TMEM columns of Q scales per k-tile
  constexpr int SF_COLS = KT_PER_STAGE * (4 + SFQ_COLS_PER_KT);    // per SF buffer
  constexpr int ACC_COLS = ACC * BN;
  static_assert(ACC_COLS + 2 * SF_COLS <= 512, "TMEM budget");
  constexpr uint32_t TMEM_COLS = tmem_cols<BN, ACC>();
  static_assert(ACC_COLS + 2 * SF_COLS <= static_cast<int>(TMEM_COLS), "TMEM allocation");
  constexpr uint32_t IDESC = ptx::idesc_nvf4(BM, BN);
  constexpr bool SPLITK_PUSH = SPLITK && BN <= 16;   // how split-K partials travel (see the comment above the kernel)
  static_assert(!SPLITK || STAGES * L::STAGE_BYTES >= BN * BM * 4, "the ring holds a partial tile");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * L::STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES] TMA -> MMA
  uint64_t* empty = bars + STAGES;          // [STAGES] MMA -> TMA
  uint64_t* acc_full = bars + 2 * STAGES;   // [ACC]    MMA -> epilogue
  uint64_t* acc_empty = acc_full + ACC;     // [ACC]    epilogue -> MMA
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  uint64_t* recv_bar = bars + 30;                                        // split-K: partials have arrived (last 16 bytes of the 256)
  float* recv = reinterpret_cast<float*>(smem + STAGES * L::STAGE_BYTES + 256);   // split-K: [slot][rank][BM]
  static_assert((2 * STAGES + 2 * ACC + 1) * 8 <= 240, "barrier area");

  pdl_launch_dependents();
  FRT_GT_DECL;
  if (threadIdx.x == 0) { FRT_GT_ZERO; FRT_GT(p, 0); }
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int total_tiles = p.p_tiles * p.q_tiles;
  const int k_stages_all = (p.k_tiles + KT_PER_STAGE - 1) / KT_PER_STAGE;
  static_assert(!SPLITK || SWAP, "split-K exists for the swapped form only");
  const int krank = SPLITK ? static_cast<int>(ptx::cluster_ctarank()) : 0;
  const int k_per = SPLITK ? k_stages_all / p.splits : k_stages_all;      // host makes it divide
  const int ks_begin = krank * k_per;
  const int k_stages = ks_begin + k_per;                                   // loop bound (exclusive)
  const int tile_first = SPLITK ? static_cast<int>(blockIdx.x) / p.splits : static_cast<int>(blockIdx.x);
  const int tile_step = SPLITK ? static_cast<int>(gridDim.x) / p.splits : static_cast<int>(gridDim.x);

  int n_pre = 0;          // thread 0: leading stages whose weight half was requested before the wait
  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { ptx::mbar_init(&full[i], 1); ptx::mbar_init(&empty[i], 1); }
    for (int i = 0; i < ACC; ++i) { ptx::mbar_init(&acc_full[i], 1); ptx::mbar_init(&acc_empty[i], 4); }
    if (SPLITK_PUSH) ptx::mbar_init(recv_bar, 1);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    if (SPLITK_PUSH) {
      // this rank owns token columns krank, krank + splits, ... of the tile: it expects every rank's 128-row
      // partial of each (the single arrival of the phase is this one; the bytes come from the peers' stores)
      const int live = min(BN, p.Q), owned = krank < live ? (live - krank + p.splits - 1) / p.splits : 0;
      if (owned) ptx::mbar_expect_tx(recv_bar, static_cast<uint32_t>(owned * p.splits * BM * 4));
    }
    ptx::prefetch_tensormap(&map_p);
    ptx::prefetch_tensormap(&map_q);
    // Small token counts: the WEIGHT halves of the first stages are requested right here, before the TMEM
    // allocation, the CTA barrier and the wait for the previous grid: weights are constants of the stream,
    // and a CTA that became resident late (its predecessor's CTAs held the SM) has no other way to hide
    // the first trip to HBM.  This thread is also the TMA producer below.
    if (SWAP && tile_first < total_tiles) {
      int pt, qt;
      tile_coords(tile_first, p, pt, qt);
      const int qblk0 = (qt * BN) >> 7;
      int nblk = 0;
      for (int b = 0; b < L::SFQ_BLOCKS; ++b) nblk += (qblk0 + b < p.sfq_row_blocks) ? 1 : 0;
      for (int ks = ks_begin; ks < k_stages && n_pre < STAGES; ++ks, ++n_pre) {
        uint8_t* st = smem + n_pre * L::STAGE_BYTES;
        const int kts = min(KT_PER_STAGE, p.k_tiles - ks * KT_PER_STAGE);
        ptx::mbar_expect_tx(&full[n_pre], L::A_BYTES + L::B_BYTES + kts * SF_TILE * (1 + nblk));
        load_p_stage(st, &map_p, &full[n_pre], ks, pt, SWAP && p.p_interleaved);
        ptx::bulk_load(st + L::A_BYTES + L::B_BYTES,
                       p.sfp + (static_cast<int64_t>(pt) * p.sf_cols + ks * KT_PER_STAGE) * SF_TILE,
                       kts * SF_TILE, &full[n_pre]);
      }
    }
    FRT_GT(p, 1);
  }
  if (warp == 1) {
    ptx::tmem_alloc(tmem_slot, TMEM_COLS);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // split-K: every CTA's receive barrier exists before anybody pushes: all threads arrive here (no
  // waiting), the epilogue warps complete the cluster barrier just before their first push
  if (SPLITK_PUSH) ptx::cluster_arrive();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above overlapped the previous kernel of the stream.  From here on global memory:
  // all warps wait for the previous grid, except the TMA thread, which first issues the loads
  // that cannot depend on it (see below).
  if (warp != 0) pdl_wait();

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {        // (thread 0: it issued the early weight loads above)
      int it = 0;
      pdl_wait();
      FRT_GT(p, 2);
      for (int t = tile_first; t < total_tiles && !*abort_flag; t += tile_step) {
        int pt, qt;
        tile_coords(t, p, pt, qt);
        const int q0 = qt * BN;
        const int qblk0 = q0 >> 7;
        for (int ks = ks_begin; ks < k_stages; ++ks, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          uint8_t* st = smem + s * L::STAGE_BYTES;
          const int kts = min(KT_PER_STAGE, p.k_tiles - ks * KT_PER_STAGE);
          int nblk = 0;
          for (int b = 0; b < L::SFQ_BLOCKS; ++b) nblk += (qblk0 + b < p.sfq_row_blocks) ? 1 : 0;
          if (it >= n_pre) {   // (the first n_pre stages were armed, and their P half loaded, above)
            if (!ptx::mbar_wait_bounded(&empty[s], ph ^ 1, WAIT_LIMIT)) {
              atomicOr(&g_status_word, 1u); *abort_flag = 1; break;
            }
            const uint32_t bytes = L::A_BYTES + L::B_BYTES + kts * SF_TILE * (1 + nblk);
            ptx::mbar_expect_tx(&full[s], bytes);
            load_p_stage(st, &map_p, &full[s], ks, pt, SWAP && p.p_interleaved);
            ptx::bulk_load(st + L::A_BYTES + L::B_BYTES,
                           p.sfp + (static_cast<int64_t>(pt) * p.sf_cols + ks * KT_PER_STAGE) * SF_TILE,
                           kts * SF_TILE, &full[s]);
          }
          ptx::tma_load_2d(st + L::A_BYTES, &map_q, &full[s], ks * 128, q0);
          for (int b = 0; b < nblk; ++b)
            ptx::bulk_load(st + L::A_BYTES + L::B_BYTES + L::SFP_BYTES + b * KT_PER_STAGE * SF_TILE,
                           p.sfq + (static_cast<int64_t>(qblk0 + b) * p.sf_cols + ks * KT_PER_STAGE) * SF_TILE,
                           kts * SF_TILE, &full[s]);
        }
      }
      // drain: wait until the MMA side has released every stage this thread armed,
      // so no bulk copy is in flight when the CTA exits
      if (!*abort_flag) {
        for (int i = 0; i < STAGES && i < it; ++i) {
          const int j = it - 1 - i;
          if (!ptx::mbar_wait_bounded(&empty[j % STAGES], (j / STAGES) & 1, WAIT_LIMIT)) {
            atomicOr(&g_status_word, 2u); break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (ptx::elect_one()) {
      // Descriptors differ between stages and k-tiles only in their low word
      // (address >> 4), so the loop adds small constants to 32-bit values.
      const uint32_t smem0 = ptx::smem_u32(smem);
      const uint64_t op_desc = ptx::desc_sw128_kmajor(smem0);
      const uint64_t sf_desc = ptx::desc_sf_32x16(smem0 + L::A_BYTES + L::B_BYTES);
      const uint32_t op_hi = static_cast<uint32_t>(op_desc >> 32), op_lo0 = static_cast<uint32_t>(op_desc);
      const uint32_t sf_hi = static_cast<uint32_t>(sf_desc >> 32), sf_lo0 = static_cast<uint32_t>(sf_desc);
      // P operand of the interleaved layout: layout type 6 (SWIZZLE_32B) in descriptor bits 61..63, 256 bytes per k-tile
      const bool p_ilv = SWAP && p.p_interleaved;
      const uint32_t p_hi = p_ilv ? ((op_hi & 0x1fffffffu) | (6u << 29)) : op_hi;
      const uint32_t p_step = p_ilv ? 16u : 2u;
      const bool copy_always = !FRT_DBG(p, 2);
      int s = 0, tl = 0;
      uint32_t ph = 0, sfbuf = 0;
      bool aborted = false;
      for (int t = tile_first; t < total_tiles && !*abort_flag; t += tile_step, ++tl) {
        const int a = tl % ACC;
        const uint32_t aph = (tl / ACC) & 1;
        if (!ptx::mbar_wait_bounded(&acc_empty[a], aph ^ 1, WAIT_LIMIT)) {
          atomicOr(&g_status_word, 4u); *abort_flag = 1; break;
        }
        ptx::tc_fence_after();
        const uint32_t d_tmem = tmem_base + a * BN;
        // tile start inside its first 128-row scale group, in 32-row TMEM columns
        int pt, qt;
        tile_coords(t, p, pt, qt);
        const uint32_t qoff = (static_cast<uint32_t>(qt * BN) & 127u) >> 5;
        for (int ks = ks_begin; ks < k_stages; ++ks) {
          if (!ptx::mbar_wait_bounded(&full[s], ph, WAIT_LIMIT)) {
            atomicOr(&g_status_word, 8u); *abort_flag = 1; aborted = true; break;
          }
          ptx::tc_fence_after();
          if (tl == 0 && ks == ks_begin) FRT_GT(p, 3);
          const uint32_t a_lo = op_lo0 + s * (L::STAGE_BYTES >> 4);
          const uint32_t b_lo = a_lo + (L::A_BYTES >> 4);
          const uint32_t sfp_lo = sf_lo0 + s * (L::STAGE_BYTES >> 4);
          const uint32_t sfq_lo = sfp_lo + (L::SFP_BYTES >> 4);
          const uint32_t sf_tmem = tmem_base + ACC_COLS + sfbuf * SF_COLS;
          const int kts = min(KT_PER_STAGE, p.k_tiles - ks * KT_PER_STAGE);
          const bool do_copy = copy_always || (tl == 0 && ks < 2);
          if (kts == KT_PER_STAGE) {
#pragma unroll
            for (int kt = 0; kt < KT_PER_STAGE; ++kt) {
              const uint32_t sfp_t = sf_tmem + kt * 4;
              const uint32_t sfq_t = sf_tmem + KT_PER_STAGE * 4 + kt * SFQ_COLS_PER_KT;
              if (do_copy) {
                ptx::tc_cp_32x128b_warpx4(sfp_t, sfp_lo + kt * (SF_TILE >> 4), sf_hi);
#pragma unroll
                for (int b = 0; b < L::SFQ_BLOCKS; ++b)
                  ptx::tc_cp_32x128b_warpx4(sfq_t + 4 * b, sfq_lo + (b * KT_PER_STAGE + kt) * (SF_TILE >> 4), sf_hi);
              }
              // +2 per k-tile: 32 bytes (64 e2m1) along K inside the 128-byte swizzle span
              ptx::tc_mma_nvf4(d_tmem, a_lo + p_step * kt, b_lo + 2 * kt, p_hi, op_hi, IDESC, sfp_t, sfq_t + qoff,
                               ks != ks_begin || kt != 0);
            }
          } else {
            for (int kt = 0; kt < kts; ++kt) {
              const uint32_t sfp_t = sf_tmem + kt * 4;
              const uint32_t sfq_t = sf_tmem + KT_PER_STAGE * 4 + kt * SFQ_COLS_PER_KT;
              ptx::tc_cp_32x128b_warpx4(sfp_t, sfp_lo + kt * (SF_TILE >> 4), sf_hi);
              for (int b = 0; b < L::SFQ_BLOCKS; ++b)
                ptx::tc_cp_32x128b_warpx4(sfq_t + 4 * b, sfq_lo + (b * KT_PER_STAGE + kt) * (SF_TILE >> 4), sf_hi);
              ptx::tc_mma_nvf4(d_tmem, a_lo + p_step * kt, b_lo + 2 * kt, p_hi, op_hi, IDESC, sfp_t, sfq_t + qoff,
                               ks != ks_begin || kt != 0);
            }
          }
          ptx::tc_commit(&empty[s]);
          sfbuf ^= 1u;
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (aborted) break;
        ptx::tc_commit(&acc_full[a]);
        FRT_GT(p, 4);
      }
    }
  } else {
    // ===================== epilogue (warps 2..5) =====================
    const int quarter = warp & 3;      // TMEM lanes [32*quarter, +32)
    int tl = 0;
    for (int t = tile_first; t < total_tiles && !*abort_flag; t += tile_step, ++tl) {
      int pt, qt;
      tile_coords(t, p, pt, qt);
      const int a = tl % ACC;
      const uint32_t aph = (tl / ACC) & 1;
      if (!ptx::mbar_wait_bounded(&acc_full[a], aph, WAIT_LIMIT)) {
        if (lane == 0) { atomicOr(&g_status_word, 16u); *abort_flag = 1; }
        break;
      }
      ptx::tc_fence_after();
      if (warp == 2 && lane == 0) FRT_GT(p, 5);
      if (SPLITK_PUSH) {                                       // every rank's receive barrier is initialised
        __syncwarp();
        ptx::cluster_wait();
      }
      const int prow = pt * BM + quarter * 32 + lane;          // index on the P axis
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + a * BN;
#pragma unroll 1
      for (int cchunk = 0; cchunk < BN / 32 || (BN % 32 && cchunk * 32 < BN); ++cchunk) {
        const int q_base = qt * BN + cchunk * 32;                // index on the Q axis
        if (q_base >= p.Q) break;                                // warp-uniform
        uint32_t r[32];
        if (BN % 32 == 0 || cchunk * 32 + 32 <= BN) {
          ptx::tc_ld_32x32b_x32(taddr + cchunk * 32, r);
          ptx::tc_wait_ld(r);
        } else {
          uint32_t r16[16];
          ptx::tc_ld_32x32b_x16(taddr + cchunk * 32, r16);
#pragma unroll
          for (int j = 0; j < 16; ++j) { r[j] = r16[j]; r[16 + j] = 0; }
        }
        ptx::tc_wait_ld();
        if (!SWAP) {
          // thread = output row prow, 32 consecutive output columns from q_base
          if (prow < p.P) {
            const int64_t off = static_cast<int64_t>(prow) * p.ldd + q_base;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = q_base + 8 * g;
              if (col >= p.Q) break;
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[8 * g + j]) * p.alpha;
              if (p.bias != nullptr) {
                float b[8];
                unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(p.bias + col)), b);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += b[j];
              }
              if (p.c != nullptr) {
                float cc[8];
                unpack_bf16x8(*reinterpret_cast<const uint4*>(p.c + off + 8 * g), cc);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += p.beta * cc[j];
              }
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]); o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]); o.w = pack_bf16x2(v[6], v[7]);
              if (!FRT_DBG(p, 1)) *reinterpret_cast<uint4*>(p.d + off + 8 * g) = o;
            }
          }
        } else {
          if (SPLITK && !SPLITK_PUSH) {
            // fp32 partial of this CTA's K share: part[token][weight row in tile], in the (idle) stage ring
            float* part = reinterpret_cast<float*>(smem);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (cchunk * 32 + j < BN) part[(cchunk * 32 + j) * BM + quarter * 32 + lane] = __uint_as_float(r[j]);
            continue;
          }
          if (SPLITK_PUSH) {
            // fp32 partial of this CTA's K share: token jt goes to rank jt % splits, where it is slot jt / splits
            // of source krank: one asynchronous remote store per value
            const uint32_t row4 = static_cast<uint32_t>(quarter * 32 + lane) * 4u;
            const uint32_t slots = static_cast<uint32_t>((BN + p.splits - 1) / p.splits);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int jt = cchunk * 32 + j;
              if (jt < BN && q_base + j < p.Q) {
                const uint32_t owner = static_cast<uint32_t>(jt % p.splits), slot = static_cast<uint32_t>(jt / p.splits);
                ptx::st_async_cluster_f32(ptx::mapa(ptx::smem_u32(recv) + row4 + (krank * slots + slot) * (BM * 4u), owner),
                                          __uint_as_float(r[j]), ptx::mapa(ptx::smem_u32(recv_bar), owner));
              }
            }
            continue;
          }
          // thread = output column prow (a weight row), columns of the tile = tokens
          const float bias = (p.bias != nullptr && prow < p.P) ? __bfloat162float(p.bias[prow]) : 0.f;
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int tok = q_base + j;
            if (tok < p.Q && prow < p.P) {
              const int64_t off = static_cast<int64_t>(tok) * p.ldd + prow;
              float v = __uint_as_float(r[j]) * p.alpha + bias;
              if (p.c != nullptr) v += p.beta * __bfloat162float(p.c[off]);
              p.d[off] = __float2bfloat16_rn(v);
            }
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&acc_empty[a]);
      if (SPLITK_PUSH) {
        const int live = min(BN, p.Q - qt * BN), owners = min(live, p.splits);
        const int slots = (BN + p.splits - 1) / p.splits;
        if (warp == 2 && lane == 0) FRT_GT(p, 6);
        if (krank < owners) {
          // this rank owns token columns krank, krank + splits, ...: all ranks' partials, summed in rank order
          if (!ptx::mbar_wait_bounded_acquire_cluster(recv_bar, 0, WAIT_LIMIT)) {
            if (lane == 0) { atomicOr(&g_status_word, 16u); *abort_flag = 1; }
            break;
          }
          if (warp == 2 && lane == 0) FRT_GT(p, 8);
          const int row = quarter * 32 + lane;
          const float bias = (p.bias != nullptr && prow < p.P) ? __bfloat162float(p.bias[prow]) : 0.f;
          for (int jt = krank; jt < live; jt += p.splits) {
            const float* src = recv + static_cast<size_t>(jt / p.splits) * BM + row;     // [source rank][slot][row]
            float part[8];
#pragma unroll
            for (int r = 0; r < 8; ++r) part[r] = r < p.splits ? src[static_cast<size_t>(r * slots) * BM] : 0.f;
            float acc = part[0];
#pragma unroll
            for (int r = 1; r < 8; ++r) acc += part[r];
            if (prow < p.P) {
              const int64_t off = static_cast<int64_t>(qt * BN + jt) * p.ldd + prow;
              float v = acc * p.alpha + bias;
              if (p.c != nullptr) v += p.beta * __bfloat162float(p.c[off]);
              p.d[off] = __float2bfloat16_rn(v);
            }
          }
          if (warp == 2 && lane == 0) FRT_GT(p, 9);
        }
      }
    }
  }

  if (SPLITK_PUSH && warp < 2) {                  // completes the cluster barrier every thread arrived on at the start
    __syncwarp();
    ptx::cluster_wait();
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0) FRT_GT(p, 7);
  if (SPLITK && !SPLITK_PUSH) {
    // more than 16 token columns: partials stay in this CTA's (idle) stage ring, and after a cluster barrier
    // every rank sums its token columns over all ranks through distributed shared memory, in rank order
    ptx::cluster_arrive();
    ptx::cluster_wait();                                  // every rank's partial tile is in its shared memory
    if (warp >= 2 && tile_first < total_tiles && !*abort_flag) {
      int pt, qt;
      tile_coords(tile_first, p, pt, qt);
      const int row = (warp & 3) * 32 + lane;
      const int prow = pt * BM + row;
      const uint32_t part0 = ptx::smem_u32(smem);
      const float bias = (p.bias != nullptr && prow < p.P) ? __bfloat162float(p.bias[prow]) : 0.f;
      // this rank's slice of the token columns; all remote loads of a column are issued
      // before the first is used, and summed in rank order
      uint32_t remote[8];
#pragma unroll
      for (int r = 0; r < 8; ++r) remote[r] = ptx::mapa(part0 + static_cast<uint32_t>(row) * 4u, r < p.splits ? r : 0);
      for (int j = krank; j < BN; j += p.splits) {
        const int tok = qt * BN + j;
        if (tok >= p.Q) break;
        float part[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
          part[r] = r < p.splits ? ptx::ld_cluster_f32(remote[r] + static_cast<uint32_t>(j * BM) * 4u) : 0.f;
        float acc = part[0];
#pragma unroll
        for (int r = 1; r < 8; ++r) acc += part[r];
        if (prow < p.P) {
          const int64_t off = static_cast<int64_t>(tok) * p.ldd + prow;
          float v = acc * p.alpha + bias;
          if (p.c != nullptr) v += p.beta * __bfloat162float(p.c[off]);
          p.d[off] = __float2bfloat16_rn(v);
        }
      }
    }
    ptx::cluster_arrive();
    ptx::cluster_wait();                                  // nobody leaves while its partial may still be read
  }
  if (warp == 1) ptx::tmem_dealloc(tmem_base, TMEM_COLS);
#ifdef FRT_DEBUG
  if (p.trace) {
    __syncthreads();
    if (threadIdx.x == 0) {
      const long long rec = atomicAdd(reinterpret_cast<unsigned long long*>(p.trace), 1ull);
      if (rec < 4000) {
        long long* o = p.trace + 16 + rec * 16;
        unsigned smid; asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        o[0] = (static_cast<long long>(p.P) << 32) | static_cast<unsigned>(p.K);
        o[1] = (static_cast<long long>(blockIdx.x) << 32) | (smid << 8) | static_cast<unsigned>(p.splits);
        for (int i = 0; i < 10; ++i) o[2 + i] = gt_ts[i];
        o[12] = frt_globaltimer();
      }
    }
  }
#endif
}

#include "gemm_pair.cuh"

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
PFN_cuTensorMapEncodeTiled_v12000 get_encode() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// packed e2m1 [rows, K/2] bytes, row-major; box = 128 bytes x box_rows, 128B swizzle
int make_operand_map(CUtensorMap* map, const void* base, int rows, int K, int box_rows) {
  auto enc = get_encode();
  if (!enc) return FRT_E_DRIVER;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K / 2), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K / 2)};
  const cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FRT_OK : FRT_E_DRIVER;
}

// packed e2m1 weights in the interleaved GEMV layout: the dense 4-D tensor [rows/8][K/64][8 rows][32 bytes];
// box = 16 row groups x 4 k-tiles x 8 rows x 32 bytes (one stage), 32-byte swizzle
int make_interleaved_map(CUtensorMap* map, const void* base, int rows, int K) {
  auto enc = get_encode();
  if (!enc) return FRT_E_DRIVER;
  const cuuint64_t kt = static_cast<cuuint64_t>(K / 64);
  const cuuint64_t dims[4] = {32, 8, kt, static_cast<cuuint64_t>(rows / 8)};
  const cuuint64_t strides[3] = {32, 256, kt * 256};
  const cuuint32_t box[4] = {32, 8, KT_PER_STAGE, BM / 8};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FRT_OK : FRT_E_DRIVER;
}

// swizzled scale buffer as [row_blocks][sf_cols][512 bytes]; box = `blocks` row groups x 4 k-tiles
int make_sf_map(CUtensorMap* map, const void* base, int rows, int sf_cols, int blocks) {
  auto enc = get_encode();
  if (!enc) return FRT_E_DRIVER;
  const cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(sf_cols), static_cast<cuuint64_t>((rows + 127) / 128)};
  const cuuint64_t strides[2] = {512, static_cast<cuuint64_t>(sf_cols) * 512};
  const cuuint32_t box[3] = {128, KT_PER_STAGE, static_cast<cuuint32_t>(blocks)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FRT_OK : FRT_E_DRIVER;
}

// bf16 output [rows, cols] with row pitch `ld` elements; box = 32 columns x 32 rows, 64-byte swizzle
int make_output_map(CUtensorMap* map, void* base, int rows, int cols, int ld) {
  auto enc = get_encode();
  if (!enc) return FRT_E_DRIVER;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {32, 32};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FRT_OK : FRT_E_DRIVER;
}

struct DeviceInfo { int sms = 0; int cc_major = 0; bool ok = false; };
DeviceInfo device_info() {
  // per-device cache (index by current device)
  static DeviceInfo cache[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return DeviceInfo{};
  if (!cache[dev].ok) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return DeviceInfo{};
    cache[dev].sms = prop.multiProcessorCount;
    cache[dev].cc_major = prop.major;
    cache[dev].ok = true;
  }
  return cache[dev];
}

template <int BN, int STAGES, int ACC, bool SWAP>
int launch_gemm(const CUtensorMap& mp, const CUtensorMap& mq, GemmParams& p, int sms, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = nvfp4_gemm_kernel<BN, STAGES, ACC, SWAP>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return FRT_E_LAUNCH;
    attr_set[dev & 63] = true;
  }
  p.q_tiles = (p.Q + BN - 1) / BN;
  p.p_tiles = (p.P + BM - 1) / BM;
  const int tiles = p.p_tiles * p.q_tiles;
  const int slots = ctas_per_sm<BN, STAGES, ACC, SWAP>() * sms;
  const int grid = tiles < slots ? tiles : slots;
  launch_pdl(kern, dim3(grid), dim3(192), L::TOTAL, st, mp, mq, p);
  return launch_result();
}

template <int BN, int STAGES>
int launch_gemm_pair(const void* p_packed, const void* q_packed, GemmParams& p, int sms, cudaStream_t st) {
  using L = PairLayout<BN, STAGES, false>;
  auto kern = nvfp4_gemm_pair_kernel<BN, STAGES, false>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return FRT_E_LAUNCH;
    attr_set[dev & 63] = true;
  }
  PairMaps maps;
  if (int rc = make_operand_map(&maps.p, p_packed, p.P, p.K, 128)) return rc;
  if (int rc = make_operand_map(&maps.q, q_packed, p.Q, p.K, BN / 2)) return rc;
  if (int rc = make_sf_map(&maps.sfp, p.sfp, p.P, p.sf_cols, 1)) return rc;
  if (int rc = make_sf_map(&maps.sfq, p.sfq, p.Q, p.sf_cols, L::SFQ_BLOCKS)) return rc;
  if (int rc = make_output_map(&maps.d, p.d, p.P, p.Q, p.ldd)) return rc;
  if (BN == 256)
    if (int rc = make_operand_map(&maps.q32, q_packed, p.Q, p.K, 32)) return rc;
  p.q_tiles = (p.Q + BN - 1) / BN;
  p.p_tiles = (p.P + 255) / 256;
  const int tiles = p.p_tiles * p.q_tiles;
  // Last wave: `left` tiles for sms/2 pairs.  Cutting each into 4 (or 2) column slices gives every
  // pair work for a fraction of a tile's time instead of leaving most of them idle for a whole one.
  // A slice still streams the whole P tile, so it costs ~0.75 of a tile: measured +2-4 % on the
  // Qwen3-8B qkv / o shapes, nothing at K = 12288 (two-way slices are kept to K < 8192).
  const int all_pairs = sms / 2;
  const int left = tiles % all_pairs;
  p.tail_split = 1;
  if (BN == 256 && left > 0 && g_opt_tail_split) {
    if (left * 4 <= all_pairs) p.tail_split = 4;
    else if (left * 2 <= all_pairs && p.K < 8192) p.tail_split = 2;
  }
  p.tail_first = p.tail_split > 1 ? tiles - left : tiles;
  p.units = p.tail_first + (tiles - p.tail_first) * p.tail_split;
  const int pairs = p.units < all_pairs ? p.units : all_pairs;
  launch_pdl(kern, dim3(2 * pairs), dim3(320), L::TOTAL, st, maps, p, static_cast<const GroupWork*>(nullptr));
  return launch_result();
}

// GEMM + SwiGLU + NVFP4 quantiser in one kernel (256 x (128 gate + 128 up) tiles).
int launch_gemm_swiglu(const void* p_packed, const void* q_packed, GemmParams& p, int sms, cudaStream_t st) {
  using L = PairLayout<256, 5, false>;
  auto kern = nvfp4_gemm_pair_kernel<256, 5, false, true>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return FRT_E_LAUNCH;
    attr_set[dev & 63] = true;
  }
  PairMaps maps{};
  if (int rc = make_operand_map(&maps.p, p_packed, p.P, p.K, 128)) return rc;
  if (int rc = make_operand_map(&maps.q, q_packed, p.Q, p.K, 128)) return rc;
  if (int rc = make_sf_map(&maps.sfp, p.sfp, p.P, p.sf_cols, 1)) return rc;
  if (int rc = make_sf_map(&maps.sfq, p.sfq, p.Q, p.sf_cols, 1)) return rc;
  p.q_tiles = p.hidden / 128;
  p.p_tiles = (p.P + 255) / 256;
  const int tiles = p.p_tiles * p.q_tiles;
  const int pairs = tiles < sms / 2 ? tiles : sms / 2;
  launch_pdl(kern, dim3(2 * pairs), dim3(576), L::TOTAL, st, maps, p, static_cast<const GroupWork*>(nullptr));
  return launch_result();
}

template <int BN, int STAGES>
int launch_gemm_splitk(const CUtensorMap& mp, const CUtensorMap& mq, GemmParams& p, cudaStream_t st) {
  using L = SmemLayout<BN, STAGES>;
  auto kern = nvfp4_gemm_kernel<BN, STAGES, 1, true, true>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL_SPLITK) != cudaSuccess)
      return FRT_E_LAUNCH;
    attr_set[dev & 63] = true;
  }
  p.q_tiles = 1;
  p.p_tiles = (p.P + BM - 1) / BM;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(static_cast<unsigned>(p.p_tiles * p.splits));
  cfg.blockDim = dim3(192);
  cfg.dynamicSmemBytes = L::TOTAL_SPLITK;
  cfg.stream = st;
  cudaLaunchAttribute attr[2] = {};
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = static_cast<unsigned>(p.splits);
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_opt_pdl ? 2 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mp, mq, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return e == cudaSuccess ? FRT_OK : FRT_E_LAUNCH;
}

// ---------------------------------------------------------------------------
// grouped (MoE): plan kernel + launch
// ---------------------------------------------------------------------------
// Windows start on a multiple of 64 rows: the scales of a window are addressed in
// TMEM as a column offset (one column per 32 rows) from a 128-row group, and the
// MMA takes that scale address only at even columns.
// Rows of the window that starts at `start` when the expert's rows end at `hi`: what is left, rounded up to
// 32, if that is at most 320; else 256.
__device__ __forceinline__ int window_rows(int start, int hi) { return grouped_window_rows(start, hi); }

__device__ __forceinline__ void emit_windows(GroupWork* work, int max_items, int lo, int hi, int expert) {
  // All windows of one expert take consecutive slots: their tiles then run at about the same
  // time on neighbouring CTA pairs and the expert's weights leave HBM once (with one slot per
  // atomic the windows of an expert ended up hundreds of tiles apart and the weights, long
  // evicted from L2, were streamed again for each).
  // A window is 256 rows, or up to 320 when that takes in the expert's last rows: the rows beyond 256 are
  // contracted by a second MMA against the weights already staged, so an expert with a few rows more than a
  // full window does not stream its weights a second time for them.
  const int first = lo & ~63;
  int n_win = 0;
  for (int start = first; start < hi; start += window_rows(start, hi)) ++n_win;
  int slot = atomicAdd(&work->count, n_win);
  // A list that does not fit (overlapping or unsorted offsets: a sorted description always fits the
  // documented workspace) is cut short, never overrun: the GEMM kernel clamps the count the same way,
  // and the status word tells the host that rows were dropped.
  if (slot + n_win > max_items) atomicOr(&g_status_word, 0x200u);
  for (int start = first; start < hi; ++slot) {
    const int len = window_rows(start, hi);
    if (slot < max_items) {
      GroupItem it{};
      it.q_row0 = start; it.n_tokens = len;
      it.lo = max(lo, start); it.hi = min(hi, start + len);
      it.expert = expert;
      work->items[slot] = it;
    }
    start += len;
  }
}

// Token-major items: the 128-row blocks an expert's rows touch, two per item (one per CTA of a pair; -1 = none).
__device__ __forceinline__ void emit_block_pairs(GroupWork* work, int max_items, int lo, int hi, int expert) {
  const int b0 = lo >> 7, b1 = (hi - 1) >> 7;
  const int n_items = (b1 - b0 + 2) / 2;
  int slot = atomicAdd(&work->count, n_items);
  if (slot + n_items > max_items) atomicOr(&g_status_word, 0x200u);
  for (int b = b0; b <= b1; b += 2, ++slot) {
    if (slot < max_items) {
      GroupItem it{};
      it.q_row0 = b;                          // block of CTA 0
      it.n_tokens = b + 1 <= b1 ? b + 1 : -1; // block of CTA 1
      it.lo = lo; it.hi = hi;
      it.expert = expert;
      work->items[slot] = it;
    }
  }
}

// Turns either description of "which expert owns which rows" into windows of
// at most 256 rows that start on a multiple of 64 (weight-major form), or into pairs of 128-row blocks
// (token-major form).
__global__ void group_plan_kernel(const int* __restrict__ offsets, const int* __restrict__ tile_expert, int tile_rows,
                                  int rows, int num_experts, int num_tiles, GroupWork* work, int max_items,
                                  int token_major) {
  pdl_launch_dependents();
  pdl_wait();
  if (gridDim.x == 1) {            // a single CTA resets the list itself (the host skips its memset)
    if (threadIdx.x == 0) work->count = 0;
    __syncthreads();
  }
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (offsets != nullptr) {
    if (i >= num_experts) return;
    const int lo = max(0, min(offsets[i], rows)), hi = max(0, min(offsets[i + 1], rows));
    if (hi > lo) {
      if (token_major) emit_block_pairs(work, max_items, lo, hi, i);
      else emit_windows(work, max_items, lo, hi, i);
    }
  } else {
    if (i >= num_tiles) return;
    const int e = tile_expert[i];
    if (e < 0 || e >= num_experts || (i > 0 && tile_expert[i - 1] == e)) return;   // not the first tile of a run
    int j = i + 1;
    while (j < num_tiles && tile_expert[j] == e) ++j;
    if (token_major) emit_block_pairs(work, max_items, i * tile_rows, j * tile_rows, e);
    else emit_windows(work, max_items, i * tile_rows, j * tile_rows, e);
  }
}

int make_weight_stack_map(CUtensorMap* map, const void* base, int n, int K, int experts, int64_t stride) {
  auto enc = get_encode();
  if (!enc) return FRT_E_DRIVER;
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(K / 2), static_cast<cuuint64_t>(n), static_cast<cuuint64_t>(experts)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(K / 2), static_cast<cuuint64_t>(stride)};
  const cuuint32_t box[3] = {128, 128, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FRT_OK : FRT_E_DRIVER;
}

int make_sf_stack_map(CUtensorMap* map, const void* base, int n, int sf_cols, int experts, int64_t stride,
                      int blocks = 1) {
  auto enc = get_encode();
  if (!enc) return FRT_E_DRIVER;
  const cuuint64_t dims[4] = {128, static_cast<cuuint64_t>(sf_cols), static_cast<cuuint64_t>((n + 127) / 128),
                              static_cast<cuuint64_t>(experts)};
  const cuuint64_t strides[3] = {512, static_cast<cuuint64_t>(sf_cols) * 512, static_cast<cuuint64_t>(stride)};
  const cuuint32_t box[4] = {128, KT_PER_STAGE, static_cast<cuuint32_t>(blocks), 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, const_cast<void*>(base), dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FRT_OK : FRT_E_DRIVER;
}

}  // namespace

// Capacity of the work list for `rows` expert-sorted rows.  Offsets form: an expert with r rows gives at most
// r / 256 + 2 windows (its first window starts on the 64-row boundary below its first row).  tile_expert form:
// a run of equal tiles gives at most as many windows as it has 16-row tiles, so rows / 16 covers any
// interleaving of experts (the reference's test pattern `arange(tiles) % experts` makes every tile a run).
int64_t grouped_max_items(int rows, int experts) { return static_cast<int64_t>(rows) / 16 + 2ll * experts + 8; }

template <int STAGES>
int run_grouped_impl(const void* a, const void* sfa, const void* b_stack, const void* sfb_stack, const void* alpha,
                const void* offsets, const void* tile_expert, int tile_rows, void* out, int rows, int N, int K,
                int experts, int64_t b_stride, int64_t sfb_stride, void* workspace, cudaStream_t st) {
  const DeviceInfo di = device_info();
  if (!di.ok || di.cc_major != 10) return FRT_E_DEVICE;
  constexpr int BN = 256;
  using L = PairLayout<BN, STAGES, true>;
  auto kern = nvfp4_gemm_pair_kernel<BN, STAGES, true>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return FRT_E_LAUNCH;
    attr_set[dev & 63] = true;
  }
  GemmParams p{};
  p.P = N; p.Q = rows; p.K = K;
  p.k_tiles = (K + 63) / 64;
  p.sf_cols = p.k_tiles;
  p.d = static_cast<__nv_bfloat16*>(out);
  p.ldd = N;
  p.alpha = 1.f;
  p.alpha_stack = static_cast<const float*>(alpha);
  p.p_tiles = (N + 255) / 256;
  p.q_tiles = 0;
  p.group_m = 1;
  p.wait_limit = wait_limit_clocks();
  p.max_items = static_cast<int>(grouped_max_items(rows, experts));
#ifdef FRT_DEBUG
  p.dbg = g_opt_gemm_debug & 0xff;
  p.trace = g_trace;
#endif
  PairMaps maps{};
  if (int rc = make_weight_stack_map(&maps.p, b_stack, N, K, experts, b_stride)) return rc;
  if (int rc = make_operand_map(&maps.q, a, rows, K, 32)) return rc;          // token windows load in 32-row boxes
  if (int rc = make_sf_stack_map(&maps.sfp, sfb_stack, N, p.sf_cols, experts, sfb_stride)) return rc;
  if (int rc = make_sf_map(&maps.sfq, sfa, rows, p.sf_cols, 1)) return rc;      // one 128-row scale group per load
  if (int rc = make_output_map(&maps.d, out, rows, N, N)) return rc;
  auto* work = static_cast<GroupWork*>(workspace);
  const int max_items = p.max_items;
  if (offsets != nullptr && experts <= L::PLAN_EXPERTS) {
    // per-expert offsets, few enough experts: the GEMM's CTAs derive the window list themselves (one launch)
    p.inline_offsets = static_cast<const int*>(offsets);
    p.num_experts = experts;
  } else {
    const int num_tiles = tile_rows > 0 ? rows / tile_rows : 0;
    const int plan_threads = offsets ? experts : num_tiles;
    if (plan_threads > 256 && cudaMemsetAsync(work, 0, 16, st) != cudaSuccess) return FRT_E_LAUNCH;   // (else the plan's one CTA does it)
    launch_pdl(group_plan_kernel, dim3((plan_threads + 255) / 256), dim3(256), 0, st, static_cast<const int*>(offsets),
               static_cast<const int*>(tile_expert), tile_rows, rows, experts, num_tiles, work, max_items, 0);
    g_launches.fetch_add(1, std::memory_order_relaxed);
  }
  launch_pdl(kern, dim3(2 * (di.sms / 2)), dim3(320), L::TOTAL, st, maps, p, static_cast<const GroupWork*>(work));
  return launch_result();
}

// Token-major grouped form: token blocks on the 256-row M axis, 256 output columns of the expert's weights on N.
int run_grouped_token_major(const void* a, const void* sfa, const void* b_stack, const void* sfb_stack,
                            const void* alpha, const void* offsets, const void* tile_expert, int tile_rows, void* out,
                            int rows, int N, int K, int experts, int64_t b_stride, int64_t sfb_stride, void* workspace,
                            cudaStream_t st) {
  const DeviceInfo di = device_info();
  if (!di.ok || di.cc_major != 10) return FRT_E_DEVICE;
  constexpr int BN = 256, STAGES = 5;
  using L = PairLayout<BN, STAGES, true, true>;
  auto kern = nvfp4_gemm_pair_kernel<BN, STAGES, true, false, true>;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return FRT_E_LAUNCH;
    attr_set[dev & 63] = true;
  }
  GemmParams p{};
  p.P = rows; p.Q = N; p.K = K;
  p.k_tiles = (K + 63) / 64;
  p.sf_cols = p.k_tiles;
  p.d = static_cast<__nv_bfloat16*>(out);
  p.ldd = N;
  p.alpha = 1.f;
  p.alpha_stack = static_cast<const float*>(alpha);
  p.p_tiles = 0;
  p.q_tiles = (N + BN - 1) / BN;
  p.group_m = 1;
  p.wait_limit = wait_limit_clocks();
  p.max_items = static_cast<int>(grouped_max_items(rows, experts));
#ifdef FRT_DEBUG
  p.dbg = g_opt_gemm_debug & 0xff;
  p.trace = g_trace;
#endif
  PairMaps maps{};
  if (int rc = make_operand_map(&maps.p, a, rows, K, 128)) return rc;
  if (int rc = make_sf_map(&maps.sfp, sfa, rows, p.sf_cols, 1)) return rc;
  if (int rc = make_weight_stack_map(&maps.q, b_stack, N, K, experts, b_stride)) return rc;      // box: 128 rows = BN / 2
  if (int rc = make_sf_stack_map(&maps.sfq, sfb_stack, N, p.sf_cols, experts, sfb_stride, L::SFQ_BLOCKS)) return rc;
  if (int rc = make_output_map(&maps.d, out, rows, N, N)) return rc;
  auto* work = static_cast<GroupWork*>(workspace);
  const int num_tiles = tile_rows > 0 ? rows / tile_rows : 0;
  const int plan_threads = offsets ? experts : num_tiles;
  if (plan_threads > 256 && cudaMemsetAsync(work, 0, 16, st) != cudaSuccess) return FRT_E_LAUNCH;   // (else the plan's one CTA does it)
  launch_pdl(group_plan_kernel, dim3((plan_threads + 255) / 256), dim3(256), 0, st, static_cast<const int*>(offsets),
             static_cast<const int*>(tile_expert), tile_rows, rows, experts, num_tiles, work, p.max_items, 1);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  launch_pdl(kern, dim3(2 * (di.sms / 2)), dim3(320), L::TOTAL, st, maps, p, static_cast<const GroupWork*>(work));
  return launch_result();
}


// Four pipeline stages (a stage holds 128 weight rows, up to 160 token rows and their scales) and two
// store-staging buffers per epilogue warp fill the shared memory of an SM.
int run_grouped(const void* a, const void* sfa, const void* b_stack, const void* sfb_stack, const void* alpha,
                const void* offsets, const void* tile_expert, int tile_rows, void* out, int rows, int N, int K,
                int experts, int64_t b_stride, int64_t sfb_stride, void* workspace, cudaStream_t st) {
  // The weight-major form is the default: on the Qwen3-30B-A3B-shaped layer (128 experts, ~256 rows each) it
  // measured 88 / 77 us for gate/up / down against 101 / 84 us for the token-major form, whose tiles always
  // contract full 128-row blocks (an unaligned expert touches three of them) while a weight-major window is as
  // long as the expert's rows.  FRT_OPT_GROUPED_FORM = 2 selects the token-major form.
  const bool token_major = g_opt_grouped_form == 2;
  if (token_major)
    return run_grouped_token_major(a, sfa, b_stack, sfb_stack, alpha, offsets, tile_expert, tile_rows, out, rows, N, K,
                                   experts, b_stride, sfb_stride, workspace, st);
  return run_grouped_impl<4>(a, sfa, b_stack, sfb_stack, alpha, offsets, tile_expert, tile_rows, out, rows, N, K,
                             experts, b_stride, sfb_stride, workspace, st);
}

unsigned* device_status_word() {
  unsigned* ptr = nullptr;
  cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_status_word);
  return ptr;
}

// Picks the kernel configuration and, for the small-M form, the split-K cluster size.
//   one CTA per tile: 1 = 128x128 (2 acc), 2 = 128x256 (1 acc), 3 = 128x192 (2 acc);
//   CTA pair per tile: 4 = 256x256, 5 = 256x192, 6 = 256x128;
//   swapped (small token counts): 11 = N16, 12 = N32, 13 = N64, 14 = N128
void select_gemm_config(int P, int Q, int K, bool swap, int requested, int sms, int& cfg, int& splits) {
  cfg = requested;
  splits = 1;
  if (cfg == 0) {
    if (swap) cfg = Q <= 16 ? 11 : Q <= 32 ? 12 : Q <= 64 ? 13 : 14;
    else if (P > 128) {
      // CTA pairs.  Estimated time = waves x cost of one tile, with the measured relative
      // tile costs 256-wide 1.0, 192-wide 0.878, 128-wide 0.665 (narrower tiles move more bytes
      // per flop through the ~64 B/clk an SM takes in from L2).  256x256 wins at every full
      // Qwen3-8B / Llama-70B shape; narrower tiles win when a column shard leaves fewer 256-wide
      // tiles than CTA pairs.
      const int pairs = sms / 2, p_tiles = (P + 255) / 256;
      const int widths[3] = {256, 192, 128}, cfgs[3] = {4, 5, 6};
      const float cost[3] = {1.0f, 0.878f, 0.665f};
      float best = 0.f;
      for (int i = 0; i < 3; ++i) {
        const int tiles = p_tiles * ((Q + widths[i] - 1) / widths[i]);
        const float t = static_cast<float>((tiles + pairs - 1) / pairs) * cost[i];
        if (i == 0 || t < best * 0.97f) { best = t; cfg = cfgs[i]; }   // prefer the wider tile on near-ties
      }
    } else {
      cfg = K >= 8192 ? 2 : 3;      // long K amortises the single-accumulator 128x256 tile
    }
  }
  const int bn = cfg == 11 ? 16 : cfg == 12 ? 32 : cfg == 13 ? 64 : 0;
  if (swap && bn && Q <= bn && g_opt_split_k) {
    // few 128-row weight tiles: split K over a cluster so that every SM streams weights
    const int tiles = (P + BM - 1) / BM, k_stages = ((K + 63) / 64 + KT_PER_STAGE - 1) / KT_PER_STAGE;
    if (g_opt_split_k >= 2) {                              // forced (measurements): taken when it divides the K stages
      if (g_opt_split_k <= 8 && k_stages % g_opt_split_k == 0) splits = g_opt_split_k;
      return;
    }
    int want = 2 * sms / tiles;                        // two CTAs of these forms fit an SM
    if (want > 8) want = 8;
    // up to 16 token columns a CTA keeps at least four K stages (o-proj of Qwen3-8B at one token: 4-way
    // 4.2 us, 8-way 4.8 us); wider tiles at least two (64 tokens: 8-way 8.4 us, 4-way 9.2 us)
    const int min_stages = bn == 16 ? 4 : 2;
    for (int s = want; s >= 2; --s)
      if (k_stages % s == 0 && k_stages / s >= min_stages) { splits = s; break; }
    if (bn == 64 && splits < 4) splits = 1;   // 64 token columns: the cross-CTA sum only pays off from 4-way
  }
}

// Shared by the dense and the small-M entry: P/Q already in kernel orientation.
int run_gemm(const void* p_packed, const void* sfp, int P, const void* q_packed, const void* sfq, int Q, int K,
             const void* bias, const void* c, void* d, int ldd, float alpha, float beta, bool swap,
             int config, cudaStream_t st, bool p_interleaved = false) {
  const DeviceInfo di = device_info();
  if (!di.ok || di.cc_major != 10) return FRT_E_DEVICE;
  GemmParams p{};
  p.P = P; p.Q = Q; p.K = K;
  p.k_tiles = (K + 63) / 64;
  p.sf_cols = p.k_tiles;
  p.sfp = static_cast<const uint8_t*>(sfp);
  p.sfq = static_cast<const uint8_t*>(sfq);
  p.sfq_row_blocks = (Q + 127) / 128;
  p.d = static_cast<__nv_bfloat16*>(d);
  p.c = static_cast<const __nv_bfloat16*>(c);
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.ldd = ldd;
  p.alpha = alpha; p.beta = beta;
  p.group_m = 16;
  p.wait_limit = wait_limit_clocks();
#ifdef FRT_DEBUG
  p.dbg = g_opt_gemm_debug & 0xff;
  p.trace = g_trace;
#endif

  int cfg = 0, splits = 1;
  select_gemm_config(P, Q, K, swap, config, di.sms, cfg, splits);
  if (cfg >= 4 && cfg <= 6) {
    if (swap) return FRT_E_UNSUPPORTED;
    switch (cfg) {
      case 4: return launch_gemm_pair<256, 5>(p_packed, q_packed, p, di.sms, st);
      case 5: return launch_gemm_pair<192, 5>(p_packed, q_packed, p, di.sms, st);
      default: return launch_gemm_pair<128, 6>(p_packed, q_packed, p, di.sms, st);
    }
  }
  int bn = 0;
  switch (cfg) {
    case 1: bn = 128; break; case 2: bn = 256; break; case 3: bn = 192; break;
    case 11: bn = 16; break; case 12: bn = 32; break; case 13: bn = 64; break; case 14: bn = 128; break;
    default: return FRT_E_UNSUPPORTED;
  }
  if ((cfg >= 11) != swap) return FRT_E_UNSUPPORTED;
  if (bn < 32 && Q > bn) return FRT_E_UNSUPPORTED;   // a 16-row tile must start a 32-row scale group
  CUtensorMap mp, mq;
  if (p_interleaved) {
    if (!swap) return FRT_E_UNSUPPORTED;
    if (int rc = make_interleaved_map(&mp, p_packed, P, K)) return rc;
  } else if (int rc = make_operand_map(&mp, p_packed, P, K, BM)) {
    return rc;
  }
  if (int rc = make_operand_map(&mq, q_packed, Q, K, bn)) return rc;
  p.p_interleaved = p_interleaved ? 1 : 0;
  p.splits = splits;
  // ring depth of the small-M forms: FRT_OPT_SMALLM_STAGES overrides the default (0) for measurements
  const int depth = g_opt_smallm_stages;
  if (p.splits > 1) {
    switch (cfg) {
      // (up to 16 token columns: the receive buffer of the split-K form takes the place of one ring stage)
      case 11: return depth == 2 ? launch_gemm_splitk<16, 2>(mp, mq, p, st)
                    : depth == 3 ? launch_gemm_splitk<16, 3>(mp, mq, p, st) : launch_gemm_splitk<16, 4>(mp, mq, p, st);
      case 12: return depth == 2 ? launch_gemm_splitk<32, 2>(mp, mq, p, st)
                    : depth == 3 ? launch_gemm_splitk<32, 3>(mp, mq, p, st) : launch_gemm_splitk<32, 4>(mp, mq, p, st);
      // 64 token columns: three stages, so that two CTAs share an SM (measured at the Qwen3-8B shapes against
      // the 8-stage ring with one CTA per SM: o 9.6 -> 8.4 us, down 13.7 -> 11.2 us, with the 8-way split that then fits)
      default: return depth == 8 ? launch_gemm_splitk<64, 8>(mp, mq, p, st) : launch_gemm_splitk<64, 3>(mp, mq, p, st);
    }
  }
  switch (cfg) {
    case 1: return launch_gemm<128, 6, 2, false>(mp, mq, p, di.sms, st);
    case 2: return launch_gemm<256, 4, 1, false>(mp, mq, p, di.sms, st);
    case 3: return launch_gemm<192, 4, 2, false>(mp, mq, p, di.sms, st);
    case 11: return depth == 2 ? launch_gemm<16, 2, 2, true>(mp, mq, p, di.sms, st)
                  : depth == 3 ? launch_gemm<16, 3, 2, true>(mp, mq, p, di.sms, st)
                               : launch_gemm<16, 5, 2, true>(mp, mq, p, di.sms, st);
    case 12: return depth == 2 ? launch_gemm<32, 2, 2, true>(mp, mq, p, di.sms, st)
                  : depth == 3 ? launch_gemm<32, 3, 2, true>(mp, mq, p, di.sms, st)
                               : launch_gemm<32, 4, 2, true>(mp, mq, p, di.sms, st);
    case 13: return depth == 8 ? launch_gemm<64, 8, 2, true>(mp, mq, p, di.sms, st)
                               : launch_gemm<64, 3, 2, true>(mp, mq, p, di.sms, st);
    case 14: return launch_gemm<128, 6, 2, true>(mp, mq, p, di.sms, st);
  }
  return FRT_E_UNSUPPORTED;
}

// [N, K/2] row-major -> [N/8][K/64][8][32 B]: one thread moves 16 bytes.
__global__ void repack_interleaved_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, int n, int kt) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;     // 16-byte piece of dst
  if (i >= static_cast<int64_t>(n) * kt * 2) return;
  const int half = static_cast<int>(i & 1);
  const int r8 = static_cast<int>((i >> 1) & 7);
  const int64_t rest = i >> 4;
  const int t = static_cast<int>(rest % kt);
  const int64_t grp = rest / kt;
  dst[i] = src[((grp * 8 + r8) * kt + t) * 2 + half];
}

}  // namespace frt

using namespace frt;

extern "C" {

#ifdef FRT_DEBUG
void frt_debug_set_trace(void* ptr) { g_trace = static_cast<long long*>(ptr); }
#endif

int frt_nvfp4_gemm_bf16(const void* a, const void* sfa, const void* b, const void* sfb, const void* bias,
                        const void* c, void* d, int M, int N, int K, float alpha, float beta, void* stream) {
  if (!a || !sfa || !b || !sfb || !d) return FRT_E_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0 || N % 8 != 0) return FRT_E_SHAPE;
  if (!aligned(a, 16) || !aligned(b, 16) || !aligned(d, 16) || !aligned(c, 16) || !aligned(bias, 16) ||
      !aligned(sfa, 16) || !aligned(sfb, 16))
    return FRT_E_ALIGN;
  if (beta != 0.f && c == nullptr) return FRT_E_NULL;
  const void* cc = beta != 0.f ? c : nullptr;
  const int cfg = g_opt_gemm_config;
  const bool swap = cfg ? cfg >= 11 : (M <= 64);
  if (swap) return run_gemm(b, sfb, N, a, sfa, M, K, bias, cc, d, N, alpha, beta, true, cfg, as_stream(stream));
  return run_gemm(a, sfa, M, b, sfb, N, K, bias, cc, d, N, alpha, beta, false, cfg, as_stream(stream));
}

int frt_nvfp4_repack_interleaved(const void* b_packed, void* b_interleaved, int N, int K, void* stream) {
  if (!b_packed || !b_interleaved) return FRT_E_NULL;
  if (N <= 0 || K <= 0 || N % 8 != 0 || K % 64 != 0) return FRT_E_SHAPE;
  if (!aligned(b_packed, 16) || !aligned(b_interleaved, 16)) return FRT_E_ALIGN;
  const int kt = K / 64;
  const int64_t pieces = static_cast<int64_t>(N) * kt * 2;
  repack_interleaved_kernel<<<static_cast<unsigned>((pieces + 255) / 256), 256, 0, as_stream(stream)>>>(
      static_cast<const uint4*>(b_packed), static_cast<uint4*>(b_interleaved), N, kt);
  return launch_result();
}

int frt_nvfp4_gemv_interleaved_bf16(const void* a, const void* sfa, const void* b_interleaved, const void* sfb,
                                    void* out, int N, int K, float alpha, void* stream) {
  if (!a || !sfa || !b_interleaved || !sfb || !out) return FRT_E_NULL;
  if (N <= 0 || K <= 0 || N % 8 != 0 || K % 64 != 0) return FRT_E_SHAPE;
  if (!aligned(a, 16) || !aligned(b_interleaved, 16) || !aligned(sfa, 16) || !aligned(sfb, 16)) return FRT_E_ALIGN;
  const int cfg = g_opt_gemm_config >= 11 && g_opt_gemm_config <= 13 ? g_opt_gemm_config : 0;
  return run_gemm(b_interleaved, sfb, N, a, sfa, 1, K, nullptr, nullptr, out, N, alpha, 0.f, true, cfg,
                  as_stream(stream), true);
}

int frt_nvfp4_gemm_plan(int M, int N, int K, int* config, int* split_k) {
  if (!config || !split_k) return FRT_E_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0 || N % 8 != 0) return FRT_E_SHAPE;
  const DeviceInfo di = device_info();
  const int sms = di.ok ? di.sms : 148;                 // no device (a build machine): the B200 count
  const int requested = g_opt_gemm_config;
  const bool swap = requested ? requested >= 11 : (M <= 64);
  if (swap) select_gemm_config(N, M, K, true, requested, sms, *config, *split_k);
  else select_gemm_config(M, N, K, false, requested, sms, *config, *split_k);
  return FRT_OK;
}

int frt_nvfp4_gemm_swiglu_nvfp4(const void* a, const void* sfa, const void* b, const void* sfb, void* out_packed,
                                void* out_sf, int M, int N2, int K, float alpha, void* stream) {
  if (!a || !sfa || !b || !sfb || !out_packed || !out_sf) return FRT_E_NULL;
  if (M <= 0 || N2 <= 0 || K <= 0 || K % 32 != 0 || N2 % 2 != 0) return FRT_E_SHAPE;
  if ((N2 / 2) % 128 != 0) return FRT_E_UNSUPPORTED;   // a tile is 128 gate + the 128 matching up columns
  if (!aligned(a, 16) || !aligned(b, 16) || !aligned(out_packed, 16) || !aligned(out_sf, 4) ||
      !aligned(sfa, 16) || !aligned(sfb, 16))
    return FRT_E_ALIGN;
  const DeviceInfo di = device_info();
  if (!di.ok || di.cc_major != 10) return FRT_E_DEVICE;
  GemmParams p{};
  p.P = M; p.Q = N2; p.K = K;
  p.k_tiles = (K + 63) / 64;
  p.sf_cols = p.k_tiles;
  p.sfp = static_cast<const uint8_t*>(sfa);
  p.sfq = static_cast<const uint8_t*>(sfb);
  p.sfq_row_blocks = (N2 + 127) / 128;
  p.alpha = alpha;
  p.group_m = 16;
  p.wait_limit = wait_limit_clocks();
#ifdef FRT_DEBUG
  p.dbg = g_opt_gemm_debug & 0xff;
  p.trace = g_trace;
#endif
  p.hidden = N2 / 2;
  p.out_packed = static_cast<uint8_t*>(out_packed);
  p.out_sf = static_cast<uint8_t*>(out_sf);
  return launch_gemm_swiglu(a, b, p, di.sms, as_stream(stream));
}

int frt_device_status(void* stream, unsigned* status_out) {
  if (!status_out) return FRT_E_NULL;
  unsigned* w = device_status_word();
  if (!w) return FRT_E_LAUNCH;
  cudaStream_t st = as_stream(stream);
  unsigned v = 0;
  if (cudaMemcpyAsync(&v, w, sizeof(v), cudaMemcpyDeviceToHost, st) != cudaSuccess) return FRT_E_LAUNCH;
  if (cudaStreamSynchronize(st) != cudaSuccess) return FRT_E_LAUNCH;
  *status_out = v;
  if (v != 0 && cudaMemsetAsync(w, 0, sizeof(v), st) != cudaSuccess) return FRT_E_LAUNCH;
  return FRT_OK;
}

}  // extern "C"
