// CTA-pair (tcgen05 cta_group::2) form of the NVFP4 GEMM for prefill shapes.
// Included by gemm.cu inside its unnamed namespace (shares GemmParams, the
// status word and the tile raster).
//
// Two CTAs on one TPC form a cluster and compute a 256 x BN output tile: CTA r
// owns rows [128 r, 128 r + 128) of the tile (its accumulator lives in its own
// TMEM) and stages only ITS half of the operands - 128 rows of P and BN/2 rows
// of Q per K stage - so every byte of P and Q crosses L2 -> shared memory once
// per pair instead of once per CTA, and the Q tile read by the tensor cores is
// gathered from both CTAs' shared memory.  Scale factors: each CTA stages the
// scales of its own P rows and of all BN Q rows.  No load is multicast.
//
//   warp 0   TMA producer of this CTA's half (tensor maps for operands AND scale
//            tiles); completion bytes of both CTAs are credited to the leader's
//            `full` barrier.
//   warp 1   leader CTA only: tcgen05.cp (scales smem -> TMEM, both CTAs) and
//            tcgen05.mma cta_group::2; tcgen05.commit multicast to both CTAs'
//            `empty` / `acc_full` barriers.
//   warps 2..9 epilogue of this CTA's 128 rows (TMEM -> registers -> swizzled staging in shared
//            memory -> TMA store); warps 2..17 in the SwiGLU form, whose epilogue computes
//            bf16(silu(gate) * up), quantises it to NVFP4 and stores packed bytes + scales.
//
// Forms (template parameters): dense bf16 output (the last, partial wave of tiles cut into column
// slices, see decode_unit), SWIGLU (gate/up tile pairs, NVFP4 output), GROUPED (one expert's weights
// on the M axis, a window of its token rows on the N axis, transposed bf16 output).
//
// TMEM (512 columns per CTA): two 128 x BN fp32 accumulators and one scale
// buffer.  For BN = 256 the accumulators overlap ([0,256) and [208,464), scales
// at [464,512)): the epilogue of tile t drains the shared columns first and
// releases them, so the mainloop of tile t+1 runs under the rest of the drain.
// The weight-major grouped form places an item's accumulator by its width: even
// tiles of a pair at [0, n), odd tiles at [448 - n, 448), scales at [448, 512).
#pragma once

struct PairMaps {
  CUtensorMap p, q, sfp, sfq;
  CUtensorMap q32;    // Q with a 32-row box (dense form: the narrow tiles of the last wave)
  CUtensorMap d;      // bf16 output [M, N], box 32 columns x 32 rows, 64-byte swizzle (dense form only)
};

// One unit of grouped work: a window of expert-sorted token rows that one
// expert's weights are applied to.  Built on the device by group_plan_kernel.
// Weight-major form: a window longer than 256 rows is contracted by two MMAs per K block against the same
// staged weights: rows [0, 256) and the rest (<= 64 rows), which is how an expert with a few rows more than
// one full window costs one pass over its weights instead of two.
struct GroupItem {
  int q_row0;      // first token row of the window (multiple of 64)
  int n_tokens;    // window length, multiple of 32, <= 320 (weight-major) 
  int lo, hi;      // token rows [lo, hi) of the window that belong to `expert`
  int expert;
  int pad[3];
};
struct GroupWork {
  int count;       // number of items
  int pad[3];
  GroupItem items[1];
};

// Dense form, last wave: when the tile count is not a multiple of the CTA-pair count, the tiles of
// the last (partial) wave are cut into 2 or 4 column slices so that every pair gets one; a work
// unit below `tail_first` is a whole tile, above it a slice of width 256 / tail_split.
__device__ __forceinline__ void decode_unit(int u, const GemmParams& p, int& pt, int& qt, int& col0, int& width) {
  int t = u;
  col0 = 0;
  width = 256;
  if (u >= p.tail_first) {
    const int v = u - p.tail_first;
    t = p.tail_first + v / p.tail_split;
    width = 256 / p.tail_split;
    col0 = (v % p.tail_split) * width;
  }
  tile_coords(t, p, pt, qt);
}

// Weight-major windows of one expert's rows [lo, hi): the first starts on the 64-row boundary below lo, every
// window but the last is 256 rows, and the last takes what is left when that is at most 320 rows.
__host__ __device__ __forceinline__ int grouped_window_rows(int start, int hi) {
  const int rem = hi - start;
  return rem <= 320 ? (rem + 31) & ~31 : 256;
}
__host__ __device__ __forceinline__ int grouped_window_count(int lo, int hi) {
  if (hi <= lo) return 0;
  const int span = hi - (lo & ~63);
  return span <= 320 ? 1 : 1 + (span - 320 + 255) / 256;
}

template <int BN, int STAGES, bool GROUPED = false, bool TM = false>
struct PairLayout {

  static constexpr int A_BYTES = 128 * 128;              // this CTA's 128 rows of P
  static constexpr int B_MAIN = (BN / 2) * 128;          // this CTA's half of the Q tile
  // weight-major grouped form: one more 32-row box for this CTA's half of the rows beyond 256
  static constexpr int B_BYTES = B_MAIN + ((GROUPED && !TM) ? 4096 : 0);
  // 128-row scale groups a Q tile can touch (a grouped window starts at any multiple of 64)
  static constexpr int SFQ_BLOCKS = (GROUPED && !TM) ? 3 : (BN <= 128 ? 1 : 2);
  static constexpr int SFP_BYTES = KT_PER_STAGE * SF_TILE;
  static constexpr int SFQ_BYTES = SFQ_BLOCKS * KT_PER_STAGE * SF_TILE;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFP_BYTES + SFQ_BYTES;
  // epilogue staging: 4 warps x 4 buffers of 32 rows x 64 bytes, written by TMA store
  // store staging: two buffers of 32 rows x 64 B per epilogue warp (8 warps stage stores)
  static constexpr int SBUFS = 2;
  static constexpr int STAGING_BYTES = 8 * SBUFS * 2048;
  static constexpr int ITEM_CACHE = GROUPED ? 96 : 0;    // this pair's first work items, copied to smem
  // weight-major grouped form with per-expert offsets: every CTA builds the window list itself (prefix of the
  // experts' window counts), so a call is one launch
  static constexpr int PLAN_EXPERTS = 256;
  static constexpr int PLAN_BYTES = (GROUPED && !TM) ? (PLAN_EXPERTS + 4) * 4 : 0;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + STAGING_BYTES + ITEM_CACHE * 32 + PLAN_BYTES + 1024 + 256;
  static constexpr int SF_COLS = KT_PER_STAGE * (4 + SFQ_BLOCKS * 4);
  // accumulator placement: disjoint when they fit, else overlapping by OVERLAP columns
  static constexpr int ACC1 = (2 * BN + SF_COLS <= 512) ? BN : 512 - SF_COLS - BN;
  static constexpr int OVERLAP = BN - ACC1;              // 0 when disjoint
  static constexpr int SF_BASE = ACC1 + BN;
  // weight-major grouped form: an item's accumulator is n_tokens columns wide; even tiles of a pair grow up
  // from column 0, odd tiles down from ACC_COLS, and what two consecutive tiles share is drained first
  static constexpr int ACC_COLS = SF_BASE;
  static_assert(SF_BASE + SF_COLS <= 512, "TMEM budget");
  static_assert(BN % 32 == 0 && OVERLAP >= 0, "tile shape");
};

// GROUPED: P = one expert's weights (3-D / 4-D tensor maps with the expert as the
// outer coordinate), Q = a window of up to 320 token rows (two MMAs per K block when it is
// longer than 256: the staged weights serve both); the output tile is written
// transposed (out[token, weight_row]) and masked to the rows of that expert.  The
// epilogue reads the accumulator as 8 x 8 block fragments (tcgen05.ld 16x256b), which
// stmatrix stores transposed into the staging buffer a TMA store (whole chunks) or
// per-row 16-byte stores (the expert's first and last rows) write out.  Measured on the
// Qwen3-30B-A3B layer: a stage is bound by what an SM takes in from L2 (~43 KB per
// CTA and K stage at ~57 B/clk); prefetching the next tile's weights into L2 changed nothing.
//
// GROUPED + TM (token-major): P = two 128-row blocks of token rows (one per CTA; blocks are aligned to the
// 128-row groups of the scale layout, so an expert's first and last block may be shared with its neighbours and
// are masked row by row in the epilogue), Q = 256 output columns of that expert's weights.  The output tile is
// row-major like the dense form's: TMA stores where a warp's 32 rows all belong to the expert, masked 16-byte
// stores at its edges.  No transpose: this is the form for experts with many rows, where the transposing
// epilogue of the weight-major form costs more than the mainloop (K = 768: three stages per tile).
//
// SWIGLU (BN = 256, dense): Q = [gate ; up] weights stacked along N (2H rows).  A tile is 128
// gate columns and the 128 matching up columns: CTA 0 stages gate rows [128 qt, +128), CTA 1
// up rows [H + 128 qt, +128), so accumulator columns [0,128) are gate and [128,256) up for the
// same 128 outputs.  The epilogue rounds both to bf16 (what a bf16 GEMM would have written),
// evaluates bf16(silu(g) * u) and rule-A quantises it: each lane owns one output row and
// whole 16-element blocks, and writes 16 packed bytes + 2 scale bytes per 32 outputs.  The
// 2H-wide bf16 intermediate never exists in memory.
// The SwiGLU form runs 16 epilogue warps (one lane quarter x one group of 32 outputs each):
// its epilogue is an exponential and a division per output, and only that many warps issue
// it in less time than the tile's mainloop takes.
template <int BN, int STAGES, bool GROUPED_ANY, bool SWIGLU = false, bool TM = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(SWIGLU ? 576 : 320, 1)
nvfp4_gemm_pair_kernel(const __grid_constant__ PairMaps maps, const GemmParams p,
                       const GroupWork* __restrict__ work) {
  using L = PairLayout<BN, STAGES, GROUPED_ANY, TM>;
  constexpr bool GROUPED = GROUPED_ANY && !TM;     // the weight-major (transposed-output) grouped form
  static_assert(!TM || GROUPED_ANY, "token-major is a grouped form");
  static_assert(!SWIGLU || (BN == 256 && !GROUPED_ANY), "the SwiGLU epilogue is a 256-wide dense tile");
  constexpr int SFQ_COLS_PER_KT = L::SFQ_BLOCKS * 4;
  constexpr uint32_t IDESC = ptx::idesc_nvf4(256, BN);
  constexpr int CHUNKS = BN / 32;
  constexpr int RELEASE_CHUNKS = (L::OVERLAP + 31) / 32;   // chunks that cover the shared columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* staging = smem + STAGES * L::STAGE_BYTES;
  GroupItem* item_cache = reinterpret_cast<GroupItem*>(staging + L::STAGING_BYTES);
  int* win_pre = reinterpret_cast<int*>(staging + L::STAGING_BYTES + L::ITEM_CACHE * 32);   // [experts + 1] windows before expert e
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + L::STAGING_BYTES + L::ITEM_CACHE * 32 + L::PLAN_BYTES);
  uint64_t* full = bars;                    // [STAGES] used in the leader: both CTAs' TMA bytes
  uint64_t* empty = bars + STAGES;          // [STAGES] in each CTA: multicast commit from the leader
  uint64_t* acc_full = bars + 2 * STAGES;   // [2] in each CTA: multicast commit from the leader
  uint64_t* acc_free = acc_full + 2;        // [1] used in the leader: 16 epilogue warps of the pair
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = ptx::cluster_ctarank();
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  pdl_launch_dependents();
  // work units: grouped: read from the plan after the wait below; dense: tiles, the last wave sliced
  int total_tiles = GROUPED_ANY ? 0 : (SWIGLU || BN != 256) ? p.p_tiles * p.q_tiles : p.units;
  constexpr bool SLICED = !GROUPED_ANY && !SWIGLU && BN == 256;
  const int per_item = TM ? p.q_tiles : p.p_tiles;          // tiles of one grouped work item
  const int k_stages = (p.k_tiles + KT_PER_STAGE - 1) / KT_PER_STAGE;

  if (threadIdx.x == 0) {
    for (int i = 0; i < STAGES; ++i) { ptx::mbar_init(&full[i], 1); ptx::mbar_init(&empty[i], 1); }
    ptx::mbar_init(&acc_full[0], 1);
    ptx::mbar_init(&acc_full[1], 1);
    ptx::mbar_init(acc_free, SWIGLU ? 32 : 16);   // epilogue warps of the pair
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&maps.p);
    ptx::prefetch_tensormap(&maps.q);
    ptx::prefetch_tensormap(&maps.sfp);
    ptx::prefetch_tensormap(&maps.sfq);
    if (!SWIGLU) ptx::prefetch_tensormap(&maps.d);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(tmem_slot, 512);
    ptx::tmem_relinquish_pair();
  }
  pdl_wait();                 // everything above overlapped the previous kernel; global memory from here on
  // item j of the inline plan: the expert whose windows contain j (binary search in the prefix), then the window
  auto make_item = [&](int j) {
    int e0 = 0, e1 = p.num_experts;               // win_pre[e0] <= j < win_pre[e1]
    while (e1 - e0 > 1) {
      const int mid = (e0 + e1) >> 1;
      if (win_pre[mid] <= j) e0 = mid; else e1 = mid;
    }
    const int lo = max(0, min(p.inline_offsets[e0], p.Q)), hi = max(0, min(p.inline_offsets[e0 + 1], p.Q));
    const int start = (lo & ~63) + 256 * (j - win_pre[e0]);
    GroupItem it{};
    it.q_row0 = start; it.n_tokens = grouped_window_rows(start, hi);
    it.lo = max(lo, start); it.hi = min(hi, start + it.n_tokens);
    it.expert = e0;
    return it;
  };
  const bool inline_plan = GROUPED && p.inline_offsets != nullptr;
  if (inline_plan) {
    // windows per expert, then their exclusive prefix (one warp, consecutive experts per lane)
    for (int e = threadIdx.x; e < p.num_experts; e += blockDim.x)
      win_pre[e + 1] = grouped_window_count(max(0, min(p.inline_offsets[e], p.Q)), max(0, min(p.inline_offsets[e + 1], p.Q)));
    if (threadIdx.x == 0) win_pre[0] = 0;
    __syncthreads();
    if (warp == 0) {
      const int per = (p.num_experts + 31) / 32, first = lane * per;
      int sum = 0;
      for (int i = 0; i < per; ++i) sum += first + i < p.num_experts ? win_pre[first + i + 1] : 0;
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
      }
      int run = incl - sum;                        // windows before this lane's experts
      for (int i = 0; i < per; ++i) {
        if (first + i < p.num_experts) {
          run += win_pre[first + i + 1];
          win_pre[first + i + 1] = run;
        }
      }
    }
    __syncthreads();
    int items = win_pre[p.num_experts];
    if (items > p.max_items) {                     // offsets that claim more rows than exist: cut short, and say so
      if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(&g_status_word, 0x200u);
      items = p.max_items;
    }
    total_tiles = items * per_item;
    for (int i = threadIdx.x; i < L::ITEM_CACHE; i += blockDim.x) {
      const int t = pair_id + i * num_pairs;
      if (t < total_tiles) item_cache[i] = make_item(t / per_item);
    }
  } else if (GROUPED_ANY) {
    total_tiles = min(work->count, p.max_items) * per_item;   // the plan never stores beyond max_items
    // tile i of this pair is global tile pair_id + i * num_pairs; its item is items[tile / per_item]
    for (int i = threadIdx.x; i < L::ITEM_CACHE; i += blockDim.x) {
      const int t = pair_id + i * num_pairs;
      if (t < total_tiles) item_cache[i] = work->items[t / per_item];
    }
  }
  // an item beyond the cached ones (weight-major form)
  auto far_item = [&](int t) { return inline_plan ? make_item(t / p.p_tiles) : work->items[t / p.p_tiles]; };
  ptx::tc_fence_before();
  __syncthreads();
  // both CTAs' barriers must be initialised before either signals the other
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ===================== TMA producer (both CTAs) =====================
    if (ptx::elect_one()) {
      const uint32_t smem0 = ptx::smem_u32(smem);
      const uint32_t full0 = ptx::smem_u32(full) & 0xFEFFFFFFu;   // the leader CTA's barrier array
      int s = 0, it = 0;
      uint32_t ph = 0;
      int ti = 0;
      for (int t = pair_id; t < total_tiles && !*abort_flag; t += num_pairs, ++ti) {
        int pt, qt, q_row, q_blk, expert = 0;
        int nq = 0, nsf = 0;       // grouped: 32-row Q boxes per CTA, 128-row scale groups the window touches
        int q_row2 = -1;           // grouped: this CTA's first row of the window's rows beyond 256 (-1: none)
        int tm_p_row = 0;
        if (TM) {
          const GroupItem item = ti < L::ITEM_CACHE ? item_cache[ti] : work->items[t / per_item];
          qt = t % per_item;
          const int blk = (rank && item.n_tokens >= 0) ? item.n_tokens : item.q_row0;   // this CTA's 128-row block
          tm_p_row = blk * 128;
          q_row = qt * BN + static_cast<int>(rank) * (BN / 2);
          q_blk = (qt * BN) >> 7;
          expert = item.expert;
          pt = 0;
        } else if (GROUPED) {
          const GroupItem item = ti < L::ITEM_CACHE ? item_cache[ti] : far_item(t);
          pt = t % p.p_tiles;
          const int main_n = min(item.n_tokens, 256), extra_n = item.n_tokens - main_n;
          q_row = item.q_row0 + static_cast<int>(rank) * (main_n >> 1);
          q_blk = item.q_row0 >> 7;
          expert = item.expert;
          nq = ((main_n >> 1) + 31) >> 5;
          nsf = ((item.q_row0 + item.n_tokens - 1) >> 7) - q_blk + 1;
          q_row2 = extra_n ? item.q_row0 + 256 + static_cast<int>(rank) * (extra_n >> 1) : -1;
        } else if (SLICED) {
          int col0, width;
          decode_unit(t, p, pt, qt, col0, width);
          q_row = qt * BN + col0 + static_cast<int>(rank) * (width >> 1);
          q_blk = (qt * BN + col0) >> 7;
          nq = width == 256 ? 0 : width >> 6;       // 32-row boxes per CTA of a slice; 0 = one 128-row box
        } else {
          tile_coords(t, p, pt, qt);
          if (SWIGLU) {
            q_row = qt * 128 + static_cast<int>(rank) * p.hidden;
            q_blk = qt;
          } else {
            q_row = qt * BN + static_cast<int>(rank) * (BN / 2);
            q_blk = (qt * BN) >> 7;
          }
        }
        const int p_row = TM ? tm_p_row : pt * 256 + static_cast<int>(rank) * 128;
        const int p_blk = p_row >> 7;
        for (int ks = 0; ks < k_stages; ++ks, ++it) {
          if (!ptx::mbar_wait_bounded(&empty[s], ph ^ 1, WAIT_LIMIT)) {
            atomicOr(&g_status_word, 1u); *abort_flag = 1; break;
          }
          const uint32_t st = smem0 + s * L::STAGE_BYTES;
          const uint32_t bar = full0 + s * 8;
          if (TM) {
            // tokens and their scales through the plain 2-D / 3-D maps, the expert's weights and weight scales
            // through the stacked maps (expert = outer coordinate); boxes past the tensors' ends are zero-filled
            if (leader) ptx::mbar_expect_tx(&full[s], 2 * L::STAGE_BYTES);
            ptx::tma_load_2d_pair(st, &maps.p, bar, ks * 128, p_row);
            ptx::tma_load_3d_pair(st + L::A_BYTES + L::B_BYTES, &maps.sfp, bar, 0, ks * KT_PER_STAGE, p_blk);
            ptx::tma_load_3d_pair(st + L::A_BYTES, &maps.q, bar, ks * 128, q_row, expert);
            ptx::tma_load_4d_pair(st + L::A_BYTES + L::B_BYTES + L::SFP_BYTES, &maps.sfq, bar, 0, ks * KT_PER_STAGE,
                                  q_blk, expert);
            if (++s == STAGES) { s = 0; ph ^= 1u; }
            continue;
          }
          if (GROUPED) {
            // the token window is loaded at its size: 32-row boxes of Q and only the scale groups it touches
            if (leader)
              ptx::mbar_expect_tx(&full[s], 2 * (L::A_BYTES + L::SFP_BYTES + (nq + (q_row2 >= 0 ? 1 : 0)) * 4096 +
                                                 nsf * KT_PER_STAGE * SF_TILE));
            ptx::tma_load_3d_pair(st, &maps.p, bar, ks * 128, p_row, expert);
            ptx::tma_load_4d_pair(st + L::A_BYTES + L::B_BYTES, &maps.sfp, bar, 0, ks * KT_PER_STAGE, p_blk, expert);
            for (int i = 0; i < nq; ++i)
              ptx::tma_load_2d_pair(st + L::A_BYTES + i * 4096, &maps.q, bar, ks * 128, q_row + 32 * i);
            if (q_row2 >= 0) ptx::tma_load_2d_pair(st + L::A_BYTES + L::B_MAIN, &maps.q, bar, ks * 128, q_row2);
            for (int b = 0; b < nsf; ++b)
              ptx::tma_load_3d_pair(st + L::A_BYTES + L::B_BYTES + L::SFP_BYTES + b * KT_PER_STAGE * SF_TILE, &maps.sfq,
                                    bar, 0, ks * KT_PER_STAGE, q_blk + b);
            if (++s == STAGES) { s = 0; ph ^= 1u; }
            continue;
          }
          if (leader) ptx::mbar_expect_tx(&full[s], 2 * (L::STAGE_BYTES - (nq ? L::B_BYTES - nq * 4096 : 0)));
          {
            ptx::tma_load_2d_pair(st, &maps.p, bar, ks * 128, p_row);
            ptx::tma_load_3d_pair(st + L::A_BYTES + L::B_BYTES, &maps.sfp, bar, 0, ks * KT_PER_STAGE, p_blk);
          }
          if (SLICED && nq) {
            for (int i = 0; i < nq; ++i)
              ptx::tma_load_2d_pair(st + L::A_BYTES + i * 4096, &maps.q32, bar, ks * 128, q_row + 32 * i);
          } else {
            ptx::tma_load_2d_pair(st + L::A_BYTES, &maps.q, bar, ks * 128, q_row);
          }
          ptx::tma_load_3d_pair(st + L::A_BYTES + L::B_BYTES + L::SFP_BYTES, &maps.sfq, bar, 0, ks * KT_PER_STAGE,
                                q_blk);
          if (SWIGLU)   // the map's box is one 128-row group: gate scales above, up scales here
            ptx::tma_load_3d_pair(st + L::A_BYTES + L::B_BYTES + L::SFP_BYTES + KT_PER_STAGE * SF_TILE, &maps.sfq, bar,
                                  0, ks * KT_PER_STAGE, (p.hidden >> 7) + q_blk);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
      }
      if (!*abort_flag) {   // drain: every armed stage has been consumed before this CTA may exit
        for (int i = 0; i < STAGES && i < it; ++i) {
          const int j = it - 1 - i;
          if (!ptx::mbar_wait_bounded(&empty[j % STAGES], (j / STAGES) & 1, WAIT_LIMIT)) {
            atomicOr(&g_status_word, 2u); break;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer (leader CTA) =====================
    if (leader && ptx::elect_one()) {
      const uint32_t smem0 = ptx::smem_u32(smem);
      const uint64_t op_desc = ptx::desc_sw128_kmajor(smem0);
      const uint64_t sf_desc = ptx::desc_sf_32x16(smem0 + L::A_BYTES + L::B_BYTES);
      const uint32_t op_hi = static_cast<uint32_t>(op_desc >> 32), op_lo0 = static_cast<uint32_t>(op_desc);
      const uint32_t sf_hi = static_cast<uint32_t>(sf_desc >> 32), sf_lo0 = static_cast<uint32_t>(sf_desc);
      const uint32_t sf_tmem = tmem_base + L::SF_BASE;
      int s = 0, tl = 0;
      uint32_t ph = 0;
      bool aborted = false;
      for (int t = pair_id; t < total_tiles && !*abort_flag; t += num_pairs, ++tl) {
        const int a = tl & 1;
        // tile tl may start once the epilogues of tile tl-1 have drained the columns the two
        // accumulators share (which also means tile tl-2, same accumulator, is fully drained)
        const bool tr = FRT_TRACING(p) && pair_id == 0 && tl < 32;
        if (tr) FRT_TRACE(p, tl * 8 + 0);
        if (tl > 0 && !ptx::mbar_wait_bounded(acc_free, (tl - 1) & 1, WAIT_LIMIT)) {
          atomicOr(&g_status_word, 4u); *abort_flag = 1; break;
        }
        ptx::tc_fence_after();
        if (tr) FRT_TRACE(p, tl * 8 + 1);
        uint32_t d_tmem = tmem_base + (a ? L::ACC1 : 0);
        uint32_t qoff, idesc = IDESC, idesc2 = 0;          // idesc2: the MMA over a grouped window's rows beyond 256
        if (TM) {
          qoff = (static_cast<uint32_t>((t % per_item) * BN) & 127u) >> 5;
        } else if (GROUPED) {
          const GroupItem item = tl < L::ITEM_CACHE ? item_cache[tl] : far_item(t);
          qoff = (static_cast<uint32_t>(item.q_row0) & 127u) >> 5;
          const int main_n = min(item.n_tokens, 256);
          idesc = ptx::idesc_nvf4(256, main_n);
          if (item.n_tokens > 256) idesc2 = ptx::idesc_nvf4(256, item.n_tokens - 256);
          d_tmem = tmem_base + (a ? L::ACC_COLS - item.n_tokens : 0);
        } else if (SLICED) {
          int pt, qt, col0, width;
          decode_unit(t, p, pt, qt, col0, width);
          qoff = (static_cast<uint32_t>(qt * BN + col0) & 127u) >> 5;
          if (width != 256) idesc = ptx::idesc_nvf4(256, width);
        } else {
          int pt, qt;
          tile_coords(t, p, pt, qt);
          qoff = SWIGLU ? 0u : (static_cast<uint32_t>(qt * BN) & 127u) >> 5;
        }
        for (int ks = 0; ks < k_stages; ++ks) {
          if (!ptx::mbar_wait_bounded(&full[s], ph, WAIT_LIMIT)) {
            atomicOr(&g_status_word, 8u); *abort_flag = 1; aborted = true; break;
          }
          ptx::tc_fence_after();
          const uint32_t a_lo = op_lo0 + s * (L::STAGE_BYTES >> 4);
          const uint32_t b_lo = a_lo + (L::A_BYTES >> 4);
          const uint32_t sfp_lo = sf_lo0 + s * (L::STAGE_BYTES >> 4);
          const uint32_t sfq_lo = sfp_lo + (L::SFP_BYTES >> 4);
          const int kts = min(KT_PER_STAGE, p.k_tiles - ks * KT_PER_STAGE);
#pragma unroll
          for (int kt = 0; kt < KT_PER_STAGE; ++kt) {
            if (kt < kts) {
              const uint32_t sfp_t = sf_tmem + kt * 4;
              const uint32_t sfq_t = sf_tmem + KT_PER_STAGE * 4 + kt * SFQ_COLS_PER_KT;
              if (!FRT_DBG(p, 2) || (tl == 0 && ks == 0)) {
                ptx::tc_cp_32x128b_warpx4_pair(sfp_t, sfp_lo + kt * (SF_TILE >> 4), sf_hi);
#pragma unroll
                for (int b = 0; b < L::SFQ_BLOCKS; ++b)
                  ptx::tc_cp_32x128b_warpx4_pair(sfq_t + 4 * b, sfq_lo + (b * KT_PER_STAGE + kt) * (SF_TILE >> 4),
                                                 sf_hi);
              }
              ptx::tc_mma_nvf4_pair(d_tmem, a_lo + 2 * kt, b_lo + 2 * kt, op_hi, idesc, sfp_t, sfq_t + qoff,
                                    (ks | kt) != 0);
              if (GROUPED && idesc2)     // same weights, the window's rows beyond 256: columns after the first 256
                ptx::tc_mma_nvf4_pair(d_tmem + 256, a_lo + 2 * kt, b_lo + (L::B_MAIN >> 4) + 2 * kt, op_hi, idesc2, sfp_t,
                                      sfq_t + qoff + 8, (ks | kt) != 0);
            }
          }
          ptx::tc_commit_pair(&empty[s], 3);
          if (++s == STAGES) { s = 0; ph ^= 1u; }
        }
        if (aborted) break;
        ptx::tc_commit_pair(&acc_full[a], 3);
        if (tr) FRT_TRACE(p, tl * 8 + 2);
      }
    }
  } else {
    // ===================== epilogue (warps 2..9, both CTAs) =====================
    // Eight warps: warp e covers TMEM lane quarter e & 3 and one half of the tile's
    // 32-column chunks.  Chunks are drained in an order that reaches the columns the two
    // accumulators share first (descending for accumulator 0, ascending for 1); the four
    // warps that own that first half release the shared columns as soon as they are in
    // registers, the other four when they start the tile.  TMEM loads run one chunk ahead of
    // the arithmetic.
    const int ew = warp - 2;
    const int quarter = warp & 3;          // a warp reaches only the TMEM lanes of sub-partition warp_id % 4
    const int half = ew >> 2;                                            // which share of the chunks (0 .. PARTS-1)
    // 8 epilogue warps split the chunks in two shares (16 in the SwiGLU form, which has its own loop below;
    // 16 warps were tried for the grouped form too: 6 % faster at K = 768, 4 % slower at K = 2048)
    constexpr int PARTS = SWIGLU ? 4 : 2;
    constexpr int NCH = CHUNKS / PARTS;                                  // chunks per warp
    constexpr int WARP_BUFS = L::SBUFS;                                  // staging buffers per warp
    static_assert(CHUNKS % PARTS == 0 && RELEASE_CHUNKS <= NCH, "chunk split");
    const uint32_t free_addr = ptx::mapa(ptx::smem_u32(acc_free), 0);   // the leader's barrier
    const uint32_t stage_base = ptx::smem_u32(staging) + ew * (WARP_BUFS * 2048);
    const int row_in_tile = static_cast<int>(rank) * 128 + quarter * 32;
    uint32_t nstore = 0;                  // TMA stores issued by this warp (2 staging buffers)
    int tl = 0;
    for (int t = pair_id; t < total_tiles && !*abort_flag; t += num_pairs, ++tl) {
      int pt, qt = 0, col0 = 0, width = BN;
      GroupItem item{};
      float alpha = p.alpha;
      int tm_row0 = 0;                      // TM: first token row of this warp's 32 TMEM lanes
      bool tm_any = false, tm_all = false;  // TM: some / all of those rows belong to the item's expert
      if (TM) {
        item = tl < L::ITEM_CACHE ? item_cache[tl] : work->items[t / per_item];
        qt = t % per_item;
        pt = 0;
        alpha = p.alpha_stack[item.expert];
        const int blk = rank ? item.n_tokens : item.q_row0;      // CTA 1 of an odd last block: nothing to write
        tm_row0 = blk * 128 + quarter * 32;
        tm_any = blk >= 0 && tm_row0 < item.hi && tm_row0 + 32 > item.lo;
        tm_all = blk >= 0 && tm_row0 >= item.lo && tm_row0 + 32 <= item.hi;
      } else if (GROUPED) {
        item = tl < L::ITEM_CACHE ? item_cache[tl] : far_item(t);
        pt = t % p.p_tiles;
        alpha = p.alpha_stack[item.expert];
      } else if (SLICED) {
        decode_unit(t, p, pt, qt, col0, width);
      } else {
        tile_coords(t, p, pt, qt);
      }
      const int a = tl & 1;
      if (!ptx::mbar_wait_bounded(&acc_full[a], (tl >> 1) & 1, WAIT_LIMIT)) {
        if (lane == 0) { atomicOr(&g_status_word, 16u); *abort_flag = 1; }
        break;
      }
      ptx::tc_fence_after();
      const int drain_rank = a ? half : PARTS - 1 - half;   // this warp owns drain positions [rank * NCH, +NCH)
      const bool first_half = drain_rank == 0;              // ... the first of which are the shared columns
      const bool tr = FRT_TRACING(p) && pair_id == 0 && tl < 32 && leader && quarter == 0 && lane == 0;
      if (tr) FRT_TRACE(p, tl * 8 + (first_half ? 3 : 6));
      const int prow = TM ? tm_row0 + lane : pt * 256 + row_in_tile + lane;   // dense / TM: output row; grouped: output column
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + (a ? L::ACC1 : 0);
      auto chunk_of = [&](int j) {                          // j-th chunk of this warp -> column chunk
        const int pos = drain_rank * NCH + j;
        return a ? pos : CHUNKS - 1 - pos;
      };
      auto chunk_live = [&](int cchunk) {                   // warp-uniform: anything to write?
        if (TM) return tm_any && qt * BN + cchunk * 32 < p.Q;
        return cchunk * 32 < width && qt * BN + col0 + cchunk * 32 < p.Q;
      };
      auto release = [&]() {
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (leader) ptx::mbar_arrive(acc_free); else ptx::mbar_arrive_cluster(free_addr);
        }
      };
      if constexpr (SWIGLU) {
        // This warp's group of 32 outputs: gate chunk c, up chunk 4 + c.  The accumulators share
        // the up chunks 2, 3 of accumulator 0 and the gate chunks 0, 1 of accumulator 1: the
        // warps that read those release after their loads, the others when they start the tile.
        const int c = ew >> 2;
        const bool owner = a ? c < 2 : c >= 2;
        uint32_t rg[32], ru[32];
        if (!owner) release();
        ptx::tc_ld_32x32b_x32(taddr + c * 32, rg);
        ptx::tc_ld_32x32b_x32(taddr + (4 + c) * 32, ru);
        ptx::tc_wait_ld(rg);
        ptx::tc_wait_ld(ru);
        if (owner) release();
        if (tr && first_half) FRT_TRACE(p, tl * 8 + 4);
        const float* inv_table = inv_scale_table();
        uint32_t pk[4];
        uint32_t sfw = 0;
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float g = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rg[16 * b + j]) * alpha));
            const float u = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ru[16 * b + j]) * alpha));
            v[j] = swiglu_bf16(g, u);
          }
          uint8_t sfb;
          const uint2 o = quantize_block16<kEncHw>(v, sfb, inv_table);
          pk[2 * b] = o.x;
          pk[2 * b + 1] = o.y;
          sfw |= static_cast<uint32_t>(sfb) << (8 * b);
        }
        if (prow < p.P && !FRT_DBG(p, 1)) {
          const int col = qt * 128 + 32 * c;                 // first of the 32 output columns
          uint8_t* dst = p.out_packed + static_cast<int64_t>(prow) * (p.hidden >> 1) + (col >> 1);
          *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          *reinterpret_cast<uint16_t*>(p.out_sf + sf_offset(prow, col >> 4, p.hidden >> 6)) =
              static_cast<uint16_t>(sfw);
        }
        if (tr) FRT_TRACE(p, tl * 8 + (first_half ? 5 : 7));
        continue;
      }
      if constexpr (GROUPED) {
        // The item's accumulator is n_tokens columns: [0, n) for even tiles of this pair, [ACC_COLS - n, ACC_COLS)
        // for odd ones, so consecutive tiles share max(0, n + n_next - ACC_COLS) columns: the top chunks of an
        // even tile, the bottom chunks of an odd one.  Chunks are drained from the shared end; the two groups of
        // four warps take alternate drain positions, so the shared chunks are split between them, and a warp
        // arrives on acc_free once its shared chunks are in registers (two register buffers: immediately after
        // the prologue loads when it owns at most two of them).
        const int nch = item.n_tokens >> 5;
        int shared = 0;
        if (t + num_pairs < total_tiles) {
          const int n_next = (tl + 1 < L::ITEM_CACHE ? item_cache[tl + 1] : far_item(t + num_pairs)).n_tokens;
          shared = max(0, (item.n_tokens + n_next - L::ACC_COLS) >> 5);
        }
        const int my_n = (nch - half + 1) >> 1;                       // drain positions half, half + 2, ...
        const int my_shared = shared > half ? (shared - half + 1) >> 1 : 0;
        const uint32_t gaddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) +
                               (a ? L::ACC_COLS - item.n_tokens : 0);
        auto chunk_at = [&](int j) { const int pos = half + 2 * j; return a ? pos : nch - 1 - pos; };
        auto live_at = [&](int j) {                                   // warp-uniform: anything to write?
          if (j >= my_n) return false;
          const int tok0 = item.q_row0 + chunk_at(j) * 32;
          return tok0 < item.hi && tok0 + 32 > item.lo;
        };
        const int n0 = pt * 256 + row_in_tile;                        // first output column of this warp
        uint32_t r[2][32];
        if (my_shared == 0) release();
        // a chunk (this warp's 32 weight rows x 32 tokens) is loaded as 8 x 8 block fragments: registers
        // [0,16) lanes 0..15, [16,32) lanes 16..31 of the warp's quarter
        auto load_chunk = [&](int j, uint32_t (&dst)[32]) {
          const uint32_t ad = gaddr + chunk_at(j) * 32;
          ptx::tc_ld_16x256b_x4<0>(ad, dst);
          ptx::tc_ld_16x256b_x4<16>(ad + (16u << 16), dst);
        };
        if (live_at(0)) load_chunk(0, r[0]);
        if (live_at(1)) load_chunk(1, r[1]);
        ptx::tc_wait_ld(r[0]);
        ptx::tc_wait_ld(r[1]);
        if (my_shared == 1 || my_shared == 2) release();
        if (tr && first_half) FRT_TRACE(p, tl * 8 + 4);
        constexpr int MAX_MINE = 5;                                   // a warp's share of an item's <= 10 chunks
#pragma unroll
        for (int j = 0; j < MAX_MINE; ++j) {
          if (j < my_n) {
            if (j >= 2) ptx::tc_wait_ld(r[j & 1]);
            if (my_shared > 2 && j == my_shared - 1) release();
            if (live_at(j)) {
              const uint32_t (&v32)[32] = r[j & 1];
              const int tok0 = item.q_row0 + chunk_at(j) * 32;
              const uint32_t buf = stage_base + (nstore % WARP_BUFS) * 2048u;
              if (nstore >= WARP_BUFS) {                     // the TMA store that last read this buffer is done
                if (lane == 0) ptx::bulk_wait_group_read<WARP_BUFS - 1>();
                __syncwarp();
              }
              // transpose through shared memory: [token][weight row], 64 bytes per token, 64-byte TMA swizzle.
              // One stmatrix per 8 tokens: its four blocks are the four groups of 8 weight rows, stored
              // transposed (thread 8m + i addresses token 8q + i, 16-byte piece m of the row).
              const uint32_t piece = static_cast<uint32_t>(lane) >> 3;
#pragma unroll
              for (uint32_t q = 0; q < 4; ++q) {
                const uint32_t token = 8u * q + (static_cast<uint32_t>(lane) & 7u);
                auto pk = [&](int i) { return pack_bf16x2(__uint_as_float(v32[i]) * alpha, __uint_as_float(v32[i + 1]) * alpha); };
                ptx::stmatrix_x4_trans(buf + token * 64u + ((piece ^ ((token >> 1) & 3u)) * 16u), pk(4 * q), pk(4 * q + 2),
                                       pk(16 + 4 * q), pk(16 + 4 * q + 2));
              }
              if (tok0 >= item.lo && tok0 + 32 <= item.hi) {
                // all 32 token rows belong to the expert: TMA writes (and clips) the box
                ptx::fence_proxy_async();
                __syncwarp();
                if (lane == 0) {
                  if (!FRT_DBG(p, 1)) ptx::tma_store_2d(&maps.d, buf, n0, tok0);
                  ptx::bulk_commit_group();
                }
                ++nstore;
              } else {
                // an edge of the expert's rows: each lane writes the 64 bytes of one token row, if the row is
                // the expert's (rows are 16-byte aligned: the output map of the TMA path demands the same)
                __syncwarp();
                const int tok = tok0 + lane;
                if (tok >= item.lo && tok < item.hi && !FRT_DBG(p, 1)) {
                  __nv_bfloat16* dst = p.d + static_cast<int64_t>(tok) * p.ldd + n0;
#pragma unroll
                  for (uint32_t g = 0; g < 4; ++g) {
                    uint4 o;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w)
                                 : "r"(buf + lane * 64u + ((g ^ ((static_cast<uint32_t>(lane) >> 1) & 3u)) * 16u))
                                 : "memory");
                    const int col = n0 + 8 * static_cast<int>(g);
                    if (col + 8 <= p.P) {
                      *reinterpret_cast<uint4*>(dst + 8 * g) = o;
                    } else {
                      const uint32_t w[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                      for (int e = 0; e < 8; ++e)
                        if (col + e < p.P)
                          reinterpret_cast<uint16_t*>(dst + 8 * g)[e] = static_cast<uint16_t>(w[e >> 1] >> (16 * (e & 1)));
                    }
                  }
                }
                __syncwarp();                                 // the buffer may be rewritten by the next chunk
              }
            }
            if (live_at(j + 2)) load_chunk(j + 2, r[j & 1]);
          }
        }
        if (tr) FRT_TRACE(p, tl * 8 + (first_half ? 5 : 7));
        continue;
      }
      uint32_t r[2][32];
      // every warp vouches that it is done with tile tl-1; the warps that own the shared columns
      // of this tile only after those columns are in their registers
      if (!first_half || RELEASE_CHUNKS == 0) release();
      // both register buffers are filled before any arithmetic: the first two chunks of the
      // first-half warps are exactly the columns the accumulators share
      static_assert(RELEASE_CHUNKS <= 2 && NCH >= 2, "release after the two prologue loads");
      if (chunk_live(chunk_of(0))) ptx::tc_ld_32x32b_x32(taddr + chunk_of(0) * 32, r[0]);
      if (chunk_live(chunk_of(1))) ptx::tc_ld_32x32b_x32(taddr + chunk_of(1) * 32, r[1]);
      ptx::tc_wait_ld(r[0]);
      ptx::tc_wait_ld(r[1]);
      if (first_half && RELEASE_CHUNKS > 0) release();
      if (tr && first_half) FRT_TRACE(p, tl * 8 + 4);
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        const int cchunk = chunk_of(j);
        const bool live = chunk_live(cchunk);
        if (j >= 2) ptx::tc_wait_ld(r[j & 1]);
        // after the arithmetic of this chunk its buffer is reloaded with chunk j+2 (see loop end)
        if (live) {
        const uint32_t (&v32)[32] = r[j & 1];
        const uint32_t buf = stage_base + (nstore % WARP_BUFS) * 2048u;
        {
          // this lane's 32 outputs of row prow -> 64 bytes of bf16 in a staging buffer laid out
          // as the 64-byte TMA swizzle expects (16-byte piece index ^ ((row >> 1) & 3))
          const int q_base = qt * BN + col0 + cchunk * 32;
          if (TM && !tm_all) {
            // an edge of the expert's rows: each lane writes its own row if it belongs to the expert
            if (prow >= item.lo && prow < item.hi) {
              __nv_bfloat16* dst = p.d + static_cast<int64_t>(prow) * p.ldd + q_base;
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                if (q_base + 8 * g < p.Q && !FRT_DBG(p, 1)) {
                  uint4 o;
                  o.x = pack_bf16x2(__uint_as_float(v32[8 * g + 0]) * alpha, __uint_as_float(v32[8 * g + 1]) * alpha);
                  o.y = pack_bf16x2(__uint_as_float(v32[8 * g + 2]) * alpha, __uint_as_float(v32[8 * g + 3]) * alpha);
                  o.z = pack_bf16x2(__uint_as_float(v32[8 * g + 4]) * alpha, __uint_as_float(v32[8 * g + 5]) * alpha);
                  o.w = pack_bf16x2(__uint_as_float(v32[8 * g + 6]) * alpha, __uint_as_float(v32[8 * g + 7]) * alpha);
                  *reinterpret_cast<uint4*>(dst + 8 * g) = o;
                }
              }
            }
          } else {
          if (nstore >= WARP_BUFS) {                         // the store that last read this buffer is done
            if (lane == 0) ptx::bulk_wait_group_read<WARP_BUFS - 1>();
            __syncwarp();
          }
          const int64_t off = static_cast<int64_t>(prow) * p.ldd + q_base;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = q_base + 8 * g;
            float v[8];
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) v[jj] = __uint_as_float(v32[8 * g + jj]) * alpha;
            if (col < p.Q) {
              if (p.bias != nullptr) {
                float bb[8];
                unpack_bf16x8(__ldg(reinterpret_cast<const uint4*>(p.bias + col)), bb);
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) v[jj] += bb[jj];
              }
              if (p.c != nullptr && prow < p.P) {
                float cc[8];
                unpack_bf16x8(*reinterpret_cast<const uint4*>(p.c + off + 8 * g), cc);
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) v[jj] += p.beta * cc[jj];
              }
            }
            const uint32_t piece = static_cast<uint32_t>(g) ^ ((static_cast<uint32_t>(lane) >> 1) & 3u);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                         ::"r"(buf + lane * 64u + piece * 16u), "r"(pack_bf16x2(v[0], v[1])),
                           "r"(pack_bf16x2(v[2], v[3])), "r"(pack_bf16x2(v[4], v[5])), "r"(pack_bf16x2(v[6], v[7]))
                         : "memory");
          }
          ptx::fence_proxy_async();
          __syncwarp();
          if (lane == 0) {
            if (!FRT_DBG(p, 1)) ptx::tma_store_2d(&maps.d, buf, q_base, TM ? tm_row0 : pt * 256 + row_in_tile);
            ptx::bulk_commit_group();
          }
          ++nstore;
          }   // whole-warp store
        }
        }   // live
        if (j + 2 < NCH && chunk_live(chunk_of(j + 2))) ptx::tc_ld_32x32b_x32(taddr + chunk_of(j + 2) * 32, r[j & 1]);
      }
      if (tr) FRT_TRACE(p, tl * 8 + (first_half ? 5 : 7));
    }
    if (lane == 0) ptx::bulk_wait_group_all();   // staging must outlive the stores that read it
  }

  // Neither CTA may free TMEM or exit while the other can still touch it.
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) ptx::tmem_dealloc_pair(tmem_base, 512);
}
