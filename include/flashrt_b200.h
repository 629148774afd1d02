/*
 * flashrt_b200.h -- C ABI of the B200 (sm_100a) NVFP4 low-bit linear path.
 *
 * Every entry point takes plain device pointers, int sizes, float scalars and
 * a CUDA stream handle (cudaStream_t passed as void*), launches asynchronously
 * on that stream and returns 0 on success or a negative FRT_E_* code.  Nothing
 * here allocates, synchronises or keeps host state between calls (except
 * where a comment says otherwise), so every call can be captured into a CUDA
 * graph.  The caller owns every buffer.
 *
 * Each declaration cites the reference interface it replaces, as
 * <path inside the reference project>:<line>.
 */
#ifndef FLASHRT_B200_H_
#define FLASHRT_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- return codes ------------------------------------------------------ */
#define FRT_OK               0
#define FRT_E_NULL          -1   /* a required pointer is null                  */
#define FRT_E_SHAPE         -2   /* a size is non-positive or not divisible     */
#define FRT_E_ALIGN         -3   /* a pointer misses its alignment              */
#define FRT_E_UNSUPPORTED   -4   /* shape outside what the kernels cover        */
#define FRT_E_LAUNCH        -5   /* the CUDA runtime refused the launch         */
#define FRT_E_DEVICE        -6   /* current device is not compute capability 10 */
#define FRT_E_DRIVER        -7   /* tensor-map encode failed                    */
#define FRT_E_TOO_LARGE     -8   /* size beyond a documented fixed maximum      */

const char* frt_error_string(int rc);

/* ---- element types ----------------------------------------------------- */
#define FRT_DTYPE_BF16 0
#define FRT_DTYPE_FP16 1

/* ---- scale-factor layout ------------------------------------------------
 * Bytes of the swizzled UE4M3 scale buffer of a [rows, dim] NVFP4 tensor:
 * ceil(rows/128) * ceil(dim/64) * 512.
 * replaces nvfp4_sf_swizzled_bytes, flashrt-nvfp4/csrc/nvfp4_sf_reshape_sm120.cuh:26 */
int64_t frt_nvfp4_sf_swizzled_bytes(int rows, int dim);

/* Byte offset of the scale of (row, element k) inside that buffer.
 * replaces sfa_offset_128x64, fp4-gemm/csrc/sfa_layout.cuh:12 */
int64_t frt_nvfp4_sf_offset(int row, int k, int dim);

/* linear [rows, dim/16] u8 -> swizzled.  The bytes that pad a row's last 64-element group
 * (dim % 64 != 0) are written as zero; rows of dst beyond `rows` are not written.
 * replaces nvfp4_sf_linear_to_swizzled, flashrt-nvfp4/csrc/nvfp4_sf_reshape_sm120.cuh:33 */
int frt_nvfp4_sf_linear_to_swizzled(const void* src_linear, void* dst_swizzled,
                                    int rows, int dim, void* stream);

/* ---- stand-alone quantiser / dequantiser --------------------------------
 * src [rows, dim] bf16 or fp16 (16-byte aligned, dim % 16 == 0) ->
 * packed [rows, dim/2] u8 (8-byte aligned) + swizzled UE4M3 scales.
 * Rule: d = max(amax/6, 1e-12); sf = e4m3_rn(d); q = v * (1/float(sf));
 * e2m1 code by thresholds {.25,.75,1.25,1.75,2.5,3.5,5} with ties to the
 * smaller magnitude; sign bit = q < 0.  The scale bytes that pad a row's last 64-element
 * group (dim % 64 != 0) are written as zero (the tensor cores read whole groups); scale
 * bytes of rows beyond `rows` are not written.
 * replaces quantize_fp4_dynamic_sfa_bf16_vec, fp4-gemm/csrc/quantize/quantize_fp4_sfa_bf16.cuh:20
 * and quantize_fp4_dynamic_sfa_fp16/_bf16, fp4-gemm/csrc/quantize/quantize_fp4_sfa.cuh:8,24 */
int frt_nvfp4_quantize(const void* src, int src_dtype, void* packed, void* sf_swizzled,
                       int rows, int dim, void* stream);

/* Bind-time weight packer: same layout as frt_nvfp4_quantize, but each block's scale is the
 * first of nine candidates e4m3(max(amax * (1/6) * m, 1e-12)), m = .375 .5 .625 .75 .875 1
 * 1.125 1.25 1.5, with the lowest squared reconstruction error.
 * replaces quantize_fp4_dynamic_sfa_mse_fp16/_bf16, fp4-gemm/csrc/quantize/quantize_fp4_sfa.cuh:32,36 */
int frt_nvfp4_quantize_mse(const void* src, int src_dtype, void* packed, void* sf_swizzled,
                           int rows, int dim, void* stream);

/* packed + swizzled scales -> fp16 [rows, dim] (exact).
 * replaces dequantize_fp4_sfa_fp16, fp4-gemm/csrc/dequantize_fp4_sfa.cuh:12 */
int frt_nvfp4_dequantize_fp16(const void* packed, const void* sf_swizzled, void* out_fp16,
                              int rows, int dim, void* stream);

/* ---- RMSNorm family (bf16) ---------------------------------------------
 * out = bf16(x * rsqrt(mean(x^2) + eps) * w); dim % 16 == 0, dim <= 16384.
 * replaces rms_norm_bf16, flashrt-residual-norm-quant/csrc/residual_norm_quant.cuh:9 */
int frt_rms_norm_bf16(const void* x, const void* weight, void* out,
                      int rows, int dim, float eps, void* stream);

/* Per-head RMSNorm IN PLACE over the leading heads of a stacked projection output (the q and k heads of one
 * q/k/v GEMM): head h of token t is head_dim contiguous elements at x + t * row_pitch + h * head_dim (elements);
 * heads [0, heads_a) use weight_a [head_dim], the next heads_b use weight_b (NULL when heads_b == 0); what lies
 * beyond them in the row (the v heads) is untouched.  head_dim in {64, 128, 256, 512}; row_pitch % 16 == 0.
 * Each head equals frt_rms_norm_bf16 of its contiguous copy bit for bit.  The reference runs such norms through
 * its kernelize RMSNorm layer, one launch per norm after a copy (demos/space/transformers-qwen3/flashrt_kernelize.py:19-40). */
int frt_rms_norm_heads_bf16(void* x, int tokens, int row_pitch, int head_dim, int heads_a, const void* weight_a,
                            int heads_b, const void* weight_b, float eps, void* stream);

/* residual <- bf16(residual + x) in place; rstd from the fp32 sums; the
 * output pass uses the rounded bf16 residual.
 * replaces residual_add_rms_norm_bf16, flashrt-residual-norm-quant/csrc/residual_norm_quant.cuh:48 */
int frt_residual_add_rms_norm_bf16(void* residual, const void* x, const void* weight, void* out,
                                   int rows, int dim, float eps, void* stream);

/* fp16 form of the fused producer, no weight: residual (fp16, in place) <- half(residual + x);
 * v = (residual + x in fp32) * rsqrt(mean(v^2) + eps); rule-A NVFP4 of v.
 * replaces residual_add_rms_norm_fp4_sfa_v2_fp16 (eps fixed at 1e-6 there),
 *   fp4-fused-ops/csrc/fused_fp4/norm_silu_fp4_sfa.cuh:39 */
int frt_residual_norm_quant_nvfp4_fp16(void* residual, const void* x, float eps, void* packed,
                                       void* sf_swizzled, int rows, int dim, void* stream);

/* LayerNorm, bf16 in / out, affine bf16 weight and bias [dim]:
 *   out = bf16(((x - mean) * rsqrt(var + eps)) * w + b), fp32 statistics (two row reductions).
 * replaces layer_norm_bf16, flashrt-residual-norm-quant/csrc/residual_norm_quant.cuh:18 */
int frt_layer_norm_bf16(const void* x, const void* weight, const void* bias, void* out,
                        int rows, int dim, float eps, void* stream);

/* (residual-add +) RMSNorm -> FP8 E4M3 with a static per-tensor scale (device scalar `scale`):
 *   residual (or null) <- bf16(residual + x);  v = (in * rstd) * w  (in = the rounded residual, or x);
 *   out_fp8[rows, dim] = e4m3_rn(clamp(v * (1 / scale), +-448)).
 * replaces rms_norm_quant_fp8_static_bf16 and residual_add_rms_norm_quant_fp8_static_bf16,
 *   flashrt-residual-norm-quant/csrc/residual_norm_quant.cuh:28,38 */
int frt_rms_norm_quant_fp8(void* residual, const void* x, const void* weight, const void* scale,
                           void* out_fp8, int rows, int dim, float eps, void* stream);

/* ---- fused (residual-add +) RMSNorm -> NVFP4 producer -------------------
 * One pass over HBM: reads x (and residual), writes residual in place,
 * packed e2m1, swizzled UE4M3 scales and, if `normed` is non-null, the bf16
 * value of the quantiser input.  Flags select the reference op's arithmetic:
 *   0 with residual : residual_add_rms_norm_quant_nvfp4_swizzled_bf16 --
 *       v = ((res+x)_fp32 * rstd) * w, not re-rounded, rule-A quantised
 *       (fp4-fused-ops/csrc/fused_fp4/cosmos3_edge_fp4.cuh:17)
 *   ONE_PLUS_W | ROUND_BF16 without residual : rms_norm_quantize_fp4_sfa_bf16
 *       (fp4-fused-ops/csrc/kernels/rms_norm_quantize_fp4_sfa_bf16.cuh:7)
 *   RNE_E2M1 | ROUND_BF16 | NORM_FROM_BF16_RESIDUAL : residual_add_rms_norm_nvfp4_bf16
 *       (fp4-fused-ops/csrc/fused_fp4/pi05_bf16_fp4_producers.cuh, rms_norm_nvfp4_bf16)
 * weight may be null (no scaling).  inv_global_scale multiplies the norm
 * result before quantisation (two-level scaling; pass 1.0f for the
 * reference's one-level recipe).  dim % 16 == 0, dim <= 16384. */
#define FRT_PRODUCER_ONE_PLUS_W               1u
#define FRT_PRODUCER_ROUND_BF16               2u
#define FRT_PRODUCER_RNE_E2M1                 4u
#define FRT_PRODUCER_NORM_FROM_BF16_RESIDUAL  8u
#define FRT_PRODUCER_WAIT_PEERS           0x100u   /* frt_norm_quant_nvfp4_bcast only: also wait for every rank's rows */
int frt_norm_quant_nvfp4(void* residual, const void* x, const void* weight, float eps,
                         float inv_global_scale, void* normed, void* packed, void* sf_swizzled,
                         int rows, int dim, unsigned flags, void* stream);

/* ---- the same producer on a row shard, fused with its exchange (one node, up to 8 GPUs) ---------------
 * For column-parallel GEMMs every GPU needs the NVFP4 activations of all M token rows.  Each rank calls this on
 * ITS rows (residual / x point at the rank's first row, `row0` is that row's index in the whole tensor; row0 and
 * rows are multiples of 128, so that a shard's scale bytes are one contiguous range) and the producer kernel
 * stores the packed codes of those rows straight into every GPU's copy of the whole [M, dim/2] buffer; a small
 * second kernel forwards the shard's scale bytes and publishes the epoch:
 *   mc_packed / mc_sf non-null : NVSwitch multicast addresses of the two buffers (one multimem.st reaches all GPUs);
 *   else dst_packed[i] / dst_sf[i], i < n_dst = n_ranks : each GPU's copy as mapped into this process (peer
 *     stores), this rank's own copy included.  dst_sf[rank] (this GPU's own copy) is needed in both modes.
 * When the grid has finished, the kernel writes `epoch` to element `rank` of every rank's flag array
 * (peer_flags[r] = rank r's array of n_ranks uint32, as mapped into this process).  `counter` is one zeroed uint32
 * of local device memory per buffer (the kernel leaves it zero).  Epochs of one buffer must increase call by call.
 * frt_peer_wait enqueues a kernel that returns once every rank's flag in the LOCAL array has reached `epoch`
 * (bounded: after about a second it sets bit 0x400 of the status word and returns); enqueue it between this call
 * and the first consumer of the buffer - or pass FRT_PRODUCER_WAIT_PEERS in `flags`, and the kernel that
 * publishes this rank's epoch performs the same bounded wait before it ends (one kernel less in the chain).  A buffer may be refilled once every rank has passed the wait of ANOTHER
 * buffer filled later (two buffers used alternately are enough for producer -> GEMMs -> producer -> GEMMs chains).
 * All buffers are the caller's (symmetric allocations, e.g. torch.distributed._symmetric_memory); nothing allocates.
 * Bytes written are those frt_norm_quant_nvfp4 writes for the same rows.  No `normed` output.  n_ranks <= 8.
 * The reference has no multi-GPU code; this entry point has no counterpart there. */
int frt_norm_quant_nvfp4_bcast(void* residual, const void* x, const void* weight, float eps,
                               float inv_global_scale, void* mc_packed, void* mc_sf,
                               void* const* dst_packed, void* const* dst_sf, int n_dst,
                               int row0, int rows, int dim, unsigned flags, void* counter,
                               void* const* peer_flags, int n_ranks, int rank, unsigned epoch, void* stream);
int frt_peer_wait(const void* flags, int n_ranks, unsigned epoch, void* stream);

/* ---- dense NVFP4 A4W4 GEMM, bf16 out ------------------------------------
 * D[M,N] = bf16(alpha * sum_k A[m,k]*SFA[m,k/16] * B[n,k]*SFB[n,k/16]
 *               (+ bias[n]) (+ beta * C[m,n])),  fp32 accumulation in TMEM.
 * A [M,K/2] u8 row-major, B [N,K/2] u8 row-major, scales swizzled, bias bf16
 * [N] or null, C bf16 [M,N] or null (may alias D), beta in {0,1}.
 * K % 32 == 0, N % 8 == 0, A/B 16-byte aligned, D/C 16-byte aligned.
 * Scale buffers must hold frt_nvfp4_sf_swizzled_bytes() bytes; rows of the
 * last 128-row group beyond M / N may hold anything; when K % 64 != 0 the
 * scale bytes that pad the last 64-element group must not be NaN patterns
 * (this library's quantisers write zeros there).
 * B / SFB are treated as constants of the stream: for M <= 64 the kernel starts
 * loading them before it waits for the previous kernel of the stream (launches
 * are programmatic dependents, see FRT_OPT_PDL).  Weights packed on the same
 * stream by frt_nvfp4_quantize / _quantize_mse / _sf_linear_to_swizzled or by an
 * ordinary kernel are complete by then (those never release their dependents
 * early); weights written by a caller's kernel that triggers programmatic
 * dependents before its last store need an event or a stream sync first.
 * replaces fp4_w4a16_gemm_sm100_bf16out (+ _widen, _pingpong),
 *   fp4-gemm/csrc/gemm/fp4/cutlass_nvfp4_w4a16_gemm_sm100.cuh, and
 *   cutlass_fp4_gemm_bias_bf16 / _bias_res_bf16,
 *   fp4-gemm/csrc/gemm/fp4/cutlass_fp4_gemm_bias_bf16_sm100.cuh;
 * small M (<= 64) is served by the same entry point through a
 * weight-streaming configuration, replacing fp4_w4a4_gemv_warpsplit_bf16 /
 * fp4_w4a4_gemm_warpsplit_mrows_bf16 (fp4-gemm/csrc/gemm/fp4/fp4_w4a4_mma_warpsplit_sm120.cuh). */
int frt_nvfp4_gemm_bf16(const void* a_packed, const void* sfa, const void* b_packed, const void* sfb,
                        const void* bias, const void* c, void* d,
                        int M, int N, int K, float alpha, float beta, void* stream);

/* The reference's bind-time weight layout of its M = 1 GEMV and the GEMV that consumes it.
 * Layout: b_interleaved viewed as [N/8][K/64][8][32 bytes] holds b_packed [N/8][8][K/64][32 bytes]
 * (groups of 8 rows x 64-element k-tiles x 8 rows x 32 B), N % 8 == 0, K % 64 == 0.
 * The GEMV reads that layout as a dense 4-D tensor (32-byte-swizzled 8-row x 32-byte atoms in shared
 * memory) and runs the same weight-streaming kernel: out[1, N] bit-equal to frt_nvfp4_gemm_bf16 at M = 1.
 * replaces fp4_w4a4_repack_b_ilv_sm120 and fp4_w4a4_mma_sm120_warpsplit_ilv_bf16out,
 *   fp4-gemm/csrc/gemm/fp4/fp4_w4a4_mma_warpsplit_ilv_sm120.cuh:15,21 */
int frt_nvfp4_repack_interleaved(const void* b_packed, void* b_interleaved, int N, int K, void* stream);
int frt_nvfp4_gemv_interleaved_bf16(const void* a_packed, const void* sfa, const void* b_interleaved,
                                    const void* sfb, void* out, int N, int K, float alpha, void* stream);

/* Which kernel configuration frt_nvfp4_gemm_bf16 would run for (M, N, K) on the current
 * device, without launching anything (a host-side query; tests use it to prove which path a
 * shape takes).  *config: 1-3 one CTA per 128-row tile (128 / 256 / 192 columns), 4-6 CTA pair
 * per 256-row tile (256 / 192 / 128 columns), 11-14 weight-streaming form for M <= 64 (16 /
 * 32 / 64 / 128 token columns); *split_k: CTAs of a cluster that share one tile's K (1 = none).
 * replaces select_sm110_variant, fp4-gemm/torch-ext/torch_binding.cpp:169 */
int frt_nvfp4_gemm_plan(int M, int N, int K, int* config, int* split_k);

/* ---- SwiGLU -> NVFP4 (the step between the two FFN GEMMs) -----------------
 * merged [rows, 2*hidden] bf16 = [gate | up] (16-byte aligned, hidden % 16 == 0) ->
 * packed [rows, hidden/2] + swizzled scales of v = bf16((g / (1 + exp(-g))) * u)
 * (fp32 arithmetic, accurate expf, IEEE division), rule-A quantised as frt_nvfp4_quantize.
 * replaces silu_mul_quantize_fp4_sfa_bf16,
 *   fp4-fused-ops/csrc/kernels/silu_mul_quantize_fp4_sfa_bf16.cuh:18 */
int frt_silu_mul_quant_nvfp4(const void* merged, void* packed, void* sf_swizzled,
                             int rows, int hidden, void* stream);

/* The same producer as the epilogue of the gate/up GEMM: B is the [gate ; up] weight
 * [N2 = 2*hidden, K/2] (gate rows first), and the result is exactly
 *   frt_silu_mul_quant_nvfp4(frt_nvfp4_gemm_bf16(A, B, alpha))
 * without the [M, 2*hidden] bf16 intermediate ever reaching memory.
 * hidden % 128 == 0, K % 32 == 0, out_packed 16-byte aligned.
 * No single reference entry point does this for SwiGLU/bf16; the nearest are the FP4-out
 * epilogues nvfp4_gemm_nvfp4 and nvfp4_gemm_geglu_nvfp4_fp16
 * (fp4-gemm/torch-ext/torch_binding.cpp:579-657), which need an interleaved weight repack and
 * a scratch buffer; this one takes the plain stacked weight and no scratch. */
int frt_nvfp4_gemm_swiglu_nvfp4(const void* a_packed, const void* sfa, const void* b_packed, const void* sfb,
                                void* out_packed, void* out_sf_swizzled,
                                int M, int N2, int K, float alpha, void* stream);

/* ---- grouped (MoE) NVFP4 GEMM, bf16 out ---------------------------------
 * Rows of `a_packed` [rows, K/2] are expert-sorted; their scales are one
 * swizzled buffer over all rows (indexed by global row).  Expert e owns the
 * stacked weights b_stack + e*b_stride (bytes) [N,K/2] and scales
 * sfb_stack + e*sfb_stride.  out[r,:] = bf16(alpha[e(r)] * A[r,:] . W[e(r)]^T).
 * Exactly one of the two descriptions of e(r) is given:
 *   expert_offsets : int32 [num_experts+1] device array, expert e owns rows
 *                    [off[e], off[e+1]); rows >= off[num_experts] untouched.
 *   tile_expert    : int32 [rows/tile_rows] device array, tile t (tile_rows in
 *                    {16,64} rows) uses expert tile_expert[t]; negative = skip
 *                    (those output rows are left untouched).
 * K % 64 == 0, N % 8 == 0.  `work` is caller-owned scratch of
 * frt_nvfp4_grouped_gemm_workspace_bytes() bytes (device, 16-byte aligned): room for
 * rows/16 + 2*num_experts + 8 row windows, which covers every sorted expert_offsets and every
 * tile_expert pattern (16-row tiles of alternating experts included).  Offsets that overlap or
 * decrease describe more rows than exist; windows that do not fit are dropped, never written past
 * the buffer, and bit 0x200 of the status word (frt_device_status) reports it.
 * (With expert_offsets and num_experts <= 256 the GEMM's CTAs derive the windows themselves and the call is
 * one launch that does not touch `work`; the same limit on the number of windows applies.  Pass the buffer
 * all the same: the tile_expert description and larger expert counts use it.)
 * replaces moe_blocktile_mma_sm120_bf16 / moe_m64_mma_sm120_bf16 / moe_m16_mma_sm120_bf16,
 *   grouped-moe-gemm/csrc/moe_blocktile_mma_sm120.cuh */
int64_t frt_nvfp4_grouped_gemm_workspace_bytes(int rows, int num_experts);
int frt_nvfp4_grouped_gemm_bf16(const void* a_packed, const void* sfa,
                                const void* b_stack, const void* sfb_stack, const void* alpha,
                                const void* expert_offsets, const void* tile_expert, int tile_rows,
                                void* out, int rows, int N, int K, int num_experts,
                                int64_t b_stride, int64_t sfb_stride,
                                void* work, void* stream);

/* Same computation for callers that cannot allocate device memory and have no
 * buffer to lend: a plug-in called from a host runtime that owns the device
 * allocator and forbids cudaMalloc on its worker threads, a serving process
 * that has already handed all free device memory to another pool (so an
 * allocation would fail), or an embedding with a fixed memory map.
 * The work list lives in a fixed array inside the library instead of `work`;
 * inputs and outputs are still the caller's.  No counterpart in the reference.
 *  - Limits: rows <= FRT_GROUPED_STATIC_MAX_ROWS and
 *    num_experts <= FRT_GROUPED_STATIC_MAX_EXPERTS, else FRT_E_TOO_LARGE.  The
 *    array (about 384 KiB) is resident on every GPU that loads the library.
 *  - The first call on a device looks up the array's device address (no
 *    allocation); make that first call before starting a stream capture.
 *  - Every call uses the same array: two calls whose kernels can overlap on the
 *    GPU (different streams, no dependency) race on it.  Calls on one stream,
 *    or otherwise ordered, are safe; the array keeps the previous call's work
 *    list and the part that must start at zero is cleared on `stream` by the call. */
#define FRT_GROUPED_STATIC_MAX_ROWS     131072
#define FRT_GROUPED_STATIC_MAX_EXPERTS  2048
int frt_nvfp4_grouped_gemm_bf16_noalloc(const void* a_packed, const void* sfa,
                                        const void* b_stack, const void* sfb_stack, const void* alpha,
                                        const void* expert_offsets, const void* tile_expert, int tile_rows,
                                        void* out, int rows, int N, int K, int num_experts,
                                        int64_t b_stride, int64_t sfb_stride, void* stream);

/* ---- MoE routing glue (the stages around the grouped GEMM) -----------------
 * Exact top-k of bf16 router logits [tokens, n_experts] -> out_idx i32 [tokens, k] and
 * out_val f32 [tokens, k] (the logits, descending; equal logits in the order the reference's
 * block reduction yields: bit-reversed low 8 index bits, then index; the caller softmaxes
 * the k values).  n_experts <= 1024, k <= 32.
 * replaces nexn2_router_topk_bf16 (one token),
 *   transformer-fused-ops/csrc/kernels/nexn2_router_topk.cuh:18 */
int frt_router_topk_bf16(const void* logits, void* out_idx, void* out_val,
                         int tokens, int n_experts, int k, void* stream);

/* The same router with the routing weights as a fourth output: out_weight f32 [tokens, k] = softmax over
 * the k selected logits (= the top-k of the full softmax, re-normalised); out_weight may be NULL. */
int frt_router_topk_softmax_bf16(const void* logits, void* out_idx, void* out_val, void* out_weight,
                                 int tokens, int n_experts, int k, void* stream);

/* Routing plan = stable sort of the (token, slot) pairs by expert, on the device:
 *   expert_offsets i32 [n_experts + 1]  rows of expert e are [offsets[e], offsets[e+1])
 *   row_of_pair    i32 [tokens * k]     expert-sorted row of pair (t, j); -1 if its index is
 *                                       outside [0, n_experts)
 *   token_of_row   i32 [tokens * k]     source token of each expert-sorted row (entries at and
 *                                       beyond expert_offsets[n_experts] are not written)
 * The reference leaves this stage to the caller ("stable routing sort, expert-tile packing
 * ... remain explicit structure-level stages", grouped-moe-gemm/README.md:13-16). */
int frt_moe_route_plan(const void* topk_idx, int tokens, int k, int n_experts,
                       void* expert_offsets, void* row_of_pair, void* token_of_row, void* stream);

/* Gather NVFP4 rows (packed [tokens, K/2] + swizzled scales) into expert-sorted order:
 * out row r = in row token_of_row[r].  K % 64 == 0.  Same README passage. */
int frt_moe_gather_nvfp4(const void* packed_in, const void* sf_in, const void* token_of_row,
                         void* packed_out, void* sf_out, int rows, int tokens, int K, void* stream);

/* Quantise bf16 token rows [tokens, K] (rule A, as frt_nvfp4_quantize) straight into expert order:
 * the NVFP4 form of token t is stored to rows row_of_pair[t, 0..k) of packed_out / sf_out (negative rows
 * skipped).  Equal to frt_nvfp4_quantize followed by frt_moe_gather_nvfp4, in one pass. */
int frt_moe_quantize_scatter_nvfp4(const void* x, const void* row_of_pair, void* packed_out, void* sf_out,
                                   int tokens, int k, int K, void* stream);

/* Weighted un-permute: out f32 [tokens, hidden] = sum_j weights[t, j] * expert_out[row[t, j], :hidden]
 * (bf16 rows of pitch `stride` elements), one fused multiply-add per slot in slot order,
 * negative rows skipped.
 * replaces moe_weighted_sum_sm120_bf16,
 *   transformer-fused-ops/csrc/kernels/moe_weighted_sum_sm120.cuh:20 */
int frt_moe_weighted_sum_bf16(const void* expert_out, const void* row_of_pair, const void* weights,
                              void* out, int tokens, int k, int hidden, int stride, void* stream);

/* ---- status / tuning -----------------------------------------------------
 * Device-side waits are bounded; a wait that runs out records a code in a
 * per-device status word and the kernel returns.  This call copies the word to
 * the host (synchronises `stream`) and clears it: 0 = no kernel gave up. */
int frt_device_status(void* stream, unsigned* status_out);

/* Number of kernels this library has launched from the calling process. */
int64_t frt_launch_count(void);

/* Tuning / debugging switches; see the FRT_OPT_* keys. Returns previous value. */
#define FRT_OPT_QUANT_ENCODER   1   /* 0 = hardware-cvt encoder (default), 1 = compare chain */
#define FRT_OPT_GEMM_CONFIG     2   /* 0 = automatic, otherwise a configuration id          */
#define FRT_OPT_PDL             4   /* 1 = launch kernels with programmatic stream serialization
                                       (default): a kernel's prologue overlaps the tail of the
                                       previous kernel of the stream; 0 = plain launches      */
#define FRT_OPT_NORM_FORM       5   /* norm kernels: 0 = by row width (default), 1 = one CTA per
                                       row group, 2 = persistent CTAs fed by bulk copies       */
#define FRT_OPT_GEMM_TAIL_SPLIT 6   /* dense CTA-pair GEMM: 1 = cut the last, partial wave of
                                       tiles into column slices (default), 0 = whole tiles     */
#define FRT_OPT_GEMM_SPLIT_K    7   /* small-M GEMM: 1 = split K over a cluster when there are
                                       fewer weight tiles than SMs (default), 0 = never,
                                       2..8 = that many CTAs per tile when it divides K / 256   */
#define FRT_OPT_SMALLM_STAGES   8   /* small-M GEMM: shared-memory ring depth, 0 = default, 2 or 3 =
                                       shallower rings (more CTAs per SM), 8 = the deep ring of the
                                       64-token form (one CTA per SM); for measurements           */
#define FRT_OPT_WAIT_LIMIT_LOG2 9   /* log2 of the SM clocks a device-side wait (mbarrier, peer flag) may
                                       spin before the kernel gives up, sets its status bit and returns:
                                       default 31 (about a second), accepted range 20..40            */
#define FRT_OPT_GROUPED_FORM   10   /* grouped GEMM: 0 / 1 = weight-major (expert weights on the 256-row axis,
                                       transposed output tile; default, the faster one measured),
                                       2 = token-major (128-row token blocks on the 256-row axis)     */
int frt_set_option(int key, int value);

#ifdef __cplusplus
}
#endif
#endif /* FLASHRT_B200_H_ */
