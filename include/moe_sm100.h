/*
 * moe_sm100.h — C ABI of libmoe_sm100.so: the B200 (sm_100a) kernels of the
 * fused Mixture-of-Experts path (group-limited top-k routing, block alignment
 * of routed tokens, the two expert grouped GEMMs and the top-k combine).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless the parameter says "host".
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it and
 *     nothing synchronises with the host, so every call can be captured in a
 *     CUDA graph (tensor maps are built on the host before the launch).
 *   - Return value: 0 on success, a negative MOE_E_* code for a rejected
 *     argument, a positive cudaError_t value when a launch failed.
 *     moe_last_error() gives the text of the last failure of the calling thread.
 *   - `status` is an optional device int32 word.  Kernels never trap: on bad
 *     data (an expert id outside the table, a wait that ran out) they OR a
 *     MOE_ST_* bit into it and carry on or return; the host reads it when it
 *     chooses to.
 *   - dtype codes: MOE_F32 0, MOE_F16 1, MOE_BF16 2, MOE_FP8E4M3 3, MOE_INT8 4.
 *
 * Each entry point names the reference interface it stands in for, as
 * path:line inside the FlagGems-vllm source tree.
 */
#ifndef MOE_SM100_H_
#define MOE_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MOE_F32 = 0, MOE_F16 = 1, MOE_BF16 = 2, MOE_FP8E4M3 = 3, MOE_INT8 = 4 };

enum {
  MOE_E_BADARG = -1,     /* null pointer, negative extent, unsupported size */
  MOE_E_DTYPE = -2,      /* dtype code not handled by this entry point */
  MOE_E_SHAPE = -3,      /* shape not supported by the requested kernel */
  MOE_E_DRIVER = -4,     /* CUDA driver entry point unavailable */
  MOE_E_TOOBIG = -5      /* exceeds a fixed capacity (see the entry point) */
};

enum {
  MOE_ST_BAD_EXPERT_ID = 1,  /* an expert id >= num_experts was skipped (negative ids = no route, silent) */
  MOE_ST_WAIT_TIMEOUT = 2,   /* a bounded barrier wait ran out; results invalid */
  MOE_ST_BAD_ROW = 4         /* a sorted row index outside its buffer was skipped */
};

/* GEMM modes (moe_gemm*_ entry points) */
enum {
  MOE_MODE_HALF = 0,
  MOE_MODE_FP8_BLOCK = 1,
  MOE_MODE_W8A16 = 2,
  MOE_MODE_FP8_ROW = 3,  /* e4m3 activations with one fp32 scale per row, e4m3 weights with one per output channel */
  MOE_MODE_INT8_ROW = 4  /* int8 activations with one fp32 scale per row, int8 weights with one per output channel */
};

/* GEMM 1 activations */
enum { MOE_ACT_SILU = 0, MOE_ACT_SWIGLUOAI = 1 };

int moe_abi_version(void);
const char* moe_last_error(void);

/*
 * Failure handling hooks; neither has a counterpart in the reference (its Triton kernels have no
 * waits of their own).
 * moe_set_wait_limit_ns: limit of every bounded barrier wait of the kernels launched afterwards
 *   (default 2 s; 0 only queries).  Returns the previous limit.  Host-side, process-wide.
 * moe_debug_wait_timeout: launches one warp that waits, with the given limit (at most 100 ms),
 *   on a barrier nobody arrives at.  The wait runs out, MOE_ST_WAIT_TIMEOUT is ORed into
 *   `status`, `gave_up[0]` (optional) becomes 1 and the kernel returns: how the status path is
 *   exercised without hanging or faulting a GPU.
 */
unsigned long long moe_set_wait_limit_ns(unsigned long long ns);
int moe_debug_wait_timeout(int32_t* status, unsigned long long limit_ns, int32_t* gave_up, void* stream);

/*
 * Group-limited top-k routing, one warp per token.
 * Stands in for grouped_topk (src/flaggems_vllm/ops/grouped_topk.py:1674-1976)
 * and its kernels (:333-794, :887-1081).  scores[M,E] with element strides
 * (stride0, stride1); bias[E] contiguous; is_padding[M] bytes or NULL.
 * Outputs topk_weights[M,topk] fp32 and topk_ids[M,topk] int32, row-major.
 * Limits: E <= 4096 (one warp per token up to 1024 experts, one CTA per token beyond), n_group <= 32,
 * topk <= 32.
 */
int moe_grouped_topk(const void* scores, int scores_dtype, int64_t stride0, int64_t stride1,
                     const void* bias, int bias_dtype, const uint8_t* is_padding,
                     int64_t M, int E, int n_group, int topk_group, int topk,
                     int renormalize, float routed_scaling_factor, int scoring_func,
                     float* topk_weights, int32_t* topk_ids, void* stream);

/*
 * Non-grouped routers: softmax (sigmoid = 0) or sigmoid (1) scores of logits[M,E]
 * (contiguous), optional fp32 selection bias[E], optional padding mask, top-k
 * with ties to the lower expert id; weights are the unbiased scores, divided by
 * their sum when renormalize (if the sum is positive), times `scale`.  Outputs
 * are caller-owned: topk_weights[M,topk] fp32, topk_indices[M,topk] (index_kind
 * 0 int32, 1 int64, 2 uint32), token_expert_indices[M,topk] int32 = slot*M + token.
 * Stands in for topk_softmax (src/flaggems_vllm/ops/topk_softmax.py:126-202) and
 * topk_sigmoid (src/flaggems_vllm/ops/topk_sigmoid.py:92-226).  Limits: E <= 1024, topk <= 32.
 */
int moe_topk_route(const void* logits, int logits_dtype, const float* bias, const uint8_t* is_padding,
                   int64_t M, int E, int topk, int sigmoid, int renormalize, float scale,
                   float* topk_weights, void* topk_indices, int index_kind,
                   int32_t* token_expert_indices, void* stream);

/*
 * Stable counting sort of the flat expert-id array with per-expert padding to
 * block_size.  Stands in for moe_align_block_size_triton
 * (src/flaggems_vllm/ops/moe_align_block_size.py:607-718; stages :414-527).
 * topk_ids: numel ids, int32 (ids_int64 = 0) or int64 (1).
 * sorted_ids[sorted_cap] is fully written (pad value = numel),
 * expert_ids[expert_cap] is fully written (unused = -1), num_post_pad[1].
 * Order inside an expert is ascending flat index (deterministic).
 * Limits: num_experts <= 4096, numel < 2^31.
 */
int moe_align_block_size(const void* topk_ids, int ids_int64, int64_t numel, int num_experts,
                         int block_size, int32_t* sorted_ids, int64_t sorted_cap,
                         int32_t* expert_ids, int64_t expert_cap, int32_t* num_post_pad,
                         int32_t* status, void* stream);

/*
 * In place: expert_ids[i] = expert_map[expert_ids[i]] for n block ids (ids outside
 * [0, num_experts), i.e. the -1 of unused blocks, become -1).  The lookup the reference does with
 * tensor indexing after the sort (src/flaggems_vllm/ops/moe_align_block_size.py:924-925).
 */
int moe_map_expert_ids(int32_t* expert_ids, int64_t n, const int32_t* expert_map, int num_experts,
                       void* stream);

/*
 * 1 x group e4m3 quantisation of rows: scale = max(amax,1e-10) * (1/448),
 * q = clamp(x / scale).  Stands in for per_token_group_quant_fp8
 * (src/flaggems_vllm/ops/per_token_group_quant_fp8.py:226-335, kernel :115-162).
 * x[rows, cols] contiguous (F32/F16/BF16); q[rows, cols]; scales row-major
 * [rows, cols/group] or, with bit 0 of scales_transposed set, [cols/group, scale_ld].
 * Bit 1 of scales_transposed rounds every scale up to a power of two (the
 * reference's scale_ue8m0 option, :153-154).  group must be 128.
 */
int moe_per_token_group_quant_fp8(const void* x, int x_dtype, int64_t rows, int64_t cols, int group,
                                  void* q, float* scales, int scales_transposed, int64_t scale_ld,
                                  void* stream);
/*
 * The same quantiser with every option of the reference function: any group size that divides
 * cols, the amax clamp `eps`, and e5m2 output (e5m2 = 1; clamp range +-57344) besides e4m3.
 * moe_per_token_group_quant_fp8 is this call with eps = 1e-10 and e4m3.
 */
int moe_per_token_group_quant_fp8_ex(const void* x, int x_dtype, int64_t rows, int64_t cols, int group, float eps,
                                     int e5m2, void* q, float* scales, int scales_transposed, int64_t scale_ld,
                                     void* stream);

/*
 * Exact widening of int8 weights to f16/bf16 (n elements, n % 16 == 0).  The
 * weight-only INT8 layer runs the tensor-core GEMMs on the widened copy and
 * applies the per-channel scale in the GEMM epilogue; the reference instead
 * multiplies the whole weight tensor by its scales in the activation dtype on
 * every call (src/flaggems_vllm/ops/fused_moe.py:2493-2500).
 */
int moe_widen_int8(const void* src, void* dst, int dst_dtype, int64_t n, void* stream);

/*
 * Router GEMM: logits[M, N] = x[M, K] . w[N, K]^T with fp32 products, fp32
 * accumulation in a fixed order (deterministic) and fp32 output, for decode-sized
 * M.  Stands in for router_gemm (src/flaggems_vllm/ops/router_gemm.py:207-237) and
 * fp32_router_gemm (src/flaggems_vllm/ops/fp32_router_gemm.py:108-145).
 *   x [M, K] F32/F16/BF16, rows x_ld elements apart (x_ld % 8 == 0, K % 8 == 0)
 *   w [N, K] contiguous F32/F16/BF16; out [M, N] fp32
 */
int moe_router_gemm(const void* x, int x_dtype, int64_t x_ld, const void* w, int w_dtype, int64_t M, int N, int K,
                    float* out, void* stream);

/*
 * Router GEMM fused with the group-limited routing, for decode batches: one launch takes the hidden
 * states to (topk_weights, topk_ids); the [M, E] logits stay in shared memory (logits_out, optional,
 * receives a copy for checks).  Logits, ids and weights equal those of moe_router_gemm followed by
 * moe_grouped_topk bit for bit.  Removes the logits round trip in front of grouped_topk
 * (src/flaggems_vllm/ops/router_gemm.py:207-237 + src/flaggems_vllm/ops/grouped_topk.py:1674-1976).
 * x [M, K] (pitch x_ld), w [E, K]: bf16/bf16, f16/f16, bf16/f32 or f32/f32; bias [E] fp32.
 */
int moe_router_gemm_grouped_topk(const void* x, int x_dtype, int64_t x_ld, const void* w, int w_dtype,
                                 const float* bias, int64_t M, int E, int K, int n_group, int topk_group, int topk,
                                 int renormalize, float routed_scaling_factor, int scoring_func, float* topk_weights,
                                 int32_t* topk_ids, float* logits_out, void* stream);

/*
 * Copy of the token rows into sorted order: out[p] = x[sorted_ids[p] / topk] for
 * the occupied slots p < num_post_pad (padding slots and the tail are left
 * untouched).  Optional first step of GEMM 1 (a_sorted = 1): with many rows per
 * expert the tensor-core kernel is faster fed by TMA boxes of this copy than by
 * its own row gather.  The reference gathers inside its GEMM kernel
 * (src/flaggems_vllm/ops/fused_moe.py:1559); this copy has no counterpart there.
 *   x [num_tokens, row_bytes] any dtype, out [rows_cap, row_bytes]; row_bytes % 16 == 0
 */
int moe_gather_rows(const void* x, int64_t num_tokens, int topk, int64_t row_bytes, const int32_t* sorted_ids,
                    const int32_t* num_post_pad, int64_t rows_cap, void* out, void* stream);

/*
 * The companion of moe_gather_rows for FP8 activations: the transposed 1x128 scales
 * [groups, num_tokens] copied into sorted order, out_t[g][p] = scales_t[g][sorted_ids[p] / topk]
 * with out_t [groups, rows_cap].  Like the row copy it has no counterpart in the reference.
 */
int moe_gather_scales_t(const float* scales_t, int groups, int64_t num_tokens, int topk, const int32_t* sorted_ids,
                        const int32_t* num_post_pad, int64_t rows_cap, float* out_t, void* stream);

/*
 * Expert grouped GEMM 1: act[p] = SiLU(x_t Wg^T) * (x_t Wu^T) for every sorted
 * row p, where t = sorted_ids[p] / topk is the token of that route.  The kernel
 * gathers the token rows itself; no sorted copy of the activations is needed
 * (a_sorted = 0), or reads rows already copied into sorted order (a_sorted = 1).
 * Stands in for fused_moe_kernel with FUSE_SILU, including its row gather
 * (src/flaggems_vllm/ops/fused_moe.py:1559, 1634-1795, launch :2078-2220).
 *   a [num_tokens, H]        activations in token order (act dtype, or e4m3 in FP8 mode);
 *     with a_sorted != 0: [rows_cap, H] rows in sorted order from moe_gather_rows
 *     (half-precision modes with use_tensor_cores 1 or 3 only)
 *   a_scales_t [H/128, num_tokens]  1x128 activation scales, transposed (FP8 mode)
 *   w1 [E, 2I, H] contiguous (act dtype, e4m3 or int8), gate rows first
 *   w1_scale: FP8 [E, 2I/128, H/128]; W8A16 [E, 2I]; HALF: NULL, or [E, 2I]
 *     per-output-channel scales applied in the epilogue (widened int8 weights)
 *   expert_ids [rows_cap / block_m], sorted_ids [rows_cap], num_post_pad[1] from the align step
 *   route_weight [num_tokens * topk]: when mul_weight != 0 gate and up are
 *     multiplied by route_weight[sorted_ids[p]] before the activation
 *   out [rows_cap, I] in sorted order: act dtype, or e4m3 with
 *     out_scales_t [I/128, rows_cap] in FP8 mode (the activation is rounded to
 *     act dtype, then quantised 1x128, as the reference does between its GEMMs)
 * use_tensor_cores: 0 = generic kernel (block_m % 16 == 0, any mode);
 *   1 = tcgen05 kernel, one CTA per 128-row align block (block_m must be 128,
 *   rows_cap % 128 == 0, I % 128 == 0, H % 128 == 0 for FP8 / H % 64 == 0 for half);
 *   2 = tcgen05 kernel, a cta_group::2 CTA pair per 256-row align block
 *   (block_m must be 256, rows_cap % 256 == 0): each weight tile is fetched once
 *   per 256 rows;
 *   3 = tcgen05 kernel, one CTA per 256-row align block with a 256x256 tile whose two
 *   accumulators fill TMEM (half precision only, block_m 256);
 *   4 = tcgen05 kernel, a cta_group::2 CTA pair per 512-row align block, 256x256 per
 *   CTA, each CTA loading half of every weight tile (half precision only, block_m 512).
 *   MOE_MODE_W8A16 accepts 0 and 1; 1 widens the int8 weights in shared memory.
 *   GEMM1 and GEMM2 of one layer must use the same block_m.
 */
int moe_gemm1(int mode, int act_dtype, const void* a, int a_sorted, const float* a_scales_t, int64_t num_tokens,
              int topk, const void* w1, const float* w1_scale, const int32_t* expert_ids,
              const int32_t* sorted_ids, const int32_t* num_post_pad, const float* route_weight,
              int mul_weight, int64_t rows_cap, int block_m, int E, int H, int I, void* out,
              float* out_scales_t, int use_tensor_cores, int32_t* status, void* stream);

/*
 * moe_gemm1 with the activation spelled out: MOE_ACT_SILU, or MOE_ACT_SWIGLUOAI
 * (min(gate, limit) * sigmoid(alpha * gate) * (clamp(up, -limit, limit) + beta) on the gate | up halves,
 * src/flaggems_vllm/ops/fused_moe.py:733-773).  The row-scaled modes MOE_MODE_FP8_ROW / MOE_MODE_INT8_ROW
 * (per-tensor and per-token W8A8, src/flaggems_vllm/ops/fused_moe.py:853-1010, scales applied to the
 * finished dot product as in :1894-1925) and every activation other than SiLU are served by the
 * generic kernel (use_tensor_cores = 0): a [num_tokens, H] in e4m3 / int8, a_scales_t [num_tokens]
 * (one per row), w1_scale [E, 2I]; the intermediate is written in the activation dtype, unquantised.
 * In moe_gemm2 the same modes take act_scales_t [rows_cap] and w2_scale [E, H].
 */
int moe_gemm1_ex(int mode, int act_dtype, const void* a, int a_sorted, const float* a_scales_t, int64_t num_tokens,
                 int topk, const void* w1, const float* w1_scale, const int32_t* expert_ids,
                 const int32_t* sorted_ids, const int32_t* num_post_pad, const float* route_weight,
                 int mul_weight, int64_t rows_cap, int block_m, int E, int H, int I, void* out,
                 float* out_scales_t, int use_tensor_cores, int activation, float alpha, float beta, float limit,
                 int32_t* status, void* stream);

/*
 * Row-wise activation quantisers of the W8A8 modes (moe_kernel_quantize_input,
 * src/flaggems_vllm/ops/fused_moe.py:1196-1220).  kind:
 *   0  int8, one dynamic scale per row: amax clamped at 1e-10 in the input dtype, scale = amax * (1/127),
 *      q = round-half-even(x / scale) in [-128, 127]            (:994-1010)
 *   1  e4m3, one dynamic scale per row: max(amax, 1e-10) / 448, at least 1 / (448 * 512)   (:899-911)
 *   2  e4m3, static per-tensor scale scale_in[0]: q = clamp(x / scale)                      (:913-917)
 *   3  e4m3, dynamic per-tensor scale: amax of the whole tensor / 448, q = clamp(x * (1 / scale)); rows whose
 *      row_ids entry is outside [0, valid_below) are skipped when row_ids is given            (:918-922)
 *   4  int8, static per-tensor scale scale_in[0]: q = round-half-even(x / scale)             (:966-969)
 * x [rows, cols] F32/F16/BF16 contiguous, q [rows, cols] bytes, scale_out [rows] (kinds 0, 1) or [1]
 * (kind 3; kinds 2 and 4 copy scale_in[0] to scale_out[0] when scale_out is given).
 */
int moe_rowwise_quant(const void* x, int x_dtype, int64_t rows, int64_t cols, int kind, const float* scale_in,
                      const int32_t* row_ids, int64_t valid_below, void* q, float* scale_out, void* stream);

/*
 * Expert grouped GEMM 2: y[sorted_ids[p], :] = (act[p] W2[e]^T) * route_weight.
 * Stands in for fused_moe_kernel as called for the down projection
 * (src/flaggems_vllm/ops/fused_moe.py:1797-1985, call :2703-2728).
 *   act_sorted [rows_cap, I] (act dtype or e4m3 with act_scales_t [I/128, rows_cap])
 *   w2 [E, H, I] contiguous; w2_scale: FP8 [E, H/128, I/128]; W8A16 [E, H];
 *     HALF: NULL or [E, H] per-output-channel scales
 *   y [numel, H] in act dtype, row = flat route index (token * topk + slot)
 */
int moe_gemm2(int mode, int act_dtype, const void* act_sorted, const float* act_scales_t,
              const void* w2, const float* w2_scale, const int32_t* expert_ids,
              const int32_t* sorted_ids, const int32_t* num_post_pad, const float* route_weight,
              int mul_weight, int64_t numel, int64_t rows_cap, int block_m, int E, int H, int I,
              void* y, int use_tensor_cores, int32_t* status, void* stream);

/*
 * moe_gemm2 on the 128-row tcgen05 kernel (use_tensor_cores = 1; FP8 block scales or half precision)
 * with the route rows written in SORTED order: y_sorted [rows_cap, H] receives row p of the sorted
 * intermediate at row p (whole tiles, staged in shared memory and written by TMA bulk stores), and
 * inv[route] = p for every routed (token, slot).  moe_sum then reads the rows through
 * row_index = inv.  Same arithmetic as moe_gemm2; only where the rows land differs.
 */
int moe_gemm2_sorted(int mode, int act_dtype, const void* act_sorted, const float* act_scales_t, const void* w2,
                     const float* w2_scale, const int32_t* expert_ids, const int32_t* sorted_ids,
                     const int32_t* num_post_pad, const float* route_weight, int mul_weight, int64_t numel,
                     int64_t rows_cap, int block_m, int E, int H, int I, void* y_sorted, int32_t* inv,
                     int32_t* status, void* stream);

/*
 * moe_gemm2_sorted over a window of the output columns: y_window [rows_cap, ncols] receives columns
 * [col0, col0 + ncols) of every row (col0 and ncols multiples of 256).  Two such calls make the
 * whole y; a caller whose next step can start on the first columns (the expert-parallel combine)
 * overlaps it with the second call, and max_ctas > 0 keeps that call off some SMs for it.  inv is
 * written by every call (the same values).  No counterpart in the reference.
 */
int moe_gemm2_sorted_cols(int mode, int act_dtype, const void* act_sorted, const float* act_scales_t, const void* w2,
                          const float* w2_scale, const int32_t* expert_ids, const int32_t* sorted_ids,
                          const int32_t* num_post_pad, const float* route_weight, int mul_weight, int64_t numel,
                          int64_t rows_cap, int block_m, int E, int H, int I, int col0, int ncols, void* y_window,
                          int32_t* inv, int max_ctas, int32_t* status, void* stream);

/*
 * Small-batch schedule of the two expert GEMMs (weight streaming, split-K): align blocks of
 * 8 routes, every routed expert's weights read once, K cut into slices whose fp32 partial
 * tiles are added in slice order by whichever CTA finishes a tile last (no floating-point
 * atomics, bitwise reproducible).  GEMM 2 also joins the top-k routes of every token in
 * slot order and writes the layer output, so no separate moe_sum pass runs.
 * Stands in for the reference's small-batch route (naive_block_assignment,
 * src/flaggems_vllm/ops/fused_moe.py:2542-2568, kernel branch :1541-1548) and, for the
 * combine, moe_sum (src/flaggems_vllm/ops/moe_sum.py:250-310).
 *
 * moe_small_m_plan: scratch sizes of one GEMM for (K, Nout, rows_cap): fp32 elements of the
 *   partial-sum buffer (0 when one K slice suffices), int32 unit counters, int32 token counters
 *   (GEMM 2 only).  k_slices >= 1 asks for at least that many K slices (more units of work
 *   when few experts are routed to).  Counters must be zero before the first launch; every
 *   launch leaves them zero.  Launches that share scratch must not overlap on the GPU.
 * moe_small_m_gemm (gemm1 = 1): a = x [num_tokens, K] in act dtype (FP8 mode: quantised
 *   1 x 128 inside the kernel), w = w1 [E, 2*Nout, K], out = intermediate [rows_cap, Nout] in
 *   act dtype, sorted order.  (gemm1 = 0): a = that intermediate (K = intermediate size),
 *   w = w2 [E, Nout, K], out = y [num_tokens * topk, Nout] scratch in act dtype,
 *   final_out = layer output [num_tokens, Nout]; rows of tokens without a valid route are
 *   zeroed.  sorted_ids / expert_ids / num_post_pad come from moe_align_block_size with
 *   block_size 8 and the GLOBAL expert count; expert_map (or NULL) maps global to local ids.
 *   w_scale as in moe_gemm1 / moe_gemm2.  Limits: topk <= 32, Nout % 64 (GEMM 1) / % 128
 *   (GEMM 2), K a multiple of 128 bytes of weights (and of 128 elements in FP8 mode).
 */
int moe_small_m_plan(int gemm1, int mode, int K, int Nout, int64_t rows_cap, int64_t num_tokens, int k_slices,
                     int64_t* partial_floats, int64_t* unit_counters, int64_t* token_counters);
int moe_small_m_gemm(int gemm1, int mode, int act_dtype, const void* a, int64_t num_tokens, int topk,
                     const void* w, const float* w_scale, const int32_t* expert_ids, const int32_t* sorted_ids,
                     const int32_t* num_post_pad, const int32_t* expert_map, int num_experts_global,
                     const float* route_weight, int mul_weight, const void* topk_ids, int ids_int64,
                     int64_t rows_cap, int E, int K, int Nout, void* out, void* final_out, int k_slices,
                     float* partial, int32_t* unit_counters, int32_t* token_counters, int32_t* status, void* stream);

/*
 * GEMM 2 of the small-batch schedule without any allocation by anyone: same inputs and output
 * as moe_small_m_gemm(gemm1 = 0, ...), but the route rows y, the partial sums and both counter
 * tables live in a fixed 8 MiB array inside the library's device image instead of in buffers
 * the caller would have to allocate.  It is for hosts that cannot get device memory at call
 * time: an engine whose pools already own all of it, or a decode loop that must not run
 * cudaMalloc / cudaFree (both stall the device).  This entry point has no counterpart in the
 * reference, which allocates its intermediates with torch on every call.
 *   - A call that needs more scratch than the array holds returns MOE_E_TOOBIG (the message
 *     gives both sizes) and launches nothing.
 *   - The first call on a device resolves the array's device address; make it before any
 *     stream capture.  Calls share the array: the counters are cleared on `stream` at the start
 *     of each call, everything else is written before it is read, and calls whose kernels
 *     overlap on the GPU race on it.
 */
int moe_small_m_gemm2_static(int mode, int act_dtype, const void* act_sorted, int64_t num_tokens, int topk,
                             const void* w2, const float* w2_scale, const int32_t* expert_ids,
                             const int32_t* sorted_ids, const int32_t* num_post_pad, const int32_t* expert_map,
                             int num_experts_global, const float* route_weight, int mul_weight, const void* topk_ids,
                             int ids_int64, int64_t rows_cap, int E, int K, int Nout, void* final_out, int k_slices,
                             int32_t* status, void* stream);

/*
 * out[m, :] = sum_j in[m, j, :] in fp32, fixed order j = 0..topk-1, stored in
 * the io dtype.  Stands in for moe_sum (src/flaggems_vllm/ops/moe_sum.py:250-310).
 * When topk_ids is given, slot j is skipped if its id is outside
 * [0, num_experts) or expert_map[id] < 0 (expert-parallel ranks).
 * When row_index is given, the row of slot (m, j) is in[row_index[m*topk + j]]
 * instead of in[m*topk + j], and a negative index skips the slot (used after the
 * expert-parallel combine, where the returned rows are ordered by the rank that
 * computed them and a token has no row from ranks it sent nothing to).
 */
int moe_sum(const void* in, void* out, int dtype, int64_t M, int topk, int64_t H,
            const void* topk_ids, int ids_int64, int num_experts, const int32_t* expert_map,
            const int32_t* row_index, void* stream);

/* moe_sum with the rows of `out` out_ld elements apart (out_ld >= H): the sum lands in a column
 * window of a wider tensor. */
int moe_sum_ld(const void* in, void* out, int64_t out_ld, int dtype, int64_t M, int topk, int64_t H,
               const void* topk_ids, int ids_int64, int num_experts, const int32_t* expert_map,
               const int32_t* row_index, void* stream);

/*
 * out[i] = SiLU(a[i]) * b[i] in fp32, rounded once to the tensors' dtype (F32/F16/BF16), n
 * contiguous elements; and its gradients da = dSiLU(a) * dgrad * b, db = dgrad * SiLU(a).
 * Stand in for silu_and_mul / silu_and_mul_out (src/flaggems_vllm/ops/silu_and_mul.py:26-70).
 */
int moe_silu_and_mul(const void* a, const void* b, void* out, int dtype, int64_t n, void* stream);
int moe_silu_and_mul_grad(const void* a, const void* b, const void* dgrad, void* da, void* db, int dtype, int64_t n,
                          void* stream);

/*
 * Expert-parallel bookkeeping (experts partitioned over `world` ranks, rank r owning experts
 * [r * experts_per_rank, (r + 1) * experts_per_rank); tokens data-parallel).  The reference
 * has no all-to-all path (its hook is expert_map with replicated tokens,
 * src/flaggems_vllm/ops/fused_moe.py:2553-2560); these three calls have no counterpart there.
 *
 * moe_ep_plan: the (token, destination rank) pairs of topk_ids [M, k] int32 (negative ids are
 *   no route), ordered by rank, then token.  index [M, world]: position of the pair or -1;
 *   counts [world]: pairs per rank; tok [M * world]: token of every pair (first sum(counts)
 *   entries).  world <= 16.
 * moe_ep_pack: send buffers of the dispatch: rows_out [pairs, row_bytes] = rows[tok[p]] and
 *   side_out [pairs, groups + 2k] fp32 = [scales[tok[p]] (groups) | expert ids | weights].
 *   scales [M, groups] row-major (groups = 0: none); topk_weights fp32.
 * moe_ep_unpack: the receiver's view of side rows: scales_t [groups, rows] (transposed),
 *   slot_ids [rows, k] = id - rank * experts_per_rank when this rank owns the expert, else -1,
 *   slot_w [rows, k].
 */
int moe_ep_plan(const int32_t* topk_ids, int64_t M, int k, int experts_per_rank, int world, int32_t* index,
                int32_t* counts, int32_t* tok, void* stream);
int moe_ep_pack(const void* rows, int64_t row_bytes, const float* scales, int groups, const int32_t* topk_ids,
                const float* topk_weights, int k, const int32_t* tok, int64_t pairs, void* rows_out, float* side_out,
                void* stream);
int moe_ep_unpack(const float* side, int64_t rows, int groups, int k, int rank, int experts_per_rank,
                  float* scales_t, int32_t* slot_ids, float* slot_w, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOE_SM100_H_ */
