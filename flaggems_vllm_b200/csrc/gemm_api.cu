// C ABI of the two expert grouped GEMMs: argument checks and the choice
// between the tcgen05 kernel and the generic kernel.
#include "tc_common.cuh"

namespace moe {
int simt_gemm(bool gemm1, int mode, int act_dtype, const void* a, const float* a_scales_t, const void* w,
              const float* w_scale, const int32_t* expert_ids, const int32_t* sorted_ids, const int32_t* npp,
              const float* route_weight, int mul_weight, int64_t numel, int64_t rows_cap, int64_t a_tokens, int topk,
              int block_m, int E, int K, int Nout, void* out, float* out_scales_t, int32_t* status, cudaStream_t st,
              int act_kind = MOE_ACT_SILU, float alpha = 0.0f, float beta = 0.0f, float limit = 0.0f);
int tc_gemm(bool gemm1, int mode, int act_dtype, const void* a, const float* a_scales_t, const void* w,
            const float* w_scale, const int32_t* expert_ids, const int32_t* sorted_ids, const int32_t* npp,
            const float* route_weight, int mul_weight, int64_t numel, int64_t rows_cap, int64_t a_tokens, int topk,
            int block_m, int E, int K, int Nout, void* out, float* out_scales_t, int32_t* status, cudaStream_t st,
            int variant, int a_sorted, int32_t* inv = nullptr, int w_row0 = 0, int w_rows = 0, int grid_limit = 0);
int w8_gemm(bool gemm1, int act_dtype, const void* a, const void* w, const float* w_scale, const int32_t* expert_ids,
            const int32_t* sorted_ids, const int32_t* npp, const float* route_weight, int mul_weight, int64_t numel,
            int64_t rows_cap, int64_t a_tokens, int topk, int block_m, int E, int K, int Nout, void* out,
            int32_t* status, cudaStream_t st);

static int check_common(const char* who, int mode, const void* a, const float* a_scales, const void* w,
                        const float* w_scale, const int32_t* expert_ids, const int32_t* sorted_ids,
                        const int32_t* npp, const float* route_weight, int mul_weight, int64_t numel,
                        int64_t rows_cap, int block_m, int E, int H, int I, const void* out) {
  if (numel < 0 || rows_cap < 0 || block_m <= 0 || E <= 0 || H <= 0 || I <= 0)
    return fail(MOE_E_BADARG, "%s: bad extent", who);
  if (!a || !w || !expert_ids || !sorted_ids || !npp || !out) return fail(MOE_E_BADARG, "%s: null pointer", who);
  if (mul_weight && !route_weight) return fail(MOE_E_BADARG, "%s: route weights missing", who);
  if ((mode == MOE_MODE_FP8_BLOCK || mode == MOE_MODE_FP8_ROW || mode == MOE_MODE_INT8_ROW) && (!a_scales || !w_scale))
    return fail(MOE_E_BADARG, "%s: scales missing", who);
  if (mode == MOE_MODE_W8A16 && !w_scale) return fail(MOE_E_BADARG, "%s: weight scales missing", who);
  return 0;
}
}  // namespace moe

extern "C" int moe_gemm1(int mode, int act_dtype, const void* a, int a_sorted, const float* a_scales_t,
                         int64_t num_tokens,
                         int topk, const void* w1, const float* w1_scale, const int32_t* expert_ids,
                         const int32_t* sorted_ids, const int32_t* num_post_pad, const float* route_weight,
                         int mul_weight, int64_t rows_cap, int block_m, int E, int H, int I, void* out,
                         float* out_scales_t, int use_tensor_cores, int32_t* status, void* stream) {
  return moe_gemm1_ex(mode, act_dtype, a, a_sorted, a_scales_t, num_tokens, topk, w1, w1_scale, expert_ids, sorted_ids,
                      num_post_pad, route_weight, mul_weight, rows_cap, block_m, E, H, I, out, out_scales_t,
                      use_tensor_cores, MOE_ACT_SILU, 0.0f, 0.0f, 0.0f, status, stream);
}

extern "C" int moe_gemm1_ex(int mode, int act_dtype, const void* a, int a_sorted, const float* a_scales_t,
                            int64_t num_tokens, int topk, const void* w1, const float* w1_scale,
                            const int32_t* expert_ids, const int32_t* sorted_ids, const int32_t* num_post_pad,
                            const float* route_weight, int mul_weight, int64_t rows_cap, int block_m, int E, int H,
                            int I, void* out, float* out_scales_t, int use_tensor_cores, int activation, float alpha,
                            float beta, float limit, int32_t* status, void* stream) {
  using namespace moe;
  if (activation != MOE_ACT_SILU && activation != MOE_ACT_SWIGLUOAI) return fail(MOE_E_BADARG, "gemm1: unknown activation %d", activation);
  if (use_tensor_cores && (activation != MOE_ACT_SILU || mode == MOE_MODE_FP8_ROW || mode == MOE_MODE_INT8_ROW))
    return fail(MOE_E_SHAPE, "gemm1: the row-scaled modes and activations other than SiLU are served by the generic kernel");
  if (num_tokens < 0 || topk <= 0) return fail(MOE_E_BADARG, "gemm1: bad token count or topk");
  const int64_t numel = num_tokens * topk;
  int rc = check_common("gemm1", mode, a, a_scales_t, w1, w1_scale, expert_ids, sorted_ids, num_post_pad,
                        route_weight, mul_weight, numel, rows_cap, block_m, E, H, I, out);
  if (rc) return rc;
  if (mode == MOE_MODE_FP8_BLOCK && !out_scales_t) return fail(MOE_E_BADARG, "gemm1: output scale buffer missing");
  if (rows_cap == 0 || numel == 0) return 0;
  if (a_sorted && !((mode == MOE_MODE_HALF && (use_tensor_cores == 1 || use_tensor_cores == 3)) ||
                    (mode == MOE_MODE_FP8_BLOCK && (use_tensor_cores == 1 || use_tensor_cores == 2))))
    return fail(MOE_E_SHAPE, "gemm1: pre-sorted rows are read by the tensor-core kernels 1 (half, fp8) and 3 (half) only");
  if (use_tensor_cores && mode == MOE_MODE_W8A16)  // int8 weights widened inside the kernel
    return w8_gemm(true, act_dtype, a, w1, w1_scale, expert_ids, sorted_ids, num_post_pad, route_weight, mul_weight,
                   numel, rows_cap, num_tokens, topk, block_m, E, H, I, out, status, (cudaStream_t)stream);
  if (use_tensor_cores)
    return tc_gemm(true, mode, act_dtype, a, a_scales_t, w1, w1_scale, expert_ids, sorted_ids, num_post_pad,
                   route_weight, mul_weight, numel, rows_cap, num_tokens, topk, block_m, E, H, I, out, out_scales_t,
                   status, (cudaStream_t)stream, use_tensor_cores, a_sorted);
  return simt_gemm(true, mode, act_dtype, a, a_scales_t, w1, w1_scale, expert_ids, sorted_ids, num_post_pad,
                   route_weight, mul_weight, numel, rows_cap, num_tokens, topk, block_m, E, H, I, out, out_scales_t,
                   status, (cudaStream_t)stream, activation, alpha, beta, limit);
}

extern "C" int moe_gemm2(int mode, int act_dtype, const void* act_sorted, const float* act_scales_t, const void* w2,
                         const float* w2_scale, const int32_t* expert_ids, const int32_t* sorted_ids,
                         const int32_t* num_post_pad, const float* route_weight, int mul_weight, int64_t numel,
                         int64_t rows_cap, int block_m, int E, int H, int I, void* y, int use_tensor_cores,
                         int32_t* status, void* stream) {
  using namespace moe;
  int rc = check_common("gemm2", mode, act_sorted, act_scales_t, w2, w2_scale, expert_ids, sorted_ids, num_post_pad,
                        route_weight, mul_weight, numel, rows_cap, block_m, E, H, I, y);
  if (rc) return rc;
  if (rows_cap == 0 || numel == 0) return 0;
  if (use_tensor_cores && (mode == MOE_MODE_FP8_ROW || mode == MOE_MODE_INT8_ROW))
    return fail(MOE_E_SHAPE, "gemm2: the row-scaled modes are served by the generic kernel");
  if (use_tensor_cores && mode == MOE_MODE_W8A16)
    return w8_gemm(false, act_dtype, act_sorted, w2, w2_scale, expert_ids, sorted_ids, num_post_pad, route_weight,
                   mul_weight, numel, rows_cap, 0, 1, block_m, E, I, H, y, status, (cudaStream_t)stream);
  if (use_tensor_cores)
    return tc_gemm(false, mode, act_dtype, act_sorted, act_scales_t, w2, w2_scale, expert_ids, sorted_ids,
                   num_post_pad, route_weight, mul_weight, numel, rows_cap, 0, 1, block_m, E, I, H, y, nullptr, status,
                   (cudaStream_t)stream, use_tensor_cores, 0);
  return simt_gemm(false, mode, act_dtype, act_sorted, act_scales_t, w2, w2_scale, expert_ids, sorted_ids,
                   num_post_pad, route_weight, mul_weight, numel, rows_cap, 0, 1, block_m, E, I, H, y, nullptr, status,
                   (cudaStream_t)stream);
}

namespace moe {
// One warp waits on a barrier nobody arrives at, with the given limit; the wait gives up, sets
// MOE_ST_WAIT_TIMEOUT and the kernel returns.  Nothing faults and nothing waits without a bound.
__global__ void wait_timeout_probe_kernel(int32_t* status, unsigned long long limit_ns, int32_t* gave_up) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const bool ok = tc::mbar_wait(&bar, 0, status, limit_ns);
  if (threadIdx.x == 0 && gave_up != nullptr) *gave_up = ok ? 0 : 1;
}
}  // namespace moe

extern "C" int moe_debug_wait_timeout(int32_t* status, unsigned long long limit_ns, int32_t* gave_up, void* stream) {
  using namespace moe;
  if (limit_ns == 0 || limit_ns > 100000000ull) return fail(MOE_E_BADARG, "debug_wait_timeout: limit must be 1 ns .. 100 ms");
  wait_timeout_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, limit_ns, gave_up);
  return check_launch("debug_wait_timeout");
}

extern "C" int moe_gemm2_sorted(int mode, int act_dtype, const void* act_sorted, const float* act_scales_t, const void* w2,
                                const float* w2_scale, const int32_t* expert_ids, const int32_t* sorted_ids,
                                const int32_t* num_post_pad, const float* route_weight, int mul_weight, int64_t numel,
                                int64_t rows_cap, int block_m, int E, int H, int I, void* y_sorted, int32_t* inv,
                                int32_t* status, void* stream) {
  using namespace moe;
  int rc = check_common("gemm2 (sorted output)", mode, act_sorted, act_scales_t, w2, w2_scale, expert_ids, sorted_ids,
                        num_post_pad, route_weight, mul_weight, numel, rows_cap, block_m, E, H, I, y_sorted);
  if (rc) return rc;
  if (!inv) return fail(MOE_E_BADARG, "gemm2 (sorted output): route index buffer missing");
  if (mode != MOE_MODE_FP8_BLOCK && mode != MOE_MODE_HALF)
    return fail(MOE_E_SHAPE, "gemm2 (sorted output): FP8 block-scale and half-precision modes only");
  if (rows_cap == 0 || numel == 0) return 0;
  return tc_gemm(false, mode, act_dtype, act_sorted, act_scales_t, w2, w2_scale, expert_ids, sorted_ids, num_post_pad,
                 route_weight, mul_weight, numel, rows_cap, 0, 1, block_m, E, I, H, y_sorted, nullptr, status,
                 (cudaStream_t)stream, 1, 0, inv);
}

// moe_gemm2_sorted over a window of the output columns [col0, col0 + ncols) of H: y_window is
// [rows_cap, ncols].  A caller that has other work for the first columns (an expert-parallel
// combine that can start on them) runs the layer's GEMM 2 as two such calls; max_ctas > 0 leaves
// the remaining SMs to that other work.
extern "C" int moe_gemm2_sorted_cols(int mode, int act_dtype, const void* act_sorted, const float* act_scales_t,
                                     const void* w2, const float* w2_scale, const int32_t* expert_ids,
                                     const int32_t* sorted_ids, const int32_t* num_post_pad, const float* route_weight,
                                     int mul_weight, int64_t numel, int64_t rows_cap, int block_m, int E, int H, int I,
                                     int col0, int ncols, void* y_window, int32_t* inv, int max_ctas, int32_t* status,
                                     void* stream) {
  using namespace moe;
  int rc = check_common("gemm2 (column window)", mode, act_sorted, act_scales_t, w2, w2_scale, expert_ids, sorted_ids,
                        num_post_pad, route_weight, mul_weight, numel, rows_cap, block_m, E, H, I, y_window);
  if (rc) return rc;
  if (!inv) return fail(MOE_E_BADARG, "gemm2 (column window): route index buffer missing");
  if (mode != MOE_MODE_FP8_BLOCK && mode != MOE_MODE_HALF)
    return fail(MOE_E_SHAPE, "gemm2 (column window): FP8 block-scale and half-precision modes only");
  if (col0 < 0 || ncols <= 0 || col0 + ncols > H) return fail(MOE_E_BADARG, "gemm2 (column window): window outside [0, H)");
  if (rows_cap == 0 || numel == 0) return 0;
  return tc_gemm(false, mode, act_dtype, act_sorted, act_scales_t, w2, w2_scale, expert_ids, sorted_ids, num_post_pad,
                 route_weight, mul_weight, numel, rows_cap, 0, 1, block_m, E, I, ncols, y_window, nullptr, status,
                 (cudaStream_t)stream, 1, 0, inv, col0, H, max_ctas);
}
