// Non-grouped top-k routers: softmax or sigmoid scores, optional selection bias,
// optional padding rows, in-place outputs.  One warp per token, the same
// ordering rule and packed keys as grouped_topk (higher value first, ties to the
// lower expert index), no scratch.
//
// Semantics follow the reference's routing kernel and its test goldens
// (src/flaggems_vllm/ops/topk_sigmoid.py:17-83, tests/test_topk_sigmoid.py:11-24,
// tests/test_topk_softmax.py:146-156):
//   p = softmax(logits) or sigmoid(logits), NaN -> 0; a softmax row holding a
//   NaN or +inf is all zeros;  choice = p + bias;  pick the k largest choices;
//   weight = p[id], divided by their sum when renormalising (sum > 0),
//   times the scaling factor;  padded rows: weight 0, id -1;
//   token_expert_indices[m, j] = j * M + m.
// Scores are evaluated in double and rounded once to fp32, so the ranking is
// reproducible bit for bit by a CPU check that does the same.
#include "moe_common.cuh"

namespace moe {
namespace {

__device__ __forceinline__ uint32_t tr_ordered_bits(float v) {
  uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ uint64_t tr_key(float v, uint32_t idx) {
  return ((uint64_t)tr_ordered_bits(v) << 32) | (uint64_t)(0xFFFFFFFFu - idx);
}
__device__ __forceinline__ uint64_t tr_warp_max(uint64_t k) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    uint64_t o = __shfl_xor_sync(0xFFFFFFFFu, k, off);
    k = o > k ? o : k;
  }
  return k;
}

template <typename LT, typename IT, int VPT>
__global__ void __launch_bounds__(128) topk_route_kernel(
    const LT* __restrict__ logits, const float* __restrict__ bias, const uint8_t* __restrict__ is_padding,
    int64_t M, int E, int topk, int sigmoid, int renormalize, float scale, float* __restrict__ out_w,
    IT* __restrict__ out_ids, int32_t* __restrict__ out_src) {
  const int lane = threadIdx.x & 31;
  const int64_t token = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= M) return;
  const bool padded = is_padding != nullptr && is_padding[token];
  const LT* row = logits + token * E;

  double x[VPT];
  bool bad = false;  // softmax: NaN or +inf anywhere zeroes the row
  double mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int e = j * 32 + lane;
    x[j] = e < E ? (double)ToF32<LT>::get(row[e]) : -INFINITY;
    if (e < E) {
      if (x[j] != x[j] || x[j] == INFINITY) bad = true;
      mx = fmax(mx, x[j]);
    }
  }
  float p[VPT];
  if (sigmoid) {
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      float v = (float)(1.0 / (1.0 + exp(-x[j])));
      p[j] = (v == v) ? v : 0.0f;
    }
  } else {
    bad = __any_sync(0xFFFFFFFFu, bad);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) mx = fmax(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, off));
    double ex[VPT], sum = 0.0;
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      ex[j] = (j * 32 + lane < E && !bad && mx > -INFINITY) ? exp(x[j] - mx) : 0.0;
      sum += ex[j];
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
#pragma unroll
    for (int j = 0; j < VPT; ++j) p[j] = sum > 0.0 ? (float)(ex[j] / sum) : 0.0f;
  }

  uint64_t key[VPT];
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int e = j * 32 + lane;
    key[j] = e < E ? tr_key(bias != nullptr ? p[j] + bias[e] : p[j], (uint32_t)e) : 0;
  }
  float my_w = 0.0f;
  uint32_t my_id = 0;
  uint64_t local = 0;
  int local_j = 0;
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    if (key[j] > local) { local = key[j]; local_j = j; }
  for (int t = 0; t < topk; ++t) {
    const uint64_t best = tr_warp_max(local);
    const uint32_t id = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFu);
    float wsel = 0.0f;
    if (local == best && best != 0) {
#pragma unroll
      for (int j = 0; j < VPT; ++j)
        if (j == local_j) { wsel = p[j]; key[j] = 0; }
      local = 0;
#pragma unroll
      for (int j = 0; j < VPT; ++j)
        if (key[j] > local) { local = key[j]; local_j = j; }
    }
    wsel = __shfl_sync(0xFFFFFFFFu, wsel, id & 31);
    if (lane == t) { my_w = wsel; my_id = id; }
  }
  float sum = lane < topk ? my_w : 0.0f;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
  if (lane < topk) {
    float w = my_w;
    if (renormalize) w = w / (sum > 0.0f ? sum : 1.0f);
    w *= scale;
    const int64_t o = token * topk + lane;
    out_w[o] = padded ? 0.0f : w;
    out_ids[o] = padded ? (IT)-1 : (IT)my_id;
    out_src[o] = (int32_t)((int64_t)lane * M + token);
  }
}

template <typename LT, typename IT>
int launch_vpt(const LT* logits, const float* bias, const uint8_t* pad, int64_t M, int E, int topk, int sigmoid,
               int renorm, float scale, float* w, IT* ids, int32_t* src, cudaStream_t st) {
  const int warps = 4;
  dim3 grid((unsigned)((M + warps - 1) / warps)), block(warps * 32);
#define MOE_TR_LAUNCH(V) \
  topk_route_kernel<LT, IT, V><<<grid, block, 0, st>>>(logits, bias, pad, M, E, topk, sigmoid, renorm, scale, w, ids, src)
  if (E <= 32) MOE_TR_LAUNCH(1);
  else if (E <= 64) MOE_TR_LAUNCH(2);
  else if (E <= 128) MOE_TR_LAUNCH(4);
  else if (E <= 256) MOE_TR_LAUNCH(8);
  else if (E <= 512) MOE_TR_LAUNCH(16);
  else MOE_TR_LAUNCH(32);
#undef MOE_TR_LAUNCH
  return check_launch("topk_route");
}

template <typename LT>
int launch_idx(const LT* logits, const float* bias, const uint8_t* pad, int64_t M, int E, int topk, int sigmoid,
               int renorm, float scale, float* w, void* ids, int index_kind, int32_t* src, cudaStream_t st) {
  switch (index_kind) {
    case 0: return launch_vpt(logits, bias, pad, M, E, topk, sigmoid, renorm, scale, w, (int32_t*)ids, src, st);
    case 1: return launch_vpt(logits, bias, pad, M, E, topk, sigmoid, renorm, scale, w, (int64_t*)ids, src, st);
    case 2: return launch_vpt(logits, bias, pad, M, E, topk, sigmoid, renorm, scale, w, (uint32_t*)ids, src, st);
    default: return fail(MOE_E_DTYPE, "topk_route: index kind must be 0 (int32), 1 (int64) or 2 (uint32)");
  }
}

}  // namespace
}  // namespace moe

extern "C" int moe_topk_route(const void* logits, int logits_dtype, const float* bias, const uint8_t* is_padding,
                              int64_t M, int E, int topk, int sigmoid, int renormalize, float scale,
                              float* topk_weights, void* topk_indices, int index_kind,
                              int32_t* token_expert_indices, void* stream) {
  using namespace moe;
  if (M < 0 || E <= 0 || topk <= 0) return fail(MOE_E_BADARG, "topk_route: non-positive extent");
  if (E > 1024) return fail(MOE_E_TOOBIG, "topk_route: at most 1024 experts (got %d)", E);
  if (topk > 32 || topk > E) return fail(MOE_E_SHAPE, "topk_route: topk must be <= min(32, experts)");
  if (M == 0) return 0;
  if (!logits || !topk_weights || !topk_indices || !token_expert_indices)
    return fail(MOE_E_BADARG, "topk_route: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  switch (logits_dtype) {
    case MOE_F32:
      return launch_idx((const float*)logits, bias, is_padding, M, E, topk, sigmoid, renormalize, scale, topk_weights,
                        topk_indices, index_kind, token_expert_indices, st);
    case MOE_F16:
      return launch_idx((const __half*)logits, bias, is_padding, M, E, topk, sigmoid, renormalize, scale,
                        topk_weights, topk_indices, index_kind, token_expert_indices, st);
    case MOE_BF16:
      return launch_idx((const __nv_bfloat16*)logits, bias, is_padding, M, E, topk, sigmoid, renormalize, scale,
                        topk_weights, topk_indices, index_kind, token_expert_indices, st);
    default:
      return fail(MOE_E_DTYPE, "topk_route: unsupported logits dtype %d", logits_dtype);
  }
}
