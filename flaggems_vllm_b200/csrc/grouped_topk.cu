// Group-limited top-k routing: one warp per token, shuffle reductions only,
// no scratch memory.
//
// Per token (fp32 throughout, as the reference's fast kernels compute it,
// src/flaggems_vllm/ops/grouped_topk.py:333-794):
//   u = sigmoid(score) or score;  r = u + bias
//   group score = sum of the two largest r in the group
//   keep the topk_group best groups, then pick the topk largest r among them
//   weight = u[id] (/ (sum + 1e-20) when renormalising) * scaling factor
// Every "largest" uses one ordering: higher value first, equal values -> lower
// index first.  It is implemented, like the reference's packed keys
// (:310-317), as an unsigned 64-bit key (order-preserving image of the fp32
// bits) << 32 | (0xFFFFFFFF - index), reduced with max.
//
// Expert e lives in lane e % 32, register e / 32, so loads are coalesced.
// The sigmoid is evaluated in double and rounded once to fp32, which makes
// the result the correctly rounded fp32 sigmoid and therefore reproducible
// bit for bit by a CPU check that does the same.
#include "moe_common.cuh"

namespace moe {
namespace {

__device__ __forceinline__ uint32_t ordered_bits(float v) {
  uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ uint64_t make_key(float v, uint32_t idx) {
  return ((uint64_t)ordered_bits(v) << 32) | (uint64_t)(0xFFFFFFFFu - idx);
}
// max of a 64-bit key over the warp with two 32-bit reductions (redux.sync): the largest high
// word, then the largest low word among the lanes that hold it
__device__ __forceinline__ uint64_t warp_max_u64(uint64_t k) {
  const uint32_t hi = (uint32_t)(k >> 32), lo = (uint32_t)k;
  const uint32_t mh = __reduce_max_sync(0xFFFFFFFFu, hi);
  const uint32_t ml = __reduce_max_sync(0xFFFFFFFFu, hi == mh ? lo : 0u);
  return ((uint64_t)mh << 32) | ml;
}
__device__ __forceinline__ float from_ordered_bits(uint32_t ob) {
  return __uint_as_float((ob & 0x80000000u) ? (ob ^ 0x80000000u) : ~ob);
}

// The routing of one token by one warp: `row` holds the token's E scores (element stride
// `stride1`; global or shared memory), the results go to w_row / id_row [topk].
template <typename ST, typename BT, int VPT>
__device__ __forceinline__ void route_row(const ST* row, int64_t stride1, const BT* __restrict__ bias, int E,
                                          int n_group, int topk_group, int topk, int renormalize, float scaling,
                                          int scoring_func, float* w_row, int32_t* id_row, int lane) {
  const int per_group = E / n_group;
  const float NEG_INF = __int_as_float(0xff800000);

  float u[VPT];      // unbiased score
  uint64_t key[VPT]; // ranking key of u + bias (0 = absent / consumed)
#pragma unroll
  for (int j = 0; j < VPT; ++j) {
    const int e = j * 32 + lane;
    if (e < E) {
      float s = ToF32<ST>::get(row[(int64_t)e * stride1]);
      if (scoring_func == 1) s = (float)(1.0 / (1.0 + exp(-(double)s)));
      u[j] = s;
      key[j] = make_key(s + ToF32<BT>::get(bias[e]), (uint32_t)e);
    } else {
      u[j] = 0.0f;
      key[j] = 0;
    }
  }

  if (n_group > 1) {
    // group of every register of this lane, computed once (-1: no expert)
    int grp[VPT];
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = j * 32 + lane;
      grp[j] = e < E ? e / per_group : -1;
    }
    // group score -> lane g holds the score of group g.  The two largest r of a group are found
    // on the order-preserving integer image of r (the key's high word; 0 = none): the lane's own
    // two, then the warp's largest, then the largest of what is left once its owner gave it up.
    float my_group_score = NEG_INF;
    for (int g = 0; g < n_group; ++g) {
      uint32_t b1 = 0, b2 = 0;
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        if (grp[j] == g) {
          const uint32_t ob = (uint32_t)(key[j] >> 32);
          if (ob > b1) { b2 = b1; b1 = ob; } else if (ob > b2) { b2 = ob; }
        }
      }
      const uint32_t top1 = __reduce_max_sync(0xFFFFFFFFu, b1);
      const int owner = __ffs(__ballot_sync(0xFFFFFFFFu, b1 == top1)) - 1;
      const uint32_t top2 = __reduce_max_sync(0xFFFFFFFFu, lane == owner ? b2 : b1);
      const float gs = per_group >= 2 ? from_ordered_bits(top1) + from_ordered_bits(top2) : from_ordered_bits(top1);
      if (lane == g) my_group_score = gs;
    }
    // choose topk_group groups
    uint32_t keep_mask = 0;
    uint64_t gkey = lane < n_group ? make_key(my_group_score, (uint32_t)lane) : 0;
    for (int t = 0; t < topk_group; ++t) {
      uint64_t best = warp_max_u64(gkey);
      uint32_t g = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFu);
      keep_mask |= 1u << (g & 31);
      if (gkey == best) gkey = 0;
    }
    // experts of dropped groups rank as -inf (still ordered by index)
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int e = j * 32 + lane;
      if (grp[j] >= 0 && !((keep_mask >> grp[j]) & 1u)) key[j] = make_key(NEG_INF, (uint32_t)e);
    }
  }

  // top-k extraction
  float my_w = 0.0f;
  int32_t my_id = 0;
  uint64_t local = 0;
  int local_j = 0;
#pragma unroll
  for (int j = 0; j < VPT; ++j)
    if (key[j] > local) { local = key[j]; local_j = j; }
  for (int t = 0; t < topk; ++t) {
    uint64_t best = warp_max_u64(local);
    uint32_t id = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFu);
    float wsel = 0.0f;
    if (local == best && best != 0) {
      // this lane owns the winner: fetch its unbiased value, consume it
#pragma unroll
      for (int j = 0; j < VPT; ++j)
        if (j == local_j) { wsel = u[j]; key[j] = 0; }
      local = 0;
#pragma unroll
      for (int j = 0; j < VPT; ++j)
        if (key[j] > local) { local = key[j]; local_j = j; }
    }
    wsel = __shfl_sync(0xFFFFFFFFu, wsel, id & 31);
    if (lane == t) { my_w = wsel; my_id = (int32_t)id; }
  }
  float sum = lane < topk ? my_w : 0.0f;
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
  if (lane < topk) {
    float w = renormalize ? my_w / (sum + 1e-20f) : my_w;
    w_row[lane] = w * scaling;
    id_row[lane] = my_id;
  }
}

template <typename ST, typename BT, int VPT>
__global__ void __launch_bounds__(128) grouped_topk_kernel(
    const ST* __restrict__ scores, int64_t stride0, int64_t stride1, const BT* __restrict__ bias,
    const uint8_t* __restrict__ is_padding, int64_t M, int E, int n_group, int topk_group, int topk,
    int renormalize, float scaling, int scoring_func, float* __restrict__ out_w,
    int32_t* __restrict__ out_ids) {
  const int lane = threadIdx.x & 31;
  const int64_t token = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (token >= M) return;
  float* w_row = out_w + token * topk;
  int32_t* id_row = out_ids + token * topk;
  if (is_padding != nullptr && is_padding[token]) {
    if (lane < topk) {
      w_row[lane] = 0.0f;
      id_row[lane] = -1;
    }
    return;
  }
  route_row<ST, BT, VPT>(scores + token * stride0, stride1, bias, E, n_group, topk_group, topk, renormalize, scaling,
                         scoring_func, w_row, id_row, lane);
}

// The same routing for more experts than a warp's registers hold (1024 < E <= 4096): one CTA of
// 256 threads per token, the unbiased scores and the ranking keys in shared memory.  The same
// ordering rules and the same arithmetic as route_row, so the ids agree with it wherever both
// apply.  A correctness path for unusually wide routers, not a tuned one.
template <typename ST, typename BT>
__global__ void __launch_bounds__(256) grouped_topk_big_kernel(
    const ST* __restrict__ scores, int64_t stride0, int64_t stride1, const BT* __restrict__ bias,
    const uint8_t* __restrict__ is_padding, int64_t M, int E, int n_group, int topk_group, int topk,
    int renormalize, float scaling, int scoring_func, float* __restrict__ out_w, int32_t* __restrict__ out_ids) {
  extern __shared__ unsigned long long big_smem[];
  uint64_t* key = reinterpret_cast<uint64_t*>(big_smem);                 // [E]
  float* u = reinterpret_cast<float*>(key + E);                          // [E]
  __shared__ uint64_t warp_best[8];
  __shared__ uint64_t best_bc;
  __shared__ float group_score[32];
  __shared__ uint32_t keep_mask_s;
  const int64_t token = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float* w_row = out_w + token * topk;
  int32_t* id_row = out_ids + token * topk;
  if (is_padding != nullptr && is_padding[token]) {
    if (tid < topk) { w_row[tid] = 0.0f; id_row[tid] = -1; }
    return;
  }
  const float NEG_INF = __int_as_float(0xff800000);
  const int per_group = E / n_group;
  const ST* row = scores + token * stride0;
  for (int e = tid; e < E; e += 256) {
    float s = ToF32<ST>::get(row[(int64_t)e * stride1]);
    if (scoring_func == 1) s = (float)(1.0 / (1.0 + exp(-(double)s)));
    u[e] = s;
    key[e] = make_key(s + ToF32<BT>::get(bias[e]), (uint32_t)e);
  }
  __syncthreads();
  if (n_group > 1) {
    for (int g = warp; g < n_group; g += 8) {  // a warp finds the two largest r of its groups
      uint32_t b1 = 0, b2 = 0;
      for (int e = g * per_group + lane; e < (g + 1) * per_group; e += 32) {
        const uint32_t ob = (uint32_t)(key[e] >> 32);
        if (ob > b1) { b2 = b1; b1 = ob; } else if (ob > b2) { b2 = ob; }
      }
      const uint32_t top1 = __reduce_max_sync(0xFFFFFFFFu, b1);
      const int owner = __ffs(__ballot_sync(0xFFFFFFFFu, b1 == top1)) - 1;
      const uint32_t top2 = __reduce_max_sync(0xFFFFFFFFu, lane == owner ? b2 : b1);
      if (lane == 0)
        group_score[g] = per_group >= 2 ? from_ordered_bits(top1) + from_ordered_bits(top2) : from_ordered_bits(top1);
    }
    __syncthreads();
    if (warp == 0) {
      uint32_t keep_mask = 0;
      uint64_t gkey = lane < n_group ? make_key(group_score[lane], (uint32_t)lane) : 0;
      for (int t = 0; t < topk_group; ++t) {
        const uint64_t best = warp_max_u64(gkey);
        keep_mask |= 1u << ((0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFu)) & 31);
        if (gkey == best) gkey = 0;
      }
      if (lane == 0) keep_mask_s = keep_mask;
    }
    __syncthreads();
    const uint32_t keep_mask = keep_mask_s;
    for (int e = tid; e < E; e += 256)
      if (!((keep_mask >> (e / per_group)) & 1u)) key[e] = make_key(NEG_INF, (uint32_t)e);
    __syncthreads();
  }
  float my_w = 0.0f;  // thread t < topk keeps result t
  int32_t my_id = 0;
  for (int t = 0; t < topk; ++t) {
    uint64_t local = 0;
    for (int e = tid; e < E; e += 256) local = key[e] > local ? key[e] : local;
    const uint64_t wb = warp_max_u64(local);
    if (lane == 0) warp_best[warp] = wb;
    __syncthreads();
    if (warp == 0) {
      const uint64_t b = warp_max_u64(lane < 8 ? warp_best[lane] : 0);
      if (lane == 0) best_bc = b;
    }
    __syncthreads();
    const uint64_t best = best_bc;
    const uint32_t id = 0xFFFFFFFFu - (uint32_t)(best & 0xFFFFFFFFu);
    if (tid == t) { my_id = (int32_t)id; my_w = best != 0 ? u[id] : 0.0f; }
    if (best != 0 && (int)(id & 255u) == tid) key[id] = 0;  // the thread that scans this expert consumes it
    __syncthreads();
  }
  if (warp == 0) {  // topk <= 32
    float sum = lane < topk ? my_w : 0.0f;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, off);
    if (lane < topk) {
      const float w = renormalize ? my_w / (sum + 1e-20f) : my_w;
      w_row[lane] = w * scaling;
      id_row[lane] = my_id;
    }
  }
}

// Router GEMM and routing in one launch for decode batches: one CTA per token computes the
// token's E logits (x[token] . w[e], fp32) into shared memory and its first warp routes them, so
// the [M, E] logits never travel through global memory.  The dot products are formed exactly as
// router_gemm_kernel forms them (128 threads per expert: 8-element chunks strided over the
// threads, shuffle tree, four warp sums in warp order), so logits, ids and weights equal those of
// the two separate launches bit for bit.  256 threads work on two experts at a time.
template <typename XT, typename WT, typename BT, int VPT>
__global__ void __launch_bounds__(256) router_topk_fused_kernel(
    const XT* __restrict__ x, int64_t x_ld, const WT* __restrict__ w, const BT* __restrict__ bias, int64_t M, int E,
    int K, int n_group, int topk_group, int topk, int renormalize, float scaling, int scoring_func,
    float* __restrict__ out_w, int32_t* __restrict__ out_ids, float* __restrict__ logits_out) {
  extern __shared__ float fused_smem[];
  float* logits = fused_smem;             // [E]
  float* part = fused_smem + E;           // [2][4]
  const int64_t token = blockIdx.x;
  const int half = threadIdx.x >> 7, t = threadIdx.x & 127, lane = threadIdx.x & 31, wq = (threadIdx.x >> 5) & 3;
  const XT* xr = x + token * x_ld;
  for (int e0 = 0; e0 < E; e0 += 2) {
    const int e = e0 + half;
    float acc = 0.0f;
    if (e < E) {
      const WT* wr = w + (int64_t)e * K;
      for (int k = t * 8; k < K; k += 128 * 8) {
        float wv[8], xv[8];
        load8<WT>(wr + k, wv);
        load8<XT>(xr + k, xv);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(xv[i], wv[i], acc);
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xFFFFFFFFu, acc, off);
    if (lane == 0) part[half * 4 + wq] = acc;
    __syncthreads();
    if (t == 0 && e < E) {
      float v = part[half * 4];
#pragma unroll
      for (int wi = 1; wi < 4; ++wi) v += part[half * 4 + wi];
      logits[e] = v;
      if (logits_out != nullptr) logits_out[token * E + e] = v;
    }
    __syncthreads();
  }
  if (threadIdx.x < 32)
    route_row<float, BT, VPT>(logits, 1, bias, E, n_group, topk_group, topk, renormalize, scaling, scoring_func,
                              out_w + token * topk, out_ids + token * topk, lane);
}

template <typename ST, typename BT>
int launch_vpt(const ST* scores, int64_t s0, int64_t s1, const BT* bias, const uint8_t* pad,
               int64_t M, int E, int n_group, int topk_group, int topk, int renorm, float scaling,
               int scoring, float* w, int32_t* ids, cudaStream_t st) {
  if (E > 1024) {
    auto kern = grouped_topk_big_kernel<ST, BT>;
    const size_t smem = (size_t)E * (sizeof(uint64_t) + sizeof(float));
    cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (ce != cudaSuccess) return fail((int)ce, "grouped_topk: shared memory attribute: %s", cudaGetErrorString(ce));
    kern<<<(unsigned)M, 256, smem, st>>>(scores, s0, s1, bias, pad, M, E, n_group, topk_group, topk, renorm, scaling,
                                        scoring, w, ids);
    return check_launch("grouped_topk (wide router)");
  }
  const int warps = 4;
  dim3 grid((unsigned)((M + warps - 1) / warps)), block(warps * 32);
#define MOE_TOPK_LAUNCH(V)                                                                     \
  grouped_topk_kernel<ST, BT, V><<<grid, block, 0, st>>>(scores, s0, s1, bias, pad, M, E,      \
                                                         n_group, topk_group, topk, renorm,   \
                                                         scaling, scoring, w, ids)
  if (E <= 32) MOE_TOPK_LAUNCH(1);
  else if (E <= 64) MOE_TOPK_LAUNCH(2);
  else if (E <= 128) MOE_TOPK_LAUNCH(4);
  else if (E <= 256) MOE_TOPK_LAUNCH(8);
  else if (E <= 512) MOE_TOPK_LAUNCH(16);
  else MOE_TOPK_LAUNCH(32);
#undef MOE_TOPK_LAUNCH
  return check_launch("grouped_topk");
}

template <typename ST>
int launch_bias(const ST* scores, int64_t s0, int64_t s1, const void* bias, int bias_dtype,
                const uint8_t* pad, int64_t M, int E, int n_group, int topk_group, int topk,
                int renorm, float scaling, int scoring, float* w, int32_t* ids, cudaStream_t st) {
  switch (bias_dtype) {
    case MOE_F32:
      return launch_vpt(scores, s0, s1, (const float*)bias, pad, M, E, n_group, topk_group, topk,
                        renorm, scaling, scoring, w, ids, st);
    case MOE_F16:
      return launch_vpt(scores, s0, s1, (const __half*)bias, pad, M, E, n_group, topk_group, topk,
                        renorm, scaling, scoring, w, ids, st);
    case MOE_BF16:
      return launch_vpt(scores, s0, s1, (const __nv_bfloat16*)bias, pad, M, E, n_group,
                        topk_group, topk, renorm, scaling, scoring, w, ids, st);
    default:
      return fail(MOE_E_DTYPE, "grouped_topk: unsupported bias dtype %d", bias_dtype);
  }
}

}  // namespace
}  // namespace moe

extern "C" int moe_grouped_topk(const void* scores, int scores_dtype, int64_t stride0,
                                int64_t stride1, const void* bias, int bias_dtype,
                                const uint8_t* is_padding, int64_t M, int E, int n_group,
                                int topk_group, int topk, int renormalize,
                                float routed_scaling_factor, int scoring_func, float* topk_weights,
                                int32_t* topk_ids, void* stream) {
  using namespace moe;
  if (M < 0 || E <= 0 || n_group <= 0 || topk <= 0 || topk_group <= 0)
    return fail(MOE_E_BADARG, "grouped_topk: non-positive extent");
  if (E > 4096) return fail(MOE_E_TOOBIG, "grouped_topk: at most 4096 experts (got %d)", E);
  if (E > 1024 && M > 2147483647ll) return fail(MOE_E_TOOBIG, "grouped_topk: too many rows");
  if (n_group > 32 || topk > 32 || topk_group > n_group || E % n_group != 0 || topk > E)
    return fail(MOE_E_SHAPE, "grouped_topk: bad group/top-k configuration");
  if (scoring_func != 0 && scoring_func != 1)
    return fail(MOE_E_BADARG, "grouped_topk: scoring_func must be 0 or 1");
  if (M == 0) return 0;
  if (!scores || !bias || !topk_weights || !topk_ids)
    return fail(MOE_E_BADARG, "grouped_topk: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  switch (scores_dtype) {
    case MOE_F32:
      return launch_bias((const float*)scores, stride0, stride1, bias, bias_dtype, is_padding, M, E,
                         n_group, topk_group, topk, renormalize, routed_scaling_factor,
                         scoring_func, topk_weights, topk_ids, st);
    case MOE_F16:
      return launch_bias((const __half*)scores, stride0, stride1, bias, bias_dtype, is_padding, M,
                         E, n_group, topk_group, topk, renormalize, routed_scaling_factor,
                         scoring_func, topk_weights, topk_ids, st);
    case MOE_BF16:
      return launch_bias((const __nv_bfloat16*)scores, stride0, stride1, bias, bias_dtype,
                         is_padding, M, E, n_group, topk_group, topk, renormalize,
                         routed_scaling_factor, scoring_func, topk_weights, topk_ids, st);
    default:
      return fail(MOE_E_DTYPE, "grouped_topk: unsupported scores dtype %d", scores_dtype);
  }
}

extern "C" int moe_router_gemm_grouped_topk(const void* x, int x_dtype, int64_t x_ld, const void* w, int w_dtype,
                                            const float* bias, int64_t M, int E, int K, int n_group, int topk_group,
                                            int topk, int renormalize, float routed_scaling_factor, int scoring_func,
                                            float* topk_weights, int32_t* topk_ids, float* logits_out, void* stream) {
  using namespace moe;
  if (M < 0 || E <= 0 || K <= 0 || n_group <= 0 || topk <= 0 || topk_group <= 0)
    return fail(MOE_E_BADARG, "router_gemm_grouped_topk: non-positive extent");
  if (E > 1024) return fail(MOE_E_TOOBIG, "router_gemm_grouped_topk: at most 1024 experts (got %d)", E);
  if (n_group > 32 || topk > 32 || topk_group > n_group || E % n_group != 0 || topk > E)
    return fail(MOE_E_SHAPE, "router_gemm_grouped_topk: bad group/top-k configuration");
  if (scoring_func != 0 && scoring_func != 1) return fail(MOE_E_BADARG, "router_gemm_grouped_topk: scoring_func must be 0 or 1");
  if (K % 8 != 0 || x_ld % 8 != 0 || x_ld < K) return fail(MOE_E_SHAPE, "router_gemm_grouped_topk: K and the row pitch must be multiples of 8");
  if (M == 0) return 0;
  if (!x || !w || !bias || !topk_weights || !topk_ids) return fail(MOE_E_BADARG, "router_gemm_grouped_topk: null pointer");
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(MOE_E_BADARG, "router_gemm_grouped_topk: operands must be 16-byte aligned");
  if (M > 65535 * 32) return fail(MOE_E_TOOBIG, "router_gemm_grouped_topk: too many rows");
  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem = (size_t)(E + 8) * sizeof(float);
#define MOE_RT_V(XT, WT, V)                                                                                         \
  router_topk_fused_kernel<XT, WT, float, V><<<(unsigned)M, 256, smem, st>>>(                                        \
      (const XT*)x, x_ld, (const WT*)w, bias, M, E, K, n_group, topk_group, topk, renormalize, routed_scaling_factor, \
      scoring_func, topk_weights, topk_ids, logits_out)
#define MOE_RT(XT, WT)                     \
  do {                                     \
    if (E <= 32) MOE_RT_V(XT, WT, 1);      \
    else if (E <= 64) MOE_RT_V(XT, WT, 2); \
    else if (E <= 128) MOE_RT_V(XT, WT, 4);\
    else if (E <= 256) MOE_RT_V(XT, WT, 8);\
    else if (E <= 512) MOE_RT_V(XT, WT, 16);\
    else MOE_RT_V(XT, WT, 32);             \
  } while (0)
  if (x_dtype == MOE_BF16 && w_dtype == MOE_BF16) MOE_RT(__nv_bfloat16, __nv_bfloat16);
  else if (x_dtype == MOE_F16 && w_dtype == MOE_F16) MOE_RT(__half, __half);
  else if (x_dtype == MOE_BF16 && w_dtype == MOE_F32) MOE_RT(__nv_bfloat16, float);
  else if (x_dtype == MOE_F32 && w_dtype == MOE_F32) MOE_RT(float, float);
  else return fail(MOE_E_DTYPE, "router_gemm_grouped_topk: unsupported dtype pair (%d, %d)", x_dtype, w_dtype);
#undef MOE_RT
#undef MOE_RT_V
  return check_launch("router_gemm_grouped_topk");
}
