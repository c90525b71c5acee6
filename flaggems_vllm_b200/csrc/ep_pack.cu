// Device-side bookkeeping of the expert-parallel step (experts partitioned over ranks, tokens
// data-parallel): which (token, destination rank) pairs exist, the send buffers of the
// dispatch all-to-all, and the receiver's view of what arrived.  The reference has no
// all-to-all path (its expert-parallel hook is expert_map with replicated tokens,
// src/flaggems_vllm/ops/fused_moe.py:2553-2560); these kernels replace some thirty small
// tensor operations per step that kept the GPU waiting on the host.
#include "moe_common.cuh"

namespace moe {
namespace {

constexpr int kPlanThreads = 1024;
constexpr int kMaxRanks = 16;

__device__ __forceinline__ uint32_t visit_mask(const int32_t* ids, int k, int experts_per_rank, int R) {
  uint32_t m = 0;
  for (int j = 0; j < k; ++j) {
    const int e = ids[j];
    if (e >= 0) m |= 1u << min(e / experts_per_rank, R - 1);
  }
  return m;
}

// One CTA.  Thread t owns the contiguous token range [t*C, (t+1)*C), so positions inside a
// rank's segment are in token order: pair (token, rank) sits at
// rank_offset[rank] + (visits of that rank by earlier tokens).
__global__ void __launch_bounds__(kPlanThreads) ep_plan_kernel(const int32_t* __restrict__ topk_ids, int64_t M, int k,
                                                               int experts_per_rank, int R,
                                                               int32_t* __restrict__ index, int32_t* __restrict__ counts,
                                                               int32_t* __restrict__ tok) {
  __shared__ int32_t warp_tot[kMaxRanks][kPlanThreads / 32];
  __shared__ int32_t rank_off[kMaxRanks + 1];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t C = (M + kPlanThreads - 1) / kPlanThreads;
  const int64_t t0 = min((int64_t)tid * C, M), t1 = min(t0 + C, M);
  int32_t cnt[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) cnt[r] = 0;
  for (int64_t t = t0; t < t1; ++t) {
    const uint32_t m = visit_mask(topk_ids + t * k, k, experts_per_rank, R);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) cnt[r] += (m >> r) & 1u;
  }
  // exclusive prefix of every rank's per-thread counts over the threads
  int32_t excl[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) {
    int32_t v = cnt[r];
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const int32_t n = __shfl_up_sync(0xFFFFFFFFu, v, off);
      if (lane >= off) v += n;
    }
    excl[r] = v - cnt[r];
    if (lane == 31) warp_tot[r][warp] = v;
  }
  __syncthreads();
  if (warp == 0) {
    for (int r = 0; r < R; ++r) {
      int32_t v = warp_tot[r][lane];
      const int32_t own = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const int32_t n = __shfl_up_sync(0xFFFFFFFFu, v, off);
        if (lane >= off) v += n;
      }
      warp_tot[r][lane] = v - own;  // exclusive offset of each warp
      if (lane == 31) rank_off[r + 1] = v;  // total of the rank
    }
    __syncwarp();
    if (lane == 0) {
      rank_off[0] = 0;
      for (int r = 0; r < R; ++r) {
        counts[r] = rank_off[r + 1];
        rank_off[r + 1] += rank_off[r];
      }
    }
  }
  __syncthreads();
  int32_t pos[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) pos[r] = r < R ? rank_off[r] + warp_tot[r][warp] + excl[r] : 0;
  for (int64_t t = t0; t < t1; ++t) {
    const uint32_t m = visit_mask(topk_ids + t * k, k, experts_per_rank, R);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < R) {
        if ((m >> r) & 1u) {
          index[t * R + r] = pos[r];
          tok[pos[r]] = (int32_t)t;
          ++pos[r];
        } else {
          index[t * R + r] = -1;
        }
      }
    }
  }
}

// One warp per pair: the token's row and one fp32 side row [scales (g) | expert ids (k) | weights (k)].
__global__ void __launch_bounds__(256) ep_pack_kernel(const uint4* __restrict__ rows, int64_t row_vec,
                                                      const float* __restrict__ scales, int g,
                                                      const int32_t* __restrict__ topk_ids,
                                                      const float* __restrict__ topk_weights, int k,
                                                      const int32_t* __restrict__ tok, int64_t P,
                                                      uint4* __restrict__ rows_out, float* __restrict__ side_out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int side = g + 2 * k;
  for (int64_t p = warp; p < P; p += warps) {
    const int64_t t = tok[p];
    const uint4* src = rows + t * row_vec;
    uint4* dst = rows_out + p * row_vec;
    int64_t c = lane;
    for (; c + 96 < row_vec; c += 128) {
      const uint4 v0 = src[c], v1 = src[c + 32], v2 = src[c + 64], v3 = src[c + 96];
      dst[c] = v0; dst[c + 32] = v1; dst[c + 64] = v2; dst[c + 96] = v3;
    }
    for (; c < row_vec; c += 32) dst[c] = src[c];
    float* so = side_out + p * side;
    for (int i = lane; i < side; i += 32) {
      float v;
      if (i < g) v = scales[t * g + i];
      else if (i < g + k) v = (float)topk_ids[t * k + (i - g)];  // expert ids < 2^24: exact in fp32
      else v = topk_weights[t * k + (i - g - k)];
      so[i] = v;
    }
  }
}

// Receiver: side rows -> transposed scales [g, n], local slot ids (or -1 for another rank's
// route) and slot weights.
__global__ void __launch_bounds__(256) ep_unpack_kernel(const float* __restrict__ side, int64_t n, int g, int k, int rank,
                                                        int experts_per_rank, float* __restrict__ scales_t,
                                                        int32_t* __restrict__ slot_ids, float* __restrict__ slot_w) {
  const int w = g + 2 * k;
  const int64_t total = n * w;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = i / w;
    const int c = (int)(i % w);
    const float v = side[i];
    if (c < g) {
      scales_t[(int64_t)c * n + p] = v;
    } else if (c < g + k) {
      const int local = (int)v - rank * experts_per_rank;
      slot_ids[p * k + (c - g)] = (v >= 0.0f && local >= 0 && local < experts_per_rank) ? local : -1;
    } else {
      slot_w[p * k + (c - g - k)] = v;
    }
  }
}

inline int grid_1d(int64_t work, int per_block, int max_blocks = 148 * 16) {
  int64_t b = (work + per_block - 1) / per_block;
  if (b < 1) b = 1;
  return (int)(b < max_blocks ? b : max_blocks);
}

}  // namespace
}  // namespace moe

extern "C" int moe_ep_plan(const int32_t* topk_ids, int64_t M, int k, int experts_per_rank, int world,
                           int32_t* index, int32_t* counts, int32_t* tok, void* stream) {
  using namespace moe;
  if (M < 0 || k <= 0 || experts_per_rank <= 0 || world <= 0) return fail(MOE_E_BADARG, "ep_plan: bad extent");
  if (world > kMaxRanks) return fail(MOE_E_TOOBIG, "ep_plan: at most %d ranks", kMaxRanks);
  if (M * world >= (1ll << 31)) return fail(MOE_E_TOOBIG, "ep_plan: tokens * ranks exceeds int32");
  if (!counts || (M > 0 && (!topk_ids || !index || !tok))) return fail(MOE_E_BADARG, "ep_plan: null pointer");
  ep_plan_kernel<<<1, kPlanThreads, 0, (cudaStream_t)stream>>>(topk_ids, M, k, experts_per_rank, world, index, counts, tok);
  return check_launch("ep_plan");
}

extern "C" int moe_ep_pack(const void* rows, int64_t row_bytes, const float* scales, int groups,
                           const int32_t* topk_ids, const float* topk_weights, int k, const int32_t* tok,
                           int64_t pairs, void* rows_out, float* side_out, void* stream) {
  using namespace moe;
  if (row_bytes <= 0 || groups < 0 || k <= 0 || pairs < 0) return fail(MOE_E_BADARG, "ep_pack: bad extent");
  if (pairs == 0) return 0;
  if (!rows || !topk_ids || !topk_weights || !tok || !rows_out || !side_out || (groups > 0 && !scales))
    return fail(MOE_E_BADARG, "ep_pack: null pointer");
  if (row_bytes % 16 != 0 || ((uintptr_t)rows & 15) || ((uintptr_t)rows_out & 15))
    return fail(MOE_E_SHAPE, "ep_pack: row size and pointers must be multiples of 16 bytes");
  ep_pack_kernel<<<grid_1d(pairs, 8), 256, 0, (cudaStream_t)stream>>>((const uint4*)rows, row_bytes / 16, scales, groups,
                                                                      topk_ids, topk_weights, k, tok, pairs,
                                                                      (uint4*)rows_out, side_out);
  return check_launch("ep_pack");
}

extern "C" int moe_ep_unpack(const float* side, int64_t rows, int groups, int k, int rank, int experts_per_rank,
                             float* scales_t, int32_t* slot_ids, float* slot_w, void* stream) {
  using namespace moe;
  if (rows < 0 || groups < 0 || k <= 0 || rank < 0 || experts_per_rank <= 0) return fail(MOE_E_BADARG, "ep_unpack: bad extent");
  if (rows == 0) return 0;
  if (!side || !slot_ids || !slot_w || (groups > 0 && !scales_t)) return fail(MOE_E_BADARG, "ep_unpack: null pointer");
  ep_unpack_kernel<<<grid_1d(rows * (groups + 2 * k), 256), 256, 0, (cudaStream_t)stream>>>(
      side, rows, groups, k, rank, experts_per_rank, scales_t, slot_ids, slot_w);
  return check_launch("ep_unpack");
}
