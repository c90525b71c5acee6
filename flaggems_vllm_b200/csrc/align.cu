// moe_align_block_size: stable counting sort of the flat expert-id array with
// each expert's run padded to a multiple of block_size.
//
// One CTA does the whole job in a single launch, entirely in shared memory:
//   phase 0  fill both output buffers with their sentinels (numel / -1)
//   phase 1  per-warp histograms: warp w owns a contiguous slice of the ids
//   phase 2  per expert: exclusive prefix over warps, padded count;
//            block-wide exclusive scan of padded counts -> expert base
//            offsets, block ids, total
//   phase 3  every warp walks its slice again in order; lanes holding the
//            same expert are ranked with __match_any_sync, so the position of
//            an id is base[expert] + (ids of that expert before it in flat
//            order).  That makes the output deterministic and identical to a
//            stable sort, which is the ordering of the reference's torch
//            golden (tests/test_moe_align_block_size.py:293-388); the
//            reference kernels rank by atomic arrival order instead
//            (src/flaggems_vllm/ops/moe_align_block_size.py:505-527).
// Ids outside [0, num_experts) are skipped; ids >= num_experts are also flagged in the
// status word (negative ids are the conventional "no route" marker and stay silent).
//
// Large inputs (thousands of ids) use the same algorithm spread over a
// thread-block cluster of 8 CTAs: each CTA owns a contiguous eighth of the ids,
// the per-CTA expert totals are exchanged through distributed shared memory
// (plain remote loads, two cluster barriers), every CTA derives the same
// expert bases and scatters its own ids.  The result is bit-identical to the
// single-CTA kernel.
#include <cooperative_groups.h>

#include "moe_common.cuh"

namespace cg = cooperative_groups;

namespace moe {
namespace {

constexpr int kAlignThreads = 1024;

template <typename IdT>
__global__ void __launch_bounds__(kAlignThreads) align_kernel(
    const IdT* __restrict__ ids, int numel, int E, int block_size, int n_warps_used,
    int32_t* __restrict__ sorted_ids, int sorted_cap, int32_t* __restrict__ expert_ids,
    int expert_cap, int32_t* __restrict__ num_post_pad, int32_t* __restrict__ status) {
  extern __shared__ int32_t smem[];
  // layout: hist[n_warps_used][E] | blk_start[E + 1] | warp_sums[32] | carry[1]
  int32_t* hist = smem;
  int32_t* blk_start = hist + (size_t)n_warps_used * E;
  int32_t* warp_sums = blk_start + (E + 1);
  int32_t* carry = warp_sums + 32;

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  const int T = blockDim.x;

  for (int i = tid; i < n_warps_used * E; i += T) hist[i] = 0;
  for (int i = tid; i < sorted_cap; i += T) sorted_ids[i] = numel;
  for (int i = tid; i < expert_cap; i += T) expert_ids[i] = -1;
  if (tid == 0) carry[0] = 0;
  __syncthreads();

  // slice of this warp: multiples of 32 so a slice is walked in whole rounds
  const int per_warp = ((numel + n_warps_used - 1) / n_warps_used + 31) & ~31;
  const int begin = warp * per_warp;
  const int end = min(numel, begin + per_warp);
  bool bad = false;
  if (warp < n_warps_used) {
    int32_t* h = hist + (size_t)warp * E;
    for (int i = begin + lane; i < end; i += 32) {
      long long e = (long long)ids[i];
      if (e >= 0 && e < E) atomicAdd(&h[(int)e], 1);
      else if (e >= E) bad = true;  // negative ids mean "no route" (padding rows, other ranks' slots)
    }
  }
  if (bad) set_status(status, MOE_ST_BAD_EXPERT_ID);
  __syncthreads();

  // phase 2: experts in chunks of T (one expert per thread per chunk)
  for (int e0 = 0; e0 < E; e0 += T) {
    const int e = e0 + tid;
    int padded = 0;
    if (e < E) {
      int run = 0;
      for (int w = 0; w < n_warps_used; ++w) {
        int c = hist[(size_t)w * E + e];
        hist[(size_t)w * E + e] = run;  // ids of expert e in earlier slices
        run += c;
      }
      padded = (run + block_size - 1) / block_size * block_size;
    }
    // exclusive scan of `padded` over the chunk
    int incl = padded;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      int o = __shfl_up_sync(0xFFFFFFFFu, incl, off);
      if (lane >= off) incl += o;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int v = lane < (T >> 5) ? warp_sums[lane] : 0;
      int s = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int o = __shfl_up_sync(0xFFFFFFFFu, s, off);
        if (lane >= off) s += o;
      }
      warp_sums[lane] = s - v;  // exclusive prefix of warp totals
    }
    __syncthreads();
    const int base = carry[0] + warp_sums[warp] + incl - padded;
    if (e < E) {
      blk_start[e] = base;
      for (int w = 0; w < n_warps_used; ++w) hist[(size_t)w * E + e] += base;
    }
    __syncthreads();
    if (tid == T - 1) carry[0] = base + padded;
    __syncthreads();
  }
  const int total = carry[0];
  if (tid == 0) {
    blk_start[E] = total;
    num_post_pad[0] = total;
  }
  __syncthreads();

  // block ids: block b belongs to the last expert whose start is <= b*bs
  const int n_blocks = total / block_size;
  for (int b = tid; b < n_blocks && b < expert_cap; b += T) {
    const int pos = b * block_size;
    int lo = 0, hi = E;  // invariant: blk_start[lo] <= pos < blk_start[hi]
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (blk_start[mid] <= pos) lo = mid; else hi = mid;
    }
    expert_ids[b] = lo;
  }

  // phase 3: ordered scatter
  if (warp < n_warps_used) {
    int32_t* h = hist + (size_t)warp * E;
    for (int i0 = begin; i0 < end; i0 += 32) {
      const int i = i0 + lane;
      long long e = i < end ? (long long)ids[i] : -1;
      const bool valid = e >= 0 && e < E;
      const unsigned vmask = __ballot_sync(0xFFFFFFFFu, valid);
      if (valid) {
        const unsigned same = __match_any_sync(vmask, (int)e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        const int leader = __ffs(same) - 1;
        int pos0 = 0;
        if (lane == leader) {
          pos0 = h[(int)e];
          h[(int)e] = pos0 + __popc(same);
        }
        pos0 = __shfl_sync(same, pos0, leader);
        const int pos = pos0 + rank;
        if (pos < sorted_cap) sorted_ids[pos] = i;
      }
      __syncwarp();
    }
  }
}


constexpr int kClusterSize = 8;

// Cluster variant.  Shared memory per CTA:
//   hist[W][E] | cta_tot[E] | blk_start[E + 1] | warp_sums[32] | carry[1]
template <typename IdT>
__global__ void __cluster_dims__(kClusterSize, 1, 1) __launch_bounds__(kAlignThreads)
align_cluster_kernel(const IdT* __restrict__ ids, int numel, int E, int block_size, int W,
                     int32_t* __restrict__ sorted_ids, int sorted_cap, int32_t* __restrict__ expert_ids,
                     int expert_cap, int32_t* __restrict__ num_post_pad, int32_t* __restrict__ status) {
  extern __shared__ int32_t smem[];
  int32_t* hist = smem;
  int32_t* cta_tot = hist + (size_t)W * E;
  int32_t* blk_start = cta_tot + E;
  int32_t* warp_sums = blk_start + (E + 1);
  int32_t* carry = warp_sums + 32;

  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, T = blockDim.x;
  const int gtid = rank * T + tid, GT = kClusterSize * T;

  for (int i = tid; i < W * E; i += T) hist[i] = 0;
  for (int i = gtid; i < sorted_cap; i += GT) sorted_ids[i] = numel;
  for (int i = gtid; i < expert_cap; i += GT) expert_ids[i] = -1;
  if (tid == 0) carry[0] = 0;
  __syncthreads();

  // slice of this CTA, then of this warp (multiples of 32)
  const int per_cta = ((numel + kClusterSize - 1) / kClusterSize + 31) & ~31;
  const int cbegin = rank * per_cta, cend = min(numel, cbegin + per_cta);
  const int per_warp = (((per_cta + W - 1) / W) + 31) & ~31;
  const int begin = cbegin + warp * per_warp;
  const int end = min(cend, begin + per_warp);
  bool bad = false;
  if (warp < W) {
    int32_t* h = hist + (size_t)warp * E;
    for (int i = begin + lane; i < end; i += 32) {
      long long e = (long long)ids[i];
      if (e >= 0 && e < E) atomicAdd(&h[(int)e], 1);
      else if (e >= E) bad = true;  // negative ids mean "no route" (padding rows, other ranks' slots)
    }
  }
  if (bad) set_status(status, MOE_ST_BAD_EXPERT_ID);
  __syncthreads();
  for (int e = tid; e < E; e += T) {
    int run = 0;
    for (int w = 0; w < W; ++w) {
      int c = hist[(size_t)w * E + e];
      hist[(size_t)w * E + e] = run;
      run += c;
    }
    cta_tot[e] = run;
  }
  cluster.sync();  // every CTA's cta_tot is final and visible cluster-wide

  for (int e0 = 0; e0 < E; e0 += T) {
    const int e = e0 + tid;
    int padded = 0, before = 0;
    if (e < E) {
      int total = 0;
#pragma unroll
      for (int r = 0; r < kClusterSize; ++r) {
        const int32_t* remote = cluster.map_shared_rank(cta_tot, r);
        const int c = remote[e];
        if (r < rank) before += c;
        total += c;
      }
      padded = (total + block_size - 1) / block_size * block_size;
    }
    int incl = padded;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      int o = __shfl_up_sync(0xFFFFFFFFu, incl, off);
      if (lane >= off) incl += o;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int v = lane < (T >> 5) ? warp_sums[lane] : 0;
      int sc = v;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        int o = __shfl_up_sync(0xFFFFFFFFu, sc, off);
        if (lane >= off) sc += o;
      }
      warp_sums[lane] = sc - v;
    }
    __syncthreads();
    const int base = carry[0] + warp_sums[warp] + incl - padded;
    if (e < E) {
      blk_start[e] = base;
      for (int w = 0; w < W; ++w) hist[(size_t)w * E + e] += base + before;
    }
    __syncthreads();
    if (tid == T - 1) carry[0] = base + padded;
    __syncthreads();
  }
  const int total = carry[0];
  if (tid == 0) blk_start[E] = total;
  if (gtid == 0) num_post_pad[0] = total;
  __syncthreads();

  const int n_blocks = total / block_size;
  for (int b = gtid; b < n_blocks && b < expert_cap; b += GT) {
    const int pos = b * block_size;
    int lo = 0, hi = E;
    while (hi - lo > 1) {
      int mid = (lo + hi) >> 1;
      if (blk_start[mid] <= pos) lo = mid; else hi = mid;
    }
    expert_ids[b] = lo;
  }
  // sentinel fill of all CTAs must be complete before anyone scatters; the
  // same barrier keeps every CTA's shared memory alive while peers read it
  cluster.sync();

  if (warp < W) {
    int32_t* h = hist + (size_t)warp * E;
    for (int i0 = begin; i0 < end; i0 += 32) {
      const int i = i0 + lane;
      long long e = i < end ? (long long)ids[i] : -1;
      const bool valid = e >= 0 && e < E;
      const unsigned vmask = __ballot_sync(0xFFFFFFFFu, valid);
      if (valid) {
        const unsigned same = __match_any_sync(vmask, (int)e);
        const int rk = __popc(same & ((1u << lane) - 1u));
        const int leader = __ffs(same) - 1;
        int pos0 = 0;
        if (lane == leader) {
          pos0 = h[(int)e];
          h[(int)e] = pos0 + __popc(same);
        }
        pos0 = __shfl_sync(same, pos0, leader);
        const int pos = pos0 + rk;
        if (pos < sorted_cap) sorted_ids[pos] = i;
      }
      __syncwarp();
    }
  }
}

}  // namespace
}  // namespace moe

extern "C" int moe_align_block_size(const void* topk_ids, int ids_int64, int64_t numel,
                                    int num_experts, int block_size, int32_t* sorted_ids,
                                    int64_t sorted_cap, int32_t* expert_ids, int64_t expert_cap,
                                    int32_t* num_post_pad, int32_t* status, void* stream) {
  using namespace moe;
  if (numel < 0 || num_experts <= 0 || block_size <= 0 || sorted_cap < 0 || expert_cap < 0)
    return fail(MOE_E_BADARG, "align: negative or zero extent");
  if (num_experts > 4096) return fail(MOE_E_TOOBIG, "align: at most 4096 experts");
  if (numel >= (1ll << 31) - 1 || sorted_cap >= (1ll << 31) - 1)
    return fail(MOE_E_TOOBIG, "align: numel must fit int32");
  if (!sorted_ids || !expert_ids || !num_post_pad || (numel > 0 && !topk_ids))
    return fail(MOE_E_BADARG, "align: null pointer");
  // worst case padded total must fit the buffers the caller gave
  // (numel + E*(bs-1) is the reference's bound); the kernel clips writes anyway.
  const int E = num_experts;
  cudaStream_t st = (cudaStream_t)stream;
  cudaError_t ce;
  if (numel >= 4096 && E <= 1024) {
    // cluster of 8 CTAs; hist[W][E] + cta_tot[E] + blk_start[E+1] + 33 words per CTA
    int W = kAlignThreads / 32;
    while (W > 1 && ((size_t)W * E + 2 * (size_t)E + 34) * 4 > 96 * 1024) W >>= 1;
    const size_t smem = ((size_t)W * E + 2 * (size_t)E + 34) * 4;
    if (ids_int64) {
      ce = cudaFuncSetAttribute(align_cluster_kernel<int64_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (ce != cudaSuccess) return fail((int)ce, "align: smem attribute: %s", cudaGetErrorString(ce));
      align_cluster_kernel<int64_t><<<kClusterSize, kAlignThreads, smem, st>>>(
          (const int64_t*)topk_ids, (int)numel, E, block_size, W, sorted_ids, (int)sorted_cap, expert_ids,
          (int)expert_cap, num_post_pad, status);
    } else {
      ce = cudaFuncSetAttribute(align_cluster_kernel<int32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (ce != cudaSuccess) return fail((int)ce, "align: smem attribute: %s", cudaGetErrorString(ce));
      align_cluster_kernel<int32_t><<<kClusterSize, kAlignThreads, smem, st>>>(
          (const int32_t*)topk_ids, (int)numel, E, block_size, W, sorted_ids, (int)sorted_cap, expert_ids,
          (int)expert_cap, num_post_pad, status);
    }
    return check_launch("align (cluster)");
  }
  // one slice (and one histogram) per 64 ids: a decode-sized call clears and scans one or two
  // histograms instead of 32
  int n_warps = kAlignThreads / 32;
  const int64_t slices = (numel + 63) / 64;
  if (slices < n_warps) n_warps = slices < 1 ? 1 : (int)slices;
  const size_t budget = 200 * 1024;
  while (n_warps > 1 && ((size_t)n_warps * E + E + 1 + 33) * 4 > budget) n_warps >>= 1;
  const size_t smem = ((size_t)n_warps * E + E + 1 + 33) * 4;
  if (ids_int64) {
    ce = cudaFuncSetAttribute(align_kernel<int64_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)smem);
    if (ce != cudaSuccess) return fail((int)ce, "align: smem attribute: %s", cudaGetErrorString(ce));
    align_kernel<int64_t><<<1, kAlignThreads, smem, st>>>(
        (const int64_t*)topk_ids, (int)numel, E, block_size, n_warps, sorted_ids, (int)sorted_cap,
        expert_ids, (int)expert_cap, num_post_pad, status);
  } else {
    ce = cudaFuncSetAttribute(align_kernel<int32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              (int)smem);
    if (ce != cudaSuccess) return fail((int)ce, "align: smem attribute: %s", cudaGetErrorString(ce));
    align_kernel<int32_t><<<1, kAlignThreads, smem, st>>>(
        (const int32_t*)topk_ids, (int)numel, E, block_size, n_warps, sorted_ids, (int)sorted_cap,
        expert_ids, (int)expert_cap, num_post_pad, status);
  }
  return check_launch("align");
}


namespace moe {
// expert_ids[i] = expert_map[expert_ids[i]]; ids outside [0, num_experts) (the -1 of unused
// blocks) become -1, which every GEMM kernel skips.
__global__ void map_expert_ids_kernel(int32_t* expert_ids, int64_t n, const int32_t* __restrict__ expert_map,
                                      int num_experts) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = expert_ids[i];
  expert_ids[i] = (e >= 0 && e < num_experts) ? expert_map[e] : -1;
}
}  // namespace moe

extern "C" int moe_map_expert_ids(int32_t* expert_ids, int64_t n, const int32_t* expert_map, int num_experts,
                                  void* stream) {
  using namespace moe;
  if (n < 0 || num_experts <= 0) return fail(MOE_E_BADARG, "map_expert_ids: negative or zero extent");
  if (n == 0) return 0;
  if (!expert_ids || !expert_map) return fail(MOE_E_BADARG, "map_expert_ids: null pointer");
  map_expert_ids_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(expert_ids, n, expert_map,
                                                                                      num_experts);
  return check_launch("map_expert_ids");
}
