// Small-batch schedule of the two expert GEMMs: weight streaming with split-K.
//
// With a handful of routes per expert the 128-row tcgen05 tiles multiply padding, and
// the layer is bound by reading every routed expert's weights once.  Here the weights
// sit on the wide side of the product: the align block is 8 routes, a unit of work is
// (align block, 128 weight rows, one slice of K), and a persistent CTA streams the
// unit's weight rows through a TMA ring while eight warps multiply them with the
// block's 8 activation rows held in shared memory,
//
//     D[16 weight rows, 8 routes] += W[16, k] . X[8, k]^T      (warp-level mma.sync),
//
// in e4m3 (FP8 block scales: every 128-wide K block goes to a fresh accumulator and is
// folded with a_scale * w_scale, the arithmetic of the reference kernel,
// src/flaggems_vllm/ops/fused_moe.py:1708-1722), f16/bf16, or int8 weights widened
// exactly in registers (weight-only int8; the channel scale is applied at the end).
// FP8 activations are quantised 1x128 by the unit itself from the rows it loads.
//
// K is cut into slices of at most 4096 bytes of an activation row (what fits beside the ring).  Every
// slice writes its fp32 partial tile to scratch and bumps a counter; the CTA that
// finds the counter complete adds the slices IN SLICE ORDER, so the result does not
// depend on which CTA finished last.  The same scheme joins the top-k routes of a
// token in GEMM 2: the CTA that writes a token's last route row for a column tile adds
// the token's rows in slot order and writes the layer output (the reference's moe_sum,
// src/flaggems_vllm/ops/moe_sum.py:250-310).  No floating-point atomics anywhere.
// Stands in for the reference's small-batch route (naive_block_assignment,
// src/flaggems_vllm/ops/fused_moe.py:2542-2568).
//
// The K order inside a 32-element group is permuted identically for both operands so
// that every lane fetches its fragment with one or two vector loads; a dot product does
// not care.  The weight tile keeps TMA's 128-byte swizzle, which also makes those loads
// conflict-free.
#include "tc_common.cuh"

namespace moe {
namespace sm {

using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::mbar_wait;
using tc::smem_u32;
using tc::tma_load_2d;

constexpr int ROWS = 8;                       // routes per align block = N of the warp MMA
constexpr int CWARPS = 8;                     // compute warps, 16 weight rows each
constexpr int TILE_W = CWARPS * 16;           // weight rows per unit
constexpr int CTHREADS = CWARPS * 32;
constexpr int THREADS = CTHREADS + 32;        // + the TMA producer warp
constexpr int STAGES = 11;
constexpr int STAGE_BYTES = TILE_W * 128;     // 128 weight rows x 128 bytes of K
constexpr int X_ROW_BYTES = 4096;             // bytes of one activation row a unit holds (one K slice)
constexpr int MAX_GROUPS = X_ROW_BYTES / 128; // FP8: 1 x 128 groups of a slice

struct Params {
  const void* a;              // GEMM1: x [tokens, K]; GEMM2: intermediate [rows_cap, K] in sorted order (act dtype)
  const float* w_scale;       // FP8: [E, rows_w/128, K/128]; weight-only int8: [E, rows_w]; else null
  const int32_t* expert_ids;  // [rows_cap / 8], global expert ids
  const int32_t* sorted_ids;  // [rows_cap]
  const int32_t* num_post_pad;
  const int32_t* expert_map;  // [num_experts_global] or null
  const float* route_weight;  // [numel]
  const void* topk_ids;       // [tokens, topk] (GEMM2: which slots of a token count)
  void* out;                  // GEMM1: intermediate [rows_cap, Nout]; GEMM2: y [numel, Nout]
  void* final_out;            // GEMM2: layer output [tokens, Nout]
  float* partial;             // [S, rows_cap, NT * 128] fp32 (S > 1)
  int32_t* unit_cnt;          // [rows_cap / 8 * NT * 8 warps], zero before and after the launch
  int32_t* tok_cnt;           // [tokens * NT * 8 warps] (GEMM2), zero before and after the launch
  int32_t* status;
  unsigned long long wait_ns;  // limit of every bounded barrier wait
  int64_t numel, rows_cap, tokens;
  int ids_int64, num_experts_global;
  int topk, mul_weight, E, K, Nout, rows_w, NT, S, chunks_total, cps;
};

template <int MODE, typename AT> struct Fmt {
  static constexpr int EW = MODE == MOE_MODE_HALF ? 2 : 1;       // bytes per weight element
  static constexpr int EX = MODE == MOE_MODE_FP8_BLOCK ? 1 : 2;  // bytes per activation element in shared memory
  static constexpr int CE = 128 / EW;                            // K elements per 128-byte chunk
  static constexpr int KSE = X_ROW_BYTES / EX;                   // K elements per slice at most
  static constexpr int XPITCH = X_ROW_BYTES + (EX == 1 ? 32 : 64);  // odd multiple of 32 / 64 bytes: conflict-free row stride
};

struct Smem {
  uint64_t full[STAGES];
  uint64_t empty[STAGES];
  float sx[ROWS][MAX_GROUPS];      // FP8: activation scale of (route, K block of the slice)
  int32_t sid[ROWS];               // flat route index of the block's rows, -1 for padding
  uint32_t mask[ROWS];             // GEMM2: valid slots of the token of each row
};

__device__ __forceinline__ void bar_compute() { asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory"); }

__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <typename AT>
__device__ __forceinline__ void mma_half(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  if constexpr (std::is_same<AT, __nv_bfloat16>::value) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  } else {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
  }
}
__device__ __forceinline__ uint2 lds64(const uint8_t* p) { return *reinterpret_cast<const uint2*>(p); }
__device__ __forceinline__ uint4 lds128(const uint8_t* p) { return *reinterpret_cast<const uint4*>(p); }
// Counter increments that publish (release) what the CTA wrote before a barrier and observe
// (acquire) what the other CTAs published: no device-wide fence per thread is needed.
__device__ __forceinline__ int atom_add_acq_rel(int32_t* p, int v) {
  int old;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
  return old;
}
// loads that must see what another CTA wrote before it bumped a counter: bypass L1
__device__ __forceinline__ float4 ldcg_f4(const float* p) {
  float4 v;
  asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ float ldcg_f(const float* p) {
  float v;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}
template <typename AT>
__device__ __forceinline__ AT ldcg_at(const AT* p) {
  unsigned short v;
  asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(v) : "l"(p));
  return *reinterpret_cast<const AT*>(&v);
}

// MODE: MOE_MODE_HALF / MOE_MODE_FP8_BLOCK / MOE_MODE_W8A16.  GEMM1: gate|up rows and the
// SiLU(gate)*up epilogue; GEMM2: route weight and the top-k combine.
template <int MODE, typename AT, bool GEMM1>
__global__ void __launch_bounds__(THREADS, 1)
small_gemm_kernel(const __grid_constant__ CUtensorMap map_w, const Params P) {
  using F = Fmt<MODE, AT>;
  constexpr bool FP8 = MODE == MOE_MODE_FP8_BLOCK;
  constexpr bool W8 = MODE == MOE_MODE_W8A16;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* ring = smem;
  uint8_t* xs = smem + (size_t)STAGES * STAGE_BYTES;  // [ROWS][XPITCH]
  Smem* aux = reinterpret_cast<Smem*>(xs + ROWS * F::XPITCH);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int npp = (int)min((int64_t)P.num_post_pad[0], P.rows_cap);
  const int nb = (npp + ROWS - 1) / ROWS;
  const int total_units = nb * P.NT * P.S;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&aux->full[s], 1);
      mbar_init(&aux->empty[s], CWARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // Unit u -> column tile nt (fastest), slice s, align block b.  A CTA takes a contiguous range
  // of units, so consecutive units mostly share (b, s) and the staged activation rows are reused.
  const int u_begin = (int)((int64_t)total_units * blockIdx.x / gridDim.x);
  const int u_end = (int)((int64_t)total_units * (blockIdx.x + 1) / gridDim.x);
  int cached_b = -1, cached_e = -1;  // expert of the block looked up last (one global load per block)
  auto unit_expert = [&](int u, int& b, int& nt, int& s) -> int {
    nt = u % P.NT;
    s = (u / P.NT) % P.S;
    b = u / (P.S * P.NT);
    if (b != cached_b) {
      int e = P.expert_ids[b];
      if (P.expert_map != nullptr) e = (e >= 0 && e < P.num_experts_global) ? P.expert_map[e] : -1;
      cached_b = b;
      cached_e = (e >= 0 && e < P.E) ? e : -1;
    }
    return cached_e;
  };

  if (warp == CWARPS) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      uint32_t it = 0;
      bool alive = true;
      for (int u = u_begin; u < u_end && alive; ++u) {
        int b, nt, s;
        const int e = unit_expert(u, b, nt, s);
        if (e < 0) continue;
        const int c0 = s * P.cps, c1 = min(P.chunks_total, c0 + P.cps);
        const int wrow = e * P.rows_w;
        for (int c = c0; c < c1; ++c, ++it) {
          const int st = it % STAGES;
          if (!mbar_wait(&aux->empty[st], ((it / STAGES) & 1) ^ 1, P.status, P.wait_ns)) { alive = false; break; }
          mbar_expect_tx(&aux->full[st], STAGE_BYTES);
          uint8_t* dst = ring + (size_t)st * STAGE_BYTES;
          if constexpr (GEMM1) {
            tma_load_2d(&map_w, &aux->full[st], dst, c * F::CE, wrow + nt * 64);
            tma_load_2d(&map_w, &aux->full[st], dst + 64 * 128, c * F::CE, wrow + P.Nout + nt * 64);
          } else {
            tma_load_2d(&map_w, &aux->full[st], dst, c * F::CE, wrow + nt * TILE_W);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ compute warps
    // Warp w owns 16 weight rows of the tile: MMA rows g and g + 8 of lane (g, q) are tile rows
    // rowA and rowB.  GEMM1 pairs gate row 8w + g with the up row of the same output column, so
    // SiLU(gate) * up never leaves the lane.  After the K loop every warp finishes its own rows
    // (partial sums, counters, epilogue) without a CTA-wide barrier; the CTA only meets to stage
    // the activation rows of a new (align block, K slice).
    const int g = lane >> 2, q = lane & 3;
    const int rowA = GEMM1 ? 8 * warp + g : 16 * warp + g;
    const int rowB = GEMM1 ? 64 + 8 * warp + g : 16 * warp + g + 8;  // (row & 7) == g for both
    const int64_t a_pitch = (int64_t)P.K;  // elements per activation row
    const int64_t tile_ld = (int64_t)P.NT * TILE_W;
    uint32_t it = 0;
    bool alive = true;

    if constexpr (!GEMM1) {
      // tokens without any valid route are written by nobody else: their output row is zero
      for (int64_t t = (int64_t)blockIdx.x * CWARPS + warp; t < P.tokens; t += (int64_t)gridDim.x * CWARPS) {
        bool ok = false;
        if (lane < P.topk) {
          const long long id = P.ids_int64 ? ((const long long*)P.topk_ids)[t * P.topk + lane]
                                           : (long long)((const int32_t*)P.topk_ids)[t * P.topk + lane];
          ok = id >= 0 && id < P.num_experts_global && (P.expert_map == nullptr || P.expert_map[id] >= 0);
        }
        if (__ballot_sync(0xFFFFFFFFu, ok) == 0u) {
          AT* o = reinterpret_cast<AT*>(P.final_out) + t * P.Nout;
          for (int c = lane; c < P.Nout; c += 32) o[c] = from_f32<AT>(0.0f);
        }
      }
    }

    int staged_b = -1, staged_s = -1;
    for (int u = u_begin; u < u_end && alive; ++u) {
      int b, nt, s;
      const int e = unit_expert(u, b, nt, s);
      if (e < 0) continue;
      const int c0 = s * P.cps, c1 = min(P.chunks_total, c0 + P.cps);
      const int nchunks = c1 - c0;
      const int klen = nchunks * F::CE;            // elements of this slice
      const int64_t k0 = (int64_t)c0 * F::CE;

      // ---------------------------------------------------------------- stage the 8 activation rows
      if (b != staged_b || s != staged_s) {
      staged_b = b; staged_s = s;
      bar_compute();  // every warp has finished the units that used the rows staged before
      if (threadIdx.x < ROWS) {
        const int64_t p = (int64_t)b * ROWS + threadIdx.x;
        const int64_t sidv = p < P.rows_cap ? (int64_t)P.sorted_ids[p] : P.numel;
        aux->sid[threadIdx.x] = (sidv >= 0 && sidv < P.numel) ? (int32_t)sidv : -1;
        if (sidv < 0 || sidv > P.numel) set_status(P.status, MOE_ST_BAD_ROW);  // the pad value is numel
      }
      bar_compute();
      if constexpr (FP8) {
        // quantise 1 x 128 groups exactly as the stand-alone quantiser does: s = max(amax, 1e-10) / 448
        const int groups = klen / 128;
        constexpr int U = 4;  // groups in flight per warp: their global loads are issued before any is used
        for (int g0 = warp; g0 < ROWS * groups; g0 += U * CWARPS) {
          uint2 raw[U];
          bool live[U];
#pragma unroll
          for (int uu = 0; uu < U; ++uu) {
            const int gi = g0 + uu * CWARPS;
            live[uu] = false;
            raw[uu] = make_uint2(0u, 0u);
            if (gi < ROWS * groups) {
              const int r = gi / groups, kb = gi % groups;
              const int sidv = aux->sid[r];
              if (sidv >= 0) {
                const int64_t src_row = GEMM1 ? (int64_t)(sidv / P.topk) : (int64_t)b * ROWS + r;
                raw[uu] = *reinterpret_cast<const uint2*>(reinterpret_cast<const AT*>(P.a) + src_row * a_pitch + k0 +
                                                          kb * 128 + lane * 4);
                live[uu] = true;
              }
            }
          }
#pragma unroll
          for (int uu = 0; uu < U; ++uu) {
            const int gi = g0 + uu * CWARPS;
            if (gi >= ROWS * groups) continue;
            const int r = gi / groups, kb = gi % groups;
            uint32_t packed = 0;
            float sc = 1.0f;
            if (live[uu]) {  // warp-uniform
              const AT* pv = reinterpret_cast<const AT*>(&raw[uu]);
              float v[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) v[i] = ToF32<AT>::get(pv[i]);
              float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
              for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
              sc = fmaxf(amax, kQuantEps) * (1.0f / kFp8Max);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float qv = fminf(fmaxf(v[i] / sc, -kFp8Max), kFp8Max);
                packed |= (uint32_t)f32_to_fp8e4m3(qv) << (8 * i);
              }
            }
            *reinterpret_cast<uint32_t*>(xs + r * F::XPITCH + kb * 128 + lane * 4) = packed;
            if (lane == 0) aux->sx[r][kb] = sc;
          }
        }
      } else {
        const int vec_per_row = klen / 8;  // 16-byte vectors
        for (int v = threadIdx.x; v < ROWS * vec_per_row; v += CTHREADS) {
          const int r = v / vec_per_row, c = v % vec_per_row;
          const int sidv = aux->sid[r];
          uint4 val = make_uint4(0, 0, 0, 0);
          if (sidv >= 0) {
            const int64_t src_row = GEMM1 ? (int64_t)(sidv / P.topk) : (int64_t)b * ROWS + r;
            val = *reinterpret_cast<const uint4*>(reinterpret_cast<const AT*>(P.a) + src_row * a_pitch + k0 + c * 8);
          }
          *reinterpret_cast<uint4*>(xs + r * F::XPITCH + c * 16) = val;
        }
      }
      if constexpr (!GEMM1) {
        // which slots of the token of route `warp` count in the combine
        const int sidv = aux->sid[warp];
        bool ok = false;
        if (sidv >= 0 && lane < P.topk) {
          const int64_t tok = sidv / P.topk;
          const long long id = P.ids_int64 ? ((const long long*)P.topk_ids)[tok * P.topk + lane]
                                           : (long long)((const int32_t*)P.topk_ids)[tok * P.topk + lane];
          ok = id >= 0 && id < P.num_experts_global && (P.expert_map == nullptr || P.expert_map[id] >= 0);
        }
        const uint32_t m = __ballot_sync(0xFFFFFFFFu, ok);
        if (lane == 0) aux->mask[warp] = m;
      }
      bar_compute();
      }  // staging of a new (block, slice)

      // FP8: weight scales of this warp's two row groups, chunk l of the slice in lane l
      [[maybe_unused]] float swA_l = 0.0f, swB_l = 0.0f;
      if constexpr (FP8) {
        const int sblk = (P.rows_w + 127) / 128, kbt = P.K / 128;
        if (lane < nchunks) {
          const int wrA = GEMM1 ? nt * 64 : nt * TILE_W, wrB = GEMM1 ? P.Nout + nt * 64 : nt * TILE_W;
          swA_l = P.w_scale[((int64_t)e * sblk + (wrA >> 7)) * kbt + c0 + lane];
          swB_l = GEMM1 ? P.w_scale[((int64_t)e * sblk + (wrB >> 7)) * kbt + c0 + lane] : swA_l;
        }
      }

      // ---------------------------------------------------------------- K loop over the slice
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
      [[maybe_unused]] float acc2[4] = {0.f, 0.f, 0.f, 0.f};
      const uint8_t* x_row = xs + g * F::XPITCH;
      for (int ci = 0; ci < nchunks; ++ci, ++it) {
        const int st = it % STAGES;
        if (!mbar_wait(&aux->full[st], (it / STAGES) & 1, P.status, P.wait_ns)) { alive = false; break; }
        const uint8_t* sa = ring + (size_t)st * STAGE_BYTES + rowA * 128;
        const uint8_t* sb = ring + (size_t)st * STAGE_BYTES + rowB * 128;
                if constexpr (MODE == MOE_MODE_HALF) {
          uint4 wa[2], wb[2], xv[2];
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const int phys = ((q + 4 * j) ^ g) << 4;
            wa[j] = lds128(sa + phys);
            wb[j] = lds128(sb + phys);
            xv[j] = lds128(x_row + (ci * 64 + 32 * j + 8 * q) * 2);
          }
          // two accumulators: consecutive MMAs do not wait for each other
          mma_half<AT>(acc, wa[0].x, wb[0].x, wa[0].y, wb[0].y, xv[0].x, xv[0].y);
          mma_half<AT>(acc2, wa[0].z, wb[0].z, wa[0].w, wb[0].w, xv[0].z, xv[0].w);
          mma_half<AT>(acc, wa[1].x, wb[1].x, wa[1].y, wb[1].y, xv[1].x, xv[1].y);
          mma_half<AT>(acc2, wa[1].z, wb[1].z, wa[1].w, wb[1].w, xv[1].z, xv[1].w);
        } else if constexpr (FP8) {
          uint2 wa[4], wb[4], xv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int phys = (((2 * j + (q >> 1)) ^ g) << 4) + 8 * (q & 1);
            wa[j] = lds64(sa + phys);
            wb[j] = lds64(sb + phys);
            xv[j] = lds64(x_row + ci * 128 + 32 * j + 8 * q);
          }
          const float swA = __shfl_sync(0xFFFFFFFFu, swA_l, ci), swB = __shfl_sync(0xFFFFFFFFu, swB_l, ci);
          const float x0 = aux->sx[2 * q][ci], x1 = aux->sx[2 * q + 1][ci];
          float d[4] = {0.f, 0.f, 0.f, 0.f}, d2[4] = {0.f, 0.f, 0.f, 0.f};
          mma_e4m3(d, wa[0].x, wb[0].x, wa[0].y, wb[0].y, xv[0].x, xv[0].y);
          mma_e4m3(d2, wa[1].x, wb[1].x, wa[1].y, wb[1].y, xv[1].x, xv[1].y);
          mma_e4m3(d, wa[2].x, wb[2].x, wa[2].y, wb[2].y, xv[2].x, xv[2].y);
          mma_e4m3(d2, wa[3].x, wb[3].x, wa[3].y, wb[3].y, xv[3].x, xv[3].y);
          // one K block done: acc += part * (a_scale[route] * w_scale[block])
          acc[0] = fmaf(d[0] + d2[0], x0 * swA, acc[0]);
          acc[1] = fmaf(d[1] + d2[1], x1 * swA, acc[1]);
          acc[2] = fmaf(d[2] + d2[2], x0 * swB, acc[2]);
          acc[3] = fmaf(d[3] + d2[3], x1 * swB, acc[3]);
        } else {
          uint2 wa[4], wb[4];
          uint4 xv[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int phys = (((2 * j + (q >> 1)) ^ g) << 4) + 8 * (q & 1);
            wa[j] = lds64(sa + phys);
            wb[j] = lds64(sb + phys);
            xv[j] = lds128(x_row + (ci * 128 + 32 * j + 8 * q) * 2);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t a01, a23, a45, a67, b01, b23, b45, b67;
            tc::widen4<AT>(wa[j].x, a01, a23);
            tc::widen4<AT>(wa[j].y, a45, a67);
            tc::widen4<AT>(wb[j].x, b01, b23);
            tc::widen4<AT>(wb[j].y, b45, b67);
            mma_half<AT>(acc, a01, b01, a23, b23, xv[j].x, xv[j].y);
            mma_half<AT>(acc2, a45, b45, a67, b67, xv[j].z, xv[j].w);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&aux->empty[st]);
      }
      if (!alive) break;
      if constexpr (!FP8) {
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[i] += acc2[i];
      }

      // ---------------------------------------------------------------- this warp's [16 rows x 8 routes]
      // lane (g, q): acc[0], acc[1] = row A of routes 2q, 2q+1; acc[2], acc[3] = row B of the same routes
      float v[4] = {acc[0], acc[1], acc[2], acc[3]};
      const int64_t pr = (int64_t)b * ROWS + 2 * q;  // sorted row of route 2q
      if (P.S > 1) {
        float* mine = P.partial + ((int64_t)s * P.rows_cap + pr) * tile_ld + (int64_t)nt * TILE_W;
        mine[rowA] = v[0]; mine[tile_ld + rowA] = v[1]; mine[rowB] = v[2]; mine[tile_ld + rowB] = v[3];
        __syncwarp();  // the warp's partial sums are written; lane 0 publishes them with its release
        int last = 0;
        if (lane == 0) {
          int32_t* cnt = &P.unit_cnt[((int64_t)b * P.NT + nt) * CWARPS + warp];
          last = atom_add_acq_rel(cnt, 1) == P.S - 1;
          if (last) *cnt = 0;  // ready for the next launch
        }
        last = __shfl_sync(0xFFFFFFFFu, last, 0);
        if (!last) continue;  // the warp of another slice finishes these rows
        v[0] = v[1] = v[2] = v[3] = 0.0f;
        for (int s2 = 0; s2 < P.S; ++s2) {  // slice order, whoever came last
          const float* part = P.partial + ((int64_t)s2 * P.rows_cap + pr) * tile_ld + (int64_t)nt * TILE_W;
          v[0] += ldcg_f(part + rowA); v[1] += ldcg_f(part + tile_ld + rowA);
          v[2] += ldcg_f(part + rowB); v[3] += ldcg_f(part + tile_ld + rowB);
        }
      }
      // weight row (inside the expert) behind tile rows A and B
      const int wrA = GEMM1 ? nt * 64 + 8 * warp + g : nt * TILE_W + rowA;
      const int wrB = GEMM1 ? P.Nout + nt * 64 + 8 * warp + g : nt * TILE_W + rowB;
      if constexpr (W8) {
        const float csA = P.w_scale[(int64_t)e * P.rows_w + wrA], csB = P.w_scale[(int64_t)e * P.rows_w + wrB];
        v[0] *= csA; v[1] *= csA; v[2] *= csB; v[3] *= csB;
      }
      const int sid0 = aux->sid[2 * q], sid1 = aux->sid[2 * q + 1];
      float rw0 = 1.0f, rw1 = 1.0f;
      if (P.mul_weight) {
        if (sid0 >= 0) rw0 = P.route_weight[sid0];
        if (sid1 >= 0) rw1 = P.route_weight[sid1];
      }
      if constexpr (GEMM1) {
        AT* o = reinterpret_cast<AT*>(P.out) + pr * P.Nout + nt * 64 + 8 * warp + g;
        if (sid0 >= 0) o[0] = from_f32<AT>(silu_mul(v[0] * rw0, v[2] * rw0));
        if (sid1 >= 0) o[P.Nout] = from_f32<AT>(silu_mul(v[1] * rw1, v[3] * rw1));
      } else {
        AT* y = reinterpret_cast<AT*>(P.out);
        if (sid0 >= 0) {
          y[(int64_t)sid0 * P.Nout + wrA] = from_f32<AT>(v[0] * rw0);
          y[(int64_t)sid0 * P.Nout + wrB] = from_f32<AT>(v[2] * rw0);
        }
        if (sid1 >= 0) {
          y[(int64_t)sid1 * P.Nout + wrA] = from_f32<AT>(v[1] * rw1);
          y[(int64_t)sid1 * P.Nout + wrB] = from_f32<AT>(v[3] * rw1);
        }
        // ---- join the routes of every token of the block for this warp's 16 columns: the warp
        // that writes a token's last row adds the token's rows in slot order
        __syncwarp();  // the rows are written; the counting lanes publish them with their release
        int last = 0;
        uint32_t mask_r = 0;
        if (lane < ROWS) {
          const int sidr = aux->sid[lane];
          if (sidr >= 0) {
            mask_r = aux->mask[lane];
            int32_t* cnt = &P.tok_cnt[((int64_t)(sidr / P.topk) * P.NT + nt) * CWARPS + warp];
            last = atom_add_acq_rel(cnt, 1) == __popc(mask_r) - 1;
            if (last) *cnt = 0;
          }
        }
        uint32_t todo = __ballot_sync(0xFFFFFFFFu, last != 0);
        while (todo) {
          const int r = __ffs(todo) - 1;
          todo &= todo - 1;
          const int64_t tok = aux->sid[r] / P.topk;
          const uint32_t mk = __shfl_sync(0xFFFFFFFFu, mask_r, r);
          if (lane < 16) {
            const int col = nt * TILE_W + 16 * warp + lane;
            float sum = 0.0f;
            for (int j = 0; j < P.topk; ++j)
              if ((mk >> j) & 1u) sum += ToF32<AT>::get(ldcg_at<AT>(y + (tok * P.topk + j) * P.Nout + col));
            reinterpret_cast<AT*>(P.final_out)[tok * P.Nout + col] = from_f32<AT>(sum);
          }
        }
      }
    }
  }
}

template <int MODE, typename AT, bool GEMM1>
static int launch(const CUtensorMap& map, const Params& P, int grid, cudaStream_t st) {
  using F = Fmt<MODE, AT>;
  auto kern = small_gemm_kernel<MODE, AT, GEMM1>;
  const size_t smem = (size_t)STAGES * STAGE_BYTES + ROWS * F::XPITCH + sizeof(Smem) + 1024;
  cudaError_t ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (ce != cudaSuccess) return fail((int)ce, "small-batch GEMM: shared memory attribute: %s", cudaGetErrorString(ce));
  kern<<<grid, THREADS, smem, st>>>(map, P);
  return check_launch(GEMM1 ? "small-batch gemm1" : "small-batch gemm2");
}

}  // namespace sm

// Scratch sizes of one small-batch GEMM for the caller's allocation.
static int small_plan(bool gemm1, int mode, int K, int Nout, int sms, int64_t rows_cap, int s_hint, sm::Params& P) {
  const int ew = mode == MOE_MODE_HALF ? 2 : 1;
  const int ce = 128 / ew;
  if (K % ce != 0) return fail(MOE_E_SHAPE, "small-batch GEMM: K must be a multiple of %d", ce);
  if (mode == MOE_MODE_FP8_BLOCK && K % 128 != 0) return fail(MOE_E_SHAPE, "small-batch GEMM (fp8): K must be a multiple of 128");
  if (gemm1 && Nout % 64 != 0) return fail(MOE_E_SHAPE, "small-batch GEMM1: intermediate size must be a multiple of 64");
  if (!gemm1 && Nout % 128 != 0) return fail(MOE_E_SHAPE, "small-batch GEMM2: hidden size must be a multiple of 128");
  P.chunks_total = K / ce;
  const int ex = mode == MOE_MODE_FP8_BLOCK ? 1 : 2;
  const int max_chunks = (sm::X_ROW_BYTES / ex) / ce;  // what one unit can hold of the activation rows
  int S = (P.chunks_total + max_chunks - 1) / max_chunks;
  if (s_hint > S) S = s_hint;
  if (S > P.chunks_total) S = P.chunks_total;
  P.cps = (P.chunks_total + S - 1) / S;
  P.S = (P.chunks_total + P.cps - 1) / P.cps;
  P.NT = gemm1 ? Nout / 64 : Nout / sm::TILE_W;
  (void)sms; (void)rows_cap;
  return 0;
}

}  // namespace moe

extern "C" int moe_small_m_plan(int gemm1, int mode, int K, int Nout, int64_t rows_cap, int64_t num_tokens, int k_slices,
                                int64_t* partial_floats, int64_t* unit_counters, int64_t* token_counters) {
  using namespace moe;
  sm::Params P;
  int rc = small_plan(gemm1 != 0, mode, K, Nout, 0, rows_cap, k_slices, P);
  if (rc) return rc;
  if (rows_cap % sm::ROWS != 0) return fail(MOE_E_SHAPE, "small-batch GEMM: row capacity must be a multiple of %d", sm::ROWS);
  if (partial_floats) *partial_floats = P.S > 1 ? (int64_t)P.S * rows_cap * P.NT * sm::TILE_W : 0;
  if (unit_counters) *unit_counters = (rows_cap / sm::ROWS) * P.NT * sm::CWARPS;
  if (token_counters) *token_counters = gemm1 ? 0 : num_tokens * P.NT * sm::CWARPS;
  return 0;
}

extern "C" int moe_small_m_gemm(int gemm1, int mode, int act_dtype, const void* a, int64_t num_tokens, int topk,
                                const void* w, const float* w_scale, const int32_t* expert_ids,
                                const int32_t* sorted_ids, const int32_t* num_post_pad, const int32_t* expert_map,
                                int num_experts_global, const float* route_weight, int mul_weight,
                                const void* topk_ids, int ids_int64, int64_t rows_cap, int E, int K, int Nout,
                                void* out, void* final_out, int k_slices, float* partial, int32_t* unit_counters,
                                int32_t* token_counters, int32_t* status, void* stream) {
  using namespace moe;
  using namespace moe::sm;
  if (num_tokens < 0 || topk <= 0 || topk > 32 || rows_cap < 0 || E <= 0 || K <= 0 || Nout <= 0)
    return fail(MOE_E_BADARG, "small-batch GEMM: bad extent (topk must be 1..32)");
  if (rows_cap == 0 || num_tokens == 0) return 0;
  if (!a || !w || !expert_ids || !sorted_ids || !num_post_pad || !out || !unit_counters)
    return fail(MOE_E_BADARG, "small-batch GEMM: null pointer");
  if (mul_weight && !route_weight) return fail(MOE_E_BADARG, "small-batch GEMM: route weights missing");
  if (!gemm1 && (!final_out || !topk_ids || !token_counters))
    return fail(MOE_E_BADARG, "small-batch GEMM2: output, topk_ids or token counters missing");
  if (mode != MOE_MODE_HALF && !w_scale) return fail(MOE_E_BADARG, "small-batch GEMM: weight scales missing");
  if (mode != MOE_MODE_HALF && mode != MOE_MODE_FP8_BLOCK && mode != MOE_MODE_W8A16)
    return fail(MOE_E_SHAPE, "small-batch GEMM: unknown mode %d", mode);
  if (act_dtype != MOE_BF16 && act_dtype != MOE_F16) return fail(MOE_E_DTYPE, "small-batch GEMM: activations must be f16 or bf16");
  if (((uintptr_t)a & 15) || ((uintptr_t)out & 15) || (final_out && ((uintptr_t)final_out & 7)))
    return fail(MOE_E_BADARG, "small-batch GEMM: buffers must be 16-byte aligned");
  Params P;
  int rc = small_plan(gemm1 != 0, mode, K, Nout, 0, rows_cap, k_slices, P);
  if (rc) return rc;
  if (rows_cap % ROWS != 0) return fail(MOE_E_SHAPE, "small-batch GEMM: row capacity must be a multiple of %d", ROWS);
  if (P.S > 1 && !partial) return fail(MOE_E_BADARG, "small-batch GEMM: %d K slices need the partial-sum scratch", P.S);
  const int rows_w = gemm1 ? 2 * Nout : Nout;
  if ((int64_t)E * rows_w >= (1ll << 31)) return fail(MOE_E_TOOBIG, "small-batch GEMM: extent exceeds int32 coordinates");
  const int eb = mode == MOE_MODE_HALF ? 2 : 1;
  const CUtensorMapDataType dt = mode != MOE_MODE_HALF ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : (act_dtype == MOE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUtensorMap map;
  rc = tc::make_map(&map, w, dt, eb, (uint64_t)E * rows_w, (uint64_t)K, gemm1 ? 64 : TILE_W, true);
  if (rc) return rc;
  P.a = a; P.w_scale = w_scale; P.expert_ids = expert_ids; P.sorted_ids = sorted_ids; P.num_post_pad = num_post_pad;
  P.expert_map = expert_map; P.route_weight = route_weight; P.topk_ids = topk_ids; P.out = out; P.final_out = final_out;
  P.partial = partial; P.unit_cnt = unit_counters; P.tok_cnt = token_counters; P.status = status; P.wait_ns = wait_limit_ns();
  P.numel = num_tokens * topk; P.rows_cap = rows_cap; P.tokens = num_tokens; P.ids_int64 = ids_int64;
  P.num_experts_global = num_experts_global; P.topk = gemm1 ? topk : topk; P.mul_weight = mul_weight; P.E = E; P.K = K;
  P.Nout = Nout; P.rows_w = rows_w;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t cap_units = (rows_cap / ROWS) * (int64_t)P.NT * P.S;
  const int grid = (int)(cap_units < sms ? cap_units : sms);
  cudaStream_t st = (cudaStream_t)stream;
#define MOE_SM_LAUNCH(M, T) (gemm1 ? launch<M, T, true>(map, P, grid, st) : launch<M, T, false>(map, P, grid, st))
#define MOE_SM_MODE(M) (act_dtype == MOE_BF16 ? MOE_SM_LAUNCH(M, __nv_bfloat16) : MOE_SM_LAUNCH(M, __half))
  if (mode == MOE_MODE_HALF) return MOE_SM_MODE(MOE_MODE_HALF);
  if (mode == MOE_MODE_FP8_BLOCK) return MOE_SM_MODE(MOE_MODE_FP8_BLOCK);
  return MOE_SM_MODE(MOE_MODE_W8A16);
#undef MOE_SM_MODE
#undef MOE_SM_LAUNCH
}

// ---------------------------------------------------------------------------------------------
// GEMM 2 of the small-batch schedule for hosts that cannot allocate.
//
// A serving engine that has handed every free byte of device memory to its own pools at
// start-up has nothing left for cudaMalloc to give, and cudaMalloc / cudaFree stall the whole
// device while they run, which a decode loop cannot afford between two kernels.  Such a host can
// call this entry point: it takes the same inputs and the same output as moe_small_m_gemm with
// gemm1 = 0, and keeps everything else -- the route rows y, the split-K partial sums and the two
// counter tables -- in the fixed array below, which lives in the library's device image.
//
//   * The array is kSmallStaticBytes (8 MiB) on every GPU that loads the library, from the load
//     to process exit.  A call whose scratch does not fit is rejected with MOE_E_TOOBIG and the
//     required size in the message; nothing is launched.
//   * No cudaMalloc, cudaFree or other allocating call is made, here or in what it calls.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress, with
//     that device current) and remembers it; make that first call outside any stream capture.
//   * All calls on a device share the one array, and it keeps what the last call left.  The
//     counter tables are cleared on `stream` at the start of every call; the rest is written
//     before it is read.  Two calls whose kernels overlap on the GPU (different streams, no
//     ordering between them) race on it: order them.
static __device__ __align__(256) unsigned char g_small_static[8u << 20];
static constexpr size_t kSmallStaticBytes = 8u << 20;
static unsigned char* g_small_static_ptr[64] = {};  // device address per device ordinal, filled on first use

static int small_static_base(unsigned char** base) {
  using namespace moe;
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return fail((int)ce, "small-batch GEMM2 (static scratch): cudaGetDevice: %s", cudaGetErrorString(ce));
  if (dev < 0 || dev >= 64) return fail(MOE_E_BADARG, "small-batch GEMM2 (static scratch): device ordinal %d not supported", dev);
  if (g_small_static_ptr[dev] == nullptr) {
    // In host code `g_small_static` names a host-side shadow of the symbol, not device memory:
    // the device address has to be asked for, once per device, with that device current.
    unsigned char* p = nullptr;
    ce = cudaGetSymbolAddress((void**)&p, g_small_static);
    if (ce != cudaSuccess || p == nullptr)
      return fail(ce != cudaSuccess ? (int)ce : MOE_E_DRIVER, "small-batch GEMM2 (static scratch): cudaGetSymbolAddress: %s",
                  cudaGetErrorString(ce));
    g_small_static_ptr[dev] = p;
  }
  *base = g_small_static_ptr[dev];
  return 0;
}

extern "C" int moe_small_m_gemm2_static(int mode, int act_dtype, const void* act_sorted, int64_t num_tokens, int topk,
                                        const void* w2, const float* w2_scale, const int32_t* expert_ids,
                                        const int32_t* sorted_ids, const int32_t* num_post_pad,
                                        const int32_t* expert_map, int num_experts_global, const float* route_weight,
                                        int mul_weight, const void* topk_ids, int ids_int64, int64_t rows_cap, int E,
                                        int K, int Nout, void* final_out, int k_slices, int32_t* status, void* stream) {
  using namespace moe;
  if (num_tokens < 0 || topk <= 0 || rows_cap < 0 || Nout <= 0) return fail(MOE_E_BADARG, "small-batch GEMM2 (static scratch): bad extent");
  if (num_tokens == 0 || rows_cap == 0) return 0;
  int64_t partial_floats = 0, unit_counters = 0, token_counters = 0;
  int rc = moe_small_m_plan(0, mode, K, Nout, rows_cap, num_tokens, k_slices, &partial_floats, &unit_counters, &token_counters);
  if (rc) return rc;
  auto up256 = [](size_t v) { return (v + 255) & ~(size_t)255; };
  const size_t counters_bytes = up256((size_t)(unit_counters + token_counters) * sizeof(int32_t));
  const size_t y_bytes = up256((size_t)num_tokens * topk * Nout * 2);  // f16 / bf16 rows
  const size_t partial_bytes = up256((size_t)partial_floats * sizeof(float));
  const size_t need = counters_bytes + y_bytes + partial_bytes;
  if (need > kSmallStaticBytes)
    return fail(MOE_E_TOOBIG, "small-batch GEMM2 (static scratch): this call needs %zu bytes of scratch, the fixed array holds %zu",
                need, kSmallStaticBytes);
  unsigned char* base = nullptr;
  rc = small_static_base(&base);
  if (rc) return rc;
  // the counter tables must start at zero whatever the previous call (or a failed one) left
  cudaError_t ce = cudaMemsetAsync(base, 0, counters_bytes, (cudaStream_t)stream);
  if (ce != cudaSuccess) return fail((int)ce, "small-batch GEMM2 (static scratch): clearing the counters: %s", cudaGetErrorString(ce));
  int32_t* unit_cnt = reinterpret_cast<int32_t*>(base);
  int32_t* tok_cnt = unit_cnt + unit_counters;
  void* y = base + counters_bytes;
  float* partial = partial_floats ? reinterpret_cast<float*>(base + counters_bytes + y_bytes) : nullptr;
  return moe_small_m_gemm(0, mode, act_dtype, act_sorted, num_tokens, topk, w2, w2_scale, expert_ids, sorted_ids, num_post_pad,
                          expert_map, num_experts_global, route_weight, mul_weight, topk_ids, ids_int64, rows_cap, E, K, Nout,
                          y, final_out, k_slices, partial, unit_cnt, tok_cnt, status, stream);
}
