// Weight-only int8 (W8A16) expert grouped GEMMs on the tcgen05 tensor cores.
//
// The reference widens every expert's int8 weights to the activation dtype in
// global memory on every call and then runs its half-precision kernel
// (src/flaggems_vllm/ops/fused_moe.py:2493-2500): one read of the int8 weights,
// one write and one more read of a copy twice their size.  Here the int8 bytes
// are the only weight traffic: TMA streams them into a raw shared-memory ring,
// converter warps widen them EXACTLY (|w| <= 128 has at most 8 significant bits)
// into the 128-byte-swizzled K-major operand tile the tensor core reads, and
// the per-output-channel fp32 scale is applied to the fp32 accumulator in the
// epilogue, so no product is rounded before the scale.
//
// Tile: 128 expert-sorted rows x 256 accumulator columns, 64 K elements per step.
//   raw ring  5 x 16 KB   int8 [256 rows x 64 B], unswizzled, one or two TMA boxes
//   B ring    2 x 32 KB   converted weights, [256 rows x 128 B] swizzled
//   A ring    4 x 16 KB   activations: cp.async gather of token rows (GEMM1) or one TMA box (GEMM2)
// Warp roles (640 threads):
//   warp 0      TMA producer of the raw weight ring
//   warp 1      MMA issuer
//   warp 2      TMEM allocation; GEMM2: TMA producer of the A ring
//   warps 2-3   GEMM1: cp.async gather of the A rows
//   warps 4-7   epilogue: accumulator -> channel scale -> SiLU*up / route weight -> store,
//               two passes of 128 columns per tile
//   warps 8-19  converters: raw int8 -> f16 / bf16 operand tile.  The conversion is integer-ALU
//               work (about 1.5 byte-permute / logic instructions per weight), the limiter
//               of this kernel, hence twelve warps of it.
// Both TMEM accumulators are used, so the epilogue of one tile overlaps the K
// loop of the next.  Every barrier wait is bounded; on expiry the kernel sets
// MOE_ST_WAIT_TIMEOUT, leaves its loops, frees TMEM and returns.
#include "tc_common.cuh"

namespace moe {
namespace w8 {
using namespace tc;

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int KBE = 64;                // K elements per step
constexpr int A_BYTES = BM * 128;
constexpr int B_BYTES = BN * 128;
constexpr int RAW_BYTES = BN * KBE;
constexpr int SA = 4, SB = 2, SR = 5;
#ifndef MOE_W8_CONV_WARPS
#define MOE_W8_CONV_WARPS 12
#define MOE_W8_LAUNCH_REGS 96
#define MOE_W8_CONV_REGS 72
#define MOE_W8_EPI_REGS 208
#endif
constexpr int EPI_WARPS = 4;
constexpr int CONV_WARPS = MOE_W8_CONV_WARPS;
constexpr int THREADS = 256 + 32 * CONV_WARPS;
constexpr int CONV_THREADS = CONV_WARPS * 32;
constexpr int GATHER_THREADS = 64;
// setmaxnreg moves registers inside the CTA's launch allocation (THREADS x LAUNCH_REGS);
// the epilogue's increase must be covered by what the other warps give up.
constexpr int LAUNCH_REGS = MOE_W8_LAUNCH_REGS;
constexpr int PRODUCER_REGS = 56;
constexpr int CONV_REGS = MOE_W8_CONV_REGS;
constexpr int EPI_REGS = MOE_W8_EPI_REGS;
static_assert(128 * PRODUCER_REGS + CONV_THREADS * CONV_REGS + EPI_WARPS * 32 * EPI_REGS <= THREADS * LAUNCH_REGS,
              "register redistribution exceeds the CTA's allocation");
static_assert(THREADS * LAUNCH_REGS <= 65536, "CTA does not fit the register file");

struct Aux {
  float cs[2][BN];  // channel scales of the tile in the epilogue, [gate | up] for GEMM1
  uint64_t a_full[SA], a_empty[SA];
  uint64_t r_full[SR], r_empty[SR];
  uint64_t b_full[SB], b_empty[SB];
  uint64_t tmem_full[2], tmem_empty[2];
  uint32_t tmem_base;
  uint32_t pad;
};
constexpr size_t SMEM_BYTES = (size_t)SA * A_BYTES + (size_t)SB * B_BYTES + (size_t)SR * RAW_BYTES + sizeof(Aux) + 1024;
static_assert(SMEM_BYTES <= 232448, "shared memory of one SM");

struct Params {
  const uint8_t* a_rows;   // GEMM1: activations [tokens, K] in token order
  const float* w_scale;    // [E, rows_w] per-output-channel scale
  const int32_t* expert_ids;
  const int32_t* sorted_ids;
  const int32_t* num_post_pad;
  const float* route_weight;
  void* out;
  int32_t* status;
  unsigned long long wait_ns;  // limit of every bounded barrier wait
  int64_t numel;
  int64_t rows_cap;
  int topk;
  int mul_weight;
  int E;
  int K;
  int Nout;     // output columns (I for GEMM1, H for GEMM2)
  int rows_w;   // weight rows per expert (2I or H)
  int n_tiles;  // column tiles per align block
  bool wide_store;  // the output is 32-byte aligned: rows are written with 32-byte stores
};

// The raw tile is fetched with as few TMA instructions as the weight layout allows: GEMM1
// two boxes of 128 rows (gate rows nt*128.. -> accumulator columns 0-127, the up rows of the
// same outputs -> columns 128-255), GEMM2 one box of 256 consecutive rows.
template <bool GEMM1> struct RawBox {
  static constexpr int COUNT = GEMM1 ? 2 : 1;
  static constexpr int ROWS = GEMM1 ? 128 : 256;
};
template <bool GEMM1>
__device__ __forceinline__ int box_row(int nt, int c, int Nout) {
  if constexpr (GEMM1) return nt * 128 + c * Nout;
  else return nt * BN;
}

// Instruction descriptor: fp32 accumulator, A/B format (f16 = 0, bf16 = 1), both K-major,
// N >> 3 at bit 17, M >> 4 at bit 24.
template <typename AT>
struct IDesc {
  static constexpr uint32_t fmt = std::is_same<AT, __nv_bfloat16>::value ? 1u : 0u;
  static constexpr uint32_t value =
      (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
};

template <typename AT, bool GEMM1>
__global__ void __launch_bounds__(THREADS, 1)
w8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, const Params P) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = sA + (size_t)SA * A_BYTES;
  uint8_t* sR = sB + (size_t)SB * B_BYTES;
  Aux* aux = reinterpret_cast<Aux*>(sR + (size_t)SR * RAW_BYTES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int KB = P.K / KBE;
  const int npp = min((int64_t)P.num_post_pad[0], P.rows_cap);
  const int total_tiles = ((npp + BM - 1) / BM) * P.n_tiles;
  const int tile0 = blockIdx.x, tile_step = gridDim.x;
#define MOE_TILE_COORDS(tile)                         \
  const int blk = (tile) / P.n_tiles;                 \
  [[maybe_unused]] const int nt = (tile) % P.n_tiles; \
  const int e = P.expert_ids[blk];

  if (threadIdx.x == 0) {
    for (int s = 0; s < SA; ++s) {
      mbar_init(&aux->a_full[s], GEMM1 ? GATHER_THREADS : 1);
      mbar_init(&aux->a_empty[s], 1);
    }
    for (int s = 0; s < SR; ++s) {
      mbar_init(&aux->r_full[s], 1);
      mbar_init(&aux->r_empty[s], CONV_WARPS);
    }
    for (int s = 0; s < SB; ++s) {
      mbar_init(&aux->b_full[s], CONV_WARPS);
      mbar_init(&aux->b_empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&aux->tmem_full[a], 1);
      mbar_init(&aux->tmem_empty[a], EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&aux->tmem_base)),
                 "r"(512));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = aux->tmem_base;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PRODUCER_REGS));
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------ raw weight ring (TMA)
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      uint32_t it = 0;
      bool alive = true;
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        const int wrow0 = e * P.rows_w;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % SR;
          if (!mbar_wait(&aux->r_empty[s], ((it / SR) & 1) ^ 1, P.status, P.wait_ns)) { alive = false; break; }
          mbar_expect_tx(&aux->r_full[s], RAW_BYTES);
#pragma unroll
          for (int c = 0; c < RawBox<GEMM1>::COUNT; ++c)
            tma_load_2d(&map_w, &aux->r_full[s], sR + (size_t)s * RAW_BYTES + c * (RawBox<GEMM1>::ROWS * KBE), kb * KBE,
                        wrow0 + box_row<GEMM1>(nt, c, P.Nout));
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = IDesc<AT>::value;
      uint32_t it = 0, acc_it = 0;
      bool alive = true;
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        const uint32_t a = acc_it & 1;
        if (!mbar_wait(&aux->tmem_empty[a], ((acc_it >> 1) & 1) ^ 1, P.status, P.wait_ns)) { alive = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int sa = it % SA, sb = it % SB;
          if (!mbar_wait(&aux->a_full[sa], (it / SA) & 1, P.status, P.wait_ns)) { alive = false; break; }
          if (!mbar_wait(&aux->b_full[sb], (it / SB) & 1, P.status, P.wait_ns)) { alive = false; break; }
          if constexpr (GEMM1) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // cp.async writes -> tensor core reads
          tc_fence_after();
          const uint64_t adesc = make_smem_desc(smem_u32(sA + (size_t)sa * A_BYTES));
          const uint64_t bdesc = make_smem_desc(smem_u32(sB + (size_t)sb * B_BYTES));
          const uint32_t d = tmem_base + a * BN;
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4)  // 32 bytes (16 elements) of K per instruction
            tc_mma<false>(d, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, (kb > 0 || k4 > 0) ? 1u : 0u);
          tc_commit(&aux->a_empty[sa]);
          tc_commit(&aux->b_empty[sb]);
        }
        if (!alive) break;
        tc_commit(&aux->tmem_full[a]);
        ++acc_it;
      }
    } else if (!GEMM1 && warp == 2 && lane == 0) {
      // ------------------------------------------------------------ A ring of GEMM2 (TMA)
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      uint32_t it = 0;
      bool alive = true;
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % SA;
          if (!mbar_wait(&aux->a_empty[s], ((it / SA) & 1) ^ 1, P.status, P.wait_ns)) { alive = false; break; }
          mbar_expect_tx(&aux->a_full[s], A_BYTES);
          tma_load_2d(&map_a, &aux->a_full[s], sA + (size_t)s * A_BYTES, kb * KBE, blk * BM);
        }
      }
    } else if (GEMM1 && warp >= 2) {
      // ------------------------------------------------------------ A-row gather (cp.async)
      // Two lanes share a row: lane pair q copies the 32-byte sector {2c, 2c+1} of rows
      // q + 32 j in step c, so every warp instruction fetches 16 whole sectors.
      const int g = threadIdx.x - 64;  // 0..63
      const int q = g >> 1, half = g & 1;
      const int64_t pitch = (int64_t)P.K * 2;
      uint32_t it = 0;
      bool alive = true;
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        const uint8_t* src[4];
        bool ok[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int64_t p = (int64_t)blk * BM + q + 32 * j;
          const int64_t sid = p < P.rows_cap ? (int64_t)P.sorted_ids[p] : P.numel;
          ok[j] = sid >= 0 && sid < P.numel;  // padding slot: the row keeps stale bytes, its results are never stored
          src[j] = P.a_rows + (ok[j] ? sid / P.topk : 0) * pitch + half * 16;
        }
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % SA;
          if (!mbar_wait(&aux->a_empty[s], ((it / SA) & 1) ^ 1, P.status, P.wait_ns)) { alive = false; break; }
          const uint32_t base = smem_u32(sA + (size_t)s * A_BYTES);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (ok[j]) {
              const int r = q + 32 * j;
              const uint8_t* sp = src[j] + (int64_t)kb * 128;
#pragma unroll
              for (int c = 0; c < 4; ++c)  // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
                cp_async16(base + (uint32_t)r * 128u + (uint32_t)(((2 * c + half) ^ (r & 7)) << 4), sp + c * 32);
            }
          }
          cp_async_arrive_noinc(&aux->a_full[s]);
        }
      }
      asm volatile("cp.async.wait_all;" ::: "memory");
    }
  } else if (warp < 4 + EPI_WARPS) {
    // -------------------------------------------------------------- epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(EPI_REGS));
    const int row = ((warp & 3) << 5) + lane;  // accumulator lane = tile row
    const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) << 5) << 16);
    uint32_t acc_it = 0;
    bool alive = true;
    // the tile loop runs to its end even after a wait has timed out: every epilogue thread must
    // reach the barrier of every tile
    for (int tile = tile0; tile < total_tiles; tile += tile_step) {
      MOE_TILE_COORDS(tile)
      if (e < 0 || e >= P.E) continue;
      const int64_t p = (int64_t)blk * BM + row;
      int64_t sid = P.numel;
      if (p < P.rows_cap) sid = (int64_t)P.sorted_ids[p];
      const bool row_ok = sid >= 0 && sid < P.numel;
      float rw = 1.0f;
      if (P.mul_weight && row_ok) rw = P.route_weight[sid];
      // the tile's 256 channel scales go through shared memory (two per thread, loaded while the
      // K loop of the tile is still running); the buffer alternates per tile, so one barrier
      // of the four epilogue warps per tile orders writes against the previous reads
      float* cs = aux->cs[acc_it & 1];
      {
        const float* gs = P.w_scale + (int64_t)e * P.rows_w;
        const int et = threadIdx.x - 128;
#pragma unroll
        for (int j = et; j < BN; j += EPI_WARPS * 32) {
          int col;
          if constexpr (GEMM1) col = nt * 128 + (j & 127) + (j >> 7) * P.Nout;
          else col = nt * BN + j;
          cs[j] = col < P.rows_w ? gs[col] : 0.0f;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(EPI_WARPS * 32) : "memory");
      }
      if (!alive) continue;
      const uint32_t a = acc_it & 1;
      if (!mbar_wait_idle(&aux->tmem_full[a], (acc_it >> 1) & 1, P.status, P.wait_ns)) { alive = false; continue; }
      tc_fence_after();
#pragma unroll 1
      for (int h = 0; h < 2; ++h) {
        float acc[128];
        uint32_t* r = reinterpret_cast<uint32_t*>(acc);
        // GEMM1: gate columns [64h, 64h+64) and up columns [128+64h, ...); GEMM2: [128h, 128h+128)
        const uint32_t t0 = t_lane + a * BN + (uint32_t)(h * (GEMM1 ? 64 : 128));
        tmem_ld64_sync(t0, r, r + 32);
        tmem_ld64_sync(t0 + (GEMM1 ? 128 : 64), r + 64, r + 96);
        if (h == 1) {  // the whole accumulator is in registers or stored: hand it back
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&aux->tmem_empty[a]);
        }
        if (!row_ok) continue;
        if constexpr (GEMM1) {
          // acc[0..63] gate, acc[64..127] up of output columns nt*128 + 64h + j
          const int n0 = nt * 128 + 64 * h;
          const float4* sg4 = reinterpret_cast<const float4*>(cs + 64 * h);
          const float4* su4 = reinterpret_cast<const float4*>(cs + 128 + 64 * h);
#pragma unroll
          for (int j4 = 0; j4 < 16; ++j4) {
            const float4 sg = sg4[j4], su = su4[j4];
            const float gs[4] = {sg.x, sg.y, sg.z, sg.w}, us[4] = {su.x, su.y, su.z, su.w};
#pragma unroll
            for (int q = 0; q < 4; ++q)
              acc[4 * j4 + q] = silu_mul_fast(acc[4 * j4 + q] * gs[q] * rw, acc[64 + 4 * j4 + q] * us[q] * rw);
          }
          uint4 pieces[8];
#pragma unroll
          for (int v = 0; v < 8; ++v)
            pieces[v] = make_uint4(pack2<AT>(acc[v * 8 + 0], acc[v * 8 + 1]), pack2<AT>(acc[v * 8 + 2], acc[v * 8 + 3]),
                                   pack2<AT>(acc[v * 8 + 4], acc[v * 8 + 5]), pack2<AT>(acc[v * 8 + 6], acc[v * 8 + 7]));
          store_row_pieces(reinterpret_cast<AT*>(P.out) + p * P.Nout + n0, pieces, P.wide_store);
        } else {
          const int n0 = nt * BN + 128 * h;
          const float4* s4 = reinterpret_cast<const float4*>(cs + 128 * h);
          AT* o = reinterpret_cast<AT*>(P.out) + sid * P.Nout + n0;
#pragma unroll
          for (int v = 0; v < 16; v += 2) {
            if (n0 + v * 8 < P.Nout) {  // Nout is a multiple of 64: the two pieces are in or out together
              uint4 pieces[2];
#pragma unroll
              for (int u = 0; u < 2; ++u) {
                const float4 s0 = s4[2 * (v + u)], s1 = s4[2 * (v + u) + 1];
                pieces[u] = make_uint4(pack2<AT>(acc[(v + u) * 8 + 0] * s0.x * rw, acc[(v + u) * 8 + 1] * s0.y * rw),
                                       pack2<AT>(acc[(v + u) * 8 + 2] * s0.z * rw, acc[(v + u) * 8 + 3] * s0.w * rw),
                                       pack2<AT>(acc[(v + u) * 8 + 4] * s1.x * rw, acc[(v + u) * 8 + 5] * s1.y * rw),
                                       pack2<AT>(acc[(v + u) * 8 + 6] * s1.z * rw, acc[(v + u) * 8 + 7] * s1.w * rw));
              }
              store_row_pieces(o + v * 8, pieces, P.wide_store);
            }
          }
        }
      }
      ++acc_it;
    }
  } else {
    // -------------------------------------------------------------- converters
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(CONV_REGS));
    const int c = threadIdx.x - (THREADS - CONV_THREADS);
    uint32_t it = 0;
    bool alive = true;
    for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
      MOE_TILE_COORDS(tile)
      if (e < 0 || e >= P.E) continue;
      for (int kb = 0; kb < KB; ++kb, ++it) {
        const int sr = it % SR, sb = it % SB;
        if (!mbar_wait(&aux->r_full[sr], (it / SR) & 1, P.status, P.wait_ns)) { alive = false; break; }
        if (!mbar_wait(&aux->b_empty[sb], ((it / SB) & 1) ^ 1, P.status, P.wait_ns)) { alive = false; break; }
        const uint8_t* raw = sR + (size_t)sr * RAW_BYTES;
        uint8_t* dst = sB + (size_t)sb * B_BYTES;
        // 1024 chunks of 16 int8; chunk q = 16 K elements (q & 3) of weight row q >> 2.  A warp
        // reads 512 contiguous bytes and writes 8 whole 128-byte rows: no bank conflicts.
        constexpr int ROUNDS = (1024 + CONV_THREADS - 1) / CONV_THREADS;
        uint4 v[ROUNDS];
#pragma unroll
        for (int i = 0; i < ROUNDS; ++i)
          if (c + CONV_THREADS * i < 1024) v[i] = *reinterpret_cast<const uint4*>(raw + (size_t)(c + CONV_THREADS * i) * 16);
#pragma unroll
        for (int i = 0; i < ROUNDS; ++i) {
          const int q = c + CONV_THREADS * i;
          if (q < 1024) {
            const int wr = q >> 2, ch = q & 3;
            uint32_t o[8];
            widen4<AT>(v[i].x, o[0], o[1]);
            widen4<AT>(v[i].y, o[2], o[3]);
            widen4<AT>(v[i].z, o[4], o[5]);
            widen4<AT>(v[i].w, o[6], o[7]);
            uint8_t* rowp = dst + (size_t)wr * 128;
            *reinterpret_cast<uint4*>(rowp + (((2 * ch) ^ (wr & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(rowp + (((2 * ch + 1) ^ (wr & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // these stores -> tensor core reads
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&aux->b_full[sb]);
          mbar_arrive(&aux->r_empty[sr]);
        }
      }
    }
  }

  // -------------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
#undef MOE_TILE_COORDS
}

template <typename AT, bool GEMM1>
static int launch(const CUtensorMap& ma, const CUtensorMap& mw, const Params& P, int grid, cudaStream_t st) {
  auto kern = w8_gemm_kernel<AT, GEMM1>;
  cudaFuncAttributes fa;
  cudaError_t ce = cudaFuncGetAttributes(&fa, kern);
  if (ce != cudaSuccess) return fail((int)ce, "int8-weight GEMM: cudaFuncGetAttributes: %s", cudaGetErrorString(ce));
  // refuse to launch rather than let setmaxnreg.inc wait for registers that do not exist
  if (128 * PRODUCER_REGS + CONV_THREADS * CONV_REGS + EPI_WARPS * 32 * EPI_REGS > THREADS * fa.numRegs ||
      fa.numRegs < CONV_REGS)
    return fail(MOE_E_DRIVER, "int8-weight GEMM: kernel was built with %d registers per thread, %d needed",
                fa.numRegs, LAUNCH_REGS);
  ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  if (ce != cudaSuccess) return fail((int)ce, "int8-weight GEMM: shared memory attribute: %s", cudaGetErrorString(ce));
  kern<<<grid, THREADS, SMEM_BYTES, st>>>(ma, mw, P);
  return check_launch(GEMM1 ? "gemm1 (int8 weights, tcgen05)" : "gemm2 (int8 weights, tcgen05)");
}

}  // namespace w8

// gemm1: `a` holds [a_tokens, K] activations in token order; gemm2: [rows_cap, K] rows in sorted order.
// `w` is int8 [E, rows_w, K], `w_scale` fp32 [E, rows_w].
int w8_gemm(bool gemm1, int act_dtype, const void* a, const void* w, const float* w_scale, const int32_t* expert_ids,
            const int32_t* sorted_ids, const int32_t* npp, const float* route_weight, int mul_weight, int64_t numel,
            int64_t rows_cap, int64_t a_tokens, int topk, int block_m, int E, int K, int Nout, void* out,
            int32_t* status, cudaStream_t st) {
  using namespace w8;
  if (act_dtype != MOE_BF16 && act_dtype != MOE_F16)
    return fail(MOE_E_DTYPE, "int8-weight tensor-core GEMM: activations must be f16 or bf16");
  if (block_m != BM) return fail(MOE_E_SHAPE, "int8-weight tensor-core GEMM: align block must be %d", BM);
  if (rows_cap % BM != 0 || rows_cap <= 0)
    return fail(MOE_E_SHAPE, "int8-weight tensor-core GEMM: row capacity must be a positive multiple of %d", BM);
  if (K % KBE != 0) return fail(MOE_E_SHAPE, "int8-weight tensor-core GEMM: K must be a multiple of %d", KBE);
  if (gemm1 && Nout % 128 != 0)
    return fail(MOE_E_SHAPE, "int8-weight tensor-core GEMM1: intermediate size must be a multiple of 128");
  if (!gemm1 && Nout % 64 != 0)
    return fail(MOE_E_SHAPE, "int8-weight tensor-core GEMM2: hidden size must be a multiple of 64");
  if (((uintptr_t)w_scale & 15) != 0 || ((uintptr_t)out & 15) != 0)
    return fail(MOE_E_BADARG, "int8-weight tensor-core GEMM: scales and output must be 16-byte aligned");
  const int rows_w = gemm1 ? 2 * Nout : Nout;
  if ((int64_t)E * rows_w >= (1ll << 31) || rows_cap >= (1ll << 31))
    return fail(MOE_E_TOOBIG, "int8-weight tensor-core GEMM: extent exceeds int32 coordinates");

  CUtensorMap ma, mw;
  int rc = 0;
  if (gemm1) {
    memset(&ma, 0, sizeof(ma));  // A rows are gathered with cp.async, no tensor map
    if (((uintptr_t)a & 15) != 0) return fail(MOE_E_BADARG, "int8-weight tensor-core GEMM1: activations not 16-byte aligned");
    if (topk <= 0 || a_tokens * topk != numel) return fail(MOE_E_BADARG, "int8-weight tensor-core GEMM1: tokens * topk != numel");
  } else {
    rc = make_map(&ma, a, act_dtype == MOE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  (uint64_t)rows_cap, (uint64_t)K, BM, false);
    if (rc) return rc;
  }
  rc = make_map(&mw, w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, (uint64_t)E * rows_w, (uint64_t)K, gemm1 ? 128 : 256, true, KBE);
  if (rc) return rc;

  Params P;
  P.a_rows = (const uint8_t*)a; P.w_scale = w_scale; P.expert_ids = expert_ids; P.sorted_ids = sorted_ids;
  P.num_post_pad = npp; P.route_weight = route_weight; P.out = out; P.status = status; P.wait_ns = wait_limit_ns(); P.numel = numel;
  P.rows_cap = rows_cap; P.topk = gemm1 ? topk : 1; P.mul_weight = mul_weight; P.E = E; P.K = K; P.Nout = Nout;
  P.rows_w = rows_w; P.n_tiles = gemm1 ? Nout / 128 : (Nout + BN - 1) / BN;
  P.wide_store = ((uintptr_t)out & 31) == 0;

  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t cap_tiles = (rows_cap / BM) * (int64_t)P.n_tiles;
  const int grid = (int)(cap_tiles < sms ? cap_tiles : sms);
  if (act_dtype == MOE_BF16)
    return gemm1 ? launch<__nv_bfloat16, true>(ma, mw, P, grid, st) : launch<__nv_bfloat16, false>(ma, mw, P, grid, st);
  return gemm1 ? launch<__half, true>(ma, mw, P, grid, st) : launch<__half, false>(ma, mw, P, grid, st);
}

}  // namespace moe
