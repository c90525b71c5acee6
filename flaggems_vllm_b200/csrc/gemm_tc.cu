// Expert grouped GEMMs on the 5th-generation tensor cores (tcgen05 / TMEM),
// fed by TMA.  One persistent CTA per SM walks a static list of
// (align block, column tile) pairs.
//
// Tile: 128 expert-sorted rows x 256 accumulator columns, K consumed 128 bytes
// per pipeline stage (128 e4m3 or 64 half elements = one 128-byte swizzle row).
//   A stage : 128 rows x 128 B.  GEMM2 reads its (already expert-sorted) input
//             with one TMA box.  GEMM1 gathers token rows: row p of the tile is
//             token sorted_ids[p] / topk, copied by 64 producer threads with
//             16-byte cp.async into the same 128-byte-swizzled layout TMA
//             would produce, so no sorted copy of the activations ever exists.
//             Two lanes share a row, so every 32-byte sector is requested once.
//   B stage : 256 rows x 128 B
// GEMM1 fetches it as two TMA boxes, 128 gate rows and the 128 up rows of the same
// 128 outputs, so one accumulator holds gate (columns 0-127) and up (128-255) of
// an output column in the same thread and SiLU(gate)*up plus the 1x128
// re-quantisation are done in registers.  GEMM2 fetches one box of 256 rows.
//
// Warp roles (384 threads):
//   warp 0      TMA producer (one lane)
//   warp 1      MMA issuer (one lane): tcgen05.mma, tcgen05.commit
//   warp 2      TMEM allocation (512 columns = two 256-column accumulators)
//   warps 2-3   GEMM1 only: cp.async gather of the A rows (2 rows per thread)
//   warps 4-11  accumulator consumers, two groups of four warps; group h owns
//               accumulator columns [128h, 128h+128) (GEMM1: gate [64h, 64h+64) and
//               up [128+64h, 128+64h+64)), warp w lanes 32*(w%4)...
// FP8 block-scaled mode: the tensor core cannot apply fp32 128x128 / 1x128
// scales, so every 128-wide K block is multiplied into a fresh TMEM
// accumulator (the two accumulators alternate) and the consumer warps fold it
// into fp32 registers with acc += part * (a_scale[row] * w_scale[block]), the
// arithmetic of the reference kernel (src/flaggems_vllm/ops/fused_moe.py:1708-1722),
// while the tensor core works on the next block.  The fold keeps two
// tcgen05.ld in flight and hands the accumulator
// back to the tensor core before its last FMAs.  The scales of the K blocks
// in flight sit in a small shared-memory ring filled by the producer side, so
// the consumers issue no global loads inside the K loop.
// Half mode: the whole K loop accumulates in TMEM; the two accumulators let
// the epilogue of one tile overlap the main loop of the next.
//
// Every barrier wait is bounded (wall-clock limit); on expiry the kernel sets
// MOE_ST_WAIT_TIMEOUT, leaves its loops, frees TMEM and returns.
#include "tc_common.cuh"
#ifdef MOE_TC_TRACE
#include <cstdlib>
#endif

namespace moe {
namespace tc {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int A_STAGE_BYTES = BM * 128;
constexpr int B_STAGE_BYTES = BN * 128;       // whole B tile (single-CTA kernel)
constexpr int B_HALF_BYTES = B_STAGE_BYTES / 2;  // what each CTA of a pair holds
constexpr int MAX_STAGES = 6;
// single CTA: 4 stages of A + B; CTA pair (cta_group::2): 6 stages of A + half of B;
// wide tile (RB = 2, half precision only): 3 stages of two A blocks + B, i.e. a 256x256
// output tile whose two accumulators fill TMEM, each B tile fetched once per 256 rows;
// wide pair: 4 stages of two A blocks + half of B, a 512x256 tile per pair, each B tile
// fetched once per 512 rows and each CTA loading only half of it
template <bool PAIR, int RB> struct Cfg {
  static constexpr int STAGES = PAIR ? (RB == 2 ? 4 : 6) : (RB == 2 ? 3 : 4);
  static constexpr int A_LOCAL = RB * A_STAGE_BYTES;
  static constexpr int STAGE_BYTES = A_LOCAL + (PAIR ? B_HALF_BYTES : B_STAGE_BYTES);
};
constexpr int THREADS = 384;
constexpr int EPI_THREADS = 256;
constexpr int GATHER_THREADS = 64;  // warps 2-3 (GEMM1)
constexpr int SCALE_THREADS = 32;   // warp 3 (FP8 GEMM2): scale staging
constexpr int SCALE_SLOTS = 8;
// setmaxnreg only moves registers inside the allocation the CTA got at launch
// (THREADS x the per-thread count ptxas reports under __launch_bounds__, 168).
// The consumers' increase must be covered by what the producer group gives
// up, otherwise setmaxnreg.inc waits forever.
constexpr int LAUNCH_REGS = 168;
constexpr int PRODUCER_REGS = 56;
constexpr int CONSUMER_REGS = 224;
static_assert((THREADS - EPI_THREADS) * PRODUCER_REGS + EPI_THREADS * CONSUMER_REGS <= THREADS * LAUNCH_REGS,
              "register redistribution exceeds the CTA's allocation");
static_assert(THREADS * LAUNCH_REGS <= 65536, "CTA does not fit the register file");

struct SmemAux {
  uint64_t full[MAX_STAGES];       // this CTA's operands (and scales) of the stage have landed
  uint64_t empty[MAX_STAGES];      // the tensor core has finished reading the stage
  uint64_t peer_full[MAX_STAGES];  // pair leader only: the partner CTA's stage has landed
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t xch_bar;
  uint32_t tmem_base;
  uint32_t pad;
  float xch[2][2][BM];  // [tile parity][consumer group][row] amax exchange
  // FP8: scales of the K blocks in flight, written by the producer-side threads
  // with cp.async and read by the consumers.  The ring is deeper than
  // STAGES + the two accumulators, so a slot is never rewritten before the
  // consumers have read it.
  float sc_a[SCALE_SLOTS][BM];  // activation scale of each tile row
  float sc_w[SCALE_SLOTS][4];   // weight scales of the two column halves
};
constexpr int OUT_STAGE_BYTES = BM * BN * 2;  // staged output tile of the TMAOUT variant
template <bool PAIR, int RB, bool TMAOUT = false> constexpr size_t smem_bytes() {
  return TMAOUT ? (size_t)3 * Cfg<PAIR, RB>::STAGE_BYTES + sizeof(SmemAux) + 1024 + OUT_STAGE_BYTES + 1024
                : (size_t)Cfg<PAIR, RB>::STAGES * Cfg<PAIR, RB>::STAGE_BYTES + sizeof(SmemAux) + 1024;
}

struct Params {
  const uint8_t* a_rows;    // GEMM1: activations [tokens, K] in token order (gathered by cp.async)
  const float* a_scales_t;  // [K/128, a_scale_ld]        (FP8)
  const float* w_scale;     // FP8: [E, rows_w/128, K/128]; half mode: optional per-row scale [E, rows_w]
  const int32_t* expert_ids;
  const int32_t* sorted_ids;
  const int32_t* num_post_pad;
  const float* route_weight;
  void* out;
  float* out_scales_t;      // [I/128, rows_cap]          (FP8 GEMM1)
  int32_t* inv;             // TMAOUT: [numel] sorted row of every route
  int32_t* status;
  unsigned long long wait_ns;  // limit of every bounded barrier wait
  int64_t numel;
  int64_t rows_cap;
  int64_t a_scale_ld;       // tokens (GEMM1) or rows_cap (GEMM2)
  int topk;
  int mul_weight;
  int E;
  int K;        // contraction length in elements
  int Nout;     // output columns (I for GEMM1, H for GEMM2)
  int rows_w;   // weight rows per expert (2I or H)
  int n_tiles;  // column tiles per align block
  int group_m;  // align blocks per group of the tile order
  int w_row0;   // GEMM2 over a window of the output columns: first weight row (output column) of the window
  bool wide_store;  // the output is 32-byte aligned: rows are written with 32-byte stores
#ifdef MOE_TC_TRACE
  long long* trace;  // [4 roles][64 K blocks][8 events] cycle stamps of CTA 0, third tile (experiment builds)
#endif
};
#ifdef MOE_TC_TRACE
#define MOE_TR(role, kb, ev) \
  do { if (blockIdx.x == 0 && tile == tile0 + 2 * tile_step && P.trace && (kb) < 64) P.trace[((role) * 64 + (kb)) * 8 + (ev)] = clock64(); } while (0)
#define MOE_TRN(role, slot, ev) \
  do { if (blockIdx.x == 0 && tile == tile0 + 3 * tile_step && P.trace) P.trace[((role) * 64 + (slot)) * 8 + (ev)] = clock64(); } while (0)
#else
#define MOE_TR(role, kb, ev) do {} while (0)
#define MOE_TRN(role, slot, ev) do {} while (0)
#endif

// Instruction descriptor: fp32 accumulator (bits 4-5 = 1), A/B element format
// (bits 7-9 / 10-12: e4m3 = 0 for kind::f8f6f4; f16 = 0, bf16 = 1 for
// kind::f16), both operands K-major, N >> 3 at bit 17, M >> 4 at bit 24.
template <bool FP8, typename AT, bool PAIR>
struct IDesc {
  static constexpr uint32_t fmt = (!FP8 && std::is_same<AT, __nv_bfloat16>::value) ? 1u : 0u;
  static constexpr uint32_t m = PAIR ? 2 * BM : BM;  // a pair multiplies 256 rows per instruction
  static constexpr uint32_t value =
      (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
};

// B tile = 256 accumulator columns = 256 weight rows, fetched with as few TMA instructions
// as the weight layout allows (every instruction costs the single producer thread issue
// time, whatever the box size).  GEMM1: columns [0,128) are gate rows nt*128.., columns
// [128,256) the up rows of the same outputs: two boxes of 128 rows (a CTA pair: one each).
// GEMM2: 256 consecutive rows, one box (a pair: 128 rows each).
template <bool GEMM1, bool PAIR> struct BBox {
  static constexpr int COUNT = (GEMM1 && !PAIR) ? 2 : 1;  // boxes per CTA and stage
  static constexpr int ROWS = (GEMM1 || PAIR) ? 128 : 256;
};
// weight row (inside the expert) of the first row of this CTA's box `c` of column tile `nt`
template <bool GEMM1, bool PAIR>
__device__ __forceinline__ int box_row(int nt, int c, int cr, int Nout) {
  if constexpr (GEMM1) return nt * 128 + (PAIR ? cr : c) * Nout;
  else return nt * BN + (PAIR ? cr * 128 : 0);
}

// PAIR = true: two CTAs of a cluster work as one cta_group::2 unit on a 256-row
// align block.  Each CTA holds its own 128 rows of A and ONE HALF of the B tile;
// the leader CTA (cluster rank 0) issues a single M=256 instruction per K step
// that reads both CTAs' shared memory and writes each CTA's own TMEM.  Every
// weight tile therefore crosses L2 -> shared memory once per 256 rows instead
// of once per 128.  Nothing is multicast: every TMA load and cp.async lands in
// the issuing CTA and signals a local barrier; the partner CTA forwards "stage
// landed" to the leader with a remote mbarrier arrive, and the leader's
// tcgen05.commit signals the stage-free / accumulator-ready barriers of both
// CTAs.
//
// RB = 2 (half precision, single CTA): the tile is 256 rows x 256 columns; both TMEM
// accumulators belong to it (rows 0-127 and 128-255), so every B stage is used by two
// instruction groups and each weight tile crosses L2 -> shared memory once per 256 rows
// without any cross-CTA traffic.  FP8 cannot use it: its fp32 fold accumulators live in
// registers and two blocks would need the whole register file.
//
// SORTED (GEMM1, half precision): the token rows were copied into sorted order beforehand
// (moe_gather_rows), so A arrives as one TMA box per 128 rows like in GEMM2 and warps 2-3 idle.
// With many rows per expert the in-kernel cp.async gather is the limiter of GEMM1 (its
// per-lane requests keep the load/store unit busier than the tensor core: 1.07 against
// 1.37 PFLOP/s for the TMA-fed GEMM2 on the Mixtral shape), and the copy costs far less.
//
// TMAOUT (GEMM2, single CTA): the output tile is staged in shared memory (bf16 / f16, the layout
// a 128-byte-swizzled tensor map expects) and written by TMA bulk stores to y in SORTED row
// order; the kernel also records where every route's row went (P.inv[route] = sorted row) for
// the combine.  A thread owns one tile row, so direct stores hand the memory system 32
// separate 32-byte sectors per warp instruction, and the consumers -- the same warps that fold
// the next tile -- sat in those stores for ~5000 cycles per tile; staged, they are done after
// sixteen conflict-free shared-memory stores.  Costs one pipeline stage of shared memory.
template <bool FP8, typename AT, bool GEMM1, bool PAIR, int RB, bool SORTED = false, bool TMAOUT = false>
__global__ void __launch_bounds__(THREADS, 1)
tc_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               const __grid_constant__ CUtensorMap map_out, const Params P) {
  static_assert(!TMAOUT || (!GEMM1 && !PAIR && RB == 1), "staged output: single-CTA GEMM2 only");
  static_assert(!SORTED || GEMM1, "pre-sorted A rows: GEMM1 only");
  constexpr bool GATHER = GEMM1 && !SORTED;  // A rows gathered inside the kernel
  static_assert(RB == 1 || (RB == 2 && !FP8), "wide tiles: half precision only");
  constexpr int STAGES = TMAOUT ? 3 : Cfg<PAIR, RB>::STAGES;
  constexpr int A_LOCAL_BYTES = Cfg<PAIR, RB>::A_LOCAL;
  constexpr int B_LOCAL_BYTES = PAIR ? B_HALF_BYTES : B_STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* sA = smem;
  uint8_t* sB = smem + (size_t)STAGES * A_LOCAL_BYTES;
  SmemAux* aux = reinterpret_cast<SmemAux*>(smem + (size_t)STAGES * Cfg<PAIR, RB>::STAGE_BYTES);
  // staged output tile: four sub-tiles of 128 rows x 64 columns (128 bytes per row), 1024-byte aligned
  [[maybe_unused]] uint8_t* s_out = smem + (((size_t)STAGES * Cfg<PAIR, RB>::STAGE_BYTES + sizeof(SmemAux) + 1023) & ~(size_t)1023);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr int KBE = FP8 ? 128 : 64;  // elements of K per stage
  const int KB = (P.K + KBE - 1) / KBE;
  const int npp = min((int64_t)P.num_post_pad[0], P.rows_cap);
  // work unit: one CTA and a 128-row align block; a CTA pair and a 256-row block; or one
  // CTA and a 256-row block (RB = 2).  UNIT = 128-row blocks per align block.
  constexpr int UNIT = PAIR ? 2 * RB : RB;
  constexpr int CTAS = PAIR ? 2 : 1;
  const int cr = PAIR ? (int)cluster_ctarank() : 0;  // rank inside the pair; 0 leads
  const int tile0 = blockIdx.x / CTAS, tile_step = gridDim.x / CTAS;
  const int nblk = (npp + UNIT * BM - 1) / (UNIT * BM);
  const int total_tiles = nblk * P.n_tiles;
  // Tile order: groups of `group_m` consecutive align blocks; inside a group the block index runs
  // fastest, then the column tile.  The CTAs that run at the same time then work on the blocks of
  // one expert for the SAME few column tiles, so a weight tile is fetched from DRAM once and
  // served to the other row blocks from L2.  (Column tile fastest sends every row block of an
  // expert over the expert's whole weight matrix at a different time; a matrix larger than L2
  // is then read once per row block.)
  auto tile_blk_nt = [&](int tile, int& blk, int& nt) {
    const int per_group = P.group_m * P.n_tiles;
    const int grp = tile / per_group;
    const int first = grp * P.group_m;
    const int gsz = min(nblk - first, P.group_m);
    const int within = tile - grp * per_group;
    nt = within / gsz;
    blk = first + within - nt * gsz;
  };
  // tile -> expert_ids index (blk), this CTA's 128-row block (mb), column tile (nt).  The expert of
  // the NEXT tile is fetched while the current one is worked on: a tile starts without waiting
  // for a global load (every role walks the same tile list with its own copy of e_next).
#define MOE_TILE_COORDS(tile)                             \
  int blk, nt;                                            \
  tile_blk_nt((tile), blk, nt);                           \
  [[maybe_unused]] const int mb = UNIT * blk + RB * cr;   \
  const int e = e_next;                                   \
  e_next = -1;                                            \
  if ((tile) + tile_step < total_tiles) {                 \
    int blk2, nt2;                                        \
    tile_blk_nt((tile) + tile_step, blk2, nt2);           \
    e_next = P.expert_ids[blk2];                          \
  }
  int e_next = -1;
  if (tile0 < total_tiles) {
    int blk0, nt0;
    tile_blk_nt(tile0, blk0, nt0);
    e_next = P.expert_ids[blk0];
  }

#ifdef MOE_TC_TRACE
  if (threadIdx.x == 0 && blockIdx.x == 0 && P.trace) { P.trace[2048] = clock64(); P.trace[2049] = (long long)now_ns(); P.trace[2052] = total_tiles; }
#endif
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&aux->full[s], GATHER ? 1 + GATHER_THREADS : (FP8 ? 1 + SCALE_THREADS : 1));
      mbar_init(&aux->empty[s], 1);
      mbar_init(&aux->peer_full[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&aux->tmem_full[a], 1);
      mbar_init(&aux->tmem_empty[a], CTAS * (EPI_THREADS / 32));  // a pair's leader also collects the partner's warps
    }
    mbar_init(&aux->xch_bar, EPI_THREADS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&aux->tmem_base)),
                   "r"(512));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&aux->tmem_base)),
                   "r"(512));
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
  }
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();  // both CTAs' barriers exist before anyone signals across
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = aux->tmem_base;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(PRODUCER_REGS));
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------ TMA producer
      if constexpr (!GATHER) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      uint32_t it = 0;
      bool alive = true;
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        [[maybe_unused]] const int row0 = mb * BM;
        const int wrow0 = e * P.rows_w + P.w_row0;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          MOE_TR(0, kb, 0);
          if (!mbar_wait(&aux->empty[s], ph ^ 1, P.status, P.wait_ns)) { alive = false; break; }
          MOE_TR(0, kb, 1);
          if constexpr (GATHER) {
            mbar_expect_tx(&aux->full[s], B_LOCAL_BYTES);  // A rows arrive by cp.async (warps 2-3)
          } else {
            mbar_expect_tx(&aux->full[s], A_LOCAL_BYTES + B_LOCAL_BYTES);
#pragma unroll
            for (int j = 0; j < RB; ++j)
              tma_load_2d(&map_a, &aux->full[s], sA + (size_t)s * A_LOCAL_BYTES + j * A_STAGE_BYTES, kb * KBE,
                          row0 + j * BM);
          }
#pragma unroll
          for (int c = 0; c < BBox<GEMM1, PAIR>::COUNT; ++c)
            tma_load_2d(&map_b, &aux->full[s], sB + (size_t)s * B_LOCAL_BYTES + c * (BBox<GEMM1, PAIR>::ROWS * 128),
                        kb * KBE, wrow0 + box_row<GEMM1, PAIR>(nt, c, cr, P.Nout));
          MOE_TR(0, kb, 2);
        }
      }
    } else if (warp == 1 && lane == 0 && cr == 0) {
      // ------------------------------------------------------------ MMA issuer (pair: leader only)
      constexpr uint32_t idesc = IDesc<FP8, AT, PAIR>::value;
      [[maybe_unused]] uint32_t it = 0;
      uint32_t acc_it = 0;
      bool alive = true;
      if constexpr (!PAIR) {
        // This thread shares its scheduler with two consumer warps that stream FMAs, and every
        // instruction it needs between "accumulator released" and "MMAs issued" waits for an issue
        // slot behind them.  So everything that does not depend on the release is done before the
        // wait for it: stage index and phase are carried (no division), the descriptors are one
        // add away from a base, and the operands' barrier (which completed long before) is waited
        // for first.  After the release only the fence, the four MMAs and the commits remain.
        const uint64_t adesc0 = make_smem_desc(smem_u32(sA));
        const uint64_t bdesc0 = make_smem_desc(smem_u32(sB));
        uint32_t s = 0, sph = 0;
        for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
          MOE_TRN(1, 61, 0);
          MOE_TILE_COORDS(tile)
          if (e < 0 || e >= P.E) continue;
          MOE_TRN(1, 61, 1);
          for (int kb = 0; kb < KB; ++kb) {
            const uint32_t a = RB == 2 ? 0u : (acc_it & 1);
            const uint32_t aph = RB == 2 ? (acc_it & 1) : ((acc_it >> 1) & 1);
            const uint64_t bdesc = bdesc0 + (uint64_t)(s * (uint32_t)(B_LOCAL_BYTES >> 4));
            const uint64_t adesc = adesc0 + (uint64_t)(s * (uint32_t)(A_LOCAL_BYTES >> 4));
            const uint32_t d0 = tmem_base + a * BN;
            MOE_TR(1, kb, 0);
            if (!mbar_wait(&aux->full[s], sph, P.status, P.wait_ns)) { alive = false; break; }
            MOE_TR(1, kb, 1);
            if constexpr (GATHER) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // cp.async writes -> tensor core reads
            if (FP8 || kb == 0) {
              if (!mbar_wait(&aux->tmem_empty[a], aph ^ 1, P.status, P.wait_ns)) { alive = false; break; }
            }
            MOE_TR(1, kb, 2);
            tc_fence_after();
#pragma unroll
            for (int j = 0; j < RB; ++j) {
              const uint64_t aj = adesc + (uint64_t)(j * (A_STAGE_BYTES >> 4));
              const uint32_t d = RB == 2 ? tmem_base + (uint32_t)j * BN : d0;
              if (FP8) {
                tc_mma_const<FP8, false>(d, aj, bdesc, idesc);
              } else {
                tc_mma<FP8>(d, aj, bdesc, idesc, kb > 0);
              }
#pragma unroll
              for (int k4 = 1; k4 < 4; ++k4)  // 32 bytes of K per instruction: start address advances by 32 B >> 4
                tc_mma_const<FP8, true>(d, aj + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc);
            }
            if (FP8 || kb == KB - 1) {
              tc_commit(&aux->tmem_full[a]);
              ++acc_it;
            }
            tc_commit(&aux->empty[s]);
            MOE_TR(1, kb, 3);
            if (kb == 0) MOE_TRN(1, 61, 2);
            if (kb == 1) MOE_TRN(1, 61, 3);
            if (kb == 2) MOE_TRN(1, 61, 4);
            if (++s == STAGES) { s = 0; sph ^= 1; }
          }
        }
      } else {
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          // accumulator barrier and phase: the two accumulators alternate (per K block in FP8
          // mode, per tile in half mode); a wide tile owns both and uses barrier 0
          const uint32_t a = RB == 2 ? 0u : (acc_it & 1);
          const uint32_t aph = RB == 2 ? (acc_it & 1) : ((acc_it >> 1) & 1);
          if (FP8 || kb == 0) {
            if (!mbar_wait<PAIR>(&aux->tmem_empty[a], aph ^ 1, P.status, P.wait_ns)) { alive = false; break; }
            tc_fence_after();
          }
          const int s = it % STAGES;
          if (!mbar_wait(&aux->full[s], (it / STAGES) & 1, P.status, P.wait_ns)) { alive = false; break; }
          if (!mbar_wait<true>(&aux->peer_full[s], (it / STAGES) & 1, P.status, P.wait_ns)) { alive = false; break; }
          if constexpr (GATHER) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // cp.async writes -> tensor core reads
          tc_fence_after();
          const uint64_t bdesc = make_smem_desc(smem_u32(sB + (size_t)s * B_LOCAL_BYTES));
#pragma unroll
          for (int j = 0; j < RB; ++j) {
            const uint64_t adesc = make_smem_desc(smem_u32(sA + (size_t)s * A_LOCAL_BYTES + j * A_STAGE_BYTES));
            const uint32_t d = tmem_base + (RB == 2 ? (uint32_t)j : a) * BN;
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              // 32 bytes of K per instruction: start address advances by 32 B >> 4
              const uint32_t accum = FP8 ? (k4 > 0) : (kb > 0 || k4 > 0);
              tc_mma_pair<FP8>(d, adesc + (uint64_t)(k4 * 2), bdesc + (uint64_t)(k4 * 2), idesc, accum);
            }
          }
          tc_commit_pair(&aux->empty[s]);
          if (FP8 || kb == KB - 1) {
            tc_commit_pair(&aux->tmem_full[a]);
            ++acc_it;
          }
        }
      }
      }
    } else if (PAIR && warp == 1 && lane == 0 && cr == 1) {
      // ------------------------------------------------------------ partner CTA: tell the leader a stage has landed
      uint32_t it = 0;
      bool alive = true;
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&aux->full[s], (it / STAGES) & 1, P.status, P.wait_ns)) { alive = false; break; }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          mbar_arrive_remote(&aux->peer_full[s], 0);
        }
      }
    } else if (GATHER && warp >= 2) {
      // ------------------------------------------------------------ A-row gather (cp.async)
      // Two lanes share a row: lane pair q copies the 32-byte sector {2c, 2c+1} of rows
      // q + 32 j in step c, so every warp instruction fetches 16 whole sectors (one lane per row
      // would touch 32 sectors per instruction and fetch every sector twice).
      const int g = threadIdx.x - 64;  // 0..63
      const int q = g >> 1, half = g & 1;
      const int64_t pitch = (int64_t)P.K * (FP8 ? 1 : 2);
      uint32_t it = 0;
      bool alive = true;
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        constexpr int RPT = 4 * RB;  // rows per lane pair
        const uint8_t* src[RPT];
        bool ok[RPT];
        // FP8: thread g also stages the activation scales of rows g and g + 64 and (g < 2) the
        // weight scale of the gate (g = 0: rows nt*128..) or up (g = 1: rows I + nt*128..) block
        [[maybe_unused]] const float* ws_src = nullptr;
        [[maybe_unused]] const float* as_src[2] = {nullptr, nullptr};
        auto row_token = [&](int r, bool& valid) -> int64_t {
          const int64_t p = (int64_t)mb * BM + r;
          const int64_t sid = p < P.rows_cap ? (int64_t)P.sorted_ids[p] : P.numel;
          valid = sid >= 0 && sid < P.numel;  // padding slot: the row keeps stale bytes, its results are never stored
          return valid ? sid / P.topk : 0;
        };
        if constexpr (FP8) {
          const int sblk_per_e = (P.rows_w + 127) / 128;
          ws_src = P.w_scale + ((int64_t)e * sblk_per_e + (g == 1 ? (P.Nout >> 7) + nt : nt)) * KB;
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            bool valid;
            const int64_t tok = row_token(g + 64 * j, valid);
            if (valid) as_src[j] = P.a_scales_t + tok;
          }
        }
#pragma unroll
        for (int j = 0; j < RPT; ++j) {
          const int64_t tok = row_token(q + 32 * j, ok[j]);
          src[j] = P.a_rows + tok * pitch + half * 16;
        }
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES;
          if (g == 0) MOE_TR(2, kb, 0);
          if (!mbar_wait(&aux->empty[s], ((it / STAGES) & 1) ^ 1, P.status, P.wait_ns)) { alive = false; break; }
          if (g == 0) MOE_TR(2, kb, 1);
          const uint32_t base = smem_u32(sA + (size_t)s * A_LOCAL_BYTES);
#pragma unroll
          for (int j = 0; j < RPT; ++j) {
            if (ok[j]) {
              const int r = q + 32 * j;  // row inside the (RB x 128)-row tile
              const uint8_t* sp = src[j] + (int64_t)kb * 128;
#pragma unroll
              for (int c = 0; c < 4; ++c)  // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
                cp_async16(base + (uint32_t)r * 128u + (uint32_t)(((2 * c + half) ^ (r & 7)) << 4), sp + c * 32);
            }
          }
          if constexpr (FP8) {
            const int slot = it % SCALE_SLOTS;
#pragma unroll
            for (int j = 0; j < 2; ++j)
              if (as_src[j] != nullptr) cp_async4(smem_u32(&aux->sc_a[slot][g + 64 * j]), as_src[j] + (int64_t)kb * P.a_scale_ld);
            if (g < 2) cp_async4(smem_u32(&aux->sc_w[slot][g]), ws_src + kb);
          }
          cp_async_arrive_noinc(&aux->full[s]);
          if (g == 0) MOE_TR(2, kb, 2);
        }
      }
      asm volatile("cp.async.wait_all;" ::: "memory");
    } else if (FP8 && !GATHER && warp == 3) {
      // ------------------------------------------------------------ scale staging (FP8, A rows read by TMA)
      uint32_t it = 0;
      bool alive = true;
      const int sblk_per_e = (P.rows_w + 127) / 128;
      for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
        MOE_TILE_COORDS(tile)
        if (e < 0 || e >= P.E) continue;
        const float* as_row = P.a_scales_t + (int64_t)mb * BM + 4 * lane;
        // GEMM2: the two 128-column weight blocks of the tile; GEMM1: the gate block and the up block
        const int wblk = GEMM1 ? (lane == 1 ? (P.Nout >> 7) + nt : nt)
                               : min((P.w_row0 >> 7) + 2 * nt + lane, sblk_per_e - 1);
        const float* ws_src = P.w_scale + ((int64_t)e * sblk_per_e + wblk) * KB;
        for (int kb = 0; kb < KB; ++kb, ++it) {
          const int s = it % STAGES;
          if (!mbar_wait(&aux->empty[s], ((it / STAGES) & 1) ^ 1, P.status, P.wait_ns)) { alive = false; break; }
          const int slot = it % SCALE_SLOTS;
          cp_async16(smem_u32(&aux->sc_a[slot][4 * lane]), as_row + (int64_t)kb * P.a_scale_ld);
          if (lane < 2) cp_async4(smem_u32(&aux->sc_w[slot][lane]), ws_src + kb);
          cp_async_arrive_noinc(&aux->full[s]);
        }
      }
      asm volatile("cp.async.wait_all;" ::: "memory");
    }
  } else {
    // -------------------------------------------------------------- consumers
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(CONSUMER_REGS));
    const int h = (warp - 4) >> 2;                  // column half owned by this group
    const int row = ((warp & 3) << 5) + lane;       // accumulator lane = tile row
    const uint32_t t_lane = tmem_base + ((uint32_t)((warp & 3) << 5) << 16) + (uint32_t)(h * (GEMM1 ? 64 : 128));
    constexpr uint32_t SECOND = GEMM1 ? 128 : 64;  // column distance of the group's second 64-column chunk
    uint32_t acc_it = 0, tile_it = 0;
    bool alive = true;
    // releasing an accumulator: the pair's leader collects the arrivals of both CTAs
    auto release_acc = [&](uint32_t a) {
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && cr == 1) mbar_arrive_remote(&aux->tmem_empty[a], 0);
        else mbar_arrive(&aux->tmem_empty[a]);
      }
    };
    // The consumers' own walk over the tile list.  Coordinates, expert and this thread's sorted id
    // of the NEXT tile are fetched inside the K loop of the current one (FP8: while the warp would
    // wait for the tensor core anyway), so a tile starts folding without integer divisions or a
    // dependent global load in front of it.
    int nx_blk = 0, nx_nt = 0, nx_e = -1;
    int64_t nx_sid = P.numel;
    auto prefetch_tile = [&](int t) {
      nx_e = -1;
      nx_sid = P.numel;
      if (t < total_tiles) {
        tile_blk_nt(t, nx_blk, nx_nt);
        nx_e = P.expert_ids[nx_blk];
        const int64_t pn = (int64_t)(UNIT * nx_blk + RB * cr) * BM + row;
        if (pn < P.rows_cap) nx_sid = (int64_t)P.sorted_ids[pn];
      }
    };
    prefetch_tile(tile0);
    for (int tile = tile0; tile < total_tiles && alive; tile += tile_step) {
      if (threadIdx.x == 128) MOE_TRN(3, 61, 0);
      const int blk = nx_blk, nt = nx_nt, e = nx_e;
      const int64_t sid_first = nx_sid;
      [[maybe_unused]] const int mb = UNIT * blk + RB * cr;
      (void)blk;
      if (!FP8 || e < 0 || e >= P.E) prefetch_tile(tile + tile_step);  // half precision has no K loop here
      if (e < 0 || e >= P.E) continue;
      if (threadIdx.x == 128) MOE_TRN(3, 61, 1);
      for (int sub = 0; sub < RB && alive; ++sub) {  // the 128-row blocks of this tile (two for wide tiles)
      const int64_t p = (int64_t)(mb + sub) * BM + row;
      int64_t sid = P.numel;
      if (sub == 0) sid = sid_first;
      else if (p < P.rows_cap) sid = (int64_t)P.sorted_ids[p];
      const bool row_ok = sid >= 0 && sid < P.numel;
      if (sid < 0 || sid > P.numel) set_status(P.status, MOE_ST_BAD_ROW);  // the pad value is numel; anything else outside is corrupt
      float acc[128];
      float rw = 1.0f;  // route weight of this row, fetched early: the epilogue must not wait for it
      if constexpr (FP8) {
#pragma unroll
        for (int i = 0; i < 128; ++i) acc[i] = 0.0f;
        // one K block: wait for its accumulator, fold it into acc, release it
        auto fold_block = [&](float s_lo, float s_hi, [[maybe_unused]] int kb) {
          const uint32_t a = acc_it & 1;
          tc_fence_after();
          const uint32_t t0 = t_lane + a * BN;
          uint32_t ra[32], rb[32];
          unsigned long long* acc2 = reinterpret_cast<unsigned long long*>(acc);
          const unsigned long long lo2 = splat2(s_lo), hi2 = splat2(s_hi);
          // The accumulator is held from the first load to the release, and the tensor core's next
          // K block into it waits for that.  The second half is therefore reloaded into each
          // 32-register staging set as soon as its FMAs have consumed it, under the FMAs of the
          // other set, and the FMAs of the second half run after the release.  Packed pair FMAs:
          // the fold's issue slots are what the MMA-issuing thread on the same scheduler competes with.
          tmem_ld64_sync(t0, ra, rb);
          if (threadIdx.x == 128) MOE_TR(3, kb, 2);
#pragma unroll
          for (int i = 0; i < 16; ++i) fma2(acc2[i], ra[2 * i], ra[2 * i + 1], lo2);
          tmem_ld32_async(t0 + SECOND, ra);
#pragma unroll
          for (int i = 0; i < 16; ++i) fma2(acc2[16 + i], rb[2 * i], rb[2 * i + 1], lo2);
          tmem_ld32_async(t0 + SECOND + 32, rb);
          tmem_wait64(ra, rb);
          release_acc(a);
          if (threadIdx.x == 128) MOE_TR(3, kb, 3);
#pragma unroll
          for (int i = 0; i < 16; ++i) fma2(acc2[32 + i], ra[2 * i], ra[2 * i + 1], hi2);
#pragma unroll
          for (int i = 0; i < 16; ++i) fma2(acc2[48 + i], rb[2 * i], rb[2 * i + 1], hi2);
          ++acc_it;
        };
        // scales come from the shared-memory ring filled by the producer side:
        // GEMM1 halves are (gate, up) -> sc_w[0], sc_w[1]; GEMM2 group h owns one weight block
        for (int kb = 0; kb < KB; ++kb) {
          const int slot = acc_it % SCALE_SLOTS;
          if (threadIdx.x == 128) MOE_TR(3, kb, 0);
          if (kb == (KB > 1 ? 1 : 0)) prefetch_tile(tile + tile_step);
          if (!mbar_wait(&aux->tmem_full[acc_it & 1], (acc_it >> 1) & 1, P.status, P.wait_ns)) { alive = false; break; }
          if (threadIdx.x == 128) MOE_TR(3, kb, 1);
          if (threadIdx.x == 128 && kb == 0) MOE_TRN(3, 61, 2);
          const float sa = aux->sc_a[slot][row];
          const float s_lo = sa * aux->sc_w[slot][GEMM1 ? 0 : h];
          const float s_hi = sa * aux->sc_w[slot][GEMM1 ? 1 : h];
          fold_block(s_lo, s_hi, kb);
          if (kb == 0 && P.mul_weight && row_ok) rw = P.route_weight[sid];  // sid arrived during the first fold
          if (threadIdx.x == 128) MOE_TR(3, kb, 4);
        }
        if (!alive) break;
      } else {
        const uint32_t a = RB == 2 ? 0u : (acc_it & 1);
        const uint32_t aph = RB == 2 ? (acc_it & 1) : ((acc_it >> 1) & 1);
        if (P.mul_weight && row_ok) rw = P.route_weight[sid];
        if (sub == 0) {
          if (!mbar_wait(&aux->tmem_full[a], aph, P.status, P.wait_ns)) { alive = false; break; }
          tc_fence_after();
        }
        const uint32_t t0 = t_lane + (RB == 2 ? (uint32_t)sub : a) * BN;
        uint32_t* r = reinterpret_cast<uint32_t*>(acc);
        tmem_ld64_sync(t0, r, r + 32);
        tmem_ld64_sync(t0 + SECOND, r + 64, r + 96);
        if (sub == RB - 1) {  // everything of this tile is in registers (or already stored)
          release_acc(a);
          ++acc_it;
        }
      }

      if (threadIdx.x == 128) MOE_TR(3, 60, 0);
      // ---------------------------------------------------------- tile epilogue
      if constexpr (!FP8) {
        if (P.w_scale != nullptr) {
          // weight-only int8: weights were widened exactly to the activation dtype, the
          // per-output-channel scale is applied here in fp32
          const float* cs = P.w_scale + (int64_t)e * P.rows_w;
          if constexpr (GEMM1) {
            const int n0 = nt * 128 + 64 * h;
#pragma unroll
            for (int j4 = 0; j4 < 16; ++j4) {
              const float4 sg = *reinterpret_cast<const float4*>(cs + n0 + 4 * j4);
              const float4 su = *reinterpret_cast<const float4*>(cs + P.Nout + n0 + 4 * j4);
              acc[4 * j4 + 0] *= sg.x; acc[4 * j4 + 1] *= sg.y; acc[4 * j4 + 2] *= sg.z; acc[4 * j4 + 3] *= sg.w;
              acc[64 + 4 * j4 + 0] *= su.x; acc[64 + 4 * j4 + 1] *= su.y;
              acc[64 + 4 * j4 + 2] *= su.z; acc[64 + 4 * j4 + 3] *= su.w;
            }
          } else {
            const int n0 = nt * BN + 128 * h;
#pragma unroll
            for (int j4 = 0; j4 < 32; ++j4) {
              if (n0 + 4 * j4 < P.Nout) {
                const float4 sc = *reinterpret_cast<const float4*>(cs + n0 + 4 * j4);
                acc[4 * j4 + 0] *= sc.x; acc[4 * j4 + 1] *= sc.y; acc[4 * j4 + 2] *= sc.z; acc[4 * j4 + 3] *= sc.w;
              }
            }
          }
        }
      }
      if constexpr (GEMM1) {
        // acc[0..63] gate, acc[64..127] up of output columns nt*128 + 64h + j
        float amax = 0.0f;
#pragma unroll
        for (int j = 0; j < 64; ++j) {
          acc[j] = round_act<AT>(silu_mul_fast(acc[j] * rw, acc[64 + j] * rw));
          amax = fmaxf(amax, fabsf(acc[j]));
        }
        const int64_t col0 = (int64_t)nt * 128 + 64 * h;
        if constexpr (FP8) {
          float* x = &aux->xch[tile_it & 1][0][0];
          x[h * BM + row] = amax;
          mbar_arrive(&aux->xch_bar);
          if (!mbar_wait(&aux->xch_bar, tile_it & 1, P.status, P.wait_ns)) { alive = false; break; }
          amax = fmaxf(amax, x[(1 - h) * BM + row]);
          const float s = fmaxf(amax, kQuantEps) * (1.0f / kFp8Max);
          const float inv_s = 1.0f / s;  // one reciprocal per row instead of 64 divisions
          if (row_ok) {
            uint4 pieces[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint32_t w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                uint32_t pk = 0;
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  const float qv = fminf(fmaxf(acc[v * 16 + q * 4 + b] * inv_s, -kFp8Max), kFp8Max);
                  pk |= (uint32_t)f32_to_fp8e4m3(qv) << (8 * b);
                }
                w[q] = pk;
              }
              pieces[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
            store_row_pieces(reinterpret_cast<uint8_t*>(P.out) + p * P.Nout + col0, pieces, P.wide_store);
            if (h == 0) P.out_scales_t[(int64_t)nt * P.rows_cap + p] = s;
          }
        } else if (row_ok) {
          uint4 pieces[8];
#pragma unroll
          for (int v = 0; v < 8; ++v)
            pieces[v] = make_uint4(pack2<AT>(acc[v * 8 + 0], acc[v * 8 + 1]), pack2<AT>(acc[v * 8 + 2], acc[v * 8 + 3]),
                                   pack2<AT>(acc[v * 8 + 4], acc[v * 8 + 5]), pack2<AT>(acc[v * 8 + 6], acc[v * 8 + 7]));
          store_row_pieces(reinterpret_cast<AT*>(P.out) + p * P.Nout + col0, pieces, P.wide_store);
        }
      } else if constexpr (TMAOUT) {
        // the previous tile's bulk stores have finished reading the staging buffer
        if (threadIdx.x == 128) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
#pragma unroll
        for (int c = 0; c < 16; ++c) {  // 16-byte chunk c of this thread's 128 columns -> sub-tile 2h + c/8, chunk c%8
          const uint4 piece = make_uint4(pack2<AT>(acc[c * 8 + 0] * rw, acc[c * 8 + 1] * rw),
                                         pack2<AT>(acc[c * 8 + 2] * rw, acc[c * 8 + 3] * rw),
                                         pack2<AT>(acc[c * 8 + 4] * rw, acc[c * 8 + 5] * rw),
                                         pack2<AT>(acc[c * 8 + 6] * rw, acc[c * 8 + 7] * rw));
          uint8_t* dst = s_out + (size_t)(2 * h + (c >> 3)) * (BM * 128) + row * 128 + (((c & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = piece;
        }
        if (row_ok && h == 0) P.inv[sid] = (int32_t)p;
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> TMA reads
        asm volatile("bar.sync 2, %0;" ::"n"(EPI_THREADS) : "memory");
        if (threadIdx.x == 128) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const int c0 = nt * BN + q4 * 64;
            if (c0 < P.Nout)
              asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&map_out), "r"(c0), "r"((int)(mb * BM)), "r"(smem_u32(s_out + (size_t)q4 * (BM * 128)))
                           : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
      } else if (row_ok) {
        const int col0 = nt * BN + 128 * h;
        AT* o = reinterpret_cast<AT*>(P.out) + sid * P.Nout + col0;
#pragma unroll
        for (int v = 0; v < 16; v += 2) {
          if (col0 + v * 8 < P.Nout) {  // Nout is a multiple of 64: the two pieces are in or out together
            uint4 pieces[2];
#pragma unroll
            for (int u = 0; u < 2; ++u)
              pieces[u] = make_uint4(pack2<AT>(acc[(v + u) * 8 + 0] * rw, acc[(v + u) * 8 + 1] * rw),
                                     pack2<AT>(acc[(v + u) * 8 + 2] * rw, acc[(v + u) * 8 + 3] * rw),
                                     pack2<AT>(acc[(v + u) * 8 + 4] * rw, acc[(v + u) * 8 + 5] * rw),
                                     pack2<AT>(acc[(v + u) * 8 + 6] * rw, acc[(v + u) * 8 + 7] * rw));
            store_row_pieces(o + v * 8, pieces, P.wide_store);
          }
        }
      }
      if (threadIdx.x == 128) MOE_TR(3, 60, 1);
      }  // sub
      ++tile_it;
    }
  }

  // -------------------------------------------------------------------- teardown
  if constexpr (TMAOUT) {
    if (threadIdx.x == 128) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // the last tile's stores are complete
  }
  tc_fence_before();
  if constexpr (PAIR) cluster_sync_all();  // no CTA leaves while its partner may still signal its barriers
  else __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    if constexpr (PAIR)
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
    else
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512));
  }
#ifdef MOE_TC_TRACE
  if (threadIdx.x == 0 && blockIdx.x == 0 && P.trace) { P.trace[2050] = clock64(); P.trace[2051] = (long long)now_ns(); }
#endif
#undef MOE_TILE_COORDS
}

// ------------------------------------------------------------------ host side
template <bool FP8, typename AT, bool GEMM1, bool PAIR, int RB, bool SORTED = false, bool TMAOUT = false>
static int launch(const CUtensorMap& ma, const CUtensorMap& mb, const Params& P, int grid, cudaStream_t st,
                  const CUtensorMap* mo = nullptr) {
  auto kern = tc_gemm_kernel<FP8, AT, GEMM1, PAIR, RB, SORTED, TMAOUT>;
  constexpr size_t smem = smem_bytes<PAIR, RB, TMAOUT>();
  cudaFuncAttributes fa;
  cudaError_t ce = cudaFuncGetAttributes(&fa, kern);
  if (ce != cudaSuccess) return fail((int)ce, "tensor-core GEMM: cudaFuncGetAttributes: %s", cudaGetErrorString(ce));
  // see LAUNCH_REGS: refuse to launch rather than let setmaxnreg.inc wait for registers that do not exist
  if ((THREADS - EPI_THREADS) * PRODUCER_REGS + EPI_THREADS * CONSUMER_REGS > THREADS * fa.numRegs)
    return fail(MOE_E_DRIVER, "tensor-core GEMM: kernel was built with %d registers per thread, %d needed",
                fa.numRegs, LAUNCH_REGS);
  ce = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (ce != cudaSuccess) return fail((int)ce, "tensor-core GEMM: shared memory attribute: %s", cudaGetErrorString(ce));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = PAIR ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  ce = cudaLaunchKernelEx(&cfg, kern, ma, mb, mo != nullptr ? *mo : ma, P);
  if (ce != cudaSuccess) return fail((int)ce, "tensor-core GEMM launch: %s", cudaGetErrorString(ce));
  return check_launch(GEMM1 ? "gemm1 (tcgen05)" : "gemm2 (tcgen05)");
}

}  // namespace tc

// gemm1: `a` holds [a_tokens, K] activations in token order (row p of a tile is token
// sorted_ids[p] / topk); gemm2: `a` holds [rows_cap, K] rows in sorted order.
int tc_gemm(bool gemm1, int mode, int act_dtype, const void* a, const float* a_scales_t, const void* w,
            const float* w_scale, const int32_t* expert_ids, const int32_t* sorted_ids, const int32_t* npp,
            const float* route_weight, int mul_weight, int64_t numel, int64_t rows_cap, int64_t a_tokens, int topk,
            int block_m, int E, int K, int Nout, void* out, float* out_scales_t, int32_t* status, cudaStream_t st,
            int variant, int a_sorted, int32_t* inv, int w_row0, int w_rows, int grid_limit) {
  // w_row0, w_rows (gemm2 with inv only; 0, 0 = the whole matrix): the call produces the Nout output
  //   columns that start at column w_row0 of a weight matrix with w_rows rows per expert, into an
  //   `out` that is Nout wide; grid_limit > 0 caps the number of CTAs (SMs left to other work)
  // inv (gemm2, variant 1): `out` is y in SORTED row order [rows_cap, Nout], written by TMA from a staged
  //   tile, and inv[route] receives the sorted row of every route
  // a_sorted (gemm1): `a` holds [rows_cap, K] rows already in sorted order (moe_gather_rows)
  // variant: 1 = one CTA per 128-row block, 2 = cta_group::2 CTA pair per 256-row block,
  //          3 = one CTA per 256-row block with a 256x256 tile (half precision only),
  //          4 = CTA pair per 512-row block, 256x256 per CTA (half precision only)
  using namespace tc;
  const bool pair = variant == 2 || variant == 4, wide = variant == 3 || variant == 4;
  if (variant < 1 || variant > 4) return fail(MOE_E_BADARG, "tensor-core GEMM: unknown kernel variant %d", variant);
  if (wide && mode != MOE_MODE_HALF) return fail(MOE_E_SHAPE, "tensor-core GEMM: the 256-row-per-CTA tiles serve half precision only");
  const bool fp8 = mode == MOE_MODE_FP8_BLOCK;
  const bool sorted = gemm1 && a_sorted != 0;
  if (sorted && ((pair && !fp8) || (fp8 && wide)))
    return fail(MOE_E_SHAPE, "tensor-core GEMM1: pre-sorted rows are served by the single-CTA kernels and the FP8 CTA pair");
  if (mode != MOE_MODE_FP8_BLOCK && mode != MOE_MODE_HALF)
    return fail(MOE_E_SHAPE, "tensor-core GEMM: mode %d is served by the generic kernel", mode);
  if (act_dtype != MOE_BF16 && act_dtype != MOE_F16)
    return fail(MOE_E_DTYPE, "tensor-core GEMM: activations must be f16 or bf16");
  const int unit_rows = BM * (pair ? 2 : 1) * (wide ? 2 : 1);
  if (block_m != unit_rows) return fail(MOE_E_SHAPE, "tensor-core GEMM: align block must be %d", unit_rows);
  if (rows_cap % unit_rows != 0 || rows_cap <= 0)
    return fail(MOE_E_SHAPE, "tensor-core GEMM: row capacity must be a positive multiple of %d", unit_rows);
  const int kbe = fp8 ? 128 : 64;
  if (K % kbe != 0) return fail(MOE_E_SHAPE, "tensor-core GEMM: K must be a multiple of %d", kbe);
  if (gemm1 && Nout % 128 != 0) return fail(MOE_E_SHAPE, "tensor-core GEMM1: intermediate size must be a multiple of 128");
  if (!gemm1 && Nout % 64 != 0) return fail(MOE_E_SHAPE, "tensor-core GEMM2: hidden size must be a multiple of 64");
  if (fp8 && !gemm1 && Nout % 128 != 0) return fail(MOE_E_SHAPE, "tensor-core GEMM2 (fp8): hidden size must be a multiple of 128");
  const bool window = w_rows > 0;
  if (window && mode == MOE_MODE_HALF && w_scale != nullptr)
    return fail(MOE_E_SHAPE, "tensor-core GEMM2: column windows do not serve per-channel scales");
  if (window && (gemm1 || inv == nullptr || w_row0 < 0 || w_row0 % 256 != 0 || Nout % 256 != 0 || w_row0 + Nout > w_rows))
    return fail(MOE_E_SHAPE, "tensor-core GEMM2: a column window starts and ends on multiples of 256 columns of the staged-output kernel");
  const int rows_w = gemm1 ? 2 * Nout : (window ? w_rows : Nout);
  if ((int64_t)E * rows_w >= (1ll << 31) || rows_cap >= (1ll << 31)) return fail(MOE_E_TOOBIG, "tensor-core GEMM: extent exceeds int32 coordinates");

  const int eb = fp8 ? 1 : 2;
  const CUtensorMapDataType dt = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                     : (act_dtype == MOE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16);
  CUtensorMap ma, mb;
  int rc = 0;
  if (gemm1 && !sorted) {
    memset(&ma, 0, sizeof(ma));  // A rows are gathered with cp.async, no tensor map
    if (((uintptr_t)a & 15) != 0) return fail(MOE_E_BADARG, "tensor-core GEMM1: activations not 16-byte aligned");
    if (topk <= 0 || a_tokens * topk != numel) return fail(MOE_E_BADARG, "tensor-core GEMM1: tokens * topk != numel");
  } else {
    rc = make_map(&ma, a, dt, eb, (uint64_t)rows_cap, (uint64_t)K, BM, false);
    if (rc) return rc;
  }
  rc = make_map(&mb, w, dt, eb, (uint64_t)E * rows_w, (uint64_t)K, (gemm1 || pair) ? 128 : 256, true);
  if (rc) return rc;

  Params P;
  if (sorted && (topk <= 0 || a_tokens * topk != numel)) return fail(MOE_E_BADARG, "tensor-core GEMM1: tokens * topk != numel");
  P.a_rows = (const uint8_t*)a; P.a_scale_ld = (gemm1 && !sorted) ? a_tokens : rows_cap; P.topk = gemm1 ? topk : 1;
  P.a_scales_t = a_scales_t; P.w_scale = w_scale; P.expert_ids = expert_ids; P.sorted_ids = sorted_ids;
  P.num_post_pad = npp; P.route_weight = route_weight; P.out = out; P.out_scales_t = out_scales_t; P.inv = nullptr;
  P.status = status; P.wait_ns = wait_limit_ns(); P.numel = numel; P.rows_cap = rows_cap; P.mul_weight = mul_weight; P.E = E; P.K = K;
  P.Nout = Nout; P.rows_w = rows_w; P.w_row0 = window ? w_row0 : 0;
  P.n_tiles = gemm1 ? Nout / 128 : (Nout + BN - 1) / BN;
  {
    // about as many blocks per group as one expert owns (rows per expert / rows per block, one of them partial)
    const int64_t per_expert = numel / (E > 0 ? E : 1);
    int64_t gm = per_expert / unit_rows + 1;
    P.group_m = (int)(gm < 1 ? 1 : (gm > 16 ? 16 : gm));
  }
  P.wide_store = ((uintptr_t)out & 31) == 0;
#ifdef MOE_TC_TRACE
  { const char* t = getenv(gemm1 ? "MOE_TRACE1" : "MOE_TRACE2"); P.trace = t ? (long long*)strtoull(t, nullptr, 0) : nullptr; }
#endif

  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t cap_tiles = (rows_cap / unit_rows) * (int64_t)P.n_tiles;
  if (grid_limit > 0 && grid_limit < sms) sms = grid_limit;
  const int units = pair ? sms / 2 : sms;  // work units resident at once: CTAs, or CTA pairs
  const int grid = (int)(cap_tiles < units ? cap_tiles : units) * (pair ? 2 : 1);

#define MOE_TC_LAUNCH2(F, T, G) \
  (pair ? launch<F, T, G, true, 1>(ma, mb, P, grid, st) : launch<F, T, G, false, 1>(ma, mb, P, grid, st))
#define MOE_TC_LAUNCH(F, T) (gemm1 ? MOE_TC_LAUNCH2(F, T, true) : MOE_TC_LAUNCH2(F, T, false))
  if (inv != nullptr) {
    if (gemm1 || variant != 1) return fail(MOE_E_SHAPE, "tensor-core GEMM: sorted output is written by GEMM2 of kernel 1 only");
    CUtensorMap mo;
    rc = make_map(&mo, out, act_dtype == MOE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                  (uint64_t)rows_cap, (uint64_t)Nout, BM, false);
    if (rc) return rc;
    P.inv = inv;
    if (fp8)
      return act_dtype == MOE_BF16 ? launch<true, __nv_bfloat16, false, false, 1, false, true>(ma, mb, P, grid, st, &mo)
                                   : launch<true, __half, false, false, 1, false, true>(ma, mb, P, grid, st, &mo);
    return act_dtype == MOE_BF16 ? launch<false, __nv_bfloat16, false, false, 1, false, true>(ma, mb, P, grid, st, &mo)
                                 : launch<false, __half, false, false, 1, false, true>(ma, mb, P, grid, st, &mo);
  }
  if (fp8 && sorted && pair)
    return act_dtype == MOE_BF16 ? launch<true, __nv_bfloat16, true, true, 1, true>(ma, mb, P, grid, st)
                                 : launch<true, __half, true, true, 1, true>(ma, mb, P, grid, st);
  if (fp8 && sorted)
    return act_dtype == MOE_BF16 ? launch<true, __nv_bfloat16, true, false, 1, true>(ma, mb, P, grid, st)
                                 : launch<true, __half, true, false, 1, true>(ma, mb, P, grid, st);
  if (fp8) return act_dtype == MOE_BF16 ? MOE_TC_LAUNCH(true, __nv_bfloat16) : MOE_TC_LAUNCH(true, __half);
  if (sorted) {
    if (act_dtype == MOE_BF16)
      return wide ? launch<false, __nv_bfloat16, true, false, 2, true>(ma, mb, P, grid, st)
                  : launch<false, __nv_bfloat16, true, false, 1, true>(ma, mb, P, grid, st);
    return wide ? launch<false, __half, true, false, 2, true>(ma, mb, P, grid, st)
                : launch<false, __half, true, false, 1, true>(ma, mb, P, grid, st);
  }
#define MOE_TC_WIDE(T, G) \
  (pair ? launch<false, T, G, true, 2>(ma, mb, P, grid, st) : launch<false, T, G, false, 2>(ma, mb, P, grid, st))
  if (wide) {
    if (act_dtype == MOE_BF16) return gemm1 ? MOE_TC_WIDE(__nv_bfloat16, true) : MOE_TC_WIDE(__nv_bfloat16, false);
    return gemm1 ? MOE_TC_WIDE(__half, true) : MOE_TC_WIDE(__half, false);
  }
#undef MOE_TC_WIDE
  return act_dtype == MOE_BF16 ? MOE_TC_LAUNCH(false, __nv_bfloat16) : MOE_TC_LAUNCH(false, __half);
#undef MOE_TC_LAUNCH
#undef MOE_TC_LAUNCH2
}

}  // namespace moe
