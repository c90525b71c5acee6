// Shared pieces of the tcgen05 grouped-GEMM kernels: PTX wrappers (mbarrier with
// bounded waits, TMA, tcgen05 MMA / commit / TMEM loads, cp.async), the
// shared-memory operand descriptor, and the host-side tensor-map encoder.
#pragma once

#include <cuda.h>

#include <cstring>
#include <type_traits>

#include "moe_common.cuh"

namespace moe {
namespace tc {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;  // 2 s: the default of moe_set_wait_limit_ns

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Arrive on the barrier at the same shared-memory offset in CTA `rank` of the cluster.
// Relaxed: what the leader consumes after this arrival is not generic-proxy data of this
// thread (TMA / cp.async results fenced to the async proxy, or TMEM already read back by
// tcgen05.wait::ld), and a release at cluster scope costs about a microsecond per call.
__device__ __forceinline__ void mbar_arrive_remote(uint64_t* bar, uint32_t rank) {
  asm volatile(
      "{\n\t.reg .b32 ra;\n\t"
      "mapa.shared::cluster.u32 ra, %0, %1;\n\t"
      "mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [ra];\n\t}"
      ::"r"(smem_u32(bar)), "r"(rank)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false when the limit ran out (status word is set).
// CLUSTER: the barrier is also arrived on by the partner CTA (acquire at cluster scope).
template <bool CLUSTER = false>
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int32_t* status,
                                          unsigned long long limit_ns = WAIT_LIMIT_NS) {
  auto probe = [&]() { return CLUSTER ? mbar_try_cluster(bar, parity) : mbar_try(bar, parity); };
  if (probe()) return true;
  const unsigned long long t0 = now_ns();
  uint32_t spins = 0;
  while (!probe()) {
    if ((++spins & 0x3FF) == 0 && now_ns() - t0 > limit_ns) {
      set_status(status, MOE_ST_WAIT_TIMEOUT);
      return false;
    }
  }
  return true;
}
// The same bounded wait for warps that expect to wait long (an epilogue warp waiting for a
// whole K loop): they sleep between probes, so their polling does not take issue slots from
// the warps that feed the tensor core.
__device__ __forceinline__ bool mbar_wait_idle(uint64_t* bar, uint32_t parity, int32_t* status,
                                               unsigned long long limit_ns = WAIT_LIMIT_NS) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = now_ns();
  uint32_t spins = 0;
  while (!mbar_try(bar, parity)) {
    __nanosleep(128);
    if ((++spins & 0xFF) == 0 && now_ns() - t0 > limit_ns) {
      set_status(status, MOE_ST_WAIT_TIMEOUT);
      return false;
    }
  }
  return true;
}
__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// cta_group::2: completion is signalled on the barrier at this offset in BOTH CTAs of the pair
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"((uint16_t)3)
      : "memory");
}
// One instruction for the pair: M = 256 (128 rows from each CTA), N = 256 (128 B rows from each CTA)
template <bool FP8>
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  if constexpr (FP8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
  }
}
template <bool FP8>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t acc) {
  if constexpr (FP8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
        : "memory");
  }
}
// The same with a compile-time accumulate flag: no predicate has to be computed at run time.
template <bool FP8, bool ACC>
__device__ __forceinline__ void tc_mma_const(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  if constexpr (FP8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC ? 1 : 0)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "n"(ACC ? 1 : 0)
        : "memory");
  }
}
// Packed fp32 pair FMA: d = a * b + d on two lanes of a 64-bit register pair.  Half the issue
// slots of two scalar FMAs, which matters for warps that share a scheduler with the thread
// that feeds the tensor core.
__device__ __forceinline__ void fma2(unsigned long long& d, uint32_t a_lo, uint32_t a_hi, unsigned long long b2) {
  unsigned long long a2;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a2) : "r"(a_lo), "r"(a_hi));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a2), "l"(b2));
}
__device__ __forceinline__ unsigned long long splat2(float v) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "r"(__float_as_uint(v)));
  return r;
}
// Two 32-column loads and the wait in ONE asm statement: the 64 results only
// become visible to the compiler after the wait, so nothing can be scheduled
// between the loads and the wait, and no extra register copies are needed.
__device__ __forceinline__ void tmem_ld64_sync(uint32_t taddr, uint32_t* a, uint32_t* b) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]),
        "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]),
        "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]),
        "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]),
        "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]),
        "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]),
        "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]),
        "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
      : "r"(taddr), "r"(taddr + 32)
      : "memory");
}
// One 32-column load WITHOUT the wait, and the wait as a statement that "rewrites" the
// destination registers, so that no use of them can be scheduled above it.
#define MOE_R8(a, o) "=r"(a[o]), "=r"(a[o + 1]), "=r"(a[o + 2]), "=r"(a[o + 3]), "=r"(a[o + 4]), "=r"(a[o + 5]), "=r"(a[o + 6]), "=r"(a[o + 7])
#define MOE_RW8(a, o) "+r"(a[o]), "+r"(a[o + 1]), "+r"(a[o + 2]), "+r"(a[o + 3]), "+r"(a[o + 4]), "+r"(a[o + 5]), "+r"(a[o + 6]), "+r"(a[o + 7])
__device__ __forceinline__ void tmem_ld32_async(uint32_t taddr, uint32_t* a) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : MOE_R8(a, 0), MOE_R8(a, 8), MOE_R8(a, 16), MOE_R8(a, 24)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_wait64(uint32_t* a, uint32_t* b) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : MOE_RW8(a, 0), MOE_RW8(a, 8), MOE_RW8(a, 16), MOE_RW8(a, 24), MOE_RW8(b, 0), MOE_RW8(b, 8), MOE_RW8(b, 16),
                 MOE_RW8(b, 24)::"memory");
}
#undef MOE_R8
#undef MOE_RW8
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src) : "memory");
}
// The barrier receives one arrival when all earlier cp.async of this thread have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 bytes per lane: a whole sector per store, so a row segment written by one thread costs
// half the sector writes of two 16-byte stores.  The address must be 32-byte aligned.
__device__ __forceinline__ void st_global_32(void* p, const uint4& a, const uint4& b) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
               "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
               : "memory");
}
// stores 2n 16-byte pieces v[0..2n) to consecutive addresses, as n 32-byte stores when `wide`
template <int N2>
__device__ __forceinline__ void store_row_pieces(void* dst, const uint4 (&v)[N2], bool wide) {
  static_assert(N2 % 2 == 0, "pairs of 16-byte pieces");
  if (wide) {
#pragma unroll
    for (int i = 0; i < N2; i += 2) st_global_32(reinterpret_cast<uint8_t*>(dst) + 16 * i, v[i], v[i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < N2; ++i) reinterpret_cast<uint4*>(dst)[i] = v[i];
  }
}
// K-major operand tile with 128-byte swizzle: rows are 128 B apart, groups of
// 8 rows 1024 B apart (stride byte offset), descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;            // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;            // descriptor version
  d |= (uint64_t)2 << 61;            // SWIZZLE_128B
  return d;
}

template <typename AT>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// SiLU(g) * u with the fast exponential and division; like the reference kernel
// (tl.exp / tl.fdiv, src/flaggems_vllm/ops/fused_moe.py:1795) it is accurate
// to a couple of ulp, far inside the layer tolerance.
__device__ __forceinline__ float silu_mul_fast(float g, float u) {
  return __fdividef(g, 1.0f + __expf(-g)) * u;
}
template <typename AT>
__device__ __forceinline__ float round_act(float v) {
  return ToF32<AT>::get(from_f32<AT>(v));
}

// Four int8 (one 32-bit word, lowest byte = lowest K index) -> four AT values in two words.
template <typename AT>
__device__ __forceinline__ void widen4(uint32_t w, uint32_t& lo, uint32_t& hi);
// bf16: with x = m - 128 s (m = low seven bits, s = sign bit), 0x4300 | m is 128 + m and
// 0x4300 | (s << 7) is 128 (1 + s), both exact, and so is their difference x
template <>
__device__ __forceinline__ void widen4<__nv_bfloat16>(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t m = w & 0x7F7F7F7Fu, sg = w & 0x80808080u;
  uint32_t a01 = __byte_perm(m, 0x43434343u, 0x4140), a23 = __byte_perm(m, 0x43434343u, 0x4342);
  uint32_t b01 = __byte_perm(sg, 0x43434343u, 0x4140), b23 = __byte_perm(sg, 0x43434343u, 0x4342);
  const __nv_bfloat162 r01 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a01), *reinterpret_cast<__nv_bfloat162*>(&b01));
  const __nv_bfloat162 r23 = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a23), *reinterpret_cast<__nv_bfloat162*>(&b23));
  lo = *reinterpret_cast<const uint32_t*>(&r01);
  hi = *reinterpret_cast<const uint32_t*>(&r23);
}
// f16: 0x6400 | u is 1024 + u; subtracting 1152 leaves x exactly
template <>
__device__ __forceinline__ void widen4<__half>(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;
  uint32_t h01 = __byte_perm(u, 0x64646464u, 0x4140);
  uint32_t h23 = __byte_perm(u, 0x64646464u, 0x4342);
  const uint32_t bias = 0x64806480u;  // (1152, 1152)
  const __half2 r01 = __hsub2(*reinterpret_cast<__half2*>(&h01), *reinterpret_cast<const __half2*>(&bias));
  const __half2 r23 = __hsub2(*reinterpret_cast<__half2*>(&h23), *reinterpret_cast<const __half2*>(&bias));
  lo = *reinterpret_cast<const uint32_t*>(&r01);
  hi = *reinterpret_cast<const uint32_t*>(&r23);
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

// 2-D row-major [rows, cols] tensor, box = `box_bytes` of a row x box_rows rows.  128-byte
// boxes use the 128-byte swizzle (tensor-core operand layout); narrower boxes land unswizzled.
static inline int make_map(CUtensorMap* m, const void* base, CUtensorMapDataType dt, int elem_bytes, uint64_t rows,
                           uint64_t cols, uint32_t box_rows, bool weights, int box_bytes = 128) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return fail(MOE_E_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  if (((uintptr_t)base & 15) != 0) return fail(MOE_E_BADARG, "tensor-core GEMM: operand not 16-byte aligned");
  if ((cols * elem_bytes) % 16 != 0) return fail(MOE_E_SHAPE, "tensor-core GEMM: row pitch must be a multiple of 16 bytes");
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstr[1] = {cols * (uint64_t)elem_bytes};
  cuuint32_t box[2] = {(cuuint32_t)(box_bytes / elem_bytes), box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, dt, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   weights ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(MOE_E_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return 0;
}

}  // namespace tc
}  // namespace moe
