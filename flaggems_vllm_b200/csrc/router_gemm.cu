// Router GEMM in front of the routers: logits[M, N] = x[M, K] . w[N, K]^T, fp32 accumulate and
// fp32 output, for decode-sized M.  Stands in for router_gemm (bf16 x bf16 -> fp32,
// src/flaggems_vllm/ops/router_gemm.py:207-237) and fp32_router_gemm (bf16/fp32 x fp32 -> fp32,
// src/flaggems_vllm/ops/fp32_router_gemm.py:108-145).
//
// One CTA of 128 threads per (expert row n, tile of 8 token rows): the weight row is read once
// per CTA (16-byte loads, each thread a strided set of 8-element chunks), the token rows come from
// L2, every product is formed in fp32 and the reduction order is fixed (lane partial sums ->
// warp shuffle tree -> four warp sums added in warp order), so the result is run-to-run
// deterministic: no split-K atomics.  Bound: latency and L2 bandwidth; algorithmic bytes
// N*K*b_w + M*K*b_x + 4*M*N.
#include <type_traits>

#include "moe_common.cuh"

namespace moe {
namespace {

constexpr int kThreads = 128;
constexpr int kRows = 8;

template <typename XT, typename WT>
__global__ void __launch_bounds__(kThreads) router_gemm_kernel(const XT* __restrict__ x, int64_t x_ld,
                                                                const WT* __restrict__ w, int64_t M, int N, int K,
                                                                float* __restrict__ out) {
  const int n = blockIdx.x;
  const int64_t m0 = (int64_t)blockIdx.y * kRows;
  const int rows = (int)min((int64_t)kRows, M - m0);
  const WT* wr = w + (int64_t)n * K;
  float acc[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;
  for (int k = threadIdx.x * 8; k < K; k += kThreads * 8) {
    float wv[8];
    load8<WT>(wr + k, wv);
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      if (r < rows) {
        float xv[8];
        load8<XT>(x + (m0 + r) * x_ld + k, xv);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r] = fmaf(xv[i], wv[i], acc[r]);
      }
    }
  }
  __shared__ float part[kThreads / 32][kRows];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int r = 0; r < kRows; ++r) {
    float v = acc[r];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, off);
    if (lane == 0) part[warp][r] = v;
  }
  __syncthreads();
  if (threadIdx.x < rows) {
    float v = part[0][threadIdx.x];
#pragma unroll
    for (int wi = 1; wi < kThreads / 32; ++wi) v += part[wi][threadIdx.x];
    out[(m0 + threadIdx.x) * N + n] = v;
  }
}

// Prefill-sized batches: warp-level tensor-core MMA (m16n8k16, fp32 accumulate), 64 x 128 output tile
// per CTA, K staged 32 elements at a time through a double-buffered cp.async ring.  The
// accumulation order is fixed, so the result is run-to-run deterministic.  f16 / bf16 operands of
// one type; K a multiple of 32.
constexpr int PM = 64, PN = 128, PK = 32, PPAD = 8, PTHREADS = 256;

__device__ __forceinline__ void cp16(void* smem_dst, const void* src, bool pred) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int bytes = pred ? 16 : 0;  // zero-fill rows beyond the matrix
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void ldsm4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}

template <typename T>
__global__ void __launch_bounds__(PTHREADS) router_gemm_mma_kernel(const T* __restrict__ x, int64_t x_ld,
                                                                   const T* __restrict__ w, int64_t M, int N, int K,
                                                                   float* __restrict__ out) {
  __shared__ __align__(16) T As[2][PM][PK + PPAD];
  __shared__ __align__(16) T Bs[2][PN][PK + PPAD];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wm = warp >> 2, wn = warp & 3;  // 2 x 4 warps, 32 x 32 outputs each
  const int64_t m0 = (int64_t)blockIdx.y * PM;
  const int n0 = blockIdx.x * PN;
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.0f;

  auto stage = [&](int buf, int k0) {
    // A: 64 rows x 4 chunks of 8 elements = 256 chunks, one per thread; B: 128 x 4 = 512, two per thread
    {
      const int r = tid >> 2, c = tid & 3;
      const bool ok = m0 + r < M;
      cp16(&As[buf][r][c * 8], x + (ok ? (m0 + r) : 0) * x_ld + k0 + c * 8, ok);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * PTHREADS, r = idx >> 2, c = idx & 3;
      const bool ok = n0 + r < N;
      cp16(&Bs[buf][r][c * 8], w + (int64_t)(ok ? (n0 + r) : 0) * K + k0 + c * 8, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  const int steps = K / PK;
  stage(0, 0);
  for (int s = 0; s < steps; ++s) {
    if (s + 1 < steps) {
      stage((s + 1) & 1, (s + 1) * PK);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const int buf = s & 1;
#pragma unroll
    for (int kk = 0; kk < PK; kk += 16) {
      uint32_t a[2][4], b[2][4];
#pragma unroll
      for (int i = 0; i < 2; ++i)  // rows 16 i + (lane & 15), k half (lane >> 4)
        ldsm4(a[i], &As[buf][wm * 32 + i * 16 + (lane & 15)][kk + ((lane >> 4) << 3)]);
#pragma unroll
      for (int j = 0; j < 2; ++j)  // two n-fragments of 8 columns each per ldmatrix.x4
        ldsm4(b[j], &Bs[buf][wn * 32 + j * 16 + ((lane >> 4) << 3) + (lane & 7)][kk + (((lane >> 3) & 1) << 3)]);
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) mma16816<T>(acc[i][j], a[i], b[j >> 1][(j & 1) * 2], b[j >> 1][(j & 1) * 2 + 1]);
    }
    __syncthreads();
  }
  const int g = lane >> 2, q = lane & 3;
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + wn * 32 + j * 8 + 2 * q;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int64_t m = m0 + wm * 32 + i * 16 + g + 8 * h;
        if (m < M) {
          if (n < N) out[m * N + n] = acc[i][j][2 * h];
          if (n + 1 < N) out[m * N + n + 1] = acc[i][j][2 * h + 1];
        }
      }
    }
}

template <typename XT>
int launch_w(const void* x, int64_t x_ld, const void* w, int w_dtype, int64_t M, int N, int K, float* out,
             cudaStream_t st) {
  const dim3 grid((unsigned)N, (unsigned)((M + kRows - 1) / kRows));
  switch (w_dtype) {
    case MOE_F32:
      router_gemm_kernel<XT, float><<<grid, kThreads, 0, st>>>((const XT*)x, x_ld, (const float*)w, M, N, K, out);
      break;
    case MOE_F16:
      router_gemm_kernel<XT, __half><<<grid, kThreads, 0, st>>>((const XT*)x, x_ld, (const __half*)w, M, N, K, out);
      break;
    case MOE_BF16:
      router_gemm_kernel<XT, __nv_bfloat16><<<grid, kThreads, 0, st>>>((const XT*)x, x_ld, (const __nv_bfloat16*)w, M, N,
                                                                     K, out);
      break;
    default: return fail(MOE_E_DTYPE, "router_gemm: unsupported weight dtype %d", w_dtype);
  }
  return check_launch("router_gemm");
}

}  // namespace
}  // namespace moe

extern "C" int moe_router_gemm(const void* x, int x_dtype, int64_t x_ld, const void* w, int w_dtype, int64_t M, int N,
                               int K, float* out, void* stream) {
  using namespace moe;
  if (M < 0 || N <= 0 || K <= 0) return fail(MOE_E_BADARG, "router_gemm: bad extent");
  if (M == 0) return 0;
  if (!x || !w || !out) return fail(MOE_E_BADARG, "router_gemm: null pointer");
  if (K % 8 != 0 || x_ld % 8 != 0 || x_ld < K) return fail(MOE_E_SHAPE, "router_gemm: K and the row pitch must be multiples of 8");
  if (((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return fail(MOE_E_BADARG, "router_gemm: operands must be 16-byte aligned");
  if ((M + kRows - 1) / kRows > 65535) return fail(MOE_E_TOOBIG, "router_gemm: serves at most %d rows", 65535 * kRows);
  cudaStream_t st = (cudaStream_t)stream;
  // prefill-sized half-precision products run on the tensor cores.  Its grid is one CTA per
  // 64 x 128 logits, a handful of CTAs for a few hundred rows (130-170 us at 128-256 rows of
  // K = 7168), where the row-streaming kernel with one CTA per logit column still wins.
  if (M > 320 && x_dtype == w_dtype && (x_dtype == MOE_BF16 || x_dtype == MOE_F16) && K % PK == 0) {
    const dim3 grid((unsigned)((N + PN - 1) / PN), (unsigned)((M + PM - 1) / PM));
    if (grid.y > 65535) return fail(MOE_E_TOOBIG, "router_gemm: serves at most %d rows", 65535 * PM);
    if (x_dtype == MOE_BF16)
      router_gemm_mma_kernel<__nv_bfloat16><<<grid, PTHREADS, 0, st>>>((const __nv_bfloat16*)x, x_ld, (const __nv_bfloat16*)w, M, N, K, out);
    else
      router_gemm_mma_kernel<__half><<<grid, PTHREADS, 0, st>>>((const __half*)x, x_ld, (const __half*)w, M, N, K, out);
    return check_launch("router_gemm (mma)");
  }
  switch (x_dtype) {
    case MOE_F32: return launch_w<float>(x, x_ld, w, w_dtype, M, N, K, out, st);
    case MOE_F16: return launch_w<__half>(x, x_ld, w, w_dtype, M, N, K, out, st);
    case MOE_BF16: return launch_w<__nv_bfloat16>(x, x_ld, w, w_dtype, M, N, K, out, st);
    default: return fail(MOE_E_DTYPE, "router_gemm: unsupported input dtype %d", x_dtype);
  }
}
