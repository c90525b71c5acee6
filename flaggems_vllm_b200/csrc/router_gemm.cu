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
#include "moe_common.cuh"

namespace moe {
namespace {

constexpr int kThreads = 128;
constexpr int kRows = 8;

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __half22float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}

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
  switch (x_dtype) {
    case MOE_F32: return launch_w<float>(x, x_ld, w, w_dtype, M, N, K, out, st);
    case MOE_F16: return launch_w<__half>(x, x_ld, w, w_dtype, M, N, K, out, st);
    case MOE_BF16: return launch_w<__nv_bfloat16>(x, x_ld, w, w_dtype, M, N, K, out, st);
    default: return fail(MOE_E_DTYPE, "router_gemm: unsupported input dtype %d", x_dtype);
  }
}
