// Generic (CUDA-core) expert grouped GEMMs.  They accept every mode, dtype and
// shape the tensor-core kernels do not (odd hidden sizes, small align blocks)
// and serve as an independent cross-check of those kernels in the tests.
// Same inputs/outputs as the tcgen05 kernels: activations in expert-sorted
// order, one expert per align block.
//
// Tile: 16 sorted rows x 128 output columns per CTA (256 threads, each 1 row x
// 8 columns), K staged through shared memory 32 at a time, operands converted
// to fp32 (and block-scaled, FP8 mode) on load, fp32 accumulation.
#include "moe_common.cuh"

namespace moe {
namespace {

constexpr int TM = 16, TN = 128, BK = 32, CPT = 8;

template <int MODE, typename AT> struct Elem;  // element types of A and W per mode
template <typename AT> struct Elem<MOE_MODE_HALF, AT> { using A = AT; using W = AT; };
template <typename AT> struct Elem<MOE_MODE_FP8_BLOCK, AT> { using A = uint8_t; using W = uint8_t; };
template <typename AT> struct Elem<MOE_MODE_W8A16, AT> { using A = AT; using W = int8_t; };
template <typename AT> struct Elem<MOE_MODE_FP8_ROW, AT> { using A = uint8_t; using W = uint8_t; };
template <typename AT> struct Elem<MOE_MODE_INT8_ROW, AT> { using A = int8_t; using W = int8_t; };

// gate/up -> activation value; `kind` is MOE_ACT_SILU or MOE_ACT_SWIGLUOAI
// (src/flaggems_vllm/ops/fused_moe.py:733-773: clamps that let NaN through, sigmoid(alpha * gate))
__device__ __forceinline__ float gated_activation(int kind, float g, float u, float alpha, float beta, float limit) {
  if (kind == MOE_ACT_SILU) return silu_mul(g, u);
  g = (g != g) ? g : fminf(g, limit);
  u = (u != u) ? u : fminf(fmaxf(u, -limit), limit);
  return g * (1.0f / (1.0f + expf(-alpha * g))) * (u + beta);
}

template <int MODE, typename T> __device__ __forceinline__ float load_a(const T* p) {
  if constexpr (MODE == MOE_MODE_FP8_BLOCK || MODE == MOE_MODE_FP8_ROW) return fp8e4m3_to_f32(*p);
  else if constexpr (MODE == MOE_MODE_INT8_ROW) return (float)(*p);
  else return ToF32<T>::get(*p);
}
template <int MODE, typename T> __device__ __forceinline__ float load_w(const T* p) {
  if constexpr (MODE == MOE_MODE_FP8_BLOCK || MODE == MOE_MODE_FP8_ROW) return fp8e4m3_to_f32(*p);
  else if constexpr (MODE == MOE_MODE_W8A16 || MODE == MOE_MODE_INT8_ROW) return (float)(*p);
  else return ToF32<T>::get(*p);
}

// GEMM1 = true : out[p, n] = silu(g) * u,  g = A[p] . W[e, n],  u = A[p] . W[e, I + n]
// GEMM1 = false: y[sorted_ids[p], n] = (A[p] . W[e, n]) * route_weight
template <int MODE, typename AT, bool GEMM1>
__global__ void __launch_bounds__(256) simt_gemm_kernel(
    const typename Elem<MODE, AT>::A* __restrict__ a, const float* __restrict__ a_scales_t,
    const typename Elem<MODE, AT>::W* __restrict__ w, const float* __restrict__ w_scale,
    const int32_t* __restrict__ expert_ids, const int32_t* __restrict__ sorted_ids,
    const int32_t* __restrict__ num_post_pad, const float* __restrict__ route_weight, int mul_weight,
    int64_t numel, int64_t rows_cap, int64_t a_tokens, int topk, int block_m, int E, int K, int Nout,
    void* __restrict__ out, float* __restrict__ out_scales_t, int32_t* __restrict__ status, int act_kind,
    float alpha, float beta, float limit) {
  using WT = typename Elem<MODE, AT>::W;
  using AE = typename Elem<MODE, AT>::A;
  __shared__ float As[TM][BK + 1];
  __shared__ float Bs[TN][BK + 1];
  __shared__ float Us[GEMM1 ? TN : 1][BK + 1];

  const int64_t row0 = (int64_t)blockIdx.y * TM;
  if (row0 >= (int64_t)num_post_pad[0] || row0 >= rows_cap) return;
  const int e = expert_ids[row0 / block_m];
  if (e < 0 || e >= E) return;  // block of an expert that lives on another rank
  const int n0 = blockIdx.x * TN;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int64_t Nw = GEMM1 ? 2 * (int64_t)Nout : (int64_t)Nout;  // rows of W per expert
  const WT* wbase = w + (int64_t)e * Nw * K;
  const int kblocks = (K + 127) / 128;

  float accg[CPT], accu[CPT];
#pragma unroll
  for (int i = 0; i < CPT; ++i) { accg[i] = 0.0f; accu[i] = 0.0f; }

  for (int k0 = 0; k0 < K; k0 += BK) {
    // A tile: 16 x 32 = 512 elements, 2 per thread
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = tid + i * 256, r = idx / BK, c = idx % BK;
      const int64_t p = row0 + r;
      float v = 0.0f;
      // GEMM1 reads token rows (row p <- token sorted_ids[p] / topk), GEMM2 sorted rows
      int64_t arow = -1, ald = rows_cap;
      if (p < rows_cap) {
        if constexpr (GEMM1) {
          const int64_t s_ = (int64_t)sorted_ids[p];
          if (s_ >= 0 && s_ < numel) arow = s_ / topk;
          ald = a_tokens;
        } else {
          arow = p;
        }
      }
      if (arow >= 0 && k0 + c < K) {
        v = load_a<MODE, AE>(a + arow * K + k0 + c);
        if constexpr (MODE == MOE_MODE_FP8_BLOCK) v *= a_scales_t[(int64_t)((k0 + c) / 128) * ald + arow];
      }
      As[r][c] = v;
    }
    // W tile(s): 128 x 32 = 4096 elements, 16 per thread
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int idx = tid + i * 256, r = idx / BK, c = idx % BK;
      const int n = n0 + r;
      float v = 0.0f, vu = 0.0f;
      if (n < Nout && k0 + c < K) {
        v = load_w<MODE, WT>(wbase + (int64_t)n * K + k0 + c);
        if constexpr (MODE == MOE_MODE_FP8_BLOCK)
          v *= w_scale[((int64_t)e * ((Nw + 127) / 128) + n / 128) * kblocks + (k0 + c) / 128];
        if constexpr (GEMM1) {
          const int64_t nu = (int64_t)Nout + n;
          vu = load_w<MODE, WT>(wbase + nu * K + k0 + c);
          if constexpr (MODE == MOE_MODE_FP8_BLOCK)
            vu *= w_scale[((int64_t)e * ((Nw + 127) / 128) + nu / 128) * kblocks + (k0 + c) / 128];
        }
      }
      Bs[r][c] = v;
      if constexpr (GEMM1) Us[r][c] = vu;
    }
    __syncthreads();
#pragma unroll 8
    for (int kk = 0; kk < BK; ++kk) {
      const float av = As[ty][kk];
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        accg[i] = fmaf(av, Bs[tx + 16 * i][kk], accg[i]);
        if constexpr (GEMM1) accu[i] = fmaf(av, Us[tx + 16 * i][kk], accu[i]);
      }
    }
    __syncthreads();
  }

  // epilogue; column of accumulator i is n0 + tx + 16*i
  const int64_t p = row0 + ty;
  const int64_t sid = p < rows_cap ? (int64_t)sorted_ids[p] : numel;
  const bool row_ok = sid >= 0 && sid < numel;
  float rw = 1.0f;
  if (mul_weight && row_ok) rw = route_weight[sid];
  constexpr bool ROW_SCALED = MODE == MOE_MODE_FP8_ROW || MODE == MOE_MODE_INT8_ROW;
  if constexpr (ROW_SCALED) {
    // one activation scale per row: of the token (GEMM1) or of the sorted intermediate row (GEMM2)
    float as = 0.0f;
    if (row_ok) as = GEMM1 ? a_scales_t[sid / topk] : a_scales_t[p];
#pragma unroll
    for (int i = 0; i < CPT; ++i) { accg[i] *= as; accu[i] *= as; }
  }
  if (ROW_SCALED || MODE == MOE_MODE_W8A16 || (MODE == MOE_MODE_HALF && w_scale != nullptr)) {
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      const int n = n0 + tx + 16 * i;
      if (n < Nout) {
        accg[i] *= w_scale[(int64_t)e * Nw + n];
        if constexpr (GEMM1) accu[i] *= w_scale[(int64_t)e * Nw + Nout + n];
      }
    }
  }
  if constexpr (GEMM1) {
    float v[CPT];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      // rounded to the activation dtype first: that is what the reference
      // stores and re-quantises (src/flaggems_vllm/ops/fused_moe.py:1969, 2658-2666)
      if constexpr (ROW_SCALED) {
        // the reference rounds GEMM 1's output to the activation dtype before the activation kernel reads it
        accg[i] = ToF32<AT>::get(from_f32<AT>(accg[i] * rw));
        accu[i] = ToF32<AT>::get(from_f32<AT>(accu[i] * rw));
        v[i] = ToF32<AT>::get(from_f32<AT>(gated_activation(act_kind, accg[i], accu[i], alpha, beta, limit)));
      } else if (act_kind != MOE_ACT_SILU) {
        // unfused activations read GEMM 1's output after it was stored in the activation dtype
        const float gq = ToF32<AT>::get(from_f32<AT>(accg[i] * rw)), uq = ToF32<AT>::get(from_f32<AT>(accu[i] * rw));
        v[i] = ToF32<AT>::get(from_f32<AT>(gated_activation(act_kind, gq, uq, alpha, beta, limit)));
      } else {
        v[i] = ToF32<AT>::get(from_f32<AT>(silu_mul(accg[i] * rw, accu[i] * rw)));
      }
      amax = fmaxf(amax, fabsf(v[i]));
    }
    if constexpr (MODE == MOE_MODE_FP8_BLOCK) {
      // the 128 columns of this tile are exactly one quantisation group,
      // held by the 16 threads of a half-warp that share `ty`
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
      const float s = fmaxf(amax, kQuantEps) * (1.0f / kFp8Max);
      if (row_ok) {
        uint8_t* o = reinterpret_cast<uint8_t*>(out) + p * Nout;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          const int n = n0 + tx + 16 * i;
          if (n < Nout) o[n] = f32_to_fp8e4m3(fminf(fmaxf(v[i] / s, -kFp8Max), kFp8Max));
        }
        if (tx == 0) out_scales_t[(int64_t)(n0 / 128) * rows_cap + p] = s;
      }
    } else if (row_ok) {
      AT* o = reinterpret_cast<AT*>(out) + p * Nout;
#pragma unroll
      for (int i = 0; i < CPT; ++i) {
        const int n = n0 + tx + 16 * i;
        if (n < Nout) o[n] = from_f32<AT>(v[i]);
      }
    }
  } else if (row_ok) {
    AT* o = reinterpret_cast<AT*>(out) + sid * Nout;
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      const int n = n0 + tx + 16 * i;
      if (n < Nout) o[n] = from_f32<AT>(accg[i] * rw);
    }
  }
  (void)status;
}

template <int MODE, typename AT, bool GEMM1>
int launch(const void* a, const float* a_scales_t, const void* w, const float* w_scale,
           const int32_t* expert_ids, const int32_t* sorted_ids, const int32_t* npp,
           const float* route_weight, int mul_weight, int64_t numel, int64_t rows_cap, int64_t a_tokens, int topk, int block_m,
           int E, int K, int Nout, void* out, float* out_scales_t, int32_t* status, cudaStream_t st, int act_kind,
           float alpha, float beta, float limit) {
  dim3 grid((unsigned)((Nout + TN - 1) / TN), (unsigned)((rows_cap + TM - 1) / TM));
  if (grid.y > 65535) return fail(MOE_E_TOOBIG, "generic GEMM: more than 65535 row tiles");
  simt_gemm_kernel<MODE, AT, GEMM1><<<grid, 256, 0, st>>>(
      (const typename Elem<MODE, AT>::A*)a, a_scales_t, (const typename Elem<MODE, AT>::W*)w, w_scale,
      expert_ids, sorted_ids, npp, route_weight, mul_weight, numel, rows_cap, a_tokens, topk, block_m, E, K, Nout, out,
      out_scales_t, status, act_kind, alpha, beta, limit);
  return check_launch(GEMM1 ? "gemm1 (generic)" : "gemm2 (generic)");
}

template <bool GEMM1, typename AT>
int dispatch_mode(int mode, const void* a, const float* a_scales_t, const void* w,
                  const float* w_scale, const int32_t* expert_ids, const int32_t* sorted_ids,
                  const int32_t* npp, const float* route_weight, int mul_weight, int64_t numel,
                  int64_t rows_cap, int64_t a_tokens, int topk, int block_m, int E, int K, int Nout, void* out,
                  float* out_scales_t, int32_t* status, cudaStream_t st, int act_kind, float alpha, float beta,
                  float limit) {
  switch (mode) {
    case MOE_MODE_HALF:
      return launch<MOE_MODE_HALF, AT, GEMM1>(a, a_scales_t, w, w_scale, expert_ids, sorted_ids, npp, route_weight, mul_weight, numel, rows_cap, a_tokens, topk, block_m, E, K, Nout, out, out_scales_t, status, st, act_kind, alpha, beta, limit);
    case MOE_MODE_FP8_BLOCK:
      return launch<MOE_MODE_FP8_BLOCK, AT, GEMM1>(a, a_scales_t, w, w_scale, expert_ids, sorted_ids, npp, route_weight, mul_weight, numel, rows_cap, a_tokens, topk, block_m, E, K, Nout, out, out_scales_t, status, st, act_kind, alpha, beta, limit);
    case MOE_MODE_W8A16:
      return launch<MOE_MODE_W8A16, AT, GEMM1>(a, a_scales_t, w, w_scale, expert_ids, sorted_ids, npp, route_weight, mul_weight, numel, rows_cap, a_tokens, topk, block_m, E, K, Nout, out, out_scales_t, status, st, act_kind, alpha, beta, limit);
    case MOE_MODE_FP8_ROW:
      return launch<MOE_MODE_FP8_ROW, AT, GEMM1>(a, a_scales_t, w, w_scale, expert_ids, sorted_ids, npp, route_weight, mul_weight, numel, rows_cap, a_tokens, topk, block_m, E, K, Nout, out, out_scales_t, status, st, act_kind, alpha, beta, limit);
    case MOE_MODE_INT8_ROW:
      return launch<MOE_MODE_INT8_ROW, AT, GEMM1>(a, a_scales_t, w, w_scale, expert_ids, sorted_ids, npp, route_weight, mul_weight, numel, rows_cap, a_tokens, topk, block_m, E, K, Nout, out, out_scales_t, status, st, act_kind, alpha, beta, limit);
    default:
      return fail(MOE_E_BADARG, "unknown GEMM mode %d", mode);
  }
}

}  // namespace

// Entry used by the C ABI functions in gemm_api.cu
int simt_gemm(bool gemm1, int mode, int act_dtype, const void* a, const float* a_scales_t,
              const void* w, const float* w_scale, const int32_t* expert_ids,
              const int32_t* sorted_ids, const int32_t* npp, const float* route_weight,
              int mul_weight, int64_t numel, int64_t rows_cap, int64_t a_tokens, int topk, int block_m, int E, int K, int Nout,
              void* out, float* out_scales_t, int32_t* status, cudaStream_t st, int act_kind, float alpha, float beta,
              float limit) {
  if (block_m % TM != 0) return fail(MOE_E_SHAPE, "generic GEMM: align block must be a multiple of 16");
  if (mode == MOE_MODE_FP8_BLOCK && (K % 128 != 0 || (gemm1 && Nout % 128 != 0)))
    return fail(MOE_E_SHAPE, "generic GEMM: FP8 block mode needs sizes that are multiples of 128");
#define MOE_SIMT_DISPATCH(G1, T)                                                                    \
  dispatch_mode<G1, T>(mode, a, a_scales_t, w, w_scale, expert_ids, sorted_ids, npp, route_weight, \
                       mul_weight, numel, rows_cap, a_tokens, topk, block_m, E, K, Nout, out, out_scales_t, status, st, \
                       act_kind, alpha, beta, limit)
  if (act_dtype == MOE_BF16) return gemm1 ? MOE_SIMT_DISPATCH(true, __nv_bfloat16) : MOE_SIMT_DISPATCH(false, __nv_bfloat16);
  if (act_dtype == MOE_F16) return gemm1 ? MOE_SIMT_DISPATCH(true, __half) : MOE_SIMT_DISPATCH(false, __half);
  if (act_dtype == MOE_F32) {
    if (mode != MOE_MODE_HALF && mode != MOE_MODE_W8A16) return fail(MOE_E_DTYPE, "8-bit activation modes need f16/bf16 as the activation dtype");
    return gemm1 ? MOE_SIMT_DISPATCH(true, float) : MOE_SIMT_DISPATCH(false, float);
  }
#undef MOE_SIMT_DISPATCH
  return fail(MOE_E_DTYPE, "generic GEMM: unsupported activation dtype %d", act_dtype);
}

}  // namespace moe
