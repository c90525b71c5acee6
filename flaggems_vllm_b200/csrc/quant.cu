// Row kernels around the grouped GEMMs:
//   * per_token_group_quant_fp8: 1x128 e4m3 quantiser (row-major or transposed scales).
//   * moe_sum: fixed-order fp32 reduction over the top-k axis.
// Quantisation follows the reference kernel exactly
// (src/flaggems_vllm/ops/per_token_group_quant_fp8.py:150-156):
//   s = max(amax, 1e-10) * (1/448);  q = clamp(x / s, -448, 448) -> e4m3 (RN).
#include "moe_common.cuh"

namespace moe {
namespace {

constexpr int kRowThreads = 256;

// One warp quantises one 128-wide group: 4 consecutive elements per lane.  The load is a
// separate step so that a warp can have the loads of several groups in flight.
template <typename T>
__device__ __forceinline__ void load_group_128(const T* __restrict__ src, int lane, float (&v)[4]) {
  if constexpr (sizeof(T) == 2) {
    uint2 raw = *reinterpret_cast<const uint2*>(src + lane * 4);
    const T* p = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = ToF32<T>::get(p[i]);
  } else {
    float4 raw = *reinterpret_cast<const float4*>(src + lane * 4);
    v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
  }
}
template <bool UE8M0>
__device__ __forceinline__ void quant_group_128(const float (&v)[4], uint8_t* __restrict__ dst,
                                                float* __restrict__ scale_out, int lane) {
  float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
  float s = fmaxf(amax, kQuantEps) * (1.0f / kFp8Max);
  // power-of-two (UE8M0) scales: exp2(ceil(log2(max(|s|, 1e-10)))), the reference's expression
  // (src/flaggems_vllm/ops/per_token_group_quant_fp8.py:153-154)
  if (UE8M0) s = exp2f(ceilf(log2f(fmaxf(fabsf(s), 1e-10f))));
  uint32_t packed = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float q = fminf(fmaxf(v[i] / s, -kFp8Max), kFp8Max);
    packed |= (uint32_t)f32_to_fp8e4m3(q) << (8 * i);
  }
  *reinterpret_cast<uint32_t*>(dst + lane * 4) = packed;
  if (lane == 0) *scale_out = s;
}

// int8 -> f16/bf16, exact; 16 elements per thread per step
template <typename T>
__global__ void __launch_bounds__(256) widen_int8_kernel(const int8_t* __restrict__ src, T* __restrict__ dst, int64_t n16) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (int64_t)gridDim.x * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(src)[i];
    const int8_t* p = reinterpret_cast<const int8_t*>(&raw);
    uint4 o[2];
    T* q = reinterpret_cast<T*>(o);
#pragma unroll
    for (int j = 0; j < 16; ++j) q[j] = from_f32<T>((float)p[j]);
    reinterpret_cast<uint4*>(dst)[2 * i] = o[0];
    reinterpret_cast<uint4*>(dst)[2 * i + 1] = o[1];
  }
}

template <typename T, bool UE8M0>
__global__ void __launch_bounds__(kRowThreads) quant_rows_kernel(
    const T* __restrict__ x, int64_t rows, int64_t cols, uint8_t* __restrict__ q,
    float* __restrict__ scales, int transposed, int64_t scale_ld) {
  const int lane = threadIdx.x & 31;
  const int64_t groups_per_row = cols / 128;
  const int64_t total = rows * groups_per_row;
  const int64_t warp0 = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * (kRowThreads / 32);
  constexpr int U = 4;  // groups in flight per warp
  for (int64_t w = warp0; w < total; w += U * stride) {
    float v[U][4];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t wu = w + u * stride;
      if (wu < total) load_group_128<T>(x + wu * 128, lane, v[u]);  // rows are contiguous: group wu starts at wu * 128
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t wu = w + u * stride;
      if (wu < total) {
        const int64_t r = wu / groups_per_row, g = wu % groups_per_row;
        float* so = transposed ? scales + g * scale_ld + r : scales + r * groups_per_row + g;
        quant_group_128<UE8M0>(v[u], q + wu * 128, so, lane);
      }
    }
  }
}

// The same quantiser for 2-byte inputs with an even number of groups per row: a warp step covers
// two neighbouring groups (8 elements = 16 bytes per lane, one half-warp per group), so a warp has
// twice the bytes in flight per load instruction.  Bit for bit the arithmetic of quant_group_128.
template <typename T>
__global__ void __launch_bounds__(kRowThreads) quant_rows_pair_kernel(
    const T* __restrict__ x, int64_t rows, int64_t cols, uint8_t* __restrict__ q, float* __restrict__ scales,
    int transposed, int64_t scale_ld) {
  static_assert(sizeof(T) == 2, "pairs of groups: 2-byte inputs");
  const int lane = threadIdx.x & 31;
  const int64_t groups_per_row = cols / 128;
  const int64_t pairs = rows * (groups_per_row / 2);
  const int64_t warp0 = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * (kRowThreads / 32);
  constexpr int U = 4;  // pairs in flight per warp
  for (int64_t w = warp0; w < pairs; w += U * stride) {
    uint4 raw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t wu = w + u * stride;
      if (wu < pairs) raw[u] = *reinterpret_cast<const uint4*>(x + wu * 256 + lane * 8);  // rows are contiguous
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t wu = w + u * stride;
      if (wu >= pairs) continue;
      const T* pv = reinterpret_cast<const T*>(&raw[u]);
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = ToF32<T>::get(pv[i]);
      float amax = 0.0f;
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
      for (int off = 8; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));  // 16 lanes = one group
      const float s = fmaxf(amax, kQuantEps) * (1.0f / kFp8Max);
      uint32_t lo = 0, hi = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        lo |= (uint32_t)f32_to_fp8e4m3(fminf(fmaxf(v[i] / s, -kFp8Max), kFp8Max)) << (8 * i);
        hi |= (uint32_t)f32_to_fp8e4m3(fminf(fmaxf(v[4 + i] / s, -kFp8Max), kFp8Max)) << (8 * i);
      }
      *reinterpret_cast<uint2*>(q + wu * 256 + lane * 8) = make_uint2(lo, hi);
      if ((lane & 15) == 0) {
        const int64_t gflat = wu * 2 + (lane >> 4);
        const int64_t r = gflat / groups_per_row, g = gflat % groups_per_row;
        *(transposed ? scales + g * scale_ld + r : scales + r * groups_per_row + g) = s;
      }
    }
  }
}

// Any group size, clamp value and 8-bit float format: one warp per group, lanes stride over the
// group (the 128-wide e4m3 kernel above is the fast case of this one).
template <typename T, bool UE8M0, bool E5M2>
__global__ void __launch_bounds__(kRowThreads) quant_rows_generic_kernel(
    const T* __restrict__ x, int64_t rows, int64_t cols, int group, float eps, uint8_t* __restrict__ q,
    float* __restrict__ scales, int transposed, int64_t scale_ld) {
  const int lane = threadIdx.x & 31;
  const float fmax_q = E5M2 ? 57344.0f : kFp8Max;
  const int64_t groups_per_row = cols / group;
  const int64_t total = rows * groups_per_row;
  const int64_t warp0 = (int64_t)blockIdx.x * (kRowThreads / 32) + (threadIdx.x >> 5);
  const int64_t stride = (int64_t)gridDim.x * (kRowThreads / 32);
  for (int64_t w = warp0; w < total; w += stride) {
    const T* src = x + w * group;  // rows are contiguous: group w starts at w * group
    float amax = 0.0f;
    for (int i = lane; i < group; i += 32) amax = fmaxf(amax, fabsf(ToF32<T>::get(src[i])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
    float s = fmaxf(amax, eps) * (1.0f / fmax_q);
    if (UE8M0) s = exp2f(ceilf(log2f(fmaxf(fabsf(s), 1e-10f))));
    for (int i = lane; i < group; i += 32) {
      const float v = fminf(fmaxf(ToF32<T>::get(src[i]) / s, -fmax_q), fmax_q);
      q[w * group + i] = E5M2 ? (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E5M2) : f32_to_fp8e4m3(v);
    }
    if (lane == 0) {
      const int64_t r = w / groups_per_row, g = w % groups_per_row;
      *(transposed ? scales + g * scale_ld + r : scales + r * groups_per_row + g) = s;
    }
  }
}

// out[m, h] = sum_j in[m, j, h]; 8 elements (16 B) of 2-byte types per thread.
template <typename T, typename IdT>
__global__ void __launch_bounds__(256) moe_sum_kernel(
    const T* __restrict__ in, T* __restrict__ out, int64_t M, int topk, int64_t H,
    const IdT* __restrict__ ids, int num_experts, const int32_t* __restrict__ expert_map,
    const int32_t* __restrict__ row_index, bool aligned, int64_t out_ld) {
  constexpr int V = 16 / sizeof(T);
  const int64_t vec_per_row = (H + V - 1) / V;
  const int64_t total = M * vec_per_row;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = idx / vec_per_row, h0 = (idx % vec_per_row) * V;
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = 0.0f;
    const bool full = aligned && (h0 + V <= H) && (H % V == 0);
    if (full) {
      // four 16-byte loads in flight per thread; the adds stay in slot order
      for (int j0 = 0; j0 < topk; j0 += 4) {
        uint4 raw[4];
        bool use[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = j0 + u;
          use[u] = j < topk;
          if (use[u] && ids != nullptr) {
            long long e = (long long)ids[m * topk + j];
            use[u] = e >= 0 && e < num_experts && (expert_map == nullptr || expert_map[e] >= 0);
          }
          if (use[u]) {
            const int64_t src_row = row_index != nullptr ? (int64_t)row_index[m * topk + j] : m * topk + j;
            use[u] = src_row >= 0;
            if (use[u]) raw[u] = *reinterpret_cast<const uint4*>(in + src_row * H + h0);
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (use[u]) {
            const T* p = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] += ToF32<T>::get(p[i]);
          }
        }
      }
    } else {
      for (int j = 0; j < topk; ++j) {
        if (ids != nullptr) {
          long long e = (long long)ids[m * topk + j];
          if (e < 0 || e >= num_experts) continue;
          if (expert_map != nullptr && expert_map[e] < 0) continue;
        }
        const int64_t src_row = row_index != nullptr ? (int64_t)row_index[m * topk + j] : m * topk + j;
        if (src_row < 0) continue;
        const T* src = in + src_row * H + h0;
        for (int i = 0; i < V && h0 + i < H; ++i) acc[i] += ToF32<T>::get(src[i]);
      }
    }
    T* dst = out + m * out_ld + h0;
    if (full) {
      uint4 raw;
      T* p = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int i = 0; i < V; ++i) p[i] = from_f32<T>(acc[i]);
      *reinterpret_cast<uint4*>(dst) = raw;
    } else {
      for (int i = 0; i < V && h0 + i < H; ++i) dst[i] = from_f32<T>(acc[i]);
    }
  }
}

int grid_for(int64_t work_items, int per_sm) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t cap = (int64_t)sms * per_sm;
  return (int)(work_items < 1 ? 1 : (work_items < cap ? work_items : cap));
}

template <typename T>
int launch_sum(const void* in, void* out, int64_t M, int topk, int64_t H, const void* ids,
               int ids_int64, int E, const int32_t* emap, const int32_t* row_index, cudaStream_t st, int64_t out_ld) {
  constexpr int V = 16 / sizeof(T);
  const int64_t total = M * ((H + V - 1) / V);
  const int grid = grid_for((total + 255) / 256, 8);
  const bool aligned = (((uintptr_t)in | (uintptr_t)out) & 15) == 0 && (out_ld * sizeof(T)) % 16 == 0;
  if (ids_int64)
    moe_sum_kernel<T, int64_t><<<grid, 256, 0, st>>>((const T*)in, (T*)out, M, topk, H,
                                                     (const int64_t*)ids, E, emap, row_index, aligned, out_ld);
  else
    moe_sum_kernel<T, int32_t><<<grid, 256, 0, st>>>((const T*)in, (T*)out, M, topk, H,
                                                     (const int32_t*)ids, E, emap, row_index, aligned, out_ld);
  return check_launch("moe_sum");
}

// out[p] = x[sorted_ids[p] / topk] for the occupied slots p < num_post_pad; one warp per row,
// 16-byte copies.  Padding slots and the unused tail are left untouched.
__global__ void gather_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ sorted_ids,
                                   const int32_t* __restrict__ num_post_pad, int64_t numel, int topk,
                                   int64_t rows_cap, int64_t row_vec, uint4* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  const int64_t npp = min((int64_t)num_post_pad[0], rows_cap);
  for (int64_t p = warp; p < npp; p += warps) {
    const int64_t sid = sorted_ids[p];
    if (sid < 0 || sid >= numel) continue;
    const uint4* src = x + (sid / topk) * row_vec;
    uint4* dst = out + p * row_vec;
    int64_t c = lane;
    for (; c + 96 < row_vec; c += 128) {  // four loads in flight
      const uint4 v0 = src[c], v1 = src[c + 32], v2 = src[c + 64], v3 = src[c + 96];
      dst[c] = v0; dst[c + 32] = v1; dst[c + 64] = v2; dst[c + 96] = v3;
    }
    for (; c < row_vec; c += 32) dst[c] = src[c];
  }
}

// Round-half-even of a value already clamped to [-128, 127]; NaN gives 0 (as the reference kernel,
// src/flaggems_vllm/ops/fused_moe.py:973-990).
__device__ __forceinline__ int8_t round_int8_even(float v) {
  if (!(v == v)) v = 0.0f;
  v = fminf(fmaxf(v, -128.0f), 127.0f);
  return (int8_t)__float2int_rn(v);
}

// One warp per row.  KIND as in moe_rowwise_quant.
template <typename T, int KIND>
__global__ void __launch_bounds__(256) rowwise_quant_kernel(const T* __restrict__ x, int64_t rows, int64_t cols,
                                                            const float* __restrict__ scale_in,
                                                            const int32_t* __restrict__ row_ids, int64_t valid_below,
                                                            uint8_t* __restrict__ q, float* __restrict__ scale_out) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  for (int64_t r = warp0; r < rows; r += warps) {
    if (row_ids != nullptr) {
      const int64_t id = row_ids[r];
      if (id < 0 || id >= valid_below) continue;
    }
    const T* src = x + r * cols;
    float scale;
    if constexpr (KIND == 0 || KIND == 1) {
      float amax = 0.0f, nan_term = 0.0f;
      for (int64_t c = lane; c < cols; c += 32) {
        const float v = ToF32<T>::get(src[c]);
        amax = fmaxf(amax, fabsf(v));
        if (!(v == v)) nan_term = v;
      }
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
        nan_term += __shfl_xor_sync(0xFFFFFFFFu, nan_term, off);
      }
      if constexpr (KIND == 0) {
        // the clamp constant takes the rounding of the input dtype (1e-10 is zero in f16)
        const float eps = ToF32<T>::get(from_f32<T>(1e-10f));
        scale = (fmaxf(amax, eps) + nan_term) * (1.0f / 127.0f);
      } else {
        scale = fmaxf(fmaxf(amax, 1e-10f) / kFp8Max, 1.0f / (kFp8Max * 512.0f));
      }
      if (lane == 0) scale_out[r] = scale;
    } else {
      scale = scale_in[0];
    }
    for (int64_t c = lane; c < cols; c += 32) {
      const float v = ToF32<T>::get(src[c]);
      uint8_t o;
      if constexpr (KIND == 0 || KIND == 4) o = (uint8_t)round_int8_even(__fdiv_rn(v, scale));
      else if constexpr (KIND == 3) o = f32_to_fp8e4m3(fminf(fmaxf(v * (1.0f / scale), -kFp8Max), kFp8Max));
      else o = f32_to_fp8e4m3(fminf(fmaxf(v / scale, -kFp8Max), kFp8Max));
      q[r * cols + c] = o;
    }
  }
}

// amax of the rows that count, as the bits of a non-negative float (atomicMax on the bits orders them)
template <typename T>
__global__ void __launch_bounds__(256) tensor_amax_kernel(const T* __restrict__ x, int64_t rows, int64_t cols,
                                                          const int32_t* __restrict__ row_ids, int64_t valid_below,
                                                          unsigned int* __restrict__ amax_bits) {
  const int lane = threadIdx.x & 31;
  const int64_t warp0 = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
  float amax = 0.0f;
  for (int64_t r = warp0; r < rows; r += warps) {
    if (row_ids != nullptr) {
      const int64_t id = row_ids[r];
      if (id < 0 || id >= valid_below) continue;
    }
    for (int64_t c = lane; c < cols; c += 32) amax = fmaxf(amax, fabsf(ToF32<T>::get(x[r * cols + c])));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xFFFFFFFFu, amax, off));
  if (lane == 0 && amax > 0.0f) atomicMax(amax_bits, __float_as_uint(amax));
}
__global__ void amax_to_scale_kernel(float* scale) {  // in place: bits of amax -> max(amax, 1e-10) / 448
  scale[0] = fmaxf(scale[0], 1e-10f) / kFp8Max;
}

// out_t[g][p] = scales_t[g][sorted_ids[p] / topk] for the occupied slots p < num_post_pad
__global__ void gather_scales_kernel(const float* __restrict__ scales_t, int groups, int64_t tokens,
                                     const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ num_post_pad,
                                     int64_t numel, int topk, int64_t rows_cap, float* __restrict__ out_t) {
  const int64_t npp = min((int64_t)num_post_pad[0], rows_cap);
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < npp; p += (int64_t)gridDim.x * blockDim.x) {
    const int64_t sid = sorted_ids[p];
    if (sid < 0 || sid >= numel) continue;
    const int64_t tok = sid / topk;
    for (int g = 0; g < groups; ++g) out_t[(int64_t)g * rows_cap + p] = scales_t[(int64_t)g * tokens + tok];
  }
}

}  // namespace
}  // namespace moe

template <typename T>
static int rowwise_quant_launch(const void* x, int64_t rows, int64_t cols, int kind, const float* scale_in,
                                const int32_t* row_ids, int64_t valid_below, void* q, float* scale_out, cudaStream_t st) {
  using namespace moe;
  const int grid = grid_for((rows + 7) / 8, 8);
#define MOE_RQ(K, SIN) rowwise_quant_kernel<T, K><<<grid, 256, 0, st>>>((const T*)x, rows, cols, SIN, row_ids, valid_below, (uint8_t*)q, scale_out)
  switch (kind) {
    case 0: MOE_RQ(0, nullptr); break;
    case 1: MOE_RQ(1, nullptr); break;
    case 2: MOE_RQ(2, scale_in); break;
    case 4: MOE_RQ(4, scale_in); break;
    case 3: {
      cudaError_t ce = cudaMemsetAsync(scale_out, 0, sizeof(float), st);
      if (ce != cudaSuccess) return fail((int)ce, "rowwise_quant: %s", cudaGetErrorString(ce));
      tensor_amax_kernel<T><<<grid, 256, 0, st>>>((const T*)x, rows, cols, row_ids, valid_below, (unsigned int*)scale_out);
      amax_to_scale_kernel<<<1, 1, 0, st>>>(scale_out);
      MOE_RQ(3, scale_out);
      break;
    }
    default: return fail(MOE_E_BADARG, "rowwise_quant: unknown kind %d", kind);
  }
#undef MOE_RQ
  return check_launch("rowwise_quant");
}

extern "C" int moe_rowwise_quant(const void* x, int x_dtype, int64_t rows, int64_t cols, int kind, const float* scale_in,
                                 const int32_t* row_ids, int64_t valid_below, void* q, float* scale_out, void* stream) {
  using namespace moe;
  if (rows < 0 || cols <= 0) return fail(MOE_E_BADARG, "rowwise_quant: bad extent");
  if (rows == 0) return 0;
  if (!x || !q) return fail(MOE_E_BADARG, "rowwise_quant: null pointer");
  if ((kind == 2 || kind == 4) && !scale_in) return fail(MOE_E_BADARG, "rowwise_quant: static scale missing");
  if ((kind == 0 || kind == 1 || kind == 3) && !scale_out) return fail(MOE_E_BADARG, "rowwise_quant: scale output missing");
  cudaStream_t st = (cudaStream_t)stream;
  if ((kind == 2 || kind == 4) && scale_out && scale_out != scale_in) {
    cudaError_t ce = cudaMemcpyAsync(scale_out, scale_in, sizeof(float), cudaMemcpyDeviceToDevice, st);
    if (ce != cudaSuccess) return fail((int)ce, "rowwise_quant: %s", cudaGetErrorString(ce));
  }
  switch (x_dtype) {
    case MOE_F32: return rowwise_quant_launch<float>(x, rows, cols, kind, scale_in, row_ids, valid_below, q, scale_out, st);
    case MOE_F16: return rowwise_quant_launch<__half>(x, rows, cols, kind, scale_in, row_ids, valid_below, q, scale_out, st);
    case MOE_BF16: return rowwise_quant_launch<__nv_bfloat16>(x, rows, cols, kind, scale_in, row_ids, valid_below, q, scale_out, st);
    default: return fail(MOE_E_DTYPE, "rowwise_quant: unsupported dtype %d", x_dtype);
  }
}

extern "C" int moe_gather_scales_t(const float* scales_t, int groups, int64_t num_tokens, int topk,
                                   const int32_t* sorted_ids, const int32_t* num_post_pad, int64_t rows_cap,
                                   float* out_t, void* stream) {
  using namespace moe;
  if (num_tokens < 0 || topk <= 0 || groups <= 0 || rows_cap < 0) return fail(MOE_E_BADARG, "gather_scales_t: bad extent");
  if (num_tokens == 0 || rows_cap == 0) return 0;
  if (!scales_t || !sorted_ids || !num_post_pad || !out_t) return fail(MOE_E_BADARG, "gather_scales_t: null pointer");
  const int grid = grid_for((rows_cap + 255) / 256, 8);
  gather_scales_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(scales_t, groups, num_tokens, sorted_ids, num_post_pad,
                                                              num_tokens * topk, topk, rows_cap, out_t);
  return check_launch("gather_scales_t");
}

extern "C" int moe_gather_rows(const void* x, int64_t num_tokens, int topk, int64_t row_bytes,
                               const int32_t* sorted_ids, const int32_t* num_post_pad, int64_t rows_cap, void* out,
                               void* stream) {
  using namespace moe;
  if (num_tokens < 0 || topk <= 0 || row_bytes <= 0 || rows_cap < 0) return fail(MOE_E_BADARG, "gather_rows: bad extent");
  if (num_tokens == 0 || rows_cap == 0) return 0;
  if (!x || !sorted_ids || !num_post_pad || !out) return fail(MOE_E_BADARG, "gather_rows: null pointer");
  if (row_bytes % 16 != 0 || ((uintptr_t)x & 15) || ((uintptr_t)out & 15))
    return fail(MOE_E_SHAPE, "gather_rows: row size and pointers must be multiples of 16 bytes");
  const int grid = grid_for((rows_cap + 7) / 8, 16);
  gather_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>((const uint4*)x, sorted_ids, num_post_pad,
                                                            num_tokens * topk, topk, rows_cap, row_bytes / 16,
                                                            (uint4*)out);
  return check_launch("gather_rows");
}

extern "C" int moe_per_token_group_quant_fp8_ex(const void* x, int x_dtype, int64_t rows, int64_t cols, int group,
                                                float eps, int e5m2, void* q, float* scales, int scales_transposed,
                                                int64_t scale_ld, void* stream) {
  using namespace moe;
  if (rows < 0 || cols <= 0 || group <= 0) return fail(MOE_E_BADARG, "quant_fp8: bad extent");
  if (cols % group != 0) return fail(MOE_E_SHAPE, "quant_fp8: cols must be a multiple of the group size %d", group);
  if (!(eps >= 0.0f)) return fail(MOE_E_BADARG, "quant_fp8: eps must be non-negative");
  if (rows == 0) return 0;
  if (!x || !q || !scales) return fail(MOE_E_BADARG, "quant_fp8: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for((rows * (cols / group) + 7) / 8, 8);
  const int transposed = scales_transposed & 1;
  const bool ue8m0 = (scales_transposed & 2) != 0;
#define MOE_QG(T, U, F) quant_rows_generic_kernel<T, U, F><<<grid, kRowThreads, 0, st>>>((const T*)x, rows, cols, group, eps, (uint8_t*)q, scales, transposed, scale_ld)
#define MOE_QG_T(T) (ue8m0 ? (e5m2 ? MOE_QG(T, true, true) : MOE_QG(T, true, false)) : (e5m2 ? MOE_QG(T, false, true) : MOE_QG(T, false, false)))
  switch (x_dtype) {
    case MOE_F32: MOE_QG_T(float); break;
    case MOE_F16: MOE_QG_T(__half); break;
    case MOE_BF16: MOE_QG_T(__nv_bfloat16); break;
    default: return fail(MOE_E_DTYPE, "quant_fp8: unsupported dtype %d", x_dtype);
  }
#undef MOE_QG_T
#undef MOE_QG
  return check_launch("per_token_group_quant_fp8");
}

extern "C" int moe_per_token_group_quant_fp8(const void* x, int x_dtype, int64_t rows, int64_t cols,
                                             int group, void* q, float* scales,
                                             int scales_transposed, int64_t scale_ld, void* stream) {
  using namespace moe;
  if (rows < 0 || cols <= 0) return fail(MOE_E_BADARG, "quant_fp8: bad extent");
  if (group != 128)  // other group sizes: the general kernel with the default clamp
    return moe_per_token_group_quant_fp8_ex(x, x_dtype, rows, cols, group, kQuantEps, 0, q, scales, scales_transposed,
                                            scale_ld, stream);
  if (cols % 128 != 0) return fail(MOE_E_SHAPE, "quant_fp8: cols must be a multiple of 128");
  if (rows == 0) return 0;
  if (!x || !q || !scales) return fail(MOE_E_BADARG, "quant_fp8: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  const int grid = grid_for((rows * (cols / 128) + 7) / 8, 8);
  const int transposed = scales_transposed & 1;
  const bool ue8m0 = (scales_transposed & 2) != 0;
#define MOE_QUANT_LAUNCH(T)                                                                                        \
  (ue8m0 ? quant_rows_kernel<T, true><<<grid, kRowThreads, 0, st>>>((const T*)x, rows, cols, (uint8_t*)q, scales,  \
                                                                    transposed, scale_ld)                          \
         : quant_rows_kernel<T, false><<<grid, kRowThreads, 0, st>>>((const T*)x, rows, cols, (uint8_t*)q, scales, \
                                                                     transposed, scale_ld))
  const bool pairs = !ue8m0 && (cols / 128) % 2 == 0 && (x_dtype == MOE_F16 || x_dtype == MOE_BF16) &&
                     (((uintptr_t)x | (uintptr_t)q) & 15) == 0;
  if (pairs) {
    const int grid2 = grid_for((rows * (cols / 256) + 7) / 8, 8);
    if (x_dtype == MOE_BF16)
      quant_rows_pair_kernel<__nv_bfloat16><<<grid2, kRowThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, (uint8_t*)q,
                                                                           scales, transposed, scale_ld);
    else
      quant_rows_pair_kernel<__half><<<grid2, kRowThreads, 0, st>>>((const __half*)x, rows, cols, (uint8_t*)q, scales,
                                                                    transposed, scale_ld);
    return check_launch("per_token_group_quant_fp8");
  }
  switch (x_dtype) {
    case MOE_F32: MOE_QUANT_LAUNCH(float); break;
    case MOE_F16: MOE_QUANT_LAUNCH(__half); break;
    case MOE_BF16: MOE_QUANT_LAUNCH(__nv_bfloat16); break;
    default: return fail(MOE_E_DTYPE, "quant_fp8: unsupported dtype %d", x_dtype);
  }
#undef MOE_QUANT_LAUNCH
  return check_launch("per_token_group_quant_fp8");
}

extern "C" int moe_widen_int8(const void* src, void* dst, int dst_dtype, int64_t n, void* stream) {
  using namespace moe;
  if (n < 0) return fail(MOE_E_BADARG, "widen_int8: negative size");
  if (n == 0) return 0;
  if (!src || !dst) return fail(MOE_E_BADARG, "widen_int8: null pointer");
  if (n % 16 != 0 || ((uintptr_t)src & 15) || ((uintptr_t)dst & 15))
    return fail(MOE_E_SHAPE, "widen_int8: size and pointers must be multiples of 16");
  cudaStream_t st = (cudaStream_t)stream;
  const int64_t n16 = n / 16;
  const int grid = grid_for((n16 + 255) / 256, 16);
  if (dst_dtype == MOE_BF16)
    widen_int8_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const int8_t*)src, (__nv_bfloat16*)dst, n16);
  else if (dst_dtype == MOE_F16)
    widen_int8_kernel<__half><<<grid, 256, 0, st>>>((const int8_t*)src, (__half*)dst, n16);
  else
    return fail(MOE_E_DTYPE, "widen_int8: destination must be f16 or bf16");
  return check_launch("widen_int8");
}

extern "C" int moe_sum_ld(const void* in, void* out, int64_t out_ld, int dtype, int64_t M, int topk, int64_t H,
                          const void* topk_ids, int ids_int64, int num_experts, const int32_t* expert_map,
                          const int32_t* row_index, void* stream) {
  using namespace moe;
  if (M < 0 || topk <= 0 || H <= 0 || out_ld < H) return fail(MOE_E_BADARG, "moe_sum: bad extent");
  if (M == 0) return 0;
  if (!in || !out) return fail(MOE_E_BADARG, "moe_sum: null pointer");
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case MOE_F32: return launch_sum<float>(in, out, M, topk, H, topk_ids, ids_int64, num_experts, expert_map, row_index, st, out_ld);
    case MOE_F16: return launch_sum<__half>(in, out, M, topk, H, topk_ids, ids_int64, num_experts, expert_map, row_index, st, out_ld);
    case MOE_BF16: return launch_sum<__nv_bfloat16>(in, out, M, topk, H, topk_ids, ids_int64, num_experts, expert_map, row_index, st, out_ld);
    default: return fail(MOE_E_DTYPE, "moe_sum: unsupported dtype %d", dtype);
  }
}

extern "C" int moe_sum(const void* in, void* out, int dtype, int64_t M, int topk, int64_t H,
                       const void* topk_ids, int ids_int64, int num_experts,
                       const int32_t* expert_map, const int32_t* row_index, void* stream) {
  return moe_sum_ld(in, out, H, dtype, M, topk, H, topk_ids, ids_int64, num_experts, expert_map, row_index, stream);
}


// ---------------------------------------------------------------------------------------------
// Stand-alone SiLU(a) * b and its gradients: the reference's silu_and_mul / silu_and_mul_out
// (src/flaggems_vllm/ops/silu_and_mul.py:26-70), which its fused_experts_impl uses on the
// un-fused GEMM1 path.  fp32 arithmetic as there: a / (1 + exp(-a)) * b, one rounding to the
// output dtype.  The layer of this library never calls it (the activation is fused into GEMM1).
namespace moe {
namespace {
template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                           T* __restrict__ out, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float x = ToF32<T>::get(a[i]), y = ToF32<T>::get(b[i]);
    out[i] = from_f32<T>((x / (1.0f + expf(-x))) * y);
  }
}
template <typename T>
__global__ void __launch_bounds__(256) silu_and_mul_grad_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                                const T* __restrict__ dgrad, T* __restrict__ da,
                                                                T* __restrict__ db, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float x = ToF32<T>::get(a[i]), y = ToF32<T>::get(b[i]), g = ToF32<T>::get(dgrad[i]);
    const float sig = 1.0f / (1.0f + expf(-x));
    da[i] = from_f32<T>(sig * (1.0f + x * (1.0f - sig)) * g * y);
    db[i] = from_f32<T>(g * (x * sig));
  }
}
}  // namespace
}  // namespace moe

extern "C" int moe_silu_and_mul(const void* a, const void* b, void* out, int dtype, int64_t n, void* stream) {
  using namespace moe;
  if (n < 0) return fail(MOE_E_BADARG, "silu_and_mul: negative size");
  if (n == 0) return 0;
  if (!a || !b || !out) return fail(MOE_E_BADARG, "silu_and_mul: null pointer");
  const int grid = grid_for((n + 255) / 256, 16);
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case MOE_F32: silu_and_mul_kernel<float><<<grid, 256, 0, st>>>((const float*)a, (const float*)b, (float*)out, n); break;
    case MOE_F16: silu_and_mul_kernel<__half><<<grid, 256, 0, st>>>((const __half*)a, (const __half*)b, (__half*)out, n); break;
    case MOE_BF16:
      silu_and_mul_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                               (__nv_bfloat16*)out, n);
      break;
    default: return fail(MOE_E_DTYPE, "silu_and_mul: unsupported dtype %d", dtype);
  }
  return check_launch("silu_and_mul");
}

extern "C" int moe_silu_and_mul_grad(const void* a, const void* b, const void* dgrad, void* da, void* db, int dtype,
                                     int64_t n, void* stream) {
  using namespace moe;
  if (n < 0) return fail(MOE_E_BADARG, "silu_and_mul_grad: negative size");
  if (n == 0) return 0;
  if (!a || !b || !dgrad || !da || !db) return fail(MOE_E_BADARG, "silu_and_mul_grad: null pointer");
  const int grid = grid_for((n + 255) / 256, 16);
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case MOE_F32:
      silu_and_mul_grad_kernel<float><<<grid, 256, 0, st>>>((const float*)a, (const float*)b, (const float*)dgrad, (float*)da,
                                                            (float*)db, n);
      break;
    case MOE_F16:
      silu_and_mul_grad_kernel<__half><<<grid, 256, 0, st>>>((const __half*)a, (const __half*)b, (const __half*)dgrad,
                                                             (__half*)da, (__half*)db, n);
      break;
    case MOE_BF16:
      silu_and_mul_grad_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                    (const __nv_bfloat16*)dgrad, (__nv_bfloat16*)da,
                                                                    (__nv_bfloat16*)db, n);
      break;
    default: return fail(MOE_E_DTYPE, "silu_and_mul_grad: unsupported dtype %d", dtype);
  }
  return check_launch("silu_and_mul_grad");
}
