// Helpers shared by the kernels of the hybrid decoder families (latent attention, state-space and matrix-memory mixers):
// element types bfloat16 / float behind one template parameter, block reductions, the exact transcendental forms.
// Everything these kernels accumulate, normalise or carry from token to token is fp32; the element type only says how
// activations, weights and cache pages are stored.
#pragma once
#include "common.cuh"

#include <cuda_bf16.h>

#define B200_DT_BF16 0
#define B200_DT_F32 1

namespace b200 {
namespace seq {

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <typename T>
__device__ __forceinline__ void stf(T* p, float v);
template <>
__device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void stf<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// element of a buffer whose type is only known at run time (dt = B200_DT_*)
__device__ __forceinline__ float ld_any(const void* p, int64_t i, int dt) {
  return dt == B200_DT_F32 ? reinterpret_cast<const float*>(p)[i] : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void st_any(void* p, int64_t i, int dt, float v) {
  if (dt == B200_DT_F32) reinterpret_cast<float*>(p)[i] = v;
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// sum over a block of up to 1024 threads; `red` is 32 floats of shared memory; every thread gets the total
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();
  if (lane_id() == 0) red[warp_id()] = v;
  __syncthreads();
  float t = lane_id() < (int)((blockDim.x + 31) / 32) ? red[lane_id()] : 0.f;
  return warp_sum(t);
}

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float logsigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

__device__ __forceinline__ void mma_m16n8k16_bf16f32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

}  // namespace seq
}  // namespace b200

#define B200_SEQ_DISPATCH(dt, T, ...)                                  \
  do {                                                                  \
    if ((dt) == B200_DT_F32) { using T = float; __VA_ARGS__; }          \
    else if ((dt) == B200_DT_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else { b200_set_last_error("unknown element type"); return B200_ERR_ARG; } \
  } while (0)
