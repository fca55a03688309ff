// layered_common.cuh — device helpers shared by the kernels of the layered architectures
// (layered_ops.cu, sequence_ops.cu): typed loads / stores over the model's element type, block
// reductions with a fixed summation order, and the dtype dispatch of the entry points.
#pragma once
#include "common.cuh"

namespace b200q {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// sum over the block (blockDim.x a multiple of 32, <= 1024); red: >= 32 floats of shared memory.
// Every thread adds the warp partials in the same order, so all threads hold the same bits.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = 0.f;
  for (int i = 0; i < nw; ++i) t += red[i];
  return t;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float siluf_(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }

static inline int grid_for(long long total, int block = 256) {
  long long g = (total + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148 * 16 ? 148 * 16 : g));
}
static inline bool is_dtype(int d) { return d == B200Q_DTYPE_BF16 || d == B200Q_DTYPE_F32; }

}  // namespace b200q

#define DISPATCH_T(dtype, ...)                   \
  do {                                           \
    if ((dtype) == B200Q_DTYPE_F32) {            \
      using T = float;                           \
      __VA_ARGS__;                               \
    } else {                                     \
      using T = bf16;                            \
      __VA_ARGS__;                               \
    }                                            \
  } while (0)
