// Shared device/host helpers for the rte_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "rte_b200.h"

#define RTE_CHECK_ARG(cond) \
  do {                      \
    if (!(cond)) return RTE_ERR_BAD_ARG; \
  } while (0)

#define RTE_LAUNCH_CHECK()                                   \
  do {                                                       \
    cudaError_t e__ = cudaPeekAtLastError();                 \
    if (e__ != cudaSuccess) return RTE_ERR_LAUNCH;           \
  } while (0)

// Device status codes written to the caller's status word.
enum : int {
  RTE_DEV_WAIT_TIMEOUT_PRODUCER = 101,
  RTE_DEV_WAIT_TIMEOUT_MMA = 102,
  RTE_DEV_WAIT_TIMEOUT_EPILOGUE = 103,
  RTE_DEV_WAIT_TIMEOUT_PEER = 104,
  RTE_DEV_INDEX_OUT_OF_RANGE = 201,
  RTE_DEV_CAPACITY_OVERFLOW = 202
};

namespace rte {

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
__host__ __device__ inline long long ceil_div64(long long a, long long b) { return (a + b - 1) / b; }

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

// Block-wide sum; `red` is shared scratch of >= 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? red[lane] : 0.f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarp) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.f + __expf(-g)); }
__device__ __forceinline__ float sigmoid_f(float g) { return 1.f / (1.f + __expf(-g)); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ float bf16_to_f(const __nv_bfloat16* p) { return __bfloat162float(*p); }

}  // namespace rte
