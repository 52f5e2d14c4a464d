// Shared helpers of the sm_100a kernels: error codes, dtype conversion, reductions.
//
// Every launcher is an extern "C" function on raw device pointers that returns
// 0 on success, a negative SI_ERR_* code when it refuses its arguments (it then
// launches nothing) or the positive cudaError_t of a failed launch.  Kernels
// run on the stream the caller passes, so a caller may capture them in a CUDA
// graph.  The reference has no native code; its Triton kernels live under
// kernels/*.py and are cited next to each kernel here.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define SI_API extern "C" __attribute__((visibility("default")))

enum SiError {
  SI_OK = 0,
  SI_ERR_ARG = -1,          // null pointer, negative size, misaligned pointer
  SI_ERR_UNSUPPORTED = -2,  // a size this build of the kernel does not take
  SI_ERR_DTYPE = -3,        // dtype code not known to the kernel
  SI_ERR_TOO_LARGE = -4,    // exceeds a stated maximum (shared memory, scratch)
};

// dtype codes shared with the Python side
enum SiDtype { SI_F32 = 0, SI_BF16 = 1 };

#define SI_LAUNCH_CHECK()                         \
  do {                                            \
    cudaError_t e__ = cudaGetLastError();         \
    if (e__ != cudaSuccess) return (int)e__;      \
  } while (0)

namespace si {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
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

// Block-wide sum, same value in every thread.  `scratch` holds 32 floats.
// The order of additions depends only on blockDim, never on the data's place
// in a batch.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from a previous call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.0f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

}  // namespace si
