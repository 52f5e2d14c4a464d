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
#include <stdlib.h>

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

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Kernels are launched with the "programmatic
// stream serialization" attribute.  pdl_wait() blocks until every earlier
// kernel of the stream has finished and its writes are visible: a kernel calls
// it before it reads or writes anything another kernel touches (weights are
// never written, so a product may request its first weights before waiting).
// pdl_trigger() lets the next kernel of the stream be scheduled once all blocks
// of this one have passed it.  The products call it when their main loop is done, so
// that the successor's launch and prologue overlap their tail and the blocks of their
// last wave are not kept off the SMs by parked successors; short kernels (norms, RoPE,
// the join of attention splits) call it at once, and so does decode attention, whose
// blocks leave room for the output projection to come in and fetch its first weights.
// Whatever a kernel needs that no kernel of the step writes (weights, the step's batch
// description, keys of earlier positions) it fetches BEFORE pdl_wait().  A captured CUDA
// graph keeps these edges.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_trigger() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch helper: returns the launch error instead of leaving it for later.
template <typename Kernel, typename... Args>
static inline cudaError_t launch(Kernel kernel, dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

#define SI_LAUNCH(kernel, grid, block, smem, stream, ...)                                  \
  do {                                                                                     \
    cudaError_t le__ = si::launch(kernel, dim3(grid), dim3(block), smem, stream, __VA_ARGS__); \
    if (le__ != cudaSuccess) return (int)le__;                                             \
  } while (0)

// Raise a kernel's dynamic shared memory limit, once per call site and device (the attribute
// belongs to the device's copy of the kernel, so a second GPU needs its own call).
#define SI_ALLOW_DYNAMIC_SMEM(kernel, bytes)                                                  \
  do {                                                                                        \
    static bool done__[64];                                                                   \
    int dev__ = 0;                                                                            \
    cudaError_t ae__ = cudaGetDevice(&dev__);                                                 \
    if (ae__ != cudaSuccess) return (int)ae__;                                                \
    if (dev__ < 0 || dev__ >= 64) return SI_ERR_TOO_LARGE;                                    \
    if (!done__[dev__]) {                                                                     \
      ae__ = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                  (int)(bytes));                                              \
      if (ae__ != cudaSuccess) return (int)ae__;                                              \
      done__[dev__] = true;                                                                   \
    }                                                                                         \
  } while (0)

// 8 consecutive elements as float, for 16-byte (bfloat16) or 32-byte (float32) vector access
template <typename T> __device__ __forceinline__ void load8(const T* p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
template <typename T> __device__ __forceinline__ void store8(T* p, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float* p, const float (&v)[8]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
template <> __device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[8]) {
  uint4 raw;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = raw;
}

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
