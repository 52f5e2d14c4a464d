// Row-wise kernels: embedding gather, RMSNorm with the residual add fused in,
// and the SwiGLU gate.  All arithmetic is float32; one rounding at the store.
//
//   embedding   x0[t] = E[id[t]]                       reference ops/embedding.py:57-60
//   RMSNorm     y = x * rsqrt(mean(x^2) + eps) * w     reference ops/rmsnorm.py:41-46,
//                                                       kernels/rmsnorm_kernel.py:105-113
//   residual    x = x + h (fused into the norm)        reference model/block.py:138,144
//   SwiGLU      h = silu(g) * u, silu(g) = g*sigmoid(g) reference ops/mlp.py:117-125,
//                                                       kernels/swiglu_kernel.py:142-150
#include "common.cuh"

namespace si {

// ---------------------------------------------------------------- embedding
template <typename T>
__global__ void embed_gather_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                    float* __restrict__ out, int hidden, int vocab) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int id = ids[t];
  float* dst = out + (size_t)t * hidden;
  if (id < 0 || id >= vocab) {
    // The host checks ids before a step; a bad id must still not read outside
    // the table.  NaN makes the fault visible in the logits.
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = __int_as_float(0x7fc00000);
    return;
  }
  const T* src = table + (size_t)id * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = to_f32<T>(src[i]);
}

// ------------------------------------------------------------------ RMSNorm
// One block per output row r.  Source row = rows ? rows[r] : r.
//   x = residual[src] (+ delta[src]);  if (!rows && delta) residual[src] = x;
//   out[r] = x * rsqrt(sum(x^2)/H + eps) * w
// The row is kept in shared memory between the two passes.
// The pending addend of a row comes either as one row of `delta` (dtype TA) or as `n_parts`
// float32 slices `parts[p][row]` (partial sums of a product whose k-range was cut across
// blocks): the slices are added in order and the sum rounded to TA, which is what the product
// would have stored had it not been cut.
struct DeltaParts {
  const float* parts;
  int n_parts;
  long long stride;  // elements between slices
};

constexpr int MAX_DELTA_PARTS = 8;

template <typename TA>
__device__ __forceinline__ void sum_parts8(const DeltaParts& dp, size_t at, float (&d)[8]) {
  // all slices are requested before the first is added (one round trip, not one per slice)
  float v[MAX_DELTA_PARTS][8];
#pragma unroll
  for (int p = 0; p < MAX_DELTA_PARTS; ++p) {
    if (p < dp.n_parts) {
      load8<float>(dp.parts + (size_t)p * dp.stride + at, v[p]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[p][j] = 0.0f;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) d[j] = v[0][j];
#pragma unroll
  for (int p = 1; p < MAX_DELTA_PARTS; ++p)
#pragma unroll
    for (int j = 0; j < 8; ++j) d[j] += v[p][j];
#pragma unroll
  for (int j = 0; j < 8; ++j) d[j] = to_f32<TA>(from_f32<TA>(d[j]));
}

template <typename TA, typename TW, bool VEC>
__global__ void rmsnorm_kernel(float* __restrict__ residual, const TA* __restrict__ delta,
                               DeltaParts dp, const TW* __restrict__ weight,
                               const int* __restrict__ rows, TA* __restrict__ out, int hidden,
                               float eps) {
  extern __shared__ float srow[];
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();  // a short kernel: let the product that follows fetch its weights meanwhile
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  const TA* del = delta ? delta + (size_t)src * hidden : nullptr;
  const bool adds = delta != nullptr || dp.n_parts > 0;
  const bool write_back = (rows == nullptr) && adds;
  TA* dst = out + (size_t)r * hidden;
  float ss = 0.0f;
  if (VEC) {  // hidden is a multiple of 8: 8 elements per thread and step
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
      float x[8];
      load8<float>(res + i, x);
      if (adds) {
        float d[8];
        if (del) load8<TA>(del + i, d);
        else sum_parts8<TA>(dp, (size_t)src * hidden + i, d);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] += d[j];
        if (write_back) store8<float>(res + i, x);
      }
      store8<float>(srow + i, x);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float x = res[i];
      if (adds) {
        if (del) {
          x += to_f32<TA>(del[i]);
        } else {
          float d = 0.0f;
          for (int p = 0; p < dp.n_parts; ++p) d += dp.parts[(size_t)p * dp.stride + (size_t)src * hidden + i];
          x += to_f32<TA>(from_f32<TA>(d));
        }
        if (write_back) res[i] = x;
      }
      srow[i] = x;
      ss += x * x;
    }
  }
  const float total = block_sum(ss, red);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (VEC) {
    for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
      float x[8], w[8];
      load8<float>(srow + i, x);
      load8<TW>(weight + i, w);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = (x[j] * rstd) * w[j];
      store8<TA>(dst + i, x);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      dst[i] = from_f32<TA>((srow[i] * rstd) * to_f32<TW>(weight[i]));
  }
}

// The same for rows that fit the block at 8 elements a thread (hidden a multiple of 8, at most
// 8 * blockDim.x): the row stays in registers between the two passes, and the gain is loaded
// before the sum is known, so a block has one round trip to memory instead of two.
template <typename TA, typename TW>
__global__ void rmsnorm_row_in_registers_kernel(float* __restrict__ residual, const TA* __restrict__ delta,
                                                DeltaParts dp, const TW* __restrict__ weight,
                                                const int* __restrict__ rows, TA* __restrict__ out,
                                                int hidden, float eps) {
  __shared__ float red[32];
  const int i = threadIdx.x * 8;
  const bool mine = i < hidden;
  float w[8];
  if (mine) load8<TW>(weight + i, w);  // the gain is not written by any kernel: fetch it before waiting
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (size_t)src * hidden;
  float x[8];
  float ss = 0.0f;
  if (mine) {
    load8<float>(res + i, x);
    if (delta || dp.n_parts > 0) {
      float d[8];
      if (delta) load8<TA>(delta + (size_t)src * hidden + i, d);
      else sum_parts8<TA>(dp, (size_t)src * hidden + i, d);
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] += d[j];
      if (rows == nullptr) store8<float>(res + i, x);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
  }
  const float total = block_sum(ss, red);
  const float rstd = rsqrtf(total / (float)hidden + eps);
  if (mine) {
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = (x[j] * rstd) * w[j];
    store8<TA>(out + (size_t)r * hidden + i, x);
  }
}

// ------------------------------------------------------------------- SwiGLU
// gu is [rows, 2*inter]: gate in columns [0, inter), up in [inter, 2*inter).
template <typename T, bool VEC>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total,
                              int inter) {
  constexpr int W = VEC ? 8 : 1;  // inter is a multiple of 8 when VEC
  pdl_wait();
  pdl_trigger();
  for (long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * W; idx < total;
       idx += (long long)gridDim.x * blockDim.x * W) {
    const long long row = idx / inter;
    const int col = (int)(idx - row * inter);
    const T* gp = gu + row * 2 * inter + col;
    if (VEC) {
      float g[8], u[8];
      load8<T>(gp, g);
      load8<T>(gp + inter, u);
#pragma unroll
      for (int j = 0; j < 8; ++j) g[j] = (g[j] / (1.0f + expf(-g[j]))) * u[j];
      store8<T>(out + idx, g);
    } else {
      const float g = to_f32<T>(gp[0]);
      const float u = to_f32<T>(gp[inter]);
      out[idx] = from_f32<T>((g / (1.0f + expf(-g))) * u);
    }
  }
}

}  // namespace si

SI_API int si_embed_gather(const void* table, int table_dtype, const int* ids, float* out,
                           int n_tokens, int hidden, int vocab, cudaStream_t stream) {
  if (!table || !ids || !out || n_tokens < 0 || hidden <= 0 || vocab <= 0) return SI_ERR_ARG;
  if (n_tokens == 0) return SI_OK;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == SI_F32)
    SI_LAUNCH(si::embed_gather_kernel<float>, n_tokens, threads, 0, stream, (const float*)table,
              ids, out, hidden, vocab);
  else if (table_dtype == SI_BF16)
    SI_LAUNCH(si::embed_gather_kernel<__nv_bfloat16>, n_tokens, threads, 0, stream,
              (const __nv_bfloat16*)table, ids, out, hidden, vocab);
  else
    return SI_ERR_DTYPE;
  return SI_OK;
}

template <typename TA, typename TW>
static int launch_rmsnorm(float* residual, const void* delta, si::DeltaParts dp, const void* weight,
                          const int* rows, void* out, int n_rows, int hidden, float eps,
                          cudaStream_t stream) {
  const size_t smem = (size_t)hidden * sizeof(float);
  if (smem > 200 * 1024) return SI_ERR_TOO_LARGE;
  const bool vec = hidden % 8 == 0 &&
                   ((((uintptr_t)residual | (uintptr_t)delta | (uintptr_t)weight | (uintptr_t)out |
                      (uintptr_t)dp.parts) & 15) == 0) && dp.stride % 4 == 0;
  auto kern = vec ? si::rmsnorm_kernel<TA, TW, true> : si::rmsnorm_kernel<TA, TW, false>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int per_thread = vec ? 8 : 1;
  int threads = (hidden / per_thread + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  if (threads < 64) threads = 64;
  if (vec && hidden <= threads * 8) {
    SI_LAUNCH((si::rmsnorm_row_in_registers_kernel<TA, TW>), n_rows, threads, 0, stream, residual,
              (const TA*)delta, dp, (const TW*)weight, rows, (TA*)out, hidden, eps);
    return SI_OK;
  }
  SI_LAUNCH(kern, n_rows, threads, smem, stream, residual, (const TA*)delta, dp, (const TW*)weight,
            rows, (TA*)out, hidden, eps);
  return SI_OK;
}

// act_dtype: dtype of delta and out.  weight_dtype: dtype of the gain.
// The addend is `delta` (one row per residual row) or, when delta is null and n_parts > 0,
// the sum of the float32 slices parts[p] (p < n_parts, part_stride elements apart, each laid
// out like delta), added in order and rounded to act_dtype.
SI_API int si_rmsnorm(float* residual, const void* delta, const float* parts, int n_parts,
                      long long part_stride, const void* weight, const int* rows,
                      void* out, int n_rows, int hidden, float eps, int act_dtype,
                      int weight_dtype, cudaStream_t stream) {
  if (!residual || !weight || !out || n_rows < 0 || hidden <= 0 || !(eps > 0.0f)) return SI_ERR_ARG;
  if (n_parts < 0 || (n_parts > 0 && (!parts || delta || part_stride < 0))) return SI_ERR_ARG;
  if (n_parts > si::MAX_DELTA_PARTS) return SI_ERR_TOO_LARGE;
  if (n_rows == 0) return SI_OK;
  si::DeltaParts dp;
  dp.parts = n_parts > 0 ? parts : nullptr;
  dp.n_parts = n_parts;
  dp.stride = part_stride;
  if (act_dtype == SI_F32 && weight_dtype == SI_F32)
    return launch_rmsnorm<float, float>(residual, delta, dp, weight, rows, out, n_rows, hidden, eps, stream);
  if (act_dtype == SI_BF16 && weight_dtype == SI_F32)
    return launch_rmsnorm<__nv_bfloat16, float>(residual, delta, dp, weight, rows, out, n_rows, hidden, eps, stream);
  if (act_dtype == SI_BF16 && weight_dtype == SI_BF16)
    return launch_rmsnorm<__nv_bfloat16, __nv_bfloat16>(residual, delta, dp, weight, rows, out, n_rows, hidden, eps, stream);
  if (act_dtype == SI_F32 && weight_dtype == SI_BF16)
    return launch_rmsnorm<float, __nv_bfloat16>(residual, delta, dp, weight, rows, out, n_rows, hidden, eps, stream);
  return SI_ERR_DTYPE;
}

SI_API int si_swiglu(const void* gu, void* out, int n_rows, int inter, int dtype,
                     cudaStream_t stream) {
  if (!gu || !out || n_rows < 0 || inter <= 0) return SI_ERR_ARG;
  if (n_rows == 0) return SI_OK;
  const long long total = (long long)n_rows * inter;
  const bool vec = inter % 8 == 0 && ((((uintptr_t)gu | (uintptr_t)out) & 31) == 0);
  const int threads = 256;
  long long blocks = (total / (vec ? 8 : 1) + threads - 1) / threads;
  if (blocks > 148LL * 16) blocks = 148LL * 16;
  if (blocks < 1) blocks = 1;
  if (dtype == SI_F32) {
    if (vec)
      SI_LAUNCH((si::swiglu_kernel<float, true>), (int)blocks, threads, 0, stream, (const float*)gu, (float*)out, total, inter);
    else
      SI_LAUNCH((si::swiglu_kernel<float, false>), (int)blocks, threads, 0, stream, (const float*)gu, (float*)out, total, inter);
  } else if (dtype == SI_BF16) {
    if (vec)
      SI_LAUNCH((si::swiglu_kernel<__nv_bfloat16, true>), (int)blocks, threads, 0, stream,
                (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, inter);
    else
      SI_LAUNCH((si::swiglu_kernel<__nv_bfloat16, false>), (int)blocks, threads, 0, stream,
                (const __nv_bfloat16*)gu, (__nv_bfloat16*)out, total, inter);
  } else {
    return SI_ERR_DTYPE;
  }
  return SI_OK;
}
