// Rotary position encoding fused with the write of keys and values into pages.
//
// Input is the fused projection output qkv [tokens, (Hq + 2*Hkv) * D] with the
// query heads first, then the key heads, then the value heads.  For every
// token at absolute position p and every pair (x_i, x_{i+D/2}), i < D/2:
//     angle = float(p) * inv_freq[i]              (float32 product)
//     a' = a*cos(angle) - b*sin(angle),  b' = b*cos(angle) + a*sin(angle)
// which is the split-half (NEOX) rotation q*cos + rotate_half(q)*sin of the
// reference (ops/rope.py:167-215; kernels/rope_kernel.py:143-150), with the
// angle formed as the reference's table does (ops/rope.py:108-110).  Unlike the
// reference's serving paths (serving/prefill.py:123-132), cos and sin are not
// rounded to the model dtype: angles, cos, sin and the products are float32 and
// the result is rounded once.
// Queries are rotated in place; rotated keys and the values go straight to
// their page (reference: serving/paged_kv_cache.py:171-182, 272-283 write the
// pages in separate copies): slot s = page * page_size + offset,
// pool[page][0=K|1=V][kv_head][offset][d].
#include "common.cuh"

namespace si {

template <typename T>
__global__ void rope_kv_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                     const float* __restrict__ inv_freq,
                                     const int* __restrict__ kv_slots, T* __restrict__ pool,
                                     int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                                     int write_kv) {
  extern __shared__ float cs[];  // cos[half], sin[half]
  pdl_trigger();
  // positions, frequencies and slots were on the device before the step's first kernel: the
  // angles are worked out while the projection before this kernel is still finishing
  const int t = blockIdx.x;
  const int half = head_dim >> 1;
  float* s_cos = cs;
  float* s_sin = cs + half;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float angle = pos * inv_freq[i];
    float s, c;
    sincosf(angle, &s, &c);
    s_cos[i] = c;
    s_sin[i] = s;
  }
  const int slot = write_kv ? kv_slots[t] : 0;
  pdl_wait();
  __syncthreads();

  const int row_width = (n_q_heads + 2 * n_kv_heads) * head_dim;
  T* row = qkv + (size_t)t * row_width;
  // head_dim is a multiple of 16, so a half is a multiple of 8: a thread rotates 8 pairs
  const int groups = half / 8;

  // queries: rotate in place
  for (int w = threadIdx.x; w < n_q_heads * groups; w += blockDim.x) {
    const int h = w / groups, i = (w - h * groups) * 8;
    T* p = row + h * head_dim + i;
    float a[8], b[8], ra[8], rb[8];
    load8<T>(p, a);
    load8<T>(p + half, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = s_cos[i + j], s = s_sin[i + j];
      ra[j] = a[j] * c - b[j] * s;
      rb[j] = b[j] * c + a[j] * s;
    }
    store8<T>(p, ra);
    store8<T>(p + half, rb);
  }
  if (!write_kv) return;

  const int page = slot / page_size, off = slot - page * page_size;
  const size_t head_stride = (size_t)page_size * head_dim;
  T* kpage = pool + ((size_t)page * 2 + 0) * n_kv_heads * head_stride + (size_t)off * head_dim;
  T* vpage = pool + ((size_t)page * 2 + 1) * n_kv_heads * head_stride + (size_t)off * head_dim;
  const T* krow = row + n_q_heads * head_dim;
  const T* vrow = krow + n_kv_heads * head_dim;

  for (int w = threadIdx.x; w < n_kv_heads * groups; w += blockDim.x) {
    const int h = w / groups, i = (w - h * groups) * 8;
    const T* p = krow + h * head_dim + i;
    float a[8], b[8], ra[8], rb[8];
    load8<T>(p, a);
    load8<T>(p + half, b);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c = s_cos[i + j], s = s_sin[i + j];
      ra[j] = a[j] * c - b[j] * s;
      rb[j] = b[j] * c + a[j] * s;
    }
    T* dst = kpage + h * head_stride + i;
    store8<T>(dst, ra);
    store8<T>(dst + half, rb);
  }
  const int v_groups = head_dim / 8;
  for (int w = threadIdx.x; w < n_kv_heads * v_groups; w += blockDim.x) {
    const int h = w / v_groups, d = (w - h * v_groups) * 8;
    float v[8];
    load8<T>(vrow + h * head_dim + d, v);
    store8<T>(vpage + h * head_stride + d, v);
  }
}

}  // namespace si

SI_API int si_rope_kv_store(void* qkv, const int* positions, const float* inv_freq,
                            const int* kv_slots, void* pool, int n_tokens, int n_q_heads,
                            int n_kv_heads, int head_dim, int page_size, int write_kv, int dtype,
                            cudaStream_t stream) {
  if (!qkv || !positions || !inv_freq || n_tokens < 0 || n_q_heads <= 0 || n_kv_heads <= 0 ||
      head_dim <= 0)
    return SI_ERR_ARG;
  if (head_dim % 16 != 0) return SI_ERR_UNSUPPORTED;
  if ((((uintptr_t)qkv | (uintptr_t)pool) & 31) != 0) return SI_ERR_ARG;
  if (write_kv && (!kv_slots || !pool || page_size <= 0)) return SI_ERR_ARG;
  if (n_tokens == 0) return SI_OK;
  const size_t smem = (size_t)head_dim * sizeof(float);
  if (smem > 48 * 1024) return SI_ERR_TOO_LARGE;
  const int work = n_q_heads * (head_dim / 16);
  int threads = (work + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  if (threads < 64) threads = 64;
  if (dtype == SI_F32)
    SI_LAUNCH(si::rope_kv_store_kernel<float>, n_tokens, threads, smem, stream, (float*)qkv,
              positions, inv_freq, kv_slots, (float*)pool, n_q_heads, n_kv_heads, head_dim,
              page_size, write_kv);
  else if (dtype == SI_BF16)
    SI_LAUNCH(si::rope_kv_store_kernel<__nv_bfloat16>, n_tokens, threads, smem, stream,
              (__nv_bfloat16*)qkv, positions, inv_freq, kv_slots, (__nv_bfloat16*)pool, n_q_heads,
              n_kv_heads, head_dim, page_size, write_kv);
  else
    return SI_ERR_DTYPE;
  return SI_OK;
}
