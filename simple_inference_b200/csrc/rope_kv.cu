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
  __syncthreads();

  const int row_width = (n_q_heads + 2 * n_kv_heads) * head_dim;
  T* row = qkv + (size_t)t * row_width;

  // queries: rotate in place
  const int q_pairs = n_q_heads * half;
  for (int w = threadIdx.x; w < q_pairs; w += blockDim.x) {
    const int h = w / half, i = w - h * half;
    T* p = row + h * head_dim;
    const float a = to_f32<T>(p[i]), b = to_f32<T>(p[i + half]);
    const float c = s_cos[i], s = s_sin[i];
    p[i] = from_f32<T>(a * c - b * s);
    p[i + half] = from_f32<T>(b * c + a * s);
  }
  if (!write_kv) return;

  const int slot = kv_slots[t];
  const int page = slot / page_size, off = slot - page * page_size;
  const size_t head_stride = (size_t)page_size * head_dim;
  T* kpage = pool + ((size_t)page * 2 + 0) * n_kv_heads * head_stride + (size_t)off * head_dim;
  T* vpage = pool + ((size_t)page * 2 + 1) * n_kv_heads * head_stride + (size_t)off * head_dim;
  const T* krow = row + n_q_heads * head_dim;
  const T* vrow = krow + n_kv_heads * head_dim;

  const int k_pairs = n_kv_heads * half;
  for (int w = threadIdx.x; w < k_pairs; w += blockDim.x) {
    const int h = w / half, i = w - h * half;
    const T* p = krow + h * head_dim;
    const float a = to_f32<T>(p[i]), b = to_f32<T>(p[i + half]);
    const float c = s_cos[i], s = s_sin[i];
    T* dst = kpage + h * head_stride;
    dst[i] = from_f32<T>(a * c - b * s);
    dst[i + half] = from_f32<T>(b * c + a * s);
  }
  const int v_elems = n_kv_heads * head_dim;
  for (int w = threadIdx.x; w < v_elems; w += blockDim.x) {
    const int h = w / head_dim, d = w - h * head_dim;
    vpage[h * head_stride + d] = vrow[w];
  }
}

}  // namespace si

SI_API int si_rope_kv_store(void* qkv, const int* positions, const float* inv_freq,
                            const int* kv_slots, void* pool, int n_tokens, int n_q_heads,
                            int n_kv_heads, int head_dim, int page_size, int write_kv, int dtype,
                            cudaStream_t stream) {
  if (!qkv || !positions || !inv_freq || n_tokens < 0 || n_q_heads <= 0 || n_kv_heads <= 0 ||
      head_dim <= 0 || (head_dim & 1))
    return SI_ERR_ARG;
  if (write_kv && (!kv_slots || !pool || page_size <= 0)) return SI_ERR_ARG;
  if (n_tokens == 0) return SI_OK;
  const size_t smem = (size_t)head_dim * sizeof(float);
  if (smem > 48 * 1024) return SI_ERR_TOO_LARGE;
  const int work = n_q_heads * (head_dim / 2);
  const int threads = work >= 1024 ? 256 : 128;
  if (dtype == SI_F32)
    si::rope_kv_store_kernel<float><<<n_tokens, threads, smem, stream>>>(
        (float*)qkv, positions, inv_freq, kv_slots, (float*)pool, n_q_heads, n_kv_heads, head_dim,
        page_size, write_kv);
  else if (dtype == SI_BF16)
    si::rope_kv_store_kernel<__nv_bfloat16><<<n_tokens, threads, smem, stream>>>(
        (__nv_bfloat16*)qkv, positions, inv_freq, kv_slots, (__nv_bfloat16*)pool, n_q_heads,
        n_kv_heads, head_dim, page_size, write_kv);
  else
    return SI_ERR_DTYPE;
  SI_LAUNCH_CHECK();
  return SI_OK;
}
