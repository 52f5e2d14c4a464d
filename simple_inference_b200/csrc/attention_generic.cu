// Attention over the paged cache, generic form: any head size that is a
// multiple of 16 up to 256, any number of heads and groups, any page size,
// float32 or bfloat16 storage, all arithmetic in float32.  It is the attention
// of the 32-bit path and the yardstick of the tensor-core kernels.
//
// For the query of token t (request s = tok_seq[t], absolute position p) and
// query head h (key/value head h / G):
//     S_j = (q . k_j) * scale          for keys j in [max(0, p-window+1), p]
//     O   = softmax_j(S) V
// computed with the online form m' = max(m, max_j S_j), P_j = exp(S_j - m'),
// l = l*exp(m-m') + sum P_j, acc = acc*exp(m-m') + sum P_j v_j, O = acc / l,
// which is the reference's recurrence (kernels/attention_kernel.py:231-244 and
// 558-581; mask rule serving/paged_kv_cache.py:366-372; grouping :188).  Keys
// are visited in tiles of 128 aligned to absolute key index, so the order of
// every sum depends on the key index alone: a token's result is the same
// whatever else is in the batch and however the prompt was cut.
//
// Key j of request s lives at pool[page][0][kvh][j % page_size][:] with
// page = block_table[s][j / page_size]; values at pool[page][1][...].
#include "common.cuh"

namespace si {

constexpr int ATT_THREADS = 128;

template <typename T> struct Vec16;  // 16 bytes of T
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ qs, const T* __restrict__ krow,
                                         int head_dim);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ qs,
                                                const float* __restrict__ krow, int head_dim) {
  float acc = 0.0f;
  for (int d = 0; d < head_dim; d += 4) {
    const float4 k = *reinterpret_cast<const float4*>(krow + d);
    acc = fmaf(qs[d], k.x, acc);
    acc = fmaf(qs[d + 1], k.y, acc);
    acc = fmaf(qs[d + 2], k.z, acc);
    acc = fmaf(qs[d + 3], k.w, acc);
  }
  return acc;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ qs,
                                                        const __nv_bfloat16* __restrict__ krow,
                                                        int head_dim) {
  float acc = 0.0f;
  for (int d = 0; d < head_dim; d += 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
    const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(k2[i]);
      acc = fmaf(qs[d + 2 * i], f.x, acc);
      acc = fmaf(qs[d + 2 * i + 1], f.y, acc);
    }
  }
  return acc;
}

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attn_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ pool,
                    const int* __restrict__ block_table, int table_stride,
                    const int* __restrict__ tok_seq, const int* __restrict__ positions,
                    T* __restrict__ out, int out_stride, int n_q_heads, int n_kv_heads,
                    int head_dim, int page_size, float scale, int window) {
  extern __shared__ float smem[];
  float* qs = smem;                       // [head_dim]
  float* ps = qs + head_dim;              // [ATT_THREADS]
  long long* voff = reinterpret_cast<long long*>(ps + ATT_THREADS);  // [ATT_THREADS]
  __shared__ float red[32];
  pdl_wait();

  const int t = blockIdx.x, h = blockIdx.y;
  const int tid = threadIdx.x;
  const int seq = tok_seq[t];
  const int pos = positions[t];
  const int group = n_q_heads / n_kv_heads;
  const int kvh = h / group;
  const int k_lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  const T* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
  for (int d = tid; d < head_dim; d += ATT_THREADS) qs[d] = to_f32<T>(qrow[d]);
  __syncthreads();

  const int* table = block_table + (size_t)seq * table_stride;
  const long long head_stride = (long long)page_size * head_dim;
  const long long v_plane = (long long)n_kv_heads * head_stride;  // K plane -> V plane

  float m_run = -INFINITY, l_run = 0.0f;
  float acc0 = 0.0f, acc1 = 0.0f;  // output dims tid and tid + ATT_THREADS

  const int tile_first = k_lo / ATT_THREADS, tile_last = pos / ATT_THREADS;
  for (int tile = tile_first; tile <= tile_last; ++tile) {
    const int j0 = tile * ATT_THREADS;
    const int jj_lo = (k_lo > j0) ? k_lo - j0 : 0;
    const int jj_hi = (pos - j0 + 1 < ATT_THREADS) ? pos - j0 + 1 : ATT_THREADS;  // exclusive
    float s = -INFINITY;
    if (tid >= jj_lo && tid < jj_hi) {
      const int j = j0 + tid;
      const int page = table[j / page_size];
      const int off = j - (j / page_size) * page_size;
      const long long kbase =
          ((long long)page * 2 * n_kv_heads + kvh) * head_stride + (long long)off * head_dim;
      voff[tid] = kbase + v_plane;
      s = dot_row<T>(qs, pool + kbase, head_dim) * scale;
    }
    const float m_tile = block_max(s, red);
    const float m_new = fmaxf(m_run, m_tile);
    const float p = (tid >= jj_lo && tid < jj_hi) ? expf(s - m_new) : 0.0f;
    ps[tid] = p;
    const float p_sum = block_sum(p, red);  // has __syncthreads: ps, voff visible after it
    const float alpha = (m_run == -INFINITY) ? 0.0f : expf(m_run - m_new);
    l_run = l_run * alpha + p_sum;
    m_run = m_new;
    acc0 *= alpha;
    acc1 *= alpha;
    if (tid < head_dim) {
      for (int jj = jj_lo; jj < jj_hi; ++jj)
        acc0 = fmaf(ps[jj], to_f32<T>(pool[voff[jj] + tid]), acc0);
    }
    if (tid + ATT_THREADS < head_dim) {
      for (int jj = jj_lo; jj < jj_hi; ++jj)
        acc1 = fmaf(ps[jj], to_f32<T>(pool[voff[jj] + tid + ATT_THREADS]), acc1);
    }
    __syncthreads();  // ps / voff are rewritten by the next tile
  }
  pdl_trigger();
  T* orow = out + (size_t)t * out_stride + (size_t)h * head_dim;
  const float inv_l = 1.0f / l_run;
  if (tid < head_dim) orow[tid] = from_f32<T>(acc0 * inv_l);
  if (tid + ATT_THREADS < head_dim) orow[tid + ATT_THREADS] = from_f32<T>(acc1 * inv_l);
}

}  // namespace si

// q: [n_tokens, q_stride] with head h at column h*head_dim; out likewise.
// window <= 0 means every earlier key is visible.
SI_API int si_attention_generic(const void* q, int q_stride, const void* pool,
                                const int* block_table, int table_stride, const int* tok_seq,
                                const int* positions, void* out, int out_stride, int n_tokens,
                                int n_q_heads, int n_kv_heads, int head_dim, int page_size,
                                float scale, int window, int dtype, cudaStream_t stream) {
  if (!q || !pool || !block_table || !tok_seq || !positions || !out) return SI_ERR_ARG;
  if (n_tokens < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || page_size <= 0 || table_stride <= 0)
    return SI_ERR_ARG;
  if (n_q_heads % n_kv_heads != 0) return SI_ERR_ARG;
  if (head_dim <= 0 || head_dim % 16 != 0 || head_dim > 2 * si::ATT_THREADS)
    return SI_ERR_UNSUPPORTED;
  if (q_stride % 8 != 0 || out_stride < n_q_heads * head_dim) return SI_ERR_ARG;
  if (n_q_heads > 65535) return SI_ERR_TOO_LARGE;
  if (n_tokens == 0) return SI_OK;
  dim3 grid(n_tokens, n_q_heads);
  const size_t smem = (size_t)head_dim * sizeof(float) + si::ATT_THREADS * sizeof(float) +
                      si::ATT_THREADS * sizeof(long long);
  if (dtype == SI_F32)
    SI_LAUNCH(si::attn_generic_kernel<float>, grid, si::ATT_THREADS, smem, stream,
        (const float*)q, q_stride, (const float*)pool, block_table, table_stride, tok_seq,
        positions, (float*)out, out_stride, n_q_heads, n_kv_heads, head_dim, page_size, scale,
        window);
  else if (dtype == SI_BF16)
    SI_LAUNCH(si::attn_generic_kernel<__nv_bfloat16>, grid, si::ATT_THREADS, smem, stream,
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pool, block_table, table_stride,
        tok_seq, positions, (__nv_bfloat16*)out, out_stride, n_q_heads, n_kv_heads, head_dim,
        page_size, scale, window);
  else
    return SI_ERR_DTYPE;
  return SI_OK;
}
