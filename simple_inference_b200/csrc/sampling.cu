// Sampling from float32 logits: greedy, temperature, top-k and top-p, one
// thread block per row.
//
// Behaviour follows the reference's sample() (sampling.py:140-172):
//   temperature == 0  -> argmax, top-k and top-p ignored           (:159-160)
//   else z = logits / temperature                                   (:39-52)
//   top-k: keep z >= the k-th largest z (ties kept); k<=0 or k>=V off (:68-83)
//   top-p: over what top-k kept, in descending order keep a token while the
//          probability mass of the tokens before it is <= p, so the token that
//          crosses p stays; p>=1 off; p<=0 keeps the top token      (:95-128)
//   then draw from softmax of what is kept                          (:169-172)
// The draw differs in mechanism, not in distribution: the reference calls
// torch.multinomial on the global generator, which depends on batch order.
// Here token = argmax_v (z_v + G_v) with Gumbel noise G_v = -log(-log(u_v)) and
// u_v a hash of (seed, stream, counter, v): a request's draw is the same alone
// or in any batch.  A row without one comparable logit (all NaN, which is how a
// failed kernel upstream marks its output) yields token -1, never an index.
// Thresholds are found by bitwise search over the ordered
// integer image of the floats (no sort, no scratch memory).
#include "common.cuh"

namespace si {

constexpr int SAMPLE_THREADS = 1024;

__device__ __forceinline__ uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}

// uniform strictly inside (0,1) for (seed, stream, counter, v): 23 bits of the hash plus a
// half, which float32 holds exactly (24 bits would round 16777215.5 up to 2^24, u = 1 and
// infinite Gumbel noise)
__device__ __forceinline__ float uniform01(uint32_t base, uint32_t v) {
  const uint32_t h = mix32(base ^ mix32(v + 0x9e3779b9U));
  return ((float)(h >> 9) + 0.5f) * (1.0f / 8388608.0f);
}

__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000U) ? ~u : (u | 0x80000000U);
}

struct ArgBest {
  float v;
  int i;
};

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {
  // larger value wins; on equal values the lower index wins
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}

__device__ __forceinline__ ArgBest block_argbest(ArgBest x, float* sv, int* si_) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = better(x, y);
  }
  __syncthreads();
  if (lane == 0) {
    sv[warp] = x.v;
    si_[warp] = x.i;
  }
  __syncthreads();
  const int nwarps = blockDim.x >> 5;
  ArgBest r;
  r.v = (lane < nwarps) ? sv[lane] : -INFINITY;
  r.i = (lane < nwarps) ? si_[lane] : 0x7fffffff;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y;
    y.v = __shfl_xor_sync(0xffffffffu, r.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, r.i, o);
    r = better(r, y);
  }
  return r;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, int ld,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const uint32_t* __restrict__ seed,
              const uint32_t* __restrict__ stream_id, const uint32_t* __restrict__ counter,
              int* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int sidx[32];
  pdl_wait();
  pdl_trigger();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const float temp = temperature[r];
  const int tid = threadIdx.x;

  if (!(temp > 0.0f)) {  // greedy
    ArgBest b{-INFINITY, 0x7fffffff};
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      // four 16-byte loads in flight per thread: a row of 128k logits is 31 such loads a thread,
      // and one after the other they took 19 us
      const float4* row4 = reinterpret_cast<const float4*>(row);
      const int n4 = vocab >> 2;
      for (int i = tid; i < n4; i += 4 * SAMPLE_THREADS) {
        float4 q[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int j = i + u * SAMPLE_THREADS;
          q[u] = j < n4 ? row4[j] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (i + u * SAMPLE_THREADS >= n4) break;   // never let a filler's index in
          const int v = (i + u * SAMPLE_THREADS) * 4;
          b = better(b, ArgBest{q[u].x, v});
          b = better(b, ArgBest{q[u].y, v + 1});
          b = better(b, ArgBest{q[u].z, v + 2});
          b = better(b, ArgBest{q[u].w, v + 3});
        }
      }
      done = n4 << 2;
    }
    for (int v = done + tid; v < vocab; v += SAMPLE_THREADS) b = better(b, ArgBest{row[v], v});
    b = block_argbest(b, sv, sidx);
    if (tid == 0) out[r] = (b.i == 0x7fffffff) ? -1 : b.i;  // -1: no comparable logit (NaN row)
    return;
  }

  const int k = top_k[r];
  const float p = top_p[r];
  uint32_t keep_key = 0;  // keep tokens whose ordered key of z is >= keep_key

  if (k > 0 && k < vocab) {
    uint32_t t = 0;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = t | (1u << bit);
      float cnt = 0.0f;  // counts up to 2^24 are exact in float
      for (int v = tid; v < vocab; v += SAMPLE_THREADS)
        cnt += (ordered_key(row[v] / temp) >= cand) ? 1.0f : 0.0f;
      cnt = block_sum(cnt, sv);
      if (cnt >= (float)k) t = cand;
    }
    keep_key = t;
  }

  if (p < 1.0f) {
    float mx = -INFINITY;
    for (int v = tid; v < vocab; v += SAMPLE_THREADS) mx = fmaxf(mx, row[v] / temp);
    mx = block_max(mx, sv);
    if (p <= 0.0f) {
      const uint32_t top = ordered_key(mx);
      keep_key = top > keep_key ? top : keep_key;
    } else {
      float denom = 0.0f;
      for (int v = tid; v < vocab; v += SAMPLE_THREADS) {
        const float z = row[v] / temp;
        if (ordered_key(z) >= keep_key) denom += expf(z - mx);
      }
      denom = block_sum(denom, sv);
      const float budget = p * denom;
      // P(t): mass of kept tokens with key > t is <= budget.  Find the largest
      // t with P(t) false; tokens with key >= t+1 are kept.
      auto mass_above = [&](uint32_t t) {
        float s = 0.0f;
        for (int v = tid; v < vocab; v += SAMPLE_THREADS) {
          const float z = row[v] / temp;
          const uint32_t key = ordered_key(z);
          if (key >= keep_key && key > t) s += expf(z - mx);
        }
        return block_sum(s, sv);
      };
      if (mass_above(0u) > budget) {
        uint32_t t = 0;
        for (int bit = 31; bit >= 0; --bit) {
          const uint32_t cand = t | (1u << bit);
          if (mass_above(cand) > budget) t = cand;
        }
        const uint32_t nucleus = t + 1u;
        keep_key = nucleus > keep_key ? nucleus : keep_key;
      }
    }
  }

  const uint32_t base = mix32(counter[r] + mix32(stream_id[r] + mix32(seed[r])));
  ArgBest b{-INFINITY, 0x7fffffff};
  for (int v = tid; v < vocab; v += SAMPLE_THREADS) {
    const float z = row[v] / temp;
    if (ordered_key(z) < keep_key) continue;
    const float u = uniform01(base, (uint32_t)v);
    const float g = -logf(-logf(u));
    b = better(b, ArgBest{z + g, v});
  }
  b = block_argbest(b, sv, sidx);
  if (tid == 0) out[r] = (b.i == 0x7fffffff) ? -1 : b.i;
}

}  // namespace si

// logits: [n_rows, ld] float32, ld >= vocab.  Per-row parameters.
SI_API int si_sample(const float* logits, int n_rows, int vocab, int ld, const float* temperature,
                     const int* top_k, const float* top_p, const uint32_t* seed,
                     const uint32_t* stream_id, const uint32_t* counter, int* out,
                     cudaStream_t stream) {
  if (!logits || !temperature || !top_k || !top_p || !seed || !stream_id || !counter || !out)
    return SI_ERR_ARG;
  if (n_rows < 0 || vocab <= 0 || ld < vocab) return SI_ERR_ARG;
  if (vocab > (1 << 24)) return SI_ERR_TOO_LARGE;
  if (n_rows == 0) return SI_OK;
  SI_LAUNCH(si::sample_kernel, n_rows, si::SAMPLE_THREADS, 0, stream, logits, vocab, ld,
            temperature, top_k, top_p, seed, stream_id, counter, out);
  return SI_OK;
}
