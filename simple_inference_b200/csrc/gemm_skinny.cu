// Matrix product for a handful of tokens (M <= 16) in bfloat16: out = X W^T with
// X [M, K] activations and W [N, K] weights in the nn.Linear layout.
//
// At these sizes the product is a stream of the weights through the SMs once
// (reference: F.linear at ops/attention.py:128-130,226, ops/mlp.py:117,128 and
// ops/embedding.py:92, i.e. cuBLAS, which picks slow kernels for M <= 16).  The
// weights are the 16-row operand of mma.sync m16n8k16 and the tokens the 8-wide
// one ("swap A and B"), so 8 tokens cost one instruction per 16 weight rows and
// 16 k.  Every lane loads 16 contiguous bytes of two weight rows per step
// straight from global memory (a warp covers 16 rows x 64 bytes: whole
// sectors), keeps several steps in flight, and never touches shared memory
// until the end.  The k index inside a 32-wide step is permuted the same way
// for both operands (lane t of a row holds k = 8t..8t+7), which leaves the dot
// products unchanged.
//
// A block is 8 warps: warps_n groups of 16 rows times warps_k shares of K; the
// shares interleave 32-wide steps so that the block reads each row
// contiguously.  Partial sums meet in shared memory in a fixed order.
//
// Epilogues: bfloat16 out; float32 out (logits); SwiGLU, where W is the stacked
// [gate; up] matrix (reference ops/mlp.py:104) and the block computes gate row n
// and up row n together and writes silu(gate) * up (reference ops/mlp.py:125,
// kernels/swiglu_kernel.py:142-150) without the [M, 2I] intermediate; and, for the
// stacked [Wq; Wk; Wv] projection, the rotary position encoding with the write of keys
// and values into their pages (the arithmetic of rope_kv.cu, reference
// ops/rope.py:167-215 and serving/paged_kv_cache.py:171-182): there a warp's 16 rows are
// 8 rows of a head's first half and the 8 rows that pair with them in its second half,
// so that both members of every rotated pair meet in one thread.
#include "common.cuh"

namespace si {

typedef __nv_bfloat16 bf16;
constexpr int SK_THREADS = 256;
constexpr int SK_WARPS = 8;
constexpr int SK_UNROLL = 4;  // 32-wide k-steps a warp requests at a time

enum SkinnyEpilogue { SK_BF16 = 0, SK_F32 = 1, SK_SWIGLU = 2, SK_ROPE = 3 };

// What the rotary epilogue needs beside the product: see rope_kv.cu for the meanings.
struct RopeEpilogue {
  const int* positions;
  const float* inv_freq;
  const int* kv_slots;
  bf16* pool;
  int n_q_heads, n_kv_heads, head_dim, page_size, write_kv;
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  // weights are read once: do not keep them in L1; let L2 fetch the row 256 bytes at a time
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// NT: n-tiles of 8 tokens (1 or 2).  MT: weight tiles per warp (2 for SwiGLU).
template <int NT, int EPI>
__global__ void __launch_bounds__(SK_THREADS)
skinny_gemm_kernel(const bf16* __restrict__ X, int ldx, const bf16* __restrict__ W,
                   void* __restrict__ out, int ldo, int M, int N, int K, int warps_k,
                   RopeEpilogue rope) {
  constexpr int MT = (EPI == SK_SWIGLU) ? 2 : 1;
  __shared__ float red[SK_WARPS][MT * 16][NT * 8 + 1];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int warps_n = SK_WARPS / warps_k;
  const int kw = warp % warps_k;
  // for SwiGLU, N is the output width I and W has 2*I rows: gate rows then up rows
  const int n0 = (blockIdx.x * warps_n + warp / warps_k) * 16;

  const bf16* wrow[MT][2];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int base = mt * N;  // the up rows follow the N gate rows
    int r0 = n0 + g, r1 = n0 + g + 8;
    if (EPI == SK_ROPE) {
      // tile n0/16 of the projection: pairs 8j..8j+7 of head hh, (x_i, x_{i + D/2})
      const int half = rope.head_dim >> 1, per_head = half >> 3;
      const int tile = n0 >> 4, hh = tile / per_head, j = tile - hh * per_head;
      r0 = hh * rope.head_dim + j * 8 + g;
      r1 = r0 + half;
    }
    if (r0 > N - 1) r0 = N - 1;
    if (r1 > N - 1) r1 = N - 1;
    wrow[mt][0] = W + (size_t)(base + r0) * K;
    wrow[mt][1] = W + (size_t)(base + r1) * K;
  }
  const bf16* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    int tok = nt * 8 + g;
    if (tok > M - 1) tok = M - 1;
    xrow[nt] = X + (size_t)tok * ldx;
  }

  float first_sin = 0.0f, first_cos = 1.0f;
  float acc[MT][NT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mt][nt][e] = 0.0f;

  // Software pipeline over batches of SK_UNROLL steps: the weights of batch i+1
  // are requested before batch i is multiplied, so a warp keeps two batches
  // (8 steps, 8 KB) in flight.  Step s of this warp is global step kw + s*warps_k.
  const int n_steps = (K + 31) / 32;
  const int my_steps = (n_steps - kw + warps_k - 1) / warps_k;
  const int n_batches = (my_steps + SK_UNROLL - 1) / SK_UNROLL;

  uint4 a0[SK_UNROLL][MT][2], a1[SK_UNROLL][MT][2];
  auto load_a = [&](uint4 (&a)[SK_UNROLL][MT][2], int batch) {
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int k = (kw + (batch * SK_UNROLL + u) * warps_k) * 32 + t * 8;
      const bool ok = k < K;  // K is a multiple of 8: a lane's 8 values are all in or all out
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) {
        a[u][mt][0] = ok ? ldg_stream(wrow[mt][0] + k) : make_uint4(0, 0, 0, 0);
        a[u][mt][1] = ok ? ldg_stream(wrow[mt][1] + k) : make_uint4(0, 0, 0, 0);
      }
    }
  };
  auto multiply = [&](const uint4 (&a)[SK_UNROLL][MT][2], int batch) {
    uint4 b[SK_UNROLL][NT];
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u) {
      const int k = (kw + (batch * SK_UNROLL + u) * warps_k) * 32 + t * 8;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        b[u][nt] = (k < K) ? *reinterpret_cast<const uint4*>(xrow[nt] + k) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < SK_UNROLL; ++u)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          mma16816(acc[mt][nt], a[u][mt][0].x, a[u][mt][1].x, a[u][mt][0].y, a[u][mt][1].y,
                   b[u][nt].x, b[u][nt].y);
          mma16816(acc[mt][nt], a[u][mt][0].z, a[u][mt][1].z, a[u][mt][0].w, a[u][mt][1].w,
                   b[u][nt].z, b[u][nt].w);
        }
  };

  if (MT == 2) {
    // two weight tiles per warp: the second buffer would cost a resident block per SM,
    // which measures slower than the latency it hides
    load_a(a0, 0);
    pdl_wait();
    multiply(a0, 0);
    for (int batch = 1; batch < n_batches; ++batch) {
      load_a(a0, batch);
      multiply(a0, batch);
    }
  } else {
    load_a(a0, 0);  // weights are never written: request the first ones before waiting
    if (EPI == SK_ROPE) {
      // positions were on the device before the step began: the angle of this thread's
      // first pair is worked out while the kernel before this one finishes
      const int pairs_cta = warps_n * 8;
      if ((int)threadIdx.x < pairs_cta * M) {
        const int p = threadIdx.x % pairs_cta, m = threadIdx.x / pairs_cta;
        const int tile = blockIdx.x * warps_n + (p >> 3), per_head = rope.head_dim >> 4;
        const int i = (tile % per_head) * 8 + (p & 7);
        sincosf((float)rope.positions[m] * rope.inv_freq[i], &first_sin, &first_cos);
      }
    }
    pdl_wait();
    for (int batch = 0; batch < n_batches; batch += 2) {
      load_a(a1, batch + 1);   // steps past the end load nothing
      multiply(a0, batch);
      load_a(a0, batch + 2);
      multiply(a1, batch + 1);
    }
  }

  pdl_trigger();
  // partial sums of this warp: rows g, g+8 of each tile, tokens 2t, 2t+1 of each n-tile
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      red[warp][mt * 16 + g][nt * 8 + 2 * t] = acc[mt][nt][0];
      red[warp][mt * 16 + g][nt * 8 + 2 * t + 1] = acc[mt][nt][1];
      red[warp][mt * 16 + g + 8][nt * 8 + 2 * t] = acc[mt][nt][2];
      red[warp][mt * 16 + g + 8][nt * 8 + 2 * t + 1] = acc[mt][nt][3];
    }
  __syncthreads();

  if (EPI == SK_ROPE) {
    const int D = rope.head_dim, half = D >> 1, per_head = half >> 3;
    const int pairs_cta = warps_n * 8;
    bf16* q_out = reinterpret_cast<bf16*>(out);
    for (int idx = threadIdx.x; idx < pairs_cta * M; idx += SK_THREADS) {
      const int p = idx % pairs_cta, m = idx / pairs_cta;
      const int wn = p >> 3, pr = p & 7;
      const int tile = blockIdx.x * warps_n + wn;
      if (tile * 16 >= N) continue;
      const int hh = tile / per_head, i = (tile - hh * per_head) * 8 + pr;
      float a = 0.0f, b = 0.0f;
      for (int k = 0; k < warps_k; ++k) {
        a += red[wn * warps_k + k][pr][m];
        b += red[wn * warps_k + k][pr + 8][m];
      }
      // rounded as the separate projection rounds its output, then rotated in float32
      a = __bfloat162float(__float2bfloat16_rn(a));
      b = __bfloat162float(__float2bfloat16_rn(b));
      const bool is_q = hh < rope.n_q_heads;
      const int kv = hh - rope.n_q_heads;  // key heads, then value heads
      if (kv < rope.n_kv_heads) {
        float sn = first_sin, cs = first_cos;
        if (idx != (int)threadIdx.x) sincosf((float)rope.positions[m] * rope.inv_freq[i], &sn, &cs);
        const float ra = a * cs - b * sn, rb = b * cs + a * sn;
        a = ra;
        b = rb;
      }
      bf16* dst;
      if (is_q) {
        dst = q_out + (size_t)m * ldo + hh * D + i;
      } else {
        if (!rope.write_kv) continue;
        const int slot = rope.kv_slots[m];
        const int page = slot / rope.page_size, off = slot - page * rope.page_size;
        const int which = kv < rope.n_kv_heads ? 0 : 1;
        const int h = kv - which * rope.n_kv_heads;
        dst = rope.pool + ((((size_t)page * 2 + which) * rope.n_kv_heads + h) * rope.page_size + off) * D + i;
      }
      dst[0] = __float2bfloat16_rn(a);
      dst[half] = __float2bfloat16_rn(b);
    }
    return;
  }

  const int rows_cta = warps_n * 16;
  const int row_base = blockIdx.x * rows_cta;
  for (int idx = threadIdx.x; idx < rows_cta * M; idx += SK_THREADS) {
    const int r = idx % rows_cta, m = idx / rows_cta;
    const int n = row_base + r;
    if (n >= N) continue;
    const int wn = r >> 4, rr = r & 15;
    float s0 = 0.0f, s1 = 0.0f;
    for (int k = 0; k < warps_k; ++k) {
      s0 += red[wn * warps_k + k][rr][m];
      if (MT == 2) s1 += red[wn * warps_k + k][16 + rr][m];
    }
    if (EPI == SK_BF16) {
      reinterpret_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(s0);
    } else if (EPI == SK_F32) {
      reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = s0;
    } else {
      const float act = s0 / (1.0f + expf(-s0));
      reinterpret_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(act * s1);
    }
  }
}

template <int NT, int EPI>
static int launch_skinny(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N,
                         int K, cudaStream_t stream, RopeEpilogue rope = RopeEpilogue()) {
  // As many rows per block as still leaves two blocks for each of the 148 SMs.
  int warps_n = 8;
  while (warps_n > 1 && (N + warps_n * 16 - 1) / (warps_n * 16) < 2 * 148) warps_n >>= 1;
  const int warps_k = SK_WARPS / warps_n;
  const int blocks = (N + warps_n * 16 - 1) / (warps_n * 16);
  SI_LAUNCH((skinny_gemm_kernel<NT, EPI>), blocks, SK_THREADS, 0, stream, (const bf16*)X, ldx,
            (const bf16*)W, out, ldo, M, N, K, warps_k, rope);
  return SI_OK;
}

}  // namespace si

// out[M, N] = X[M, K] W[N, K]^T for M <= 16.  epilogue 0: bfloat16 out, 1: float32 out,
// 2: SwiGLU (W has 2*N rows, gate rows first; out is bfloat16 [M, N]).
// K must be a multiple of 8; X rows, W and ldx must keep 16-byte alignment.
SI_API int si_gemm_skinny_bf16(const void* X, int ldx, const void* W, void* out, int ldo, int M,
                               int N, int K, int epilogue, cudaStream_t stream) {
  if (!X || !W || !out || M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N) return SI_ERR_ARG;
  if (M > 16 || K % 8 != 0 || ldx % 8 != 0) return SI_ERR_UNSUPPORTED;
  if (((uintptr_t)X | (uintptr_t)W) & 15) return SI_ERR_ARG;
  if (M == 0) return SI_OK;
  using namespace si;
  if (M <= 8) {
    if (epilogue == SK_BF16) return launch_skinny<1, SK_BF16>(X, ldx, W, out, ldo, M, N, K, stream);
    if (epilogue == SK_F32) return launch_skinny<1, SK_F32>(X, ldx, W, out, ldo, M, N, K, stream);
    if (epilogue == SK_SWIGLU) return launch_skinny<1, SK_SWIGLU>(X, ldx, W, out, ldo, M, N, K, stream);
  } else {
    if (epilogue == SK_BF16) return launch_skinny<2, SK_BF16>(X, ldx, W, out, ldo, M, N, K, stream);
    if (epilogue == SK_F32) return launch_skinny<2, SK_F32>(X, ldx, W, out, ldo, M, N, K, stream);
    if (epilogue == SK_SWIGLU) return launch_skinny<2, SK_SWIGLU>(X, ldx, W, out, ldo, M, N, K, stream);
  }
  return SI_ERR_ARG;
}

// The stacked projection [Wq; Wk; Wv] of M <= 16 tokens with the rotary encoding and the
// cache write in its epilogue: rotated queries go to the first n_q_heads*head_dim columns
// of qkv (the other columns are left alone), rotated keys and the values to slot
// kv_slots[m] of the pool [pages, 2, n_kv_heads, page_size, head_dim] unless write_kv is 0.
SI_API int si_gemm_skinny_rope_kv_bf16(const void* X, int ldx, const void* W, void* qkv, int ldo,
                                       int M, int K, const int* positions, const float* inv_freq,
                                       const int* kv_slots, void* pool, int n_q_heads,
                                       int n_kv_heads, int head_dim, int page_size, int write_kv,
                                       cudaStream_t stream) {
  if (!X || !W || !qkv || !positions || !inv_freq || M < 0 || K <= 0 || n_q_heads <= 0 ||
      n_kv_heads <= 0 || head_dim <= 0 || ldx < K)
    return SI_ERR_ARG;
  if (write_kv && (!kv_slots || !pool || page_size <= 0)) return SI_ERR_ARG;
  if (M > 16 || K % 8 != 0 || ldx % 8 != 0 || head_dim % 16 != 0) return SI_ERR_UNSUPPORTED;
  if (((uintptr_t)X | (uintptr_t)W) & 15) return SI_ERR_ARG;
  const int N = (n_q_heads + 2 * n_kv_heads) * head_dim;
  if (ldo < n_q_heads * head_dim) return SI_ERR_ARG;
  if (M == 0) return SI_OK;
  using namespace si;
  RopeEpilogue rope;
  rope.positions = positions;
  rope.inv_freq = inv_freq;
  rope.kv_slots = kv_slots;
  rope.pool = (bf16*)pool;
  rope.n_q_heads = n_q_heads;
  rope.n_kv_heads = n_kv_heads;
  rope.head_dim = head_dim;
  rope.page_size = page_size;
  rope.write_kv = write_kv;
  if (M <= 8) return launch_skinny<1, SK_ROPE>(X, ldx, W, qkv, ldo, M, N, K, stream, rope);
  return launch_skinny<2, SK_ROPE>(X, ldx, W, qkv, ldo, M, N, K, stream, rope);
}
