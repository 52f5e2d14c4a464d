// Tensor-core attention over the paged cache for bfloat16, compiled for one
// head size (-DSI_HEAD_DIM=D, D a multiple of 16 up to 256).
//
// Three kernels share one softmax recurrence:
//
//   attn_prefill_kernel  one block per (64-query tile of a sequence, query head):
//                        the flash-attention forward of the reference
//                        (kernels/attention_kernel.py:108-251) reading keys and
//                        values through the block table instead of a gathered copy
//                        (serving/paged_kv_cache.py:188-256).
//   attn_decode_kernel   sequences that bring one token: one block per (sequence,
//                        key/value head, split of the keys); the G query heads of
//                        the group are the rows of one 16-row tile, so keys and
//                        values are read once per group, not once per head, and
//                        the keys are split over blocks (the reference's paged
//                        decode, kernels/attention_kernel.py:496-586, has one
//                        program per query head and no split).  Partial results
//                        go to scratch memory and attn_merge_kernel joins them.
//   attn_decode_tma_kernel  the same, for head sizes that are multiples of 64 and pages
//                        of 8 to 64 tokens: keys and values arrive as TMA boxes
//                        (cp.async.bulk.tensor, 128-byte swizzle) announced by
//                        mbarriers, and no thread computes an address.  A fifth warp
//                        looks the pages up and issues the copies, so the four computing
//                        warps never stand behind a table read or a copy's issue.
//
// Both compute S = (Q K^T) * scale with mma.sync m16n8k16 (bf16 in, float32
// accumulate), mask by absolute position (key j visible to a query at position
// p iff p - window < j <= p), run the online softmax in float32
// (kernels/attention_kernel.py:231-241: m' = max(m, rowmax), P = exp(S - m'),
// l = l*exp(m-m') + sum P, acc = acc*exp(m-m') + P V), round P to bfloat16 for
// the P V product as the reference does (:240), and divide by l at the end.
// Key tiles are 64 keys aligned to absolute key index, so the order of every
// sum depends on key indices only.
//
// Shared-memory rows are padded by 16 bytes: the row stride is then an odd
// multiple of 16 bytes modulo 128, which makes every ldmatrix conflict-free for
// any D that is a multiple of 16.
#include "tma.cuh"

#ifndef SI_HEAD_DIM
#error "compile with -DSI_HEAD_DIM=<head size>"
#endif

namespace si {

constexpr int D = SI_HEAD_DIM;
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "head size must be a multiple of 16 in [16, 256]");
constexpr int STRIDE = D + 8;        // elements per shared-memory row
constexpr int KV_TILE = 64;          // keys per tile of the decode kernel
constexpr int PF_TILE = 32;          // keys per tile of the prefill kernel
constexpr int PF_STAGES = 3;         // tiles in flight in the prefill kernel
constexpr int Q_TILE = 64;           // query rows per prefill block
constexpr int THREADS = 128;
constexpr int CHUNKS = D / 8;        // 16-byte chunks per row
constexpr float LOG2E = 1.4426950408889634f;

typedef __nv_bfloat16 bf16;

// ------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
      "{%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// --------------------------------------------------------------- tile loader
// Keys [key0, key0+64) of one sequence and one kv head into sK, sV.  Keys
// outside [k_lo, k_hi] are zero-filled and their pages are not touched (a page
// before the window may already belong to someone else).
// Where the pages of one (sequence, kv head) lie: everything the loader needs that does
// not change from tile to tile, so that a 16-byte copy costs a handful of instructions.
struct PageWalk {
  const bf16* base;        // pool + kvh * page_size * D
  const int* table;        // block table row of the sequence
  long long page_stride;   // elements between pages: 2 * n_kv_heads * page_size * D
  long long v_offset;      // from a key row to its value row: n_kv_heads * page_size * D
  int page_size;
  int page_shift;          // log2(page_size) if it is a power of two, else -1
};

__device__ __forceinline__ PageWalk make_page_walk(const bf16* pool, const int* table, int kvh,
                                                   int n_kv_heads, int page_size) {
  PageWalk w;
  const long long head_stride = (long long)page_size * D;
  w.base = pool + (long long)kvh * head_stride;
  w.table = table;
  w.page_stride = 2LL * n_kv_heads * head_stride;
  w.v_offset = (long long)n_kv_heads * head_stride;
  w.page_size = page_size;
  w.page_shift = (page_size & (page_size - 1)) == 0 ? __ffs(page_size) - 1 : -1;
  return w;
}

template <int ROWS>
__device__ __forceinline__ void load_kv_tile(bf16* sK, bf16* sV, const PageWalk& w, int key0,
                                             int k_lo, int k_hi) {
  // Consecutive threads copy consecutive 16-byte chunks of a row, so a warp's
  // request covers whole rows (full sectors).  A thread keeps its chunk column
  // and walks down the rows when the thread count is a multiple of the row's chunks.
  constexpr int TOTAL = ROWS * CHUNKS;
#pragma unroll
  for (int i = 0; i < (TOTAL + THREADS - 1) / THREADS; ++i) {
    const int idx = threadIdx.x + i * THREADS;
    if (TOTAL % THREADS != 0 && idx >= TOTAL) break;
    const int row = idx / CHUNKS, chunk = idx - row * CHUNKS;  // CHUNKS is a constant
    const int j = key0 + row;
    const bool valid = (j >= k_lo) && (j <= k_hi);
    const bf16* kptr = w.base;
    if (valid) {
      const int lp = w.page_shift >= 0 ? (j >> w.page_shift) : (j / w.page_size);
      const int off = j - lp * w.page_size;
      kptr = w.base + (long long)w.table[lp] * w.page_stride + (off * D + chunk * 8);
    }
    cp_async16(sK + row * STRIDE + chunk * 8, kptr, valid);
    cp_async16(sV + row * STRIDE + chunk * 8, kptr + w.v_offset, valid);
  }
}

// rows [0, n_rows) of a [rows][D] tile whose row r starts at src + r * row_stride
__device__ __forceinline__ void load_q_rows(bf16* sQ, const bf16* __restrict__ src,
                                            long long row_stride, int n_rows, int tile_rows) {
  for (int idx = threadIdx.x; idx < tile_rows * CHUNKS; idx += THREADS) {
    const int row = idx / CHUNKS, chunk = idx - row * CHUNKS;
    const bool valid = row < n_rows;
    cp_async16(sQ + row * STRIDE + chunk * 8, src + (valid ? row * row_stride + chunk * 8 : 0), valid);
  }
}

// One warp's S = Q_rows K_keys^T for 16 query rows and NT*8 keys.
// sQrow0: first of the 16 query rows in shared memory; sKrow0: first key row.
template <int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const bf16* sQrow0, const bf16* sKrow0) {
  static_assert(NT % 2 == 0, "n-tiles come in pairs");
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t a[4];
    ldsm_x4(a, sQrow0 + ((lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + ks * 16 + 8 * (lane >> 4));
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      ldsm_x4(b, sKrow0 + (np * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + ks * 16 +
                     8 * ((lane >> 3) & 1));
      mma_bf16(s[2 * np], a, b[0], b[1]);
      mma_bf16(s[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// o += P V for one warp: P is 16 rows x NT*8 keys (already exponentiated, in s),
// V rows start at sVrow0.
template <int NT>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&s)[NT][4],
                                        const bf16* sVrow0) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b[4];
      ldsm_x4_trans(b, sVrow0 + (kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + dp * 16 +
                           8 * (lane >> 4));
      mma_bf16(o[2 * dp], a, b[0], b[1]);
      mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Online-softmax update of one warp's rows.  s holds scaled, masked scores in
// the log2 domain (-inf where masked) and is overwritten with P.  m, l are per
// thread for its two rows (lane/4 and lane/4 + 8); l is the thread's partial sum.
template <int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&m)[2], float (&l)[2],
                                               float (&o)[D / 8][4]) {
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[r], mx);
    const float m_use = (m_new == -INFINITY) ? 0.0f : m_new;  // row fully masked so far
    const float alpha = exp2f(m[r] - m_use);                  // m = -inf gives 0
    float sum = 0.0f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float p0 = exp2f(s[nt][2 * r] - m_use);
      const float p1 = exp2f(s[nt][2 * r + 1] - m_use);
      s[nt][2 * r] = p0;
      s[nt][2 * r + 1] = p1;
      sum += p0 + p1;
    }
    l[r] = l[r] * alpha + sum;
    m[r] = m_new;
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      o[dt][2 * r] *= alpha;
      o[dt][2 * r + 1] *= alpha;
    }
  }
}

// ------------------------------------------------------------------- prefill
// grid (pairs of 64-query tiles, query heads).  With a causal mask the later tiles
// of a prompt see the most keys; the host pairs the longest tile with the
// shortest, the second longest with the second shortest and so on (tile_pairs),
// and a block runs its two tiles one after the other, so that all blocks take
// about the same time and none is left running alone at the end.  Keys come in
// tiles of 32 through a three-stage cp.async ring (one barrier per tile): small
// tiles keep the score registers few, so three blocks fit on an SM.
__global__ void __launch_bounds__(THREADS)
attn_prefill_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ pool,
                    const int* __restrict__ block_table, int table_stride,
                    const int* __restrict__ cu_q, const int* __restrict__ positions,
                    const int* __restrict__ tile_seq, const int* __restrict__ tile_start,
                    const int* __restrict__ tile_pairs, bf16* __restrict__ out, int out_stride,
                    int n_q_heads, int n_kv_heads, int page_size, float scale_log2, int window) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);          // [Q_TILE][STRIDE]
  bf16* sKV = sQ + Q_TILE * STRIDE;                      // PF_STAGES x (K, V) x [PF_TILE][STRIDE]
  constexpr int STAGE_ELEMS = 2 * PF_TILE * STRIDE;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  for (int which = 0; which < 2; ++which) {
  const int tile_id = tile_pairs[2 * blockIdx.x + which];
  if (tile_id < 0) break;
  if (which) __syncthreads();  // the first tile's shared memory is free to reuse
  const int seq = tile_seq[tile_id];
  const int tok0 = cu_q[seq] + tile_start[tile_id];
  int n_rows = cu_q[seq + 1] - tok0;
  if (n_rows > Q_TILE) n_rows = Q_TILE;
  const int h = blockIdx.y;
  const int kvh = h / (n_q_heads / n_kv_heads);
  const int pos0 = positions[tok0];  // rows of a tile are consecutive positions
  const int k_hi = pos0 + n_rows - 1;
  const int k_lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const PageWalk walk = make_page_walk(pool, block_table + (long long)seq * table_stride, kvh,
                                       n_kv_heads, page_size);

  const int tile_first = k_lo / PF_TILE, tile_last = k_hi / PF_TILE;
  // prologue: Q and the first PF_STAGES-1 key tiles, one commit group per tile
  load_q_rows(sQ, q + (long long)tok0 * q_stride + (long long)h * D, q_stride, n_rows, Q_TILE);
#pragma unroll
  for (int st = 0; st < PF_STAGES - 1; ++st) {
    if (tile_first + st <= tile_last) {
      bf16* dK = sKV + st * STAGE_ELEMS;
      load_kv_tile<PF_TILE>(dK, dK + PF_TILE * STRIDE, walk, (tile_first + st) * PF_TILE, k_lo,
                            k_hi);
    }
    cp_async_commit();
  }

  float o[D / 8][4];
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  const int row_lo = warp * 16;
  for (int tile = tile_first; tile <= tile_last; ++tile) {
    const int it = tile - tile_first;
    cp_async_wait<PF_STAGES - 2>();  // this tile has landed (one newer group may be in flight)
    __syncthreads();                 // ... for every thread; and everyone is done with tile-1
    {                                // refill the stage that tile-1 used
      const int nt = tile + PF_STAGES - 1;
      if (nt <= tile_last) {
        bf16* dK = sKV + ((it + PF_STAGES - 1) % PF_STAGES) * STAGE_ELEMS;
        load_kv_tile<PF_TILE>(dK, dK + PF_TILE * STRIDE, walk, nt * PF_TILE, k_lo, k_hi);
      }
      cp_async_commit();
    }
    const bf16* sK = sKV + (it % PF_STAGES) * STAGE_ELEMS;
    const bf16* sV = sK + PF_TILE * STRIDE;

    // A warp whose 16 rows are all past n_rows, or all before this tile's keys
    // (causal), skips the arithmetic.
    const bool active = row_lo < n_rows && (pos0 + min(row_lo + 15, n_rows - 1)) >= tile * PF_TILE;
    if (active) {
      float s[PF_TILE / 8][4];
      qk_tile<PF_TILE / 8>(s, sQ + row_lo * STRIDE, sK);
      const int key0 = tile * PF_TILE;
#pragma unroll
      for (int nt = 0; nt < PF_TILE / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int row = row_lo + (lane >> 2) + 8 * (e >> 1);
          const int j = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int p = pos0 + row;
          const bool ok = row < n_rows && j <= p && (window <= 0 || j > p - window);
          s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
        }
      softmax_update<PF_TILE / 8>(s, m, l, o);
      pv_tile<PF_TILE / 8>(o, s, sV);
    }
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float lt = l[r];
    lt += __shfl_xor_sync(0xffffffffu, lt, 1);
    lt += __shfl_xor_sync(0xffffffffu, lt, 2);
    const int row = warp * 16 + (lane >> 2) + 8 * r;
    if (row < n_rows) {
      const float inv = 1.0f / lt;  // the query's own key is always visible, so lt > 0
      bf16* dst = out + (long long)(tok0 + row) * out_stride + (long long)h * D + (lane & 3) * 2;
#pragma unroll
      for (int dt = 0; dt < D / 8; ++dt) {
        *reinterpret_cast<__nv_bfloat162*>(dst + dt * 8) =
            __floats2bfloat162_rn(o[dt][2 * r] * inv, o[dt][2 * r + 1] * inv);
      }
    }
  }
  cp_async_wait<0>();  // only empty groups can be pending here
  }  // which
  pdl_trigger();
}

// -------------------------------------------------------------------- decode
// grid (sequences with one token, kv heads * head chunks, splits).  Rows of the
// 16-row tile are the query heads kvh*G + chunk*16 + r.  Warp w works on keys
// [16w, 16w+16) of every 64-key tile of this block's split; the four warps'
// states are merged in shared memory.  With n_splits > 1 the block writes
// (m, l, unnormalised acc) to scratch for attn_merge_kernel.
__global__ void __launch_bounds__(THREADS)
attn_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ pool,
                   const int* __restrict__ block_table, int table_stride,
                   const int* __restrict__ cu_q, const int* __restrict__ positions,
                   const int* __restrict__ single_seqs, bf16* __restrict__ out, int out_stride,
                   float* __restrict__ part_acc, float* __restrict__ part_ml, int n_q_heads,
                   int n_kv_heads, int page_size, float scale_log2, int window, int n_splits) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sQ = reinterpret_cast<bf16*>(smem_raw);          // [16][STRIDE]
  bf16* sKV = sQ + 16 * STRIDE;                          // 2 stages x (K, V) x [KV_TILE][STRIDE]

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  pdl_wait();
  const int group = n_q_heads / n_kv_heads;
  const int chunks_per_kv = (group + 15) / 16;
  const int kvh = blockIdx.y / chunks_per_kv;
  const int head0 = kvh * group + (blockIdx.y % chunks_per_kv) * 16;
  int n_heads_here = kvh * group + group - head0;
  if (n_heads_here > 16) n_heads_here = 16;
  const int seq = single_seqs[blockIdx.x];
  const int tok = cu_q[seq];
  const int pos = positions[tok];
  const int k_lo_all = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const PageWalk walk = make_page_walk(pool, block_table + (long long)seq * table_stride, kvh,
                                       n_kv_heads, page_size);

  // this block's share of the key tiles [tile_a, tile_b)
  const int tile_first = k_lo_all / KV_TILE, tile_end = pos / KV_TILE + 1;
  const int n_tiles = tile_end - tile_first;
  const int per = (n_tiles + n_splits - 1) / n_splits;
  const int tile_a = tile_first + blockIdx.z * per;
  int tile_b = tile_a + per;
  if (tile_b > tile_end) tile_b = tile_end;

  float o[D / 8][4];
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  if (tile_a < tile_b) {
    // Q rows: one per query head of the chunk, the rest zero
    load_q_rows(sQ, q + (long long)tok * q_stride + (long long)head0 * D, D, n_heads_here, 16);
    load_kv_tile<KV_TILE>(sKV, sKV + KV_TILE * STRIDE, walk, tile_a * KV_TILE, k_lo_all, pos);
    cp_async_commit();
    for (int tile = tile_a; tile < tile_b; ++tile) {
      const int stage = (tile - tile_a) & 1;
      bf16* sK = sKV + stage * 2 * KV_TILE * STRIDE;
      bf16* sV = sK + KV_TILE * STRIDE;
      if (tile + 1 < tile_b) {
        bf16* nK = sKV + (stage ^ 1) * 2 * KV_TILE * STRIDE;
        load_kv_tile<KV_TILE>(nK, nK + KV_TILE * STRIDE, walk, (tile + 1) * KV_TILE, k_lo_all, pos);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const int key0 = tile * KV_TILE + warp * 16;
      if (key0 <= pos && key0 + 15 >= k_lo_all) {
        float s[2][4];
        qk_tile<2>(s, sQ, sK + warp * 16 * STRIDE);
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int j = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
            const bool ok = j <= pos && j >= k_lo_all;
            s[nt][e] = ok ? s[nt][e] * scale_log2 : -INFINITY;
          }
        softmax_update<2>(s, m, l, o);
        pv_tile<2>(o, s, sV + warp * 16 * STRIDE);
      }
      __syncthreads();
    }
  }

  pdl_trigger();
  // ---- merge the four warps (each saw different keys) in shared memory
  // layout: wm[4][16], wl[4][16], wacc[4][16][D] floats, over the K/V stages
  float* wm = reinterpret_cast<float*>(sKV);
  float* wl = wm + 4 * 16;
  float* wacc = wl + 4 * 16;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float lt = l[r];
    lt += __shfl_xor_sync(0xffffffffu, lt, 1);
    lt += __shfl_xor_sync(0xffffffffu, lt, 2);
    const int row = (lane >> 2) + 8 * r;
    if ((lane & 3) == 0) {
      wm[warp * 16 + row] = m[r];
      wl[warp * 16 + row] = lt;
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      float* dst = wacc + ((warp * 16 + row) * D) + dt * 8 + (lane & 3) * 2;
      dst[0] = o[dt][2 * r];
      dst[1] = o[dt][2 * r + 1];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < n_heads_here * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, wm[w * 16 + row]);
    float acc = 0.0f, lsum = 0.0f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(wm[w * 16 + row] - mm);
        acc += f * wacc[(w * 16 + row) * D + d];
        lsum += f * wl[w * 16 + row];
      }
    }
    const int head = head0 + row;
    if (n_splits == 1) {
      out[(long long)tok * out_stride + (long long)head * D + d] = from_f32<bf16>(acc / lsum);
    } else {
      const long long p = ((long long)blockIdx.x * n_q_heads + head) * n_splits + blockIdx.z;
      part_acc[p * D + d] = acc;
      if (d == 0) {
        part_ml[p * 2] = mm;
        part_ml[p * 2 + 1] = lsum;
      }
    }
  }
}

// ------------------------------------------------------- decode, keys by TMA
// The same kernel with keys and values brought in by the tensor memory accelerator
// (head sizes that are multiples of 64, page sizes 8, 16, 32 or 64).  The pool of one layer
// is a 2-D tensor [pages*2*kv_heads*page_size rows, D columns]; the keys (or values) of
// one page and kv head are page_size consecutive rows, so one lane issues, per page and
// 64-column half, one cp.async.bulk.tensor box with the 128-byte swizzle, and an mbarrier
// with the expected byte count tells the four warps when a 64-key stage is complete.  The
// warps hand a stage back through a second mbarrier, so there is no block-wide barrier in
// the loop and nobody spends instructions on addresses.  ldmatrix applies the swizzle
// (16-byte chunk c of row r lives at chunk c ^ (r & 7) of its 128-byte row).
constexpr int TMA_STAGES = 2;  // measured: a third stage costs a resident block per SM and 25 % of the bandwidth
constexpr int HALVES = D / 64;                                   // 64-column halves of a row
constexpr int HALF_BYTES = KV_TILE * 128;                        // 64 rows x 128 B
constexpr int TMA_STAGE_BYTES = 2 * (D >= 64 ? HALVES : 1) * HALF_BYTES;

__device__ __forceinline__ const bf16* sw_addr(const bf16* half_base, int row, int chunk) {
  return half_base + row * 64 + ((chunk ^ (row & 7)) << 3);
}

// S = Q K^T for one warp's 16 keys (rows row0..row0+15 of the stage's key halves).
__device__ __forceinline__ void qk_tile_sw(float (&s)[2][4], const bf16* sQ, const bf16* sKhalves,
                                           int row0) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) s[nt][e] = 0.0f;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t a[4], b[4];
    ldsm_x4(a, sQ + ((lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + ks * 16 + 8 * (lane >> 4));
    const int row = row0 + (lane & 7) + 8 * (lane >> 4);
    const int chunk = (ks & 3) * 2 + ((lane >> 3) & 1);
    ldsm_x4(b, sw_addr(sKhalves + (ks >> 2) * (HALF_BYTES / 2), row, chunk));
    mma_bf16(s[0], a, b[0], b[1]);
    mma_bf16(s[1], a, b[2], b[3]);
  }
}

// o += P V for one warp's 16 keys.
__device__ __forceinline__ void pv_tile_sw(float (&o)[D / 8][4], const float (&s)[2][4],
                                           const bf16* sVhalves, int row0) {
  const int lane = threadIdx.x & 31;
  uint32_t a[4];
  a[0] = pack_bf16(s[0][0], s[0][1]);
  a[1] = pack_bf16(s[0][2], s[0][3]);
  a[2] = pack_bf16(s[1][0], s[1][1]);
  a[3] = pack_bf16(s[1][2], s[1][3]);
  const int row = row0 + (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
  for (int dp = 0; dp < D / 16; ++dp) {
    uint32_t b[4];
    const int chunk = (dp & 3) * 2 + (lane >> 4);
    ldsm_x4_trans(b, sw_addr(sVhalves + (dp >> 2) * (HALF_BYTES / 2), row, chunk));
    mma_bf16(o[2 * dp], a, b[0], b[1]);
    mma_bf16(o[2 * dp + 1], a, b[2], b[3]);
  }
}

constexpr int DECODE_TMA_THREADS = THREADS + 32;  // four computing warps and a producer warp
__device__ __forceinline__ void compute_warps_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__global__ void __launch_bounds__(DECODE_TMA_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap pool_map, const bf16* __restrict__ q,
                       int q_stride, const int* __restrict__ block_table, int table_stride,
                       const int* __restrict__ cu_q, const int* __restrict__ positions,
                       const int* __restrict__ single_seqs, bf16* __restrict__ out, int out_stride,
                       float* __restrict__ part_acc, float* __restrict__ part_ml, int n_q_heads,
                       int n_kv_heads, int page_size, float scale_log2, int window, int n_splits) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // [stages, 1024-byte aligned][Q tile][barriers]
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t stages0 = (raw + 1023u) & ~1023u;
  unsigned char* stages_ptr = smem_raw + (stages0 - raw);
  bf16* sQ = reinterpret_cast<bf16*>(stages_ptr + TMA_STAGES * TMA_STAGE_BYTES);
  const uint32_t bars = stages0 + TMA_STAGES * TMA_STAGE_BYTES + 16 * STRIDE * 2;  // 8-byte aligned
  const uint32_t full0 = bars, empty0 = bars + 8 * TMA_STAGES;
  __shared__ int failed;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int group = n_q_heads / n_kv_heads;
  const int chunks_per_kv = (group + 15) / 16;
  const int kvh = blockIdx.y / chunks_per_kv;
  const int head0 = kvh * group + (blockIdx.y % chunks_per_kv) * 16;
  int n_heads_here = kvh * group + group - head0;
  if (n_heads_here > 16) n_heads_here = 16;

  // set-up that needs nothing from earlier kernels: barriers, zeroed stages (rows of pages
  // that are not loaded must hold finite numbers: they meet P = 0)
  if (tid == 0) {
    failed = 0;
    for (int st = 0; st < TMA_STAGES; ++st) {
      mbar_init(full0 + 8 * st, 1);
      mbar_init(empty0 + 8 * st, 4);  // one arrival per warp
    }
    mbar_init_fence();
  }
  // The kernels after this one (the join of the splits, then the output projection) are let in
  // at once: the projection's blocks fit beside these and fetch their first weights meanwhile
  // (measured: 1.2 % of a decode step at batch 8).
  pdl_trigger();
  // The step's batch description (positions, block tables) was copied to the device before
  // any kernel of the step began, and pages below the current position were written by earlier
  // steps: this block reads them, and fetches its first keys, BEFORE it waits for the preceding
  // kernel.  Only the tile that holds the current position (whose key and value that kernel
  // writes) and the query wait.
  const int seq = single_seqs[blockIdx.x];
  const int tok = cu_q[seq];
  const int pos = positions[tok];
  const int k_lo_all = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* table = block_table + (long long)seq * table_stride;

  const int tile_first = k_lo_all / KV_TILE, tile_end = pos / KV_TILE + 1;
  const int n_tiles_all = tile_end - tile_first;
  const int per = (n_tiles_all + n_splits - 1) / n_splits;
  const int tile_a = tile_first + blockIdx.z * per;
  int tile_b = tile_a + per;
  if (tile_b > tile_end) tile_b = tile_end;
  const int n_my = tile_b - tile_a;

  // Rows of pages that are not loaded (past the last key, or before the window) must hold
  // finite numbers, since they meet P = 0.  A stage that a complete tile filled before is
  // fine; only a stage whose FIRST tile is such a partial one is cleared here.
  for (int st = 0; st < TMA_STAGES && st < n_my; ++st) {
    const int t = tile_a + st;
    const bool partial = (t == tile_end - 1 && (pos + 1) % KV_TILE != 0) ||
                         (t == tile_first && k_lo_all % KV_TILE != 0);
    if (partial) {
      uint4* z = reinterpret_cast<uint4*>(stages_ptr + st * TMA_STAGE_BYTES);
      for (int i = tid; i < TMA_STAGE_BYTES / 16; i += DECODE_TMA_THREADS) z[i] = make_uint4(0, 0, 0, 0);
    }
  }
  fence_proxy_async_smem();
  __syncthreads();  // barriers initialised, stages zeroed

  // Warp 4 issues the boxes of tile number `i` of this block into stage i % TMA_STAGES: lane pg
  // looks up and fetches page pg of the tile, so a tile's table reads are in flight together
  // and the next tile's are under way while this one is computed.
  const int pages_per_tile = KV_TILE / page_size;
  auto lookup = [&](int i) {
    if (i >= n_my || lane >= pages_per_tile) return -1;
    const int j0 = (tile_a + i) * KV_TILE + lane * page_size;
    return (j0 <= pos && j0 + page_size - 1 >= k_lo_all) ? table[j0 / page_size] : -1;
  };
  auto issue = [&](int i, int page) {
    const int st = i % TMA_STAGES;
    const uint32_t dst0 = stages0 + st * TMA_STAGE_BYTES + lane * page_size * 128;
    const int n_boxes = __popc(__ballot_sync(0xffffffffu, page >= 0));
    if (lane == 0)
      mbar_expect_tx(full0 + 8 * st, (uint32_t)n_boxes * 2u * HALVES * page_size * 128u);
    __syncwarp();
    if (page >= 0) {
      const int krow = ((page * 2) * n_kv_heads + kvh) * page_size;
      const int vrow = krow + n_kv_heads * page_size;
#pragma unroll
      for (int h = 0; h < HALVES; ++h) {
        tma_load_2d(dst0 + h * HALF_BYTES, &pool_map, full0 + 8 * st, h * 64, krow);
        tma_load_2d(dst0 + (HALVES + h) * HALF_BYTES, &pool_map, full0 + 8 * st, h * 64, vrow);
      }
    }
  };
  if (warp == 4) {
    // The producer warp.  A tile below the current position holds keys of earlier steps and is
    // fetched at once; only the tile that holds the current position (whose key and value the
    // kernel before this one writes) waits for that kernel.
    bool waited = false;
    int page = lookup(0);
    for (int nx = 0; nx < n_my; ++nx) {
      const int page_after = lookup(nx + 1);  // under way while this tile is issued
      const int nst = nx % TMA_STAGES;
      const uint32_t nuse = (uint32_t)(nx / TMA_STAGES);
      if (tile_a + nx == tile_end - 1 && !waited) {
        pdl_wait();
        waited = true;
      }
      const bool free_now = nuse == 0 || mbar_wait_bounded(empty0 + 8 * nst, (nuse - 1) & 1u);
      if (!__all_sync(0xffffffffu, free_now)) {
        if (lane == 0) atomicExch(&failed, 1);
        break;
      }
      issue(nx, page);
      page = page_after;
    }
    return;
  }
  pdl_wait();
  // Q rows by cp.async: one per query head of the chunk, the rest zero
  if (n_my > 0) load_q_rows(sQ, q + (long long)tok * q_stride + (long long)head0 * D, D, n_heads_here, 16);
  cp_async_commit();
  cp_async_wait<0>();
  compute_warps_sync();  // Q in place

  float o[D / 8][4];
#pragma unroll
  for (int dt = 0; dt < D / 8; ++dt)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[dt][e] = 0.0f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

  bool ok = true;
  for (int i = 0; i < n_my && ok; ++i) {
    const int st = i % TMA_STAGES;
    const uint32_t use = (uint32_t)(i / TMA_STAGES);  // how often this stage was used before
    if (!mbar_wait_bounded(full0 + 8 * st, use & 1u)) {
      atomicExch(&failed, 1);
      ok = false;
      break;
    }
    const bf16* sK = reinterpret_cast<const bf16*>(stages_ptr + st * TMA_STAGE_BYTES);
    const bf16* sV = sK + HALVES * (HALF_BYTES / 2);
    const int key0 = (tile_a + i) * KV_TILE + warp * 16;
    if (key0 <= pos && key0 + 15 >= k_lo_all) {
      float s[2][4];
      qk_tile_sw(s, sQ, sK, warp * 16);
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const bool in = j <= pos && j >= k_lo_all;
          s[nt][e] = in ? s[nt][e] * scale_log2 : -INFINITY;
        }
      softmax_update<2>(s, m, l, o);
      pv_tile_sw(o, s, sV, warp * 16);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty0 + 8 * st);
  }
  compute_warps_sync();  // every warp has left the stages: the space is reused for the merge
  const bool bad = failed != 0;

  float* wm = reinterpret_cast<float*>(stages_ptr);
  float* wl = wm + 4 * 16;
  float* wacc = wl + 4 * 16;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    float lt = l[r];
    lt += __shfl_xor_sync(0xffffffffu, lt, 1);
    lt += __shfl_xor_sync(0xffffffffu, lt, 2);
    const int row = (lane >> 2) + 8 * r;
    if ((lane & 3) == 0) {
      wm[warp * 16 + row] = m[r];
      wl[warp * 16 + row] = lt;
    }
#pragma unroll
    for (int dt = 0; dt < D / 8; ++dt) {
      float* dst = wacc + ((warp * 16 + row) * D) + dt * 8 + (lane & 3) * 2;
      dst[0] = o[dt][2 * r];
      dst[1] = o[dt][2 * r + 1];
    }
  }
  compute_warps_sync();
  for (int idx = tid; idx < n_heads_here * D; idx += THREADS) {
    const int row = idx / D, d = idx - row * D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, wm[w * 16 + row]);
    float acc = 0.0f, lsum = 0.0f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(wm[w * 16 + row] - mm);
        acc += f * wacc[(w * 16 + row) * D + d];
        lsum += f * wl[w * 16 + row];
      }
    }
    if (bad) acc = __int_as_float(0x7fc00000);  // a wait ran out: make the failure visible
    const int head = head0 + row;
    if (n_splits == 1) {
      out[(long long)tok * out_stride + (long long)head * D + d] = from_f32<bf16>(acc / lsum);
    } else {
      const long long p = ((long long)blockIdx.x * n_q_heads + head) * n_splits + blockIdx.z;
      part_acc[p * D + d] = acc;
      if (d == 0) {
        part_ml[p * 2] = bad ? 0.0f : mm;
        part_ml[p * 2 + 1] = bad ? 1.0f : lsum;
      }
    }
  }
}

// grid (sequences with one token, query heads); joins the splits' partial results.
// Every load of the partial results is issued before anything waits on one: a lane per split
// fetches (m, l) and the weights exp2(m - max) are formed by warp shuffles; then each thread
// sums its column over the splits eight loads at a time.
constexpr int MERGE_MAX_SPLITS = 64;
__global__ void attn_merge_kernel(const float* __restrict__ part_acc,
                                  const float* __restrict__ part_ml,
                                  const int* __restrict__ cu_q,
                                  const int* __restrict__ single_seqs, bf16* __restrict__ out,
                                  int out_stride, int n_q_heads, int n_splits) {
  __shared__ float weight[MERGE_MAX_SPLITS];
  __shared__ float inv_l;
  const int head = blockIdx.y;
  const int tok = cu_q[single_seqs[blockIdx.x]];   // not written by any kernel of the step
  const long long base = ((long long)blockIdx.x * n_q_heads + head) * n_splits;
  pdl_wait();
  pdl_trigger();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m[MERGE_MAX_SPLITS / 32], l[MERGE_MAX_SPLITS / 32];
    float mm = -INFINITY;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      const int z = lane + 32 * i;
      const float2 ml = z < n_splits ? *reinterpret_cast<const float2*>(part_ml + (base + z) * 2)
                                     : make_float2(-INFINITY, 0.0f);
      m[i] = ml.x;
      l[i] = ml.y;
      mm = fmaxf(mm, ml.x);
    }
    mm = warp_max(mm);
    float lsum = 0.0f;
#pragma unroll
    for (int i = 0; i < MERGE_MAX_SPLITS / 32; ++i) {
      const int z = lane + 32 * i;
      const float f = m[i] == -INFINITY ? 0.0f : exp2f(m[i] - mm);   // a split with no keys weighs nothing
      if (z < n_splits) weight[z] = f;
      lsum += f * l[i];
    }
    // the sum over splits in a fixed order (a butterfly), whatever the batch
    lsum = warp_sum(lsum);
    if (lane == 0) inv_l = 1.0f / lsum;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float* col = part_acc + base * D + d;
    float acc = 0.0f;
    int z = 0;
    for (; z + 8 <= n_splits; z += 8) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = weight[z + j] != 0.0f ? col[(long long)(z + j) * D] : 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) acc += weight[z + j] * v[j];
    }
    for (; z < n_splits; ++z) acc += weight[z] != 0.0f ? weight[z] * col[(long long)z * D] : 0.0f;
    out[(long long)tok * out_stride + (long long)head * D + d] = from_f32<bf16>(acc * inv_l);
  }
}

constexpr size_t PREFILL_SMEM =
    (size_t)(Q_TILE + PF_STAGES * 2 * PF_TILE) * STRIDE * sizeof(bf16);
constexpr size_t DECODE_KV_SMEM = (size_t)4 * KV_TILE * STRIDE * sizeof(bf16);
constexpr size_t DECODE_MERGE_SMEM = (size_t)(2 * 4 * 16 + 4 * 16 * D) * sizeof(float);
constexpr size_t DECODE_TMA_SMEM =
    1024 + (size_t)TMA_STAGES * TMA_STAGE_BYTES + 16 * STRIDE * sizeof(bf16) + 16 * TMA_STAGES + 64;
constexpr size_t DECODE_SMEM =
    (size_t)16 * STRIDE * sizeof(bf16) +
    (DECODE_KV_SMEM > DECODE_MERGE_SMEM ? DECODE_KV_SMEM : DECODE_MERGE_SMEM);

}  // namespace si

SI_API int si_attn_head_dim() { return si::D; }

// Attention for the 64-query tiles listed in tile_seq/tile_start; tile_pairs holds n_pairs
// pairs of tile indices (the second may be -1), one pair per block.
SI_API int si_attn_prefill(const void* q, int q_stride, const void* pool, const int* block_table,
                           int table_stride, const int* cu_q, const int* positions,
                           const int* tile_seq, const int* tile_start, const int* tile_pairs,
                           int n_pairs, void* out, int out_stride, int n_q_heads, int n_kv_heads, int page_size,
                           float scale, int window, cudaStream_t stream) {
  if (!q || !pool || !block_table || !cu_q || !positions || !tile_seq || !tile_start ||
      !tile_pairs || !out)
    return SI_ERR_ARG;
  const int n_tiles = n_pairs;
  if (n_tiles < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 ||
      page_size <= 0 || table_stride <= 0 || q_stride % 8 != 0 || out_stride % 2 != 0)
    return SI_ERR_ARG;
  if (n_q_heads > 65535) return SI_ERR_TOO_LARGE;
  if (n_tiles == 0) return SI_OK;
  SI_ALLOW_DYNAMIC_SMEM((si::attn_prefill_kernel), (int)si::PREFILL_SMEM);
  dim3 grid(n_tiles, n_q_heads);
  SI_LAUNCH(si::attn_prefill_kernel, grid, si::THREADS, si::PREFILL_SMEM, stream,
      (const si::bf16*)q, q_stride, (const si::bf16*)pool, block_table, table_stride, cu_q,
      positions, tile_seq, tile_start, tile_pairs, (si::bf16*)out, out_stride, n_q_heads,
      n_kv_heads, page_size, scale * si::LOG2E, window);
  return SI_OK;
}

// Floats of scratch the decode path needs: part_acc then part_ml.
SI_API long long si_attn_decode_scratch_floats(int n_single, int n_q_heads, int n_splits) {
  if (n_splits <= 1) return 0;
  return (long long)n_single * n_q_heads * n_splits * (si::D + 2);
}

// Attention for the sequences listed in single_seqs (one token each).
// scratch: si_attn_decode_scratch_floats(...) floats, may be null when n_splits == 1.
// n_pages: pages in the pool (for the bounds of the tensor map).
SI_API int si_attn_decode(const void* q, int q_stride, const void* pool, int n_pages,
                          const int* block_table, int table_stride, const int* cu_q,
                          const int* positions, const int* single_seqs, int n_single, void* out,
                          int out_stride, float* scratch, int n_q_heads, int n_kv_heads,
                          int page_size, float scale, int window, int n_splits,
                          cudaStream_t stream) {
  if (!q || !pool || !block_table || !cu_q || !positions || !single_seqs || !out)
    return SI_ERR_ARG;
  if (n_single < 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads != 0 ||
      page_size <= 0 || table_stride <= 0 || q_stride % 8 != 0 || n_splits < 1)
    return SI_ERR_ARG;
  if (n_splits > 1 && !scratch) return SI_ERR_ARG;
  const int group = n_q_heads / n_kv_heads;
  const int grid_y = n_kv_heads * ((group + 15) / 16);
  if (grid_y > 65535 || n_splits > si::MERGE_MAX_SPLITS || n_q_heads > 65535) return SI_ERR_TOO_LARGE;
  if (n_single == 0) return SI_OK;
  SI_ALLOW_DYNAMIC_SMEM((si::attn_decode_kernel), (int)si::DECODE_SMEM);
  float* part_acc = scratch;
  float* part_ml = scratch ? scratch + (long long)n_single * n_q_heads * n_splits * si::D : nullptr;
  dim3 grid(n_single, grid_y, n_splits);
  // keys by TMA when the shapes allow it (see attn_decode_tma_kernel)
  const bool tma_shapes = si::D % 64 == 0 && page_size >= 8 && page_size <= 64 &&
                          (page_size & (page_size - 1)) == 0 && n_pages > 0 &&
                          (((uintptr_t)pool) & 15) == 0;
  CUtensorMap pool_map;
  if (tma_shapes &&
      si::make_bf16_map(&pool_map, pool, (long long)n_pages * 2 * n_kv_heads * page_size, si::D,
                        si::D, page_size)) {
    SI_ALLOW_DYNAMIC_SMEM((si::attn_decode_tma_kernel), (int)si::DECODE_TMA_SMEM);
    SI_LAUNCH(si::attn_decode_tma_kernel, grid, si::DECODE_TMA_THREADS, si::DECODE_TMA_SMEM, stream, pool_map,
              (const si::bf16*)q, q_stride, block_table, table_stride, cu_q, positions, single_seqs,
              (si::bf16*)out, out_stride, part_acc, part_ml, n_q_heads, n_kv_heads, page_size,
              scale * si::LOG2E, window, n_splits);
    if (n_splits > 1) {
      dim3 mgrid(n_single, n_q_heads);
      SI_LAUNCH(si::attn_merge_kernel, mgrid, si::D >= 128 ? 128 : 64, 0, stream, part_acc, part_ml,
                cu_q, single_seqs, (si::bf16*)out, out_stride, n_q_heads, n_splits);
    }
    return SI_OK;
  }
  SI_LAUNCH(si::attn_decode_kernel, grid, si::THREADS, si::DECODE_SMEM, stream,
      (const si::bf16*)q, q_stride, (const si::bf16*)pool, block_table, table_stride, cu_q,
      positions, single_seqs, (si::bf16*)out, out_stride, part_acc, part_ml, n_q_heads, n_kv_heads,
      page_size, scale * si::LOG2E, window, n_splits);
  if (n_splits > 1) {
    dim3 mgrid(n_single, n_q_heads);
    SI_LAUNCH(si::attn_merge_kernel, mgrid, si::D >= 128 ? 128 : 64, 0, stream,
        part_acc, part_ml, cu_q, single_seqs, (si::bf16*)out, out_stride, n_q_heads, n_splits);
    }
  return SI_OK;
}

// ---------------------------------------------------------------------------
// The variant that allocates nothing (declared and explained in no_alloc.h).
// ---------------------------------------------------------------------------
#include "no_alloc.h"

// In host code this name is only a handle for cudaGetSymbolAddress, never an address
// to hand to a kernel.
static __device__ __align__(256) float si_static_scratch[SI_ATTN_STATIC_SCRATCH_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_static_scratch[kMaxDevices];  // device address of si_static_scratch, per device
}  // namespace

SI_API int si_attn_decode_static(const void* q, int q_stride, const void* pool, int n_pages,
                                 const int* block_table, int table_stride, const int* cu_q,
                                 const int* positions, const int* single_seqs, int n_single,
                                 void* out, int out_stride, int n_q_heads, int n_kv_heads,
                                 int page_size, float scale, int window, int n_splits,
                                 cudaStream_t stream) {
  if (n_single < 0 || n_q_heads <= 0 || n_splits < 1) return SI_ERR_ARG;
  // each factor is bounded before the product is formed, so the product cannot wrap
  if (n_splits > 65535 || n_q_heads > 65535 || n_single > SI_ATTN_STATIC_SCRATCH_FLOATS)
    return SI_ERR_TOO_LARGE;
  if (si_attn_decode_scratch_floats(n_single, n_q_heads, n_splits) > SI_ATTN_STATIC_SCRATCH_FLOATS)
    return SI_ERR_TOO_LARGE;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return SI_ERR_TOO_LARGE;
  if (g_static_scratch[dev] == nullptr) {  // set-up, once per device, with that device current
    float* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, si_static_scratch);
    if (e != cudaSuccess) return (int)e;
    if (ptr == nullptr) return SI_ERR_ARG;
    g_static_scratch[dev] = ptr;
  }
  return si_attn_decode(q, q_stride, pool, n_pages, block_table, table_stride, cu_q, positions, single_seqs,
                        n_single, out, out_stride, g_static_scratch[dev], n_q_heads, n_kv_heads,
                        page_size, scale, window, n_splits, stream);
}
