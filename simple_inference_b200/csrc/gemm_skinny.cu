// Matrix product for a handful of tokens (M <= 16) in bfloat16: out = X W^T with
// X [M, K] activations and W [N, K] weights in the nn.Linear layout.
//
// At these sizes the product is one pass of the weights through the SMs
// (reference: F.linear at ops/attention.py:128-130,226, ops/mlp.py:117,128 and
// ops/embedding.py:92, i.e. cuBLAS, which picks slow kernels for M <= 16), and a
// whole matrix is only a few times what the memory system holds in flight.  So the
// kernel is built to have every SM asking for weights from its first cycle to its
// last:
//
//   * A block is four warps that share 16 weight rows and split the block's k-range
//     between them, 128 k at a time, interleaved, so that the block reads each row
//     in one piece.  Every warp owns a private ring of stages in shared memory
//     (16 rows x 128 k = 4 KB a stage) that it fills with cp.async (16 bytes a
//     lane, no registers held) and drains with 16-byte shared loads laid out so
//     that a quarter warp reads 128 contiguous bytes.  A warp syncs with nobody
//     but itself until the final sum.
//   * The ring is filled BEFORE the wait on the preceding kernel (weights are never
//     written), so under programmatic dependent launch the weights of this product
//     stream in while the kernel before it (a norm, attention's join) still runs.
//   * A product runs as at most four blocks an SM (48 KB of rings each), all resident from
//     the start, each working through its share of the row tiles with its rings running on
//     from tile to tile.  The trigger for the NEXT kernel is the block's first instruction:
//     as this product's blocks leave, the next product's blocks settle in their place and
//     fill their own rings while this one still streams, so the weight stream does not stop
//     at a kernel boundary.  (Two blocks an SM, leaving half of each SM to the successor from
//     the start, was slower: a product needs the depth more than the overlap.)
//   * The k-range of the products that feed the residual stream (which the next
//     RMSNorm adds up anyway) is cut across blocks, so that a matrix of 3072 rows
//     still fills the SMs.  Partial sums go out as float32 slices
//     [splits, M, N] that the consumer adds in a fixed order.
//
// The weights are the 16-row operand of mma.sync m16n8k16 and the tokens the 8-wide
// one ("swap A and B"), so 8 tokens cost one instruction per 16 weight rows and 16 k.
// The k index inside a 32-wide step is permuted the same way for both operands (lane
// t of a row holds k = 8t..8t+7), which leaves the dot products unchanged.
//
// Epilogues: bfloat16 out; float32 out (logits); float32 partial sums; SwiGLU, where W
// is the stacked [gate; up] matrix (reference ops/mlp.py:104), a block's 16 rows are 8
// gate rows and the 8 up rows of the same outputs, and it writes silu(gate) * up
// (reference ops/mlp.py:125, kernels/swiglu_kernel.py:142-150) without the [M, 2I]
// intermediate; and, for the stacked [Wq; Wk; Wv] projection, the rotary position
// encoding with the write of keys and values into their pages (the arithmetic of
// rope_kv.cu, reference ops/rope.py:167-215 and serving/paged_kv_cache.py:171-182):
// there a block's 16 rows are 8 rows of a head's first half and the 8 rows that pair
// with them in its second half, so that both members of every rotated pair meet in one
// thread.
#include "common.cuh"

namespace si {

typedef __nv_bfloat16 bf16;
constexpr int SK_WARPS = 4;
constexpr int SK_THREADS = SK_WARPS * 32;
constexpr int SK_STAGE_K = 128;                       // k-values a warp fetches per stage
constexpr int SK_STAGE_BYTES = 16 * SK_STAGE_K * 2;   // 16 weight rows of them
constexpr int SK_STAGES = 3;                          // stages in a warp's ring: 12 KB in flight
constexpr int SK_BLOCKS_PER_SM = 4;                   // blocks of a product resident on an SM
constexpr bool SK_EARLY_TRIGGER = true;
constexpr int SK_RING_BYTES = SK_WARPS * SK_STAGES * SK_STAGE_BYTES;
constexpr int SK_MAX_SPLITS = 8;

enum SkinnyEpilogue { SK_BF16 = 0, SK_F32 = 1, SK_SWIGLU = 2, SK_ROPE = 3, SK_PARTIAL = 4 };

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

// 16 bytes from global to shared memory past the registers and L1; weights are read once, and
// L2 may fetch the row 256 bytes at a time.  bytes == 0 writes zeros and reads nothing.
__device__ __forceinline__ void cp_async_stream16(unsigned smem, const void* gmem, int bytes) {
  asm volatile("cp.async.cg.shared.global.L2::256B [%0], [%1], 16, %2;\n" ::"r"(smem), "l"(gmem),
               "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit_group() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint4 lds128(unsigned smem) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem));
  return v;
}

// Rows of W behind the 16 rows of tile `tile`: rows [0, 8) start at row_a, rows [8, 16) at row_b.
template <int EPI>
__device__ __forceinline__ void tile_rows(int tile, int N, const RopeEpilogue& rope, int& row_a,
                                          int& row_b) {
  if (EPI == SK_SWIGLU) {          // N is the output width I; W has 2 I rows, gate rows first
    row_a = tile * 8;
    row_b = N + tile * 8;
  } else if (EPI == SK_ROPE) {     // pairs 8j..8j+7 of head hh: (x_i, x_{i + D/2})
    const int half = rope.head_dim >> 1, per_head = half >> 3;
    const int hh = tile / per_head, j = tile - hh * per_head;
    row_a = hh * rope.head_dim + j * 8;
    row_b = row_a + half;
  } else {
    row_a = tile * 16;
    row_b = row_a + 8;
  }
}

// NT: n-tiles of 8 tokens (1 or 2).
// grid (blocks, k splits).  A block works on tiles blockIdx.x, blockIdx.x + gridDim.x, ... of
// the n_tiles row tiles, one after the other, with its warps' rings running on across the
// tiles.  k_per_block: a multiple of SK_WARPS * SK_STAGE_K.
template <int NT, int EPI>
__global__ void __launch_bounds__(SK_THREADS, SK_BLOCKS_PER_SM)
skinny_gemm_kernel(const bf16* __restrict__ X, int ldx, const bf16* __restrict__ W,
                   void* __restrict__ out, int ldo, int M, int N, int K, int k_per_block,
                   int n_tiles, RopeEpilogue rope) {
  extern __shared__ __align__(128) unsigned char sk_smem[];
  // two buffers for up to 8 tokens, so that a tile costs one barrier; one for 16 tokens, where
  // a second would take the fourth block's place on the SM
  constexpr int RED_BUFS = NT == 1 ? 2 : 1;
  __shared__ float red[RED_BUFS][SK_WARPS][16][NT * 8 + 1];

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n_rows_w = EPI == SK_SWIGLU ? 2 * N : N;

  // ---- this warp's stages of a tile: stage i of the warp is stage warp + i*SK_WARPS of the block
  const int k_begin = blockIdx.y * k_per_block;
  int k_end = k_begin + k_per_block;
  if (k_end > K) k_end = K;
  const int block_stages = (k_end - k_begin + SK_STAGE_K - 1) / SK_STAGE_K;
  const int my_stages = block_stages > warp ? (block_stages - warp + SK_WARPS - 1) / SK_WARPS : 0;
  const int my_tiles = (n_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int total = my_tiles * my_stages;   // stages of this warp over all its tiles

  // a lane copies 16 bytes of rows (2 it + lane/16), it = 0..7, at k-chunk lane%16 of the stage
  const int cc = lane & 15;
  const bf16* src_row[8];
  auto point_at = [&](int tile) {
    int row_a, row_b;
    tile_rows<EPI>(tile, N, rope, row_a, row_b);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 2 + (lane >> 4);
      int row = r < 8 ? row_a + r : row_b + (r - 8);
      if (row > n_rows_w - 1) row = n_rows_w - 1;   // rows past the end are read again, never stored
      src_row[it] = W + (size_t)row * K + cc * 8;
    }
  };
  const unsigned ring = (unsigned)__cvta_generic_to_shared(sk_smem) +
                        warp * (SK_STAGES * SK_STAGE_BYTES);
  // within a stage: [4 k-steps of 32][16 rows][32 k], so that lane (g, t) finds its 16 bytes of
  // rows g and g+8 of a step at g*64 + t*16 (+512): a quarter warp reads 128 contiguous bytes
  const unsigned dst_off = (cc >> 2) * 1024 + (lane >> 4) * 64 + (cc & 3) * 16;

  int f_q = 0, f_i = 0, f_tile = blockIdx.x;   // the next stage to fetch: flat index, index in its tile, tile
  auto fetch = [&]() {   // the warp's next stage into its slot of the ring
    if (f_q < total) {
      if (f_i == 0) point_at(f_tile);
      const int k0 = k_begin + (warp + f_i * SK_WARPS) * SK_STAGE_K;
      const int bytes = (k0 + cc * 8 < k_end) ? 16 : 0;   // K is a multiple of 8
      const unsigned slot = ring + (f_q % SK_STAGES) * SK_STAGE_BYTES + dst_off;
#pragma unroll
      for (int it = 0; it < 8; ++it)
        cp_async_stream16(slot + it * 128, src_row[it] + (bytes ? k0 : 0), bytes);
      ++f_q;
      if (++f_i == my_stages) {
        f_i = 0;
        f_tile += gridDim.x;
      }
    }
    cp_async_commit_group();   // an empty group keeps the count of groups uniform
  };

  // All blocks of this product are resident from the start (the grid is no larger than four
  // blocks an SM), so the kernel after it may be scheduled at once: its blocks settle where
  // this product's blocks leave and fill their own rings while the rest still run.
  if (SK_EARLY_TRIGGER) pdl_trigger();
#pragma unroll
  for (int i = 0; i < SK_STAGES; ++i) fetch();   // weights are never written: ask before waiting

  const bf16* xrow[NT];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    int tok = nt * 8 + g;
    if (tok > M - 1) tok = M - 1;
    xrow[nt] = X + (size_t)tok * ldx + t * 8;
  }
  float first_sin = 0.0f, first_cos = 1.0f;
  if (EPI == SK_ROPE) {
    // positions were on the device before the step began: the angle of this thread's pair in
    // the block's first tile is worked out while the kernel before this one finishes
    if ((int)threadIdx.x < 8 * M) {
      const int p = threadIdx.x & 7, m = threadIdx.x >> 3, per_head = rope.head_dim >> 4;
      const int i = ((int)blockIdx.x % per_head) * 8 + p;
      sincosf((float)rope.positions[m] * rope.inv_freq[i], &first_sin, &first_cos);
    }
  }
  float acc[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[nt][e] = 0.0f;

  pdl_wait();

  uint4 xb[2][4][NT];   // the tokens' part of a stage, fetched one stage ahead
  int x_i = 0;          // index in its tile of the next stage whose tokens are fetched
  auto fetch_x = [&](uint4 (&b)[4][NT]) {
    const int k0 = k_begin + (warp + x_i * SK_WARPS) * SK_STAGE_K;
    if (++x_i == my_stages) x_i = 0;
#pragma unroll
    for (int st = 0; st < 4; ++st) {
      const int k = k0 + st * 32;
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
        b[st][nt] = (k + t * 8 < k_end) ? *reinterpret_cast<const uint4*>(xrow[nt] + k)
                                        : make_uint4(0, 0, 0, 0);
    }
  };
  auto multiply = [&](const uint4 (&b)[4][NT], int q) {
    const unsigned slot = ring + (q % SK_STAGES) * SK_STAGE_BYTES + g * 64 + t * 16;
#pragma unroll
    for (int st = 0; st < 4; ++st) {
      const uint4 lo = lds128(slot + st * 1024), hi = lds128(slot + st * 1024 + 512);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mma16816(acc[nt], lo.x, hi.x, lo.y, hi.y, b[st][nt].x, b[st][nt].y);
        mma16816(acc[nt], lo.z, hi.z, lo.w, hi.w, b[st][nt].z, b[st][nt].w);
      }
    }
  };

  // ---- the end of a tile: the four warps' sums meet in shared memory, then the epilogue
  int m_i = 0, m_tile = blockIdx.x, m_j = 0;   // stage in its tile, tile, and how many tiles are done
  auto finish_tile = [&]() {
    float (*rd)[16][NT * 8 + 1] = red[m_j % RED_BUFS];
    // partial sums of this warp: rows g, g+8 of the tile, tokens 2t, 2t+1 of each n-tile
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      rd[warp][g][nt * 8 + 2 * t] = acc[nt][0];
      rd[warp][g][nt * 8 + 2 * t + 1] = acc[nt][1];
      rd[warp][g + 8][nt * 8 + 2 * t] = acc[nt][2];
      rd[warp][g + 8][nt * 8 + 2 * t + 1] = acc[nt][3];
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[nt][e] = 0.0f;
    }
    __syncthreads();
    const int tile = m_tile;
    if (EPI == SK_ROPE) {
      const int D = rope.head_dim, half = D >> 1, per_head = half >> 3;
      bf16* q_out = reinterpret_cast<bf16*>(out);
      for (int idx = threadIdx.x; idx < 8 * M; idx += SK_THREADS) {
        const int pr = idx & 7, m = idx >> 3;
        const int hh = tile / per_head, i = (tile - hh * per_head) * 8 + pr;
        float a = 0.0f, b = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) {
          a += rd[w][pr][m];
          b += rd[w][pr + 8][m];
        }
        // rounded as the separate projection rounds its output, then rotated in float32
        a = __bfloat162float(__float2bfloat16_rn(a));
        b = __bfloat162float(__float2bfloat16_rn(b));
        const bool is_q = hh < rope.n_q_heads;
        const int kv = hh - rope.n_q_heads;  // key heads, then value heads
        if (kv < rope.n_kv_heads) {
          float sn = first_sin, cs = first_cos;
          if (m_j != 0 || idx != (int)threadIdx.x)
            sincosf((float)rope.positions[m] * rope.inv_freq[i], &sn, &cs);
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
    } else if (EPI == SK_SWIGLU) {
      for (int idx = threadIdx.x; idx < 8 * M; idx += SK_THREADS) {
        const int r = idx & 7, m = idx >> 3;
        const int n = tile * 8 + r;
        if (n >= N) continue;
        float gate = 0.0f, up = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) {
          gate += rd[w][r][m];
          up += rd[w][r + 8][m];
        }
        const float act = gate / (1.0f + expf(-gate));
        reinterpret_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(act * up);
      }
    } else {
      for (int idx = threadIdx.x; idx < 16 * M; idx += SK_THREADS) {
        const int r = idx & 15, m = idx >> 4;
        const int n = tile * 16 + r;
        if (n >= N) continue;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < SK_WARPS; ++w) s += rd[w][r][m];
        if (EPI == SK_BF16) {
          reinterpret_cast<bf16*>(out)[(size_t)m * ldo + n] = __float2bfloat16_rn(s);
        } else if (EPI == SK_F32) {
          reinterpret_cast<float*>(out)[(size_t)m * ldo + n] = s;
        } else {  // SK_PARTIAL: slice blockIdx.y of [splits, M, ldo]
          reinterpret_cast<float*>(out)[((size_t)blockIdx.y * M + m) * ldo + n] = s;
        }
      }
    }
    if (RED_BUFS == 1) __syncthreads();   // everyone has read the sums before the next tile's are written
    m_tile += gridDim.x;
    ++m_j;
  };
  auto stage_done = [&]() {   // after a stage's products: hand the slot back, close the tile
    __syncwarp();             // every lane has read the slot before it is filled again
    fetch();
    if (++m_i == my_stages) {
      m_i = 0;
      finish_tile();
    }
  };

  if (total > 0) fetch_x(xb[0]);
  for (int q = 0; q < total; q += 2) {
    // two stages per trip so that the two token buffers are named at compile time
    cp_async_wait_group<SK_STAGES - 1>();
    __syncwarp();
    if (q + 1 < total) fetch_x(xb[1]);
    multiply(xb[0], q);
    stage_done();
    if (q + 1 < total) {
      cp_async_wait_group<SK_STAGES - 1>();
      __syncwarp();
      if (q + 2 < total) fetch_x(xb[0]);
      multiply(xb[1], q + 1);
      stage_done();
    }
  }
  cp_async_wait_group<0>();   // only empty groups can be pending here
  if (!SK_EARLY_TRIGGER) pdl_trigger();
  // A warp without stages of its own (a k-range shorter than the four warps' round) still has
  // to meet the others at every tile's barrier.
  if (my_stages == 0)
    for (int j = 0; j < my_tiles; ++j) finish_tile();
}

template <int NT, int EPI>
static int launch_skinny(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N,
                         int K, int splits, cudaStream_t stream, RopeEpilogue rope = RopeEpilogue()) {
  const int rows_per_tile = EPI == SK_SWIGLU ? 8 : 16;   // outputs a block's 16 weight rows make
  const int tiles = (N + rows_per_tile - 1) / rows_per_tile;
  const int unit = SK_WARPS * SK_STAGE_K;
  const int k_per_block = ((K + splits - 1) / splits + unit - 1) / unit * unit;
  if (splits > 65535) return SI_ERR_TOO_LARGE;
  // as many blocks as are resident at once; the tiles go round them in turn
  const long long resident = (long long)SK_BLOCKS_PER_SM * 148 / splits;
  const int blocks = tiles < resident ? tiles : (int)(resident < 1 ? 1 : resident);
  SI_ALLOW_DYNAMIC_SMEM((skinny_gemm_kernel<NT, EPI>), SK_RING_BYTES);
  SI_LAUNCH((skinny_gemm_kernel<NT, EPI>), dim3(blocks, splits), SK_THREADS, SK_RING_BYTES, stream,
            (const bf16*)X, ldx, (const bf16*)W, out, ldo, M, N, K, k_per_block, tiles, rope);
  return SI_OK;
}

}  // namespace si

// How many slices of partial sums si_gemm_skinny_bf16 writes for epilogue 4 at these sizes:
// as many k-ranges as still let every block of the product be resident at once (four blocks
// an SM), each range no shorter than one round of the four warps.
SI_API int si_gemm_skinny_splits(int N, int K) {
  using namespace si;
  if (N <= 0 || K <= 0) return 1;
  const int tiles = (N + 15) / 16;
  int splits = (SK_BLOCKS_PER_SM * 148) / tiles;
  const int most = K / (SK_WARPS * SK_STAGE_K);
  if (splits > most) splits = most;
  if (splits > SK_MAX_SPLITS) splits = SK_MAX_SPLITS;
  return splits < 1 ? 1 : splits;
}

// out[M, N] = X[M, K] W[N, K]^T for M <= 16.  epilogue 0: bfloat16 out, 1: float32 out,
// 2: SwiGLU (W has 2*N rows, gate rows first; out is bfloat16 [M, N]), 4: float32 partial
// sums, out is [splits, M, ldo] with splits = si_gemm_skinny_splits(N, K), to be added up
// in order of the slices.
// K must be a multiple of 8; X rows, W and ldx must keep 16-byte alignment.
SI_API int si_gemm_skinny_bf16(const void* X, int ldx, const void* W, void* out, int ldo, int M,
                               int N, int K, int epilogue, cudaStream_t stream) {
  if (!X || !W || !out || M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N) return SI_ERR_ARG;
  if (M > 16 || K % 8 != 0 || ldx % 8 != 0) return SI_ERR_UNSUPPORTED;
  if (((uintptr_t)X | (uintptr_t)W) & 15) return SI_ERR_ARG;
  if (M == 0) return SI_OK;
  using namespace si;
  const int splits = epilogue == SK_PARTIAL ? si_gemm_skinny_splits(N, K) : 1;
  if (M <= 8) {
    if (epilogue == SK_BF16) return launch_skinny<1, SK_BF16>(X, ldx, W, out, ldo, M, N, K, 1, stream);
    if (epilogue == SK_F32) return launch_skinny<1, SK_F32>(X, ldx, W, out, ldo, M, N, K, 1, stream);
    if (epilogue == SK_SWIGLU) return launch_skinny<1, SK_SWIGLU>(X, ldx, W, out, ldo, M, N, K, 1, stream);
    if (epilogue == SK_PARTIAL) return launch_skinny<1, SK_PARTIAL>(X, ldx, W, out, ldo, M, N, K, splits, stream);
  } else {
    if (epilogue == SK_BF16) return launch_skinny<2, SK_BF16>(X, ldx, W, out, ldo, M, N, K, 1, stream);
    if (epilogue == SK_F32) return launch_skinny<2, SK_F32>(X, ldx, W, out, ldo, M, N, K, 1, stream);
    if (epilogue == SK_SWIGLU) return launch_skinny<2, SK_SWIGLU>(X, ldx, W, out, ldo, M, N, K, 1, stream);
    if (epilogue == SK_PARTIAL) return launch_skinny<2, SK_PARTIAL>(X, ldx, W, out, ldo, M, N, K, splits, stream);
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
  if (M <= 8) return launch_skinny<1, SK_ROPE>(X, ldx, W, qkv, ldo, M, N, K, 1, stream, rope);
  return launch_skinny<2, SK_ROPE>(X, ldx, W, qkv, ldo, M, N, K, 1, stream, rope);
}
