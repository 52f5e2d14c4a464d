// bfloat16 matrix product on the fifth-generation tensor cores: out = X W^T with
// X [M, K] activations and W [N, K] weights (nn.Linear layout), float32
// accumulation in tensor memory.  It serves every product with many rows
// (prompt portions); the reference calls cuBLAS for them (F.linear,
// ops/attention.py:128-130,226; ops/mlp.py:117,128).
//
// One persistent block per SM walks over 128 x 256 output tiles.  Roles:
//   warp 0, one lane   TMA producer: cp.async.bulk.tensor loads of a 128 x 64 tile
//                      of X and a 256 x 64 tile of W per k-step into a four-stage
//                      ring of 128-byte-swizzled shared memory; mbarriers with
//                      expected byte counts say when a stage is full.  Loads are
//                      plain tiled loads of this GPU's own memory, one per block.
//   warp 1, one lane   MMA issuer: four tcgen05.mma (M128 N256 K16, kind::f16,
//                      operands by shared-memory descriptor) per k-step into one
//                      of two 256-column accumulators in tensor memory;
//                      tcgen05.commit frees the stage, and after the last k-step
//                      tells the epilogue that the accumulator is complete.
//   warps 2..5         epilogue: each warp reads its 32 lanes of the accumulator
//                      with tcgen05.ld, rounds once to bfloat16 and stores; then
//                      hands the accumulator back.  With two accumulators the
//                      epilogue of one tile overlaps the products of the next.
//
// Epilogue 2 (SwiGLU): W is the stacked [gate; up] matrix (reference
// ops/mlp.py:104).  A tile's 256 weight rows are 128 gate rows and the 128 up
// rows of the same output columns (two TMA boxes), so the epilogue has g and u
// of an output side by side in tensor memory and writes silu(g) * u (reference
// ops/mlp.py:125) without ever storing the [M, 2I] intermediate.
//
// Every wait on an mbarrier is bounded.  If one runs out, the block records a
// code in *status, stops issuing work, still meets its final barrier, frees its
// tensor memory and returns; the host reads *status and raises.
#include "tcgen05.cuh"

namespace si {

typedef __nv_bfloat16 bf16;

constexpr int TC_BM = 128, TC_BN_MAX = 256, TC_BK = 64, TC_STAGES = 4;
constexpr int TC_THREADS = 192;
constexpr uint32_t TC_A_BYTES = TC_BM * TC_BK * 2;       // 16 KiB
constexpr uint32_t TC_B_BYTES = TC_BN_MAX * TC_BK * 2;   // 32 KiB reserved; a narrower tile fills less
constexpr uint32_t TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr uint32_t TC_TMEM_COLS = 512;                   // two accumulators of up to 256 columns
constexpr uint32_t TC_SMEM_BYTES = TC_STAGES * TC_STAGE_BYTES + 1024 /*alignment*/ + 256 /*barriers*/;

enum TcStatus { TC_OK = 0, TC_TIMEOUT_PRODUCER = 1, TC_TIMEOUT_MMA = 2, TC_TIMEOUT_EPILOGUE = 3 };
enum TcEpilogue { TC_EPI_BF16 = 0, TC_EPI_SWIGLU = 2 };

// ------------------------------------------------------------------ PTX helpers
// (mbarrier and TMA helpers are in tma.cuh)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_wait_bounded(bar, parity)) return true;
  atomicCAS(status, 0, code);
  return false;
}
// ----------------------------------------------------------------------- kernel
// n_out: output columns (N, or I for SwiGLU).  up_row0: first up row of W (I) for SwiGLU.
// BN: weight rows (accumulator columns) per tile, a multiple of 16 up to 256.
template <int EPI, int BN>
__global__ void __launch_bounds__(TC_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
               bf16* __restrict__ out, int ldo, int M, int n_out, int K, int up_row0,
               int* __restrict__ status) {
  constexpr int TILE_N_OUT = (EPI == TC_EPI_SWIGLU) ? BN / 2 : BN;
  constexpr uint32_t STAGE_TX_BYTES = TC_A_BYTES + BN * TC_BK * 2;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + TC_STAGES * TC_STAGE_BYTES;
  // barrier addresses (8 bytes each): full[4], empty[4], acc_full[2], acc_empty[2]; then the TMEM slot
  const uint32_t full0 = bars, empty0 = bars + 8 * TC_STAGES;
  const uint32_t acc_full0 = bars + 16 * TC_STAGES, acc_empty0 = acc_full0 + 16;
  const uint32_t tmem_slot = acc_empty0 + 16;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + TC_BM - 1) / TC_BM;
  const int tiles_n = (n_out + TILE_N_OUT - 1) / TILE_N_OUT;
  const int n_tiles = tiles_m * tiles_n;
  const int k_blocks = (K + TC_BK - 1) / TC_BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);  // one arrival per epilogue warp
    }
    mbar_init_fence();
  }
  // The inputs must be complete, and only then is tensor memory taken: a block that is resident
  // while the kernel before it still runs must not hold its SM's 512 columns through the wait
  // (a block of an earlier kernel that has yet to allocate there would never get them).
  pdl_wait();
  if (warp == 1) {  // the whole warp allocates tensor memory, and later frees it
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(tmem_slot), "r"(TC_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tmem_fence_before();
  }
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {  // ---------------------------------------------- TMA producer
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
        const int m0 = (tile % tiles_m) * TC_BM;       // m fastest: neighbours share the W tile
        const int n0 = (tile / tiles_m) * TILE_N_OUT;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % TC_STAGES, ph = (it / TC_STAGES) & 1u;
          if (!mbar_wait(empty0 + 8 * s, ph ^ 1u, status, TC_TIMEOUT_PRODUCER)) { ok = false; break; }
          const uint32_t a_dst = base + s * TC_STAGE_BYTES, b_dst = a_dst + TC_A_BYTES;
          mbar_expect_tx(full0 + 8 * s, STAGE_TX_BYTES);
          tma_load_2d(a_dst, &map_x, full0 + 8 * s, kb * TC_BK, m0);
          if (EPI == TC_EPI_SWIGLU) {
            tma_load_2d(b_dst, &map_w, full0 + 8 * s, kb * TC_BK, n0);
            tma_load_2d(b_dst + BN * TC_BK, &map_w, full0 + 8 * s, kb * TC_BK, up_row0 + n0);
          } else {
            tma_load_2d(b_dst, &map_w, full0 + 8 * s, kb * TC_BK, n0);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ------------------------------------------------ MMA issuer
      constexpr uint32_t idesc = umma_idesc(TC_BM, BN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x, ++acc_it) {
        const uint32_t buf = acc_it & 1u, aph = (acc_it >> 1) & 1u;
        if (!mbar_wait(acc_empty0 + 8 * buf, aph ^ 1u, status, TC_TIMEOUT_MMA)) break;
        tmem_fence_after();
        const uint32_t d_tmem = tmem_base + buf * TC_BN_MAX;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t s = it % TC_STAGES, ph = (it / TC_STAGES) & 1u;
          if (!mbar_wait(full0 + 8 * s, ph, status, TC_TIMEOUT_MMA)) { ok = false; break; }
          tmem_fence_after();
          const uint32_t a_src = base + s * TC_STAGE_BYTES;
          const uint64_t da = umma_desc(a_src), db = umma_desc(a_src + TC_A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)  // 16 columns = 32 bytes further along each row
            umma_bf16(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
          umma_commit(empty0 + 8 * s);  // the stage is free once these products have read it
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);
      }
      pdl_trigger();  // this block has issued all its products
    }
  } else {  // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;  // a warp may read lanes [32*(warp%4), +32) of tensor memory
    uint32_t acc_it = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++acc_it) {
      const uint32_t buf = acc_it & 1u, aph = (acc_it >> 1) & 1u;
      if (!mbar_wait(acc_full0 + 8 * buf, aph, status, TC_TIMEOUT_EPILOGUE)) break;
      tmem_fence_after();
      const int m0 = (tile % tiles_m) * TC_BM, n0 = (tile / tiles_m) * TILE_N_OUT;
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + buf * TC_BN_MAX + ((uint32_t)(quarter * 32) << 16);
      bf16* orow = out + (size_t)row * ldo + n0;
      if (EPI == TC_EPI_SWIGLU) {
#pragma unroll 1
        for (int c = 0; c < TILE_N_OUT / 32; ++c) {
          uint32_t g[32], u[32];
          float v[32];
          tmem_ld32(taddr + c * 32, g);
          tmem_ld32(taddr + BN / 2 + c * 32, u);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float gi = __uint_as_float(g[i]);
            v[i] = (gi / (1.0f + expf(-gi))) * __uint_as_float(u[i]);
          }
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = n0 + c * 32 + j * 8;
              if (col < n_out) {  // n_out is a multiple of 8
                float w8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) w8[i] = v[j * 8 + i];
                store8<bf16>(orow + c * 32 + j * 8, w8);
              }
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < TILE_N_OUT / 32; ++c) {  // two 16-column loads in flight per turn
          uint32_t a[16], b[16];
          tmem_ld16(taddr + c * 32, a);
          tmem_ld16(taddr + c * 32 + 16, b);
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = n0 + c * 32 + j * 8;
              if (col < n_out) {
                float w8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i)
                  w8[i] = __uint_as_float(j < 2 ? a[j * 8 + i] : b[(j - 2) * 8 + i]);
                store8<bf16>(orow + c * 32 + j * 8, w8);
              }
            }
          }
        }
        if (TILE_N_OUT % 32 != 0) {  // a last half-width chunk of 16 columns
          constexpr int c0 = TILE_N_OUT / 32 * 32;
          uint32_t a[16];
          tmem_ld16(taddr + c0, a);
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
              const int col = n0 + c0 + j * 8;
              if (col < n_out) {
                float w8[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) w8[i] = __uint_as_float(a[j * 8 + i]);
                store8<bf16>(orow + c0 + j * 8, w8);
              }
            }
          }
        }
      }
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty0 + 8 * buf);
    }
  }

  tmem_fence_before();
  __syncthreads();
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"(TC_TMEM_COLS) : "memory");
  }
}

// ------------------------------------------------------------------------- host
static bool make_map(CUtensorMap* map, const void* ptr, int rows, int cols, int ld, int box_rows) {
  return make_bf16_map(map, ptr, rows, cols, ld, box_rows);
}

// Tile width for an [M, N] output on n_sms persistent blocks: the widest tile is the most
// efficient per tile, but the blocks finish together only if the tile count divides well.
// Score = (mean tiles per block / most tiles of a block) * a mild preference for wide tiles.
static int choose_bn(int M, int N, int n_sms) {
  const int tiles_m = (M + TC_BM - 1) / TC_BM;
  int best = 256;
  double best_score = -1.0;
  for (int bn = 256; bn >= 128; bn -= 16) {
    const long long tiles = (long long)tiles_m * ((N + bn - 1) / bn);
    const long long per_block = (tiles + n_sms - 1) / n_sms;
    const double balance = (double)tiles / ((double)per_block * n_sms);
    const double used = (double)N / ((double)((N + bn - 1) / bn) * bn);  // part of the tiles inside N
    // a narrower tile re-reads X more often per product: about 1% per 16 columns below 256
    const double width = 1.0 - 0.01 * (256 - bn) / 16;
    const double score = balance * used * width;
    if (score > best_score + 1e-9) {
      best_score = score;
      best = bn;
    }
  }
  return best;
}

template <int EPI, int BN>
static int launch_tc(const CUtensorMap& map_x, const CUtensorMap& map_w, bf16* out, int ldo, int M,
                     int N, int K, int up_row0, int* status, int n_sms, cudaStream_t stream) {
  SI_ALLOW_DYNAMIC_SMEM((gemm_tc_kernel<EPI, BN>), TC_SMEM_BYTES);
  constexpr int tile_n = EPI == TC_EPI_SWIGLU ? BN / 2 : BN;
  const int n_tiles = ((M + TC_BM - 1) / TC_BM) * ((N + tile_n - 1) / tile_n);
  const int grid = n_tiles < n_sms ? n_tiles : n_sms;
  SI_LAUNCH((gemm_tc_kernel<EPI, BN>), grid, TC_THREADS, TC_SMEM_BYTES, stream, map_x, map_w, out,
            ldo, M, N, K, up_row0, status);
  return SI_OK;
}

}  // namespace si

// out[M, N] = X[M, K] W[N, K]^T in bfloat16 (epilogue 0), or out[M, N] = silu(X Wg^T) * (X Wu^T)
// with W = [Wg; Wu] of 2N rows (epilogue 2).  K and N multiples of 8, ldx and ldo multiples of 8,
// all pointers 16-byte aligned.  status: one int in device memory, 0 while all is well.
SI_API int si_gemm_tc_bf16(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N,
                           int K, int epilogue, int* status, cudaStream_t stream) {
  using namespace si;
  if (!X || !W || !out || !status || M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N)
    return SI_ERR_ARG;
  if (K % 8 != 0 || N % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) return SI_ERR_UNSUPPORTED;
  if (((uintptr_t)X | (uintptr_t)W | (uintptr_t)out) & 15) return SI_ERR_ARG;
  if (epilogue != TC_EPI_BF16 && epilogue != TC_EPI_SWIGLU) return SI_ERR_ARG;
  if (M == 0) return SI_OK;
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
  }
  CUtensorMap map_x, map_w;
  if (!make_map(&map_x, X, M, K, ldx, TC_BM)) return SI_ERR_UNSUPPORTED;
  if (epilogue == TC_EPI_SWIGLU) {
    if (!make_map(&map_w, W, 2 * N, K, K, 128)) return SI_ERR_UNSUPPORTED;
    return launch_tc<TC_EPI_SWIGLU, 256>(map_x, map_w, (bf16*)out, ldo, M, N, K, N, status, n_sms,
                                         stream);
  }
  const int bn = choose_bn(M, N, n_sms);
  if (!make_map(&map_w, W, N, K, K, bn)) return SI_ERR_UNSUPPORTED;
#define SI_TC_CASE(W)                                                                         \
  case W:                                                                                     \
    return launch_tc<TC_EPI_BF16, W>(map_x, map_w, (bf16*)out, ldo, M, N, K, 0, status, n_sms, \
                                     stream)
  switch (bn) {
    SI_TC_CASE(256);
    SI_TC_CASE(240);
    SI_TC_CASE(224);
    SI_TC_CASE(208);
    SI_TC_CASE(192);
    SI_TC_CASE(176);
    SI_TC_CASE(160);
    SI_TC_CASE(144);
    default:
      return launch_tc<TC_EPI_BF16, 128>(map_x, map_w, (bf16*)out, ldo, M, N, K, 0, status, n_sms,
                                         stream);
  }
#undef SI_TC_CASE
}
