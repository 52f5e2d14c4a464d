// bfloat16 matrix product on pairs of SMs: out = X W^T as in gemm_tc.cu, but every output tile
// is 256 rows tall and belongs to a cluster of two blocks whose tensor cores work as one
// (tcgen05.mma.cta_group::2).  Block r of the pair holds rows [128 r, 128 r + 128) of the X
// tile and half of the tile's weight rows in its own shared memory; the instruction reads both
// halves, so per output element each SM fetches about a third less from L2 than with
// 128-row tiles, which is what bounds the one-block kernel on large products.  (The reference
// calls cuBLAS for these products: F.linear, ops/attention.py:128-130,226; ops/mlp.py:117,128.)
//
// Roles per block (192 threads), as in gemm_tc.cu:
//   warp 0, one lane   TMA producer: its block's 128 x 64 tile of X and (BN/2) x 64 tile of W
//                      per 64 columns of K, two such pairs per stage of a three-stage ring.  Both blocks' loads report their
//                      bytes to the FIRST block's `full` barrier (cp.async.bulk.tensor with
//                      .cta_group::2); no load is a multicast.
//   warp 1, one lane   in the first block only: the MMA issuer.  Four tcgen05.mma (M256 N=BN
//                      K16) per 64 columns; tcgen05.commit with a two-block mask frees the stage
//                      in both blocks, and after the last k-step tells both epilogues.
//   warps 2..5         epilogue of the block's own 128 rows (its own tensor memory); all
//                      eight epilogue warps of the pair hand the accumulator back to the
//                      first block's barrier.
// SwiGLU: the first block loads the 128 gate rows of a tile, the second the 128 up rows, so
// the accumulator has g in columns [0, 128) and u in [128, 256) as in gemm_tc.cu.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in *status, and
// the block goes on to the closing cluster barrier, frees its tensor memory and returns.
#include <cstdlib>

#include "tcgen05.cuh"

namespace si {

typedef __nv_bfloat16 bf16;

constexpr int T2_BM = 128;            // rows per block; a tile has 2 * T2_BM
constexpr int T2_BK = 64;     // columns of one TMA box (a 128-byte swizzled row)
constexpr int T2_SUB = 2;     // boxes along K per stage: one barrier round per 128 columns (measured: a
                              // 2048-token prefill takes 12.9 ms with 3 stages of 2 boxes, 13.9 ms with
                              // 6 of 1, 13.7 ms with 2 of 3)
constexpr int T2_STAGES = 3;
constexpr int T2_THREADS = 192;
constexpr uint32_t T2_A_BYTES = T2_BM * T2_BK * 2;   // 16 KiB
constexpr uint32_t T2_B_BYTES = 128 * T2_BK * 2;     // 16 KiB reserved: half of at most 256 weight rows
constexpr uint32_t T2_SUB_BYTES = T2_A_BYTES + T2_B_BYTES;
constexpr uint32_t T2_STAGE_BYTES = T2_SUB * T2_SUB_BYTES;
constexpr uint32_t T2_TMEM_COLS = 512;
constexpr uint32_t T2_SMEM_BYTES = T2_STAGES * T2_STAGE_BYTES + 1024 + 256;

enum { T2_EPI_BF16 = 0, T2_EPI_SWIGLU = 2, T2_EPI_PARTIAL = 4 };
constexpr int T2_MAX_SPLITS = 8;
enum { T2_TIMEOUT_PRODUCER = 1, T2_TIMEOUT_MMA = 2, T2_TIMEOUT_EPILOGUE = 3 };

__device__ __forceinline__ bool t2_wait(uint32_t bar, uint32_t parity, int* status, int code) {
  if (mbar_wait_bounded(bar, parity)) return true;
  atomicCAS(status, 0, code);
  return false;
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// the address, in the cluster's shared window, of `addr` in the block of rank `rank`
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
// tiled load into this block's shared memory whose bytes are counted by a barrier that may lie
// in the partner block (`bar` is an address in the cluster's shared window)
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
// arrives, once the products issued so far are done, at `bar` (same offset) in both blocks
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3) : "memory");
}

template <int EPI, int BN>
__global__ void __launch_bounds__(T2_THREADS, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                void* __restrict__ out_any, int ldo, int M, int n_out, int K, int up_row0, int splits,
                int* __restrict__ status) {
  bf16* const out = reinterpret_cast<bf16*>(out_any);
  constexpr int TILE_N_OUT = (EPI == T2_EPI_SWIGLU) ? BN / 2 : BN;
  constexpr uint32_t STAGE_TX_BYTES = 2 * (T2_A_BYTES + (BN / 2) * T2_BK * 2);  // both blocks' loads
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + T2_STAGES * T2_STAGE_BYTES;
  // full[stages], empty[stages], acc_full[2], acc_empty[2], then the tensor-memory slot
  const uint32_t full0 = bars, empty0 = bars + 8 * T2_STAGES;
  const uint32_t acc_full0 = bars + 16 * T2_STAGES, acc_empty0 = acc_full0 + 16;
  const uint32_t tmem_slot = acc_empty0 + 16;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int tiles_m = (M + 2 * T2_BM - 1) / (2 * T2_BM);
  const int tiles_n = (n_out + TILE_N_OUT - 1) / TILE_N_OUT;
  const int n_tiles = tiles_m * tiles_n;
  const int k_boxes = (K + T2_BK - 1) / T2_BK;
  const int k_blocks = (k_boxes + T2_SUB - 1) / T2_SUB;  // stages per tile
  // A unit is (tile, k-range): unit u works on tile u % n_tiles over stages [kb0, kb1) of part
  // u / n_tiles.  One part (splits == 1) unless the epilogue writes partial sums.
  const int n_units = n_tiles * splits;
  auto part_of = [&](int u, int& tile, int& kb0, int& kb1) {
    tile = u % n_tiles;
    const int part = u / n_tiles;
    kb0 = (int)((long long)part * k_blocks / splits);
    kb1 = (int)((long long)(part + 1) * k_blocks / splits);
    return part;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < T2_STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);   // used in the first block: its producer's arrival plus all bytes
      mbar_init(empty0 + 8 * s, 1);  // one commit, delivered to both blocks
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 8);  // used in the first block: the pair's eight epilogue warps
    }
    mbar_init_fence();
  }
  // Tensor memory is taken only AFTER the wait on the preceding kernel.  A block of this kernel
  // may be resident while the kernel before it still runs; holding all 512 columns of its SM
  // through that wait starves any block of an earlier kernel that has yet to allocate there
  // (seen as a stall of whole steps with long prompt portions beside decoded tokens).
  pdl_wait();
  if (warp == 1) {  // one warp of each block: the pair's tensor memory is allocated together
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(tmem_slot), "r"(T2_TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    tmem_fence_before();
  }
  __syncthreads();
  cluster_sync();  // both blocks' barriers exist before either signals the other's
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  if (warp == 0) {
    if (lane == 0) {  // ---------------------------------------------- TMA producer
      const uint32_t full_first = map_to_rank(full0, 0);  // the first block counts the bytes
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair; ok && u < n_units; u += n_pairs) {
        int tile, kb0, kb1;
        part_of(u, tile, kb0, kb1);
        const int m0 = (tile % tiles_m) * 2 * T2_BM + rank * T2_BM;  // m fastest: neighbours share W
        const int n0 = (tile / tiles_m) * TILE_N_OUT;
        const int w_row = (EPI == T2_EPI_SWIGLU) ? (rank == 0 ? n0 : up_row0 + n0)
                                                 : n0 + (int)rank * (BN / 2);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % T2_STAGES, ph = (it / T2_STAGES) & 1u;
          if (!t2_wait(empty0 + 8 * s, ph ^ 1u, status, T2_TIMEOUT_PRODUCER)) { ok = false; break; }
          const int nsub = k_boxes - kb * T2_SUB < T2_SUB ? k_boxes - kb * T2_SUB : T2_SUB;
          if (rank == 0) mbar_expect_tx(full0 + 8 * s, STAGE_TX_BYTES * nsub);
          for (int j = 0; j < nsub; ++j) {
            const uint32_t a_dst = base + s * T2_STAGE_BYTES + j * T2_SUB_BYTES, b_dst = a_dst + T2_A_BYTES;
            tma_load_2d_pair(a_dst, &map_x, full_first + 8 * s, (kb * T2_SUB + j) * T2_BK, m0);
            tma_load_2d_pair(b_dst, &map_w, full_first + 8 * s, (kb * T2_SUB + j) * T2_BK, w_row);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {  // ------------------------------------ MMA issuer
      constexpr uint32_t idesc = umma_idesc(2 * T2_BM, BN);
      uint32_t it = 0, acc_it = 0;
      bool ok = true;
      for (int u = pair; ok && u < n_units; u += n_pairs, ++acc_it) {
        int tile, kb0, kb1;
        part_of(u, tile, kb0, kb1);
        const uint32_t buf = acc_it & 1u, aph = (acc_it >> 1) & 1u;
        if (!t2_wait(acc_empty0 + 8 * buf, aph ^ 1u, status, T2_TIMEOUT_MMA)) break;
        tmem_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const uint32_t s = it % T2_STAGES, ph = (it / T2_STAGES) & 1u;
          if (!t2_wait(full0 + 8 * s, ph, status, T2_TIMEOUT_MMA)) { ok = false; break; }
          tmem_fence_after();
          const int nsub = k_boxes - kb * T2_SUB < T2_SUB ? k_boxes - kb * T2_SUB : T2_SUB;
          for (int j = 0; j < nsub; ++j) {
            const uint32_t a_src = base + s * T2_STAGE_BYTES + j * T2_SUB_BYTES;
            const uint64_t da = umma_desc(a_src), db = umma_desc(a_src + T2_A_BYTES);
#pragma unroll
            for (int k = 0; k < T2_BK / 16; ++k)
              umma_bf16_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb != kb0 || (j | k) != 0) ? 1u : 0u);
          }
          umma_commit_pair(empty0 + 8 * s);
        }
        if (ok) umma_commit_pair(acc_full0 + 8 * buf);
      }
    }
    if (lane == 0) pdl_trigger();
  } else {  // ------------------------------------------------------------ epilogue
    const int quarter = warp & 3;
    const uint32_t acc_empty_first = map_to_rank(acc_empty0, 0);
    uint32_t acc_it = 0;
    for (int u = pair; u < n_units; u += n_pairs, ++acc_it) {
      int tile, kb0, kb1;
      const int part = part_of(u, tile, kb0, kb1);
      const uint32_t buf = acc_it & 1u, aph = (acc_it >> 1) & 1u;
      if (!t2_wait(acc_full0 + 8 * buf, aph, status, T2_TIMEOUT_EPILOGUE)) break;
      tmem_fence_after();
      const int m0 = (tile % tiles_m) * 2 * T2_BM + rank * T2_BM, n0 = (tile / tiles_m) * TILE_N_OUT;
      const int row = m0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + buf * 256 + ((uint32_t)(quarter * 32) << 16);
      bf16* orow = out + (size_t)row * ldo + n0;
      if (EPI == T2_EPI_SWIGLU) {
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
      } else if (EPI == T2_EPI_PARTIAL) {
        // float32 partial sums of this k-range into slice `part` of out[splits][M][ldo]
        float* prow = reinterpret_cast<float*>(out_any) + ((size_t)part * M + row) * ldo + n0;
#pragma unroll 1
        for (int c = 0; c < TILE_N_OUT / 16; ++c) {
          uint32_t a[16];
          tmem_ld16(taddr + c * 16, a);
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = n0 + c * 16 + j * 4;
              if (col < n_out)   // n_out is a multiple of 8
                *reinterpret_cast<float4*>(prow + c * 16 + j * 4) =
                    make_float4(__uint_as_float(a[j * 4]), __uint_as_float(a[j * 4 + 1]),
                                __uint_as_float(a[j * 4 + 2]), __uint_as_float(a[j * 4 + 3]));
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < TILE_N_OUT / 32; ++c) {
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
      if (lane == 0) mbar_arrive_cluster(acc_empty_first + 8 * buf);
    }
  }

  // Neither block may leave while its partner can still reach into its shared memory
  // (operand reads, barrier arrivals) or tensor memory.
  tmem_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"(T2_TMEM_COLS) : "memory");
  }
}

// Tile width on n_pairs persistent pairs: a multiple of 16 (each block holds half of the weight
// rows, in whole 8-row swizzle groups) that spreads the tiles evenly and wastes little of the
// last tile.  The time of a tile grows with its width, so a narrower tile that fills the last
// round is better than a wide one that leaves pairs idle.
static int choose_bn2(int M, int N, int n_pairs) {
  const int tiles_m = (M + 2 * T2_BM - 1) / (2 * T2_BM);
  int best = 256;
  double best_score = -1.0;
  for (int bn = 256; bn >= 128; bn -= 16) {
    const long long tiles = (long long)tiles_m * ((N + bn - 1) / bn);
    const long long per_pair = (tiles + n_pairs - 1) / n_pairs;
    const double balance = (double)tiles / ((double)per_pair * n_pairs);
    const double used = (double)N / ((double)((N + bn - 1) / bn) * bn);
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
static int launch_tc2(const CUtensorMap& map_x, const CUtensorMap& map_w, void* out, int ldo, int M,
                      int N, int K, int up_row0, int splits, int* status, int n_sms,
                      cudaStream_t stream) {
  SI_ALLOW_DYNAMIC_SMEM((gemm_tc2_kernel<EPI, BN>), T2_SMEM_BYTES);
  constexpr int tile_n = EPI == T2_EPI_SWIGLU ? BN / 2 : BN;
  const long long n_units =
      (long long)((M + 2 * T2_BM - 1) / (2 * T2_BM)) * ((N + tile_n - 1) / tile_n) * splits;
  int pairs = n_sms / 2;
  if (pairs > n_units) pairs = (int)n_units;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(T2_THREADS);
  cfg.dynamicSmemBytes = T2_SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<EPI, BN>, map_x, map_w, out, ldo, M, N, K,
                                     up_row0, splits, status);
  return e == cudaSuccess ? SI_OK : (int)e;
}

}  // namespace si

// The product of gemm_tc.cu's si_gemm_tc_bf16 (same arguments and conditions) on pairs of SMs.
SI_API int si_gemm_tc2_bf16(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N,
                            int K, int epilogue, int* status, cudaStream_t stream) {
  using namespace si;
  if (!X || !W || !out || !status || M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N)
    return SI_ERR_ARG;
  if (K % 8 != 0 || N % 8 != 0 || ldx % 8 != 0 || ldo % 8 != 0) return SI_ERR_UNSUPPORTED;
  if (((uintptr_t)X | (uintptr_t)W | (uintptr_t)out) & 15) return SI_ERR_ARG;
  if (epilogue != T2_EPI_BF16 && epilogue != T2_EPI_SWIGLU) return SI_ERR_ARG;
  if (M == 0) return SI_OK;
  static int n_sms = 0;
  if (n_sms == 0) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
  }
  if (n_sms < 2) return SI_ERR_UNSUPPORTED;
  CUtensorMap map_x, map_w;
  if (!make_bf16_map(&map_x, X, M, K, ldx, T2_BM)) return SI_ERR_UNSUPPORTED;
  if (epilogue == T2_EPI_SWIGLU) {
    if (!make_bf16_map(&map_w, W, 2 * N, K, K, 128)) return SI_ERR_UNSUPPORTED;
    return launch_tc2<T2_EPI_SWIGLU, 256>(map_x, map_w, out, ldo, M, N, K, N, 1, status, n_sms,
                                          stream);
  }
  const int bn = choose_bn2(M, N, n_sms / 2);
  if (!make_bf16_map(&map_w, W, N, K, K, bn / 2)) return SI_ERR_UNSUPPORTED;
#define SI_T2_CASE(W)                                                                          \
  case W:                                                                                      \
    return launch_tc2<T2_EPI_BF16, W>(map_x, map_w, out, ldo, M, N, K, 0, 1, status, n_sms, \
                                      stream)
  switch (bn) {
    SI_T2_CASE(256);
    SI_T2_CASE(240);
    SI_T2_CASE(224);
    SI_T2_CASE(208);
    SI_T2_CASE(192);
    SI_T2_CASE(176);
    SI_T2_CASE(160);
    SI_T2_CASE(144);
    default:
      return launch_tc2<T2_EPI_BF16, 128>(map_x, map_w, out, ldo, M, N, K, 0, 1, status, n_sms,
                                          stream);
  }
#undef SI_T2_CASE
}

// Into how many k-ranges si_gemm_tc2_partial should cut the product of M rows, N weight rows and
// K columns, for a consumer that adds float32 slices anyway (the RMSNorm after a projection
// that feeds the residual stream).  With few rows a product has fewer 256 x 256 tiles than the
// GPU has pairs of SMs, and one tile's pass over K bounds its time; cutting K fills the pairs.
// Every further range costs a float32 slice of M x N that is written and read again.  Returns
// 1 where cutting does not pay: the caller then takes the ordinary product.
SI_API int si_gemm_tc2_splits(int M, int N, int K) {
  using namespace si;
  if (M <= 0 || N <= 0 || K <= 0) return 1;
  int dev = 0, n_sms = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms < 2)
    return 1;
  const int pairs = n_sms / 2;
  const long long tiles = (long long)((M + 2 * T2_BM - 1) / (2 * T2_BM)) * ((N + 255) / 256);
  const int stages = ((K + T2_BK - 1) / T2_BK + T2_SUB - 1) / T2_SUB;
  // microseconds: a stage of a 256-wide tile, a unit's fixed cost, and the slices' way through
  // L2 and the norm (bytes / 2.5 TB/s, once written and once read)
  const double t_stage = 0.75, t_unit = 2.5;
  int best = 1;
  double best_time = 1e30;
  for (int s = 1; s <= T2_MAX_SPLITS && stages / s >= 2; ++s) {
    const long long rounds = (tiles * s + pairs - 1) / pairs;
    double t = (double)rounds * ((double)((stages + s - 1) / s) * t_stage + t_unit);
    if (s > 1) t += 2.0 * (double)s * M * N * 4.0 / 2.5e6;
    if (t < best_time - 1e-9) {
      best_time = t;
      best = s;
    }
  }
  return best;
}

// float32 partial sums of X[M, K] W[N, K]^T over `splits` k-ranges: out[splits][M][ldo], slice p
// holding range p, to be added in order.  Same conditions as si_gemm_tc2_bf16; ldo a multiple of 4.
SI_API int si_gemm_tc2_partial(const void* X, int ldx, const void* W, void* out, int ldo, int M, int N,
                               int K, int splits, int* status, cudaStream_t stream) {
  using namespace si;
  if (!X || !W || !out || !status || M < 0 || N <= 0 || K <= 0 || ldx < K || ldo < N || splits < 1)
    return SI_ERR_ARG;
  if (K % 8 != 0 || N % 8 != 0 || ldx % 8 != 0 || ldo % 4 != 0) return SI_ERR_UNSUPPORTED;
  if (splits > T2_MAX_SPLITS) return SI_ERR_TOO_LARGE;
  if (((uintptr_t)X | (uintptr_t)W | (uintptr_t)out) & 15) return SI_ERR_ARG;
  if (M == 0) return SI_OK;
  int dev = 0, n_sms = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return (int)e;
  if (n_sms < 2) return SI_ERR_UNSUPPORTED;
  const int stages = ((K + T2_BK - 1) / T2_BK + T2_SUB - 1) / T2_SUB;
  if (splits > stages) return SI_ERR_ARG;   // every slice must get at least one stage
  CUtensorMap map_x, map_w;
  if (!make_bf16_map(&map_x, X, M, K, ldx, T2_BM)) return SI_ERR_UNSUPPORTED;
  if (!make_bf16_map(&map_w, W, N, K, K, 128)) return SI_ERR_UNSUPPORTED;
  return launch_tc2<T2_EPI_PARTIAL, 256>(map_x, map_w, out, ldo, M, N, K, 0, splits, status, n_sms,
                                         stream);
}
