// Prefill attention on the fifth-generation tensor cores (head sizes 128 and 64, pages of 8 to 64
// tokens): the flash-attention forward of the reference (kernels/attention_kernel.py:108-251)
// over the paged cache, with both matrix products as tcgen05.mma and their results in tensor
// memory.
//
// One block per (128-query tile of a sequence, query head); keys in tiles of 128.  Twelve
// warps (the first four, with the light roles, give registers to the eight softmax warps:
// setmaxnreg), each kind of work with a thread of its own, because a wait on an mbarrier costs the
// waiting thread some 200 cycles even when the barrier is already complete, and a thread that
// makes several such waits per tile sets the pace of the whole block:
//   warps 0 and 3      TMA producers, one for the key tiles (and the Q tile, once: two
//                      64-column halves straight from the qkv buffer), one for the value
//                      tiles: per tile the rows of its pages (one cp.async.bulk.tensor box per
//                      page: all its rows, both column halves, 128-byte swizzle; one lane per
//                      page) into a ring of slots that K and V tiles share, in the order the
//                      products need them; mbarriers count the bytes.  The block-table entries
//                      of a tile are fetched two tiles ahead (cp.async into shared memory).
//   warp 1, one lane   issues S = Q K^T (M128 N128, eight K16 steps; Q and K are K-major)
//                      into one of two S buffers in tensor memory; S(t) follows the
//                      completion of PV(t-2), which read P from the same buffer.
//   warp 2, one lane   issues PV = P V (P is read from tensor memory, where the softmax
//                      warps put it over the S it came from; V is MN-major: its rows are
//                      keys) into one of two output buffers (tiles of equal parity add up in
//                      the same one).
//   warps 4..11        softmax, in two sets of four warps, one thread per query row.  Set b
//                      owns tiles b, b+2, ...: it reads the row of S with tcgen05.ld (four
//                      loads, one wait: the softmax lies on the chain S -> P -> PV -> next S
//                      of its set), masks edge tiles by absolute position, runs the
//                      online softmax in float32 (kernels/attention_kernel.py:231-241) with
//                      two-wide fma and ex2.approx, rounds P to bfloat16 (:240) and stores it
//                      to tensor memory as the next product's A operand.  The set's output
//                      adds up in tensor memory (the products accumulate); it is rescaled
//                      only when a row's maximum has grown by more than 2^8, every term of a
//                      row staying relative to one maximum.  At the end the two sets' (m, l,
//                      O) are joined like the parts of a split, divided by l and stored.
// Every mbarrier wait is bounded; a block whose wait runs out writes NaN to its outputs.
#include "tcgen05.cuh"

#ifndef SI_HEAD_DIM
#error "compile with -DSI_HEAD_DIM=<head size>"
#endif

#if SI_HEAD_DIM == 128 || SI_HEAD_DIM == 64

namespace si {

typedef __nv_bfloat16 bf16;
constexpr int TQ = 128, TK = 128, HD = SI_HEAD_DIM;
constexpr int HALVES_TC = HD / 64;                   // 64-column halves of a row: 128 bytes each
constexpr uint32_t HALF_BYTES_TC = 128 * 128;        // 128 rows x 64 bf16
constexpr uint32_t TILE_BYTES = HALVES_TC * HALF_BYTES_TC;   // 128 x HD bf16: 32 KiB (heads of 128), 16 KiB (64)
constexpr uint32_t ROW_BYTES_TC = HD * 2;            // a row of a key or value tile
constexpr uint32_t GROUP_BYTES_TC = 8 * ROW_BYTES_TC;  // eight rows: their halves side by side
constexpr int ATC_THREADS = 384;  // key producer, S issuer, eight softmax warps, P V issuer, value producer
constexpr int PV_WARP = 2, V_WARP = 3, SOFTMAX_WARP0 = 4;  // warps 0..3: the light roles, one warpgroup
constexpr int LIGHT_REGS = 56, SOFTMAX_REGS = 224;     // 128 x 56 + 256 x 224 registers = 63 K of the SM's 64 K
constexpr int RING = HD == 128 ? 5 : 8;   // K and V tiles share one ring of slots of a tile each
constexpr uint32_t ATC_SMEM = 1024 + (1 + RING) * TILE_BYTES + 256;  // Q, the ring, barriers

// Tiles enter the ring in the order the tensor core needs them: K0, K1, V0, K2, V1, ...,
// K(n-1), V(n-2), V(n-1).
__device__ __forceinline__ int k_item(int t) { return t == 0 ? 0 : 2 * t - 1; }
__device__ __forceinline__ int v_item(int t, int n) { return t < n - 1 ? 2 * t + 2 : 2 * t + 1; }
constexpr float LOG2E_TC = 1.4426950408889634f;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(ATC_THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap q_map,
                       const __grid_constant__ CUtensorMap kv_map,
                       const int* __restrict__ block_table, int table_stride,
                       const int* __restrict__ cu_q, const int* __restrict__ positions,
                       const int* __restrict__ tile_seq, const int* __restrict__ tile_start,
                       bf16* __restrict__ out, int out_stride, int n_q_heads, int n_kv_heads,
                       int page_size, float scale_log2, int window) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t sQ = base, ring = base + TILE_BYTES;
  const uint32_t bars = base + (1 + RING) * TILE_BYTES;
  // barriers, 8 bytes each
  const uint32_t q_full = bars, s_full0 = bars + 8, p_full0 = bars + 24, o_full0 = bars + 40,
                 tmem_slot = bars + 72, slot_full0 = bars + 80,
                 slot_empty0 = slot_full0 + 8 * RING;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(base_ptr + (1 + RING) * TILE_BYTES + 72);
  __shared__ int failed;
  __shared__ int tile_pages_of[2][4][32];  // per producer warp: block-table entries of four tiles in turn, one page per lane
  __shared__ float xmax[2][2][TQ];  // [tile parity][part][row]: the two threads of a row trade maxima
  __shared__ float xsum[2][TQ];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    failed = 0;
    mbar_init(q_full, 1);
    for (int i = 0; i < RING; ++i) {
      mbar_init(slot_full0 + 8 * i, 1);
      mbar_init(slot_empty0 + 8 * i, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(s_full0 + 8 * i, 1);
      mbar_init(p_full0 + 8 * i, 4);   // the four warps of the set that owns the buffer
      mbar_init(o_full0 + 8 * i, 1);
    }
    mbar_init_fence();
  }
  // ---- this block's tile (the step's batch description was on the device before its first
  // kernel: read it before waiting for the kernel that wrote Q, K and V)
  const int tile_id = blockIdx.y;  // the host lists the longest tiles first; heads vary fastest
  const int seq = tile_seq[tile_id];
  const int tok0 = cu_q[seq] + tile_start[tile_id];
  int n_rows = cu_q[seq + 1] - tok0;
  if (n_rows > TQ) n_rows = TQ;
  const int h = blockIdx.x;
  const int kvh = h / (n_q_heads / n_kv_heads);
  const int pos0 = positions[tok0];
  const int k_hi = pos0 + n_rows - 1;
  const int k_lo = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
  const int tile_first = k_lo / TK, tile_last = k_hi / TK;
  const int n_tiles = tile_last - tile_first + 1;
  const int* table = block_table + (long long)seq * table_stride;

  // Rows of pages that are not loaded (past the last key, before the window) meet P = 0 and
  // must hold finite numbers.  A slot that an earlier tile filled does (keys and values are
  // finite); only a slot whose FIRST tile is such a partial one is cleared here.
  for (int slot = 0; slot < RING && slot < 2 * n_tiles; ++slot) {
    const int i = slot;  // the item that uses the slot first
    const bool is_v = i != 0 && ((i & 1) == 0 || i == 2 * n_tiles - 1);
    const int t = i == 0 ? 0 : (is_v ? (i == 2 * n_tiles - 1 ? n_tiles - 1 : (i - 2) / 2) : (i + 1) / 2);
    const bool partial = (t == n_tiles - 1 && (k_hi + 1) % TK != 0) || (t == 0 && k_lo % TK != 0);
    if (partial) {
      uint4* z = reinterpret_cast<uint4*>(base_ptr + TILE_BYTES + slot * TILE_BYTES);
      for (int j = threadIdx.x; j < (int)(TILE_BYTES / 16); j += ATC_THREADS) z[j] = make_uint4(0, 0, 0, 0);
    }
  }
  fence_proxy_async_smem();
  // Tensor memory is taken only after the wait on the preceding kernel: a block that is resident
  // while an earlier kernel still runs must not hold its SM's 512 columns through that wait (a
  // block of the earlier kernel that has yet to allocate there would never get them).
  pdl_wait();
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(tmem_slot), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    tmem_fence_before();
  }
  __syncthreads();
  tmem_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;
  // The softmax warps hold a row of S (128 values) and the P they make of it: the first
  // warpgroup (producers and issuers) hands them the registers it does not need.
  // (the two instructions stand at the head of the two branches below)

  // Tensor memory: S of tile t in columns [128 b, 128 b + 128) with b = t & 1; P of tile t,
  // bfloat16 pairs, over the first 64 columns of the same buffer once S has been read;
  // P V of tile t in columns [256 + 128 b, 256 + 128 b + 128).

  if (warp < SOFTMAX_WARP0) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(LIGHT_REGS));
  if (warp == 0 || warp == V_WARP) {  // ------------------------------------------ TMA producers
    // Two warps, one for the key tiles and one for the value tiles: a tile is one copy per
    // page, issued lane by lane, and one warp issuing both kinds took as long per tile as all
    // the rest of the block.  Lane i looks up and fetches page i of a tile.
    const bool my_kind_is_v = warp == V_WARP;
    int (*tile_pages)[32] = tile_pages_of[my_kind_is_v ? 1 : 0];
    if (warp == 0 && lane == 0) {
      mbar_expect_tx(q_full, TILE_BYTES);
#pragma unroll
      for (int half = 0; half < HALVES_TC; ++half)
        tma_load_2d(sQ + half * HALF_BYTES_TC, &q_map, q_full, h * HD + 64 * half, tok0);
    }
    const int pages_per_tile = TK / page_size;  // at most 16
    const int n_items = 2 * n_tiles;
    // item i: keys (odd i, and i = 0) or values of which tile
    auto tile_of = [&](int i, bool& is_v) {
      is_v = i != 0 && ((i & 1) == 0 || i == n_items - 1);
      return i == 0 ? 0 : (is_v ? (i == n_items - 1 ? n_tiles - 1 : (i - 2) / 2) : (i + 1) / 2);
    };
    // The block-table entries of tile t travel to shared memory two tiles ahead of their first
    // use (cp.async, no register waits on them): a load issued when it is needed would put a
    // trip to L2 into every item of this loop, and the loop sets the pace of the block.
    auto wanted = [&](int t) {
      const int j0 = (tile_first + t) * TK + lane * page_size;
      return lane < pages_per_tile && j0 <= k_hi && j0 + page_size - 1 >= k_lo;
    };
    auto fetch_pages = [&](int t) {
      if (t < n_tiles && wanted(t)) {
        const int j0 = (tile_first + t) * TK + lane * page_size;
        const uint32_t dst = smem_u32(&tile_pages[t & 3][lane]);
        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(table + j0 / page_size) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch_pages(0);
    fetch_pages(1);
    for (int i = 0; i < n_items; ++i) {
      const int slot = i % RING;
      bool is_v;
      const int tile = tile_of(i, is_v);
      if (is_v != my_kind_is_v) continue;
      // this warp's entries of the tile were asked for two tiles ago
      fetch_pages(tile + 2);
      asm volatile("cp.async.wait_group 2;" ::: "memory");
      const int page = wanted(tile) ? tile_pages[tile & 3][lane] : -1;
      bool ok = true;
      if (i >= RING) ok = mbar_wait_bounded(slot_empty0 + 8 * slot, ((i / RING) - 1) & 1);
      if (!__all_sync(0xffffffffu, ok)) {
        if (lane == 0) atomicExch(&failed, 1);
        break;
      }
      const int n_pages = __popc(__ballot_sync(0xffffffffu, page >= 0));
      if (lane == 0)
        mbar_expect_tx(slot_full0 + 8 * slot, (uint32_t)n_pages * page_size * ROW_BYTES_TC);
      __syncwarp();
      if (page >= 0) {
        // the page's rows of this kv head, both column halves, in one copy (see make_page_map);
        // in the slot, page i of the tile is page_size rows from page i - 1
        const uint32_t dst = ring + slot * TILE_BYTES + lane * page_size * ROW_BYTES_TC;
        const int group0 = ((page * 2) * n_kv_heads + kvh) * (page_size >> 3);
        tma_load_5d(dst, &kv_map, slot_full0 + 8 * slot, 0, 0, 0, group0, is_v ? 1 : 0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {  // ------------------------------------------------- issuer of S = Q K^T
      // Two threads issue the products, one the S = Q K^T of every tile, the other the P V:
      // a wait on a barrier costs a thread some 200 cycles even when the barrier is complete,
      // and one thread doing all four waits of a tile kept the tensor core idle half the time.
      // S(t) overwrites the buffer that P(t-2) was read from, so it follows the completion of
      // PV(t-2) (the barrier o_full of that buffer); everything else is ordered through the
      // softmax warps (s_full -> p_full).
      constexpr uint32_t idesc_s = umma_idesc(TQ, TK, false);   // Q K^T: both K-major
      bool ok = mbar_wait_bounded(q_full, 0);
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int b = t & 1;
        // the keys are usually there long before the buffer is free: that wait comes first
        const int item = k_item(t), slot = item % RING;
        if (!mbar_wait_bounded(slot_full0 + 8 * slot, (item / RING) & 1)) ok = false;
        if (ok && t >= 2 && !mbar_wait_bounded(o_full0 + 8 * b, ((t - 2) >> 1) & 1)) ok = false;
        if (!ok) break;
        tmem_fence_after();
        const uint32_t kbase = ring + slot * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {  // 16 columns of d per step; halves of 64 columns
          // Q: two half tiles of 128 rows; K: the halves of every 8-row group side by side
          const uint32_t q_off = (k >> 2) * HALF_BYTES_TC + (k & 3) * 32;
          const uint32_t k_off = (k >> 2) * 1024 + (k & 3) * 32;
          umma_bf16(tmem_base + b * 128, umma_desc(sQ + q_off), umma_desc(kbase + k_off, GROUP_BYTES_TC),
                    idesc_s, k != 0 ? 1u : 0u);
        }
        umma_commit(s_full0 + 8 * b);
        umma_commit(slot_empty0 + 8 * slot);
      }
      if (!ok) atomicExch(&failed, 1);
    }
  } else {  // warp == PV_WARP
    if (lane == 0) {  // ----------------------------------------------------- issuer of P V
      // PV(t) is issued once the softmax warps have read S(t) and written P(t) over it.
      constexpr uint32_t idesc_o = umma_idesc(TQ, HD, true);    // P V: V is MN-major
      bool ok = true;
      for (int t = 0; ok && t < n_tiles; ++t) {
        const int b = t & 1;
        const int item = v_item(t, n_tiles), slot = item % RING;
        if (!mbar_wait_bounded(slot_full0 + 8 * slot, (item / RING) & 1)) ok = false;   // values first: see above
        if (ok && !mbar_wait_bounded(p_full0 + 8 * b, (t >> 1) & 1)) ok = false;
        if (!ok) break;
        tmem_fence_after();
        const uint32_t vbase = ring + slot * TILE_BYTES;
#pragma unroll
        for (int k = 0; k < TK / 16; ++k) {  // 16 keys per step: 8 columns of packed P, two 8-row groups of V
          // the set's output adds up over its tiles (tiles b, b + 2, ...): only its first starts anew
          // V: 16 keys are two 8-row groups, a group's second column half 1024 bytes after its first
          umma_bf16_ts(tmem_base + 256 + b * 128, tmem_base + b * 128 + k * 8,
                       umma_desc_mn(vbase + k * 2 * GROUP_BYTES_TC, 1024, GROUP_BYTES_TC), idesc_o,
                       (t >= 2 || k != 0) ? 1u : 0u);
        }
        umma_commit(o_full0 + 8 * b);
        umma_commit(slot_empty0 + 8 * slot);
      }
      if (!ok) atomicExch(&failed, 1);
    }
  }
  } else {  // ------------------------------------------------------- softmax and epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(SOFTMAX_REGS));
    // Two sets of four warps; set b owns the tiles b, b + 2, ... (S buffer b, output buffer b)
    // and runs its own online softmax over them, one thread per query row, so the sets work
    // out of step and neither waits for the other until the end, where their (m, l, O) join
    // like the parts of a split.  A set's output stays in tensor memory and adds up there;
    // it is rescaled only when a row's maximum grows by more than 2^RESCALE_AT (the sums
    // stay exact: every term of a row is relative to the same stale maximum).
    constexpr float RESCALE_AT = 8.0f;
    const int quarter = warp & 3;
    const int set = (warp - SOFTMAX_WARP0) >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
    const int my_pos = pos0 + row;
    const bool row_ok = row < n_rows;
    const uint32_t s_addr = tmem_base + set * 128 + lane_off;        // S of the set's tiles, then P over it
    const uint32_t o_addr = tmem_base + 256 + set * 128 + lane_off;  // the set's output
    float m_run = -INFINITY, l_run = 0.0f;
    bool ok = true;

    for (int t = set, j = 0; t < n_tiles; t += 2, ++j) {  // j: number of the tile within the set
      const int key0 = (tile_first + t) * TK;
      // interior tiles need no mask: every key is at or before every row and inside the window
      const bool need_mask = key0 + TK - 1 > pos0 || (window > 0 && key0 <= k_hi - window);
      if (ok && !mbar_wait_bounded(s_full0 + 8 * set, j & 1)) ok = false;
      tmem_fence_after();
      auto visible = [&](int key) {
        return row_ok && key <= my_pos && (window <= 0 || key > my_pos - window);
      };
      // The whole row of S comes into registers at once (four loads, one wait): the softmax of a
      // tile lies on the chain S -> P -> P V -> next S of its set, so the latency of a
      // tensor-memory load is paid once a tile and P is worked out from the registers.
      uint32_t r0[32], r1[32], r2[32], r3[32];
      auto mask_chunk = [&](uint32_t (&r)[32], int c) {
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (!visible(key0 + c * 32 + i)) r[i] = 0xff800000u;  // -inf: never the maximum, exp2 gives 0
        }
      };
      auto max_chunk = [&](const uint32_t (&r)[32]) {
        float a = fmaxf(__uint_as_float(r[0]), __uint_as_float(r[1]));
#pragma unroll
        for (int i = 2; i < 32; i += 2) a = fmax3(a, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        return a;
      };
      tmem_ld32(s_addr, r0);
      tmem_ld32(s_addr + 32, r1);
      tmem_ld32(s_addr + 64, r2);
      tmem_ld32(s_addr + 96, r3);
      tmem_ld_wait();
      mask_chunk(r0, 0);
      mask_chunk(r1, 1);
      mask_chunk(r2, 2);
      mask_chunk(r3, 3);
      const float mx = fmaxf(fmaxf(max_chunk(r0), max_chunk(r1)), fmaxf(max_chunk(r2), max_chunk(r3)));
      const float m_new = fmaxf(m_run, mx * scale_log2);
      if (j == 0) {
        m_run = m_new;  // nothing added up yet
      } else {
        const bool grow = m_new > m_run + RESCALE_AT || (m_run == -INFINITY && m_new != -INFINITY);
        if (__any_sync(0xffffffffu, grow)) {
          // the set's previous product must have landed before its output is touched
          if (ok && !mbar_wait_bounded(o_full0 + 8 * set, (j - 1) & 1)) ok = false;
          tmem_fence_after();
          const float m_to = grow ? m_new : m_run;
          const float alpha = (m_to == -INFINITY) ? 1.0f : ex2_approx(m_run - m_to);
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(o_addr + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
            tmem_st32(o_addr + c * 32, r);
          }
          tmem_st_wait();
          l_run *= alpha;
          m_run = m_to;
        }
      }
      const float m_use = (m_run == -INFINITY) ? 0.0f : m_run;
      // P = exp2(S * scale - m), rounded to bfloat16, stored over the S it came from
      const float2 sc2 = make_float2(scale_log2, scale_log2), nm2 = make_float2(-m_use, -m_use);
      float2 acc = make_float2(0.0f, 0.0f);
      auto p_chunk = [&](const uint32_t (&r)[32], int c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          float2 x = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), sc2, nm2);
          x.x = ex2_approx(x.x);
          x.y = ex2_approx(x.y);
          acc = __fadd2_rn(acc, x);
          pk[i] = pack_bf16(x.x, x.y);
        }
        tmem_st16(s_addr + c * 16, pk);  // 32 keys = 16 packed columns
      };
      p_chunk(r0, 0);
      p_chunk(r1, 1);
      p_chunk(r2, 2);
      p_chunk(r3, 3);
      tmem_st_wait();
      tmem_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full0 + 8 * set);
      l_run += acc.x + acc.y;
    }

    // ---- join the two sets: thread (set, row) writes output columns [HD/2 set, HD/2 set + HD/2)
    xmax[0][set][row] = m_run;
    xsum[set][row] = l_run;
    const int n_mine[2] = {(n_tiles + 1) / 2, n_tiles / 2};
    for (int b = 0; b < 2; ++b)  // both sets' last products
      if (ok && n_mine[b] > 0 && !mbar_wait_bounded(o_full0 + 8 * b, (n_mine[b] - 1) & 1)) ok = false;
    tmem_fence_after();
    if (!ok) atomicExch(&failed, 1);
    asm volatile("bar.sync 1, 256;" ::: "memory");
    {
      // (tcgen05.ld is a warp-wide instruction: every lane runs the loads, rows past the tile's
      // end only skip the stores)
      const float m0 = xmax[0][0][row], m1 = xmax[0][1][row];
      const float mm = fmaxf(m0, m1);
      const bool two = n_mine[1] > 0;  // the same for the whole block
      const float w0 = (m0 == -INFINITY) ? 0.0f : ex2_approx(m0 - mm);
      const float w1 = (!two || m1 == -INFINITY) ? 0.0f : ex2_approx(m1 - mm);
      float inv = 1.0f / (xsum[0][row] * w0 + xsum[1][row] * w1);
      if (!ok || *reinterpret_cast<volatile int*>(&failed)) inv = __int_as_float(0x7fc00000);  // make it visible
      bf16* dst = out + (long long)(tok0 + row) * out_stride + (long long)h * HD + set * (HD / 2);
#pragma unroll 1
      for (int c = 0; c < HD / 64; ++c) {
        uint32_t r0[32], r1[32];
        tmem_ld32(tmem_base + 256 + lane_off + set * (HD / 2) + c * 32, r0);
        if (two) tmem_ld32(tmem_base + 384 + lane_off + set * (HD / 2) + c * 32, r1);
        tmem_ld_wait();
#pragma unroll
        for (int q8 = 0; q8 < 4; ++q8) {
          float w8[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float v = __uint_as_float(r0[q8 * 8 + i]) * w0;
            if (two && w1 != 0.0f) v += __uint_as_float(r1[q8 * 8 + i]) * w1;
            w8[i] = v * inv;
          }
          if (row_ok) store8<bf16>(dst + c * 32 + q8 * 8, w8);
        }
      }
    }
  }

  tmem_fence_before();
  __syncthreads();
  pdl_trigger();
  if (warp == 1) {
    tmem_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;"
                 ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace si

SI_API int si_attn_prefill_tc_supported() { return 1; }

// Attention for the 128-query tiles listed in tile_seq/tile_start (longest first).
// q: the qkv buffer [n_tokens, q_stride] (query heads in its first columns).
SI_API int si_attn_prefill_tc(const void* q, int q_stride, int n_tokens, const void* pool,
                              int n_pages, const int* block_table, int table_stride,
                              const int* cu_q, const int* positions, const int* tile_seq,
                              const int* tile_start, int n_tiles, void* out, int out_stride,
                              int n_q_heads, int n_kv_heads, int page_size, float scale, int window,
                              cudaStream_t stream) {
  using namespace si;
  if (!q || !pool || !block_table || !cu_q || !positions || !tile_seq || !tile_start || !out)
    return SI_ERR_ARG;
  if (n_tiles < 0 || n_tokens <= 0 || n_pages <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 ||
      n_q_heads % n_kv_heads != 0 || table_stride <= 0 || q_stride % 8 != 0 || out_stride % 8 != 0)
    return SI_ERR_ARG;
  if (page_size < 8 || page_size > 64 || (page_size & (page_size - 1)) != 0) return SI_ERR_UNSUPPORTED;
  if ((((uintptr_t)q | (uintptr_t)pool | (uintptr_t)out) & 15) != 0) return SI_ERR_ARG;
  if (n_tiles > 65535) return SI_ERR_TOO_LARGE;
  if (!(scale > 0.0f)) return SI_ERR_ARG;  // the row maximum is taken before scaling
  if (n_tiles == 0) return SI_OK;
  CUtensorMap q_map, kv_map;
  if (!make_bf16_map(&q_map, q, n_tokens, n_q_heads * HD, q_stride, TQ)) return SI_ERR_UNSUPPORTED;
  if (!make_page_map(&kv_map, pool, n_pages, n_kv_heads, page_size, HD, 1)) return SI_ERR_UNSUPPORTED;
  SI_ALLOW_DYNAMIC_SMEM((attn_prefill_tc_kernel), ATC_SMEM);
  dim3 grid(n_q_heads, n_tiles);
  SI_LAUNCH(attn_prefill_tc_kernel, grid, ATC_THREADS, ATC_SMEM, stream, q_map, kv_map, block_table,
            table_stride, cu_q, positions, tile_seq, tile_start, (bf16*)out, out_stride, n_q_heads,
            n_kv_heads, page_size, scale * LOG2E_TC, window);
  return SI_OK;
}

#else  // other head sizes: the mma.sync kernel of attention_mma.cu serves them

#include "common.cuh"
SI_API int si_attn_prefill_tc_supported() { return 0; }
SI_API int si_attn_prefill_tc(const void*, int, int, const void*, int, const int*, int, const int*,
                              const int*, const int*, const int*, int, void*, int, int, int, int,
                              float, int, cudaStream_t) {
  return SI_ERR_UNSUPPORTED;
}

#endif
