// Tensor-map and mbarrier helpers shared by the kernels that use the tensor memory
// accelerator (TMA): encoding 2-D maps of bfloat16 matrices on the host (cached, because an
// encode costs tens of microseconds and a step asks for the same few maps again and again),
// and the device-side PTX for bulk tensor loads and bounded mbarrier waits.  All loads are
// plain tiled loads of this GPU's own memory by one block.
#pragma once

#include <cuda.h>

#include <functional>
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace si {

constexpr unsigned long long TMA_WAIT_LIMIT_NS = 1000000000ull;  // one second per wait

// ---------------------------------------------------------------------------- device
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait for the phase with the given parity; false after TMA_WAIT_LIMIT_NS.  The clock
// is read only once the barrier has been found closed a few times: reading %globaltimer costs
// hundreds of cycles, which a wait that succeeds at once (the common case in a full pipeline)
// must not pay.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done) : "r"(bar), "r"(parity) : "memory");
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
#pragma unroll 1
  for (int i = 0; i < 16; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 63u && global_ns() - t0 > TMA_WAIT_LIMIT_NS) return false;
  }
}
// x: innermost coordinate (its byte offset must be a multiple of 16), y: row
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
// five coordinates, innermost first (the innermost one's byte offset a multiple of 16)
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4) : "memory");
}
// orders earlier generic-proxy writes to shared memory before later async-proxy (TMA) writes
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ------------------------------------------------------------------------------ host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

struct MapKey {
  const void* ptr;
  long long rows;
  int cols, ld, box_rows;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = std::hash<const void*>()(k.ptr);
    for (long long v : {k.rows, (long long)k.cols, (long long)k.ld, (long long)k.box_rows})
      h = h * 1000003u + (size_t)v;
    return h;
  }
};

// Map of a rows x cols bfloat16 matrix with `ld` elements between rows, for boxes of
// box_rows x 64 columns written to shared memory with the 128-byte swizzle.
static inline bool make_bf16_map(CUtensorMap* map, const void* ptr, long long rows, int cols, int ld,
                                 int box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  static std::mutex mutex;
  const MapKey key{ptr, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> lock(mutex);
  auto it = maps.find(key);
  if (it != maps.end()) {
    *map = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * sizeof(__nv_bfloat16)};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t elem[2] = {1, 1};
  if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (maps.size() > 4096) maps.clear();
  maps.emplace(key, *map);
  return true;
}

// Map of a paged key/value pool [pages, 2, kv_heads, page_size, head_dim] (bfloat16, head_dim a
// multiple of 64, page_size a multiple of 8) that fetches a whole page of one kv head with ONE
// copy.  Its five dimensions are: 64 columns of a row; the 8 rows of a group; the head_dim/64
// column halves of a row; the 8-row groups of the pool, counted through all pages and heads;
// keys or values.  A box of (64, 8, halves, page_size/8, kv) lands in shared memory as
// [kv][group][half][8 rows x 128 bytes, swizzled]: for every column half the 8-row groups are
// halves * 1024 bytes apart, which both ldmatrix and the tcgen05 operand descriptors take.
// A copy costs the TMA unit about as much whatever its size, so a page in one copy instead of
// one per half and per K/V is what lets small pages stream at full rate.
// kv_in_box: 2 = keys and values of the page in one box (values behind keys), 1 = one of them
// per box (coordinate 4 chooses).  The row coordinate (3) of page p, head h is
// ((2 p) * kv_heads + h) * page_size / 8.
static inline bool make_page_map(CUtensorMap* map, const void* pool, long long n_pages, int n_kv_heads,
                                 int page_size, int head_dim, int kv_in_box) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> maps;
  static std::mutex mutex;
  const MapKey key{pool, n_pages, n_kv_heads, page_size * 1024 + head_dim, kv_in_box};
  std::lock_guard<std::mutex> lock(mutex);
  auto it = maps.find(key);
  if (it != maps.end()) {
    *map = it->second;
    return true;
  }
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn || head_dim % 64 != 0 || page_size % 8 != 0 || n_pages <= 0) return false;
  const cuuint64_t row_bytes = (cuuint64_t)head_dim * 2;
  const cuuint64_t kv_rows = (cuuint64_t)n_kv_heads * page_size;  // from a key row to its value row
  const cuuint64_t groups = (cuuint64_t)n_pages * 2 * kv_rows / 8;
  cuuint64_t dims[5] = {64, 8, (cuuint64_t)head_dim / 64, groups - kv_rows / 8, 2};
  cuuint64_t strides[4] = {row_bytes, 128, 8 * row_bytes, kv_rows * row_bytes};
  cuuint32_t box[5] = {64, 8, (cuuint32_t)head_dim / 64, (cuuint32_t)page_size / 8, (cuuint32_t)kv_in_box};
  cuuint32_t elem[5] = {1, 1, 1, 1, 1};
  if (fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, const_cast<void*>(pool), dims, strides, box, elem,
         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (maps.size() > 4096) maps.clear();
  maps.emplace(key, *map);
  return true;
}

}  // namespace si
