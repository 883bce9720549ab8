// tcgen05 / TMA / mbarrier helpers shared by the tensor-core units (sm_100a).
//
// Device side: inline PTX for mbarriers (with a bounded wait), TMA tile loads, tensor memory
// and tcgen05.mma, and the shared-memory matrix descriptor of a K-major, 128-byte-swizzled
// tile.  Host side: tensor maps for row-major bfloat16 matrices cut into [rows, 64] boxes and for
// result matrices, encoded through the driver entry point (no link against libcuda) and
// remembered by key.
// No load here uses cluster multicast.
#pragma once

#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace {

// Polls of an mbarrier before a wait gives up.  A test build may shorten it
// (-DGB_TEST_WAIT_LIMIT=n) so that a wait which nothing completes runs out in microseconds.
#ifdef GB_TEST_WAIT_LIMIT
constexpr uint32_t WAIT_LIMIT = GB_TEST_WAIT_LIMIT;
#else
constexpr uint32_t WAIT_LIMIT = 1u << 22;
#endif
constexpr int TC_BOX_COLS = 64;             // 64 bfloat16 = one 128-byte swizzle row

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; false when the limit ran out (the caller records it and leaves its loop).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}
// A tile of shared memory to global memory through a tensor map: stored, or added (the map's type:
// float32).  The requests of a thread form groups; tma_store_wait_read<N> returns when all but the
// last N groups have been read out of shared memory, tma_store_wait_all when they are all written.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_add_2d(const CUtensorMap* map, const void* src, int x, int y) {
  asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// What this thread wrote to shared memory becomes visible to TMA (the asynchronous proxy).
__device__ __forceinline__ void fence_smem_to_tma() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t cluster_size() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// A float to the same place in the shared memory of CTA `rank` of the cluster, its 4 bytes counted
// on the mbarrier at `local_bar`'s place in that CTA: the receiver waits for the bytes it expects
// instead of for a barrier of the whole cluster.
__device__ __forceinline__ void st_peer_f32_counted(float* local, uint32_t rank, float v, uint64_t* local_bar) {
  uint32_t addr, bar;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(smem_u32(local_bar)), "r"(rank));
  asm volatile("st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.b32 [%0], %1, [%2];"
               ::"r"(addr), "r"(__float_as_uint(v)), "r"(bar) : "memory");
}
// Shared-memory matrix descriptor of a K-major tile with 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3ffff) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}

// ------------------------------------------------------------------ host side: tensor maps
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_fn() {
  static EncodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiled)p;
  });
  return fn;
}

struct MapKey {
  const void* base;
  uint64_t rows, cols, pitch;
  uint32_t box_rows, kind;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && pitch == o.pitch && box_rows == o.box_rows && kind == o.kind;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = (size_t)k.base;
    for (uint64_t v : {k.rows, k.cols, k.pitch, (uint64_t)k.box_rows, (uint64_t)k.kind}) h = h * 1000003u ^ (size_t)v;
    return h;
  }
};

// Maps are remembered: weights and reused activation buffers are encoded once.
bool tensor_map_any(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch, uint32_t box_rows,
                    uint32_t box_cols, CUtensorMapDataType type, CUtensorMapSwizzle swizzle, uint32_t kind) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{base, rows, cols, pitch, box_rows, kind};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  EncodeTiled fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {pitch};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t elem[2] = {1, 1};
  if (fn(out, type, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
    return false;
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// A [rows, cols] bfloat16 matrix with rows `pitch` bytes apart, cut into [box_rows, 64] boxes
// (operands of the products: 128-byte swizzle).
bool tensor_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch, uint32_t box_rows) {
  return tensor_map_any(out, base, rows, cols, pitch, box_rows, TC_BOX_COLS, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                        CU_TENSOR_MAP_SWIZZLE_128B, 0);
}

// A [rows, cols] result matrix (bfloat16 or float32) written in [piece_rows, piece_cols] pieces
// (up to TC_OUT_ROWS x TC_OUT_COLS) that lie row after row in shared memory.  False when TMA
// cannot address it (base and pitch must be multiples of 16 bytes): the caller then stores with
// plain instructions.
constexpr int TC_OUT_ROWS = 32, TC_OUT_COLS = 32;
bool tensor_map_out(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch, uint32_t piece_rows,
                    uint32_t piece_cols, bool f32) {
  if (((uintptr_t)base & 15) || (pitch & 15) || piece_rows > (uint32_t)TC_OUT_ROWS || piece_cols > (uint32_t)TC_OUT_COLS ||
      (piece_cols * (f32 ? 4 : 2)) % 16)
    return false;
  return tensor_map_any(out, base, rows, cols, pitch, piece_rows, piece_cols,
                        f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                        CU_TENSOR_MAP_SWIZZLE_NONE, (f32 ? 2 : 1) | (piece_cols << 4));
}

}  // namespace
