// Shared helpers of the gemmars_b200 CUDA units (sm_100a).
//
// Conventions of every unit:
//  * entry points are `extern "C"`, take raw device pointers, sizes and a stream, launch
//    asynchronously and return the cudaError_t of the launch (0 = success), or a negative
//    code for an argument they refuse;
//  * element types are passed as a code: 0 = float32, 1 = bfloat16;
//  * softmax, norms, rotation angles and residual sums are computed in float32.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define GB_EXPORT extern "C" __attribute__((visibility("default")))

enum { GB_F32 = 0, GB_BF16 = 1 };
enum { GB_ERR_DTYPE = -2, GB_ERR_SIZE = -3, GB_ERR_ARG = -4 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(bf16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads, the same value in every thread.  The order of the
// additions depends on the block size alone, never on the data or the batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// The paged cache.  Keys: [pages, kv_heads, page_size, head_dim] (a key's dims contiguous).
// Values are kept transposed inside a page: [pages, kv_heads, head_dim, page_size] (a dim's
// positions contiguous), so that both products of attention contract over the contiguous axis.
// page_table: [slots, table_width]; a ring when the sequence is longer than the table is wide.
struct PagedKV {
  const int* page_table;
  int table_width;
  int page_size;
  int num_kv_heads;
  int head_dim;
  __device__ __forceinline__ size_t row(int slot, int pos, int kv_head) const {
    const int lp = pos / page_size;
    const int page = page_table[(size_t)slot * table_width + lp % table_width];
    return (((size_t)page * num_kv_heads + kv_head) * page_size + pos % page_size) * head_dim;
  }
  // Index of dim 0 of the value at `pos`; dim d is d * page_size further.
  __device__ __forceinline__ size_t vcol(int slot, int pos, int kv_head) const {
    const int lp = pos / page_size;
    const int page = page_table[(size_t)slot * table_width + lp % table_width];
    return ((size_t)page * num_kv_heads + kv_head) * page_size * head_dim + pos % page_size;
  }
};

static inline int gb_launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch (units compiled with -DGB_PDL=1).  A kernel launched with the
// attribute may start while the kernel before it in the stream is still running; it then does
// what does not depend on that kernel (set-up, asking for its first weights) and calls
// pdl_wait_prior() before it touches anything the earlier kernel wrote, or writes anything the
// earlier kernel may still read.  pdl_release_next() lets the kernel after this one start in that
// way once every CTA of this one has called it: the small kernels call it at their start, the
// large ones when their last load is on its way (earlier, the CTAs of the kernels to come take the
// room that this kernel's own CTAs need, and the chain runs ahead by many kernels).
// Measured on the Qwen3-8B shape, decode steps replayed from a graph: +8 % tokens/s at batch 1,
// +4 % at batch 8, +-1 % at batch 64; a 2,048-token prompt gets 2 % shorter.  Each unit exists in
// two builds; the engine uses the GB_PDL=1 build inside its steps.
#ifndef GB_PDL
#define GB_PDL 0
#endif
// A unit whose kernels should never start early defines GB_PDL_EARLY_START 0 before this header.
#ifndef GB_PDL_EARLY_START
#define GB_PDL_EARLY_START GB_PDL
#endif
__device__ __forceinline__ void pdl_wait_prior() {
#if GB_PDL
  asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_release_next() {
#if GB_PDL
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

template <typename Kernel, typename... Args>
static inline void gb_launch(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = GB_PDL_EARLY_START ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<Args&&>(args)...);
}
