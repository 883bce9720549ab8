// Warp-level bfloat16 MMA helpers shared by the attention units.
#pragma once

#include "common.cuh"

// D = A * B + D for one m16n8k16 tile, float32 accumulation.  Thread (g = lane / 4, c = lane % 4):
//   A: a0 (row g, k 2c..2c+1), a1 (row g + 8, same k), a2 (row g, k 2c+8..2c+9), a3 (row g + 8, same k)
//   B: b0 (k 2c..2c+1, column g), b1 (k 2c+8..2c+9, column g)
//   D: d0, d1 (row g, columns 2c, 2c+1), d2, d3 (row g + 8, same columns)
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}
__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}
