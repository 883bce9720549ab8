// Plain CUDA-core matrix product  y[t, o] = sum_i W[o, i] * x[t, i] (+ bias[o])
// (src/kernels.rs:54-57), for float32 and for bfloat16 inputs, accumulating in float32 with
// FFMA only: no tensor-core or reduced-precision matrix mode is compiled into this unit.
//
// It is the whole matrix path of the float32 engine and the plain reference of the bfloat16
// tensor-core kernels.  Every output element is accumulated by one thread over i = 0..K-1 in
// ascending order, so a row's result does not depend on how many rows the call has
// (the property the reference tests as batch invariance, src/qwen_mtp.rs:748-776).
#include "common.cuh"

enum { OUT_STORE = 0, OUT_ACCUMULATE_F32 = 1 };

constexpr int BM = 64, BN = 64, BK = 16;

template <typename TI, typename TO, int MODE>
__global__ void __launch_bounds__(256) gemm_ref_kernel(const TI* __restrict__ x, const TI* __restrict__ w,
                                                       const float* __restrict__ bias, TO* __restrict__ y, int M,
                                                       int N, int K, long long ldx, long long ldy) {
  pdl_release_next();
  pdl_wait_prior();
  __shared__ float xs[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int e = tid; e < BM * BK; e += 256) {
      const int r = e / BK, c = e % BK;
      const int gm = m0 + r, gk = k0 + c;
      xs[c][r] = (gm < M && gk < K) ? to_f32(x[(size_t)gm * ldx + gk]) : 0.f;
      const int gn = n0 + r;
      ws[c][r] = (gn < N && gk < K) ? to_f32(w[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = xs[kk][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) b[j] = ws[kk][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + tm + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tn + j;
      if (gn >= N) continue;
      float v = acc[i][j] + (bias ? bias[gn] : 0.f);
      TO* dst = y + (size_t)gm * ldy + gn;
      if (MODE == OUT_ACCUMULATE_F32)
        *dst = from_f32<TO>(to_f32(*dst) + v);
      else
        *dst = from_f32<TO>(v);
    }
  }
}

// x: [M, K] rows ldx apart; w: [N, K]; y: [M, N] rows ldy apart.
// mode OUT_STORE writes y in out_dtype; OUT_ACCUMULATE_F32 adds into a float32 y.
GB_EXPORT int gb_gemm_ref(const void* x, const void* w, int in_dtype, const float* bias, void* y, int out_dtype,
                          int mode, int M, int N, int K, long long ldx, long long ldy, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return GB_ERR_SIZE;
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (mode == OUT_ACCUMULATE_F32 && out_dtype != GB_F32) return GB_ERR_DTYPE;
#define LAUNCH(TI, TO, MODE) \
  gb_launch(gemm_ref_kernel<TI, TO, MODE>, grid, 256, 0, stream, (const TI*)x, (const TI*)w, bias, (TO*)y, M, N, K, ldx, ldy)
  if (in_dtype == GB_F32) {
    if (out_dtype != GB_F32) return GB_ERR_DTYPE;
    if (mode == OUT_ACCUMULATE_F32) LAUNCH(float, float, OUT_ACCUMULATE_F32);
    else LAUNCH(float, float, OUT_STORE);
  } else if (in_dtype == GB_BF16) {
    if (mode == OUT_ACCUMULATE_F32) LAUNCH(bf16, float, OUT_ACCUMULATE_F32);
    else if (out_dtype == GB_F32) LAUNCH(bf16, float, OUT_STORE);
    else if (out_dtype == GB_BF16) LAUNCH(bf16, bf16, OUT_STORE);
    else return GB_ERR_DTYPE;
  } else {
    return GB_ERR_DTYPE;
  }
#undef LAUNCH
  return gb_launch_status();
}
