// Plain causal grouped-query attention over the paged cache, for prompts and for decoding alike.
//
// One block per (token, query head).  The query at position p of head h uses kv head
// h / (nh / nkv) and the keys lo..p, lo = max(0, p + 1 - window) with a window, else 0
// (src/model.rs:1187-1226).  Softmax is m = max, e = exp(s - m), e / sum (src/kernels.rs:1550-1561),
// computed online over chunks of 128 keys that start at lo.  The arithmetic for one
// (token, head) is a function of its position and of the cache contents alone, so whole
// prompts, single tokens and any batch give the same bits.  Everything is float32 arithmetic;
// it is the attention of the float32 engine and the plain reference of the faster kernels.
#include "common.cuh"

constexpr int CHUNK = 128;

template <typename T>
__global__ void __launch_bounds__(CHUNK) attention_ref_kernel(
    const T* __restrict__ q, long long q_stride, T* __restrict__ out, long long out_stride,
    const T* __restrict__ kcache, const T* __restrict__ vcache, PagedKV kv, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_seq, const int* __restrict__ seq_slot, int nh, int window) {
  extern __shared__ float smem[];
  pdl_release_next();
  pdl_wait_prior();
  const int hd = kv.head_dim;
  float* qs = smem;                    // [hd]
  float* p = qs + hd;                  // [CHUNK]
  float* scratch = p + CHUNK;          // [33]
  // [CHUNK]; 8-byte aligned whatever the head size (the launcher adds the 8 bytes this may skip)
  size_t* rows = (size_t*)(((uintptr_t)(scratch + 34) + 7) & ~(uintptr_t)7);
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int g = h / (nh / kv.num_kv_heads);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int hi = pos + 1;
  const int lo = window > 0 ? max(0, hi - window) : 0;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * hd;
  for (int i = tid; i < hd; i += CHUNK) qs[i] = to_f32(qrow[i]);
  __syncthreads();
  float m = -INFINITY, l = 0.f, acc[2] = {0.f, 0.f};
  for (int c0 = lo; c0 < hi; c0 += CHUNK) {
    const int j = c0 + tid;
    float s = -INFINITY;
    if (j < hi) {
      const T* kr = kcache + kv.row(slot, j, g);
      rows[tid] = kv.vcol(slot, j, g);
      float d = 0.f;
      for (int i = 0; i < hd; ++i) d = fmaf(qs[i], to_f32(kr[i]), d);
      s = d;
    }
    const float m_new = fmaxf(m, block_max(s, scratch));
    const float pj = j < hi ? expf(s - m_new) : 0.f;
    p[tid] = pj;
    const float csum = block_sum(pj, scratch);  // also orders the writes of p and rows
    const float alpha = expf(m - m_new);
    l = l * alpha + csum;
    const int n = min(CHUNK, hi - c0);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int d = tid + u * CHUNK;
      if (d < hd) {
        float a = acc[u] * alpha;
        for (int jj = 0; jj < n; ++jj) a = fmaf(p[jj], to_f32(vcache[rows[jj] + (size_t)d * kv.page_size]), a);
        acc[u] = a;
      }
    }
    m = m_new;
    __syncthreads();
  }
  T* orow = out + (size_t)t * out_stride + (size_t)h * hd;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int d = tid + u * CHUNK;
    if (d < hd) orow[d] = from_f32<T>(acc[u] / l);
  }
}

// q: [ntok, nh, hd] rows q_stride apart (already normed, rotated, scaled); out likewise.
GB_EXPORT int gb_attention_ref(const void* q, long long q_stride, void* out, long long out_stride, int dtype,
                               const void* kcache, const void* vcache, const int* page_table, int table_width,
                               int page_size, int nkv, int hd, const int* tok_pos, const int* tok_seq,
                               const int* seq_slot, int ntok, int nh, int window, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (hd <= 0 || hd > 2 * CHUNK || nkv <= 0 || nh % nkv) return GB_ERR_SIZE;
  PagedKV kv{page_table, table_width, page_size, nkv, hd};
  const size_t smem = (size_t)(hd + CHUNK + 34) * sizeof(float) + CHUNK * sizeof(size_t) + 8;
  dim3 grid(ntok, nh);
  if (dtype == GB_F32)
    gb_launch(attention_ref_kernel<float>, grid, CHUNK, smem, stream, (const float*)q, q_stride, (float*)out, out_stride,
                                                              (const float*)kcache, (const float*)vcache, kv,
                                                              tok_pos, tok_seq, seq_slot, nh, window);
  else if (dtype == GB_BF16)
    gb_launch(attention_ref_kernel<bf16>, grid, CHUNK, smem, stream, (const bf16*)q, q_stride, (bf16*)out, out_stride,
                                                             (const bf16*)kcache, (const bf16*)vcache, kv, tok_pos,
                                                             tok_seq, seq_slot, nh, window);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}
