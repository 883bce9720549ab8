// bfloat16 causal grouped-query attention of whole prompts (or chunks of them) over the paged
// cache: the prefill kernel.  Compiled for one head size (-DGB_HEAD_DIM=...).
//
// Same mathematics as the decode kernel (src/model.rs:1187-1226, src/kernels.rs:1550-1561) and
// the same way of feeding the tensor cores straight from the cache (keys contiguous in the
// dims, values contiguous in the positions; see attention_decode.cu).  Here the 16 rows of an
// MMA are 16 consecutive tokens of one sequence for one query head, each row masked at its own
// position (and window).  A CTA covers 64 tokens of one sequence and up to two query heads
// that share a kv head: 4 x 2 warps that read the same keys and values, which the L1 cache
// then serves.  The step's keys are already in the cache when this runs, so a token sees the
// earlier tokens of its own step there.
#include "mma.cuh"

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 128
#endif

namespace {

constexpr int HD = GB_HEAD_DIM;
constexpr int KEYS = 32;
constexpr int TILE = 64;        // tokens per CTA
constexpr int MT = TILE / 16;   // row groups of 16 tokens
constexpr int RH = 2;           // query heads per CTA at most
constexpr float LOG2E = 1.4426950408889634f;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");

// grid (token tiles upper bound, kv heads * head chunks); block MT * heads_per_cta * 32.
__global__ void __launch_bounds__(MT * RH * 32)
attention_prefill_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                         const bf16* __restrict__ kcache, const bf16* __restrict__ vcache, PagedKV kv,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                         const int* __restrict__ seq_slot, int n_seqs, int nh, int window, int heads_per_cta) {
  pdl_release_next();
  pdl_wait_prior();
  // ---- which sequence and which 64-token tile of it
  int b = 0, tile = blockIdx.x;
  for (; b < n_seqs; ++b) {
    const int tiles = (cu_seqlens[b + 1] - cu_seqlens[b] + TILE - 1) / TILE;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (b >= n_seqs) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int mt = warp % MT, hr = warp / MT;
  const int rep = nh / kv.num_kv_heads;
  const int chunks = (rep + heads_per_cta - 1) / heads_per_cta;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int hl = chunk * heads_per_cta + hr;          // head within the kv group
  if (hl >= rep) return;
  const int head = kvh * rep + hl;
  const int seq_len = cu_seqlens[b + 1] - cu_seqlens[b];
  const int first = tile * TILE + mt * 16;            // first token of this warp within the sequence's step
  if (first >= seq_len) return;
  const int slot = seq_slot[b], start = seq_start[b];
  const int tok0 = cu_seqlens[b] + first;
  const bool v0 = first + g < seq_len, v1 = first + g + 8 < seq_len;
  const int pos0 = v0 ? start + first + g : -1, pos1 = v1 ? start + first + g + 8 : -1;   // -1: no key passes
  const int last = start + min(first + 15, seq_len - 1);                                    // last position of the warp
  const int lo_first = window > 0 ? max(0, start + first + 1 - window) : 0;
  const int lo0 = window > 0 ? max(0, pos0 + 1 - window) : 0, lo1 = window > 0 ? max(0, pos1 + 1 - window) : 0;

  constexpr int KB = HD / 32, TAIL = HD % 32;
  uint32_t qa[KB + 1][4], qb[KB + 1][4];
  {
    const bf16* q0 = q + (size_t)(tok0 + g) * q_stride + (size_t)head * HD;
    const bf16* q1 = q0 + 8 * q_stride;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      uint4 a = v0 ? *(const uint4*)(q0 + kb * 32 + c * 8) : make_uint4(0, 0, 0, 0);
      qa[kb][0] = a.x; qa[kb][1] = a.y; qa[kb][2] = a.z; qa[kb][3] = a.w;
      uint4 bb = v1 ? *(const uint4*)(q1 + kb * 32 + c * 8) : make_uint4(0, 0, 0, 0);
      qb[kb][0] = bb.x; qb[kb][1] = bb.y; qb[kb][2] = bb.z; qb[kb][3] = bb.w;
    }
    if (TAIL) {
      uint2 a = v0 ? *(const uint2*)(q0 + KB * 32 + c * 4) : make_uint2(0, 0);
      qa[KB][0] = a.x; qa[KB][1] = a.y;
      uint2 bb = v1 ? *(const uint2*)(q1 + KB * 32 + c * 4) : make_uint2(0, 0);
      qb[KB][0] = bb.x; qb[KB][1] = bb.y;
    }
  }

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  for (int blk = lo_first / KEYS; blk * KEYS <= last; ++blk) {
    const int key0 = blk * KEYS;
    const int page = kv.page_table[(size_t)slot * kv.table_width + (key0 / kv.page_size) % kv.table_width];
    const size_t page_base = ((size_t)page * kv.num_kv_heads + kvh) * kv.page_size * HD;
    const int in_page = key0 % kv.page_size;
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      const bf16* krow = kcache + page_base + (size_t)(in_page + 8 * (g >> 1) + 2 * j + (g & 1)) * HD;
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        const uint4 k4 = *(const uint4*)(krow + kb * 32 + c * 8);
        mma16816(s[j], qa[kb][0], qb[kb][0], qa[kb][1], qb[kb][1], k4.x, k4.y);
        mma16816(s[j], qa[kb][2], qb[kb][2], qa[kb][3], qb[kb][3], k4.z, k4.w);
      }
      if (TAIL) {
        const uint2 k2 = *(const uint2*)(krow + KB * 32 + c * 4);
        mma16816(s[j], qa[KB][0], qb[KB][0], qa[KB][1], qb[KB][1], k2.x, k2.y);
      }
    }
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + 8 * c + 2 * j + e;
        s[j][e] = (key >= lo0 && key <= pos0) ? s[j][e] * LOG2E : -INFINITY;
        s[j][2 + e] = (key >= lo1 && key <= pos1) ? s[j][2 + e] * LOG2E : -INFINITY;
        mx0 = fmaxf(mx0, s[j][e]);
        mx1 = fmaxf(mx1, s[j][2 + e]);
      }
    const float n0 = fmaxf(m0, quad_max(mx0)), n1 = fmaxf(m1, quad_max(mx1));
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;
    const float alpha0 = exp2f(m0 - u0), alpha1 = exp2f(m1 - u1);
    m0 = n0;
    m1 = n1;
    uint32_t p[4][2];
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = exp2f(s[j][0] - u0), bb = exp2f(s[j][1] - u0);
      const float cc = exp2f(s[j][2] - u1), d = exp2f(s[j][3] - u1);
      sum0 += a + bb;
      sum1 += cc + d;
      p[j][0] = pack_bf16(a, bb);
      p[j][1] = pack_bf16(cc, d);
    }
    l0 = l0 * alpha0 + sum0;
    l1 = l1 * alpha1 + sum1;
    const bf16* vbase = vcache + page_base + in_page + 8 * c;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      const uint4 v4 = *(const uint4*)(vbase + (size_t)(d * 8 + g) * kv.page_size);
      o[d][0] *= alpha0; o[d][1] *= alpha0; o[d][2] *= alpha1; o[d][3] *= alpha1;
      mma16816(o[d], p[0][0], p[0][1], p[1][0], p[1][1], v4.x, v4.y);
      mma16816(o[d], p[2][0], p[2][1], p[3][0], p[3][1], v4.z, v4.w);
    }
  }
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  if (v0) {
    const float inv = 1.0f / l0;
    bf16* dst = out + (size_t)(tok0 + g) * out_stride + (size_t)head * HD + 2 * c;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) *(uint32_t*)(dst + d * 8) = pack_bf16(o[d][0] * inv, o[d][1] * inv);
  }
  if (v1) {
    const float inv = 1.0f / l1;
    bf16* dst = out + (size_t)(tok0 + g + 8) * out_stride + (size_t)head * HD + 2 * c;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) *(uint32_t*)(dst + d * 8) = pack_bf16(o[d][2] * inv, o[d][3] * inv);
  }
}

}  // namespace

// q, out: [ntok, nh * HD] bfloat16, tokens of all sequences packed (cu_seqlens: [n_seqs + 1]);
// seq_start: cache length of each sequence before this step; the cache already holds this
// step's keys and values.  q rows and out rows must be 16-byte / 4-byte aligned.
GB_EXPORT int gb_attention_prefill(const void* q, long long q_stride, void* out, long long out_stride,
                                   const void* kcache, const void* vcache, const int* page_table, int table_width,
                                   int page_size, int nkv, int hd, const int* cu_seqlens, const int* seq_start,
                                   const int* seq_slot, int n_seqs, int ntok, int nh, int window,
                                   cudaStream_t stream) {
  if (ntok <= 0 || n_seqs <= 0) return 0;
  if (hd != HD || nkv <= 0 || nh % nkv || page_size % KEYS) return GB_ERR_SIZE;
  if (((uintptr_t)q & 15) || (q_stride % 8) || ((uintptr_t)out & 3) || (out_stride % 2) || ((uintptr_t)kcache & 15) ||
      ((uintptr_t)vcache & 15))
    return GB_ERR_SIZE;
  PagedKV kv{page_table, table_width, page_size, nkv, hd};
  const int rep = nh / nkv;
  const int heads_per_cta = rep < RH ? rep : RH;
  const int chunks = (rep + heads_per_cta - 1) / heads_per_cta;
  dim3 grid((ntok + TILE - 1) / TILE + n_seqs, nkv * chunks);
  gb_launch(attention_prefill_kernel, grid, MT * heads_per_cta * 32, 0, stream,
      (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache, kv, cu_seqlens,
      seq_start, seq_slot, n_seqs, nh, window, heads_per_cta);
  return gb_launch_status();
}
