// bfloat16 grouped-query attention of single query positions over the paged cache, split along
// the keys: the decode kernel.  Compiled for one head size (-DGB_HEAD_DIM=...).
//
// For the query at position p of head h (kv head g = h / (nh / nkv)): s_j = q . K[j] for the keys
// lo..p, softmax (m = max, e = exp(s - m), e / sum; src/kernels.rs:1550-1561), o = sum p_j V[j]
// (src/model.rs:1187-1226).  The query is already normed, rotated and scaled.
//
// A CTA serves one token, one kv head (all the query heads that share it, up to 16 at a time)
// and one contiguous share of the keys; its warps take blocks of 32 keys in turn.  Keys and
// values go from global memory straight into tensor-core fragments: both products contract
// over the axis that is contiguous in the cache (dims for q.K, positions for p.V, values being
// stored transposed inside a page), so each thread's 16-byte load is eight consecutive elements
// of the contraction and the MMA's inner index is simply assigned to them in that order, on
// both operands alike.  The keys of a block are assigned to MMA columns so that the scores a
// thread gets are the ones it needs as the p.V operand: no shuffles, no shared memory in the loop.
//
// Each CTA leaves (m, l, o) per head in scratch; a second kernel merges the shares in order.
// With one share the first kernel writes the result itself.
// These kernels never start under the kernel before them: measured, the step got slower when the
// attention CTAs, one to an SM, moved in early (batch 8: -6 %, batch 64: -14 %).
#define GB_PDL_EARLY_START 0
#include "mma.cuh"

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 128
#endif

namespace {

constexpr int HD = GB_HEAD_DIM;
constexpr int WARPS = 8;
constexpr int KEYS = 32;                       // keys per block
constexpr float LOG2E = 1.4426950408889634f;
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");

// grid (shares, kv heads * head chunks, tokens); block WARPS * 32.
// part_o: [tokens, nh, shares, HD]; part_ml: [tokens, nh, shares, 2] (m in log2 units, l).
template <bool UPPER>   // UPPER: more than 8 query heads per chunk (rows 8..15 of the MMA in use)
__global__ void __launch_bounds__(WARPS * 32, 1)
attention_decode_kernel(const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out, long long out_stride,
                        const bf16* __restrict__ kcache, const bf16* __restrict__ vcache, PagedKV kv,
                        const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                        const int* __restrict__ seq_slot, int nh, int window, float* __restrict__ part_o,
                        float* __restrict__ part_ml, int rows_per_chunk) {
  extern __shared__ float smem[];
  pdl_wait_prior();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const int shares = gridDim.x, share = blockIdx.x;
  const int rep = nh / kv.num_kv_heads;
  const int chunks = (rep + rows_per_chunk - 1) / rows_per_chunk;
  const int kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks;
  const int t = blockIdx.z;
  const int head0 = kvh * rep + chunk * rows_per_chunk;                 // first query head of this CTA
  const int rows = min(rows_per_chunk, rep - chunk * rows_per_chunk);    // query heads of this CTA
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int hi = pos + 1;
  const int lo = window > 0 ? max(0, hi - window) : 0;
  const int blk_first = lo / KEYS, blk_end = (hi + KEYS - 1) / KEYS;
  const int nblk = blk_end - blk_first;
  const int b_begin = blk_first + (int)((long long)nblk * share / shares);
  const int b_end = blk_first + (int)((long long)nblk * (share + 1) / shares);

  // ---- the query fragments: row g (and g + 8) of the MMA = query head head0 + g (+ 8)
  constexpr int KB = HD / 32, TAIL = HD % 32;     // 32-dim blocks, and a 16-dim tail
  uint32_t qa[KB + 1][4], qb[KB + 1][4];           // qb: rows 8..15
  {
    const bf16* q0 = q + (size_t)t * q_stride + (size_t)(head0 + g) * HD;
    const bool v0 = g < rows, v1 = UPPER && (g + 8 < rows);
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      uint4 a = v0 ? *(const uint4*)(q0 + kb * 32 + c * 8) : make_uint4(0, 0, 0, 0);
      qa[kb][0] = a.x; qa[kb][1] = a.y; qa[kb][2] = a.z; qa[kb][3] = a.w;
      uint4 b = v1 ? *(const uint4*)(q0 + 8 * HD + kb * 32 + c * 8) : make_uint4(0, 0, 0, 0);
      qb[kb][0] = b.x; qb[kb][1] = b.y; qb[kb][2] = b.z; qb[kb][3] = b.w;
    }
    if (TAIL) {
      uint2 a = v0 ? *(const uint2*)(q0 + KB * 32 + c * 4) : make_uint2(0, 0);
      qa[KB][0] = a.x; qa[KB][1] = a.y;
      uint2 b = v1 ? *(const uint2*)(q0 + 8 * HD + KB * 32 + c * 4) : make_uint2(0, 0);
      qb[KB][0] = b.x; qb[KB][1] = b.y;
    }
  }

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8; m in log2 units
  float o[HD / 8][4];
#pragma unroll
  for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

  // the page of a block is looked up one block ahead, so that the lookup's round trip to memory
  // runs under the block before and not in front of this block's loads
  const int* table_row = kv.page_table + (size_t)slot * kv.table_width;
  int next_page = b_begin + warp < b_end ? table_row[((b_begin + warp) * KEYS / kv.page_size) % kv.table_width] : 0;
  for (int blk = b_begin + warp; blk < b_end; blk += WARPS) {
    const int key0 = blk * KEYS;
    const int page = next_page;
    if (blk + WARPS < b_end) next_page = table_row[((blk + WARPS) * KEYS / kv.page_size) % kv.table_width];
    const size_t page_base = ((size_t)page * kv.num_kv_heads + kvh) * kv.page_size * HD;
    const int in_page = key0 % kv.page_size;
    // ---- the block's values are asked for now, before the scores are computed: their loads are
    // in flight during the first product and the softmax (the kernel lives on loads in flight)
    const bf16* vbase = vcache + page_base + in_page + 8 * c;
    uint4 vv[HD / 8];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) vv[d] = *(const uint4*)(vbase + (size_t)(d * 8 + g) * kv.page_size);
    // ---- scores: group j of 8 MMA columns; column n holds key 8 (n / 2) + 2 j + (n % 2)
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      const bf16* krow = kcache + page_base + (size_t)(in_page + 8 * (g >> 1) + 2 * j + (g & 1)) * HD;
#pragma unroll
      for (int kb = 0; kb < KB; ++kb) {
        const uint4 k4 = *(const uint4*)(krow + kb * 32 + c * 8);
        mma16816(s[j], qa[kb][0], UPPER ? qb[kb][0] : 0u, qa[kb][1], UPPER ? qb[kb][1] : 0u, k4.x, k4.y);
        mma16816(s[j], qa[kb][2], UPPER ? qb[kb][2] : 0u, qa[kb][3], UPPER ? qb[kb][3] : 0u, k4.z, k4.w);
      }
      if (TAIL) {
        const uint2 k2 = *(const uint2*)(krow + KB * 32 + c * 4);
        mma16816(s[j], qa[KB][0], UPPER ? qb[KB][0] : 0u, qa[KB][1], UPPER ? qb[KB][1] : 0u, k2.x, k2.y);
      }
    }
    // ---- mask, running maximum, probabilities (this thread: keys key0 + 8 c + 2 j + e)
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = key0 + 8 * c + 2 * j + e;
        const bool ok = key >= lo && key < hi;
        s[j][e] = ok ? s[j][e] * LOG2E : -INFINITY;
        s[j][2 + e] = ok ? s[j][2 + e] * LOG2E : -INFINITY;
        mx0 = fmaxf(mx0, s[j][e]);
        mx1 = fmaxf(mx1, s[j][2 + e]);
      }
    const float n0 = fmaxf(m0, quad_max(mx0)), n1 = fmaxf(m1, quad_max(mx1));
    const float u0 = n0 == -INFINITY ? 0.f : n0, u1 = n1 == -INFINITY ? 0.f : n1;
    const float alpha0 = exp2f(m0 - u0), alpha1 = exp2f(m1 - u1);
    m0 = n0;
    m1 = n1;
    uint32_t p[4][2];   // p[j][0]: row g, keys (8c+2j, +1); p[j][1]: row g + 8
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = exp2f(s[j][0] - u0), b = exp2f(s[j][1] - u0);
      const float cc = exp2f(s[j][2] - u1), d = exp2f(s[j][3] - u1);
      sum0 += a + b;
      sum1 += cc + d;
      p[j][0] = pack_bf16(a, b);
      p[j][1] = pack_bf16(cc, d);
    }
    l0 = l0 * alpha0 + sum0;
    l1 = l1 * alpha1 + sum1;
    // ---- o = o * alpha + p . V; values are [dim][position] inside the page
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) {
      const uint4 v4 = vv[d];
      o[d][0] *= alpha0; o[d][1] *= alpha0; o[d][2] *= alpha1; o[d][3] *= alpha1;
      mma16816(o[d], p[0][0], UPPER ? p[0][1] : 0u, p[1][0], UPPER ? p[1][1] : 0u, v4.x, v4.y);
      mma16816(o[d], p[2][0], UPPER ? p[2][1] : 0u, p[3][0], UPPER ? p[3][1] : 0u, v4.z, v4.w);
    }
  }
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);

  pdl_release_next();   // this warp's keys are done: the next kernel may move in while the CTAs merge
  // ---- merge the warps of the CTA in warp order (shared memory: [WARPS][rows_per_chunk][HD + 2])
  const int R = rows_per_chunk, W = HD + 2;
  float* mine = smem + (size_t)warp * R * W;
  if (g < rows) {
    float* r = mine + (size_t)g * W;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) { r[d * 8 + 2 * c] = o[d][0]; r[d * 8 + 2 * c + 1] = o[d][1]; }
    if (c == 0) { r[HD] = m0; r[HD + 1] = l0; }
  }
  if (UPPER && g + 8 < rows) {
    float* r = mine + (size_t)(g + 8) * W;
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) { r[d * 8 + 2 * c] = o[d][2]; r[d * 8 + 2 * c + 1] = o[d][3]; }
    if (c == 0) { r[HD] = m1; r[HD + 1] = l1; }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < rows * HD; i += WARPS * 32) {
    const int r = i / HD, d = i % HD;
    float M = -INFINITY;
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, smem[((size_t)w * R + r) * W + HD]);
    const float U = M == -INFINITY ? 0.f : M;
    float L = 0.f, acc = 0.f;
    for (int w = 0; w < WARPS; ++w) {
      const float* src = smem + ((size_t)w * R + r) * W;
      const float f = exp2f(src[HD] - U);
      L += src[HD + 1] * f;
      acc += src[d] * f;
    }
    const int head = head0 + r;
    if (shares == 1) {
      out[(size_t)t * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(acc / L);
    } else {
      const size_t pi = ((size_t)t * nh + head) * shares + share;
      part_o[pi * HD + d] = acc;
      if (d == 0) { part_ml[pi * 2] = M; part_ml[pi * 2 + 1] = L; }
    }
  }
}

// Merges the shares of one (token, head) in share order.
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       bf16* __restrict__ out, long long out_stride, int nh, int shares) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x, head = blockIdx.y;
  const size_t base = ((size_t)t * nh + head) * shares;
  float M = -INFINITY;
  for (int s = 0; s < shares; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  const float U = M == -INFINITY ? 0.f : M;
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float L = 0.f, acc = 0.f;
    for (int s = 0; s < shares; ++s) {
      const float f = exp2f(part_ml[(base + s) * 2] - U);
      L += part_ml[(base + s) * 2 + 1] * f;
      acc += part_o[(base + s) * HD + d] * f;
    }
    out[(size_t)t * out_stride + (size_t)head * HD + d] = __float2bfloat16_rn(acc / L);
  }
}

int launch_decode(const bf16* q, long long q_stride, bf16* out, long long out_stride, const bf16* kc, const bf16* vc,
                  PagedKV kv, const int* tok_pos, const int* tok_seq, const int* seq_slot, int ntok, int nh, int window,
                  int shares, float* part_o, float* part_ml, cudaStream_t stream) {
  const int rep = nh / kv.num_kv_heads;
  const int rows = rep <= 8 ? rep : (rep <= 16 ? rep : 16);
  const int chunks = (rep + rows - 1) / rows;
  const size_t smem = (size_t)WARPS * rows * (HD + 2) * sizeof(float);
  dim3 grid(shares, kv.num_kv_heads * chunks, ntok);
  if (rows <= 8) {
    auto k = attention_decode_kernel<false>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    gb_launch(k, grid, WARPS * 32, smem, stream, q, q_stride, out, out_stride, kc, vc, kv, tok_pos, tok_seq, seq_slot, nh,
                                          window, part_o, part_ml, rows);
  } else {
    auto k = attention_decode_kernel<true>;
    if (smem > 48 * 1024 && cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return (int)cudaGetLastError();
    gb_launch(k, grid, WARPS * 32, smem, stream, q, q_stride, out, out_stride, kc, vc, kv, tok_pos, tok_seq, seq_slot, nh,
                                          window, part_o, part_ml, rows);
  }
  int rc = gb_launch_status();
  if (rc != 0 || shares == 1) return rc;
  gb_launch(attention_merge_kernel, dim3(ntok, nh), HD >= 128 ? 128 : 64, 0, stream, part_o, part_ml, out, out_stride, nh, shares);
  return gb_launch_status();
}

}  // namespace

GB_EXPORT int gb_attention_decode_head_dim() { return HD; }

// q, out: [ntok, nh * HD] bfloat16 (row strides free; q 16-byte aligned rows).  The cache as in
// common.cuh.  shares: CTAs along the keys per (token, kv head); scratch (float32) must hold
// ntok * nh * shares * (HD + 2) values when shares > 1: part_o first, then part_ml.
GB_EXPORT int gb_attention_decode(const void* q, long long q_stride, void* out, long long out_stride,
                                  const void* kcache, const void* vcache, const int* page_table, int table_width,
                                  int page_size, int nkv, int hd, const int* tok_pos, const int* tok_seq,
                                  const int* seq_slot, int ntok, int nh, int window, int shares, float* scratch,
                                  cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (hd != HD || nkv <= 0 || nh % nkv || page_size % KEYS || shares < 1 || shares > 65535) return GB_ERR_SIZE;
  if (((uintptr_t)q & 15) || (q_stride % 8) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15)) return GB_ERR_SIZE;
  if (shares > 1 && !scratch) return GB_ERR_ARG;
  PagedKV kv{page_table, table_width, page_size, nkv, hd};
  float* part_o = scratch;
  float* part_ml = scratch ? scratch + (size_t)ntok * nh * shares * HD : nullptr;
  return launch_decode((const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)kcache, (const bf16*)vcache, kv,
                       tok_pos, tok_seq, seq_slot, ntok, nh, window, shares, part_o, part_ml, stream);
}

// ------------------------------------------------------------------ the entry point that allocates nothing
// See attention_decode_static.h.  The shares' partial results go to a fixed array in device
// memory instead of a buffer from the caller.  Nothing in it has to start at zero: every
// element the merge kernel reads was written by the first kernel of the same call.
#include <mutex>

#include "attention_decode_static.h"

namespace {

static __device__ __align__(256) float g_static_scratch[GB_ATTENTION_DECODE_STATIC_FLOATS];

// The array's device address, per device.  In host code the name g_static_scratch stands for a
// host-side shadow, not for device memory, so its address is asked for once per device, with
// that device current, and only that pointer is ever handed to a kernel.
float* static_scratch_address(int* error) {
  static float* address[64] = {};
  static std::mutex mu;
  int dev = -1;
  *error = (int)cudaGetDevice(&dev);
  if (*error != 0) return nullptr;
  if (dev < 0 || dev >= 64) {
    *error = GB_ERR_ARG;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (!address[dev]) {
    void* p = nullptr;
    *error = (int)cudaGetSymbolAddress(&p, g_static_scratch);
    if (*error != 0) return nullptr;
    address[dev] = (float*)p;
  }
  return address[dev];
}

}  // namespace

GB_EXPORT int gb_attention_decode_static(const void* q, long long q_stride, void* out, long long out_stride,
                                         const void* kcache, const void* vcache, const int* page_table,
                                         int table_width, int page_size, int nkv, int hd, const int* tok_pos,
                                         const int* tok_seq, const int* seq_slot, int ntok, int nh, int window,
                                         int shares, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  // sizes first, each against its own bound, so that the product below cannot wrap
  if (hd != HD || nkv <= 0 || nh <= 0 || nh % nkv || shares < 1 || shares > 65535) return GB_ERR_SIZE;
  float* scratch = nullptr;
  if (shares > 1) {
    const unsigned long long per_share = (unsigned long long)(HD + 2) * (unsigned)shares;   // < 2^25
    const unsigned long long rows_allowed = GB_ATTENTION_DECODE_STATIC_FLOATS / per_share;
    if ((unsigned long long)ntok > rows_allowed || (unsigned long long)ntok * (unsigned)nh > rows_allowed)
      return GB_ERR_STATIC_SCRATCH;
    // one share writes its result itself and needs no scratch: the array's address is looked up
    // only when it is used
    int error = 0;
    scratch = static_scratch_address(&error);
    if (!scratch) return error;
  }
  return gb_attention_decode(q, q_stride, out, out_stride, kcache, vcache, page_table, table_width, page_size, nkv, hd,
                             tok_pos, tok_seq, seq_slot, ntok, nh, window, shares, scratch, stream);
}
