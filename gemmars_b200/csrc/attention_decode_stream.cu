// bfloat16 attention of single positions over the paged cache, with the cache streamed through
// shared memory by TMA (sm_100a; head sizes that are multiples of 64, of which the package uses and tests 64 and 128;
// at most 16 query heads per kv head):
//
//     s_j = q_h . K[j, g]   for lo <= j <= p,      p_j = softmax(s)_j,      o_h = sum_j p_j V[j, g]
//     (src/model.rs:1199-1226; src/kernels.rs:1550-1561; q arrives scaled by head_dim^-0.5)
//
// Decoding reads every cached key and value once, so the kernel is a stream of pages and its
// time is how evenly and how steadily the SMs pull their share of them.  The pages to read are
// one flat list: token by token, kv head by kv head, page by page; CTA i of G takes the
// contiguous pages [i P / G, (i + 1) P / G), whatever the lengths of the sequences.  A producer
// thread asks for them in that order, a page of keys and the same page of values per stage
// (16 KB each at head size 128, 128-byte swizzle), stages ahead of the four consumer warps.
//
// A consumer warp owns 16 of a page's 64 keys: scores with mma.sync m16n8k16 (rows = the query
// heads of the kv head, padded to 16), an online softmax in log2 units, and the p.V product from
// the transposed value page, all operands through ldmatrix.  At the end of a segment (the part
// of one (token, kv head) that lies in the CTA's range) the four warps are merged in warp order;
// a whole (token, kv head) is written out at once, a part goes to one of the CTA's two scratch
// slots (only the first and the last segment of a range can be parts) and a second kernel adds
// the parts in key order.
//
// Every wait on an mbarrier is bounded; a wait that runs out sets the status word and the CTA's
// abort flag, after which its warps only walk their loops to the end.
#include "mma.cuh"
#include "tc_common.cuh"

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 128
#endif
#ifndef GB_STREAM_STAGES
#define GB_STREAM_STAGES 3
#endif

namespace {

constexpr int HD = GB_HEAD_DIM;
constexpr int KEYS = 64;                       // positions per page
constexpr int CW = 4;                          // consumer warps: 16 keys of a page each
constexpr int THREADS = (CW + 1) * 32;
constexpr int STAGES = GB_STREAM_STAGES;
constexpr int QH = HD / 64;                    // 64-wide boxes per key row
constexpr int MAX_TOKENS = 4096;
constexpr uint32_t K_BYTES = KEYS * HD * 2, V_BYTES = HD * KEYS * 2, STAGE_BYTES = K_BYTES + V_BYTES;
constexpr float LOG2E = 1.4426950408889634f;
static_assert(HD % 64 == 0 && HD >= 64 && HD <= 256, "head size: 64, 128, 192 or 256");

__device__ int g_stream_status;   // 0, or the first wait that ran out (1 free stage, 2 page)

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort, int code) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && *abort) return false;
  }
  *abort = 1;
  atomicCAS(&g_stream_status, 0, code);
  return false;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

// What a token asks of the cache: its slot, the first page it reads and how many.
struct TokenSpan {
  int slot, lo, hi, first_page, pages;
};
// A token whose slot is skip_slot belongs to no sequence (a row that pads a captured step): it
// asks for nothing and its row of the result is zero.  (Left in, 8 such rows x 8 kv heads
// were 64 one-page segments at the end of the list, all in the last CTA's range, and made a step
// of 24 sequences slower than one of 32.)
__device__ __forceinline__ TokenSpan token_span(int t, const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                               int window, int skip_slot) {
  TokenSpan s;
  const int pos = tok_pos[t];
  s.slot = seq_slot[tok_seq[t]];
  s.hi = pos + 1;
  s.lo = window > 0 ? max(0, s.hi - window) : 0;
  s.first_page = s.lo / KEYS;
  s.pages = s.slot == skip_slot ? 0 : (s.hi - 1) / KEYS - s.first_page + 1;
  return s;
}

// The flat list of pages: token t's pages of kv head h start at (prefix[t] * nkv + h * pages_t).
// Finds the token that flat index p falls into (prefix is non-decreasing, prefix[ntok] * nkv > p):
// the last token whose pages start at or before p, which is never a token without pages.
__device__ __forceinline__ int token_of(const int* prefix, int ntok, int nkv, long long p) {
  int lo = 0, hi = ntok - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if ((long long)prefix[mid] * nkv <= p) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

// grid: G CTAs; block: THREADS.  part: [G * 2][rep][HD + 2] (o, then m in log2 units, then l);
// prefix_out: [ntok + 1], written by CTA 0 for the merge kernel.
__global__ void __launch_bounds__(THREADS, 1)
attention_decode_stream_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                               const bf16* __restrict__ q, long long q_stride, bf16* __restrict__ out,
                               long long out_stride, const int* __restrict__ page_table, int table_width, int nkv,
                               const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                               const int* __restrict__ seq_slot, int ntok, int nh, int window, int skip_slot,
                               float* __restrict__ part, int* __restrict__ prefix_out) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  volatile int* abort = (volatile int*)(empty_bar + STAGES);
  int* prefix = (int*)(abort + 2);                              // [ntok + 1]
  float* merge = (float*)(prefix + ((ntok + 1 + 3) & ~3));      // [CW][rep][HD + 2]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int rep = nh / nkv;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], CW);
    }
    *abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // Positions, slots and the page table are the step's inputs, not the work of the kernel before
  // this one: the lists of pages are made before waiting for it; q and the cache are read after.
  // ---- pages per token, then their running sum (warp 0, 32 tokens a round)
  for (int t = threadIdx.x; t < ntok; t += THREADS) prefix[t + 1] = token_span(t, tok_pos, tok_seq, seq_slot, window, skip_slot).pages;
  __syncthreads();
  if (warp == 0) {
    int carry = 0;
    for (int base = 0; base < ntok; base += 32) {
      const int t = base + lane;
      int v = t < ntok ? prefix[t + 1] : 0;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += up;
      }
      if (t < ntok) prefix[t + 1] = carry + v;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
    if (lane == 0) prefix[0] = 0;
  }
  __syncthreads();
  const long long P = (long long)prefix[ntok] * nkv, G = gridDim.x;
  const long long p0 = (long long)blockIdx.x * P / G, p1 = ((long long)blockIdx.x + 1) * P / G;

  if (warp == CW) {
    // ---------------- producer: one page of keys and of values per stage.  Which rows of the
    // cache a page is takes a chain of loads (position, slot, page table), so the warp looks up
    // 32 pages at a time, a lane each, one round ahead of the lane that issues the copies.
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    auto lookup = [&](long long p) -> int {   // row of the cache (page * nkv + kv head) of flat page p
      if (p >= p1) return 0;
      const int t = token_of(prefix, ntok, nkv, p);
      const TokenSpan sp = token_span(t, tok_pos, tok_seq, seq_slot, window, skip_slot);
      const long long r = p - (long long)prefix[t] * nkv;
      const int kvh = (int)(r / sp.pages), page = (int)(r % sp.pages);
      return page_table[(size_t)sp.slot * table_width + (sp.first_page + page) % table_width] * nkv + kvh;
    };
    int next_row = lookup(p0 + lane);
    pdl_wait_prior();
    uint32_t it = 0;
    bool ok = true;
    for (long long base = p0; base < p1; base += 32) {
      const int my_row = next_row;
      next_row = lookup(base + 32 + lane);
      const int n = (int)min((long long)32, p1 - base);
      for (int i = 0; i < n; ++i, ++it) {
        const int row = __shfl_sync(0xffffffffu, my_row, i);
        if (lane == 0 && ok) {
          const uint32_t s = it % STAGES;
          ok = it < STAGES || wait_or_abort(&empty_bar[s], ((it / STAGES) - 1) & 1, abort, 1);
          if (ok) {
            uint8_t* k_smem = smem + s * STAGE_BYTES;
            mbar_expect_tx(&full_bar[s], STAGE_BYTES);
#pragma unroll
            for (int h = 0; h < QH; ++h) tma_load_2d(k_smem + h * (KEYS * 128), &map_k, h * 64, row * KEYS, &full_bar[s]);
            tma_load_2d(k_smem + K_BYTES, &map_v, 0, row * HD, &full_bar[s]);
          }
        }
        __syncwarp();
      }
    }
    if (lane == 0) pdl_release_next();   // the last page is on its way: the next kernel may move in
    __syncwarp();
    return;
  }

  // ---------------- consumers
  const int g = lane >> 2, c = lane & 3;
  const int W = HD + 2;
  float* mine = merge + (size_t)warp * rep * W;
  // the address part of ldmatrix that does not change: this lane supplies row (lane % 8) of
  // matrix (lane / 8); matrices 0, 1 are the low and high 16-byte chunk of the first 8 rows,
  // matrices 2, 3 of the next 8 rows
  const int mat = lane >> 3, mrow = (mat >> 1) * 8 + (lane & 7), mchunk = mat & 1;
  bool ok = true;
  uint32_t it = 0, seg = 0;
  long long p = p0;
  int t = p0 < p1 ? token_of(prefix, ntok, nkv, p0) : 0;
  pdl_wait_prior();
  if (blockIdx.x == 0)
    for (int i = threadIdx.x; i <= ntok; i += CW * 32) prefix_out[i] = prefix[i];
  while (p < p1) {
    // ---- the segment: (token t, kv head kvh), pages [a, b) of the token's span
    const TokenSpan sp = token_span(t, tok_pos, tok_seq, seq_slot, window, skip_slot);
    const long long r = p - (long long)prefix[t] * nkv;
    const int kvh = (int)(r / sp.pages), a = (int)(r % sp.pages);
    const int b = (int)min((long long)sp.pages, a + (p1 - p));
    const bool whole = a == 0 && b == sp.pages;
    const int head0 = kvh * rep;
    // q as the A operand: rows g and g + 8 are query heads head0 + g and head0 + g + 8
    uint32_t qa[HD / 16][4];
    {
      const bf16* q0 = q + (size_t)t * q_stride + (size_t)(head0 + g) * HD + 2 * c;
      const bf16* q1 = q0 + 8 * HD;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        qa[ks][0] = g < rep ? *(const uint32_t*)(q0 + ks * 16) : 0u;
        qa[ks][1] = g + 8 < rep ? *(const uint32_t*)(q1 + ks * 16) : 0u;
        qa[ks][2] = g < rep ? *(const uint32_t*)(q0 + ks * 16 + 8) : 0u;
        qa[ks][3] = g + 8 < rep ? *(const uint32_t*)(q1 + ks * 16 + 8) : 0u;
      }
    }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;   // rows g and g + 8; m in log2 units
    float o[HD / 8][4];
#pragma unroll
    for (int d = 0; d < HD / 8; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;

    for (int page = a; page < b; ++page, ++it) {
      const uint32_t s = it % STAGES;
      if (ok) ok = wait_or_abort(&full_bar[s], (it / STAGES) & 1, abort, 2);
      if (!ok) continue;
      const uint32_t k_smem = smem_u32(smem + s * STAGE_BYTES), v_smem = k_smem + K_BYTES;
      const int key0 = (sp.first_page + page) * KEYS + warp * 16;   // position of this warp's first key
      // ---- scores of 16 keys: two n-tiles of 8
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      {
        const int krow = warp * 16 + mrow;
        const uint32_t row_addr = k_smem + krow * 128;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const int chunk = (ks & 3) * 2 + mchunk;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(row_addr + (ks >> 2) * (KEYS * 128) + ((chunk ^ (krow & 7)) << 4), b0, b1, b2, b3);
          mma16816(s0, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
          mma16816(s1, qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
        }
      }
      // ---- mask, online softmax (log2 units)
      const int ka = key0 + 2 * c, kb = ka + 8;
      const bool va0 = ka >= sp.lo && ka < sp.hi, va1 = ka + 1 >= sp.lo && ka + 1 < sp.hi;
      const bool vb0 = kb >= sp.lo && kb < sp.hi, vb1 = kb + 1 >= sp.lo && kb + 1 < sp.hi;
      s0[0] = va0 ? s0[0] * LOG2E : -INFINITY;
      s0[1] = va1 ? s0[1] * LOG2E : -INFINITY;
      s0[2] = va0 ? s0[2] * LOG2E : -INFINITY;
      s0[3] = va1 ? s0[3] * LOG2E : -INFINITY;
      s1[0] = vb0 ? s1[0] * LOG2E : -INFINITY;
      s1[1] = vb1 ? s1[1] * LOG2E : -INFINITY;
      s1[2] = vb0 ? s1[2] * LOG2E : -INFINITY;
      s1[3] = vb1 ? s1[3] * LOG2E : -INFINITY;
      const float n0 = fmaxf(m0, quad_max(fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]))));
      const float n1 = fmaxf(m1, quad_max(fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]))));
      const float r0 = n0 == -INFINITY ? 0.f : n0, r1 = n1 == -INFINITY ? 0.f : n1;   // all masked so far
      const float al0 = exp2f(m0 - r0), al1 = exp2f(m1 - r1);
      m0 = n0;
      m1 = n1;
      s0[0] = exp2f(s0[0] - r0);
      s0[1] = exp2f(s0[1] - r0);
      s1[0] = exp2f(s1[0] - r0);
      s1[1] = exp2f(s1[1] - r0);
      s0[2] = exp2f(s0[2] - r1);
      s0[3] = exp2f(s0[3] - r1);
      s1[2] = exp2f(s1[2] - r1);
      s1[3] = exp2f(s1[3] - r1);
      l0 = l0 * al0 + (s0[0] + s0[1] + s1[0] + s1[1]);
      l1 = l1 * al1 + (s0[2] + s0[3] + s1[2] + s1[3]);
      const uint32_t pa0 = pack_bf16(s0[0], s0[1]), pa1 = pack_bf16(s0[2], s0[3]);
      const uint32_t pa2 = pack_bf16(s1[0], s1[1]), pa3 = pack_bf16(s1[2], s1[3]);
      // ---- o = o * alpha + p . V over this warp's 16 keys: two n-tiles of 8 dims per ldmatrix
      {
        const int chunk = warp * 2 + mchunk;
#pragma unroll
        for (int j = 0; j < HD / 16; ++j) {
          const int vrow = j * 16 + mrow;
          uint32_t b0, b1, b2, b3;
          ldmatrix_x4(v_smem + vrow * 128 + ((chunk ^ (vrow & 7)) << 4), b0, b1, b2, b3);
          o[2 * j][0] *= al0;
          o[2 * j][1] *= al0;
          o[2 * j][2] *= al1;
          o[2 * j][3] *= al1;
          o[2 * j + 1][0] *= al0;
          o[2 * j + 1][1] *= al0;
          o[2 * j + 1][2] *= al1;
          o[2 * j + 1][3] *= al1;
          mma16816(o[2 * j], pa0, pa1, pa2, pa3, b0, b1);
          mma16816(o[2 * j + 1], pa0, pa1, pa2, pa3, b2, b3);
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty_bar[s])) : "memory");
    }

    // ---- merge the four warps in warp order
    l0 = quad_sum(l0);
    l1 = quad_sum(l1);
    if (g < rep) {
      float* row = mine + (size_t)g * W;
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) *(float2*)(row + d * 8 + 2 * c) = make_float2(o[d][0], o[d][1]);
      if (c == 0) { row[HD] = m0; row[HD + 1] = l0; }
    }
    if (g + 8 < rep) {
      float* row = mine + (size_t)(g + 8) * W;
#pragma unroll
      for (int d = 0; d < HD / 8; ++d) *(float2*)(row + d * 8 + 2 * c) = make_float2(o[d][2], o[d][3]);
      if (c == 0) { row[HD] = m1; row[HD + 1] = l1; }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    float* slot = part + ((size_t)blockIdx.x * 2 + (seg == 0 ? 0 : 1)) * rep * W;
    for (int i = threadIdx.x; i < rep * HD; i += CW * 32) {
      const int rr = i / HD, d = i % HD;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < CW; ++w) M = fmaxf(M, merge[((size_t)w * rep + rr) * W + HD]);
      float L = 0.f, O = 0.f;
#pragma unroll
      for (int w = 0; w < CW; ++w) {
        const float* src = merge + ((size_t)w * rep + rr) * W;
        const float mw = src[HD];
        const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
        L += src[HD + 1] * f;
        O += src[d] * f;
      }
      if (whole) {
        out[(size_t)t * out_stride + (size_t)(head0 + rr) * HD + d] = __float2bfloat16_rn(O / L);
      } else {
        slot[(size_t)rr * W + d] = O;
        if (d == 0) {
          slot[(size_t)rr * W + HD] = M;
          slot[(size_t)rr * W + HD + 1] = L;
        }
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(CW * 32) : "memory");
    // ---- on to the next segment
    p += b - a;
    ++seg;
    if (p < p1) t = token_of(prefix, ntok, nkv, p);   // the next token that has pages
  }
}

// One CTA per (token, kv head): adds the parts that the stream kernel left for it, in key order.
// Nothing to do when one CTA had the whole of it.  A thread owns one output value (up to
// MERGE_EPT when there are more than 1,024); the parts' maxima and sums are fetched by all
// threads at once and turned into one factor per part and head, so that the thread's own loads
// of o depend on nothing and go out together.  More than MERGE_ROUND parts take several rounds.
constexpr int MAX_CTAS = 1024, MERGE_ROUND = 64, MERGE_EPT = 4, MAX_REP = 16, MERGE_COUNT_ITSELF = 256;
__global__ void __launch_bounds__(1024)
attention_decode_stream_merge_kernel(bf16* __restrict__ out, long long out_stride, const float* __restrict__ part,
                                     const int* __restrict__ prefix, const int* __restrict__ tok_pos,
                                     const int* __restrict__ tok_seq, const int* __restrict__ seq_slot, int window,
                                     int skip_slot, int ntok, int nkv, int nh, int G) {
  __shared__ int slot_of[MERGE_ROUND];   // scratch slot of a part; -1: that CTA had no pages at all
  __shared__ float fac[MERGE_ROUND][MAX_REP], sum[MERGE_ROUND][MAX_REP];
  __shared__ float run_m[MAX_REP], run_l[MAX_REP], scale[MAX_REP];
  __shared__ int span[3];                // pages before token t, through token t, of all tokens
  pdl_release_next();
  const int t = blockIdx.x / nkv, kvh = blockIdx.x % nkv;
  const bool early = ntok <= MERGE_COUNT_ITSELF;
  if (early) {
    // with few tokens the CTA counts the pages itself, from the step's inputs, while the stream
    // kernel is still running; else it reads the stream kernel's list once that is done
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      int carry = 0;
      for (int base = 0; base < ntok; base += 32) {
        const int i = base + lane;
        int v = 0;
        if (i < ntok) v = token_span(i, tok_pos, tok_seq, seq_slot, window, skip_slot).pages;
        int incl = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const int up = __shfl_up_sync(0xffffffffu, incl, d);
          if (lane >= d) incl += up;
        }
        if (i == t) {
          span[0] = carry + incl - v;
          span[1] = carry + incl;
        }
        carry += __shfl_sync(0xffffffffu, incl, 31);
      }
      if (lane == 0) span[2] = carry;
    }
  } else {
    pdl_wait_prior();
    if (threadIdx.x == 0) {
      span[0] = prefix[t];
      span[1] = prefix[t + 1];
      span[2] = prefix[ntok];
    }
  }
  __syncthreads();
  const int rep = nh / nkv, W = HD + 2;
  const long long P = (long long)span[2] * nkv;
  const int pages = span[1] - span[0];
  const long long u0 = (long long)span[0] * nkv + (long long)kvh * pages, u1 = u0 + pages;
  const int first = (int)(((u0 + 1) * G - 1) / P), last = (int)((u1 * G - 1) / P);
  const int n = last - first + 1, tid = threadIdx.x, nthr = blockDim.x;
  // which scratch slot each part lies in: known from the page counts alone
  auto slots_of_round = [&](int base, int cn) {
    if (tid < cn) {
      const long long j = first + base + tid, start = j * P / G;
      // a CTA's part of this (token, kv head) is its first segment if its range starts inside it
      slot_of[tid] = start == (j + 1) * P / G ? -1 : (int)j * 2 + (start >= u0 ? 0 : 1);
    }
  };
  if (tid < MAX_REP) {
    run_m[tid] = -INFINITY;
    run_l[tid] = 0.f;
  }
  if (n > 1) slots_of_round(0, min(MERGE_ROUND, n));
  if (early) pdl_wait_prior();   // every CTA waits, also one with nothing to add: the kernel after this one relies on it
  if (pages == 0) {   // a row of no sequence: zeros, so that what follows stays finite
    for (int i = tid; i < rep * HD; i += nthr)
      out[(size_t)t * out_stride + (size_t)(kvh * rep + i / HD) * HD + i % HD] = __float2bfloat16_rn(0.f);
    return;
  }
  if (n == 1) return;
  float acc[MERGE_EPT];
#pragma unroll
  for (int e = 0; e < MERGE_EPT; ++e) acc[e] = 0.f;
  // parts of the thread's first value asked for before the factors are known: a lone sequence of
  // 8,192 tokens is cut into about 19 parts per kv head, which then come in one round trip
  constexpr int AHEAD = 24;
  for (int base = 0; base < n; base += MERGE_ROUND) {
    const int cn = min(MERGE_ROUND, n - base);
    __syncthreads();
    if (base > 0) slots_of_round(base, cn);
    __syncthreads();
    float ahead[AHEAD];
    {
      const int rr = tid / HD, d = tid % HD;
      const float* src = part + (size_t)rr * W + d;
#pragma unroll
      for (int jj = 0; jj < AHEAD; ++jj) {
        const int sl = jj < cn ? slot_of[jj] : -1;
        ahead[jj] = (sl >= 0 && tid < rep * HD) ? src[(size_t)sl * rep * W] : 0.f;
      }
    }
    for (int i = tid; i < cn * rep; i += nthr) {
      const int jj = i / rep, rr = i % rep, sl = slot_of[jj];
      const float* src = part + ((size_t)max(sl, 0) * rep + rr) * W;
      fac[jj][rr] = sl >= 0 ? src[HD] : -INFINITY;
      sum[jj][rr] = sl >= 0 ? src[HD + 1] : 0.f;
    }
    __syncthreads();
    if (tid < rep * 32) {
      // warp rr: the factors of head rr's parts, two parts a lane (the block has rep * HD >= rep * 64 threads)
      const int rr = tid >> 5, ln = tid & 31;
      static_assert(MERGE_ROUND == 64, "two parts a lane");
      const float m0 = ln < cn ? fac[ln][rr] : -INFINITY, m1 = ln + 32 < cn ? fac[ln + 32][rr] : -INFINITY;
      const float before = run_m[rr], l_before = run_l[rr];
      float m = fmaxf(before, fmaxf(m0, m1));
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, d));
      const float f0 = m0 == -INFINITY ? 0.f : exp2f(m0 - m), f1 = m1 == -INFINITY ? 0.f : exp2f(m1 - m);
      float l = (ln < cn ? sum[ln][rr] * f0 : 0.f) + (ln + 32 < cn ? sum[ln + 32][rr] * f1 : 0.f);
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) l += __shfl_xor_sync(0xffffffffu, l, d);
      const float sc = before == -INFINITY ? 0.f : exp2f(before - m);
      if (ln < cn) fac[ln][rr] = f0;
      if (ln + 32 < cn) fac[ln + 32][rr] = f1;
      __syncwarp();
      if (ln == 0) {
        run_m[rr] = m;
        run_l[rr] = l_before * sc + l;
        scale[rr] = sc;
      }
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < MERGE_EPT; ++e) {
      const int i = tid + e * nthr;
      if (i < rep * HD) {
        const int rr = i / HD, d = i % HD;
        const float* src = part + (size_t)rr * W + d;
        float a = acc[e] * scale[rr];
        int jj = 0;
        if (e == 0) {
#pragma unroll
          for (; jj < AHEAD; ++jj)
            if (jj < cn) a += fac[jj][rr] * ahead[jj];   // 0 where the slot is empty
        }
#pragma unroll 8
        for (; jj < cn; ++jj) {
          const int sl = slot_of[jj];
          if (sl >= 0) a += fac[jj][rr] * src[(size_t)sl * rep * W];
        }
        acc[e] = a;
      }
    }
  }
#pragma unroll
  for (int e = 0; e < MERGE_EPT; ++e) {
    const int i = tid + e * nthr;
    if (i < rep * HD) {
      const int rr = i / HD, d = i % HD;
      out[(size_t)t * out_stride + (size_t)(kvh * rep + rr) * HD + d] = __float2bfloat16_rn(acc[e] / run_l[rr]);
    }
  }
}

}  // namespace

GB_EXPORT int gb_attention_decode_stream_head_dim() { return HD; }

// Shared memory one CTA needs for `ntok` tokens and `rep` query heads per kv head.
static size_t stream_smem(int ntok, int rep) {
  return (size_t)STAGES * STAGE_BYTES + 2 * STAGES * 8 + 8 + (size_t)((ntok + 1 + 3) & ~3) * 4 +
         (size_t)CW * rep * (HD + 2) * 4 + 1024;
}

// q, out: [ntok, nh * HD] bfloat16 (q rows 4-byte aligned).  kcache: [pages, nkv, 64, HD],
// vcache: [pages, nkv, HD, 64], 16-byte aligned.  ctas: CTAs to launch (0: two per SM when they
// fit, else one).  skip_slot: tokens of this slot belong to no sequence: nothing is read for them
// and their rows of out are zero (-1: none).  scratch: float32, at least
// gb_attention_decode_stream_scratch(...) values.
GB_EXPORT long long gb_attention_decode_stream_scratch(int ntok, int nh, int nkv, int ctas) {
  if (nkv <= 0) return 0;
  return (long long)ctas * 2 * (nh / nkv) * (HD + 2) + ntok + 1;
}

GB_EXPORT int gb_attention_decode_stream(const void* q, long long q_stride, void* out, long long out_stride,
                                         const void* kcache, const void* vcache, long long pages,
                                         const int* page_table, int table_width, int page_size, int nkv, int hd,
                                         const int* tok_pos, const int* tok_seq, const int* seq_slot, int ntok, int nh,
                                         int window, int skip_slot, int ctas, float* scratch, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (hd != HD || page_size != KEYS || nkv <= 0 || nh % nkv || nh / nkv > 16 || ntok > MAX_TOKENS || ctas <= 0 || ctas > MAX_CTAS)
    return GB_ERR_SIZE;
  if (((uintptr_t)q & 3) || (q_stride & 1) || !scratch) return GB_ERR_ARG;
  const int rep = nh / nkv;
  CUtensorMap mk, mv;
  if (!tensor_map(&mk, kcache, (uint64_t)pages * nkv * KEYS, (uint64_t)HD, (uint64_t)HD * 2, KEYS)) return GB_ERR_ARG;
  if (!tensor_map(&mv, vcache, (uint64_t)pages * nkv * HD, (uint64_t)KEYS, (uint64_t)KEYS * 2, HD)) return GB_ERR_ARG;
  const size_t smem = stream_smem(ntok, rep);
  if (smem > 227 * 1024) return GB_ERR_SIZE;
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(attention_decode_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return (int)cudaGetLastError();
    configured = smem;
  }
  float* part = scratch;
  int* prefix = (int*)(scratch + (size_t)ctas * 2 * rep * (HD + 2));
  gb_launch(attention_decode_stream_kernel, dim3(ctas), dim3(THREADS), smem, stream, mk, mv, (const bf16*)q, q_stride,
            (bf16*)out, out_stride, page_table, table_width, nkv, tok_pos, tok_seq, seq_slot, ntok, nh, window, skip_slot,
            part, prefix);
  const int merge_threads = rep * HD >= 1024 ? 1024 : (rep * HD + 31) / 32 * 32;
  gb_launch(attention_decode_stream_merge_kernel, dim3(ntok * nkv), dim3(merge_threads), 0, stream, (bf16*)out, out_stride,
            (const float*)part, (const int*)prefix, tok_pos, tok_seq, seq_slot, window, skip_slot, ntok, nkv, nh, ctas);
  return gb_launch_status();
}

GB_EXPORT int gb_attention_decode_stream_smem(int ntok, int rep) { return (int)stream_smem(ntok, rep); }

GB_EXPORT int gb_attention_decode_stream_status(int reset) {
  int v = -1;
  if (cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset) {
    int zero = 0;
    cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
  }
  return v;
}
