// bfloat16 matrix product on the 5th-generation tensor cores (tcgen05, sm_100a):
//
//     y[t, o] = sum_i W[o, i] * x[t, i] (+ bias[o])          (src/kernels.rs:54-57)
//
// written in bfloat16 or float32, or added into a float32 y (the residual stream).
//
// The product is computed "swapped": a CTA owns 128 output features (rows of W, the MMA's M) by
// BN tokens (rows of x, the MMA's N, 16..256).  Both operands are K-major in memory as they
// are, so TMA brings [128 x 64] tiles of W and [BN x 64] tiles of x into 128-byte-swizzled
// shared memory, one elected thread issues tcgen05.mma with the accumulator in tensor memory
// (lane = feature, column = token), and four warps read it back with tcgen05.ld: for one
// token, the 32 lanes of a warp hold 32 consecutive features.  A result that TMA can address
// leaves as TMA stores of 32 tokens x 32 features staged in shared memory (TileOut), any other
// with plain stores.
//
// Two kernels.  gemm_tc_kernel, one tile per CTA, serves decoding (BN = 16..64, where the CTA
// only streams its rows of W at memory speed): when that leaves too few tiles for the 148 SMs,
// the inner dimension is split over the CTAs of a thread-block cluster, whose partial sums meet
// in the shared memory of the rank that finishes the token and are added there in rank order:
// no atomics, the same bits every run.
// gemm_tc_persistent_kernel serves prompts (BN = 128 or 256): one CTA per SM walks the tiles
// with two accumulator buffers, so a tile's epilogue runs under the next tile's MMAs.
//
// Warp roles (192 threads): warps 0-3 epilogue (tensor-memory lane quarter = warp id),
// warp 4 TMA producer, warp 5 tensor-memory allocation and MMA issue.
//
// Every wait on an mbarrier is bounded: after WAIT_LIMIT polls the thread records a code in
// the status word and goes on to the common exit, where tensor memory is freed.
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;          // output features per CTA (MMA M)
constexpr int BK = 64;           // inner elements per stage: 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int THREADS = 192;

// EPI_SWIGLU_BF16: W stacks a gate matrix over an up matrix ([2N, K]) and the kernel writes
// silu(gate) * up in bfloat16, so the [M, 2N] intermediate never exists.  gemm_tc_kernel keeps two
// accumulators (gate rows and up rows of the same 128 features against one tile of x);
// gemm_tc_persistent_kernel one, whose 128 rows are 64 gate rows and the same features' up rows.
enum { EPI_STORE_BF16 = 0, EPI_STORE_F32 = 1, EPI_ACCUMULATE_F32 = 2, EPI_SWIGLU_BF16 = 3, EPI_QKV_BF16 = 4 };

// EPI_QKV_BF16: the q/k/v product of a decode step whose head size is the tile's 128 features: a
// tile is one head of one kind, and the epilogue does what the per-head kernel would do next on
// the value it holds in a register: RMSNorm over the head, rotation at the token's position, the
// query's scale; queries go to y as bfloat16, keys and values straight into the paged cache
// (src/qwen.rs:737-785).  What that needs beyond the product:
// An RMSNorm that sits between two products, taken into them (decode steps, where the norm's own
// kernel costs more waiting than work).  The product before it, which adds into the residual r,
// also leaves bf16(r * g), g being the norm's weight, and its tile's part of every token's sum
// of squares; the product after it takes those rows as its input and multiplies each token's
// results by 1 / sqrt(mean(r^2) + eps), which is what the norm would have done to its input.
// Statistics and the scale are float32; the parts are added in tile order (the same bits every run).
struct NormLink {
  const float* in_partial;   // this product's input rows are unscaled: [in_tiles][64] sums of squares; null: rows are plain
  int in_tiles;
  float in_eps, in_inv_width;
  const float* out_weight;   // this product adds into the residual and a norm follows: its weight; null: nothing to leave
  bf16* out_rows;            // [M][N] rows out_ld apart: bf16(residual * weight)
  long long out_ld;
  float* out_partial;        // [tiles of this product][64]
};

struct QkvTail {
  const float* q_weight;    // [128] or null: no norm
  const float* k_weight;
  const float* inv_freq;    // [64] or null: no rotation
  const int* tok_pos;
  const int* tok_seq;
  const int* seq_slot;
  const int* page_table;    // null: keys and values are not cached (they go to y like the queries)
  bf16* kcache;
  bf16* vcache;
  float eps, q_scale;
  int nh, nkv, table_width, page_size;
  const float2* rope_table; // prompts: [tokens][64] (cos, sin) of each packed token's angles, or null
  const int2* token_place;  // prompts: [tokens] (page, position in the page) of each packed token
  NormLink link;            // any mode of gemm_tc_kernel: a norm taken into this product (all null: none)
  int recv_apart;           // gemm_tc_kernel with a split inner dimension: the ranks' partial sums arrive in
                            // memory of their own behind the stages (see the exchange), not in the stages
};
enum { ST_OK = 0, ST_TIMEOUT_FULL = 1, ST_TIMEOUT_EMPTY = 2, ST_TIMEOUT_TMEM = 3, ST_TIMEOUT_PART = 4, ST_TIMEOUT_RECV = 5 };

__device__ int g_status;   // first failure of any launch; 0 when all waits completed



// silu(g) * u with the hardware's exp2 and reciprocal (two special-function instructions): the
// result is rounded to bfloat16, whose step is a thousand times their error, and the four epilogue
// warps have nothing to hide a longer chain behind (measured: the exact expf and division made
// the gated tile's epilogue 11.5 us per 128 tokens).  For g below -88 the quotient is 0, the limit.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

template <int MODE>
__device__ __forceinline__ void emit(void* y, size_t idx, float v) {
  if (MODE == EPI_STORE_BF16 || MODE == EPI_SWIGLU_BF16) ((bf16*)y)[idx] = __float2bfloat16_rn(v);
  else if (MODE == EPI_STORE_F32) ((float*)y)[idx] = v;
  else ((float*)y)[idx] += v;
}

// The way out of a tile for results that TMA can address.  An epilogue warp holds 32 features (one
// per lane) of 16 tokens at a time; written to the result with plain stores that is 16 requests of
// 64 or 128 bytes per warp, and the requests, not their bytes, were what the epilogue waited for
// (measured: 0.55 us per 16 tokens whatever the type, 4.6 us for a tile of 128 tokens; a quarter of
// the stores took a third of the time).  Here the warp puts the piece into shared memory, token
// after token, and one lane sends it as a single TMA store (or float32 add: the residual), two
// pieces in flight per warp.  TMA drops the tokens and features beyond the result's edges.  A
// piece's cost is its fence and its request (about 400 cycles, whatever its size), so a piece is
// 32 tokens wherever the tile has that many.
constexpr int PIECE_TOKENS = TC_OUT_ROWS, PIECE_FEATURES = TC_OUT_COLS;
constexpr int PIECE_BYTES = PIECE_TOKENS * PIECE_FEATURES * 4;          // float32; bfloat16 uses half
constexpr int PIECES = 2;                                               // pieces of a warp in flight
constexpr int OUT_STAGING_BYTES = 4 * PIECES * PIECE_BYTES;             // four warps

template <int MODE, int SLOT_BYTES = PIECE_BYTES>
struct TileOut {
  static constexpr int FEATURES = PIECE_FEATURES;
  const CUtensorMap* map;
  uint8_t* pieces;   // this warp's pieces, 128-byte aligned
  uint32_t sent;
  __device__ __forceinline__ TileOut(const CUtensorMap* m, uint8_t* staging, int warp)
      : map(m), pieces(staging + warp * PIECES * SLOT_BYTES), sent(0) {}
  __device__ __forceinline__ static void put(uint8_t* p, int token, int lane, float r) {
    if (MODE == EPI_STORE_BF16 || MODE == EPI_SWIGLU_BF16 || MODE == EPI_QKV_BF16)
      ((bf16*)p)[token * FEATURES + lane] = __float2bfloat16_rn(r);
    else
      ((float*)p)[token * FEATURES + lane] = r;
  }
  // the piece to fill next; waits until the request that last used its memory has read it
  __device__ __forceinline__ uint8_t* next(int lane) {
    if (sent >= PIECES) {
      if (lane == 0) tma_store_wait_read<PIECES - 1>();
      __syncwarp();
    }
    return pieces + (sent % PIECES) * SLOT_BYTES;
  }
  // after every lane has put its values: one request for the whole piece
  __device__ __forceinline__ void post(uint8_t* p, int lane, int x, int row, int N) {
    fence_smem_to_tma();
    __syncwarp();
    if (lane == 0 && x < N) {
      if (MODE == EPI_ACCUMULATE_F32) tma_add_2d(map, p, x, row);
      else tma_store_2d(map, p, x, row);
      tma_store_commit();
    }
    ++sent;
  }
  // lo, hi: tokens 0-15 and (with `both`) 16-31 of this lane's feature; x: the warp's first
  // feature; row: the first token.  The map's pieces are 32 tokens long with `both`, else 16.
  __device__ __forceinline__ void send(const uint32_t (&lo)[16], const uint32_t (&hi)[16], bool both, float bias, int lane,
                                       int x, int row, int N) {
    uint8_t* p = next(lane);
#pragma unroll
    for (int j = 0; j < 16; ++j) put(p, j, lane, __uint_as_float(lo[j]) + bias);
    if (both) {
#pragma unroll
      for (int j = 0; j < 16; ++j) put(p, 16 + j, lane, __uint_as_float(hi[j]) + bias);
    }
    post(p, lane, x, row, N);
  }
  // before the shared memory is given up and the kernel ends
  __device__ __forceinline__ void finish(int lane) {
    if (lane == 0) tma_store_wait_all();
    __syncwarp();
  }
};

// 16 tokens (from m_first) of feature n with plain stores: results that TMA cannot address.
template <int MODE>
__device__ __forceinline__ void store_direct(void* y, long long ldy, const uint32_t (&v)[16], float bias, int m_first, int M,
                                             int n, int N) {
  if (n >= N) return;
  if (MODE == EPI_ACCUMULATE_F32) {
    // all 16 loads first, then the stores: a load after a store to the same array would
    // wait for it, and the chunk would take 16 round trips to memory instead of one
    float old[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) old[j] = m_first + j < M ? ((const float*)y)[(size_t)(m_first + j) * ldy + n] : 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (m_first + j < M) ((float*)y)[(size_t)(m_first + j) * ldy + n] = old[j] + __uint_as_float(v[j]) + bias;
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j)
      if (m_first + j < M) emit<MODE>(y, (size_t)(m_first + j) * ldy + n, __uint_as_float(v[j]) + bias);
  }
}

// The accumulator columns [c, c + 16) of this warp's 32 lanes, gated when the tile has two
// accumulators BN columns apart; the caller waits (tc_wait_ld) before it reads v, then calls gate.
template <bool DUAL>
__device__ __forceinline__ void acc_load(uint32_t acc, int up_offset, int c, uint32_t (&v)[16], uint32_t (&u)[16]) {
  tc_ld16(acc + c, v);
  if (DUAL) tc_ld16(acc + up_offset + c, u);
}
template <bool DUAL>
__device__ __forceinline__ void gate(uint32_t (&v)[16], const uint32_t (&u)[16]) {
  if (DUAL) {
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(silu_mul(__uint_as_float(v[j]), __uint_as_float(u[j])));
  }
}

// The gated product of the persistent kernel keeps gate and up rows of W in one tile of 128 rows:
// 64 gate rows, then the up rows of the same 64 features.  Epilogue warps 0 and 1 then hold gate
// values (32 features each, one per lane), warps 2 and 3 the up values of the same features, and
// warp w and w + 2 are a pair: of 32 tokens the gate warp finishes the first 16 and the up warp
// the last 16, each handing the other, through shared memory, the 16 values it lacks (of 16
// tokens the gate warp finishes all).  GateExchange is one pair's memory: two rounds (a warp
// writes round r + 2 only after the pair's barrier of round r + 1, which its partner reaches
// after it has read round r), two directions, 16 tokens x 32 lanes of float32.
constexpr int EXCHANGE_BYTES = 2 * 2 * 2 * 16 * 32 * 4;   // two pairs
struct GateExchange {
  float* base;      // this pair's [round & 1][direction][16][32]
  uint32_t round;
  int pair;
  __device__ __forceinline__ GateExchange(uint8_t* mem, int warp) : base((float*)mem + (warp & 1) * 2 * 2 * 16 * 32), round(0), pair(warp & 1) {}
  // give: the 16 values of this lane that the partner finishes; returns in `got` the partner's
  __device__ __forceinline__ void swap(const uint32_t (&give)[16], bool is_up, int lane, uint32_t (&got)[16]) {
    float* mine = base + ((round & 1) * 2 + (is_up ? 1 : 0)) * 16 * 32;
    const float* theirs = base + ((round & 1) * 2 + (is_up ? 0 : 1)) * 16 * 32;
#pragma unroll
    for (int j = 0; j < 16; ++j) mine[j * 32 + lane] = __uint_as_float(give[j]);
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
#pragma unroll
    for (int j = 0; j < 16; ++j) got[j] = __float_as_uint(theirs[j * 32 + lane]);
    ++round;
  }
};

// One value of one token of one head tile, held by epilogue thread f = feature; all 128 epilogue
// threads call it together.  red: 4 floats, xs: 128 floats of shared memory.
__device__ __forceinline__ void qkv_finish(const QkvTail& tl, void* y, long long ldy, int m, int n0, int f, float value,
                                           float* red, float* xs) {
  const int head = n0 / BM;
  const int pos = tl.tok_pos[m];
  const bool is_q = head < tl.nh, is_k = !is_q && head < tl.nh + tl.nkv;
  size_t cache_row = 0;   // (page * kv heads + kv head): the page's rows of this kv head
  if (!is_q && tl.page_table) {
    const int slot = tl.seq_slot[tl.tok_seq[m]];
    const int page = tl.page_table[(size_t)slot * tl.table_width + (pos / tl.page_size) % tl.table_width];
    cache_row = (size_t)page * tl.nkv + (head - tl.nh - (is_k ? 0 : tl.nkv));
  }
  if (!is_q && !is_k) {   // a value head: as it is, into the transposed page
    if (tl.page_table) tl.vcache[(cache_row * BM + f) * tl.page_size + pos % tl.page_size] = __float2bfloat16_rn(value);
    else ((bf16*)y)[(size_t)m * ldy + n0 + f] = __float2bfloat16_rn(value);
    return;
  }
  const float* w = is_q ? tl.q_weight : tl.k_weight;
  float c = 1.f, sn = 0.f;
  if (tl.inv_freq) sincosf((float)pos * tl.inv_freq[f & 63], &sn, &c);
  float x = value;
  if (w) {
    const float part = warp_sum(value * value);
    if ((f & 31) == 0) red[f >> 5] = part;
    asm volatile("bar.sync 1, 128;" ::: "memory");
    x = value * (1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)BM + tl.eps)) * w[f];
  }
  xs[f] = x;
  asm volatile("bar.sync 1, 128;" ::: "memory");
  const float other = xs[f ^ 64];
  asm volatile("bar.sync 1, 128;" ::: "memory");   // red and xs may be written again
  // rotate-half: dims i and i + 64 are a pair (a, b): a' = a cos - b sin, b' = b cos + a sin
  float r = f < 64 ? x * c - other * sn : x * c + other * sn;
  if (is_q) r *= tl.q_scale;
  const bf16 o = __float2bfloat16_rn(r);
  if (is_q || !tl.page_table) ((bf16*)y)[(size_t)m * ldy + n0 + f] = o;
  else tl.kcache[(cache_row * tl.page_size + pos % tl.page_size) * BM + f] = o;
}

// ---- the same per-head work for prompts, in the persistent kernel's epilogue -------------------
// There a warp holds, for its lane's feature, 32 tokens of the tile at a time (x[0..31]), and the
// four epilogue warps together hold the head's 128 features of those tokens.
//
// Sum over the warp's 32 lanes of each of 32 values, lane l ending up with the sum of value l:
// at every step a lane keeps one half of its values and gives the other half to its partner,
// 31 shuffles in all instead of five per value.
__device__ __forceinline__ float lanes_sum_32(float (&v)[32], int lane) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
    const bool upper = (lane & off) != 0;
#pragma unroll
    for (int i = 0; i < off; ++i) {
      const float give = upper ? v[i] : v[i + off];
      const float keep = upper ? v[i + off] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, give, off);
    }
  }
  return v[0];
}

__device__ __forceinline__ uint32_t pack_two_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(const uint32_t*)&v;
}

// Shared memory of the prompt tail: the epilogue warps' exchange (the other half of a rotation
// pair lives 64 features away, in warp w ^ 2; value tiles are transposed through the same memory)
// and the warps' partial sums of squares.
struct PromptTailShared {
  float* exchange;   // [4 warps][32 tokens][32 lanes]
  float* partial;    // [4 warps][32 tokens]
};

// One round: tokens m_first .. m_first + 31 of head `head` (features 32 * warp + lane), the raw
// products in x.  Queries leave through `tile_out`; keys and values go to the cache.
// `warp`: which quarter of the head's features the warp holds (0 .. 3); `bar`: the named barrier of
// the four warps that share the round.
template <int MODE, int SLOT>
__device__ __forceinline__ void qkv_prompt_round(const QkvTail& tl, float (&x)[32], int head, int warp, int lane, int m_first,
                                                 int M, int Nq, const PromptTailShared& sh, TileOut<MODE, SLOT>& tile_out,
                                                 int bar) {
  const int f = warp * 32 + lane;
  const bool is_q = head < tl.nh, is_k = !is_q && head < tl.nh + tl.nkv;
  // Asked for first, used last: where this lane's token (m_first + lane) lives in the cache, and
  // the angles of the round's 32 tokens for this lane's dim.  Both are tables made once a step
  // from the step's inputs, so nothing here waits on a chain of lookups.
  int cache_row = 0, pos_in_page = 0;
  if (!is_q) {
    const int2 place = tl.token_place[min(m_first + lane, M - 1)];
    pos_in_page = place.y;
    cache_row = place.x * tl.nkv + (head - tl.nh - (is_k ? 0 : tl.nkv));
  }
  float2 cs[32];
  if (tl.rope_table && (is_q || is_k)) {
    const float2* tab = tl.rope_table + (f & 63);
#pragma unroll
    for (int j = 0; j < 32; ++j) cs[j] = tab[(size_t)min(m_first + j, M - 1) * 64];
  }
  if (!is_q && !is_k) {
    // ---- a value head: as it is, transposed into the page ([dim][position]).  Through shared
    // memory (two tokens to a word, rows 17 words apart: no two lanes in one bank), so that a
    // store covers 8 positions of one dim (16 bytes) where the 32 tokens are consecutive positions
    // of one page that start on a multiple of 8.
    uint32_t* mine = (uint32_t*)(sh.exchange + warp * 32 * 32);      // [32 features][17]
#pragma unroll
    for (int j = 0; j < 16; ++j) mine[lane * 17 + j] = pack_two_bf16(x[2 * j], x[2 * j + 1]);
    __syncwarp();
    const int row0 = __shfl_sync(0xffffffffu, cache_row, 0), p0 = __shfl_sync(0xffffffffu, pos_in_page, 0);
    const bool run = __all_sync(0xffffffffu, cache_row == row0 && pos_in_page == p0 + lane) && (p0 & 7) == 0 &&
                     m_first + 31 < M;
    if (run) {
      const int fl = lane >> 2, ch = lane & 3;              // 8 features an instruction, 4 chunks of 8 tokens
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int ff = 8 * i + fl;
        const uint32_t* src = mine + ff * 17 + 4 * ch;
        const uint4 v = make_uint4(src[0], src[1], src[2], src[3]);
        *(uint4*)(tl.vcache + ((size_t)row0 * BM + warp * 32 + ff) * tl.page_size + p0 + 8 * ch) = v;
      }
    } else {
      const bf16* mine16 = (const bf16*)mine;
      for (int j = 0; j < 32; ++j) {
        const int row = __shfl_sync(0xffffffffu, cache_row, j), pp = __shfl_sync(0xffffffffu, pos_in_page, j);
        if (m_first + j < M) tl.vcache[((size_t)row * BM + f) * tl.page_size + pp] = mine16[lane * 34 + j];
      }
    }
    __syncwarp();
    return;
  }
  // ---- a query or key head: RMSNorm over the head's 128 features, per token
  const float* w = is_q ? tl.q_weight : tl.k_weight;
  if (w) {
    float sq[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) sq[j] = x[j] * x[j];
    sh.partial[warp * 32 + lane] = lanes_sum_32(sq, lane);     // token `lane`, this warp's 32 features
    asm volatile("bar.sync %0, 128;" ::"r"(bar) : "memory");
    const float total = sh.partial[lane] + sh.partial[32 + lane] + sh.partial[64 + lane] + sh.partial[96 + lane];
    const float inv = 1.0f / sqrtf(total / (float)BM + tl.eps), wf = w[f];
#pragma unroll
    for (int j = 0; j < 32; ++j) x[j] = x[j] * __shfl_sync(0xffffffffu, inv, j) * wf;
  }
  // ---- rotation: dims i and i + 64 are a pair (a, b): a' = a cos - b sin, b' = b cos + a sin
  if (tl.rope_table) {
    float* mine = sh.exchange + warp * 32 * 32;
    const float* theirs = sh.exchange + (warp ^ 2) * 32 * 32;
#pragma unroll
    for (int j = 0; j < 32; ++j) mine[j * 32 + lane] = x[j];
    asm volatile("bar.sync %0, 128;" ::"r"(bar) : "memory");
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float other = theirs[j * 32 + lane];
      x[j] = f < 64 ? x[j] * cs[j].x - other * cs[j].y : x[j] * cs[j].x + other * cs[j].y;
    }
  }
  if (is_q) {
    uint8_t* p = tile_out.next(lane);
#pragma unroll
    for (int j = 0; j < 32; ++j) tile_out.put(p, j, lane, x[j] * tl.q_scale);
    tile_out.post(p, lane, head * BM + warp * 32, m_first, Nq);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int row = __shfl_sync(0xffffffffu, cache_row, j), pp = __shfl_sync(0xffffffffu, pos_in_page, j);
      if (m_first + j < M) tl.kcache[((size_t)row * tl.page_size + pp) * BM + f] = __float2bfloat16_rn(x[j]);
    }
  }
  // With both steps on, the barrier of each keeps the other's memory safe for the next round;
  // with one alone, a warp could write the next round's values while another still reads these.
  if ((w != nullptr) != (tl.rope_table != nullptr)) asm volatile("bar.sync %0, 128;" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ------------------------------------------------------------------ the kernel
// grid = (token tiles, feature tiles, K splits); a cluster spans the K splits of one tile.
template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
               const __grid_constant__ CUtensorMap map_y, int y_tma, const float* __restrict__ bias,
               void* __restrict__ y, int M, int N, int K, long long ldy, const __grid_constant__ QkvTail tail) {
  constexpr bool DUAL = MODE == EPI_SWIGLU_BF16;
  __shared__ float qkv_red[MODE == EPI_QKV_BF16 ? 4 : 1], qkv_xs[MODE == EPI_QKV_BF16 ? BM : 1];
  constexpr uint32_t W_BYTES = BM * BK * 2, A_BYTES = (DUAL ? 2 : 1) * W_BYTES, B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t ACC_COLS = (DUAL ? 2 : 1) * BN, TMEM_COLS = ACC_COLS < 32 ? 32 : ACC_COLS;
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "tensor memory columns: a power of two up to 512");
  constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = (uint32_t*)(tmem_bar + 1);
  uint64_t* recv_bar = tmem_bar + 2;             // the other ranks' partial sums for this rank's tokens have arrived

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * BN, n0 = blockIdx.y * BM;
  const uint32_t nsplit = cluster_size(), split = cluster_rank();
  const int kb_total = (K + BK - 1) / BK;
  const int kb_begin = (int)((long long)kb_total * split / nsplit), kb_end = (int)((long long)kb_total * (split + 1) / nsplit);
  const int kb_count = kb_end - kb_begin;
  // with the inner dimension split, every rank adds a share of the tile's real tokens over all ranks
  const int real = min(M - m0, BN), share = (real + (int)nsplit - 1) / (int)nsplit;
  const int c0 = min(real, (int)split * share), c1 = min(real, c0 + share);
  // what this rank will receive then: every rank's 128 threads send one float per accumulator for
  // each of this rank's tokens, and each float counts its bytes on recv_bar where it lands
  const uint32_t recv_bytes = nsplit * (uint32_t)(c1 - c0) * (DUAL ? 2 : 1) * BM * 4;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tmem_bar, 1);
    mbar_init(recv_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (nsplit > 1) mbar_expect_tx(recv_bar, recv_bytes);
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  // With memory of its own for what the other ranks send, a rank may be written to at any time: all
  // that the senders need is that its mbarrier exists, which this barrier of the cluster says, long
  // before anyone has anything to send (its wait stands where the sending starts).
  const bool recv_apart = nsplit > 1 && tail.recv_apart != 0;
  if (recv_apart) cluster_arrive();

  if (warp == 4) {
    // ---------------- TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      // the weights do not depend on the kernel before this one: the first stages' W tiles are
      // asked for at once, x only after that kernel has finished
      const int pre = kb_count < STAGES ? kb_count : STAGES;
      for (int i = 0; i < pre; ++i) {
        uint8_t* a = smem + i * STAGE_BYTES;
        mbar_expect_tx(&full_bar[i], STAGE_BYTES);
        tma_load_2d(a, &map_w, (kb_begin + i) * BK, n0, &full_bar[i]);
        if (DUAL) tma_load_2d(a + W_BYTES, &map_w, (kb_begin + i) * BK, N + n0, &full_bar[i]);   // the up rows
      }
      pdl_wait_prior();
      for (int i = 0; i < pre; ++i) {
#ifdef GB_TEST_WITHHOLD_LOAD
        // Test build only: the tokens of the last block are never asked for, so its stage never
        // fills and the MMA thread's bounded wait runs out.  It shows that a wait which gives up
        // sets the status word and that the CTA still leaves through the common exit.
        if (i == kb_count - 1) continue;
#endif
        tma_load_2d(smem + i * STAGE_BYTES + A_BYTES, &map_x, (kb_begin + i) * BK, m0, &full_bar[i]);
      }
      for (int i = pre; i < kb_count; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1)) {
          atomicCAS(&g_status, ST_OK, ST_TIMEOUT_EMPTY);
          break;
        }
        uint8_t* a = smem + s * STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(a, &map_w, (kb_begin + i) * BK, n0, &full_bar[s]);
        if (DUAL) tma_load_2d(a + W_BYTES, &map_w, (kb_begin + i) * BK, N + n0, &full_bar[s]);   // the up rows
#ifdef GB_TEST_WITHHOLD_LOAD
        if (i == kb_count - 1) continue;
#endif
        tma_load_2d(a + A_BYTES, &map_x, (kb_begin + i) * BK, m0, &full_bar[s]);
      }
      // the last load is on its way: the next kernel may move in and ask for its first weights
      // while this one finishes (earlier, its CTAs would only take room from this kernel's)
      pdl_release_next();
    }
    __syncwarp();
  } else if (warp == 5) {
    // ---------------- MMA issue
    if (lane == 0) {
      bool ok = true;
      for (int i = 0; i < kb_count && ok; ++i) {
        const int s = i % STAGES;
        if (!mbar_wait(&full_bar[s], (i / STAGES) & 1)) {
          atomicCAS(&g_status, ST_OK, ST_TIMEOUT_FULL);
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a = smem_u32(smem + s * STAGE_BYTES);
        const uint64_t adesc = smem_desc(a), bdesc = smem_desc(a + A_BYTES), udesc = smem_desc(a + W_BYTES);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k) {  // 32 bytes further along the swizzled row per step
          tc_mma(tmem, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), IDESC, (i > 0 || k > 0) ? 1u : 0u);
          if (DUAL) tc_mma(tmem + BN, udesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), IDESC, (i > 0 || k > 0) ? 1u : 0u);
        }
        tc_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
      }
      tc_commit(tmem_bar);         // the accumulator is complete once everything issued has run
    }
    __syncwarp();
  }

  // ---------------- epilogue (warps 0-3); the other warps wait at the barriers below
  bool have_acc = false;
  float bias_v = 0.f, old[8];
  __shared__ float row_scale[64], sq_part[4][32];
  const NormLink& link = tail.link;
  if (warp < 4) {
    pdl_wait_prior();   // y may be read (accumulate) and is written: not before the kernel before is done
    const int n = n0 + warp * 32 + lane;
    bias_v = (bias && n < N) ? bias[n] : 0.f;
    if (link.in_partial) {
      // The scale of each of the tile's tokens, while the products run.  A token's sums of squares
      // (one per tile of the product that left them) are shared out over 128 / BN adjacent lanes,
      // four loads in flight each, and added up in a fixed order: the same bits every run.
      constexpr int TOK = BN < 64 ? BN : 64, PER = 128 / TOK;      // PER: 8, 4 or 2 lanes a token
      const int t = warp * 32 + lane, tok = t / PER, j = t % PER;
      float ss = 0.f;
      if (m0 + tok < M) {
        const float* col = link.in_partial + m0 + tok;
        for (int i = j; i < link.in_tiles; i += 4 * PER) {
          const float a = col[i * 64];
          const float b = i + PER < link.in_tiles ? col[(i + PER) * 64] : 0.f;
          const float c = i + 2 * PER < link.in_tiles ? col[(i + 2 * PER) * 64] : 0.f;
          const float d = i + 3 * PER < link.in_tiles ? col[(i + 3 * PER) * 64] : 0.f;
          ss += (a + b) + (c + d);
        }
      }
#pragma unroll
      for (int o = 1; o < PER; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (j == 0) row_scale[tok] = 1.0f / sqrtf(ss * link.in_inv_width + link.in_eps);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    if (MODE == EPI_ACCUMULATE_F32 && nsplit > 1) {
      // what this thread will add to: asked for now, so that the answer is there after the products
#pragma unroll
      for (int i = 0; i < 8; ++i) old[i] = (c0 + i < c1 && n < N) ? ((const float*)y)[(size_t)(m0 + c0 + i) * ldy + n] : 0.f;
    }
    if (kb_count > 0) {
      have_acc = __all_sync(0xffffffffu, mbar_wait(tmem_bar, 0));   // the same answer in every lane
      if (!have_acc && lane == 0) atomicCAS(&g_status, ST_OK, ST_TIMEOUT_TMEM);
    }
    tc_fence_after();
  }
  if (nsplit > 1) {
    // Every rank sends each token's partial sums to the rank that finishes the token, into that
    // rank's shared memory (remote stores do not wait for an answer; each counts its bytes on the
    // receiver's mbarrier), and a rank adds what it received, in rank order, from its own shared
    // memory as soon as its own tokens' sums are all there: no second barrier of the cluster.
    // (Publishing in place and reading the other ranks' memory cost a round trip per token and a
    // second barrier before anyone could leave: 4.1 us from the last MMA to the last store with
    // eight ranks, measured inside a decode step.)  The memory is the pipeline's stages, so a rank
    // may be written to only when its MMAs are done: that is the one barrier, which every
    // thread arrives at as soon as this rank's accumulator is complete.  A rank may leave while
    // its own sends are still on their way: they need nothing of the sender any more, and the
    // receivers stay until everything they expect has arrived.
    float* recv = recv_apart ? (float*)(smem + STAGES * STAGE_BYTES + 1024) : (float*)smem;   // [rank][token of this rank's share][accumulator][BM]
    constexpr int NACC = DUAL ? 2 : 1;
    if (!recv_apart) cluster_arrive();   // in the stages: not before every rank's MMAs have read them
    cluster_wait();
    if (warp < 4) {
      const int f = warp * 32 + lane;
      const uint32_t acc = tmem + ((uint32_t)(warp * 32) << 16);
      int owner = 0, local = 0;   // of token c + j
#pragma unroll 1
      for (int c = 0; c < BN && c < real; c += 16) {
        uint32_t v[16], u[16];
        if (have_acc) {
          acc_load<DUAL>(acc, BN, c, v, u);
          tc_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = u[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c + j < real) {
            float* slot = recv + ((size_t)((int)split * share + local) * NACC) * BM + f;
            st_peer_f32_counted(slot, (uint32_t)owner, __uint_as_float(v[j]), recv_bar);
            if (DUAL) st_peer_f32_counted(slot + BM, (uint32_t)owner, __uint_as_float(u[j]), recv_bar);
            if (++local == share) {
              local = 0;
              ++owner;
            }
          }
        }
      }
    }
    if (warp < 4) {
      // no barrier of the cluster: this rank goes on when its own tokens' sums are all there
      if (!__all_sync(0xffffffffu, mbar_wait(recv_bar, 0)) && lane == 0) atomicCAS(&g_status, ST_OK, ST_TIMEOUT_RECV);
      const int f = warp * 32 + lane, n = n0 + f;
      const float out_g = (MODE == EPI_ACCUMULATE_F32 && link.out_weight && n < N) ? link.out_weight[n] : 0.f;
#pragma unroll 1
      for (int c = c0; c < c1; ++c) {
        const float* mine = recv + ((size_t)(c - c0) * NACC) * BM + f;
        const size_t rank_stride = (size_t)share * NACC * BM;
        float part[8], part_up[8];
#pragma unroll
        for (uint32_t r = 0; r < 8; ++r) {
          part[r] = r < nsplit ? mine[r * rank_stride] : 0.f;
          if (DUAL) part_up[r] = r < nsplit ? mine[r * rank_stride + BM] : 0.f;
        }
        float sum = part[0];
#pragma unroll
        for (int r = 1; r < 8; ++r) sum += part[r];
        const float sc = link.in_partial ? row_scale[c] : 1.f;
        sum *= sc;
        if (MODE == EPI_QKV_BF16) {   // every thread has the same tokens: they finish one together
          qkv_finish(tail, y, ldy, m0 + c, n0, f, sum + bias_v, qkv_red, qkv_xs);
          continue;
        }
        float final_r = 0.f;
        if (n < N) {
          if (DUAL) {
            float up = part_up[0];
#pragma unroll
            for (int r = 1; r < 8; ++r) up += part_up[r];
            sum = silu_mul(sum, up * sc);
          }
          const size_t idx = (size_t)(m0 + c) * ldy + n;
          if (MODE == EPI_ACCUMULATE_F32) {
            float prev = c - c0 < 8 ? 0.f : ((const float*)y)[idx];   // the first eight were asked for early
#pragma unroll
            for (int q = 0; q < 8; ++q) prev = (c - c0 == q) ? old[q] : prev;
            final_r = prev + sum + bias_v;
            ((float*)y)[idx] = final_r;
            if (link.out_weight) link.out_rows[(size_t)(m0 + c) * link.out_ld + n] = __float2bfloat16_rn(final_r * out_g);
          } else {
            emit<MODE>(y, idx, sum + bias_v);
          }
        }
        if (MODE == EPI_ACCUMULATE_F32 && link.out_weight) {   // this warp's 32 features of the token's sum of squares
          const float sq = warp_sum(final_r * final_r);
          if (lane == 0 && c - c0 < 32) sq_part[warp][c - c0] = sq;
        }
      }
      if (MODE == EPI_ACCUMULATE_F32 && link.out_weight) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int t = warp * 32 + lane;
        if (t < c1 - c0)
          link.out_partial[(size_t)blockIdx.y * 64 + m0 + c0 + t] = sq_part[0][t] + sq_part[1][t] + sq_part[2][t] + sq_part[3][t];
      }
    }
  } else if (warp < 4 && have_acc) {
    const int f = warp * 32 + lane, n = n0 + f;
    const float b = bias_v;
    // the pipeline's stages are idle by now: the pieces on their way out lie there
    TileOut<MODE> tile_out(&map_y, smem, warp);
    const bool by_tma = MODE != EPI_QKV_BF16 && y_tma != 0;
    constexpr bool BOTH = BN >= 32;   // 32 tokens per round
    const uint32_t acc = tmem + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
    for (int c = 0; c < BN; c += BOTH ? 32 : 16) {
      if (m0 + c >= M) break;
      uint32_t v[16], u[16], v2[16], u2[16];
      acc_load<DUAL>(acc, BN, c, v, u);
      if (BOTH) acc_load<DUAL>(acc, BN, c + 16, v2, u2);
      tc_wait_ld();
      if (link.in_partial) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float s1 = row_scale[c + j], s2 = BOTH ? row_scale[c + 16 + j] : 1.f;
          v[j] = __float_as_uint(__uint_as_float(v[j]) * s1);
          if (DUAL) u[j] = __float_as_uint(__uint_as_float(u[j]) * s1);
          if (BOTH) v2[j] = __float_as_uint(__uint_as_float(v2[j]) * s2);
          if (BOTH && DUAL) u2[j] = __float_as_uint(__uint_as_float(u2[j]) * s2);
        }
      }
      gate<DUAL>(v, u);
      if (BOTH) gate<DUAL>(v2, u2);
      if (by_tma) {
        tile_out.send(v, v2, BOTH, b, lane, n0 + warp * 32, m0 + c, N);
      } else if (MODE == EPI_QKV_BF16) {
        for (int j = 0; j < 16; ++j)   // the token count is the same for every thread
          if (m0 + c + j < M) qkv_finish(tail, y, ldy, m0 + c + j, n0, f, __uint_as_float(v[j]) + b, qkv_red, qkv_xs);
        if (BOTH)
          for (int j = 0; j < 16; ++j)
            if (m0 + c + 16 + j < M) qkv_finish(tail, y, ldy, m0 + c + 16 + j, n0, f, __uint_as_float(v2[j]) + b, qkv_red, qkv_xs);
      } else {
        store_direct<MODE>(y, ldy, v, b, m0 + c, M, n, N);
        if (BOTH) store_direct<MODE>(y, ldy, v2, b, m0 + c + 16, M, n, N);
      }
    }
    if (by_tma) tile_out.finish(lane);
  }
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  if (warp == 5) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
}

// ------------------------------------------------------------------ the persistent kernel for prompts
// One CTA per SM walks the output tiles (token tile fastest, so the CTAs that run together
// share the same rows of W).  The accumulator in tensor memory is double-buffered: while the
// four epilogue warps read tile i out of one buffer and store it, the MMA warp already fills the
// other with tile i + 1, and the TMA warp runs ahead through the shared-memory stages across
// tile borders.  In gated mode a tile's 128 rows of W are 64 gate rows and the 64 up rows of the same
// features, and the tile gives 64 features of the result: one accumulator and as
// many shared-memory bytes per MMA cycle as the plain product (two accumulators over 128 tokens
// read the tokens twice and ran at 735 cycles a block of 64 inner elements, against 547).
// Tile t of the walk: token tiles come in groups of 2,048 tokens; inside a group the token tile
// runs fastest and the feature tile slowest, and the groups follow one another.  The CTAs that run
// together then share a few rows of W and one group's rows of x (16 MB at 4,096 wide), which stay
// in L2 while W streams past once per group; with the token tile fastest over all tokens, a
// 16,384-token step read x again for every feature tile (measured: 2.5 GB from memory for the
// q/k/v product, whose operands are 0.18 GB).
__device__ __forceinline__ void tile_origin(int t, int tiles_m, int tiles_n, int bn, int tile_features, int& m0, int& n0) {
  const int group = max(1, 2048 / bn), per_group = group * tiles_n;
  const int g = t / per_group, r = t - g * per_group;
  const int gm = min(group, tiles_m - g * group);
  m0 = (g * group + r % gm) * bn;
  n0 = (r / gm) * tile_features;
}


// The work of one CTA of the persistent kernel: tiles blockIdx.x, + gridDim.x, and so on.  Where
// the last round of tiles would leave SMs idle, a product that adds into its result (`split` > 1)
// cuts each tile of that round into `split` parts along the inner dimension, and the CTAs walk
// those parts the same way, part 0 of every tile first: the CTAs stay in step along the inner
// dimension, as they are in the whole rounds, so that what one fetches the others find in L2.
// (Equal shares of all tiles' blocks laid end to end keep every SM as busy, but each CTA is then
// at another place of the inner dimension: measured 6 % slower over a prompt of 8B layer sizes,
// whose 100 MB of W and 50 MB of x in the down product no longer pass through L2 once.)
struct TileWalk {
  int t, kb0, kb1, part;   // the segment: blocks [kb0, kb1) of tile t; which part of the tile it is
  int at, whole, last, split, kb_total;
  __device__ __forceinline__ TileWalk(int tiles, int kb_total_, int split_) : at(blockIdx.x), split(split_), kb_total(kb_total_) {
    whole = split > 1 ? tiles - tiles % (int)gridDim.x : tiles;   // tiles of the full rounds
    last = tiles - whole;                                          // tiles of the round that is cut
    set();
  }
  __device__ __forceinline__ void set() {
    if (at < whole) {
      t = at;
      part = 0;
      kb0 = 0;
      kb1 = kb_total;
    } else if (more()) {
      const int p = at - whole;
      part = p / last;
      t = whole + p - part * last;
      kb0 = (int)((long long)part * kb_total / split);
      kb1 = (int)((long long)(part + 1) * kb_total / split);
    }
  }
  __device__ __forceinline__ bool more() const { return at < whole + last * split; }
  __device__ __forceinline__ bool shared() const { return at >= whole; }   // one of several parts of its tile
  __device__ __forceinline__ void next() {
    at += gridDim.x;
    set();
  }
};

// The q/k/v mode has eight epilogue warps, two to each quarter of tensor memory's lanes (a warp
// reaches the quarter warp % 4): warps 0-3 take the even rounds of 32 tokens of a tile, warps 6-9
// the odd ones.  Its epilogue is work, not stores (a round is 2.9 us for four warps), and at
// short inner dimensions (2,560: 16 us of MMAs a tile) it, not the MMAs, set the product's time.
constexpr int PERSISTENT_QKV_THREADS = 320, QKV_STAGING_BYTES = 65 * 1024;   // pieces 32 KB, exchange 2 x 16 KB, sums 1 KB

template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(MODE == EPI_QKV_BF16 ? PERSISTENT_QKV_THREADS : THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                          const __grid_constant__ CUtensorMap map_y, int y_tma, const float* __restrict__ bias,
                          void* __restrict__ y, int M, int N, int K, long long ldy, int bn,
                          const __grid_constant__ QkvTail tail, int split_last, int* __restrict__ part_flags) {
  constexpr bool GATED = MODE == EPI_SWIGLU_BF16;   // rows of a tile: 16 gate, 16 up, ... (see gate_rows)
  // the last round's tiles in parts along the inner dimension: only where parts can be added
  const int split = MODE == EPI_ACCUMULATE_F32 ? max(split_last, 1) : 1;
  constexpr bool QKV = MODE == EPI_QKV_BF16;        // a tile is one head: norm, rotation, cache write (qkv_prompt_round)
  constexpr int TILE_F = GATED ? BM / 2 : BM;       // features of the result per tile
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
  constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t ACC_COLS = BN, TMEM_COLS = 2 * ACC_COLS;
  static_assert(TMEM_COLS == 256 || TMEM_COLS == 512, "two accumulator buffers: 256 or 512 columns");
  // bn: tokens per tile, a multiple of 16 up to BN (BN sizes the stages and the accumulators)
  const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
  const uint32_t stage_tx = A_BYTES + (uint32_t)bn * BK * 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* full_bar = (uint64_t*)(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* acc_full = empty_bar + STAGES;     // 2: the MMA warp has finished a tile in that buffer
  uint64_t* acc_empty = acc_full + 2;          // 2: the epilogue warps have read it out
  uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
  uint8_t* out_staging = smem + STAGES * STAGE_BYTES + 1024;   // past the barriers; OUT_STAGING_BYTES
  // gated: the pieces are 16 tokens of bfloat16 (1 KB), and the pairs' exchange has the upper half
  constexpr int SLOT = (GATED || QKV) ? OUT_STAGING_BYTES / 2 / (4 * PIECES) : PIECE_BYTES;
  static_assert(!GATED || (SLOT >= 16 * PIECE_FEATURES * 2 && OUT_STAGING_BYTES / 2 >= EXCHANGE_BYTES), "gated staging");
  // q/k/v: eight warps' bfloat16 pieces of 32 tokens (32 KB), then each group of four warps' exchange
  // (16 KB each), then their partial sums
  static_assert(!QKV || (SLOT >= PIECE_TOKENS * PIECE_FEATURES * 2 && 8 * PIECES * SLOT == 32 * 1024), "q/k/v staging");
  static_assert((2 * STAGES + 4) * 8 + 16 <= 1024, "the barriers have 1 KB");
  constexpr int EPI_WARPS = QKV ? 8 : 4;
  __shared__ int epilogue_gave_up;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (M + bn - 1) / bn, tiles_n = (N + TILE_F - 1) / TILE_F, tiles = tiles_m * tiles_n;
  const int kb_total = (K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], EPI_WARPS);
    }
    epilogue_gave_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    // ---------------- TMA producer: all of this CTA's tiles, one stream of stages
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
      pdl_wait_prior();
      uint32_t it = 0;
      bool ok = true;
      for (TileWalk w(tiles, kb_total, split); w.more() && ok; w.next()) {
        int m0, n0;
        tile_origin(w.t, tiles_m, tiles_n, bn, TILE_F, m0, n0);
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          if (it >= STAGES && !mbar_wait(&empty_bar[s], ((it / STAGES) - 1) & 1)) {
            atomicCAS(&g_status, ST_OK, ST_TIMEOUT_EMPTY);
            ok = false;
            break;
          }
          uint8_t* a = smem + s * STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], stage_tx);
          if (GATED) {   // map_w is cut into boxes of 64 rows: the gate rows, then the same features' up rows
            // (a request costs the issuing thread about 75 cycles: boxes of 16 rows, which would let a
            // warp gate without shared memory, made nine requests a block and the producer the limit)
            tma_load_2d(a, &map_w, kb * BK, n0, &full_bar[s]);
            tma_load_2d(a + A_BYTES / 2, &map_w, kb * BK, N + n0, &full_bar[s]);
          } else {
            tma_load_2d(a, &map_w, kb * BK, n0, &full_bar[s]);
          }
          tma_load_2d(a + A_BYTES, &map_x, kb * BK, m0, &full_bar[s]);
        }
      }
      pdl_release_next();   // all loads issued: the next kernel may move in
    }
    __syncwarp();
  } else if (warp == 5) {
    // ---------------- MMA issue
    if (lane == 0) {
      uint32_t it = 0, i = 0;
      bool ok = true;
      for (TileWalk w(tiles, kb_total, split); w.more() && ok; w.next(), ++i) {
        const uint32_t b = i & 1;
        if (i >= 2 && !mbar_wait(&acc_empty[b], ((i >> 1) - 1) & 1)) {   // the epilogue has read this buffer out
          atomicCAS(&g_status, ST_OK, ST_TIMEOUT_TMEM);
          break;
        }
        tc_fence_after();
        const uint32_t d = tmem + b * ACC_COLS;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const uint32_t s = it % STAGES;
          if (!mbar_wait(&full_bar[s], (it / STAGES) & 1)) {
            atomicCAS(&g_status, ST_OK, ST_TIMEOUT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a = smem_u32(smem + s * STAGE_BYTES);
          const uint64_t adesc = smem_desc(a), bdesc = smem_desc(a + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma(d, adesc + (uint64_t)(k * 2), bdesc + (uint64_t)(k * 2), idesc, (kb > w.kb0 || k > 0) ? 1u : 0u);
          tc_commit(&empty_bar[s]);
        }
        tc_commit(&acc_full[b]);
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue warps: lane = feature, column = token
    pdl_wait_prior();
    const int quarter = warp & 3, group = warp >= 6 ? 1 : 0;          // group 1: the q/k/v mode's second four
    const int f = GATED ? (warp & 1) * 32 + lane : quarter * 32 + lane;   // this lane's feature of the tile
    const bool is_up = GATED && warp >= 2;
    TileOut<MODE, SLOT> tile_out(&map_y, out_staging, group * 4 + quarter);
    GateExchange exchange(out_staging + OUT_STAGING_BYTES / 2, warp);
    const PromptTailShared tail_shared{(float*)(out_staging + 32 * 1024 + group * 16 * 1024),
                                       (float*)(out_staging + 64 * 1024) + group * 4 * 32};
    const bool both = bn % 32 == 0;   // 32 tokens per round; the result's map is cut to match
    uint32_t i = 0;
    for (TileWalk w(tiles, kb_total, split); w.more(); w.next(), ++i) {
      const uint32_t b = i & 1;
      int m0, n0;
      tile_origin(w.t, tiles_m, tiles_n, bn, TILE_F, m0, n0);
      const int n = n0 + f;
      bool have = __all_sync(0xffffffffu, mbar_wait(&acc_full[b], (i >> 1) & 1));
      if (!have && lane == 0) atomicCAS(&g_status, ST_OK, ST_TIMEOUT_TMEM);
      if (GATED || QKV) {   // the warps meet at barriers below: they leave together or not at all
        if (!have && lane == 0) epilogue_gave_up = 1;
        asm volatile("bar.sync 3, %0;" ::"n"(EPI_WARPS * 32) : "memory");
        have = epilogue_gave_up == 0;
      }
      if (!have) break;
      tc_fence_after();
      const float bv = (bias && n < N && w.kb0 == 0) ? bias[n] : 0.f;
      // The parts of a tile are added in their order along the inner dimension, so that the sums
      // have the same bits every run: a word per tile and warp counts the parts whose sums are in
      // memory, part q adds when it reads q (its predecessors were walked earlier, or at the same
      // time by CTAs that wait for nothing later than this one does), and the last part puts the
      // word back to zero.
      int* word = w.shared() ? part_flags + (w.t - w.whole) * 4 + warp : nullptr;
      if (MODE == EPI_ACCUMULATE_F32 && word && w.part > 0) {
        if (lane == 0) {
          bool there = false;
          for (uint32_t spin = 0; spin < WAIT_LIMIT && !there; ++spin) {
            int v;
            asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
            there = v == w.part;
          }
          if (!there) atomicCAS(&g_status, ST_OK, ST_TIMEOUT_PART);
        }
        __syncwarp();
      }
      const uint32_t acc = tmem + ((uint32_t)(quarter * 32) << 16) + b * ACC_COLS;
#pragma unroll 1
      for (int c = QKV ? 32 * group : 0; c < bn; c += QKV ? 64 : (both ? 32 : 16)) {
        if (m0 + c >= M) break;
        uint32_t v[16], v2[16];
        tc_ld16(acc + c, v);
        if (both) tc_ld16(acc + c + 16, v2);
        tc_wait_ld();
        if (GATED) {
          // 32 tokens: the gate warp gives its last 16 and finishes the first 16, the up warp the other
          // way round; 16 tokens: the up warp gives, the gate warp finishes
          uint32_t got[16];
          exchange.swap((both && !is_up) ? v2 : v, is_up, lane, got);
          if (both || !is_up) {
            const uint32_t (&g)[16] = is_up ? got : v;
            const uint32_t (&u)[16] = is_up ? v2 : got;
            const int row = m0 + c + (is_up ? 16 : 0);
            float r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = silu_mul(__uint_as_float(g[j]), __uint_as_float(u[j]));
            if (y_tma) {
              uint8_t* p = tile_out.next(lane);
#pragma unroll
              for (int j = 0; j < 16; ++j) tile_out.put(p, j, lane, r[j]);
              tile_out.post(p, lane, n0 + (warp & 1) * 32, row, N);
            } else if (n < N) {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (row + j < M) emit<MODE>(y, (size_t)(row + j) * ldy + n, r[j]);
            }
          }
        } else if (QKV) {
          float x[32];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            x[j] = __uint_as_float(v[j]) + bv;
            x[16 + j] = __uint_as_float(v2[j]) + bv;
          }
          qkv_prompt_round<MODE, SLOT>(tail, x, n0 / BM, quarter, lane, m0 + c, M, tail.nh * BM, tail_shared, tile_out, 1 + group);
        } else if (y_tma) {
          tile_out.send(v, v2, both, bv, lane, n0 + warp * 32, m0 + c, N);
        } else {
          store_direct<MODE>(y, ldy, v, bv, m0 + c, M, n, N);
          if (both) store_direct<MODE>(y, ldy, v2, bv, m0 + c + 16, M, n, N);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[b]);
      if (MODE == EPI_ACCUMULATE_F32 && word) {
        if (lane == 0) {
          tma_store_wait_all();    // this warp's sums are in memory
          __threadfence();
          asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(word), "r"(w.part + 1 < split ? w.part + 1 : 0) : "memory");
        }
        __syncwarp();
      }
    }
    if (y_tma || QKV) tile_out.finish(lane);
  }
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  if (warp == 5) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
}

// cos and sin of every packed token's angles, once per step for all layers: table[t][i] =
// (cos, sin)(float32(position of t) * inv_freq[i]) (src/kernels.rs:1525-1531).
__global__ void rope_table_kernel(const int* __restrict__ tok_pos, const float* __restrict__ inv_freq,
                                  float2* __restrict__ table, int ntok, int half) {
  pdl_release_next();
  pdl_wait_prior();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= ntok * half) return;
  float s, c;
  sincosf((float)tok_pos[i / half] * inv_freq[i % half], &s, &c);
  table[i] = make_float2(c, s);
}

// Where every packed token lives in a group's cache: place[t] = (page, position in the page), once
// per step for all the layers that share the group's page table.
__global__ void token_place_kernel(const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                   const int* __restrict__ seq_slot, const int* __restrict__ page_table, int table_width,
                                   int page_size, int2* __restrict__ place, int ntok) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= ntok) return;
  const int pos = tok_pos[t], slot = seq_slot[tok_seq[t]];
  place[t] = make_int2(page_table[(size_t)slot * table_width + (pos / page_size) % table_width], pos % page_size);
}

// ------------------------------------------------------------------ host side

// The result's tensor map, and whether TMA can address the result at all.
struct OutMap {
  CUtensorMap map;
  int usable;
};
// bn: tokens per tile; the kernels send 32 tokens at a time where a tile has that many.
OutMap out_map(const void* y, int mode, int M, int N, long long ldy, int bn) {
  OutMap o = {};
  const bool f32 = mode == EPI_STORE_F32 || mode == EPI_ACCUMULATE_F32;
  o.usable = mode != EPI_QKV_BF16 && tensor_map_out(&o.map, y, (uint64_t)M, (uint64_t)N, (uint64_t)ldy * (f32 ? 4 : 2),
                                                    bn % 32 == 0 ? 32 : 16, 32, f32);
  return o;
}

template <int BN, int STAGES, int MODE>
int launch(const CUtensorMap& mw, const CUtensorMap& mx, const OutMap& my, const float* bias, void* y, int M, int N, int K,
           long long ldy, int splits, cudaStream_t stream, const QkvTail& tail = QkvTail{}) {
  constexpr int NW = MODE == EPI_SWIGLU_BF16 ? 2 : 1;
  constexpr size_t STAGE = (size_t)NW * BM * BK * 2 + BN * BK * 2;
  constexpr size_t SMEM0 = (size_t)STAGES * STAGE + (2 * STAGES + 1) * 8 + 16 + 1024;
  static_assert(SMEM0 <= 227 * 1024, "stages do not fit in shared memory");
  // The ranks' partial sums in memory of their own (no barrier of the cluster before the exchange)
  // where that costs no CTA an SM its place: [ranks][tokens a rank finishes][accumulators][128] floats
  // behind the stages and their kilobyte of barriers.
  size_t SMEM = SMEM0;
  QkvTail tail_ = tail;
  tail_.recv_apart = 0;
  if (splits > 1 && BN <= 64) {
    static int sms = 0;
    if (!sms) {
      int dev = 0;
      cudaGetDevice(&dev);
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    }
    const int real = M < BN ? M : BN, share = (real + splits - 1) / splits;
    const size_t recv = (size_t)splits * share * NW * BM * 4, apart = (size_t)STAGES * STAGE + 2048 + recv;
    const long long ctas = (long long)((M + BN - 1) / BN) * ((N + BM - 1) / BM) * splits;
    const int wanted = (int)((ctas + sms - 1) / sms), fit_now = (int)(227 * 1024 / (SMEM0 + 1024)), fit_apart = (int)(227 * 1024 / (apart + 1024));
    // ... and leaves half of an SM's shared memory to the CTAs of the next kernel, which start under
    // this one's tail and ask for their first weights: with the memory of their own, 8B layer sizes
    // at batch 1 got 3.5 % slower a step (two CTAs of 79 KB an SM), 0.6B sizes 4.2 % faster (one).
    if (sms > 0 && fit_apart >= (wanted < fit_now ? wanted : fit_now) && (size_t)wanted * (apart + 1024) <= 114 * 1024) {
      SMEM = apart;
      tail_.recv_apart = 1;
    }
  }
  static_assert(BN > 64 || (size_t)NW * (BN + 8) * BM * 4 <= (size_t)STAGES * STAGE, "the ranks' partial sums need the stage memory");
  static_assert((size_t)OUT_STAGING_BYTES <= (size_t)STAGES * STAGE, "the pieces on their way out need the stage memory");
  auto kernel = gemm_tc_kernel<BN, STAGES, MODE>;
  static size_t configured = 0;
  if (SMEM > configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return (int)cudaGetLastError();
    configured = SMEM;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((M + BN - 1) / BN, (N + BM - 1) / BM, splits);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = SMEM;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = GB_PDL ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, kernel, mw, mx, my.map, my.usable, bias, y, M, N, K, ldy, tail_);
}

template <int BN, int STAGES>
int launch_mode(int mode, const CUtensorMap& mw, const CUtensorMap& mx, const OutMap& my, const float* bias, void* y, int M,
                int N, int K, long long ldy, int splits, cudaStream_t stream, const QkvTail& tail = QkvTail{}) {
  switch (mode) {
    case EPI_STORE_BF16: return launch<BN, STAGES, EPI_STORE_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    case EPI_STORE_F32: return launch<BN, STAGES, EPI_STORE_F32>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    case EPI_ACCUMULATE_F32: return launch<BN, STAGES, EPI_ACCUMULATE_F32>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
  }
  return GB_ERR_ARG;
}

template <int BN, int STAGES, int MODE>
int launch_persistent(const CUtensorMap& mw, const CUtensorMap& mx, const OutMap& my, const float* bias, void* y, int M,
                      int N, int K, long long ldy, int bn, int ctas, cudaStream_t stream, const QkvTail& tail = QkvTail{},
                      int* part_flags = nullptr) {
  // stages, 1 KB of barriers, the pieces on their way out, 1 KB to align the base
  constexpr size_t STAGING = MODE == EPI_QKV_BF16 ? QKV_STAGING_BYTES : OUT_STAGING_BYTES;
  constexpr size_t SMEM = (size_t)STAGES * ((size_t)BM * BK * 2 + BN * BK * 2) + 1024 + STAGING + 1024;
  constexpr int NTHREADS = MODE == EPI_QKV_BF16 ? PERSISTENT_QKV_THREADS : THREADS;
  static_assert(SMEM <= 227 * 1024, "stages do not fit in shared memory");
  static_assert((2 * STAGES + 4) * 8 + 16 <= 1024, "the barriers have 1 KB");
  constexpr int TILE_F = MODE == EPI_SWIGLU_BF16 ? BM / 2 : BM;
  auto kernel = gemm_tc_persistent_kernel<BN, STAGES, MODE>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return (int)cudaGetLastError();
    configured = true;
  }
  const int tiles = ((M + bn - 1) / bn) * ((N + TILE_F - 1) / TILE_F);
  // Where the last round of tiles would leave SMs idle and TMA adds the sums into the result: that
  // round's tiles in `split` parts along the inner dimension.  What a split costs, in blocks of the
  // inner dimension: the rounds of parts it makes, and, since the parts of a tile add one after the
  // other, a wait of about one tile's way out (its adds and their completion: about 9 blocks' time
  // at 256 tokens) for every further part of the same tile that is walked in the same round.
  int split = 1, grid = tiles < ctas ? tiles : ctas;
  if (MODE == EPI_ACCUMULATE_F32 && part_flags && my.usable && tiles % ctas != 0) {
    const int last = tiles % ctas, kb_total = (K + BK - 1) / BK;
    const double way_out = 9.0 * bn / 256 + 1.0;
    double best = 0.92 * kb_total;
    for (int sp = 2; sp <= 8 && kb_total / sp >= 4; ++sp) {
      const int rounds = (last * sp + ctas - 1) / ctas;
      const int together = sp < (ctas + last - 1) / last ? sp : (ctas + last - 1) / last;   // parts of a tile in one round
      const double cost = (double)rounds * kb_total / sp + (together - 1) * way_out + (rounds - 1) * 1.0;
      if (cost < best) {
        best = cost;
        split = sp;
      }
    }
    if (split > 1) grid = last * split < ctas && tiles < ctas ? last * split : ctas;
  }
  gb_launch(kernel, dim3(grid), dim3(NTHREADS), SMEM, stream, mw, mx, my.map, my.usable, bias, y, M, N, K, ldy, bn, tail,
            split, part_flags);
  return gb_launch_status();
}

}  // namespace

// x: [M, K] bfloat16, rows ldx elements apart; w: [N, K] bfloat16 contiguous; y: [M, N], rows ldy apart.
// mode: 0 store bfloat16, 1 store float32, 2 add into float32, 3 w = [gate; up] of 2N rows and
// y[M, N] = silu(x gate^T) * (x up^T) in bfloat16.  bn: tokens per tile (16, 32, 64, 128, 256);
// splits: CTAs of a cluster sharing the inner dimension (1, 2, 4, 8; only with bn <= 64);
// stages: pipeline depth for bn <= 64 (4 or 8; other tiles have a fixed depth).
// Needs K % 8 == 0, ldx % 8 == 0 and 16-byte aligned x and w (TMA rules).
static int gemm_tc_with_link(const void* x, const void* w, const float* bias, void* y, int mode, int M, int N, int K,
                             long long ldx, long long ldy, int bn, int splits, int stages, const NormLink& link,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  QkvTail tail{};
  tail.link = link;
  if (link.in_partial && (M > 64 || bn > 64 || link.in_tiles <= 0)) return GB_ERR_SIZE;
  // leaving rows for a norm is the work of the ranks that finish a token: it needs the inner dimension split
  if (link.out_weight && (mode != EPI_ACCUMULATE_F32 || splits < 2 || M > 64 || !link.out_rows || !link.out_partial)) return GB_ERR_ARG;
  if (K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return GB_ERR_SIZE;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return GB_ERR_ARG;
  if (splits > 1 && bn > 64) return GB_ERR_ARG;
  CUtensorMap mw, mx;
  const bool swiglu = mode == EPI_SWIGLU_BF16;   // w is [2N, K]: gate rows, then up rows
  if (swiglu && bias) return GB_ERR_ARG;
  if (!tensor_map(&mw, w, (uint64_t)N * (swiglu ? 2 : 1), (uint64_t)K, (uint64_t)K * 2, BM)) return GB_ERR_ARG;
  if (!tensor_map(&mx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)bn)) return GB_ERR_ARG;
  const OutMap my = out_map(y, mode, M, N, ldy, bn);
  if (swiglu) {
    switch (bn) {
      case 16: return launch<16, 3, EPI_SWIGLU_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
      case 32: return launch<32, 3, EPI_SWIGLU_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
      case 64: return launch<64, 3, EPI_SWIGLU_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
      case 128: return launch<128, 4, EPI_SWIGLU_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
      case 256: return launch<256, 3, EPI_SWIGLU_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    }
    return GB_ERR_SIZE;
  }
  switch (bn) {
    // decoding: `stages` = 4 leaves room for three CTAs on an SM (their tiles then finish together),
    // 8 gives one CTA a deeper pipeline
    case 16:
      return stages == 8 ? launch_mode<16, 8>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail)
                         : launch_mode<16, 4>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    case 32:
      return stages == 8 ? launch_mode<32, 8>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail)
                         : launch_mode<32, 4>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    case 64:
      return stages == 8 ? launch_mode<64, 8>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail)
                         : launch_mode<64, 4>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    case 128:   // stages = 3: two CTAs fit an SM, and one's epilogue runs under the other's MMAs
      return stages == 3 ? launch_mode<128, 3>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail)
                         : launch_mode<128, 6>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    case 256: return launch_mode<256, 4>(mode, mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
  }
  return GB_ERR_SIZE;
}

GB_EXPORT int gb_gemm_tc(const void* x, const void* w, const float* bias, void* y, int mode, int M, int N, int K,
                         long long ldx, long long ldy, int bn, int splits, int stages, cudaStream_t stream) {
  return gemm_tc_with_link(x, w, bias, y, mode, M, N, K, ldx, ldy, bn, splits, stages, NormLink{}, stream);
}

// gb_gemm_tc with an RMSNorm taken into it (see NormLink; at most 64 tokens).  in_partial non-null:
// x holds bf16(residual * norm weight) and every token's results are multiplied by
// 1 / sqrt(sum of in_partial[0 .. in_tiles)[token] / in_width + in_eps).  out_weight non-null
// (mode 2, splits >= 2): besides adding into y, the kernel writes bf16(y * out_weight) to out_rows
// (rows out_ld apart) and this product's tiles' sums of squares to out_partial [ceil(N / 128)][64].
GB_EXPORT int gb_gemm_tc_linked(const void* x, const void* w, const float* bias, void* y, int mode, int M, int N, int K,
                                long long ldx, long long ldy, int bn, int splits, int stages, const float* in_partial,
                                int in_tiles, float in_eps, int in_width, const float* out_weight, void* out_rows,
                                long long out_ld, float* out_partial, cudaStream_t stream) {
  NormLink link{in_partial, in_tiles, in_eps, in_width > 0 ? 1.0f / (float)in_width : 0.f, out_weight, (bf16*)out_rows, out_ld,
                out_partial};
  return gemm_tc_with_link(x, w, bias, y, mode, M, N, K, ldx, ldy, bn, splits, stages, link, stream);
}

// The q/k/v product of a decode step with the per-head work in its epilogue (head size 128, at most
// 64 tokens): y[M, N] gets the queries (normed, rotated, scaled; N = (nh + 2 nkv) * 128, rows ldy
// apart; the key and value columns of y are written only when page_table is null), the cache the
// keys and values.  q_weight / k_weight null: no norm; inv_freq null: no rotation.
GB_EXPORT int gb_gemm_tc_qkv(const void* x, const void* w, const float* bias, void* y, int M, int N, int K, long long ldx,
                             long long ldy, int bn, int splits, const float* q_weight, const float* k_weight,
                             const float* inv_freq, float eps, float q_scale, int nh, int nkv, const int* tok_pos,
                             const int* tok_seq, const int* seq_slot, const int* page_table, int table_width,
                             int page_size, void* kcache, void* vcache, const float* in_partial, int in_tiles,
                             float in_eps, int in_width, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15)) return GB_ERR_SIZE;
  if (splits != 1 && splits != 2 && splits != 4 && splits != 8) return GB_ERR_ARG;
  if (in_partial && (in_tiles <= 0 || in_width <= 0)) return GB_ERR_ARG;
  if (M > 64 || nh <= 0 || nkv < 0 || N != (nh + 2 * nkv) * BM || !tok_pos) return GB_ERR_SIZE;
  if (page_table && (!tok_seq || !seq_slot || !kcache || !vcache || page_size <= 0)) return GB_ERR_ARG;
  if ((q_weight == nullptr) != (k_weight == nullptr)) return GB_ERR_ARG;
  CUtensorMap mw, mx;
  if (!tensor_map(&mw, w, (uint64_t)N, (uint64_t)K, (uint64_t)K * 2, BM)) return GB_ERR_ARG;
  if (!tensor_map(&mx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)bn)) return GB_ERR_ARG;
  const OutMap my = out_map(y, EPI_QKV_BF16, M, N, ldy, bn);   // not used: the tail writes to the cache
  QkvTail tail{q_weight, k_weight, inv_freq, tok_pos, tok_seq, seq_slot, page_table, (bf16*)kcache, (bf16*)vcache,
               eps, q_scale, nh, nkv, table_width, page_size};
  tail.link.in_partial = in_partial;     // x holds unscaled rows: see NormLink
  tail.link.in_tiles = in_tiles;
  tail.link.in_eps = in_eps;
  tail.link.in_inv_width = in_partial ? 1.0f / (float)in_width : 0.f;
  switch (bn) {
    case 16: return launch<16, 4, EPI_QKV_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    case 32: return launch<32, 4, EPI_QKV_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
    case 64: return launch<64, 4, EPI_QKV_BF16>(mw, mx, my, bias, y, M, N, K, ldy, splits, stream, tail);
  }
  return GB_ERR_SIZE;
}

// The same product for prompts (M > 64): one CTA per SM walks the tiles and the epilogue of a tile
// runs under the MMAs of the next.  mode as gb_gemm_tc; bn: tokens per tile, a multiple of 16 up to
// 256; ctas: CTAs to launch.  part_flags: null, or 4 * ctas int32 zeros: a product that adds into y
// may then cut the tiles of a last round that is not full into parts along the inner dimension;
// every launch leaves the words zero, and two launches that use the same words must not run at
// the same time.
GB_EXPORT int gb_gemm_tc_persistent(const void* x, const void* w, const float* bias, void* y, int mode, int M, int N,
                                    int K, long long ldx, long long ldy, int bn, int ctas, int* part_flags,
                                    cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ctas <= 0) return GB_ERR_SIZE;
  if (bn < 16 || bn > 256 || (bn % 16)) return GB_ERR_SIZE;
  const bool swiglu = mode == EPI_SWIGLU_BF16;
  if (swiglu && bias) return GB_ERR_ARG;
  CUtensorMap mw, mx;
  // gated: W in boxes of 64 rows; a tile is 64 gate rows and the same features' 64 up rows
  if (!tensor_map(&mw, w, (uint64_t)N * (swiglu ? 2 : 1), (uint64_t)K, (uint64_t)K * 2, swiglu ? BM / 2 : BM)) return GB_ERR_ARG;
  if (!tensor_map(&mx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)bn)) return GB_ERR_ARG;
  const OutMap my = out_map(y, mode, M, N, ldy, swiglu ? 16 : bn);   // gated: a warp sends 16 tokens at a time
  if (swiglu) {
    if (bn > 128) return launch_persistent<256, 4, EPI_SWIGLU_BF16>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream);
    return launch_persistent<128, 6, EPI_SWIGLU_BF16>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream);
  }
  if (bn > 128) {
    switch (mode) {
      case EPI_STORE_BF16: return launch_persistent<256, 4, EPI_STORE_BF16>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream);
      case EPI_STORE_F32: return launch_persistent<256, 4, EPI_STORE_F32>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream);
      case EPI_ACCUMULATE_F32:
        return launch_persistent<256, 4, EPI_ACCUMULATE_F32>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream, QkvTail{}, part_flags);
    }
  } else {
    switch (mode) {
      case EPI_STORE_BF16: return launch_persistent<128, 6, EPI_STORE_BF16>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream);
      case EPI_STORE_F32: return launch_persistent<128, 6, EPI_STORE_F32>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream);
      case EPI_ACCUMULATE_F32:
        return launch_persistent<128, 6, EPI_ACCUMULATE_F32>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream, QkvTail{}, part_flags);
    }
  }
  return GB_ERR_ARG;
}

// (cos, sin) of every packed token's angles: table [ntok][half] float2, for gb_gemm_tc_qkv_prompt.
GB_EXPORT int gb_rope_table(const int* tok_pos, const float* inv_freq, void* table, int ntok, int half,
                            cudaStream_t stream) {
  if (ntok <= 0 || half <= 0) return 0;
  if (!tok_pos || !inv_freq || !table) return GB_ERR_ARG;
  const long long total = (long long)ntok * half;
  gb_launch(rope_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, tok_pos, inv_freq,
            (float2*)table, ntok, half);
  return gb_launch_status();
}

// (page, position in the page) of every packed token: place [ntok] int2, for gb_gemm_tc_qkv_prompt.
GB_EXPORT int gb_token_place(const int* tok_pos, const int* tok_seq, const int* seq_slot, const int* page_table,
                             int table_width, int page_size, void* place, int ntok, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (!tok_pos || !tok_seq || !seq_slot || !page_table || !place || page_size <= 0 || table_width <= 0) return GB_ERR_ARG;
  gb_launch(token_place_kernel, dim3((ntok + 255) / 256), dim3(256), 0, stream, tok_pos, tok_seq, seq_slot, page_table,
            table_width, page_size, (int2*)place, ntok);
  return gb_launch_status();
}

// The q/k/v product of a prompt step (more than 64 tokens) with the per-head work in its epilogue
// (head size 128): y [M, nh * 128] (rows ldy apart) gets the queries, normed, rotated and scaled;
// the keys (normed, rotated) and the values go straight into the paged cache, at the places
// token_place ([M] (page, position in the page), see gb_token_place) names.  q_weight / k_weight
// null: no norm; rope_table ([M][64] (cos, sin), see gb_rope_table) null: no rotation.  ctas: CTAs
// to launch.
GB_EXPORT int gb_gemm_tc_qkv_prompt(const void* x, const void* w, const float* bias, void* y, int M, int N, int K,
                                    long long ldx, long long ldy, int ctas, const float* q_weight, const float* k_weight,
                                    const void* rope_table, float eps, float q_scale, int nh, int nkv,
                                    const void* token_place, int page_size, void* kcache, void* vcache,
                                    cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15) || ctas <= 0) return GB_ERR_SIZE;
  if (nh <= 0 || nkv < 0 || N != (nh + 2 * nkv) * BM) return GB_ERR_SIZE;
  if (nkv > 0 && (!token_place || !kcache || !vcache || page_size <= 0 || (page_size % 8))) return GB_ERR_ARG;
  if ((q_weight == nullptr) != (k_weight == nullptr)) return GB_ERR_ARG;
  if ((ldy % 8) || ((uintptr_t)y & 15)) return GB_ERR_SIZE;    // the queries leave by TMA
  const int bn = M <= 128 ? 128 : 256;
  CUtensorMap mw, mx;
  if (!tensor_map(&mw, w, (uint64_t)N, (uint64_t)K, (uint64_t)K * 2, BM)) return GB_ERR_ARG;
  if (!tensor_map(&mx, x, (uint64_t)M, (uint64_t)K, (uint64_t)ldx * 2, (uint32_t)bn)) return GB_ERR_ARG;
  const OutMap my = out_map(y, EPI_STORE_BF16, M, nh * BM, ldy, 32);
  if (!my.usable) return GB_ERR_ARG;
  QkvTail tail{q_weight, k_weight, nullptr, nullptr, nullptr, nullptr, nullptr, (bf16*)kcache, (bf16*)vcache,
               eps, q_scale, nh, nkv, 1, page_size, (const float2*)rope_table, (const int2*)token_place};
  if (bn > 128) return launch_persistent<256, 3, EPI_QKV_BF16>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream, tail);
  return launch_persistent<128, 4, EPI_QKV_BF16>(mw, mx, my, bias, y, M, N, K, ldy, bn, ctas, stream, tail);
}

// The status word: 0, or the first wait that ran out (1 operands, 2 free stage, 3 accumulator,
// 4 the other part of a shared tile, 5 the other ranks' partial sums).
// Synchronizes the device; for tests and health checks, not for the step.
GB_EXPORT int gb_gemm_tc_status(int reset) {
  int v = -1;
  if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset) {
    int zero = 0;
    cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
  }
  return v;
}
