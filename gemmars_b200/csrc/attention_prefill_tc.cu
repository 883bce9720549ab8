// bfloat16 causal grouped-query attention of packed prompts on the 5th-generation tensor cores
// (tcgen05, sm_100a), for head sizes 64 and 128.  Compiled for one head size (-DGB_HEAD_DIM=...).
//
// Mathematics as everywhere (src/model.rs:1187-1226, src/kernels.rs:1550-1561): the query at
// position p sees the keys lo..p of its own sequence, softmax in float32, o = sum p_j V[j].
//
// A CTA owns 128 consecutive tokens of one sequence for one query head and walks the cache one
// page (64 keys) at a time:
//   * the TMA warp brings the page's keys [64 x hd] and transposed values [hd x 64] into
//     128-byte-swizzled shared memory (two stages); both are K-major tiles as the cache stores them;
//   * the MMA warp issues S = Q K^T (M = 128 tokens, N = 64 keys) into one of two S buffers in
//     tensor memory, one page ahead of the softmax, and then O += P V (N = hd) once P is there;
//   * four softmax warps, one thread per token row, read their row of S with tcgen05.ld, mask it,
//     keep the running maximum and sum, write P in bfloat16 into shared memory in the operand
//     layout, and rescale the O accumulator in tensor memory when the maximum has moved.
// Two CTAs fit an SM (112 KB of shared memory, 256 columns of tensor memory each), so one CTA's
// softmax overlaps the other's MMAs.  Every mbarrier wait is bounded; a wait that runs out sets
// the status word and an abort flag that ends the CTA's other loops, and tensor memory is freed.
#include "tc_common.cuh"

#ifndef GB_HEAD_DIM
#define GB_HEAD_DIM 128
#endif

namespace {

constexpr int HD = GB_HEAD_DIM;
static_assert(HD == 64 || HD == 128, "the tensor-core prefill kernel takes head sizes 64 and 128");
constexpr int ROWS = 128, KEYS = 64, QH = HD / 64;
constexpr uint32_t Q_BYTES = ROWS * HD * 2, K_BYTES = KEYS * HD * 2, V_BYTES = HD * KEYS * 2, P_BYTES = ROWS * KEYS * 2;
constexpr uint32_t SMEM_TILES = Q_BYTES + 2 * K_BYTES + 2 * V_BYTES + P_BYTES;
constexpr uint32_t TMEM_COLS = 256, S_COL0 = 0, S_COL1 = 64, O_COL = 128;
constexpr uint32_t IDESC_S = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(KEYS >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(ROWS >> 4) << 24);
constexpr float RESCALE_STEP = 8.0f;   // how far a row's maximum may outgrow its reference before O is rescaled
constexpr float LOG2E = 1.4426950408889634f;

__device__ int g_attn_status;   // 0, or the barrier whose wait ran out first (1..6)

__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t* v) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
        "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]),
        "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]),
        "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// A bounded wait that also gives up when another warp of the CTA already has.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort, int code) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255) == 255 && *abort) return false;
  }
  *abort = 1;
  atomicCAS(&g_attn_status, 0, code);
  return false;
}


__device__ __forceinline__ float ex2(float x) {   // 2^x, one instruction; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}

// grid (query heads, token tiles upper bound); block 192: warps 0-3 softmax, 4 TMA, 5 MMA.
__global__ void __launch_bounds__(192, 2)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out, long long out_stride,
                            const int* __restrict__ page_table, int table_width, int nkv,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ seq_start,
                            const int* __restrict__ seq_slot, int n_seqs, int nh, int window) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* q_smem = smem;
  uint8_t* k_smem = q_smem + Q_BYTES;          // two stages
  uint8_t* v_smem = k_smem + 2 * K_BYTES;      // two stages
  uint8_t* p_smem = v_smem + 2 * V_BYTES;
  uint64_t* bars = (uint64_t*)(smem + SMEM_TILES);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2: a page of keys has arrived
  uint64_t* k_empty = bars + 3;       // 2: the S product that read it is done
  uint64_t* v_full = bars + 5;        // 2: a page of values has arrived
  uint64_t* v_empty = bars + 7;       // 2: the P V product that read it is done
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* s_empty = bars + 11;      // 2
  uint64_t* p_full = bars + 13;       // 1
  uint64_t* o_done = bars + 14;       // 1
  uint32_t* tmem_slot = (uint32_t*)(bars + 15);
  volatile int* abort = (volatile int*)(tmem_slot + 1);

  pdl_wait_prior();
  // ---- which sequence and which 128-token tile of it.  The grid is (heads, tiles) and the tiles are
  // taken from the last down: a causal tile's work grows with its place in the sequence (2 to 34
  // pages in a 2,048-token prompt), and CTAs start in the order of the grid, so the long ones of
  // all heads go first and the short ones fill the end of the kernel.
  int b = 0, tile = gridDim.y - 1 - blockIdx.y;
  for (; b < n_seqs; ++b) {
    const int tiles = (cu_seqlens[b + 1] - cu_seqlens[b] + ROWS - 1) / ROWS;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (b >= n_seqs) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int head = blockIdx.x, kvh = head / (nh / nkv);
  const int seq_len = cu_seqlens[b + 1] - cu_seqlens[b];
  const int first = tile * ROWS;
  const int rows_valid = min(ROWS, seq_len - first);
  const int slot = seq_slot[b], start = seq_start[b];
  const int tok0 = cu_seqlens[b] + first;
  const int pos_last = start + first + rows_valid - 1;
  const int lo_first = window > 0 ? max(0, start + first + 1 - window) : 0;
  const int kt_begin = lo_first / KEYS, n_tiles = pos_last / KEYS + 1 - kt_begin;

  if (threadIdx.x == 0) {
    if (smem_u32(smem) & 1023u) {   // the swizzled tiles need 1024-byte alignment
      *abort = 1;
      atomicCAS(&g_attn_status, 0, 7);
    } else {
      *abort = 0;
    }
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(o_done, 1);
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
    // ---------------- TMA: the query tile once, then one page of keys and values per step
    if (lane == 0 && !*abort) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
      mbar_expect_tx(q_full, Q_BYTES);
      for (int h = 0; h < QH; ++h) tma_load_2d(q_smem + h * (ROWS * 128), &map_q, head * HD + h * 64, tok0, q_full);
      // Keys and values have stages and barriers of their own: a stage of keys is free as soon as
      // the S product that read it is done, long before the P V product frees the values of the same
      // page, so the keys of page j + 2 are on their way while page j is still being worked on
      // (with one barrier for both, the next S product waited a full round trip to memory behind
      // every P V product: 3,400 cycles a page against 640 of MMAs).  The thread takes whichever
      // load can go next.
      int jk = 0, jv = 0;
      uint32_t spins = 0;
      while ((jk < n_tiles || jv < n_tiles) && !*abort) {
        bool moved = false;
        if (jk < n_tiles && (jk < 2 || mbar_try_wait(&k_empty[jk & 1], ((jk >> 1) - 1) & 1))) {
          const int sidx = jk & 1;
          const int page = page_table[(size_t)slot * table_width + (kt_begin + jk) % table_width];
          const int row = page * nkv + kvh;
          mbar_expect_tx(&k_full[sidx], K_BYTES);
          for (int h = 0; h < QH; ++h)
            tma_load_2d(k_smem + sidx * K_BYTES + h * (KEYS * 128), &map_k, h * 64, row * KEYS, &k_full[sidx]);
          ++jk;
          moved = true;
        }
        if (jv < n_tiles && jv < jk && (jv < 2 || mbar_try_wait(&v_empty[jv & 1], ((jv >> 1) - 1) & 1))) {
          const int sidx = jv & 1;
          const int page = page_table[(size_t)slot * table_width + (kt_begin + jv) % table_width];
          const int row = page * nkv + kvh;
          mbar_expect_tx(&v_full[sidx], V_BYTES);
          tma_load_2d(v_smem + sidx * V_BYTES, &map_v, 0, row * HD, &v_full[sidx]);
          ++jv;
          moved = true;
        }
        if (moved) {
          spins = 0;
        } else if (++spins > WAIT_LIMIT) {
          *abort = 1;
          atomicCAS(&g_attn_status, 0, 1);
          break;
        }
      }
    }
    if (lane == 0) pdl_release_next();   // the last page is on its way: the next kernel may move in
    __syncwarp();
  } else if (warp == 5) {
    // ---------------- MMA issue: S up to two pages ahead of the softmax, and O += P V as soon as a
    // P is there; whichever can go next (neither waits for the other's operands)
    if (lane == 0 && !*abort && wait_or_abort(q_full, 0, abort, 2)) {
      int js = 0, jp = 0;   // next S, next P V
      uint32_t spins = 0;
      while (jp < n_tiles && !*abort) {
        bool moved = false;
        if (js < n_tiles && mbar_try_wait(&k_full[js & 1], (js >> 1) & 1) &&
            (js < 2 || mbar_try_wait(&s_empty[js & 1], ((js >> 1) - 1) & 1))) {
          const int sidx = js & 1;
          tc_fence_after();
          const uint32_t d = tmem + (sidx ? S_COL1 : S_COL0);
#pragma unroll
          for (int h = 0; h < QH; ++h) {
            const uint64_t qd = smem_desc(smem_u32(q_smem + h * (ROWS * 128)));
            const uint64_t kd = smem_desc(smem_u32(k_smem + sidx * K_BYTES + h * (KEYS * 128)));
#pragma unroll
            for (int k = 0; k < 4; ++k) tc_mma(d, qd + (uint64_t)(k * 2), kd + (uint64_t)(k * 2), IDESC_S, (h > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&s_full[sidx]);
          tc_commit(&k_empty[sidx]);
          ++js;
          moved = true;
        }
        if (jp < js && mbar_try_wait(p_full, jp & 1) && mbar_try_wait(&v_full[jp & 1], (jp >> 1) & 1)) {
          tc_fence_after();
          const uint64_t pd = smem_desc(smem_u32(p_smem));
          const uint64_t vd = smem_desc(smem_u32(v_smem + (jp & 1) * V_BYTES));
#pragma unroll
          for (int k = 0; k < 4; ++k) tc_mma(tmem + O_COL, pd + (uint64_t)(k * 2), vd + (uint64_t)(k * 2), IDESC_PV, (jp > 0 || k > 0) ? 1u : 0u);
          tc_commit(o_done);
          tc_commit(&v_empty[jp & 1]);
          ++jp;
          moved = true;
        }
        if (moved) {
          spins = 0;
        } else if (++spins > WAIT_LIMIT) {
          *abort = 1;
          atomicCAS(&g_attn_status, 0, 3);
          break;
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- softmax: thread = token row = tensor-memory lane
    const int r = warp * 32 + lane;
    const bool valid = r < rows_valid;
    const int pos = valid ? start + first + r : -1;
    const int lo = (window > 0 && valid) ? max(0, pos + 1 - window) : 0;
    const uint32_t lane_addr = tmem + ((uint32_t)(warp * 32) << 16);
    float m = -INFINITY, l = 0.f;
    bool ok = !*abort;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int sb = j & 1;
      ok = __all_sync(0xffffffffu, wait_or_abort(&s_full[sb], (j >> 1) & 1, abort, 6));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[64];
      tc_ld32(lane_addr + (sb ? S_COL1 : S_COL0), sv);
      tc_ld32(lane_addr + (sb ? S_COL1 : S_COL0) + 32, sv + 32);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);     // this warp has its rows of S: the buffer may be written again
      const int key0 = (kt_begin + j) * KEYS;
      // Only the pages on the diagonal and at a window's lower edge hold keys that a row must not
      // see; the others skip the two comparisons and the select per score (the loop is bound by
      // the number of instructions the four softmax warps issue, not by the exponentials).
      if (__any_sync(0xffffffffu, key0 + KEYS - 1 > pos || key0 < lo)) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int key = key0 + c;
          if (!(key >= lo && key <= pos)) sv[c] = __float_as_uint(-INFINITY);
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sv[c]));
        mx1 = fmaxf(mx1, __uint_as_float(sv[c + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sv[c + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sv[c + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * LOG2E;   // log2 units from here on
      // m is the reference the exponentials are taken against, not always the running maximum: it
      // moves only when the maximum has outgrown it by more than RESCALE_STEP (in log2 units), so
      // that O, which would have to be rescaled with it, is left alone on most pages.  p can then
      // be as large as 2^RESCALE_STEP, which bfloat16 and the float32 sums take without loss;
      // numerator and denominator carry the same factor.
      const float m_new = (m == -INFINITY || mx > m + RESCALE_STEP) ? fmaxf(m, mx) : m;
      const float u = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m - u);
      m = m_new;
      float sum0 = 0.f, sum1 = 0.f;
      uint32_t pk[32];
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        // one multiply-add and one ex2 per score: 2^(s * log2(e) - reference); a masked score is
        // -inf and gives 0
        const float a = ex2(fmaf(__uint_as_float(sv[2 * c]), LOG2E, -u));
        const float bq = ex2(fmaf(__uint_as_float(sv[2 * c + 1]), LOG2E, -u));
        sum0 += a;
        sum1 += bq;
        pk[c] = pack2(a, bq);
      }
      l = l * alpha + (sum0 + sum1);
      if (j > 0) {
        // O of the pages before is complete; bring it to the new maximum where that moved
        ok = __all_sync(0xffffffffu, wait_or_abort(o_done, (j - 1) & 1, abort, 6));
        if (!ok) break;
        tc_fence_after();
        if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < HD; c += 32) {
            uint32_t ov[32];
            tc_ld32(lane_addr + O_COL + c, ov);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tc_st32(lane_addr + O_COL + c, ov);
          }
          tc_wait_st();
        }
      }
      // P in the operand layout: row r is 128 bytes, its 16-byte chunk c sits at chunk c ^ (r & 7)
      uint8_t* prow = p_smem + r * 128;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *(uint4*)(prow + ((c ^ (r & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    if (ok) ok = __all_sync(0xffffffffu, wait_or_abort(o_done, (n_tiles - 1) & 1, abort, 6));
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      bf16* dst = out + (size_t)(tok0 + r) * out_stride + (size_t)head * HD;
#pragma unroll 1
      for (int c = 0; c < HD; c += 32) {
        uint32_t ov[32];
        tc_ld32(lane_addr + O_COL + c, ov);
        tc_wait_ld();
        if (valid) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack2(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv);
            w.y = pack2(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv);
            w.z = pack2(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv);
            w.w = pack2(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv);
            *(uint4*)(dst + c + 8 * i) = w;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  __syncwarp();
  if (warp == 5) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
}

}  // namespace

// q, out: [ntok, nh * HD] bfloat16, tokens of all sequences packed (cu_seqlens: [n_seqs + 1]); q rows
// q_stride elements apart.  kcache: [pages, nkv, 64, HD]; vcache: [pages, nkv, HD, 64] (pages counts
// every page of the layer, the spare one included).  seq_start: cache length of each sequence before
// this step; the cache already holds this step's keys and values.
GB_EXPORT int gb_attention_prefill_tc(const void* q, long long q_stride, void* out, long long out_stride,
                                      const void* kcache, const void* vcache, long long pages, const int* page_table,
                                      int table_width, int page_size, int nkv, int hd, const int* cu_seqlens,
                                      const int* seq_start, const int* seq_slot, int n_seqs, int ntok, int nh,
                                      int window, cudaStream_t stream) {
  if (ntok <= 0 || n_seqs <= 0) return 0;
  if (hd != HD || page_size != KEYS || nkv <= 0 || nh % nkv || pages <= 0) return GB_ERR_SIZE;
  if (((uintptr_t)q & 15) || (q_stride % 8) || ((uintptr_t)out & 15) || (out_stride % 8) || ((uintptr_t)kcache & 15) ||
      ((uintptr_t)vcache & 15))
    return GB_ERR_SIZE;
  CUtensorMap mq, mk, mv;
  if (!tensor_map(&mq, q, (uint64_t)ntok, (uint64_t)nh * HD, (uint64_t)q_stride * 2, ROWS)) return GB_ERR_ARG;
  if (!tensor_map(&mk, kcache, (uint64_t)pages * nkv * KEYS, (uint64_t)HD, (uint64_t)HD * 2, KEYS)) return GB_ERR_ARG;
  if (!tensor_map(&mv, vcache, (uint64_t)pages * nkv * HD, (uint64_t)KEYS, (uint64_t)KEYS * 2, HD)) return GB_ERR_ARG;
  constexpr size_t SMEM = SMEM_TILES + 15 * 8 + 16;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attention_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
      return (int)cudaGetLastError();
    configured = true;
  }
  dim3 grid(nh, (ntok + ROWS - 1) / ROWS + n_seqs);
  gb_launch(attention_prefill_tc_kernel, grid, 192, SMEM, stream, mq, mk, mv, (bf16*)out, out_stride, page_table,
            table_width, nkv, cu_seqlens, seq_start, seq_slot, n_seqs, nh, window);
  return gb_launch_status();
}

// 0, or the code of the first bounded wait that ran out (synchronizes the device).

GB_EXPORT int gb_attention_prefill_tc_status(int reset) {
  int v = -1;
  if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess) return -1;
  if (reset) {
    int zero = 0;
    cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
  }
  return v;
}
