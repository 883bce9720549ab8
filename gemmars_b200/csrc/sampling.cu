// Token sampling on the device: greedy, or temperature + top-k + top-p, one block per row.
//
// Reference: src/sampler.rs.  Greedy is the first maximum (:125-135).  Otherwise the k largest
// logits are taken in decreasing order (:43-61), p_i = exp((l_i - l_max) / T) / sum (:62-68),
// the shortest prefix whose running sum reaches top_p is kept (:70-81), and the draw walks that
// prefix with r = u * total, r -= p_i until r <= 0 (:109-122).  The uniform number u comes from
// the caller (the reference's xorshift64* generator runs on the host, one per sequence).
// Sums are sequential float32 sums in candidate order, as in the reference.  Equal logits are
// ordered by token id (the reference leaves their order open).  Up to 1,024 candidates live in
// shared memory (sample_kernel); more, or all tokens, are sorted in global scratch (sample_wide_kernel).
#include "common.cuh"

constexpr int SAMPLE_THREADS = 1024;
constexpr int MAX_TOP_K = 1024;

__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Exclusive prefix sum of one flag per thread over the block; total in *total.
__device__ __forceinline__ int block_exclusive_count(bool flag, int* warp_totals, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned ballot = __ballot_sync(0xffffffffu, flag);
  const int before = __popc(ballot & ((1u << lane) - 1));
  __syncthreads();
  if (lane == 0) warp_totals[warp] = __popc(ballot);
  __syncthreads();
  int base = 0, sum = 0;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
    const int c = warp_totals[w];
    if (w < warp) base += c;
    sum += c;
  }
  *total = sum;
  return base + before;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_kernel(
    const float* __restrict__ logits, long long stride, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
    int* __restrict__ out) {
  __shared__ unsigned long long cand[MAX_TOP_K];
  __shared__ float probs[MAX_TOP_K];
  __shared__ int hist[256];
  __shared__ int warp_totals[32];
  __shared__ float red_v[32];
  __shared__ int red_i[32];
  __shared__ unsigned sh_prefix;
  __shared__ int sh_remaining, sh_count;
  pdl_release_next();
  pdl_wait_prior();
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* l = logits + (size_t)row * stride;
  const float temp = temperature ? temperature[row] : 0.f;

  if (!(temp > 0.f)) {  // greedy: first maximum
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
      const float v = l[i];
      if (v > bv) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((tid & 31) == 0) { red_v[tid >> 5] = bv; red_i[tid >> 5] = bi; }
    __syncthreads();
    if (tid < 32) {
      bv = red_v[tid]; bi = red_i[tid];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (tid == 0) out[row] = bi == 0x7fffffff ? 0 : bi;
    }
    return;
  }

  int k = top_k[row];
  if (k <= 0 || k > MAX_TOP_K) k = MAX_TOP_K;  // the host refuses these; never index out of range
  if (k > vocab) k = vocab;

  // ---- the k-th largest key, by radix selection from the top byte down
  if (tid == 0) { sh_prefix = 0; sh_remaining = k; }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const unsigned prefix = sh_prefix;
    const unsigned mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
      const unsigned key = ordered_key(l[i]);
      if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 255], 1);
    }
    __syncthreads();
    if (tid == 0) {
      int remaining = sh_remaining, d = 255;
      for (; d > 0; --d) {
        if (hist[d] >= remaining) break;
        remaining -= hist[d];
      }
      sh_prefix = prefix | ((unsigned)d << shift);
      sh_remaining = remaining;
    }
    __syncthreads();
  }
  const unsigned kth = sh_prefix;
  const int need_equal = sh_remaining;  // how many keys equal to kth belong to the top k

  // ---- collect: every key above kth, and the need_equal lowest token ids at kth
  if (tid == 0) sh_count = 0;
  for (int i = tid; i < MAX_TOP_K; i += SAMPLE_THREADS) cand[i] = 0ull;
  __syncthreads();
  int equal_seen = 0;
  for (int base = 0; base < vocab; base += SAMPLE_THREADS) {
    const int i = base + tid;
    const unsigned key = i < vocab ? ordered_key(l[i]) : 0u;
    const bool above = i < vocab && key > kth;
    const bool equal = i < vocab && key == kth;
    if (above) {
      const int at = atomicAdd(&sh_count, 1);
      cand[at] = ((unsigned long long)key << 32) | (unsigned)(0xffffffffu - (unsigned)i);
    }
    if (equal_seen < need_equal) {  // uniform across the block
      int total;
      const int before = block_exclusive_count(equal, warp_totals, &total);
      if (equal && equal_seen + before < need_equal) {
        const int at = k - need_equal + equal_seen + before;
        cand[at] = ((unsigned long long)key << 32) | (unsigned)(0xffffffffu - (unsigned)i);
      }
      equal_seen += total;
    }
  }
  __syncthreads();

  // ---- sort decreasing by (logit, then increasing token id): bitonic over MAX_TOP_K entries
  for (int size = 2; size <= MAX_TOP_K; size <<= 1) {
    for (int step = size >> 1; step > 0; step >>= 1) {
      const int i = tid, j = i ^ step;
      if (j > i) {
        const unsigned long long a = cand[i], b = cand[j];
        const bool descending = (i & size) == 0;
        if (descending ? a < b : a > b) { cand[i] = b; cand[j] = a; }
      }
      __syncthreads();
    }
  }

  // ---- probabilities, cut and draw
  const float inv_t = 1.0f / temp;
  const float lmax = l[0xffffffffu - (unsigned)(cand[0] & 0xffffffffu)];
  if (tid < k) {
    const int id = (int)(0xffffffffu - (unsigned)(cand[tid] & 0xffffffffu));
    probs[tid] = expf((l[id] - lmax) * inv_t);
  }
  __syncthreads();
  if (tid == 0) {
    float sum = 0.f;
    for (int i = 0; i < k; ++i) sum += probs[i];
    int cut = k;
    const float tp = top_p[row];
    float acc = 0.f, total = 0.f;
    if (tp < 1.0f) {
      for (int i = 0; i < k; ++i) {
        acc += probs[i] / sum;
        if (acc >= tp) { cut = i + 1; break; }
      }
    }
    for (int i = 0; i < cut; ++i) total += probs[i] / sum;
    float r = uniform[row] * total;
    int pick = cut - 1;
    for (int i = 0; i < cut; ++i) {
      r -= probs[i] / sum;
      if (r <= 0.f) { pick = i; break; }
    }
    out[row] = (int)(0xffffffffu - (unsigned)(cand[pick] & 0xffffffffu));
  }
}

// ------------------------------------------------------------------ more than 1,024 candidates
// top_k = 0 (every token is a candidate, src/sampler.rs:43-47) or top_k > 1,024: the candidates do
// not fit shared memory, so the row's tokens are sorted in global scratch: a stable radix sort by
// the ordered key, 4 bits a pass from the lowest, larger digits first, starting from increasing
// token ids (so equal logits stay ordered by token id, as in the narrow kernel).  A thread owns a
// contiguous run of the array and a column of the 16 x 1024 digit counts, so no atomics are
// needed and the scatter is stable.  Then the same sequential float32 sums as above, over as many
// candidates as there are.  One block per row; rows that the narrow kernel serves return at once.
constexpr int WIDE_BINS = 16;

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_wide_kernel(
    const float* __restrict__ logits, long long stride, int vocab, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
    int* __restrict__ out, unsigned* __restrict__ keys, unsigned* __restrict__ ids, float* __restrict__ probs) {
  extern __shared__ int hist[];   // [WIDE_BINS][SAMPLE_THREADS]
  __shared__ int warp_sums[32];
  pdl_release_next();
  pdl_wait_prior();
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float temp = temperature ? temperature[row] : 0.f;
  int k = top_k[row];
  if (!(temp > 0.f) || (k >= 1 && k <= MAX_TOP_K)) return;
  if (k <= 0 || k > vocab) k = vocab;
  const float* l = logits + (size_t)row * stride;
  unsigned* key_buf[2] = {keys + (size_t)row * 2 * vocab, keys + (size_t)row * 2 * vocab + vocab};
  unsigned* id_buf[2] = {ids + (size_t)row * 2 * vocab, ids + (size_t)row * 2 * vocab + vocab};
  float* pr = probs + (size_t)row * vocab;
  for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
    key_buf[0][i] = ordered_key(l[i]);
    id_buf[0][i] = (unsigned)i;
  }
  __syncthreads();
  const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
  const int lo = min(vocab, tid * chunk), hi = min(vocab, lo + chunk);
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 4 * pass, src = pass & 1, dst = src ^ 1;
    for (int d = 0; d < WIDE_BINS; ++d) hist[d * SAMPLE_THREADS + tid] = 0;
    for (int i = lo; i < hi; ++i) ++hist[(15 - ((key_buf[src][i] >> shift) & 15)) * SAMPLE_THREADS + tid];
    __syncthreads();
    // exclusive running sum over the counts, digit by digit and thread by thread within a digit
    int local[WIDE_BINS], sum = 0;
    for (int j = 0; j < WIDE_BINS; ++j) {
      local[j] = hist[tid * WIDE_BINS + j];
      sum += local[j];
    }
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += warp_sums[w];
    int run = base + incl - sum;
    for (int j = 0; j < WIDE_BINS; ++j) {
      hist[tid * WIDE_BINS + j] = run;
      run += local[j];
    }
    __syncthreads();
    for (int i = lo; i < hi; ++i) {
      const unsigned key = key_buf[src][i];
      const int at = hist[(15 - ((key >> shift) & 15)) * SAMPLE_THREADS + tid]++;
      key_buf[dst][at] = key;
      id_buf[dst][at] = id_buf[src][i];
    }
    __syncthreads();
  }
  // eight passes: the sorted order is back in the first buffers
  const unsigned* order = id_buf[0];
  const float inv_t = 1.0f / temp, lmax = l[order[0]];
  for (int i = tid; i < k; i += SAMPLE_THREADS) pr[i] = expf((l[order[i]] - lmax) * inv_t);
  __syncthreads();
  if (tid == 0) {
    float sum = 0.f;
    for (int i = 0; i < k; ++i) sum += pr[i];
    int cut = k;
    const float tp = top_p[row];
    float acc = 0.f, total = 0.f;
    if (tp < 1.0f) {
      for (int i = 0; i < k; ++i) {
        acc += pr[i] / sum;
        if (acc >= tp) { cut = i + 1; break; }
      }
    }
    for (int i = 0; i < cut; ++i) total += pr[i] / sum;
    float r = uniform[row] * total;
    int pick = cut - 1;
    for (int i = 0; i < cut; ++i) {
      r -= pr[i] / sum;
      if (r <= 0.f) { pick = i; break; }
    }
    out[row] = (int)order[pick];
  }
}

// logits: [rows, vocab] float32, rows `stride` apart.  temperature may be null (all greedy).
// Rows with temperature <= 0 take the first maximum; rows with 1 <= top_k <= 1024 are served from
// shared memory; other rows (top_k = 0: all tokens, or more than 1,024) need `wide`, float32
// scratch of 5 * rows * vocab values, and are sorted in it (null: such rows are refused).
GB_EXPORT int gb_sample(const float* logits, long long stride, int rows, int vocab, const float* temperature,
                        const int* top_k, const float* top_p, const float* uniform, int* out, float* wide,
                        cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return GB_ERR_SIZE;
  if (temperature && (!top_k || !top_p || !uniform)) return GB_ERR_ARG;
  gb_launch(sample_kernel, rows, SAMPLE_THREADS, 0, stream, logits, stride, vocab, temperature, top_k, top_p, uniform, out);
  if (wide && temperature) {
    constexpr size_t SMEM = (size_t)WIDE_BINS * SAMPLE_THREADS * sizeof(int);
    static bool configured = false;
    if (!configured) {
      if (cudaFuncSetAttribute(sample_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) != cudaSuccess)
        return (int)cudaGetLastError();
      configured = true;
    }
    unsigned* keys = (unsigned*)wide;
    unsigned* ids = keys + (size_t)2 * rows * vocab;
    float* probs = wide + (size_t)4 * rows * vocab;
    gb_launch(sample_wide_kernel, rows, SAMPLE_THREADS, SMEM, stream, logits, stride, vocab, temperature, top_k, top_p,
              uniform, out, keys, ids, probs);
  }
  return gb_launch_status();
}
