// Token sampling on the device: greedy, or temperature + top-k + top-p.
//
// Reference: src/sampler.rs.  Greedy is the first maximum (:125-135).  Otherwise the k largest
// logits are taken in decreasing order (:43-61), p_i = exp((l_i - l_max) / T) / sum (:62-68),
// the shortest prefix whose running sum reaches top_p is kept (:70-81), and the draw walks that
// prefix with r = u * total, r -= p_i until r <= 0 (:109-122).  The uniform number u comes from
// the caller (the reference's xorshift64* generator runs on the host, one per sequence).
// Sums are sequential float32 sums in candidate order, as in the reference.  Equal logits are
// ordered by token id (the reference leaves their order open).
//
// Up to 1,024 candidates a row: two kernels.  A row of logits is cut into slices and every
// slice goes to a CTA of its own (a row of 152 thousand logits is 600 KB: read by one CTA it
// takes longer than a decode step's attention, read by ten it does not), which keeps its
// slice in registers and finds the slice's k best (sample_slice_kernel); then one CTA per row
// takes the slices' candidates, finds the k best of those, sorts them, and draws
// (sample_merge_kernel).  Greedy rows are the case k = 1.  A token is the 64-bit value
// (ordered logit bits, complement of the token id): all values differ, a larger value is a
// better candidate, and "the k best" has one answer whatever the ties, found by radix selection
// over the 8 bytes from the top.  More candidates, or all tokens: sample_wide_kernel below.
#include "common.cuh"

constexpr int SAMPLE_THREADS = 1024;
constexpr int MAX_TOP_K = 1024;
constexpr int PER_THREAD = 16;                                // values a thread keeps in registers
constexpr int SELECT_MAX = SAMPLE_THREADS * PER_THREAD;       // values one CTA can select from

__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ unsigned long long candidate(float logit, int token) {
  return ((unsigned long long)ordered_key(logit) << 32) | (unsigned)(0xffffffffu - (unsigned)token);
}
__device__ __forceinline__ int candidate_token(unsigned long long c) { return (int)(0xffffffffu - (unsigned)(c & 0xffffffffu)); }

struct SelectShared {
  int hist[256];
  unsigned long long prefix;
  int remaining, count, done;
};

// The k largest of the block's values (v[e] of every thread; 0 = no value; all others differ),
// written to out[0 .. k) in no particular order; k must not exceed the number of values.
// Radix selection of the k-th largest from the top byte down, then one pass that collects.
__device__ void select_largest(const unsigned long long (&v)[PER_THREAD], int k, unsigned long long* out, SelectShared& s) {
  const int tid = threadIdx.x, lane = tid & 31;
  if (tid == 0) { s.prefix = 0ull; s.remaining = k; s.count = 0; s.done = 0; }
  for (int pass = 0; pass < 8; ++pass) {
    const int shift = 56 - 8 * pass;
    if (tid < 256) s.hist[tid] = 0;
    __syncthreads();
    const unsigned long long prefix = s.prefix;
    const unsigned long long mask = pass == 0 ? 0ull : (~0ull << (shift + 8));
#pragma unroll
    for (int e = 0; e < PER_THREAD; ++e) {
      const bool in = v[e] != 0ull && (v[e] & mask) == prefix;
      const int bin = (int)((v[e] >> shift) & 255);
      if (pass == 0) {
        // the logits of a row share their top byte: lanes that count into the same bin send one
        // addition, where thirty-two additions to one address would run one after the other
        const unsigned active = __ballot_sync(0xffffffffu, in);
        if (in) {
          const unsigned same = __match_any_sync(active, bin);
          if (lane == __ffs(same) - 1) atomicAdd(&s.hist[bin], __popc(same));
        }
      } else if (in) {
        atomicAdd(&s.hist[bin], 1);     // further down the values spread over the bins
      }
    }
    __syncthreads();
    if (tid < 32) {
      // bins from the top: lane L holds bins 255 - 8 L down to 248 - 8 L
      int mine[8], sum = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { mine[j] = s.hist[255 - 8 * lane - j]; sum += mine[j]; }
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
      }
      const int remaining = s.remaining;
      const unsigned reached = __ballot_sync(0xffffffffu, incl >= remaining);
      const int owner = reached ? __ffs(reached) - 1 : 31;
      if (lane == owner) {
        int left = remaining - (incl - sum), j = 7, in_bin = mine[7];
        bool found = false;
#pragma unroll
        for (int q = 0; q < 7; ++q) {
          if (!found) {
            if (mine[q] >= left) {
              found = true;
              j = q;
              in_bin = mine[q];
            } else {
              left -= mine[q];
            }
          }
        }
        s.prefix = prefix | ((unsigned long long)(255 - 8 * lane - j) << shift);
        s.remaining = left;
        // every value of the chosen bin is wanted: the bytes below cannot change the answer
        s.done = in_bin == left;
      }
    }
    __syncthreads();
    if (s.done) break;
  }
  const unsigned long long kth = s.prefix;      // the k-th largest, or (stopped early) its leading bytes
#pragma unroll
  for (int e = 0; e < PER_THREAD; ++e)
    if (v[e] != 0ull && v[e] >= kth) {
      const int at = atomicAdd(&s.count, 1);
      if (at < k) out[at] = v[e];
    }
  __syncthreads();
}

__device__ __forceinline__ int row_k(const float* temperature, const int* top_k, int row, int vocab) {
  const float temp = temperature ? temperature[row] : 0.f;
  if (!(temp > 0.f)) return 1;                     // greedy: the first maximum
  int k = top_k[row];
  if (k <= 0 || k > MAX_TOP_K) k = MAX_TOP_K;      // such rows belong to the wide kernel; never index out of range
  return min(k, vocab);
}

// grid (slices, rows).  Slice s of a row is tokens [s * slice_len, (s + 1) * slice_len); its
// min(k, tokens in the slice) best go to cand[(row * slices + s) * cap ...], their number to counts.
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_slice_kernel(
    const float* __restrict__ logits, long long stride, int vocab, int slice_len, const float* __restrict__ temperature,
    const int* __restrict__ top_k, unsigned long long* __restrict__ cand, int* __restrict__ counts, int cap) {
  __shared__ SelectShared sel;
  __shared__ unsigned long long best[MAX_TOP_K];
  pdl_release_next();
  pdl_wait_prior();
  const int slice = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
  const int lo = slice * slice_len, n = max(0, min(vocab - lo, slice_len));
  const float* l = logits + (size_t)row * stride + lo;
  const int k = min(min(row_k(temperature, top_k, row, vocab), cap), n);
  unsigned long long v[PER_THREAD];
#pragma unroll
  for (int e = 0; e < PER_THREAD; ++e) {
    const int i = e * SAMPLE_THREADS + tid;
    v[e] = i < n ? candidate(l[i], lo + i) : 0ull;
  }
  if (k > 0) select_largest(v, k, best, sel);
  unsigned long long* mine = cand + ((size_t)row * gridDim.x + slice) * cap;
  for (int i = tid; i < k; i += SAMPLE_THREADS) mine[i] = best[i];
  if (tid == 0) counts[row * gridDim.x + slice] = k;
}

// One block per row: the k best of the slices' candidates, in decreasing order, then the draw.
__global__ void __launch_bounds__(SAMPLE_THREADS) sample_merge_kernel(
    const float* __restrict__ logits, long long stride, int vocab, int slices, const float* __restrict__ temperature,
    const int* __restrict__ top_k, const float* __restrict__ top_p, const float* __restrict__ uniform,
    const unsigned long long* __restrict__ cand, const int* __restrict__ counts, int cap, int* __restrict__ out) {
  __shared__ SelectShared sel;
  __shared__ unsigned long long best[MAX_TOP_K];
  __shared__ float probs[MAX_TOP_K];
  pdl_release_next();
  pdl_wait_prior();
  const int row = blockIdx.x, tid = threadIdx.x;
  const float temp = temperature ? temperature[row] : 0.f;
  const int k = min(row_k(temperature, top_k, row, vocab), cap * slices);
  unsigned long long v[PER_THREAD];
  int have = 0;
#pragma unroll
  for (int e = 0; e < PER_THREAD; ++e) {
    const int i = e * SAMPLE_THREADS + tid, s = i / cap, j = i - s * cap;
    v[e] = (s < slices && j < counts[row * slices + s]) ? cand[((size_t)row * slices + s) * cap + j] : 0ull;
  }
  for (int s = 0; s < slices; ++s) have += counts[row * slices + s];
  const int kk = min(k, have);
  for (int i = tid; i < MAX_TOP_K; i += SAMPLE_THREADS) best[i] = 0ull;
  __syncthreads();
  select_largest(v, kk, best, sel);
  if (!(temp > 0.f)) {
    if (tid == 0) out[row] = kk > 0 ? candidate_token(best[0]) : 0;
    return;
  }
  // ---- sort decreasing (logit, then increasing token id): bitonic over the next power of two
  int width = 2;
  while (width < kk) width <<= 1;
  for (int size = 2; size <= width; size <<= 1) {
    for (int step = size >> 1; step > 0; step >>= 1) {
      const int i = tid, j = i ^ step;
      if (i < width && j > i) {
        const unsigned long long a = best[i], b = best[j];
        const bool descending = (i & size) == 0;
        if (descending ? a < b : a > b) { best[i] = b; best[j] = a; }
      }
      __syncthreads();
    }
  }
  // ---- probabilities, cut and draw
  const float* l = logits + (size_t)row * stride;
  const float inv_t = 1.0f / temp;
  const float lmax = l[candidate_token(best[0])];
  if (tid < kk) probs[tid] = expf((l[candidate_token(best[tid])] - lmax) * inv_t);
  __syncthreads();
  if (tid == 0) {
    float sum = 0.f;
    for (int i = 0; i < kk; ++i) sum += probs[i];
    int cut = kk;
    const float tp = top_p[row];
    float acc = 0.f, total = 0.f;
    if (tp < 1.0f) {
      for (int i = 0; i < kk; ++i) {
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
    out[row] = candidate_token(best[pick]);
  }
}

// ------------------------------------------------------------------ all rows greedy
// The first maximum of every row, without any selection: a slice's largest value by a plain
// reduction (the value's order is "larger logit first, then smaller token id"), then the largest of
// the slices' results.
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long other = __shfl_xor_sync(0xffffffffu, v, o);
    v = other > v ? other : v;
  }
  return v;
}

constexpr int ARGMAX_THREADS = 256;

__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_slice_kernel(const float* __restrict__ logits, long long stride, int vocab,
                                                                     int slice_len, unsigned long long* __restrict__ cand) {
  __shared__ unsigned long long warp_best[ARGMAX_THREADS / 32];
  pdl_release_next();
  pdl_wait_prior();
  const int slice = blockIdx.x, row = blockIdx.y, tid = threadIdx.x;
  const int lo = slice * slice_len, hi = min(vocab, lo + slice_len);
  const float* l = logits + (size_t)row * stride;
  unsigned long long best = 0ull;
  for (int i = lo + tid; i < hi; i += ARGMAX_THREADS) {
    const unsigned long long c = candidate(l[i], i);
    best = c > best ? c : best;
  }
  best = warp_max_u64(best);
  if ((tid & 31) == 0) warp_best[tid >> 5] = best;
  __syncthreads();
  if (tid < 32) {
    best = warp_max_u64(tid < ARGMAX_THREADS / 32 ? warp_best[tid] : 0ull);
    if (tid == 0) cand[(size_t)row * gridDim.x + slice] = best;
  }
}

__global__ void __launch_bounds__(32) argmax_merge_kernel(const unsigned long long* __restrict__ cand, int slices,
                                                          int* __restrict__ out) {
  pdl_release_next();
  pdl_wait_prior();
  const int row = blockIdx.x;
  unsigned long long best = 0ull;
  for (int i = threadIdx.x; i < slices; i += 32) {
    const unsigned long long c = cand[(size_t)row * slices + i];
    best = c > best ? c : best;
  }
  best = warp_max_u64(best);
  if (threadIdx.x == 0) out[row] = best ? candidate_token(best) : 0;
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

// How a row is cut for the two kernels: (slices, tokens per slice) for `rows` rows of `vocab`
// logits with at most `cap` candidates a row, on a device of `sms` multiprocessors.  About two
// CTAs per multiprocessor in all; a slice is at most SELECT_MAX tokens and the slices' candidates
// together at most SELECT_MAX.  Returns 0 slices when no cut does both.
static void sample_cut(int rows, int vocab, int cap, int sms, int* slices, int* slice_len) {
  const int least = (vocab + SELECT_MAX - 1) / SELECT_MAX, most = SELECT_MAX / cap;
  int n = (2 * sms + rows - 1) / rows;
  if (n < least) n = least;
  if (n > most) n = most;
  if (n > 64) n = 64;
  if (n < least) {
    *slices = 0;
    *slice_len = 0;
    return;
  }
  const int len = (vocab + n - 1) / n;
  *slice_len = len;
  *slices = (vocab + len - 1) / len;
}

// Bytes of scratch gb_sample wants for the narrow path (8-byte aligned), or -1 when the sizes
// cannot be served (a vocabulary beyond 64 slices of 16,384 tokens, or too many candidates for it).
GB_EXPORT long long gb_sample_scratch_bytes(int rows, int vocab, int cap, int sms) {
  if (rows <= 0 || vocab <= 0 || cap < 1 || cap > MAX_TOP_K || sms <= 0) return -1;
  int slices, slice_len;
  sample_cut(rows, vocab, cap, sms, &slices, &slice_len);
  if (slices == 0) return -1;
  return (long long)rows * slices * cap * 8 + (((long long)rows * slices * 4 + 7) & ~7ll);
}

// logits: [rows, vocab] float32, rows `stride` apart.  temperature may be null (all greedy).
// Rows with temperature <= 0 take the first maximum; rows with 1 <= top_k <= 1024 are served by
// the slice and merge kernels; `cap` is the largest such top_k among the rows (1 when all are
// greedy) and `scratch` holds gb_sample_scratch_bytes(rows, vocab, cap, sms) bytes.  Other rows
// (top_k = 0: all tokens, or more than 1,024) need `wide`, float32 scratch of 5 * rows * vocab
// values, and are sorted in it (null: such rows are refused by the caller).
GB_EXPORT int gb_sample(const float* logits, long long stride, int rows, int vocab, const float* temperature,
                        const int* top_k, const float* top_p, const float* uniform, int* out, float* wide,
                        void* scratch, int cap, int sms, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || cap < 1 || cap > MAX_TOP_K || sms <= 0) return GB_ERR_SIZE;
  if (temperature && (!top_k || !top_p || !uniform)) return GB_ERR_ARG;
  if (!scratch) return GB_ERR_ARG;
  int slices, slice_len;
  sample_cut(rows, vocab, cap, sms, &slices, &slice_len);
  if (slices == 0) return GB_ERR_SIZE;
  unsigned long long* cand = (unsigned long long*)scratch;
  int* counts = (int*)(cand + (size_t)rows * slices * cap);
  if (!temperature) {   // every row takes its first maximum
    gb_launch(argmax_slice_kernel, dim3(slices, rows), ARGMAX_THREADS, 0, stream, logits, stride, vocab, slice_len, cand);
    gb_launch(argmax_merge_kernel, rows, 32, 0, stream, (const unsigned long long*)cand, slices, out);
    return gb_launch_status();
  }
  gb_launch(sample_slice_kernel, dim3(slices, rows), SAMPLE_THREADS, 0, stream, logits, stride, vocab, slice_len,
            temperature, top_k, cand, counts, cap);
  gb_launch(sample_merge_kernel, rows, SAMPLE_THREADS, 0, stream, logits, stride, vocab, slices, temperature, top_k, top_p,
            uniform, (const unsigned long long*)cand, (const int*)counts, cap, out);
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
