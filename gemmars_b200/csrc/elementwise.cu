// Memory-bound kernels of the step: embedding gather, RMSNorm, the fused per-head
// norm + rotation + scale + cache write, and the gated activation.
//
// Reference formulas: embedding src/qwen.rs:669-672; RMSNorm src/kernels.rs:1385-1392;
// rotation src/kernels.rs:1521-1548 with inv_freq from src/qwen.rs:529-533; q scale after the
// rotation src/qwen.rs:737-761; keys cached normed and rotated, values raw src/qwen.rs:775-785;
// silu(a) * b src/kernels.rs:1416-1426.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// x[t, :] = table[tok[t], :] * scale, into the float32 residual stream.
template <typename W>
__global__ void embed_gather_kernel(const W* __restrict__ table, const int* __restrict__ tok, float* __restrict__ x,
                                    int hidden, int vocab, float scale) {
  pdl_release_next();
  pdl_wait_prior();
  const int t = blockIdx.x;
  int id = tok[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // ids are checked on the host; never read outside
  const W* row = table + (size_t)id * hidden;
  float* out = x + (size_t)t * hidden;
  if (sizeof(W) == 2 && (hidden & 7) == 0 && (((uintptr_t)table | (uintptr_t)x) & 15) == 0) {
    // 16 bytes of the row per load, all of a thread's loads asked for before the first is used: a
    // decode step's few rows are a handful of round trips to memory, not one per two bytes
    constexpr int U = 4;
    const uint4* row8 = (const uint4*)row;
    float4* out4 = (float4*)out;
    const int n8 = hidden / 8;
    for (int base = 0; base < n8; base += U * blockDim.x) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + threadIdx.x + u * blockDim.x;
        v[u] = i < n8 ? row8[i] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int i = base + threadIdx.x + u * blockDim.x;
        if (i < n8) {
          const float2 a = __bfloat1622float2(*(const __nv_bfloat162*)&v[u].x), b = __bfloat1622float2(*(const __nv_bfloat162*)&v[u].y);
          const float2 c = __bfloat1622float2(*(const __nv_bfloat162*)&v[u].z), d = __bfloat1622float2(*(const __nv_bfloat162*)&v[u].w);
          out4[2 * i] = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
          out4[2 * i + 1] = make_float4(c.x * scale, c.y * scale, d.x * scale, d.y * scale);
        }
      }
    }
    return;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) out[i] = to_f32(row[i]) * scale;
}

GB_EXPORT int gb_embed_gather(const void* table, int table_dtype, const int* tok, float* x, int ntok, int hidden,
                              int vocab, float scale, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  const int threads = hidden >= 1024 ? 256 : 128;
  if (table_dtype == GB_F32)
    gb_launch(embed_gather_kernel<float>, ntok, threads, 0, stream, (const float*)table, tok, x, hidden, vocab, scale);
  else if (table_dtype == GB_BF16)
    gb_launch(embed_gather_kernel<bf16>, ntok, threads, 0, stream, (const bf16*)table, tok, x, hidden, vocab, scale);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// ------------------------------------------------------------------ RMSNorm
// out[r, :] = x[src(r), :] * (mean(x^2) + eps)^-1/2 * w, statistics in float32.
// rows_index (optional) gathers: src(r) = rows_index[r].
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                               const int* __restrict__ rows_index, int n, float eps) {
  __shared__ float scratch[33];
  pdl_release_next();
  constexpr int KEEP = 4;            // float4s a thread keeps in registers between the two passes
  const bool vec = (n & 3) == 0, keep = vec && n / 4 <= KEEP * (int)blockDim.x;
  float4 gain[KEEP];
  if (keep) {
    // the weights do not depend on the kernel before this one: asked for before waiting for it
#pragma unroll
    for (int u = 0; u < KEEP; ++u) {
      const int i = threadIdx.x + u * blockDim.x;
      gain[u] = i < n / 4 ? ((const float4*)w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  }
  pdl_wait_prior();
  const int r = blockIdx.x;
  const float* row = x + (size_t)(rows_index ? rows_index[r] : r) * n;
  T* o = out + (size_t)r * n;
  // four elements at a time when the row allows it (rows of x and out are then 16-byte aligned);
  // the order of the additions depends on n and the block size alone
  if (vec) {
    const float4* row4 = (const float4*)row;
    const float4* w4 = (const float4*)w;
    float4 held[KEEP];
    float ss = 0.f;
    if (keep) {
#pragma unroll
      for (int u = 0; u < KEEP; ++u) {
        const int i = threadIdx.x + u * blockDim.x;
        held[u] = i < n / 4 ? row4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < KEEP; ++u) ss += held[u].x * held[u].x + held[u].y * held[u].y + held[u].z * held[u].z + held[u].w * held[u].w;
    } else {
      for (int i = threadIdx.x; i < n / 4; i += blockDim.x) {
        const float4 v = row4[i];
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
      }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (int u = 0, i = threadIdx.x; i < n / 4; i += blockDim.x, ++u) {
      const float4 v = keep ? held[u < KEEP ? u : 0] : row4[i], g = keep ? gain[u < KEEP ? u : 0] : w4[i];
      const float a = v.x * inv * g.x, b = v.y * inv * g.y, c = v.z * inv * g.z, d = v.w * inv * g.w;
      if (sizeof(T) == 4) {
        ((float4*)o)[i] = make_float4(a, b, c, d);
      } else {
        __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
        ((uint2*)o)[i] = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
      }
    }
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += row[i] * row[i];
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) o[i] = from_f32<T>(row[i] * inv * w[i]);
}

// Many rows (a prompt), bfloat16 out: one warp per row, no block barrier.  The row is read twice
// (the second time from L1) with eight 16-byte loads of a lane in flight, which is what the
// kernel lives on when there are thousands of rows; the float32 engine keeps the kernel above
// for every number of rows, since the block's shape fixes the order of the additions.
__global__ void __launch_bounds__(256) rmsnorm_rows_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                           bf16* __restrict__ out, const int* __restrict__ rows_index,
                                                           int rows, int n, float eps) {
  pdl_release_next();
  pdl_wait_prior();
  const int lane = threadIdx.x & 31, r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const float4* row4 = (const float4*)(x + (size_t)(rows_index ? rows_index[r] : r) * n);
  const float4* w4 = (const float4*)w;
  const int n4 = n / 4;
  float ss = 0.f;
  for (int base = 0; base < n4; base += 32 * 8) {
    float4 v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + lane + 32 * u;
      v[u] = i < n4 ? row4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
  }
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
  uint2* o = (uint2*)(out + (size_t)r * n);
  for (int base = 0; base < n4; base += 32 * 8) {
    float4 v[8], g[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + lane + 32 * u;
      if (i < n4) {
        v[u] = row4[i];
        g[u] = w4[i];
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = base + lane + 32 * u;
      if (i < n4) {
        __nv_bfloat162 lo = __floats2bfloat162_rn(v[u].x * inv * g[u].x, v[u].y * inv * g[u].y);
        __nv_bfloat162 hi = __floats2bfloat162_rn(v[u].z * inv * g[u].z, v[u].w * inv * g[u].w);
        o[i] = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
      }
    }
  }
}

// The same for rows of up to 32 * 4 * U values: the row stays in the lane's registers (U 16-byte
// loads in flight at once, nothing read twice), and the norm's weights are put into shared memory
// once per CTA before the kernel waits for the one before it, so that a row is one round trip to
// memory, not two.  A prompt of 2,048 rows of 4,096: 20 us with the kernel above inside a prompt
// step, where the rows come out of L2.
template <int U>
__global__ void __launch_bounds__(128) rmsnorm_rows_held_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                                                bf16* __restrict__ out, const int* __restrict__ rows_index,
                                                                int rows, int n, float eps) {
  extern __shared__ float4 weights[];   // [n / 4]
  pdl_release_next();
  const int n4 = n / 4;
  for (int i = threadIdx.x; i < n4; i += blockDim.x) weights[i] = ((const float4*)w)[i];
  pdl_wait_prior();
  const int lane = threadIdx.x & 31, r = min(blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), rows - 1);
  const bool mine = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5) < rows;   // a warp beyond the rows only keeps the barrier
  const float4* row4 = (const float4*)(x + (size_t)(rows_index ? rows_index[r] : r) * n);
  float4 v[U];
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int i = lane + 32 * u;
    v[u] = i < n4 ? row4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float ss = 0.f;
#pragma unroll
  for (int u = 0; u < U; ++u) ss += v[u].x * v[u].x + v[u].y * v[u].y + v[u].z * v[u].z + v[u].w * v[u].w;
  const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
  __syncthreads();   // the weights are in shared memory
  if (!mine) return;
  uint2* o = (uint2*)(out + (size_t)r * n);
#pragma unroll
  for (int u = 0; u < U; ++u) {
    const int i = lane + 32 * u;
    if (i < n4) {
      const float4 g = weights[i];
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[u].x * inv * g.x, v[u].y * inv * g.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v[u].z * inv * g.z, v[u].w * inv * g.w);
      o[i] = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
    }
  }
}

template <int U>
static void launch_rows_held(const float* x, const float* w, bf16* out, const int* rows_index, int rows, int n, float eps,
                             cudaStream_t stream) {
  gb_launch(rmsnorm_rows_held_kernel<U>, (rows + 3) / 4, 128, (size_t)n * 4, stream, x, w, out, rows_index, rows, n, eps);
}

GB_EXPORT int gb_rmsnorm(const float* x, const float* w, void* out, int out_dtype, const int* rows_index, int rows,
                         int n, float eps, cudaStream_t stream) {
  if (rows <= 0) return 0;
  const int threads = n >= 1024 ? 256 : 128;
  if (out_dtype == GB_F32)
    gb_launch(rmsnorm_kernel<float>, rows, threads, 0, stream, x, w, (float*)out, rows_index, n, eps);
  else if (out_dtype == GB_BF16 && rows >= 512 && (n & 3) == 0 && n <= 32 * 4 * 8)
    launch_rows_held<8>(x, w, (bf16*)out, rows_index, rows, n, eps, stream);
  else if (out_dtype == GB_BF16 && rows >= 512 && (n & 3) == 0 && n <= 32 * 4 * 16)
    launch_rows_held<16>(x, w, (bf16*)out, rows_index, rows, n, eps, stream);
  else if (out_dtype == GB_BF16 && rows >= 512 && (n & 3) == 0 && n <= 32 * 4 * 24)
    launch_rows_held<24>(x, w, (bf16*)out, rows_index, rows, n, eps, stream);
  else if (out_dtype == GB_BF16 && rows >= 512 && (n & 3) == 0 && n <= 32 * 4 * 32)
    launch_rows_held<32>(x, w, (bf16*)out, rows_index, rows, n, eps, stream);
  else if (out_dtype == GB_BF16 && rows >= 512 && (n & 3) == 0 && n <= 32 * 4 * 40)
    launch_rows_held<40>(x, w, (bf16*)out, rows_index, rows, n, eps, stream);
  else if (out_dtype == GB_BF16 && rows >= 512 && (n & 3) == 0)
    gb_launch(rmsnorm_rows_kernel, (rows + 7) / 8, 256, 0, stream, x, w, (bf16*)out, rows_index, rows, n, eps);
  else if (out_dtype == GB_BF16)
    gb_launch(rmsnorm_kernel<bf16>, rows, threads, 0, stream, x, w, (bf16*)out, rows_index, n, eps);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}

// ------------------------------------------------------------------ per-head norm + rotation + cache write
// qkv: [ntok, (nh + 2 nkv) * hd], heads in the order q.., k.., v...  One warp per (token, head).
//   q heads: optional RMSNorm over hd (weight qw), optional rotation of the first `rot` dims at
//            the token's position, then * q_scale; written back in place.
//   k heads: optional RMSNorm (weight kw), optional rotation; written back in place and, with
//            FLAG_CACHE, into the paged key cache.
//   v heads: with FLAG_CACHE copied into the paged value cache (transposed inside the page).
//   FLAG_SINGLE: the tokens are single positions of different sequences (a decode step).
enum { FLAG_NORM = 1, FLAG_ROPE = 2, FLAG_CACHE = 4, FLAG_INPLACE = 8, FLAG_V_TILED = 16, FLAG_SINGLE = 32 };

// One head of one token, by one warp.  cs / sn: cos and sin of the token's angles (rot / 2 each).
template <typename T>
__device__ __forceinline__ void head_norm_rope_cache_one(T* __restrict__ qkv, int t, int h, int pos, int nh, int nkv, int hd,
                                                         int rot, const float* __restrict__ qw,
                                                         const float* __restrict__ kw, float eps,
                                                         const float* __restrict__ cs, const float* __restrict__ sn,
                                                         float q_scale, int page, const PagedKV& kv,
                                                         T* __restrict__ kcache, T* __restrict__ vcache, int flags) {
  const int lane = threadIdx.x & 31;
  const int heads = nh + 2 * nkv;
  T* src = qkv + ((size_t)t * heads + h) * hd;
  const bool cache = flags & FLAG_CACHE;
  if (h >= nh + nkv) {  // value head
    if (!cache || (flags & FLAG_V_TILED)) return;   // tiled: value_cache_tile_kernel writes the values
    T* dst = vcache + ((size_t)page * nkv + (h - nh - nkv)) * kv.page_size * hd + pos % kv.page_size;
    for (int i = lane; i < hd; i += 32) dst[(size_t)i * kv.page_size] = src[i];
    return;
  }
  const bool is_q = h < nh;
  if (is_q && !(flags & FLAG_INPLACE)) return;
  const float* w = is_q ? qw : kw;
  if (sizeof(T) == 2 && (flags & FLAG_ROPE) && rot == hd && (hd & 3) == 0) {
    // bfloat16, all dims rotated: each lane keeps two adjacent dims of each half (4-byte loads and
    // stores), so the head is read once for the norm and the rotation alike
    const int half = hd / 2;
    const float scale = is_q ? q_scale : 1.f;
    bf16* cdst = (!is_q && cache) ? (bf16*)kcache + (((size_t)page * nkv + (h - nh)) * kv.page_size + pos % kv.page_size) * hd
                                  : nullptr;
    const bf16* s16 = (const bf16*)src;
    float2 a[2], b[2];   // up to head size 256: two rounds of 64 dims per half
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = 2 * lane + 64 * r;
      if (i < half) {
        a[r] = __bfloat1622float2(*(const __nv_bfloat162*)(s16 + i));
        b[r] = __bfloat1622float2(*(const __nv_bfloat162*)(s16 + i + half));
        ss += a[r].x * a[r].x + a[r].y * a[r].y + b[r].x * b[r].x + b[r].y * b[r].y;
      }
    }
    float2 wa[2], wb[2];   // the norm's weights for the same dims, asked for before the sum is known
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = 2 * lane + 64 * r;
      if ((flags & FLAG_NORM) && i < half) {
        wa[r] = *(const float2*)(w + i);
        wb[r] = *(const float2*)(w + i + half);
      }
    }
    float inv = 1.f;
    if (flags & FLAG_NORM) inv = 1.0f / sqrtf(warp_sum(ss) / (float)hd + eps);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int i = 2 * lane + 64 * r;
      if (i < half) {
        float ax = a[r].x * inv, ay = a[r].y * inv, bx = b[r].x * inv, by = b[r].y * inv;
        if (flags & FLAG_NORM) {
          ax *= wa[r].x; ay *= wa[r].y; bx *= wb[r].x; by *= wb[r].y;
        }
        const float s0 = sn[i], c0 = cs[i], s1 = sn[i + 1], c1 = cs[i + 1];
        const __nv_bfloat162 ra = __floats2bfloat162_rn((ax * c0 - bx * s0) * scale, (ay * c1 - by * s1) * scale);
        const __nv_bfloat162 rb = __floats2bfloat162_rn((bx * c0 + ax * s0) * scale, (by * c1 + ay * s1) * scale);
        if (flags & FLAG_INPLACE) {
          *(__nv_bfloat162*)((bf16*)src + i) = ra;
          *(__nv_bfloat162*)((bf16*)src + i + half) = rb;
        }
        if (cdst) {
          *(__nv_bfloat162*)(cdst + i) = ra;
          *(__nv_bfloat162*)(cdst + i + half) = rb;
        }
      }
    }
    return;
  }
  float inv = 1.f;
  if (flags & FLAG_NORM) {
    float ss = 0.f;
    for (int i = lane; i < hd; i += 32) {
      const float v = to_f32(src[i]);
      ss += v * v;
    }
    ss = warp_sum(ss);
    inv = 1.0f / sqrtf(ss / (float)hd + eps);
  }
  const float scale = is_q ? q_scale : 1.f;
  T* cdst = (!is_q && cache) ? kcache + (((size_t)page * nkv + (h - nh)) * kv.page_size + pos % kv.page_size) * hd : nullptr;
  const bool inplace = flags & FLAG_INPLACE;
  const bool rope = flags & FLAG_ROPE;
  const int half = rope ? rot / 2 : 0;
  for (int i = lane; i < half; i += 32) {
    float a = to_f32(src[i]) * inv, b = to_f32(src[i + half]) * inv;
    if (flags & FLAG_NORM) {
      a *= w[i];
      b *= w[i + half];
    }
    const float s = sn[i], c = cs[i];
    const T ra = from_f32<T>((a * c - b * s) * scale), rb = from_f32<T>((b * c + a * s) * scale);
    if (inplace) {
      src[i] = ra;
      src[i + half] = rb;
    }
    if (cdst) {
      cdst[i] = ra;
      cdst[i + half] = rb;
    }
  }
  for (int i = 2 * half + lane; i < hd; i += 32) {  // dims that are not rotated
    float a = to_f32(src[i]) * inv;
    if (flags & FLAG_NORM) a *= w[i];
    const T ra = from_f32<T>(a * scale);
    if (inplace) src[i] = ra;
    if (cdst) cdst[i] = ra;
  }
}

// Prompts, bfloat16, all dims rotated, head size 16 * 2^j: a head is taken by hd / 16 lanes, each
// with 8 adjacent dims of either half (16-byte loads and stores), so a warp takes 32 / (hd / 16)
// heads at once and a token's query and key heads are a dozen warp tasks instead of forty.  One
// CTA per token, a warp per task.  Value heads are not touched here.
template <int LANES>   // lanes per head = hd / 16
__global__ void __launch_bounds__(320, 3) head_norm_rope_cache_wide_kernel(bf16* __restrict__ qkv, int ntok, int nh, int nkv, int hd,
                                                 const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                                 const float* __restrict__ inv_freq, float q_scale,
                                                 const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                                 const int* __restrict__ seq_slot, PagedKV kv,
                                                 bf16* __restrict__ kcache, int flags) {
  extern __shared__ float trig[];   // cos [hd / 2], sin [hd / 2]
  pdl_release_next();
  const int t = blockIdx.x, half = hd / 2;
  const int pos = tok_pos[t];
  float* cs = trig;
  float* sn = trig + half;
  int page = 0;   // needed for the key heads' stores only: its loads run under the heads' loads
  if (flags & FLAG_CACHE)
    page = kv.page_table[(size_t)seq_slot[tok_seq[t]] * kv.table_width + (pos / kv.page_size) % kv.table_width];
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
  __syncthreads();
  pdl_wait_prior();   // the angles and the page came from the step's inputs; q, k, v from the kernel before
  constexpr int HEADS = 32 / LANES;
  const int lane = threadIdx.x & 31, sub = lane % LANES, which = lane / LANES;
  const int heads = nh + 2 * nkv, qk = nh + nkv;
  for (int h0 = (threadIdx.x >> 5) * HEADS; h0 < qk; h0 += (blockDim.x >> 5) * HEADS) {
    const int h = h0 + which;
    const bool live = h < qk;
    const bool is_q = h < nh;
    bf16* src = qkv + ((size_t)t * heads + (live ? h : 0)) * hd;
    const int i = 8 * sub;   // this lane: dims i .. i + 7 and i + half .. i + half + 7
    uint4 ra = make_uint4(0, 0, 0, 0), rb = ra;
    if (live) {
      ra = *(const uint4*)(src + i);
      rb = *(const uint4*)(src + i + half);
    }
    const float* w = is_q ? qw : kw;
    float wa[8], wb[8], a[8], b[8];
    if ((flags & FLAG_NORM) && live) {
      *(float4*)&wa[0] = *(const float4*)(w + i);
      *(float4*)&wa[4] = *(const float4*)(w + i + 4);
      *(float4*)&wb[0] = *(const float4*)(w + i + half);
      *(float4*)&wb[4] = *(const float4*)(w + i + half + 4);
    }
    const __nv_bfloat162* pa = (const __nv_bfloat162*)&ra;
    const __nv_bfloat162* pb = (const __nv_bfloat162*)&rb;
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 fa = __bfloat1622float2(pa[j]), fb = __bfloat1622float2(pb[j]);
      a[2 * j] = fa.x; a[2 * j + 1] = fa.y; b[2 * j] = fb.x; b[2 * j + 1] = fb.y;
      ss += fa.x * fa.x + fa.y * fa.y + fb.x * fb.x + fb.y * fb.y;
    }
    float inv = 1.f;
    if (flags & FLAG_NORM) {
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      inv = 1.0f / sqrtf(ss / (float)hd + eps);
    }
    if (!live) continue;
    const float scale = is_q ? q_scale : 1.f;
    float c[8], sgn[8];
    *(float4*)&c[0] = *(const float4*)(cs + i);
    *(float4*)&c[4] = *(const float4*)(cs + i + 4);
    *(float4*)&sgn[0] = *(const float4*)(sn + i);
    *(float4*)&sgn[4] = *(const float4*)(sn + i + 4);
    uint4 oa, ob;
    __nv_bfloat162* qa = (__nv_bfloat162*)&oa;
    __nv_bfloat162* qb = (__nv_bfloat162*)&ob;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float lo[2], hi[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int d = 2 * j + e;
        float x = a[d] * inv, y = b[d] * inv;
        if (flags & FLAG_NORM) {
          x *= wa[d];
          y *= wb[d];
        }
        lo[e] = (x * c[d] - y * sgn[d]) * scale;
        hi[e] = (y * c[d] + x * sgn[d]) * scale;
      }
      qa[j] = __floats2bfloat162_rn(lo[0], lo[1]);
      qb[j] = __floats2bfloat162_rn(hi[0], hi[1]);
    }
    *(uint4*)(src + i) = oa;
    *(uint4*)(src + i + half) = ob;
    if (!is_q && (flags & FLAG_CACHE)) {
      bf16* cdst = kcache + (((size_t)page * nkv + (h - nh)) * kv.page_size + pos % kv.page_size) * hd;
      *(uint4*)(cdst + i) = oa;
      *(uint4*)(cdst + i + half) = ob;
    }
  }
}

// A CTA takes `heads_per_cta` heads of one token (grid: tokens x groups of heads): the token's
// rot / 2 angles (float32(position) * inv_freq, as the reference) and their cos and sin are computed
// once into shared memory and the token's page is looked up once, while the heads' loads are already
// on their way; then the warps take the heads in turn.  Prompts give a CTA all heads of a token (the
// angles are computed once per token); decoding gives every warp one head, since there the kernel
// is a chain of latencies and not work.
template <typename T>
__global__ void head_norm_rope_cache_kernel(T* __restrict__ qkv, int ntok, int nh, int nkv, int hd, int rot,
                                            const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                            const float* __restrict__ inv_freq, float q_scale,
                                            const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                                            const int* __restrict__ seq_slot, PagedKV kv, T* __restrict__ kcache,
                                            T* __restrict__ vcache, int flags, int heads_per_cta) {
  extern __shared__ float trig[];   // cos [rot / 2], sin [rot / 2]
  pdl_release_next();
  // positions, slots and the page table are the step's inputs: the angles and the page are worked
  // out while the kernel before this one (which makes q, k and v) is still running
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = (flags & FLAG_ROPE) ? rot / 2 : 0;
  float* cs = trig;
  float* sn = trig + half;
  int page = 0;
  if (flags & FLAG_CACHE)
    page = kv.page_table[(size_t)seq_slot[tok_seq[t]] * kv.table_width + (pos / kv.page_size) % kv.table_width];
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf((float)pos * inv_freq[i], &sn[i], &cs[i]);
  __syncthreads();
  pdl_wait_prior();
  const int heads = nh + 2 * nkv, h0 = blockIdx.y * heads_per_cta;
  const int h1 = min(heads, h0 + heads_per_cta);
  for (int h = h0 + (threadIdx.x >> 5); h < h1; h += blockDim.x >> 5)
    head_norm_rope_cache_one<T>(qkv, t, h, pos, nh, nkv, hd, rot, qw, kw, eps, cs, sn, q_scale, page, kv, kcache, vcache,
                                flags);
}

// The values of 32 consecutive packed tokens for one kv head, written into the cache through a
// shared-memory transpose: rows are read 16 bytes at a time, and each store instruction of a warp
// then covers one dim of 32 tokens, which are consecutive positions of a page for a prompt (64
// contiguous bytes instead of 32 scattered two-byte stores).
template <typename T>
__global__ void __launch_bounds__(128) value_cache_tile_kernel(const T* __restrict__ qkv, int ntok, int nh, int nkv, int hd,
                                                               const int* __restrict__ tok_pos,
                                                               const int* __restrict__ tok_seq,
                                                               const int* __restrict__ seq_slot, PagedKV kv,
                                                               T* __restrict__ vcache) {
  extern __shared__ unsigned char tile_raw[];
  T* tile = (T*)tile_raw;                 // [32][hd + 2]
  pdl_release_next();
  pdl_wait_prior();
  const int t0 = blockIdx.x * 32, kvh = blockIdx.y, pitch = hd + 2;
  const int heads = nh + 2 * nkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < 32; r += 4) {
    const int t = t0 + r;
    if (t < ntok) {
      const T* src = qkv + ((size_t)t * heads + nh + nkv + kvh) * hd;
      for (int i = lane; i < hd; i += 32) tile[r * pitch + i] = src[i];
    }
  }
  __syncthreads();
  const int t = t0 + lane;
  if (t >= ntok) return;
  T* dst = vcache + kv.vcol(seq_slot[tok_seq[t]], tok_pos[t], kvh);
  for (int d = warp; d < hd; d += 4) dst[(size_t)d * kv.page_size] = tile[lane * pitch + d];
}

GB_EXPORT int gb_head_norm_rope_cache(void* qkv, int dtype, int ntok, int nh, int nkv, int hd, int rot,
                                      const float* qw, const float* kw, float eps, const float* inv_freq,
                                      float q_scale, const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                      const int* page_table, int table_width, int page_size, void* kcache,
                                      void* vcache, int flags, cudaStream_t stream) {
  if (ntok <= 0) return 0;
  if (rot < 0 || rot > hd || (rot & 1)) return GB_ERR_SIZE;
  if ((flags & FLAG_NORM) && (!qw || !kw)) return GB_ERR_ARG;
  if ((flags & FLAG_ROPE) && !inv_freq) return GB_ERR_ARG;
  PagedKV kv{page_table, table_width, page_size, nkv, hd};
  // prompts: values through the transposing kernel (FLAG_SINGLE: every token is a single position
  // of another sequence, where that kernel would gather nothing)
  const bool v_tiled = (flags & FLAG_CACHE) && !(flags & FLAG_SINGLE) && nkv > 0 && ntok >= 64;
  if (v_tiled) flags |= FLAG_V_TILED;
  const int heads = nh + 2 * nkv;
  const int lanes = hd / 16;
  if (v_tiled && dtype == GB_BF16 && (flags & FLAG_ROPE) && (flags & FLAG_INPLACE) && rot == hd && hd % 16 == 0 &&
      (lanes & (lanes - 1)) == 0 && lanes <= 16 && (((uintptr_t)qkv | (uintptr_t)kcache) & 15) == 0) {
    const int tasks = ((nh + nkv) * lanes + 31) / 32;
    const int threads = 32 * (tasks < 10 ? tasks : 10);   // 10 warps: three CTAs share an SM
    const size_t trig_bytes = (size_t)hd * sizeof(float);
#define GB_WIDE(L) \
  gb_launch(head_norm_rope_cache_wide_kernel<L>, ntok, threads, trig_bytes, stream, (bf16*)qkv, ntok, nh, nkv, hd, qw, kw, eps, \
            inv_freq, q_scale, tok_pos, tok_seq, seq_slot, kv, (bf16*)kcache, flags)
    switch (lanes) {
      case 1: GB_WIDE(1); break;
      case 2: GB_WIDE(2); break;
      case 4: GB_WIDE(4); break;
      case 8: GB_WIDE(8); break;
      default: GB_WIDE(16); break;
    }
#undef GB_WIDE
    int rc = gb_launch_status();
    if (rc != 0) return rc;
    dim3 vgrid((ntok + 31) / 32, nkv);
    gb_launch(value_cache_tile_kernel<bf16>, vgrid, 128, (size_t)32 * (hd + 2) * 2, stream, (const bf16*)qkv, ntok, nh, nkv,
              hd, tok_pos, tok_seq, seq_slot, kv, (bf16*)vcache);
    return gb_launch_status();
  }
  const int threads = heads >= 8 ? 256 : 32 * heads;
  const int heads_per_cta = ntok >= 64 ? heads : threads / 32;
  const dim3 grid(ntok, (heads + heads_per_cta - 1) / heads_per_cta);
  const size_t trig_bytes = (size_t)rot * sizeof(float);
  if (dtype == GB_F32)
    gb_launch(head_norm_rope_cache_kernel<float>, grid, threads, trig_bytes, stream,
        (float*)qkv, ntok, nh, nkv, hd, rot, qw, kw, eps, inv_freq, q_scale, tok_pos, tok_seq, seq_slot, kv,
        (float*)kcache, (float*)vcache, flags, heads_per_cta);
  else if (dtype == GB_BF16)
    gb_launch(head_norm_rope_cache_kernel<bf16>, grid, threads, trig_bytes, stream,
        (bf16*)qkv, ntok, nh, nkv, hd, rot, qw, kw, eps, inv_freq, q_scale, tok_pos, tok_seq, seq_slot, kv,
        (bf16*)kcache, (bf16*)vcache, flags, heads_per_cta);
  else
    return GB_ERR_DTYPE;
  int rc = gb_launch_status();
  if (rc != 0 || !v_tiled) return rc;
  dim3 vgrid((ntok + 31) / 32, nkv);
  if (dtype == GB_F32)
    gb_launch(value_cache_tile_kernel<float>, vgrid, 128, (size_t)32 * (hd + 2) * 4, stream, (const float*)qkv, ntok, nh, nkv,
              hd, tok_pos, tok_seq, seq_slot, kv, (float*)vcache);
  else
    gb_launch(value_cache_tile_kernel<bf16>, vgrid, 128, (size_t)32 * (hd + 2) * 2, stream, (const bf16*)qkv, ntok, nh, nkv,
              hd, tok_pos, tok_seq, seq_slot, kv, (bf16*)vcache);
  return gb_launch_status();
}

// ------------------------------------------------------------------ gated activation
// out[t, i] = silu(gu[t, i]) * gu[t, inter + i];  silu(a) = a / (1 + exp(-a)).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, long long total, int inter) {
  pdl_release_next();
  pdl_wait_prior();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / inter;
  const int i = (int)(idx % inter);
  const float g = to_f32(gu[t * 2 * inter + i]), u = to_f32(gu[t * 2 * inter + inter + i]);
  out[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
}

GB_EXPORT int gb_silu_mul(const void* gu, void* out, int dtype, int ntok, int inter, cudaStream_t stream) {
  const long long total = (long long)ntok * inter;
  if (total <= 0) return 0;
  const unsigned grid = (unsigned)((total + 255) / 256);
  if (dtype == GB_F32)
    gb_launch(silu_mul_kernel<float>, grid, 256, 0, stream, (const float*)gu, (float*)out, total, inter);
  else if (dtype == GB_BF16)
    gb_launch(silu_mul_kernel<bf16>, grid, 256, 0, stream, (const bf16*)gu, (bf16*)out, total, inter);
  else
    return GB_ERR_DTYPE;
  return gb_launch_status();
}
