// Token sampling on the device: greedy, temperature, top-k and top-p, one CTA per row.
//
// Meaning of the options (as in umarhassan-cloud/kvforge, src/tokenvault/sampling.py:40-66):
// temperature 0 picks the argmax of the logits; otherwise logits are divided by the
// temperature; top-k keeps the k largest; top-p keeps, in descending order, the entries
// whose mass *before* them is below top_p (so the top entry always stays); the token is
// drawn from the softmax of what is kept.
//
// How: no sort.  The k-th largest value and the top-p cut are found by a radix descent over
// the order-preserving integer image of the floats (4 levels of 8 bits), by count for
// top-k and by probability mass for top-p.  Masses are exp(x - max) in 2^-40 fixed point
// summed as 64-bit integers, so every sum is exact and independent of the order of
// addition: the same row, options and random key always give the same token.  Values tied
// with the k-th largest all stay.  The draw is the inverse CDF in index order with a
// uniform integer in [0, total mass).
#include "common.cuh"

using namespace kvf;

namespace {

constexpr int THREADS = 512;
constexpr int NWARPS = THREADS / 32;
constexpr float FIX_ONE = 1099511627776.0f;  // 2^40

__device__ __forceinline__ unsigned ordered_key(float v) {
  const unsigned b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const unsigned long long t = __shfl_xor_sync(0xffffffffu, v, o);
    v = t > v ? t : v;
  }
  return v;
}

constexpr int MAX_BLOCKS = 512;  // stretches of the vocabulary whose masses the draw keeps in shared memory

struct Shared {
  unsigned long long hist[NWARPS][256];  // per-warp histograms (count or mass)
  unsigned long long red[NWARPS];
  unsigned long long bcast[3];
  unsigned long long blk[MAX_BLOCKS];    // mass of each stretch, in index order
  float fred[32];
};

// f(i, row[i]) for every i < V, each thread taking its share.  Rows that start on a 16-byte boundary
// are read four values at a time, and four such reads are in flight per thread: a pass over the
// row is bound by L2 latency otherwise (one CTA reads a whole row).
template <typename F>
__device__ __forceinline__ void for_each(const float* __restrict__ row, int V, F f) {
  if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(row);
    const int n4 = V >> 2;
#pragma unroll 4
    for (int i = threadIdx.x; i < n4; i += THREADS) {
      const float4 v = r4[i];
      f(4 * i, v.x);
      f(4 * i + 1, v.y);
      f(4 * i + 2, v.z);
      f(4 * i + 3, v.w);
    }
    for (int i = (n4 << 2) + threadIdx.x; i < V; i += THREADS) f(i, row[i]);
  } else {
#pragma unroll 4
    for (int i = threadIdx.x; i < V; i += THREADS) f(i, row[i]);
  }
}

// One level of the radix descent.  Among entries with key >= lo_key whose bits above
// `shift + 8` equal `prefix`, histogram (count or mass) by the digit at `shift`, then walk
// digits from 255 down until the running total reaches `remaining`.  Returns the digit and
// updates `remaining` to what is still wanted inside that digit.
template <bool BY_MASS>
__device__ int radix_level(Shared& sh, const float* row, int V, float temp, float mx, unsigned lo_key,
                           unsigned prefix, int shift, unsigned long long& remaining) {
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < NWARPS * 256; i += THREADS) (&sh.hist[0][0])[i] = 0ull;
  __syncthreads();
  for_each(row, V, [&](int, float raw) {
    const float x = raw / temp;
    const unsigned key = ordered_key(x);
    if (key < lo_key) return;
    if (shift < 24 && (key >> (shift + 8)) != prefix) return;
    const unsigned digit = (key >> shift) & 255u;
    const unsigned long long w = BY_MASS ? __float2ull_rz(expf(x - mx) * FIX_ONE) : 1ull;
    if (!BY_MASS && shift == 24) {
      // Counting at the top level (sign and exponent), where nearly all values share a digit: the
      // lanes with the same digit are counted at once and one of them adds to the histogram.
      // (For masses the grouping costs more than the atomics it saves: measured.)
      const unsigned peers = __match_any_sync(__activemask(), digit);
      if ((int)(threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&sh.hist[warp][digit], (unsigned long long)__popc(peers));
    } else {
      atomicAdd(&sh.hist[warp][digit], w);  // integer sums: the order does not matter
    }
  });
  __syncthreads();
  // fold the per-warp histograms: thread t < 256 owns digit t
  if (threadIdx.x < 256) {
    unsigned long long s = 0;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) s += sh.hist[w][threadIdx.x];
    sh.hist[0][threadIdx.x] = s;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long cum = 0;
    int chosen = 0;
    unsigned long long rem = remaining;
    bool found = false;
    for (int dgt = 255; dgt >= 0; --dgt) {
      const unsigned long long c = sh.hist[0][dgt];
      if (cum + c >= remaining) {
        chosen = dgt;
        rem = remaining - cum;
        found = true;
        break;
      }
      cum += c;
    }
    if (!found) {  // fewer than wanted exist under this prefix: take everything
      chosen = 0;
      rem = 0;
    }
    sh.bcast[0] = (unsigned long long)chosen;
    sh.bcast[1] = rem;
  }
  __syncthreads();
  remaining = sh.bcast[1];
  const int chosen = (int)sh.bcast[0];
  __syncthreads();
  return chosen;
}

__global__ void __launch_bounds__(THREADS, 2)
sample_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temps,
              const int* __restrict__ top_ks, const float* __restrict__ top_ps,
              const unsigned long long* __restrict__ rand_keys, int* __restrict__ out_tokens,
              float* __restrict__ probs_out) {
  __shared__ Shared sh;
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  float* prow = probs_out ? probs_out + (size_t)r * V : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float T = temps ? temps[r] : 0.f;

  if (T == 0.f) {
    // ---- greedy: highest logit, lowest index among equals
    unsigned long long best = 0;
    for_each(row, V, [&](int i, float x) {
      const unsigned long long c = ((unsigned long long)ordered_key(x) << 32) | (0xFFFFFFFFu - (unsigned)i);
      best = c > best ? c : best;
    });
    best = warp_max_u64(best);
    if (lane == 0) sh.red[warp] = best;
    __syncthreads();
    if (warp == 0) {
      unsigned long long v = lane < NWARPS ? sh.red[lane] : 0ull;
      v = warp_max_u64(v);
      if (lane == 0) sh.bcast[0] = v;
    }
    __syncthreads();
    const int tok = (int)(0xFFFFFFFFu - (unsigned)(sh.bcast[0] & 0xFFFFFFFFull));
    if (threadIdx.x == 0) out_tokens[r] = tok;
    if (prow)
      for (int i = threadIdx.x; i < V; i += THREADS) prow[i] = (i == tok) ? 1.f : 0.f;
    return;
  }

  // ---- maximum of the scaled row
  float mx = -INFINITY;
  for_each(row, V, [&](int, float x) { mx = fmaxf(mx, x / T); });
  mx = block_max(mx, sh.fred);
  __syncthreads();

  unsigned lo_key = 0u;  // entries with key >= lo_key are kept
  const int k = top_ks ? top_ks[r] : 0;
  if (k > 0 && k < V) {
    unsigned prefix = 0u;
    unsigned long long remaining = (unsigned long long)k;
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      const int dgt = radix_level<false>(sh, row, V, T, mx, 0u, prefix, shift, remaining);
      prefix = (prefix << 8) | (unsigned)dgt;
    }
    lo_key = prefix;  // the k-th largest key
  }

  const float top_p = top_ps ? top_ps[r] : 1.f;
  if (top_p < 1.f) {
    // mass of what top-k kept
    unsigned long long z = 0;
    for_each(row, V, [&](int, float raw) {
      const float x = raw / T;
      if (ordered_key(x) >= lo_key) z += __float2ull_rz(expf(x - mx) * FIX_ONE);
    });
    z = warp_sum_u64(z);
    if (lane == 0) sh.red[warp] = z;
    __syncthreads();
    if (threadIdx.x == 0) {
      unsigned long long s = 0;
      for (int w = 0; w < NWARPS; ++w) s += sh.red[w];
      unsigned long long tgt = (unsigned long long)ceil((double)top_p * (double)s);
      if (tgt < 1ull) tgt = 1ull;
      if (tgt > s) tgt = s;
      sh.bcast[0] = tgt;
    }
    __syncthreads();
    unsigned long long remaining = sh.bcast[0];
    __syncthreads();
    unsigned prefix = 0u;
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      const int dgt = radix_level<true>(sh, row, V, T, mx, lo_key, prefix, shift, remaining);
      prefix = (prefix << 8) | (unsigned)dgt;
    }
    lo_key = prefix > lo_key ? prefix : lo_key;
  }

  // ---- draw: the inverse CDF in index order.  The row is cut into stretches of `bs` entries (at
  // most MAX_BLOCKS of them); warps sum the kept mass of each stretch, one thread finds the
  // stretch the target falls into, one warp walks that stretch 32 entries at a time.
  const int bs = 1024 * ((V + 1024 * MAX_BLOCKS - 1) / (1024 * MAX_BLOCKS));
  const int nblk = (V + bs - 1) / bs;
  auto mass_at = [&](int i) -> unsigned long long {
    if (i >= V) return 0ull;
    const float x = row[i] / T;
    return ordered_key(x) >= lo_key ? __float2ull_rz(expf(x - mx) * FIX_ONE) : 0ull;
  };
  for (int b = warp; b < nblk; b += NWARPS) {
    unsigned long long part = 0;
    for (int c0 = b * bs; c0 < (b + 1) * bs; c0 += 1024) {
#pragma unroll 8
      for (int j = 0; j < 32; ++j) part += mass_at(c0 + 32 * j + lane);
    }
    part = warp_sum_u64(part);
    if (lane == 0) sh.blk[b] = part;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned long long total = 0;
    for (int b = 0; b < nblk; ++b) total += sh.blk[b];
    const unsigned long long rnd = splitmix64(rand_keys ? rand_keys[r] : 0ull);
    const unsigned long long target = __umul64hi(rnd, total);  // uniform in [0, total)
    int b_sel = nblk - 1;
    unsigned long long before = 0;
    for (int b = 0; b < nblk; ++b) {
      if (target < before + sh.blk[b]) {
        b_sel = b;
        break;
      }
      before += sh.blk[b];
    }
    sh.bcast[0] = target - before;
    sh.bcast[1] = total;
    sh.bcast[2] = (unsigned long long)b_sel;
  }
  __syncthreads();
  const int b_sel = (int)sh.bcast[2];
  const unsigned long long total = sh.bcast[1];
  if (warp == 0) {
    unsigned long long rem = sh.bcast[0];
    int tok = -1, last_kept = -1;
    const int s_begin = b_sel * bs, s_end = min(V, s_begin + bs);
    for (int base = s_begin; base < s_end && tok < 0; base += 32) {
      const unsigned long long w = mass_at(base + lane);
      unsigned long long incl = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
      }
      const unsigned hit = __ballot_sync(0xffffffffu, w > 0 && incl > rem);
      const unsigned kept = __ballot_sync(0xffffffffu, w > 0);
      if (kept) last_kept = base + 31 - __clz(kept);
      if (hit) {
        tok = base + __ffs(hit) - 1;
      } else {
        rem -= __shfl_sync(0xffffffffu, incl, 31);
      }
    }
    if (tok < 0) tok = last_kept >= 0 ? last_kept : 0;
    if (lane == 0) out_tokens[r] = tok;
  }
  if (prow) {
    const float inv = 1.f / (float)total;
    for (int i = threadIdx.x; i < V; i += THREADS) {
      const float x = row[i] / T;
      const unsigned long long w = ordered_key(x) >= lo_key ? __float2ull_rz(expf(x - mx) * FIX_ONE) : 0ull;
      prow[i] = (float)w * inv;
    }
  }
}

// ---- greedy for a whole batch in two short kernels: many CTAs per row find the best
// (value, lowest index) of a stretch of the vocabulary, one warp per row picks among them.
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, long long ld, int V, int chunks,
                      unsigned long long* __restrict__ partial) {
  __shared__ unsigned long long red[8];
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.y, c = blockIdx.x;
  const int len = (V + chunks - 1) / chunks;
  const int lo = c * len, hi = min(V, lo + len);
  const float* row = logits + (size_t)r * ld;
  unsigned long long best = 0;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const unsigned long long v = ((unsigned long long)ordered_key(row[i]) << 32) | (0xFFFFFFFFu - (unsigned)i);
    best = v > best ? v : best;
  }
  best = warp_max_u64(best);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = best;
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned long long v = threadIdx.x < 8 ? red[threadIdx.x] : 0ull;
    v = warp_max_u64(v);
    if (threadIdx.x == 0) partial[(size_t)r * chunks + c] = v;
  }
}

__global__ void __launch_bounds__(32)
argmax_final_kernel(const unsigned long long* __restrict__ partial, int chunks, int* __restrict__ out_tokens) {
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.x;
  unsigned long long best = 0;
  for (int c = threadIdx.x; c < chunks; c += 32) {
    const unsigned long long v = partial[(size_t)r * chunks + c];
    best = v > best ? v : best;
  }
  best = warp_max_u64(best);
  if (threadIdx.x == 0) out_tokens[r] = (int)(0xFFFFFFFFu - (unsigned)(best & 0xFFFFFFFFull));
}

}  // namespace

// logits: [R, V] float with row stride ld.  temps/top_ks/top_ps/rand_keys: [R] (null temps =
// all greedy).  out_tokens: [R] int.  probs_out: optional [R, V] float, the distribution
// each token was drawn from (for tests).
KVF_API int kvf_sample_f32(const float* logits, long long ld, int R, int V, const float* temps,
                           const int* top_ks, const float* top_ps, const unsigned long long* rand_keys,
                           int* out_tokens, float* probs_out, cudaStream_t st) {
  if (R <= 0) return 0;
  if (V <= 0) return (int)cudaErrorInvalidValue;
  return launch(sample_kernel, dim3(R), dim3(THREADS), 0, st, logits, ld, V, temps, top_ks, top_ps, rand_keys,
                out_tokens, probs_out);
}

// Greedy tokens of float logits [R, V] (row stride ld): the highest logit, the lowest index
// among equals.  `partial` is scratch of R * chunks 64-bit words.
KVF_API int kvf_argmax_f32(const float* logits, long long ld, int R, int V, unsigned long long* partial, int chunks,
                           int* out_tokens, cudaStream_t st) {
  if (R <= 0) return 0;
  if (V <= 0 || chunks <= 0 || !partial || (unsigned)R > 65535u) return (int)cudaErrorInvalidValue;
  int rc = launch(argmax_partial_kernel, dim3(chunks, R), dim3(256), 0, st, logits, ld, V, chunks, partial);
  if (rc) return rc;
  return launch(argmax_final_kernel, dim3(R), dim3(32), 0, st, (const unsigned long long*)partial, chunks, out_tokens);
}
