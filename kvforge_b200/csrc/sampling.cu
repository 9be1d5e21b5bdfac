// Token sampling on the device: greedy, temperature, top-k and top-p.  A row is shared by a
// thread-block cluster of up to 8 CTAs (each takes a slice of the vocabulary); what the CTAs of a
// row find (maximum, histograms, masses) meets through distributed shared memory, and every CTA
// works out the same decisions from the same sums, so nothing has to be sent back.
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
// uniform integer in [0, total mass).  A pass that puts the row into coarse buckets below its
// maximum comes first: when the buckets down to the one with the cut (the k-th largest, or the
// top-p share of the mass) hold at most 512 entries, those are gathered in the first CTA's
// shared memory and the cuts and the draw are worked out there, by the same rules, instead of by
// radix passes over the row.  Under top-p alone on a flat row (more entries than that over the
// cut) only the entries of the bucket the cut falls into are gathered, since all of the buckets
// above it stay; the cut is found among them and the draw goes over the row.  The radix passes
// remain for crowded buckets, many equal values and large k.
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
constexpr int MAX_CLUSTER = 8;
constexpr int CAND_MAX = 512;  // up to this many entries are gathered in the first CTA and finished there (7 arrays: 14 KB + 4 KB)

struct Shared {
  unsigned long long hist[NWARPS][256];  // per-warp histograms (count or mass); [0] holds the CTA's fold
  unsigned long long tot[256];           // the row's histogram (all CTAs of the cluster)
  unsigned long long red[NWARPS];
  unsigned long long bcast[4];
  unsigned long long blk[MAX_BLOCKS];    // mass of each stretch, in index order
  unsigned long long xu;                 // what this CTA offers to the others (a sum or a maximum)
  unsigned n_cand;                       // the first CTA's: how many entries passed top-k
  float xf;
  float fred[32];
};

__device__ __forceinline__ uint32_t sm32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// the address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t in_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ unsigned long long ld_cluster_u64(uint32_t addr) {
  unsigned long long v;
  asm volatile("ld.shared::cluster.u64 %0, [%1];" : "=l"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_cluster_u32(uint32_t addr) {
  unsigned v;
  asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void st_cluster_u32(uint32_t addr, unsigned v) {
  asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}
// every thread of every CTA of the cluster
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// The cluster's view of a row: CTA `rank` of `nranks` owns entries [lo, hi).
struct Slice {
  const float* row;
  int V, lo, hi;
  uint32_t rank, nranks;
};

// f(i, row[i]) for every i of the slice, each thread taking its share.  Slices start at multiples of
// 4; rows that start on a 16-byte boundary are read four values at a time, and four such reads are
// in flight per thread: a pass is bound by L2 latency otherwise.
template <typename F>
__device__ __forceinline__ void for_each(const Slice& s, F f) {
  if ((reinterpret_cast<uintptr_t>(s.row) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(s.row);
    const int b4 = s.lo >> 2, e4 = s.hi >> 2;  // whole float4s inside the slice
#pragma unroll 4
    for (int i = b4 + threadIdx.x; i < e4; i += THREADS) {
      const float4 v = r4[i];
      f(4 * i, v.x);
      f(4 * i + 1, v.y);
      f(4 * i + 2, v.z);
      f(4 * i + 3, v.w);
    }
    for (int i = (e4 << 2) + threadIdx.x; i < s.hi; i += THREADS) f(i, s.row[i]);
  } else {
#pragma unroll 4
    for (int i = s.lo + threadIdx.x; i < s.hi; i += THREADS) f(i, s.row[i]);
  }
}

// Sums / maxima over the cluster: each CTA offers its value, all read all.  Two barriers: one before
// the reads, one after (the slot may be written again).
__device__ __forceinline__ unsigned long long cluster_sum_u64(Shared& sh, const Slice& s, unsigned long long mine) {
  if (threadIdx.x == 0) sh.xu = mine;
  cluster_barrier();
  unsigned long long total = 0;
  for (uint32_t c = 0; c < s.nranks; ++c) total += ld_cluster_u64(in_cta(sm32(&sh.xu), c));
  cluster_barrier();
  return total;
}
__device__ __forceinline__ unsigned long long cluster_max_u64(Shared& sh, const Slice& s, unsigned long long mine) {
  if (threadIdx.x == 0) sh.xu = mine;
  cluster_barrier();
  unsigned long long best = 0;
  for (uint32_t c = 0; c < s.nranks; ++c) {
    const unsigned long long v = ld_cluster_u64(in_cta(sm32(&sh.xu), c));
    best = v > best ? v : best;
  }
  cluster_barrier();
  return best;
}
__device__ __forceinline__ float cluster_max_f32(Shared& sh, const Slice& s, float mine) {
  if (threadIdx.x == 0) sh.xf = mine;
  cluster_barrier();
  float best = -INFINITY;
  for (uint32_t c = 0; c < s.nranks; ++c) best = fmaxf(best, ld_cluster_f32(in_cta(sm32(&sh.xf), c)));
  cluster_barrier();
  return best;
}
// the CTA's sum of a per-thread value
__device__ __forceinline__ unsigned long long block_sum_u64(Shared& sh, unsigned long long v) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  v = warp_sum_u64(v);
  __syncthreads();
  if (lane == 0) sh.red[warp] = v;
  __syncthreads();
  unsigned long long s = 0;
#pragma unroll
  for (int w = 0; w < NWARPS; ++w) s += sh.red[w];
  return s;
}

__device__ __forceinline__ unsigned block_max_u32(Shared& sh, unsigned v) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = max(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) sh.red[warp] = v;
  __syncthreads();
  unsigned m = 0;
#pragma unroll
  for (int w = 0; w < NWARPS; ++w) m = max(m, (unsigned)sh.red[w]);
  return m;
}

// The first position (in walking order) at which the running total of a[.] reaches (REACH: >=) or
// passes (!REACH: >) `want`, found by one warp: lane l sums the positions l*per .. l*per+per-1 of the
// walk, a scan over the lanes finds the lane, the lane walks its own stretch.  a(i) gives the value
// at walk position i.  Returns the position, or -1 if the total never gets there; `before` is the
// total ahead of the returned position.
template <bool REACH, typename A>
__device__ __forceinline__ int warp_find(int n, A a, unsigned long long want, unsigned long long& before) {
  const int lane = threadIdx.x & 31;
  const int per = (n + 31) / 32;
  unsigned long long mine = 0;
  for (int j = 0; j < per; ++j) {
    const int i = lane * per + j;
    if (i < n) mine += a(i);
  }
  unsigned long long incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const bool got = REACH ? incl >= want : incl > want;
  const unsigned hit = __ballot_sync(0xffffffffu, got && mine > 0);
  if (!hit) return -1;
  const int src = __ffs(hit) - 1;
  int pos = -1;
  unsigned long long cum = incl - mine;  // ahead of this lane's stretch
  if (lane == src) {
    for (int j = 0; j < per; ++j) {
      const int i = lane * per + j;
      const unsigned long long v = i < n ? a(i) : 0ull;
      if (v > 0 && (REACH ? cum + v >= want : cum + v > want)) {
        pos = i;
        break;
      }
      cum += v;
    }
  }
  pos = __shfl_sync(0xffffffffu, pos, src);
  before = __shfl_sync(0xffffffffu, cum, src);
  return pos;
}

// One level of the radix descent.  Among entries with key >= lo_key whose bits above
// `shift + 8` equal `prefix`, histogram (count or mass) by the digit at `shift`, then walk
// digits from 255 down until the running total reaches `remaining`.  Returns the digit and
// updates `remaining` to what is still wanted inside that digit.  Every CTA of the cluster
// histograms its slice, sums all the CTAs' histograms and takes the same walk.
template <bool BY_MASS>
__device__ int radix_level(Shared& sh, const Slice& sl, float temp, float mx, unsigned lo_key, unsigned prefix, int shift,
                           unsigned long long& remaining) {
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < NWARPS * 256; i += THREADS) (&sh.hist[0][0])[i] = 0ull;
  __syncthreads();
  for_each(sl, [&](int, float raw) {
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
  cluster_barrier();  // every CTA's fold is there
  if (threadIdx.x < 256) {
    unsigned long long s = 0;
    for (uint32_t c = 0; c < sl.nranks; ++c) s += ld_cluster_u64(in_cta(sm32(&sh.hist[0][threadIdx.x]), c));
    sh.tot[threadIdx.x] = s;
  }
  cluster_barrier();  // the folds have been read: the histograms may be cleared again
  if (threadIdx.x < 32) {
    // walk the digits from 255 down until the running total reaches what is wanted
    unsigned long long before = 0;
    const int at = warp_find<true>(256, [&](int i) { return sh.tot[255 - i]; }, remaining, before);
    if (threadIdx.x == 0) {
      // (fewer than wanted exist under this prefix: take everything)
      sh.bcast[0] = at >= 0 ? (unsigned long long)(255 - at) : 0ull;
      sh.bcast[1] = at >= 0 ? remaining - before : 0ull;
    }
  }
  __syncthreads();
  remaining = sh.bcast[1];
  const int chosen = (int)sh.bcast[0];
  __syncthreads();
  return chosen;
}

// Buckets of an eighth of a nat below the row's maximum, 255 for the maximum itself down to 0 for
// 32 nats or more below it: a coarse order of the values (a larger value never has a smaller
// bucket) in which a peaked row's k largest, or its top-p part, fill a few sparse buckets.
__device__ __forceinline__ unsigned linear_bucket(float x, float mx) { return 255u - min(255u, __float2uint_rz((mx - x) * 8.f)); }

// Histogram (count or mass) of the whole row by linear_bucket, then the walk from bucket 255 down
// until the running total reaches what is wanted: `want` itself (counts), or the share `top_p` of
// the row's whole mass, which the histogram gives (masses).  Returns the bucket where that
// happens; `upto` says how many entries lie in the buckets down to and including it (by mass: a
// lower bound worked out from the masses), `all` is the total of the row, `above` the total of the
// buckets over the returned one.
template <bool BY_MASS>
__device__ int linear_level(Shared& sh, const Slice& sl, float temp, float mx, unsigned long long want, float top_p,
                            unsigned long long& upto, unsigned long long& all, unsigned long long& above) {
  const int warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < NWARPS * 256; i += THREADS) (&sh.hist[0][0])[i] = 0ull;
  __syncthreads();
  for_each(sl, [&](int, float raw) {
    const float x = raw / temp;
    const unsigned digit = linear_bucket(x, mx);
    // (a row spreads over many buckets, so the lanes of a warp seldom meet in one)
    atomicAdd(&sh.hist[warp][digit], BY_MASS ? __float2ull_rz(expf(x - mx) * FIX_ONE) : 1ull);
  });
  __syncthreads();
  if (threadIdx.x < 256) {
    unsigned long long s = 0;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) s += sh.hist[w][threadIdx.x];
    sh.hist[0][threadIdx.x] = s;
  }
  cluster_barrier();  // every CTA's fold is there
  if (threadIdx.x < 256) {
    unsigned long long s = 0;
    for (uint32_t c = 0; c < sl.nranks; ++c) s += ld_cluster_u64(in_cta(sm32(&sh.hist[0][threadIdx.x]), c));
    sh.tot[threadIdx.x] = s;
  }
  cluster_barrier();  // the folds have been read
  if (threadIdx.x < 32) {
    unsigned long long total = 0;
    for (int i = threadIdx.x; i < 256; i += 32) total += sh.tot[i];
    total = warp_sum_u64(total);
    unsigned long long wanted = want;
    if (BY_MASS) {
      wanted = (unsigned long long)ceil((double)top_p * (double)total);
      if (wanted < 1ull) wanted = 1ull;
      if (wanted > total) wanted = total;
    }
    unsigned long long before = 0;
    const int at = warp_find<true>(256, [&](int i) { return sh.tot[255 - i]; }, wanted, before);
    if (threadIdx.x == 0) {
      const int bucket = at >= 0 ? 255 - at : 0;  // (fewer than wanted exist: everything)
      sh.bcast[0] = (unsigned long long)bucket;
      sh.bcast[1] = at >= 0 ? before + sh.tot[bucket] : total;
      sh.bcast[2] = total;
      sh.bcast[3] = at >= 0 ? before : 0ull;
      if (BY_MASS) {
        // how many entries that is, at least: a bucket's entries weigh at most exp(-(255 - b) / 8) each
        float least = 0.f;
        for (int b = 255; b >= bucket; --b) least += (float)sh.tot[b] / (expf(-0.125f * (float)(255 - b)) * FIX_ONE);
        sh.bcast[1] = bucket == 0 ? ~0ull : (unsigned long long)least;
      }
    }
  }
  __syncthreads();
  const int bucket = (int)sh.bcast[0];
  upto = sh.bcast[1];
  all = sh.bcast[2];
  above = sh.bcast[3];
  __syncthreads();
  return bucket;
}

// grid (cluster size, rows); the cluster spans x
__global__ void __launch_bounds__(THREADS, 2)
sample_kernel(const float* __restrict__ logits, long long ld, int V, const float* __restrict__ temps,
              const int* __restrict__ top_ks, const float* __restrict__ top_ps,
              const unsigned long long* __restrict__ rand_keys, int* __restrict__ out_tokens,
              float* __restrict__ probs_out) {
  __shared__ Shared sh;
  pdl_launch();
  pdl_wait();
  const int r = blockIdx.y;
  const float* row = logits + (size_t)r * ld;
  float* prow = probs_out ? probs_out + (size_t)r * V : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float T = temps ? temps[r] : 0.f;
  Slice sl;
  sl.row = row;
  sl.V = V;
  sl.rank = blockIdx.x;
  sl.nranks = gridDim.x;
  {
    const int per = (((V + (int)gridDim.x - 1) / (int)gridDim.x) + 3) & ~3;  // a multiple of 4
    sl.lo = min(V, (int)blockIdx.x * per);
    sl.hi = min(V, sl.lo + per);
  }

  if (T == 0.f) {
    // ---- greedy: highest logit, lowest index among equals
    unsigned long long best = 0;
    for_each(sl, [&](int i, float x) {
      const unsigned long long c = ((unsigned long long)ordered_key(x) << 32) | (0xFFFFFFFFu - (unsigned)i);
      best = c > best ? c : best;
    });
    best = warp_max_u64(best);
    if (lane == 0) sh.red[warp] = best;
    __syncthreads();
    unsigned long long v = 0;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) v = sh.red[w] > v ? sh.red[w] : v;
    v = cluster_max_u64(sh, sl, v);
    const int tok = (int)(0xFFFFFFFFu - (unsigned)(v & 0xFFFFFFFFull));
    if (threadIdx.x == 0 && sl.rank == 0) out_tokens[r] = tok;
    if (prow)
      for (int i = sl.lo + threadIdx.x; i < sl.hi; i += THREADS) prow[i] = (i == tok) ? 1.f : 0.f;
    return;
  }

  // ---- maximum of the scaled row
  float mx = -INFINITY;
  for_each(sl, [&](int, float x) { mx = fmaxf(mx, x / T); });
  mx = block_max(mx, sh.fred);
  mx = cluster_max_f32(sh, sl, mx);

  const int k = top_ks ? top_ks[r] : 0;
  const float top_p = top_ps ? top_ps[r] : 1.f;
  const bool by_count = k > 0 && k < V;
  bool have_all = false;  // the row's whole mass is known (from the histogram by mass)
  unsigned long long row_mass = 0;

  // ---- the short way: one more pass puts the row into coarse buckets (by count for top-k, else by
  // mass for top-p); the entries of the buckets down to the one that holds the cut are gathered in
  // the first CTA's shared memory (over the histograms, which are done with), if they are few, and
  // top-k, top-p and the draw are finished there on the exact values: the same masses, the same
  // cuts and the same draw in index order as the passes over the row further down.
  bool cut_found = false;  // the top-p cut is known already (lo_key): no radix descent by mass
  unsigned lo_key = 0u;    // entries with key >= lo_key are kept
  if ((by_count && k <= CAND_MAX) || (!by_count && top_p < 1.f)) {
    unsigned long long upto = 0, all = 0, above = 0;
    const int bucket = by_count ? linear_level<false>(sh, sl, T, mx, (unsigned long long)k, 1.f, upto, all, above)
                                : linear_level<true>(sh, sl, T, mx, 0ull, top_p, upto, all, above);
    unsigned* c_idx = reinterpret_cast<unsigned*>(&sh.hist[0][0]);
    unsigned* c_key = c_idx + CAND_MAX;
    float* c_val = reinterpret_cast<float*>(c_key + CAND_MAX);
    unsigned long long* c_mass = reinterpret_cast<unsigned long long*>(c_val + CAND_MAX);
    unsigned long long* c_kept = c_mass + CAND_MAX;
    have_all = !by_count;
    row_mass = all;
    // Gathers the entries of the buckets from `bucket` up (or of `bucket` alone) in the first CTA's
    // arrays, if they are at most CAND_MAX; returns how many they are (more than CAND_MAX: nothing was
    // sent).  Every CTA first collects what it finds in its own shared memory (it stops collecting when
    // it has more than fit: a flat row would otherwise queue up on the counter), then the CTAs learn one
    // another's numbers and, if all fit, put theirs into the first CTA's arrays one after another.
    auto gather = [&](bool only_cut) -> int {
      unsigned* l_idx = reinterpret_cast<unsigned*>(&sh.hist[8][0]);  // 16 KB in: behind the first CTA's arrays (14 KB)
      float* l_val = reinterpret_cast<float*>(l_idx + CAND_MAX);
      if (threadIdx.x == 0) sh.n_cand = 0u;
      __syncthreads();
      for_each(sl, [&](int i, float raw) {
        const float x = raw / T;
        const unsigned b = linear_bucket(x, mx);
        if ((only_cut ? b == (unsigned)bucket : b >= (unsigned)bucket) && *(volatile unsigned*)&sh.n_cand <= (unsigned)CAND_MAX) {
          const unsigned slot = atomicAdd(&sh.n_cand, 1u);
          if (slot < (unsigned)CAND_MAX) {
            l_idx[slot] = (unsigned)i;
            l_val[slot] = x;
          }
        }
      });
      cluster_barrier();  // every CTA's number stands (and every CTA is done with the histograms)
      int n = 0, offset = 0;
      for (uint32_t c = 0; c < sl.nranks; ++c) {
        const int theirs = (int)ld_cluster_u32(in_cta(sm32(&sh.n_cand), c));
        if (c < sl.rank) offset += theirs;
        n = (theirs > CAND_MAX || n > CAND_MAX) ? 2 * CAND_MAX : n + theirs;
      }
      if (n <= CAND_MAX) {
        const int mine = (int)sh.n_cand;
        const uint32_t a_idx = in_cta(sm32(c_idx), 0), a_val = in_cta(sm32(c_val), 0);
        for (int i = threadIdx.x; i < mine; i += THREADS) {
          st_cluster_u32(a_idx + 4u * (uint32_t)(offset + i), l_idx[i]);
          st_cluster_u32(a_val + 4u * (uint32_t)(offset + i), __float_as_uint(l_val[i]));
        }
      }
      cluster_barrier();  // all of them are in the first CTA (or nobody sent any)
      return n;
    };
    if (upto <= (unsigned long long)CAND_MAX) {  // (by mass this is a lower bound: the true number shows when they are gathered)
      const int n = gather(false);
      if (n <= CAND_MAX) {
        if (sl.rank == 0) {
          for (int i = threadIdx.x; i < n; i += THREADS) {
            c_key[i] = ordered_key(c_val[i]);
            c_mass[i] = __float2ull_rz(expf(c_val[i] - mx) * FIX_ONE);
          }
          __syncthreads();
          if (by_count) {
            // top-k: an entry stays if fewer than k are strictly larger (values tied with the k-th stay)
            for (int i = threadIdx.x; i < n; i += THREADS) {
              int larger = 0;
              const unsigned mine = c_key[i];
              for (int j = 0; j < n; ++j) larger += c_key[j] > mine ? 1 : 0;
              c_kept[i] = larger < k ? c_mass[i] : 0ull;
            }
            __syncthreads();
            for (int i = threadIdx.x; i < n; i += THREADS) c_mass[i] = c_kept[i];
            __syncthreads();
          }
          if (top_p < 1.f) {
            // top-p of the mass that top-k kept (of the whole row without top-k: the entries that were
            // not gathered are all smaller than these): an entry stays if the mass of the strictly
            // larger ones is below the target
            unsigned long long s = all;
            if (by_count) {
              unsigned long long z = 0;
              for (int i = threadIdx.x; i < n; i += THREADS) z += c_mass[i];
              s = block_sum_u64(sh, z);
            }
            unsigned long long remaining = (unsigned long long)ceil((double)top_p * (double)s);
            if (remaining < 1ull) remaining = 1ull;
            if (remaining > s) remaining = s;
            for (int i = threadIdx.x; i < n; i += THREADS) {
              unsigned long long above = 0;
              const unsigned mine = c_key[i];
              for (int j = 0; j < n; ++j) above += c_key[j] > mine ? c_mass[j] : 0ull;
              c_kept[i] = above < remaining ? c_mass[i] : 0ull;
            }
          } else {
            for (int i = threadIdx.x; i < n; i += THREADS) c_kept[i] = c_mass[i];
          }
          __syncthreads();
          unsigned long long z = 0;
          unsigned lowest = 0xFFFFFFFFu;  // the smallest key that stays
          for (int i = threadIdx.x; i < n; i += THREADS) {
            z += c_kept[i];
            if (c_kept[i] > 0ull) lowest = min(lowest, c_key[i]);
          }
          const unsigned long long total = block_sum_u64(sh, z);
          lowest = ~block_max_u32(sh, ~lowest);
          const unsigned long long rnd = splitmix64(rand_keys ? rand_keys[r] : 0ull);
          const unsigned long long target = __umul64hi(rnd, total);  // uniform in [0, total)
          for (int i = threadIdx.x; i < n; i += THREADS) {
            unsigned long long before = 0;
            const unsigned mine = c_idx[i];
            for (int j = 0; j < n; ++j) before += c_idx[j] < mine ? c_kept[j] : 0ull;
            if (before <= target && target - before < c_kept[i]) out_tokens[r] = (int)mine;  // exactly one entry
          }
          if (threadIdx.x == 0) {
            sh.bcast[0] = (unsigned long long)lowest;
            sh.bcast[1] = total;
          }
        }
        if (!prow) return;
        cluster_barrier();  // the cut and the total stand in the first CTA
        const unsigned cut_key = (unsigned)ld_cluster_u64(in_cta(sm32(&sh.bcast[0]), 0));
        const unsigned long long total = ld_cluster_u64(in_cta(sm32(&sh.bcast[1]), 0));
        cluster_barrier();  // read by all
        const float inv = 1.f / (float)total;
        for (int i = sl.lo + threadIdx.x; i < sl.hi; i += THREADS) {
          const float x = row[i] / T;
          const unsigned long long w = ordered_key(x) >= cut_key ? __float2ull_rz(expf(x - mx) * FIX_ONE) : 0ull;
          prow[i] = (float)w * inv;
        }
        return;
      }
    }
    // ---- the middle way (top-p alone, too many entries over the cut to gather): every entry of the
    // buckets over the cut's bucket stays, so only that bucket's entries decide where the cut lies.  If
    // they are few, the first CTA finds the cut among them by the same rule (an entry stays if the mass
    // of the strictly larger ones, `above` included, is below the target), every CTA learns the cut's
    // key, and the draw goes over the row as after the radix descents.  (Bucket 0 holds everything far
    // below the maximum: no.)
    if (!by_count && bucket > 0) {
      const int n = gather(true);
      if (n <= CAND_MAX) {
        if (sl.rank == 0) {
          for (int i = threadIdx.x; i < n; i += THREADS) {
            c_key[i] = ordered_key(c_val[i]);
            c_mass[i] = __float2ull_rz(expf(c_val[i] - mx) * FIX_ONE);
          }
          __syncthreads();
          unsigned long long remaining = (unsigned long long)ceil((double)top_p * (double)all);
          if (remaining < 1ull) remaining = 1ull;
          if (remaining > all) remaining = all;
          unsigned lowest = 0xFFFFFFFFu;
          for (int i = threadIdx.x; i < n; i += THREADS) {
            unsigned long long larger = above;
            const unsigned mine = c_key[i];
            for (int j = 0; j < n; ++j) larger += c_key[j] > mine ? c_mass[j] : 0ull;
            if (larger < remaining) lowest = min(lowest, mine);
          }
          lowest = ~block_max_u32(sh, ~lowest);
          if (threadIdx.x == 0) sh.bcast[0] = (unsigned long long)lowest;
        }
        cluster_barrier();  // the cut stands in the first CTA
        lo_key = (unsigned)ld_cluster_u64(in_cta(sm32(&sh.bcast[0]), 0));
        cluster_barrier();  // read by all
        cut_found = true;
      }
    }
  }

  // ---- the long way (a flat row, many equal values, or a large k): exact radix descents over the row
  if (by_count) {
    unsigned prefix = 0u;
    unsigned long long remaining = (unsigned long long)k;
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      const int dgt = radix_level<false>(sh, sl, T, mx, 0u, prefix, shift, remaining);
      prefix = (prefix << 8) | (unsigned)dgt;
    }
    lo_key = prefix;  // the k-th largest key
  }
  if (top_p < 1.f && !cut_found) {
    // mass of what top-k kept (of the whole row without top-k: the histogram by mass has it)
    unsigned long long s = row_mass;
    if (!have_all) {
      unsigned long long z = 0;
      for_each(sl, [&](int, float raw) {
        const float x = raw / T;
        if (ordered_key(x) >= lo_key) z += __float2ull_rz(expf(x - mx) * FIX_ONE);
      });
      s = cluster_sum_u64(sh, sl, block_sum_u64(sh, z));
    }
    unsigned long long remaining = (unsigned long long)ceil((double)top_p * (double)s);
    if (remaining < 1ull) remaining = 1ull;
    if (remaining > s) remaining = s;
    unsigned prefix = 0u;
    for (int level = 0; level < 4; ++level) {
      const int shift = 24 - 8 * level;
      const int dgt = radix_level<true>(sh, sl, T, mx, lo_key, prefix, shift, remaining);
      prefix = (prefix << 8) | (unsigned)dgt;
    }
    lo_key = prefix > lo_key ? prefix : lo_key;
  }

  // ---- draw: the inverse CDF in index order.  The row is cut into stretches of `bs` entries (at
  // most MAX_BLOCKS of them); stretch b belongs to CTA b % nranks, whose warps sum its kept mass;
  // every CTA then gathers all the sums and finds the stretch the target falls into; the first CTA
  // walks that stretch 32 entries at a time.
  const int bs = 1024 * ((V + 1024 * MAX_BLOCKS - 1) / (1024 * MAX_BLOCKS));
  const int nblk = (V + bs - 1) / bs;
  auto mass_at = [&](int i) -> unsigned long long {
    if (i >= V) return 0ull;
    const float x = row[i] / T;
    return ordered_key(x) >= lo_key ? __float2ull_rz(expf(x - mx) * FIX_ONE) : 0ull;
  };
  for (int b = (int)sl.rank + (int)sl.nranks * warp; b < nblk; b += (int)sl.nranks * NWARPS) {
    unsigned long long part = 0;
    for (int c0 = b * bs; c0 < (b + 1) * bs; c0 += 1024) {
#pragma unroll 8
      for (int j = 0; j < 32; ++j) part += mass_at(c0 + 32 * j + lane);
    }
    part = warp_sum_u64(part);
    if (lane == 0) sh.blk[b] = part;
  }
  cluster_barrier();  // every stretch's mass is with its owner
  for (int b = threadIdx.x; b < nblk; b += THREADS) {
    const uint32_t owner = (uint32_t)b % sl.nranks;
    if (owner != sl.rank) sh.blk[b] = ld_cluster_u64(in_cta(sm32(&sh.blk[b]), owner));
  }
  cluster_barrier();  // gathered (and nobody reads this CTA's shared memory after this)
  __syncthreads();
  if (threadIdx.x < 32) {
    unsigned long long total = 0;
    for (int b = threadIdx.x; b < nblk; b += 32) total += sh.blk[b];
    total = warp_sum_u64(total);
    const unsigned long long rnd = splitmix64(rand_keys ? rand_keys[r] : 0ull);
    const unsigned long long target = __umul64hi(rnd, total);  // uniform in [0, total)
    unsigned long long before = 0;
    int b_sel = warp_find<false>(nblk, [&](int i) { return sh.blk[i]; }, target, before);
    if (b_sel < 0) {  // (cannot happen: target < total)
      b_sel = nblk - 1;
      before = total - sh.blk[nblk - 1];
    }
    if (threadIdx.x == 0) {
      sh.bcast[0] = target - before;
      sh.bcast[1] = total;
      sh.bcast[2] = (unsigned long long)b_sel;
    }
  }
  __syncthreads();
  const int b_sel = (int)sh.bcast[2];
  const unsigned long long total = sh.bcast[1];
  if (sl.rank == 0) {
    // the chosen stretch, 1,024 entries at a time: every thread works out two masses (all reads in
    // flight at once), then one warp finds where the running mass passes what is left of the target
    unsigned long long* sel = &sh.hist[0][0];  // 1,024 entries (the histograms are done with)
    unsigned long long rem = sh.bcast[0];
    const int s_begin = b_sel * bs, s_end = min(V, s_begin + bs);
    int tok = -1;
    for (int c0 = s_begin; c0 < s_end && tok < 0; c0 += 1024) {
      __syncthreads();
      sel[threadIdx.x] = mass_at(c0 + threadIdx.x < s_end ? c0 + threadIdx.x : V);
      sel[threadIdx.x + THREADS] = mass_at(c0 + THREADS + threadIdx.x < s_end ? c0 + THREADS + threadIdx.x : V);
      __syncthreads();
      if (warp == 0) {
        unsigned long long before = 0;
        const int at = warp_find<false>(1024, [&](int i) { return sel[i]; }, rem, before);
        if (lane == 0) {
          unsigned long long chunk = 0;
          if (at < 0)
            for (int i = 0; i < 1024; ++i) chunk += sel[i];  // (only a stretch longer than 1,024 gets here)
          sh.bcast[0] = at >= 0 ? (unsigned long long)(c0 + at) : ~0ull;
          sh.bcast[1] = rem - chunk;
        }
      }
      __syncthreads();
      if (sh.bcast[0] != ~0ull) tok = (int)sh.bcast[0];
      rem = sh.bcast[1];
    }
    if (tok < 0) {  // (cannot happen: the target is below the stretch's mass) the last kept entry of the stretch
      for (int i = s_end - 1; i >= s_begin && tok < 0; --i)
        if (mass_at(i) > 0) tok = i;
      if (tok < 0) tok = 0;
    }
    if (threadIdx.x == 0) out_tokens[r] = tok;
  }
  if (prow) {
    const float inv = 1.f / (float)total;
    for (int i = sl.lo + threadIdx.x; i < sl.hi; i += THREADS) {
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
  // a cluster per row: as many CTAs (a power of two up to 8) as the row has stretches of 8,192 entries
  // ... as long as all the clusters fit the device at once (two CTAs per SM)
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  int c = 1;
  while (c < MAX_CLUSTER && (long long)c * 8192 < V && (long long)2 * c * R <= 2ll * sms) c <<= 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(c, R);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = c;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled ? 2 : 1;
  return (int)cudaLaunchKernelEx(&cfg, sample_kernel, logits, ld, V, temps, top_ks, top_ps, rand_keys, out_tokens, probs_out);
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
