// Embedding gather, residual-add + RMSNorm, rotary encoding + cache write, SiLU gate.
//
// The residual stream is held in float for both storage types, so the residual sum is a
// 32-bit sum; norms, rotation angles and the gate are computed in float and rounded once.
#include "common.cuh"

using namespace kvf;

// ---------------------------------------------------------------- embedding
// resid[n, :] = float(table[ids[n], :]).  An id outside the table writes zeros and raises
// the error flag (the host validates ids before; this only keeps a bad id from reading
// outside the table).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ resid, int H, int vocab, int* __restrict__ err) {
  const int n = blockIdx.x;
  const int id = ids[n];
  const bool ok = (id >= 0 && id < vocab);
  if (!ok && threadIdx.x == 0 && err) atomicOr(err, 1);
  const T* row = table + (size_t)(ok ? id : 0) * H;
  float* out = resid + (size_t)n * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) out[i] = ok ? to_float<T>(row[i]) : 0.f;
}

// ---------------------------------------------------------------- add + RMSNorm
// v = resid[src,:] (+ float(delta[src,:]) if delta) (+ sum over slices of partials[s][src,:]);
// src = rows ? rows[r] : r.  `partials` are the float slices a split-K product leaves.
// out[r,:] = T( v * rsqrt(mean(v^2) + eps) * weight[:] )
// Without `rows` the sum is written back to resid (the residual stream moves on); with
// `rows` (a gather of the wanted rows before the output head) resid is left untouched, so a
// row may be named twice.  One CTA per row; the reduction tree depends on H only.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                   const float* __restrict__ partials, int nsplit, size_t split_stride,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   const int* __restrict__ rows, int H, float eps) {
  __shared__ float red[32];
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* h = resid + (size_t)src * H;
  const T* dl = delta ? delta + (size_t)src * H : nullptr;
  const float* pt = partials ? partials + (size_t)src * H : nullptr;
  const bool pending = (dl != nullptr) || (pt != nullptr);
  const bool write_back = pending && (rows == nullptr);
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = h[i];
    if (dl) v += to_float<T>(dl[i]);
    if (pt) {
      float d = 0.f;
      for (int s = 0; s < nsplit; ++s) d += pt[(size_t)s * split_stride + i];  // slice order: reproducible
      v += d;
    }
    if (write_back) h[i] = v;
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* o = out + (size_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = h[i];
    if (pending && !write_back) {
      if (dl) v += to_float<T>(dl[i]);
      if (pt) {
        float d = 0.f;
        for (int s = 0; s < nsplit; ++s) d += pt[(size_t)s * split_stride + i];
        v += d;
      }
    }
    o[i] = from_float<T>(v * inv * weight[i]);
  }
}

// resid[r,:] += float(delta[r,:]) without a norm (used after the last layer when the
// final norm reads gathered rows).
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ resid, const T* __restrict__ delta, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) resid[i] += to_float<T>(delta[i]);
}

// ---------------------------------------------------------------- rotary + cache write
// qkv: [N, (nh + 2*nkv) * d] with q heads first, then k heads, then v heads.
// Rotates q in place, rotates k, and writes k and v of token n to its cache slot.
// Pair (j, j + rot/2) of the first `rot` dims turns by angle float(pos) * inv_freq[j];
// dims >= rot pass through.  Cache layout per layer: [num_blocks][nkv][block_size][d].
// slot < 0 means "do not write" (a call that reads another call's cache).
// The projections come from `qkv`, or (partials != nullptr) as the sum of the float slices of
// a split-K product; q then goes to `q_out` [N, nh*d].
template <typename T>
__global__ void rope_cache_kernel(T* __restrict__ qkv, const float* __restrict__ partials, int nsplit,
                                  size_t split_stride, T* __restrict__ q_out, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                  T* __restrict__ kcache, T* __restrict__ vcache, int nh, int nkv, int d,
                                  int rot, int block_size, long long num_slots, int* __restrict__ err) {
  const int n = blockIdx.x;
  const int half = rot >> 1;
  const int stride = (nh + 2 * nkv) * d;
  T* row = qkv ? qkv + (size_t)n * stride : nullptr;
  const float* prow = partials ? partials + (size_t)n * stride : nullptr;
  // element `idx` of this token's projections: from the bfloat16/float row, or the sum of the
  // float slices of a split-K product (in slice order)
  auto value = [&](int idx) -> float {
    if (prow) {
      float v = 0.f;
      for (int s = 0; s < nsplit; ++s) v += prow[(size_t)s * split_stride + idx];
      return v;
    }
    return to_float<T>(row[idx]);
  };
  T* qdst = q_out ? q_out + (size_t)n * nh * d : row;
  const float pos = (float)positions[n];
  long long slot = slots ? (long long)slots[n] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && err) atomicOr(err, 2);
    slot = -1;
  }
  const long long blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? (int)(slot % block_size) : 0;

  // q and k heads: one thread per (head, pair)
  const int rot_work = (nh + nkv) * half;
  for (int w = threadIdx.x; w < rot_work; w += blockDim.x) {
    const int head = w / half, j = w - head * half;
    float s, c;
    sincosf(pos * inv_freq[j], &s, &c);
    const float x1 = value(head * d + j), x2 = value(head * d + j + half);
    const T y1 = from_float<T>(x1 * c - x2 * s);
    const T y2 = from_float<T>(x2 * c + x1 * s);
    if (head < nh) {
      qdst[(size_t)head * d + j] = y1;
      qdst[(size_t)head * d + j + half] = y2;
    } else if (slot >= 0) {
      const int kvh = head - nh;
      T* dst = kcache + (((size_t)blk * nkv + kvh) * block_size + off) * d;
      dst[j] = y1;
      dst[j + half] = y2;
    }
  }
  // pass-through dims (partial rotation) of q when it moves to another buffer, and of k
  const int pass = d - rot;
  if (q_out)
    for (int w = threadIdx.x; w < nh * pass; w += blockDim.x) {
      const int head = w / pass, j = rot + (w - head * pass);
      qdst[(size_t)head * d + j] = from_float<T>(value(head * d + j));
    }
  if (slot < 0) return;
  for (int w = threadIdx.x; w < nkv * pass; w += blockDim.x) {
    const int kvh = w / pass, j = rot + (w - kvh * pass);
    kcache[(((size_t)blk * nkv + kvh) * block_size + off) * d + j] = from_float<T>(value((nh + kvh) * d + j));
  }
  for (int w = threadIdx.x; w < nkv * d; w += blockDim.x) {
    const int kvh = w / d, j = w - kvh * d;
    vcache[(((size_t)blk * nkv + kvh) * block_size + off) * d + j] = from_float<T>(value((nh + nkv + kvh) * d + j));
  }
}

// ---------------------------------------------------------------- SiLU gate
// out[n, i] = T( silu(float(g_i)) * float(u_i) ),  silu(t) = t / (1 + exp(-t)).
// Columns of gu [N, 2I]: gates then ups (block == 0), or alternating in blocks of `block`
// ([g0..b-1, u0..b-1, gb.., ...]), the order the decode product wants its weight rows in.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int block, size_t total) {
  size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t n = idx / I;
  const int i = (int)(idx - n * I);
  const int cg = block ? (i / block) * 2 * block + (i % block) : i;
  const int cu = block ? cg + block : I + i;
  const float g = to_float<T>(gu[n * 2 * (size_t)I + cg]);
  const float u = to_float<T>(gu[n * 2 * (size_t)I + cu]);
  out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
}

// ---------------------------------------------------------------- cast
// float -> T rows (used when a float tensor feeds a T-typed product).
template <typename T>
__global__ void cast_from_float_kernel(const float* __restrict__ in, T* __restrict__ out, size_t n) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_float<T>(in[i]);
}

static inline int norm_threads(int H) {
  int t = 32;
  while (t < 1024 && t * 4 < H) t <<= 1;
  return t;
}

#define KVF_ELEMENTWISE_API(SUF, T)                                                                      \
  KVF_API int kvf_embed_##SUF(const void* table, const int* ids, float* resid, int N, int H, int vocab,  \
                              int* err, cudaStream_t st) {                                               \
    if (N <= 0) return 0;                                                                                \
    embed_kernel<T><<<N, 256, 0, st>>>((const T*)table, ids, resid, H, vocab, err);                      \
    return KVF_LAUNCH_STATUS();                                                                          \
  }                                                                                                      \
  KVF_API int kvf_add_rmsnorm_##SUF(float* resid, const void* delta, const float* partials, int nsplit, \
                                    long long split_stride, const float* weight, void* out,              \
                                    const int* rows, int n_rows, int H, float eps, cudaStream_t st) {    \
    if (n_rows <= 0) return 0;                                                                           \
    add_rmsnorm_kernel<T><<<n_rows, norm_threads(H), 0, st>>>(resid, (const T*)delta, partials, nsplit,  \
                                                              (size_t)split_stride, weight, (T*)out,     \
                                                              rows, H, eps);                             \
    return KVF_LAUNCH_STATUS();                                                                          \
  }                                                                                                      \
  KVF_API int kvf_add_residual_##SUF(float* resid, const void* delta, long long n, cudaStream_t st) {    \
    if (n <= 0) return 0;                                                                                \
    add_residual_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(resid, (const T*)delta, (size_t)n); \
    return KVF_LAUNCH_STATUS();                                                                          \
  }                                                                                                      \
  KVF_API int kvf_rope_cache_##SUF(void* qkv, const float* partials, int nsplit, long long split_stride, \
                                   void* q_out, const int* positions, const float* inv_freq,             \
                                   const int* slots, void* kcache, void* vcache, int N, int nh, int nkv, \
                                   int d, int rot, int block_size, long long num_slots, int* err,        \
                                   cudaStream_t st) {                                                    \
    if (N <= 0) return 0;                                                                                \
    if (rot < 0 || rot > d || (rot & 1)) return (int)cudaErrorInvalidValue;                              \
    if (!qkv && !(partials && q_out)) return (int)cudaErrorInvalidValue;                                 \
    rope_cache_kernel<T><<<N, 256, 0, st>>>((T*)qkv, partials, nsplit, (size_t)split_stride, (T*)q_out,  \
                                            positions, inv_freq, slots, (T*)kcache, (T*)vcache, nh, nkv, \
                                            d, rot, block_size, num_slots, err);                         \
    return KVF_LAUNCH_STATUS();                                                                          \
  }                                                                                                      \
  KVF_API int kvf_silu_mul_##SUF(const void* gu, void* out, long long N, int I, int block,               \
                                 cudaStream_t st) {                                                      \
    const size_t total = (size_t)N * I;                                                                  \
    if (total == 0) return 0;                                                                            \
    if (block < 0 || (block && I % block)) return (int)cudaErrorInvalidValue;                            \
    silu_mul_kernel<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const T*)gu, (T*)out, I, block, \
                                                                        total);                          \
    return KVF_LAUNCH_STATUS();                                                                          \
  }                                                                                                      \
  KVF_API int kvf_cast_from_float_##SUF(const float* in, void* out, long long n, cudaStream_t st) {      \
    if (n <= 0) return 0;                                                                                \
    cast_from_float_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(in, (T*)out, (size_t)n);      \
    return KVF_LAUNCH_STATUS();                                                                          \
  }

KVF_ELEMENTWISE_API(f32, float)
KVF_ELEMENTWISE_API(bf16, bf16)
