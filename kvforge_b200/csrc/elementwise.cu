// Embedding gather, residual-add + RMSNorm, rotary encoding + cache write, SiLU gate.
//
// The residual stream is held in float for both storage types, so the residual sum is a
// 32-bit sum; norms, rotation angles and the gate are computed in float and rounded once.
#include "common.cuh"

using namespace kvf;

// ---------------------------------------------------------------- embedding
// resid[n, :] = float(table[id, :]) with id = ids[n], or, where feedback_rows[n] >= 0, the
// token that the sampling kernel of the step before left at feedback[feedback_rows[n]] (so a
// decoded token goes round on the device and the host need not have read it yet).  An id
// outside the table writes zeros and raises the error flag (the host validates ids before;
// this only keeps a bad id from reading outside the table).
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             const int* __restrict__ feedback_rows, const int* __restrict__ feedback,
                             float* __restrict__ resid, int H, int vocab, int* __restrict__ err) {
  pdl_launch();
  pdl_wait();
  const int n = blockIdx.x;
  int id = ids[n];
  if (feedback_rows && feedback_rows[n] >= 0) id = feedback[feedback_rows[n]];
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
  pdl_launch();
  pdl_wait();
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

// The same for H % 4 == 0: 16-byte loads, the slices of a split product loaded side by side,
// and the summed row kept in shared memory so that global memory is read once.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
  static __device__ __forceinline__ float4 load(const bf16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
    return make_float4(a.x, a.y, b.x, b.y);
  }
  static __device__ __forceinline__ void store(bf16* p, float4 v) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&a);
    u.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = u;
  }
};

template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                       const float* __restrict__ partials, int nsplit, size_t split_stride,
                                       const float* __restrict__ weight, T* __restrict__ out,
                                       const int* __restrict__ rows, int H, float eps) {
  pdl_launch();
  extern __shared__ __align__(16) float rowbuf[];  // H floats
  __shared__ float red[32];
  const int r = blockIdx.x;
  // the norm's weight does not come from the kernel ahead: a thread's first four are fetched before the wait
  const int i0 = threadIdx.x * 4;
  const float4 w0 = i0 < H ? *reinterpret_cast<const float4*>(weight + i0) : make_float4(0.f, 0.f, 0.f, 0.f);
  const int src = rows ? rows[r] : r;
  pdl_wait();
  float* h = resid + (size_t)src * H;
  const T* dl = delta ? delta + (size_t)src * H : nullptr;
  const float* pt = partials ? partials + (size_t)src * H : nullptr;
  const bool write_back = ((dl != nullptr) || (pt != nullptr)) && (rows == nullptr);
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    float4 v = *reinterpret_cast<const float4*>(h + i);
    if (dl) {
      const float4 d = Vec4<T>::load(dl + i);
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    }
    if (pt) {
      float4 d = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
      for (int s = 0; s < nsplit; ++s) {  // slice order: reproducible
        const float4 q = *reinterpret_cast<const float4*>(pt + (size_t)s * split_stride + i);
        d.x += q.x; d.y += q.y; d.z += q.z; d.w += q.w;
      }
      v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
    }
    if (write_back) *reinterpret_cast<float4*>(h + i) = v;
    *reinterpret_cast<float4*>(rowbuf + i) = v;
    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  T* o = out + (size_t)r * H;
  for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
    const float4 v = *reinterpret_cast<const float4*>(rowbuf + i);
    const float4 w = i == i0 ? w0 : *reinterpret_cast<const float4*>(weight + i);
    Vec4<T>::store(o + i, make_float4(v.x * inv * w.x, v.y * inv * w.y, v.z * inv * w.z, v.w * inv * w.w));
  }
}

// Without slices of a split product, for H % 4 == 0 and H <= 512 * VPT: a CTA of 128 threads per
// row, the row in registers (VPT 16-byte loads per thread, all in flight at once, the norm's
// weight among them since it does not wait for the sum), one reduction over four warps.  Small
// CTAs with few registers: sixteen rows are on an SM at a time, which is what keeps the memory
// pipe full when there are thousands of rows (2,048 rows of 4,096: 6.4 us; a row per warp, with
// its row in 128 registers, took 21 us, a row per CTA of 1,024 threads 22 us), and it is no
// slower than those on a handful of rows.  The reduction tree depends on H alone.
template <typename T, int VPT>
__global__ void __launch_bounds__(128) add_rmsnorm_rows_kernel(float* __restrict__ resid, const T* __restrict__ delta,
                                                               const float* __restrict__ weight, T* __restrict__ out,
                                                               const int* __restrict__ rows, int H, float eps) {
  pdl_launch();
  __shared__ float red[32];
  const int r = blockIdx.x;
  float4 w[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {  // the weight comes from no kernel ahead: fetched before the wait
    const int i = (k * 128 + threadIdx.x) * 4;
    w[k] = i < H ? *reinterpret_cast<const float4*>(weight + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  const int src = rows ? rows[r] : r;
  pdl_wait();
  float* h = resid + (size_t)src * H;
  const T* dl = delta ? delta + (size_t)src * H : nullptr;
  float4 v[VPT];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = (k * 128 + threadIdx.x) * 4;
    v[k] = i < H ? *reinterpret_cast<const float4*>(h + i) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (dl) {
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int i = (k * 128 + threadIdx.x) * 4;
      if (i < H) {
        const float4 d = Vec4<T>::load(dl + i);
        v[k].x += d.x; v[k].y += d.y; v[k].z += d.z; v[k].w += d.w;
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) ss += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
  ss = block_sum(ss, red);
  const float inv = rsqrtf(ss / (float)H + eps);
  const bool write_back = dl != nullptr && rows == nullptr;
  T* o = out + (size_t)r * H;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = (k * 128 + threadIdx.x) * 4;
    if (i < H) {
      if (write_back) *reinterpret_cast<float4*>(h + i) = v[k];
      Vec4<T>::store(o + i, make_float4(v[k].x * inv * w[k].x, v[k].y * inv * w[k].y, v[k].z * inv * w[k].z, v[k].w * inv * w[k].w));
    }
  }
}

// resid[r,:] += float(delta[r,:]) without a norm (used after the last layer when the
// final norm reads gathered rows).
template <typename T>
__global__ void add_residual_kernel(float* __restrict__ resid, const T* __restrict__ delta, size_t n) {
  pdl_launch();
  pdl_wait();
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
  pdl_launch();
  pdl_wait();
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
    float r1, r2;
    rotate_pair(x1, x2, c, s, r1, r2);
    const T y1 = from_float<T>(r1);
    const T y2 = from_float<T>(r2);
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

// The same with one thread per (head, pair): grid (tokens, groups of heads), so that a few
// tokens still spread over many SMs, and the slices of a split product loaded side by side.
// Needs rot == d (the whole head turns) and an even d.
template <typename T>
__global__ void rope_cache_heads_kernel(T* __restrict__ qkv, const float* __restrict__ partials, int nsplit,
                                        size_t split_stride, T* __restrict__ q_out,
                                        const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                        const int* __restrict__ slots, T* __restrict__ kcache,
                                        T* __restrict__ vcache, int nh, int nkv, int d, int block_size,
                                        long long num_slots, int heads_per_cta, int* __restrict__ err) {
  pdl_launch();
  const int n = blockIdx.x;
  const int half = d >> 1;
  const int total_heads = nh + 2 * nkv;
  const int stride = total_heads * d;
  const int head = blockIdx.y * heads_per_cta + threadIdx.x / half;
  const int j = threadIdx.x % half;
  const bool mine = threadIdx.x < heads_per_cta * half && head < total_heads;
  // positions, slots and frequencies come with the step, not from the kernel ahead: the angle is
  // worked out before the wait
  float sn = 0.f, cs = 1.f;
  long long slot = -1;
  if (mine) {
    if (head < nh + nkv) sincosf((float)positions[n] * inv_freq[j], &sn, &cs);
    slot = slots ? (long long)slots[n] : -1;
  }
  pdl_wait();
  if (!mine) return;
  T* row = qkv ? qkv + (size_t)n * stride : nullptr;
  const float* prow = partials ? partials + (size_t)n * stride : nullptr;
  const int i1 = head * d + j, i2 = i1 + half;
  float x1, x2;
  if (prow) {
    x1 = x2 = 0.f;
#pragma unroll 8
    for (int s = 0; s < nsplit; ++s) {  // slice order: reproducible
      x1 += prow[(size_t)s * split_stride + i1];
      x2 += prow[(size_t)s * split_stride + i2];
    }
  } else {
    x1 = to_float<T>(row[i1]);
    x2 = to_float<T>(row[i2]);
  }
  if (slot >= num_slots) {
    if (j == 0 && err) atomicOr(err, 2);
    slot = -1;
  }
  T y1, y2;
  if (head < nh + nkv) {
    float r1, r2;
    rotate_pair(x1, x2, cs, sn, r1, r2);
    y1 = from_float<T>(r1);
    y2 = from_float<T>(r2);
  } else {
    y1 = from_float<T>(x1);
    y2 = from_float<T>(x2);
  }
  if (head < nh) {
    T* qdst = q_out ? q_out + (size_t)n * nh * d : row;
    qdst[(size_t)head * d + j] = y1;
    qdst[(size_t)head * d + j + half] = y2;
  } else if (slot >= 0) {
    const bool is_k = head < nh + nkv;
    const int kvh = is_k ? head - nh : head - nh - nkv;
    T* dst = (is_k ? kcache : vcache) + (((size_t)(slot / block_size) * nkv + kvh) * block_size + (slot % block_size)) * d;
    dst[j] = y1;
    dst[j + half] = y2;
  }
}

// The same again for many tokens: one CTA per token, each thread moves 8 consecutive dims of a
// head (16-byte loads and stores for bfloat16) together with the 8 dims half a head further on
// that they pair with.  Needs rot == d and d % 16 == 0.
template <typename T> struct Ld8;
template <> struct Ld8<bf16> {
  static __device__ __forceinline__ void load(const bf16* p, float* f) { bf16x8_to_float(*reinterpret_cast<const uint4*>(p), f); }
  static __device__ __forceinline__ void store(bf16* p, const float* f) {
    uint4 u;
    uint32_t* w = reinterpret_cast<uint32_t*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 v = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&v);
    }
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Ld8<float> {
  static __device__ __forceinline__ void load(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
  }
};

template <typename T>
__global__ void rope_cache_vec_kernel(T* __restrict__ qkv, const float* __restrict__ partials, int nsplit,
                                      size_t split_stride, T* __restrict__ q_out,
                                      const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                      const int* __restrict__ slots, T* __restrict__ kcache,
                                      T* __restrict__ vcache, int nh, int nkv, int d, int block_size,
                                      long long num_slots, int* __restrict__ err) {
  pdl_launch();
  extern __shared__ __align__(16) float cs_sn[];  // cos then sin of this token's d/2 angles
  const int n = blockIdx.x;
  const int half = d >> 1, cph = half >> 3;  // chunks of 8 pairs per head
  {
    // the angles depend on the position alone: once per token, not once per head
    const float pos0 = (float)positions[n];
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos0 * inv_freq[j], &cs_sn[half + j], &cs_sn[j]);
  }
  pdl_wait();
  __syncthreads();
  const int stride = (nh + 2 * nkv) * d;
  T* row = qkv ? qkv + (size_t)n * stride : nullptr;
  const float* prow = partials ? partials + (size_t)n * stride : nullptr;
  auto load8 = [&](int idx, float* f) {
    if (prow) {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
      for (int s = 0; s < nsplit; ++s) {  // slice order: reproducible
        float g[8];
        Ld8<float>::load(prow + (size_t)s * split_stride + idx, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] += g[e];
      }
    } else {
      Ld8<T>::load(row + idx, f);
    }
  };
  long long slot = slots ? (long long)slots[n] : -1;
  if (slot >= num_slots) {
    if (threadIdx.x == 0 && err) atomicOr(err, 2);
    slot = -1;
  }
  const size_t cache_row = slot >= 0 ? ((size_t)(slot / block_size) * nkv) * block_size + (slot % block_size) : 0;
  T* qdst = q_out ? q_out + (size_t)n * nh * d : row;
  // One pass over two kinds of items, so that a token's values are on their way while its heads
  // turn: rotated heads (q then k), one item = 8 pairs of one head; then values, plain copies of
  // 8 dims per item.  (CTAs of 128 threads from 512 tokens on: with 256 the 2,048-token prompt step of the 1B shape takes 4.09 instead of
  // 4.05 ms, the 8B shape's 24.1 instead of 23.7 ms.  Two items in flight per thread were no faster.)
  const int rot_items = (nh + nkv) * cph;
  const int v_chunks = d >> 3;
  const int v_items = slot >= 0 ? nkv * v_chunks : 0;
  for (int w = threadIdx.x; w < rot_items + v_items; w += blockDim.x) {
    if (w < rot_items) {
      const int head = w / cph, j0 = (w - head * cph) << 3;
      float x1[8], x2[8], y1[8], y2[8];
      load8(head * d + j0, x1);
      load8(head * d + half + j0, x2);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float cs = cs_sn[j0 + e], sn = cs_sn[half + j0 + e];
        rotate_pair(x1[e], x2[e], cs, sn, y1[e], y2[e]);
      }
      T* dst = nullptr;
      if (head < nh) {
        dst = qdst + (size_t)head * d;
      } else if (slot >= 0) {
        dst = kcache + (cache_row + (size_t)(head - nh) * block_size) * d;
      }
      if (dst) {
        Ld8<T>::store(dst + j0, y1);
        Ld8<T>::store(dst + half + j0, y2);
      }
    } else {
      const int v = w - rot_items;
      const int kvh = v / v_chunks, j0 = (v - kvh * v_chunks) << 3;
      float f[8];
      load8((nh + nkv + kvh) * d + j0, f);
      Ld8<T>::store(vcache + (cache_row + (size_t)kvh * block_size) * d + j0, f);
    }
  }
}

// ---------------------------------------------------------------- SiLU gate
// out[n, i] = T( silu(float(g_i)) * float(u_i) ),  silu(t) = t / (1 + exp(-t)).
// Columns of gu [N, 2I]: gates then ups (block == 0), or alternating in blocks of `block`
// ([g0..b-1, u0..b-1, gb.., ...]), the order the decode product wants its weight rows in.
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int I, int block, size_t total) {
  pdl_launch();
  pdl_wait();
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

// The same, 8 bfloat16 outputs (one 16-byte load of gates, one of ups, one 16-byte store) per
// thread; needs I % 8 == 0, which the interleaved layout (blocks of 8) has by construction.
__global__ void silu_mul_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int I, int block,
                                       size_t groups) {
  pdl_launch();
  pdl_wait();
  const size_t gidx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gidx >= groups) return;
  const int per_row = I >> 3;
  const size_t n = gidx / per_row;
  const int i0 = (int)(gidx - n * per_row) << 3;
  const int cg = block ? (i0 / block) * 2 * block + (i0 % block) : i0;
  const int cu = block ? cg + block : I + i0;
  const bf16* row = gu + n * 2 * (size_t)I;
  const uint4 gv = *reinterpret_cast<const uint4*>(row + cg);
  const uint4 uv = *reinterpret_cast<const uint4*>(row + cu);
  float g[8], u[8];
  bf16x8_to_float(gv, g);
  bf16x8_to_float(uv, u);
  uint4 o;
  uint32_t* op = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    const float a = g[2 * e] / (1.f + expf(-g[2 * e])) * u[2 * e];
    const float b = g[2 * e + 1] / (1.f + expf(-g[2 * e + 1])) * u[2 * e + 1];
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    op[e] = *reinterpret_cast<uint32_t*>(&v);
  }
  *reinterpret_cast<uint4*>(out + n * (size_t)I + i0) = o;
}

template <typename T>
int launch_silu_mul(const void* gu, void* out, long long N, int I, int block, cudaStream_t st) {
  const size_t total = (size_t)N * I;
  return launch(silu_mul_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, (const T*)gu, (T*)out, I, block, total);
}
template <>
int launch_silu_mul<bf16>(const void* gu, void* out, long long N, int I, int block, cudaStream_t st) {
  const size_t total = (size_t)N * I;
  const bool aligned = ((((uintptr_t)gu) | ((uintptr_t)out)) & 15) == 0;
  if ((I & 7) == 0 && (block == 0 || block == 8) && aligned) {
    const size_t groups = total >> 3;
    return launch(silu_mul_bf16x8_kernel, dim3((unsigned)((groups + 255) / 256)), dim3(256), 0, st, (const bf16*)gu,
                  (bf16*)out, I, block, groups);
  }
  return launch(silu_mul_kernel<bf16>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, st, (const bf16*)gu,
                (bf16*)out, I, block, total);
}

// ---------------------------------------------------------------- cast
// float -> T rows (used when a float tensor feeds a T-typed product).
template <typename T>
__global__ void cast_from_float_kernel(const float* __restrict__ in, T* __restrict__ out, size_t n) {
  pdl_launch();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = from_float<T>(in[i]);
}

static inline int norm_threads(int H) {
  int t = 32;
  while (t < 1024 && t * 4 < H) t <<= 1;
  return t;
}

#define KVF_ELEMENTWISE_API(SUF, T)                                                                      \
  KVF_API int kvf_embed_##SUF(const void* table, const int* ids, const int* feedback_rows,               \
                              const int* feedback, float* resid, int N, int H, int vocab, int* err,      \
                              cudaStream_t st) {                                                         \
    if (N <= 0) return 0;                                                                                \
    return launch(embed_kernel<T>, dim3(N), dim3(256), 0, st, (const T*)table, ids, feedback_rows,       \
                  feedback, resid, H, vocab, err);                                                       \
  }                                                                                                      \
  KVF_API int kvf_add_rmsnorm_##SUF(float* resid, const void* delta, const float* partials, int nsplit, \
                                    long long split_stride, const float* weight, void* out,              \
                                    const int* rows, int n_rows, int H, float eps, cudaStream_t st) {    \
    if (n_rows <= 0) return 0;                                                                           \
    if ((H & 3) == 0 && H <= 4096 && !partials) {                                                        \
      const dim3 g(n_rows), b(128);                                                                      \
      if (H <= 512)                                                                                      \
        return launch(add_rmsnorm_rows_kernel<T, 1>, g, b, 0, st, resid, (const T*)delta, weight,        \
                      (T*)out, rows, H, eps);                                                            \
      if (H <= 1024)                                                                                     \
        return launch(add_rmsnorm_rows_kernel<T, 2>, g, b, 0, st, resid, (const T*)delta, weight,        \
                      (T*)out, rows, H, eps);                                                            \
      if (H <= 2048)                                                                                     \
        return launch(add_rmsnorm_rows_kernel<T, 4>, g, b, 0, st, resid, (const T*)delta, weight,        \
                      (T*)out, rows, H, eps);                                                            \
      return launch(add_rmsnorm_rows_kernel<T, 8>, g, b, 0, st, resid, (const T*)delta, weight,          \
                    (T*)out, rows, H, eps);                                                              \
    }                                                                                                    \
    if ((H & 3) == 0 && H <= 32768 && (split_stride & 3) == 0) {                                         \
      int t = 32;                                                                                        \
      while (t < 1024 && t * 4 < H) t <<= 1;                                                             \
      const size_t smem = (size_t)H * sizeof(float);                                                     \
      if (smem > 48 * 1024) {                                                                            \
        cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_vec_kernel<T>,                                  \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
        if (e != cudaSuccess) return (int)e;                                                             \
      }                                                                                                  \
      return launch(add_rmsnorm_vec_kernel<T>, dim3(n_rows), dim3(t), smem, st, resid, (const T*)delta,   \
                    partials, nsplit, (size_t)split_stride, weight, (T*)out, rows, H, eps);              \
    }                                                                                                    \
    return launch(add_rmsnorm_kernel<T>, dim3(n_rows), dim3(norm_threads(H)), 0, st, resid,              \
                  (const T*)delta, partials, nsplit, (size_t)split_stride, weight, (T*)out, rows, H,     \
                  eps);                                                                                  \
  }                                                                                                      \
  KVF_API int kvf_add_residual_##SUF(float* resid, const void* delta, long long n, cudaStream_t st) {    \
    if (n <= 0) return 0;                                                                                \
    return launch(add_residual_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, resid,    \
                  (const T*)delta, (size_t)n);                                                           \
  }                                                                                                      \
  KVF_API int kvf_rope_cache_##SUF(void* qkv, const float* partials, int nsplit, long long split_stride, \
                                   void* q_out, const int* positions, const float* inv_freq,             \
                                   const int* slots, void* kcache, void* vcache, int N, int nh, int nkv, \
                                   int d, int rot, int block_size, long long num_slots, int* err,        \
                                   cudaStream_t st) {                                                    \
    if (N <= 0) return 0;                                                                                \
    if (rot < 0 || rot > d || (rot & 1)) return (int)cudaErrorInvalidValue;                              \
    if (!qkv && !(partials && q_out)) return (int)cudaErrorInvalidValue;                                 \
    if (rot == d && (d & 15) == 0 && N > 16 && (split_stride & 3) == 0) {                                \
      /* a CTA per token: small CTAs when the tokens fill the SMs several times over, larger ones for a few dozen */ \
      return launch(rope_cache_vec_kernel<T>, dim3(N), dim3(N >= 512 ? 128 : 256), (size_t)d * sizeof(float), st, (T*)qkv, partials, nsplit, \
                    (size_t)split_stride, (T*)q_out, positions, inv_freq, slots, (T*)kcache, (T*)vcache, \
                    nh, nkv, d, block_size, num_slots, err);                                             \
    }                                                                                                    \
    if (rot == d && d >= 2 && d <= 512) {                                                                \
      const int half = d / 2;                                                                            \
      int hpc = 128 / half;                                                                              \
      if (hpc < 1) hpc = 1;                                                                              \
      const int heads = nh + 2 * nkv;                                                                    \
      dim3 grid(N, (heads + hpc - 1) / hpc);                                                             \
      if (grid.y <= 65535u) {                                                                            \
        return launch(rope_cache_heads_kernel<T>, grid, dim3(hpc * half), 0, st, (T*)qkv, partials,      \
                      nsplit, (size_t)split_stride, (T*)q_out, positions, inv_freq, slots, (T*)kcache,   \
                      (T*)vcache, nh, nkv, d, block_size, num_slots, hpc, err);                          \
      }                                                                                                  \
    }                                                                                                    \
    return launch(rope_cache_kernel<T>, dim3(N), dim3(256), 0, st, (T*)qkv, partials, nsplit,            \
                  (size_t)split_stride, (T*)q_out, positions, inv_freq, slots, (T*)kcache, (T*)vcache,   \
                  nh, nkv, d, rot, block_size, num_slots, err);                                          \
  }                                                                                                      \
  KVF_API int kvf_silu_mul_##SUF(const void* gu, void* out, long long N, int I, int block,               \
                                 cudaStream_t st) {                                                      \
    const size_t total = (size_t)N * I;                                                                  \
    if (total == 0) return 0;                                                                            \
    if (block < 0 || (block && I % block)) return (int)cudaErrorInvalidValue;                            \
    return launch_silu_mul<T>(gu, out, N, I, block, st);                                                 \
  }                                                                                                      \
  KVF_API int kvf_cast_from_float_##SUF(const float* in, void* out, long long n, cudaStream_t st) {      \
    if (n <= 0) return 0;                                                                                \
    return launch(cast_from_float_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, in,    \
                  (T*)out, (size_t)n);                                                                   \
  }

// Turn programmatic dependent launch on or off for every launch of this library.
KVF_API int kvf_set_pdl(int enabled) {
  kvf::g_pdl_enabled = enabled ? 1 : 0;
  return 0;
}

KVF_ELEMENTWISE_API(f32, float)
KVF_ELEMENTWISE_API(bf16, bf16)
