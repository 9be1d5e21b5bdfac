// Paged grouped-query attention over block tables on the FP32 pipes, for any head size
// (a multiple of 8, at most 256), any number of heads and groups, and any mix of
// query lengths in one flat batch.  This is the attention of the true 32-bit path and
// the fall-back of the bfloat16 path for head sizes that have no tensor-core kernel.
//
// Contract (what every attention kernel of this engine computes): sequence b has
// ctx_b keys in its pages after this step's writes and q_b = qsl[b+1]-qsl[b] queries;
// query i sits at position p = ctx_b - q_b + i and sees key j iff j <= p (and
// j > p - window when window > 0).  S = scale * (q . k) in float, softmax in float,
// O = P V in float, one rounding to T.
//
// Exactness: keys are walked in tiles of 32 that start at absolute positions (multiples
// of 32), each score is one thread's sequential dot product, and a fully masked tile
// leaves a row's state untouched.  So the result for a query does not depend on how the
// prompt was cut, on the other rows of its tile, or on the physical pages.
//
// Cache layout per layer: K and V each [num_blocks][nkv][block_size][d].
#include "common.cuh"

using namespace kvf;

namespace {

constexpr int TK = 32;        // keys per tile = one per lane
constexpr int WARPS = 4;      // warps per CTA
constexpr int RPW = 4;        // query rows per warp
constexpr int ROWS = WARPS * RPW;

struct AttnParams {
  const void* q;
  void* out;
  const void* kcache;
  const void* vcache;
  const int* block_tables;
  const int* qsl;
  const int* ctx_lens;
  float* part_acc;  // split mode: [B][nh][splits][d]
  float* part_ml;   // split mode: [B][nh][splits][2]
  int q_stride, out_stride, bt_stride;
  int nh, nkv, d, block_size;
  int gh, chunks, tq;  // heads per CTA, head chunks per kv head, tokens per CTA
  int window;
  int split_size, max_splits;
  float scale;
};

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<bf16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void load_vec_to_float(const T* src, float* dst);
template <>
__device__ __forceinline__ void load_vec_to_float<float>(const float* src, float* dst) {
  const float4 v = *reinterpret_cast<const float4*>(src);
  dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
template <>
__device__ __forceinline__ void load_vec_to_float<bf16>(const bf16* src, float* dst) {
  const uint4 v = *reinterpret_cast<const uint4*>(src);
  bf16x8_to_float(v, dst);
}

// DPL = output dims per lane = ceil(d / 32).  SPLIT: every sequence has one query and
// grid.x walks key ranges of split_size; partial (m, l, acc) go to scratch.
template <typename T, int DPL, bool SPLIT>
__global__ void __launch_bounds__(WARPS * 32) paged_attn_generic_kernel(const AttnParams p) {
  extern __shared__ __align__(16) float smem[];
  const int d = p.d, ldk = d + 4;
  float* Ks = smem;                    // [TK][ldk]
  float* Vs = Ks + TK * ldk;           // [TK][ldk]
  float* Qs = Vs + TK * ldk;           // [ROWS][d]
  float* Ps = Qs + ROWS * d;           // [WARPS][RPW][TK]

  const int b = blockIdx.y;
  const int kvh = blockIdx.z / p.chunks, chunk = blockIdx.z - kvh * p.chunks;
  const int g = p.nh / p.nkv;
  const int q_begin = p.qsl[b], q_len = p.qsl[b + 1] - q_begin;
  const int ctx = p.ctx_lens[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (q_len <= 0 || ctx <= 0) return;

  int q0, kv_lo, kv_hi;  // first query token of this CTA; key range [kv_lo, kv_hi)
  if (SPLIT) {
    q0 = q_len - 1;  // one query per sequence (the last, if a caller passes more)
    kv_lo = blockIdx.x * p.split_size;
    if (kv_lo >= ctx) return;  // a range past the context: the merge never reads it
    kv_hi = min(ctx, kv_lo + p.split_size);
    if (p.window > 0) kv_lo = max(kv_lo, ((max(0, ctx - p.window)) / TK) * TK);
    if (kv_lo >= kv_hi) {
      // a range that lies wholly before the window is empty, and says so to the merge
      for (int r = threadIdx.x; r < p.gh; r += blockDim.x) {
        const int head = kvh * g + chunk * p.gh + r;
        if (head < (kvh + 1) * g) {
          float* ml = p.part_ml + (((size_t)b * p.nh + head) * p.max_splits + blockIdx.x) * 2;
          ml[0] = -INFINITY;
          ml[1] = 0.f;
        }
      }
      return;
    }
  } else {
    q0 = blockIdx.x * p.tq;
    if (q0 >= q_len) return;
    const int p_first = ctx - q_len + q0;
    const int p_last = ctx - q_len + min(q0 + p.tq, q_len) - 1;
    kv_lo = 0;
    if (p.window > 0) kv_lo = (max(0, p_first - p.window + 1) / TK) * TK;
    kv_hi = p_last + 1;
  }
  const int n_tok = SPLIT ? 1 : min(p.tq, q_len - q0);

  // ---- stage the query rows as float.  Row r -> (token r / gh, head r % gh).
  const T* qg = (const T*)p.q;
  for (int idx = threadIdx.x; idx < ROWS * d; idx += blockDim.x) {
    const int r = idx / d, j = idx - r * d;
    const int tok = r / p.gh, hh = chunk * p.gh + (r - tok * p.gh);
    float v = 0.f;
    if (tok < n_tok && hh < g)
      v = to_float<T>(qg[(size_t)(q_begin + q0 + tok) * p.q_stride + (size_t)(kvh * g + hh) * d + j]);
    Qs[idx] = v;
  }

  // per-row state; row of (warp, slot i) is r = i * WARPS + warp
  float m[RPW], l[RPW], acc[RPW][DPL];
  int pos[RPW];
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    const int r = i * WARPS + warp;
    const int tok = r / p.gh, hh = chunk * p.gh + (r - tok * p.gh);
    const bool valid = (tok < n_tok) && (hh < g);
    pos[i] = valid ? (ctx - q_len + q0 + tok) : -1;  // -1: sees nothing
    m[i] = -INFINITY;
    l[i] = 0.f;
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[i][e] = 0.f;
  }

  const T* kc = (const T*)p.kcache;
  const T* vc = (const T*)p.vcache;
  const int* bt = p.block_tables + (size_t)b * p.bt_stride;
  constexpr int VN = Vec<T>::N;
  const int vec_per_row = d / VN;

  for (int t0 = kv_lo; t0 < kv_hi; t0 += TK) {
    __syncthreads();  // previous tile consumed (and Qs staged, first time)
    // ---- load the K and V tile as float; keys >= ctx and released pages are zero-filled
    for (int idx = threadIdx.x; idx < TK * vec_per_row; idx += blockDim.x) {
      const int key = idx / vec_per_row, c = (idx - key * vec_per_row) * VN;
      const int kp = t0 + key;
      float kf[VN], vf[VN];
      const int blk = kp < ctx ? bt[kp / p.block_size] : -1;
      if (blk >= 0) {  // a page given back (-1) lies wholly outside every window: zeros
        const int off = kp % p.block_size;
        const size_t base = (((size_t)blk * p.nkv + kvh) * p.block_size + off) * d + c;
        load_vec_to_float<T>(kc + base, kf);
        load_vec_to_float<T>(vc + base, vf);
      } else {
#pragma unroll
        for (int e = 0; e < VN; ++e) kf[e] = vf[e] = 0.f;
      }
#pragma unroll
      for (int e = 0; e < VN; ++e) {
        Ks[key * ldk + c + e] = kf[e];
        Vs[key * ldk + c + e] = vf[e];
      }
    }
    __syncthreads();

    // ---- scores: lane = key, RPW rows at once
    float s[RPW];
#pragma unroll
    for (int i = 0; i < RPW; ++i) s[i] = 0.f;
    const float* krow = Ks + lane * ldk;
    for (int c = 0; c < d; c += 4) {
      const float4 kv4 = *reinterpret_cast<const float4*>(krow + c);
#pragma unroll
      for (int i = 0; i < RPW; ++i) {
        const float4 q4 = *reinterpret_cast<const float4*>(Qs + (i * WARPS + warp) * d + c);
        s[i] = fmaf(q4.x, kv4.x, s[i]);
        s[i] = fmaf(q4.y, kv4.y, s[i]);
        s[i] = fmaf(q4.z, kv4.z, s[i]);
        s[i] = fmaf(q4.w, kv4.w, s[i]);
      }
    }
    const int kp = t0 + lane;
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      bool vis = (kp <= pos[i]) && (kp < kv_hi);
      if (p.window > 0) vis = vis && (kp > pos[i] - p.window);
      if (SPLIT) vis = vis && (kp >= kv_lo);
      const float sc = vis ? s[i] * p.scale : -INFINITY;
      const float tmax = warp_max(sc);
      const float m_new = fmaxf(m[i], tmax);
      float pj = 0.f, corr = 1.f;
      if (m_new != -INFINITY) {  // warp-uniform
        corr = expf(m[i] - m_new);
        pj = vis ? expf(sc - m_new) : 0.f;
        m[i] = m_new;
      }
      l[i] = l[i] * corr + warp_sum(pj);
#pragma unroll
      for (int e = 0; e < DPL; ++e) acc[i][e] *= corr;
      Ps[(warp * RPW + i) * TK + lane] = pj;
    }
    __syncwarp();
    // ---- O += P V : lane owns dims lane, lane+32, ...
    for (int j = 0; j < TK; j += 4) {
      float4 p4[RPW];
#pragma unroll
      for (int i = 0; i < RPW; ++i) p4[i] = *reinterpret_cast<const float4*>(Ps + (warp * RPW + i) * TK + j);
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
          const int dim = lane + 32 * e;
          const float v = (dim < d) ? Vs[(j + jj) * ldk + dim] : 0.f;
#pragma unroll
          for (int i = 0; i < RPW; ++i) {
            const float pv = jj == 0 ? p4[i].x : jj == 1 ? p4[i].y : jj == 2 ? p4[i].z : p4[i].w;
            acc[i][e] = fmaf(pv, v, acc[i][e]);
          }
        }
      }
    }
    __syncwarp();
  }

  // ---- write
#pragma unroll
  for (int i = 0; i < RPW; ++i) {
    if (pos[i] < 0) continue;
    const int r = i * WARPS + warp;
    const int tok = r / p.gh, head = kvh * g + chunk * p.gh + (r - tok * p.gh);
    if (SPLIT) {
      const size_t slot = ((size_t)b * p.nh + head) * p.max_splits + blockIdx.x;
      if (lane == 0) {
        p.part_ml[slot * 2] = m[i];
        p.part_ml[slot * 2 + 1] = l[i];
      }
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int dim = lane + 32 * e;
        if (dim < d) p.part_acc[slot * d + dim] = acc[i][e];
      }
    } else {
      const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
      T* o = (T*)p.out + (size_t)(q_begin + q0 + tok) * p.out_stride + (size_t)head * d;
#pragma unroll
      for (int e = 0; e < DPL; ++e) {
        const int dim = lane + 32 * e;
        if (dim < d) o[dim] = from_float<T>(acc[i][e] * inv);
      }
    }
  }
}

// Merge the partial results of the key ranges of one (sequence, head), in range order.
template <typename T>
__global__ void attn_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                                    T* __restrict__ out, const int* __restrict__ qsl,
                                    const int* __restrict__ ctx_lens, int nh, int d, int out_stride,
                                    int split_size, int max_splits) {
  const int b = blockIdx.y, head = blockIdx.x;
  const int q_begin = qsl[b], q_len = qsl[b + 1] - q_begin;
  const int ctx = ctx_lens[b];
  if (q_len <= 0 || ctx <= 0) return;
  const int ns = min(max_splits, (ctx + split_size - 1) / split_size);
  const size_t base = ((size_t)b * nh + head) * max_splits;
  float M = -INFINITY;
  for (int s = 0; s < ns; ++s) M = fmaxf(M, part_ml[(base + s) * 2]);
  float L = 0.f;
  for (int s = 0; s < ns; ++s) {
    const float ms = part_ml[(base + s) * 2];
    if (ms != -INFINITY) L += expf(ms - M) * part_ml[(base + s) * 2 + 1];
  }
  const float inv = L > 0.f ? 1.f / L : 0.f;
  T* o = out + (size_t)(q_begin + q_len - 1) * out_stride + (size_t)head * d;
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < ns; ++s) {
      const float ms = part_ml[(base + s) * 2];
      if (ms != -INFINITY) a += expf(ms - M) * part_acc[(base + s) * d + j];
    }
    o[j] = from_float<T>(a * inv);
  }
}

template <typename T, int DPL, bool SPLIT>
int launch_generic(const AttnParams& p, dim3 grid, cudaStream_t st) {
  const size_t smem = (size_t)(2 * TK * (p.d + 4) + ROWS * p.d + WARPS * RPW * TK) * sizeof(float);
  auto kern = paged_attn_generic_kernel<T, DPL, SPLIT>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  kern<<<grid, WARPS * 32, smem, st>>>(p);
  return KVF_LAUNCH_STATUS();
}

template <typename T, bool SPLIT>
int dispatch_dpl(const AttnParams& p, dim3 grid, cudaStream_t st) {
  if (p.d <= 32) return launch_generic<T, 1, SPLIT>(p, grid, st);
  if (p.d <= 64) return launch_generic<T, 2, SPLIT>(p, grid, st);
  if (p.d <= 128) return launch_generic<T, 4, SPLIT>(p, grid, st);
  return launch_generic<T, 8, SPLIT>(p, grid, st);
}

template <typename T>
int paged_attention_generic(const void* q, void* out, const void* kcache, const void* vcache,
                            const int* block_tables, const int* qsl, const int* ctx_lens, int B,
                            int max_q_len, int q_stride, int out_stride, int bt_stride, int nh, int nkv,
                            int d, int block_size, float scale, int window, int split_size, int max_splits,
                            int grid_splits, float* part_acc, float* part_ml, cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (d <= 0 || d > 256 || (d % 8) != 0 || nkv <= 0 || nh % nkv != 0 || block_size <= 0)
    return (int)cudaErrorInvalidValue;
  AttnParams p;
  p.q = q; p.out = out; p.kcache = kcache; p.vcache = vcache;
  p.block_tables = block_tables; p.qsl = qsl; p.ctx_lens = ctx_lens;
  p.part_acc = part_acc; p.part_ml = part_ml;
  p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride;
  p.nh = nh; p.nkv = nkv; p.d = d; p.block_size = block_size;
  const int g = nh / nkv;
  p.gh = g < ROWS ? g : ROWS;
  p.chunks = (g + p.gh - 1) / p.gh;
  p.tq = ROWS / p.gh;
  p.window = window; p.scale = scale;
  p.split_size = split_size; p.max_splits = max_splits;
  if ((unsigned)B > 65535u || (unsigned)(nkv * p.chunks) > 65535u) return (int)cudaErrorInvalidValue;
  if (split_size > 0) {
    // decode form: one query per sequence, key ranges in grid.x, then a merge
    if (split_size % TK != 0 || max_splits <= 0 || !part_acc || !part_ml) return (int)cudaErrorInvalidValue;
    p.tq = 1;
    // grid over the ranges that can be non-empty; max_splits is the scratch's stride
    dim3 grid(grid_splits > 0 && grid_splits < max_splits ? grid_splits : max_splits, B, nkv * p.chunks);
    int rc = dispatch_dpl<T, true>(p, grid, st);
    if (rc) return rc;
    attn_combine_kernel<T><<<dim3(nh, B), 64, 0, st>>>(part_acc, part_ml, (T*)out, qsl, ctx_lens, nh, d,
                                                       out_stride, split_size, max_splits);
    return KVF_LAUNCH_STATUS();
  }
  dim3 grid((max_q_len + p.tq - 1) / p.tq, B, nkv * p.chunks);
  return dispatch_dpl<T, false>(p, grid, st);
}

}  // namespace

#define KVF_ATTN_API(SUF, T)                                                                              \
  KVF_API int kvf_paged_attention_generic_##SUF(                                                          \
      const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables,          \
      const int* qsl, const int* ctx_lens, int B, int max_q_len, int q_stride, int out_stride,            \
      int bt_stride, int nh, int nkv, int d, int block_size, float scale, int window, int split_size,     \
      int max_splits, int grid_splits, float* part_acc, float* part_ml, cudaStream_t st) {                \
    return paged_attention_generic<T>(q, out, kcache, vcache, block_tables, qsl, ctx_lens, B, max_q_len,  \
                                      q_stride, out_stride, bt_stride, nh, nkv, d, block_size, scale,     \
                                      window, split_size, max_splits, grid_splits, part_acc, part_ml,     \
                                      st);                                                                \
  }

KVF_ATTN_API(f32, float)
KVF_ATTN_API(bf16, bf16)
