// Paged grouped-query attention for bfloat16 on the tensor cores (mma.sync m16n8k16), head
// sizes 64 and 128.  Same contract as attention_generic.cu: sequence b has ctx_b keys after
// this step's writes and q_b queries; query i sits at p = ctx_b - q_b + i and sees key j
// iff j <= p (and j > p - window when window > 0); softmax in float, one rounding.
//
// One CTA serves one kv head of one sequence.  The MMA's 16 rows are (query token, head of
// the group) pairs, so the g query heads that share a kv head share every K/V tile that is
// brought into shared memory.
//   * tile form:  the CTA's 4 warps hold 64 rows (64/g query tokens) and walk the keys in
//     tiles of 64.  Serves prompts, portions and mixed batches.
//   * split form: every sequence has one query (16 rows hold the g heads); grid.x walks key
//     ranges; the 4 warps take 16 keys each of every tile and merge at the end; partial
//     (m, l, acc) go to scratch and a second kernel merges the ranges.
// Keys are walked in tiles that start at multiples of 64 from position 0, so a query's
// result does not depend on how the prompt was cut or on what else is in the batch.
// K/V tiles come in by cp.async (16-byte chunks, XOR-swizzled rows, two stages).
//
// Cache layout per layer: K and V each [num_blocks][nkv][block_size][D].
#include "common.cuh"
#include "attention_merge.cuh"

using namespace kvf;

namespace {

constexpr int BN = 64;       // keys per tile
constexpr int NWARPS = 4;
constexpr int BM = 16 * NWARPS;

struct MmaParams {
  const bf16* q;
  bf16* out;
  const bf16* kcache;
  const bf16* vcache;
  const int* block_tables;
  const int* qsl;
  const int* ctx_lens;
  float* part_acc;  // split form: [B][nh][max_splits][D]
  float* part_ml;   // split form: [B][nh][max_splits][2]  (m in natural-log units, l)
  int* tickets;     // split form: [B][nkv] counters, zero between launches; null: a merge kernel follows
  int q_stride, out_stride, bt_stride;
  int nh, nkv, block_size;
  int bs_shift;  // log2(block_size) if it is a power of two, else -1
  int window;
  int split_size, max_splits;  // max_splits: slices the scratch has room for per (sequence, head)
  int grid_splits;             // ranges that can be non-empty: ceil(longest context / split_size)
  float scale_log2;  // scale * log2(e)
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;  // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of the 16-byte chunk `chunk` of row `row` in a swizzled [rows][D] bf16 tile.
template <int D> __device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
  return (uint32_t)(row * D * 2 + ((chunk ^ (row & 7)) << 4));
}

// Bring keys [t0, t0+BN) of one kv head into a K and a V tile.  Keys at or past `ctx` and
// keys in pages that were given back (table entry < 0) are zero-filled.  What does not
// change from tile to tile (which keys and chunk a thread moves, where they land in the
// swizzled tile) is worked out once.
template <int D>
struct TileLoader {
  static constexpr int CH = D / 8;                       // 16-byte chunks per key
  static constexpr int ITER = BN * CH / (NWARPS * 32);   // chunks per thread and tile
  static constexpr int KEY_STEP = (NWARPS * 32) / CH;    // keys between a thread's chunks
  int key0, chunk;
  uint32_t soff[ITER];
  __device__ __forceinline__ void init() {
    key0 = threadIdx.x / CH;
    chunk = threadIdx.x % CH;
#pragma unroll
    for (int i = 0; i < ITER; ++i) soff[i] = tile_off<D>(key0 + i * KEY_STEP, chunk);
  }
  __device__ __forceinline__ void load(const MmaParams& p, const int* bt, int kvh, int ctx, int t0, uint32_t ks,
                                       uint32_t vs) const {
#pragma unroll
    for (int i = 0; i < ITER; ++i) {
      const int kp = t0 + key0 + i * KEY_STEP;
      int blk = -1, off = 0;
      if (kp < ctx) {
        if (p.bs_shift >= 0) {
          blk = bt[kp >> p.bs_shift];
          off = kp & (p.block_size - 1);
        } else {
          blk = bt[kp / p.block_size];
          off = kp % p.block_size;
        }
      }
      const bool valid = blk >= 0;
      const size_t base = valid ? (((size_t)blk * p.nkv + kvh) * p.block_size + off) * D + chunk * 8 : 0;
      cp_async16(ks + soff[i], p.kcache + base, valid);
      cp_async16(vs + soff[i], p.vcache + base, valid);
    }
  }
};

// S[16 x (8*NT)] += Q[16 x D] K^T for the n-tiles [nt0, nt0+NT) of the K tile at `ks`.
template <int D, int NT>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const uint32_t (&qf)[D / 16][4], uint32_t ks, int nt0, int lane) {
#pragma unroll
  for (int j = 0; j < NT; j += 2) {
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t b[4];
      const int key = (nt0 + j) * 8 + ((lane >> 4) << 3) + (lane & 7);
      const int chunk = 2 * kk + ((lane >> 3) & 1);
      ldmatrix_x4(b, ks + tile_off<D>(key, chunk));
      mma_16816(s[j], qf[kk], b[0], b[1]);
      mma_16816(s[j + 1], qf[kk], b[2], b[3]);
    }
  }
}

// O[16 x D] += P[16 x 16*KS] V for key-steps [ks0, ks0+KS) of the V tile at `vs`; P comes
// from the score accumulators of n-tiles 2*(ks-ks0), 2*(ks-ks0)+1.
template <int D, int KS>
__device__ __forceinline__ void pv_tile(float (&o)[D / 8][4], const float (&s)[2 * KS][4], uint32_t vs, int ks0, int lane) {
#pragma unroll
  for (int k = 0; k < KS; ++k) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * k][0], s[2 * k][1]);
    a[1] = pack_bf16(s[2 * k][2], s[2 * k][3]);
    a[2] = pack_bf16(s[2 * k + 1][0], s[2 * k + 1][1]);
    a[3] = pack_bf16(s[2 * k + 1][2], s[2 * k + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      uint32_t b[4];
      const int key = (ks0 + k) * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
      const int chunk = 2 * dp + (lane >> 4);
      ldmatrix_x4_trans(b, vs + tile_off<D>(key, chunk));
      mma_16816(o[2 * dp], a, b[0], b[1]);
      mma_16816(o[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Mask, running maximum, exponentials and running sum for the two rows a thread holds
// (lane/4 and lane/4 + 8) over NT n-tiles whose first key is `key0`.  Row r sees keys
// lo[r] <= k <= hi[r].  Scores come in as raw dot products and leave as probabilities
// relative to the new maximum.
template <int NT, int ND>
__device__ __forceinline__ void softmax_step(float (&s)[NT][4], float (&o)[ND][4], float (&m)[2], float (&l)[2],
                                             const int (&lo)[2], const int (&hi)[2], int key0, float scale_log2,
                                             int lane, bool need_mask) {
  float mx[2] = {-INFINITY, -INFINITY};
  if (need_mask) {  // warp-uniform: only tiles that straddle an edge of what the rows see
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int r = e >> 1;
        const int kp = key0 + j * 8 + ((lane & 3) << 1) + (e & 1);
        const bool vis = (kp <= hi[r]) && (kp >= lo[r]);
        const float v = vis ? s[j][e] * scale_log2 : -INFINITY;
        s[j][e] = v;
        mx[r] = fmaxf(mx[r], v);
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = s[j][e] * scale_log2;
        s[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
  }
  float corr[2], m_use[2];
  bool changed = false;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float m_new = fmaxf(m[r], mx[r]);
    changed = changed || (m_new != m[r]);
    m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;  // a row that has seen nothing yet
    corr[r] = fast_exp2(m[r] - m_use[r]);
    m[r] = m_new;
  }
  float sum[2] = {0.f, 0.f};
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float pv = fast_exp2(s[j][e] - m_use[e >> 1]);
      s[j][e] = pv;
      sum[e >> 1] += pv;
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 1);
    sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], 2);
  }
  if (__any_sync(0xffffffffu, changed)) {  // a maximum moved: old sums shrink (else the factor is exactly 1)
    l[0] *= corr[0];
    l[1] *= corr[1];
#pragma unroll
    for (int j = 0; j < ND; ++j) {
      o[j][0] *= corr[0];
      o[j][1] *= corr[0];
      o[j][2] *= corr[1];
      o[j][3] *= corr[1];
    }
  }
  l[0] += sum[0];
  l[1] += sum[1];
}

// Query fragments of 16 rows straight from global memory.  Row r of the CTA is
// (token r / g, head r % g); rows past the tile's tokens read zeros.
template <int D>
__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[D / 16][4], const MmaParams& p, int q_token0, int n_tok,
                                             int kvh, int g, int row_base, int lane) {
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = row_base + (lane >> 2) + 8 * h;
    const int tok = r / g, hh = r - tok * g;
    const bool valid = tok < n_tok;
    const bf16* src = p.q + (size_t)(q_token0 + (valid ? tok : 0)) * p.q_stride + (size_t)(kvh * g + hh) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int col = kk * 16 + ((lane & 3) << 1);
      qf[kk][h] = valid ? *reinterpret_cast<const uint32_t*>(src + col) : 0u;
      qf[kk][2 + h] = valid ? *reinterpret_cast<const uint32_t*>(src + col + 8) : 0u;
    }
  }
}

// ------------------------------------------------------------------ tile form
template <int D>
__global__ void __launch_bounds__(NWARPS * 32) attn_mma_tile_kernel(const MmaParams p) {
  pdl_launch();
  pdl_wait();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int TILE_BYTES = BN * D * 2;
  const uint32_t smem = smem_u32(smem_raw);  // stage s: K at s*2*TILE, V at (s*2+1)*TILE

  const int b = blockIdx.y, kvh = blockIdx.z;
  const int g = p.nh / p.nkv;
  const int tq = BM / g;  // query tokens per CTA
  const int q_begin = p.qsl[b], q_len = p.qsl[b + 1] - q_begin;
  const int ctx = p.ctx_lens[b];
  const int q0 = blockIdx.x * tq;
  if (q_len <= 0 || ctx <= 0 || q0 >= q_len) return;
  const int n_tok = min(tq, q_len - q0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p_first = ctx - q_len + q0;
  const int kv_hi = p_first + n_tok;  // one past the last position any row sees
  const int kv_lo = p.window > 0 ? (max(0, p_first - p.window + 1) / BN) * BN : 0;
  const int* bt = p.block_tables + (size_t)b * p.bt_stride;

  TileLoader<D> loader;
  loader.init();
  uint32_t qf[D / 16][4];
  load_q_frags<D>(qf, p, q_begin + q0, n_tok, kvh, g, warp * 16, lane);
  int pos[2], lo[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int tok = (warp * 16 + (lane >> 2) + 8 * h) / g;
    pos[h] = tok < n_tok ? p_first + tok : -1;  // -1: a row past the tile's tokens sees nothing
    lo[h] = p.window > 0 ? pos[h] - p.window + 1 : 0;
  }
  // a warp whose rows all lie past the tile's tokens still helps with the loads
  const bool warp_active = (warp * 16) / g < n_tok;

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  const int n_tiles = (kv_hi - kv_lo + BN - 1) / BN;
  // the warp's rows all see every key of a tile that ends at or before the first row's position
  // and starts at or after the last row's window
  const int warp_tok0 = (warp * 16) / g, warp_tok1 = min(n_tok - 1, (warp * 16 + 15) / g);
  const int all_hi = p_first + warp_tok0;  // keys <= this are seen by every valid row of the warp
  const int all_lo = p.window > 0 ? p_first + warp_tok1 - p.window + 1 : 0;
  const bool rows_full = (warp * 16 + 15) / g < n_tok;  // no row of the warp lies past the tile's tokens
  loader.load(p, bt, kvh, ctx, kv_lo, smem, smem + TILE_BYTES);
  cp_async_commit();
  for (int t = 0; t < n_tiles; ++t) {
    const int st = t & 1;
    if (t + 1 < n_tiles) {
      loader.load(p, bt, kvh, ctx, kv_lo + (t + 1) * BN, smem + (st ^ 1) * 2 * TILE_BYTES,
                  smem + ((st ^ 1) * 2 + 1) * TILE_BYTES);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (warp_active) {
      const uint32_t ks = smem + st * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
      float s[BN / 8][4];
#pragma unroll
      for (int j = 0; j < BN / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
      qk_tile<D, BN / 8>(s, qf, ks, 0, lane);
      const int key0 = kv_lo + t * BN;
      const bool need_mask = !rows_full || key0 + BN - 1 > all_hi || key0 < all_lo;
      softmax_step<BN / 8, D / 8>(s, o, m, l, lo, pos, key0, p.scale_log2, lane, need_mask);
      pv_tile<D, BN / 16>(o, s, vs, 0, lane);
    }
    __syncthreads();  // the stage is free for the load after next
  }

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if (pos[h] < 0) continue;
    const int r = warp * 16 + (lane >> 2) + 8 * h;
    const int tok = r / g, hh = r - tok * g;
    const float inv = l[h] > 0.f ? 1.f / l[h] : 0.f;
    bf16* dst = p.out + (size_t)(q_begin + q0 + tok) * p.out_stride + (size_t)(kvh * g + hh) * D + ((lane & 3) << 1);
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
      *reinterpret_cast<uint32_t*>(dst + j * 8) = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
  }
}

// ------------------------------------------------------------------ split form
// ------------------------------------------------------------------ split form
// Of the keys a range holds, only the newest (position ctx-1, written by the kernel ahead of
// this one in the stream) can change during a step; lengths and block tables were uploaded
// before the step.  So a CTA whose range ends before that key starts fetching its tiles before
// it waits for the kernel ahead.
template <int D>
__global__ void __launch_bounds__(NWARPS * 32) attn_mma_split_kernel(const MmaParams p) {
  pdl_launch();
  extern __shared__ __align__(128) unsigned char smem_raw[];
  __shared__ int s_last;
  constexpr int TILE_BYTES = BN * D * 2;
  const uint32_t smem = smem_u32(smem_raw);

  const int b = blockIdx.y, kvh = blockIdx.z, split = blockIdx.x;
  const int g = p.nh / p.nkv;  // <= 16
  const int q_begin = p.qsl[b], q_len = p.qsl[b + 1] - q_begin;
  const int ctx = p.ctx_lens[b];
  int kv_lo = split * p.split_size;
  // dead: no query, or a range past the context (the merge never reads it)
  const bool live = q_len > 0 && ctx > 0 && kv_lo < ctx;
  const int kv_hi = min(ctx, kv_lo + p.split_size);
  const int key_lo = kv_lo;
  if (p.window > 0) kv_lo = max(kv_lo, (max(0, ctx - p.window) / BN) * BN);
  const bool empty = kv_lo >= kv_hi;  // wholly before the window
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int* bt = p.block_tables + (size_t)b * p.bt_stride;
  TileLoader<D> loader;
  loader.init();
  const int n_tiles = (live && !empty) ? (kv_hi - kv_lo + BN - 1) / BN : 0;
  int issued = 0;
  if (n_tiles > 0 && kv_hi < ctx) {
    for (; issued < 2 && issued < n_tiles; ++issued) {
      loader.load(p, bt, kvh, kv_hi, kv_lo + issued * BN, smem + issued * 2 * TILE_BYTES, smem + (issued * 2 + 1) * TILE_BYTES);
      cp_async_commit();
    }
  }
  pdl_wait();
  if (!live) return;
  const size_t slot0 = ((size_t)b * p.nh + (size_t)kvh * g) * p.max_splits + split;  // + head * max_splits
  // ranges of this sequence that write a partial result
  const int ns = min(min(p.max_splits, p.grid_splits), (ctx + p.split_size - 1) / p.split_size);
  if (empty) {  // an empty range, and it says so
    for (int h = threadIdx.x; h < g; h += blockDim.x) {
      p.part_ml[(slot0 + (size_t)h * p.max_splits) * 2] = -INFINITY;
      p.part_ml[(slot0 + (size_t)h * p.max_splits) * 2 + 1] = 0.f;
    }
  } else {
  // rows are the heads of the group: row r is head r of this kv head; rows >= g are zero
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + 8 * h;
    const bool valid = r < g;
    const bf16* src = p.q + (size_t)(q_begin + q_len - 1) * p.q_stride + (size_t)(kvh * g + (valid ? r : 0)) * D;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      const int col = kk * 16 + ((lane & 3) << 1);
      qf[kk][h] = valid ? *reinterpret_cast<const uint32_t*>(src + col) : 0u;
      qf[kk][2 + h] = valid ? *reinterpret_cast<const uint32_t*>(src + col + 8) : 0u;
    }
  }
  // every row sees the keys of this range that lie inside the window; keys at or past
  // kv_hi were zero-filled and are masked
  const int first_seen = max(key_lo, p.window > 0 ? ctx - p.window : 0);
  const int lo[2] = {first_seen, first_seen};
  const int hi[2] = {kv_hi - 1, kv_hi - 1};

  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  if (issued == 0) {
    loader.load(p, bt, kvh, kv_hi, kv_lo, smem, smem + TILE_BYTES);
    cp_async_commit();
    issued = 1;
  }
  for (int t = 0; t < n_tiles; ++t) {
    const int st = t & 1;
    if (issued == t + 1 && t + 1 < n_tiles) {  // its stage was read in iteration t-1
      loader.load(p, bt, kvh, kv_hi, kv_lo + (t + 1) * BN, smem + (st ^ 1) * 2 * TILE_BYTES,
                  smem + ((st ^ 1) * 2 + 1) * TILE_BYTES);
      cp_async_commit();
      ++issued;
    }
    if (issued > t + 1)
      cp_async_wait<1>();
    else
      cp_async_wait<0>();
    __syncthreads();
    {
      const uint32_t ks = smem + st * 2 * TILE_BYTES, vs = ks + TILE_BYTES;
      float s[2][4];
      s[0][0] = s[0][1] = s[0][2] = s[0][3] = 0.f;
      s[1][0] = s[1][1] = s[1][2] = s[1][3] = 0.f;
      qk_tile<D, 2>(s, qf, ks, 2 * warp, lane);  // this warp's 16 keys of the tile
      const int key0 = kv_lo + t * BN + warp * 16;
      const bool need_mask = key0 < first_seen || key0 + 15 > kv_hi - 1;
      softmax_step<2, D / 8>(s, o, m, l, lo, hi, key0, p.scale_log2, lane, need_mask);
      pv_tile<D, 1>(o, s, vs, warp, lane);
    }
    __syncthreads();
  }

  // ---- merge the 4 warps (each saw a quarter of the keys) through shared memory
  float* red = reinterpret_cast<float*>(smem_raw);  // [NWARPS][16][D + 2]; the tiles are done with
  constexpr int LD = D + 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int r = (lane >> 2) + 8 * h;
    float* row = red + ((size_t)warp * 16 + r) * LD;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      row[j * 8 + ((lane & 3) << 1)] = o[j][2 * h];
      row[j * 8 + ((lane & 3) << 1) + 1] = o[j][2 * h + 1];
    }
    if ((lane & 3) == 0) {
      row[D] = m[h];
      row[D + 1] = l[h];
    }
  }
  __syncthreads();
  const float LN2 = 0.6931471805599453f;
  for (int idx = threadIdx.x; idx < g * D; idx += blockDim.x) {
    const int r = idx / D, dcol = idx - r * D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, red[((size_t)w * 16 + r) * LD + D]);
    float acc = 0.f, L = 0.f;
#pragma unroll
    for (int w = 0; w < NWARPS; ++w) {
      const float mw = red[((size_t)w * 16 + r) * LD + D];
      const float f = (mw == -INFINITY) ? 0.f : fast_exp2(mw - M);
      acc += f * red[((size_t)w * 16 + r) * LD + dcol];
      L += f * red[((size_t)w * 16 + r) * LD + D + 1];
    }
    const size_t slot = slot0 + (size_t)r * p.max_splits;
    p.part_acc[slot * D + dcol] = acc;
    if (dcol == 0) {
      p.part_ml[slot * 2] = (M == -INFINITY) ? -INFINITY : M * LN2;  // natural-log units for the merge
      p.part_ml[slot * 2 + 1] = L;
    }
  }
  }  // a range with keys

  if (p.tickets == nullptr) return;
  // ---- the CTA that finishes last among the ranges of this (sequence, kv head) merges them
  if (!last_of_ranges(p.tickets + (size_t)b * p.nkv + kvh, ns, &s_last)) return;
  float* wgt = reinterpret_cast<float*>(smem_raw) + warp * 1024;  // ns <= 1024
  bf16* orow = p.out + (size_t)(q_begin + q_len - 1) * p.out_stride;
  for (int h = warp; h < g; h += NWARPS) {
    const int head = kvh * g + h;
    merge_ranges_warp<D>(p.part_acc, p.part_ml, ((size_t)b * p.nh + head) * p.max_splits, ns, wgt, orow + (size_t)head * D, lane);
  }
}

// Merge the partial results of the key ranges of one (sequence, head), in range order.
// One CTA of 128 threads per (sequence, head): weights of the ranges first, then each thread
// one output dim.
__global__ void __launch_bounds__(128)
attn_mma_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                      bf16* __restrict__ out, const int* __restrict__ qsl, const int* __restrict__ ctx_lens,
                      int nh, int d, int out_stride, int split_size, int max_splits) {
  pdl_launch();
  pdl_wait();
  __shared__ float wgt[1024];
  __shared__ float red[32];
  const int b = blockIdx.y, head = blockIdx.x;
  const int q_begin = qsl[b], q_len = qsl[b + 1] - q_begin;
  const int ctx = ctx_lens[b];
  if (q_len <= 0 || ctx <= 0) return;
  const int ns = min(min(max_splits, 1024), (ctx + split_size - 1) / split_size);
  const size_t base = ((size_t)b * nh + head) * max_splits;
  float mx = -INFINITY;
  for (int s = threadIdx.x; s < ns; s += blockDim.x) {
    const float ms = part_ml[(base + s) * 2];
    wgt[s] = ms;
    mx = fmaxf(mx, ms);
  }
  const float M = block_max(mx, red);
  float lsum = 0.f;
  for (int s = threadIdx.x; s < ns; s += blockDim.x) {
    const float ms = wgt[s];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - M);
    wgt[s] = w;
    lsum += w * part_ml[(base + s) * 2 + 1];
  }
  const float L = block_sum(lsum, red);  // also orders the writes of wgt before the reads below
  const float inv = L > 0.f ? 1.f / L : 0.f;
  bf16* o = out + (size_t)(q_begin + q_len - 1) * out_stride + (size_t)head * d;
  for (int j = threadIdx.x; j < d; j += blockDim.x) {
    float a = 0.f;
#pragma unroll 4
    for (int s = 0; s < ns; ++s) {
      const float w = wgt[s];
      if (w != 0.f) a += w * part_acc[(base + s) * d + j];  // an empty range wrote no sums
    }
    o[j] = __float2bfloat16_rn(a * inv);
  }
}

template <int D>
int launch_mma(const MmaParams& p, int B, int max_q_len, cudaStream_t st) {
  const size_t smem = (size_t)2 * 2 * BN * D * 2;
  const int g = p.nh / p.nkv;
  if (p.split_size > 0) {
    auto kern = attn_mma_split_kernel<D>;
    size_t need = smem > (size_t)NWARPS * 16 * (D + 2) * 4 ? smem : (size_t)NWARPS * 16 * (D + 2) * 4;
    if (p.tickets && need < (size_t)NWARPS * 1024 * 4) need = (size_t)NWARPS * 1024 * 4;  // the merge's weights
    if (need > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
      if (e != cudaSuccess) return (int)e;
    }
    int rc = launch(kern, dim3(p.grid_splits, B, p.nkv), dim3(NWARPS * 32), need, st, p);
    if (rc || p.tickets) return rc;
    return launch(attn_mma_merge_kernel, dim3(p.nh, B), dim3(128), 0, st, (const float*)p.part_acc,
                  (const float*)p.part_ml, p.out, p.qsl, p.ctx_lens, p.nh, D, p.out_stride, p.split_size, p.max_splits);
  }
  auto kern = attn_mma_tile_kernel<D>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  const int tq = BM / g;
  return launch(kern, dim3((max_q_len + tq - 1) / tq, B, p.nkv), dim3(NWARPS * 32), smem, st, p);
}

}  // namespace

// bfloat16 only; d in {64, 128}; nh/nkv <= 64 (tile form) or <= 16 (split form, chosen by
// split_size > 0: one query per sequence, split_size a multiple of 64).  Anything else is
// refused with cudaErrorInvalidValue: the caller falls back to the generic kernel.
static int run_mma(const void* q, void* out, const void* kcache, const void* vcache, const int* block_tables,
                   const int* qsl, const int* ctx_lens, int B, int max_q_len, int q_stride, int out_stride,
                   int bt_stride, int nh, int nkv, int d, int block_size, float scale, int window, int split_size,
                   int max_splits, int grid_splits, float* part_acc, float* part_ml, int* tickets, cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if ((d != 64 && d != 128) || nkv <= 0 || nh % nkv != 0 || block_size <= 0) return (int)cudaErrorInvalidValue;
  const int g = nh / nkv;
  if (g > BM || (unsigned)B > 65535u || (unsigned)nkv > 65535u) return (int)cudaErrorInvalidValue;
  if ((q_stride & 1) || (out_stride & 1)) return (int)cudaErrorInvalidValue;
  MmaParams p;
  p.q = (const bf16*)q; p.out = (bf16*)out; p.kcache = (const bf16*)kcache; p.vcache = (const bf16*)vcache;
  p.block_tables = block_tables; p.qsl = qsl; p.ctx_lens = ctx_lens;
  p.part_acc = part_acc; p.part_ml = part_ml; p.tickets = split_size > 0 ? tickets : nullptr;
  p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride;
  p.nh = nh; p.nkv = nkv; p.block_size = block_size; p.window = window;
  p.bs_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == block_size) p.bs_shift = sh;
  p.split_size = split_size; p.max_splits = max_splits;
  p.grid_splits = grid_splits > 0 && grid_splits < max_splits ? grid_splits : max_splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  if (split_size > 0) {
    if (g > 16 || split_size % BN != 0 || max_splits <= 0 || max_splits > 1024 || !part_acc || !part_ml || max_q_len != 1)
      return (int)cudaErrorInvalidValue;
  }
  return d == 64 ? launch_mma<64>(p, B, max_q_len, st) : launch_mma<128>(p, B, max_q_len, st);
}

KVF_API int kvf_paged_attention_mma_bf16(const void* q, void* out, const void* kcache, const void* vcache,
                                         const int* block_tables, const int* qsl, const int* ctx_lens, int B,
                                         int max_q_len, int q_stride, int out_stride, int bt_stride, int nh,
                                         int nkv, int d, int block_size, float scale, int window, int split_size,
                                         int max_splits, int grid_splits, float* part_acc, float* part_ml,
                                         cudaStream_t st) {
  return run_mma(q, out, kcache, vcache, block_tables, qsl, ctx_lens, B, max_q_len, q_stride, out_stride, bt_stride, nh,
                 nkv, d, block_size, scale, window, split_size, max_splits, grid_splits, part_acc, part_ml, nullptr, st);
}

// The split form in one launch: `tickets` holds B * nkv counters that are zero before the first
// launch (each launch leaves them zero); the CTA that finishes last among the ranges of a
// (sequence, kv head) merges them.  Launches that share `tickets` must not overlap.
KVF_API int kvf_paged_attention_decode_fused_bf16(const void* q, void* out, const void* kcache, const void* vcache,
                                                  const int* block_tables, const int* qsl, const int* ctx_lens, int B,
                                                  int q_stride, int out_stride, int bt_stride, int nh, int nkv, int d,
                                                  int block_size, float scale, int window, int split_size,
                                                  int max_splits, int grid_splits, float* part_acc, float* part_ml,
                                                  int* tickets, cudaStream_t st) {
  if (!tickets || split_size <= 0) return (int)cudaErrorInvalidValue;
  return run_mma(q, out, kcache, vcache, block_tables, qsl, ctx_lens, B, 1, q_stride, out_stride, bt_stride, nh, nkv, d,
                 block_size, scale, window, split_size, max_splits, grid_splits, part_acc, part_ml, tickets, st);
}
