// Paged grouped-query attention for decoding (one query per sequence): bfloat16, head size 64
// or 128, at most 8 query heads per kv head, pages of a multiple of 16 tokens.  Same contract
// and the same partial-result layout as the decode form in attention_mma.cu.
//
// Decoding streams the cache once; what a key costs in instructions decides the speed.  So:
//   * A page of one kv head is one contiguous run of the cache.  It comes in by TMA, 16 keys
//     (one box of [16][64] per 64 dims, 128-byte swizzle) per copy and tensor, issued by one
//     lane; pages that were given back, and keys past the context, come from a row past the
//     tensor's end, which the copy fills with zeros.
//   * Keys ride the 16-row side of the MMA and the heads of the group its 8-column side:
//     S^T[16 keys x 8 heads] = K Q^T, then O^T[d x 8 heads] += V^T P^T, the probabilities
//     turned from accumulator to B-operand layout by movmatrix.  Half of the tensor work is
//     real (a quarter with heads on the 16-row side).
//   * A warp owns its units of 16 keys, its shared-memory ring and its mbarriers: nothing in
//     the main loop waits for another warp.
//   * The maximum the probabilities are scaled by is raised only when a score exceeds it by
//     more than 8 (log2 units), so most units cost no cross-lane reduction and no rescaling.
// CTA = (key range, sequence, kv head), 4 warps; warp w takes units w, w+4, ... of the range.
// A range whose keys were all written by earlier steps starts its copies before it waits for
// the kernel ahead of it in the stream.  The four warps' results are merged through shared
// memory into the range's partial result; the CTA that finishes last among the ranges of a
// (sequence, kv head) merges the ranges in range order.
//
// With CLUSTER the CTAs of the ranges of one (sequence, kv head) are one thread-block cluster
// (up to 16), and the merge goes through distributed shared memory: every CTA leaves its partial
// result in its own shared memory, a cluster barrier, then CTA r merges a slice of the outputs by
// reading all the others', in range order, and writes it out; a second barrier keeps every CTA's
// shared memory alive until it has been read.  No partial results in global memory, no fence, no
// ticket.  CTAs of ranges past the context stay for the barriers.
//
// Every mbarrier wait is bounded; if one runs out the kernel raises bit 4 of the error flag.
#include <cuda.h>

#include "attention_merge.cuh"
#include "common.cuh"

using namespace kvf;

namespace {

constexpr int NWARPS = 4;
constexpr int UNIT = 16;  // keys per copy and per MMA row tile
constexpr uint32_t SPIN_LIMIT = 1u << 20;
constexpr float RESCALE_STEP = 8.f;

struct DecParams {
  const bf16* q;
  bf16* out;
  const int* block_tables;
  const int* qsl;
  const int* ctx_lens;
  float* part_acc;  // [B][nh][max_splits][D]
  float* part_ml;   // [B][nh][max_splits][2]  (m in natural-log units, l)
  int* tickets;     // [B][nkv], zero between launches
  int* err;
  int q_stride, out_stride, bt_stride;
  int nh, nkv, block_size;
  int window;
  int single_only;  // sequences that bring more than one query are left alone (another kernel's)
  int split_size, max_splits, grid_splits;
  int wave_target;  // > 0: the range size doubles until the ranges of the longest context are at most this many CTAs
  int total_rows;  // rows of the cache seen as [rows][D]: a copy from this row reads zeros
  float scale_log2;
};

__device__ __forceinline__ uint32_t sm32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, int* err) {
  {  // a phase that is already over is told by a test, which does not suspend the thread
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  if (err) atomicOr(err, 4);
  return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// an 8 x 8 matrix of 16-bit values held one row per four lanes, transposed across the warp
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(d) : "r"(a));
  return d;
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}

// the address of the same shared-memory location in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t in_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ float ld_cluster(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
// every thread of every CTA of the cluster
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// Byte offset of the 16-byte chunk c (0 .. D/8-1) of key `row` (0..15) inside a unit: one box of
// [16][64] (2 KB, 128-byte swizzle) per 64 dims.
__device__ __forceinline__ uint32_t unit_off(int row, int c) {
  return (uint32_t)((c >> 3) * 2048 + row * 128 + (((c & 7) ^ (row & 7)) << 4));
}

// ST: units in flight per warp.  Four of 4 KB (head size 64) keep a warp's whole share of a
// short range in flight; two leave room for seven CTAs on an SM, which suits grids of
// several waves.
template <int D, int ST> struct Shape {
  static constexpr int STAGES = ST;
  static constexpr uint32_t TENSOR_BYTES = UNIT * D * 2;  // K (or V) of one unit
  static constexpr uint32_t STAGE_BYTES = 2 * TENSOR_BYTES;
  static constexpr uint32_t WARP_BYTES = STAGES * STAGE_BYTES;
  static constexpr uint32_t TILES_BYTES = NWARPS * WARP_BYTES;
  static constexpr uint32_t FLAG_OFFSET = TILES_BYTES + NWARPS * STAGES * 8;  // one int: "this CTA merges"
  // CLUSTER: this CTA's partial result [8 heads][D + 2] floats, after the four warps' [4][8][D + 2]
  static constexpr uint32_t RED_BYTES = NWARPS * 8 * (D + 2) * 4;
  static constexpr uint32_t CPART_OFFSET = RED_BYTES;
  static_assert(CPART_OFFSET + 8 * (D + 2) * 4 <= TILES_BYTES, "the partial results lie in the tile area");
  static constexpr uint32_t SMEM_BYTES = FLAG_OFFSET + 16;
};

template <int D, int ST, bool CLUSTER>
__global__ void __launch_bounds__(NWARPS * 32)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                       const DecParams p) {
  using S = Shape<D, ST>;
  constexpr int STAGES = S::STAGES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];  // nothing static beside it: it starts the CTA's window
  pdl_launch();
  const uint32_t base = sm32(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.y, kvh = blockIdx.z, split = blockIdx.x;
  const int g = p.nh / p.nkv;  // <= 8
  const int q_begin = p.qsl[b], q_len = p.qsl[b + 1] - q_begin;
  const int ctx = p.ctx_lens[b];
  // The range size of the launch, or a multiple of it: with few (sequence, kv head) pairs a long
  // context makes more CTAs than run at once, and a second, small wave costs more than longer
  // ranges do.  Every CTA works the size out for itself from the step's longest context, so all
  // agree; the grid was made for the launch's size, and ranges that get no keys leave below.
  int split_size = p.split_size;
  if (p.wave_target > 0) {
    int longest = 0;
    for (int i = lane; i < (int)gridDim.y; i += 32) longest = max(longest, p.ctx_lens[i]);
    longest = __reduce_max_sync(0xffffffffu, longest);
    const int pairs = (int)(gridDim.y * gridDim.z);
    while (split_size < 8192 && (long long)pairs * ((longest + split_size - 1) / split_size) > p.wave_target) split_size <<= 1;
  }
  const int range_lo = split * split_size;
  // dead: no query, a range past the context (the merge never reads it), or shared memory that
  // does not start where the swizzle needs it (refused: bit 8 of the error flag)
  const bool aligned = (base & 1023u) == 0;
  const bool seq_live = (p.single_only ? q_len == 1 : q_len > 0) && ctx > 0;  // the same for all ranges of a sequence: for a whole cluster
  const bool live = seq_live && range_lo < ctx && aligned;
  const int kv_hi = min(ctx, range_lo + split_size);
  const int first_seen = max(range_lo, p.window > 0 ? ctx - p.window : 0);  // first key this range may show
  const int kv_lo = (first_seen / UNIT) * UNIT;
  const bool empty = kv_lo >= kv_hi;  // wholly before the window
  const int n_units = (live && !empty) ? (kv_hi - kv_lo + UNIT - 1) / UNIT : 0;
  const int n_mine = n_units > warp ? (n_units - warp + NWARPS - 1) / NWARPS : 0;
  const int* bt = p.block_tables + (size_t)b * p.bt_stride;
  // A CTA with nothing to do leaves at once and frees its place for one that has; the first CTA
  // of the grid stays to the wait, so that the grid is never done before the kernel ahead of it.
  // With CLUSTER a CTA leaves early only if its whole cluster does (a sequence without query or context).
  if ((CLUSTER ? !seq_live : (!live && aligned)) && (blockIdx.x | blockIdx.y | blockIdx.z) != 0) return;

  const uint32_t tiles = base + warp * S::WARP_BYTES;
  const uint32_t bars = base + S::TILES_BYTES + warp * STAGES * 8;
  if (lane == 0) {
#pragma unroll
    for (int s = 0; s < STAGES; ++s) bar_init(bars + 8 * s, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();

  // unit i of this warp: keys kv_lo + 16 * (warp + 4 i) ...; one lane issues its copies
  auto issue = [&](int i) {
    if (lane == 0) {
      const int key0 = kv_lo + UNIT * (warp + NWARPS * i);
      const int blk = bt[key0 / p.block_size];
      const int row = blk >= 0 ? (blk * p.nkv + kvh) * p.block_size + key0 % p.block_size : p.total_rows;
      const uint32_t bar = bars + 8 * (i % STAGES);
      const uint32_t ks = tiles + (i % STAGES) * S::STAGE_BYTES, vs = ks + S::TENSOR_BYTES;
      bar_expect_tx(bar, S::STAGE_BYTES);
#pragma unroll
      for (int h = 0; h < D / 64; ++h) {
        tma_load_2d(ks + h * 2048, &map_k, h * 64, row, bar);
        tma_load_2d(vs + h * 2048, &map_v, h * 64, row, bar);
      }
    }
  };
  const int token = q_begin + q_len - 1;
  int issued = 0;
  if (kv_hi < ctx) {  // no key of this range is written during this step
    for (; issued < STAGES && issued < n_mine; ++issued) issue(issued);
  }
  pdl_wait();
  if (!aligned && threadIdx.x == 0 && p.err) atomicOr(p.err, 8);
  if (CLUSTER ? !seq_live : !live) return;
  const size_t slot0 = ((size_t)b * p.nh + (size_t)kvh * g) * p.max_splits + split;  // + head * max_splits
  const int ns = min(min(p.max_splits, p.grid_splits), (ctx + split_size - 1) / split_size);

  float* cpart = reinterpret_cast<float*>(smem_raw + S::CPART_OFFSET);  // CLUSTER: [8][D + 2]
  if (empty || !live) {  // (not live: only with CLUSTER) nothing to add, and it says so
    for (int h = threadIdx.x; h < g; h += blockDim.x) {
      if (CLUSTER) {
        cpart[h * (D + 2) + D] = -INFINITY;
        cpart[h * (D + 2) + D + 1] = 0.f;
      } else {
        p.part_ml[(slot0 + (size_t)h * p.max_splits) * 2] = -INFINITY;
        p.part_ml[(slot0 + (size_t)h * p.max_splits) * 2 + 1] = 0.f;
      }
    }
  } else {
    for (; issued < STAGES && issued < n_mine; ++issued) issue(issued);

    // Q^T as B operand: this lane holds head lane/4, dims 16 kk + 2 (lane%4) + {0,1} (+8)
    uint32_t qf[D / 16][2];
    {
      const int head = lane >> 2;
      const bool valid = head < g;
      {
        const bf16* src = p.q + (size_t)token * p.q_stride + (size_t)(kvh * g + (valid ? head : 0)) * D;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const int col = kk * 16 + ((lane & 3) << 1);
          qf[kk][0] = valid ? *reinterpret_cast<const uint32_t*>(src + col) : 0u;
          qf[kk][1] = valid ? *reinterpret_cast<const uint32_t*>(src + col + 8) : 0u;
        }
      }
    }
    // this lane's two heads: n0 = 2 (lane%4), n0 + 1.  o[mt][e]: dim 16 mt + lane/4 (+8 for e >= 2), head n0 + (e & 1)
    float o[D / 16][4];
#pragma unroll
    for (int mt = 0; mt < D / 16; ++mt) o[mt][0] = o[mt][1] = o[mt][2] = o[mt][3] = 0.f;
    float m_ref[2] = {-INFINITY, -INFINITY}, l_part[2] = {0.f, 0.f};

    bool ok = true;
    for (int i = 0; i < n_mine && ok; ++i) {
      const int st = i % STAGES;
      const uint32_t ks = tiles + st * S::STAGE_BYTES, vs = ks + S::TENSOR_BYTES;
      const int key0 = kv_lo + UNIT * (warp + NWARPS * i);
      ok = __all_sync(0xffffffffu, bar_wait(bars + 8 * st, (i / STAGES) & 1, p.err));
      if (!ok) break;
      const bool edge = key0 < first_seen || key0 + UNIT > kv_hi;
      if (key0 + UNIT > kv_hi) {
        // keys at or past kv_hi inside a live page hold whatever was there: their values are zeroed
        // (their scores are masked below), so that nothing of them reaches the sum
        const int r0 = kv_hi - key0;
        for (int idx = r0 * (D / 8) + lane; idx < UNIT * (D / 8); idx += 32) {
          const uint32_t dst = vs + unit_off(idx / (D / 8), idx % (D / 8));
          asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
        }
        __syncwarp();
      }
      // S^T = K Q^T: rows are keys lane/4 (c0, c1) and lane/4 + 8 (c2, c3), columns the heads n0, n0 + 1
      float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t a[4];
        ldsm_x4(a, ks + unit_off((lane & 7) + (((lane >> 3) & 1) << 3), 2 * kk + (lane >> 4)));
        mma16816(c, a, qf[kk][0], qf[kk][1]);
      }
      float s0 = c[0] * p.scale_log2, s1 = c[1] * p.scale_log2, s2 = c[2] * p.scale_log2, s3 = c[3] * p.scale_log2;
      if (edge) {  // warp-uniform
        const int ka = key0 + (lane >> 2), kb = ka + 8;
        if (ka < first_seen || ka >= kv_hi) s0 = s1 = -INFINITY;
        if (kb < first_seen || kb >= kv_hi) s2 = s3 = -INFINITY;
      }
      const float t0 = fmaxf(s0, s2), t1 = fmaxf(s1, s3);
      if (__any_sync(0xffffffffu, t0 > m_ref[0] + RESCALE_STEP || t1 > m_ref[1] + RESCALE_STEP)) {
        // the maximum over the unit's keys: the 8 lanes that share lane % 4 hold a head's column
        float c0 = t0, c1 = t1;
#pragma unroll
        for (int off = 4; off < 32; off <<= 1) {
          c0 = fmaxf(c0, __shfl_xor_sync(0xffffffffu, c0, off));
          c1 = fmaxf(c1, __shfl_xor_sync(0xffffffffu, c1, off));
        }
        const float n0 = fmaxf(m_ref[0], c0), n1 = fmaxf(m_ref[1], c1);
        const float f0 = (n0 == -INFINITY) ? 1.f : ex2(m_ref[0] - n0);
        const float f1 = (n1 == -INFINITY) ? 1.f : ex2(m_ref[1] - n1);
        m_ref[0] = n0;
        m_ref[1] = n1;
        l_part[0] *= f0;
        l_part[1] *= f1;
#pragma unroll
        for (int mt = 0; mt < D / 16; ++mt) {
          o[mt][0] *= f0;
          o[mt][1] *= f1;
          o[mt][2] *= f0;
          o[mt][3] *= f1;
        }
      }
      const float u0 = (m_ref[0] == -INFINITY) ? 0.f : m_ref[0], u1 = (m_ref[1] == -INFINITY) ? 0.f : m_ref[1];
      const float p0 = ex2(s0 - u0), p1 = ex2(s1 - u1), p2 = ex2(s2 - u0), p3 = ex2(s3 - u1);
      l_part[0] += p0 + p2;
      l_part[1] += p1 + p3;
      // P^T as B operand: keys 2 (lane%4) + {0,1} (+8), head lane/4
      const uint32_t b0 = movmatrix_trans(kvf_pack_bf16x2(p0, p1));
      const uint32_t b1 = movmatrix_trans(kvf_pack_bf16x2(p2, p3));
      // O^T += V^T P^T: A = V^T through transposing loads of the [key][dim] tile
#pragma unroll
      for (int mt = 0; mt < D / 16; ++mt) {
        uint32_t a[4];
        ldsm_x4_trans(a, vs + unit_off((lane & 7) + ((lane >> 4) << 3), 2 * mt + ((lane >> 3) & 1)));
        mma16816(o[mt], a, b0, b1);
      }
      __syncwarp();  // every lane has read the stage
      if (i + STAGES < n_mine) issue(i + STAGES);
    }

    // ---- this warp's sums over the lanes that share a head, then the four warps through shared memory
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l_part[0] += __shfl_xor_sync(0xffffffffu, l_part[0], off);
      l_part[1] += __shfl_xor_sync(0xffffffffu, l_part[1], off);
    }
    __syncthreads();  // all warps are done with their tiles
    constexpr int LD = D + 2;
    float* red = reinterpret_cast<float*>(smem_raw);  // [NWARPS][8 heads][D + 2]
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      float* row = red + ((size_t)warp * 8 + ((lane & 3) << 1) + e) * LD;
#pragma unroll
      for (int mt = 0; mt < D / 16; ++mt) {
        row[mt * 16 + (lane >> 2)] = o[mt][e];
        row[mt * 16 + (lane >> 2) + 8] = o[mt][2 + e];
      }
      if ((lane >> 2) == 0) {
        row[D] = m_ref[e];
        row[D + 1] = l_part[e];
      }
    }
    __syncthreads();
    const float LN2 = 0.6931471805599453f;
    for (int idx = threadIdx.x; idx < g * D; idx += blockDim.x) {
      const int r = idx / D, dcol = idx - r * D;
      float M = -INFINITY;
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) M = fmaxf(M, red[((size_t)w * 8 + r) * LD + D]);
      float acc = 0.f, L = 0.f;
#pragma unroll
      for (int w = 0; w < NWARPS; ++w) {
        const float mw = red[((size_t)w * 8 + r) * LD + D];
        const float f = (mw == -INFINITY) ? 0.f : ex2(mw - M);
        acc += f * red[((size_t)w * 8 + r) * LD + dcol];
        L += f * red[((size_t)w * 8 + r) * LD + D + 1];
      }
      if (CLUSTER) {
        cpart[r * LD + dcol] = acc;
        if (dcol == 0) {
          cpart[r * LD + D] = M;  // log2 units
          cpart[r * LD + D + 1] = L;
        }
        continue;
      }
      if (ns == 1) {  // the only range of its sequence: this is the result
        p.out[(size_t)(q_begin + q_len - 1) * p.out_stride + (size_t)(kvh * g + r) * D + dcol] =
            __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        continue;
      }
      const size_t slot = slot0 + (size_t)r * p.max_splits;
      p.part_acc[slot * D + dcol] = acc;
      if (dcol == 0) {
        p.part_ml[slot * 2] = (M == -INFINITY) ? -INFINITY : M * LN2;  // natural-log units for the merge
        p.part_ml[slot * 2 + 1] = L;
      }
    }
    if (!CLUSTER && ns == 1) return;
  }

  if (CLUSTER) {
    // ---- every CTA of the cluster merges a slice of the g * D outputs over the ns ranges, in range order
    cluster_barrier();
    uint32_t nranks;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nranks));
    const int per = (g * D + (int)nranks - 1) / (int)nranks;
    // (the cluster spans x: the rank is blockIdx.x)
    for (int local = threadIdx.x; local < per; local += blockDim.x) {
      const int idx = (int)blockIdx.x * per + local;
      if (idx >= g * D) break;
      const int r = idx / D, dcol = idx - r * D;
      const uint32_t mine = sm32(cpart + r * (D + 2));
      float M = -INFINITY;
      for (int s2 = 0; s2 < ns; ++s2) M = fmaxf(M, ld_cluster(in_cta(mine + D * 4, (uint32_t)s2)));
      float acc = 0.f, L = 0.f;
      for (int s2 = 0; s2 < ns; ++s2) {
        const uint32_t theirs = in_cta(mine, (uint32_t)s2);
        const float ms = ld_cluster(theirs + D * 4);
        if (ms == -INFINITY) continue;  // an empty range left no sums
        const float w = ex2(ms - M);
        acc += w * ld_cluster(theirs + dcol * 4);
        L += w * ld_cluster(theirs + (D + 1) * 4);
      }
      p.out[(size_t)(q_begin + q_len - 1) * p.out_stride + (size_t)(kvh * g + r) * D + dcol] =
          __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
    }
    cluster_barrier();  // nobody leaves while its shared memory may still be read
    return;
  }

  // ---- the CTA that finishes last among the ranges of this (sequence, kv head) merges them
  if (!last_of_ranges(p.tickets + (size_t)b * p.nkv + kvh, ns, reinterpret_cast<int*>(smem_raw + S::FLAG_OFFSET))) return;
  float* wgt = reinterpret_cast<float*>(smem_raw) + warp * 1024;  // ns <= 1024
  bf16* orow = p.out + (size_t)(q_begin + q_len - 1) * p.out_stride;
  for (int h = warp; h < g; h += NWARPS) {
    const int head = kvh * g + h;
    merge_ranges_warp<D>(p.part_acc, p.part_ml, ((size_t)b * p.nh + head) * p.max_splits, ns, wgt, orow + (size_t)head * D, lane);
  }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// The cache as [rows][d] bfloat16; boxes of [16][64], 128-byte swizzle, zeros past the end.
int cache_map(CUtensorMap* map, const void* ptr, long long rows, int d) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)UNIT};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int D, int ST>
int launch_dec(const CUtensorMap& mk, const CUtensorMap& mv, const DecParams& p, int B, bool cluster, cudaStream_t st) {
  size_t smem = Shape<D, ST>::SMEM_BYTES;
  static_assert(Shape<D, ST>::FLAG_OFFSET >= NWARPS * 1024 * 4, "the range merge's weights lie in the tile area");
  const dim3 grid(p.grid_splits, B, p.nkv);
  if (cluster) {
    // the ranges of a (sequence, kv head) as one cluster; more than 8 CTAs need the non-portable size
    auto kern = attn_decode_tma_kernel<D, ST, true>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess && p.grid_splits > 8) e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = grid;
      cfg.blockDim = dim3(NWARPS * 32);
      cfg.dynamicSmemBytes = smem;
      cfg.stream = st;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = p.grid_splits;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = g_pdl_enabled ? 2 : 1;
      e = cudaLaunchKernelEx(&cfg, kern, mk, mv, p);
      if (e == cudaSuccess) return 0;
    }
    (void)cudaGetLastError();  // a cluster this size does not fit here: the ticket form does the same work
  }
  auto kern = attn_decode_tma_kernel<D, ST, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  return launch(kern, grid, dim3(NWARPS * 32), smem, st, mk, mv, p);
}

}  // namespace

namespace {

int run_dec(const void* q, void* out, const void* kcache, const void* vcache,
            const int* block_tables, const int* qsl, const int* ctx_lens, int B, int q_stride, int out_stride,
            int bt_stride, int nh, int nkv, int d, int block_size, long long num_blocks, float scale, int window,
            int split_size, int max_splits, int grid_splits, float* part_acc, float* part_ml, int* tickets, int* err,
            int flags, int wave_target, cudaStream_t st) {
  if (B <= 0) return 0;
  const int cluster = flags & 1;
  if ((d != 64 && d != 128) || nkv <= 0 || nh <= 0 || nh % nkv != 0 || nh / nkv > 8) return (int)cudaErrorInvalidValue;
  if (block_size <= 0 || block_size % UNIT != 0 || num_blocks <= 0) return (int)cudaErrorInvalidValue;
  const long long rows = num_blocks * nkv * block_size;
  if (rows >= (1ll << 31) - UNIT) return (int)cudaErrorInvalidValue;
  if (split_size <= 0 || split_size % UNIT != 0 || max_splits <= 0 || max_splits > 1024 || !part_acc || !part_ml || !tickets)
    return (int)cudaErrorInvalidValue;
  if ((q_stride & 1) || (out_stride & 1) || ((((uintptr_t)kcache) | ((uintptr_t)vcache)) & 15)) return (int)cudaErrorInvalidValue;
  if ((unsigned)B > 65535u || (unsigned)nkv > 65535u) return (int)cudaErrorInvalidValue;
  if (!q) return (int)cudaErrorInvalidValue;
  CUtensorMap mk, mv;
  int rc = cache_map(&mk, kcache, rows, d);
  if (rc) return rc;
  rc = cache_map(&mv, vcache, rows, d);
  if (rc) return rc;
  DecParams p;
  p.q = (const bf16*)q; p.out = (bf16*)out; p.block_tables = block_tables; p.qsl = qsl; p.ctx_lens = ctx_lens;
  p.part_acc = part_acc; p.part_ml = part_ml; p.tickets = tickets; p.err = err;
  p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride;
  p.nh = nh; p.nkv = nkv; p.block_size = block_size; p.window = window;
  p.single_only = (flags & 2) ? 1 : 0;
  p.split_size = split_size; p.max_splits = max_splits; p.wave_target = wave_target > 0 ? wave_target : 0;
  p.grid_splits = grid_splits > 0 && grid_splits < max_splits ? grid_splits : max_splits;
  p.total_rows = (int)rows;
  p.scale_log2 = scale * 1.4426950408889634f;
  // more CTAs than fit at four stages: two stages, so that they run in fewer waves
  const long long ctas = (long long)p.grid_splits * B * nkv;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const bool small = ctas <= 3ll * sms;
  const bool cl = cluster != 0 && p.grid_splits <= 16;
  if (d == 64) return small ? launch_dec<64, 4>(mk, mv, p, B, cl, st) : launch_dec<64, 2>(mk, mv, p, B, cl, st);
  return launch_dec<128, 2>(mk, mv, p, B, cl, st);
}

}  // namespace

// One query per sequence.  kcache/vcache: [num_blocks][nkv][block_size][d] bfloat16, 16-byte
// aligned.  Takes d in {64, 128}, nh/nkv <= 8, block_size a multiple of 16, fewer than 2^31 - 16
// cache rows; refuses anything else with cudaErrorInvalidValue (the caller has other kernels).
// `tickets`: B * nkv counters, zero before the first launch and left zero by every launch;
// launches that share them must not overlap.  flags bit 0: with at most 16 ranges, merge them
// through a thread-block cluster's shared memory instead (scratch and tickets are then unused,
// unless such a cluster cannot be launched here).  flags bit 1: only sequences that bring exactly
// one query are computed (the others of a mixed batch belong to the kernel of prompts).
// wave_target > 0: the kernel doubles split_size (up to 8,192) until the ranges of the longest
// context of the batch, over all B * nkv pairs, are at most that many.
KVF_API int kvf_paged_attention_decode_tma_bf16(const void* q, void* out, const void* kcache, const void* vcache,
                                                const int* block_tables, const int* qsl, const int* ctx_lens, int B,
                                                int q_stride, int out_stride, int bt_stride, int nh, int nkv, int d,
                                                int block_size, long long num_blocks, float scale, int window,
                                                int split_size, int max_splits, int grid_splits, float* part_acc,
                                                float* part_ml, int* tickets, int* err, int flags, int wave_target,
                                                cudaStream_t st) {
  return run_dec(q, out, kcache, vcache, block_tables, qsl, ctx_lens, B, q_stride, out_stride, bt_stride, nh,
                 nkv, d, block_size, num_blocks, scale, window, split_size, max_splits, grid_splits, part_acc, part_ml,
                 tickets, err, flags, wave_target, st);
}
