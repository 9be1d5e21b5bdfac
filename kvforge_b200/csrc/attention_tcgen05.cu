// Paged grouped-query attention for many queries (prompts, portions, mixed batches) on the
// tcgen05 tensor cores; bfloat16, head size 64 or 128.  Same contract as attention_generic.cu.
//
// One CTA serves 128 rows of one kv head of one sequence; a row is a (query token, head of the
// group) pair, so 128/g tokens.  Which tokens: an entry (sequence, first query) of a list made
// on the host with the step, longest walk over the keys first; without a list, the grid's y and
// z.  Keys are walked in tiles of 64 from position 0 (or from the tile that holds the window's
// first key).  Per tile t:
//   S = Q K^T      tcgen05.mma 128 x 64 x (head size), Q and the K tile in 128-byte-swizzled shared
//                  memory (K-major; a 128-wide tile as two 64-wide halves), S in tensor memory;
//   softmax        thread r owns row r (tensor-memory lane r): it reads the 64 scores once with
//                  tcgen05.ld, keeps the running maximum and sum in registers, and writes
//                  P = exp2(S * scale - m) as bfloat16 into shared memory in the swizzled K-major
//                  layout of an A operand (packed f32x2 fma and add, a three-input maximum);
//   O += P V       tcgen05.mma 128 x 64 x 64 per 64 output dims, the V tile [keys][64] as an
//                  MN-major B operand; O stays in tensor memory over all tiles.
// Two groups of four softmax warps take the even and the odd tiles, each with its own S buffer,
// P buffer, O accumulator, maximum and sum; at the end group 0 merges the two.
// The maximum m that P is scaled by follows the row's true maximum lazily: a thread raises it
// only when the true maximum has grown by more than 8 (in log2 units), so P <= 256; then the
// warp multiplies its rows of O by exp2(m_old - m_new) in tensor memory (tcgen05.ld / st) before
// the next P V.  The sum l carries the same factor, so O / l is the exact softmax average.
// Whether a thread rescales depends on its own row only: a row's result does not depend on the
// rows beside it.
// Warps 0-7 do the softmax.  Warp 8 brings Q in with cp.async and the K/V tiles as tensor-map
// boxes of a page's keys (16, 32 or 64 rows of 128 bytes; with pages that are no multiple of 16
// keys, and for a last tile that ends inside a page, key by key with cp.async) through a ring of
// 4 stages (5 at head size 128).  One thread of warp 9 issues the MMAs: when P(t) arrives, first
// S(t+2), which is all its group waits for, then P(t) V(t).  Two CTAs fit an SM at head size 64
// (112 KB of shared memory and 256 tensor-memory columns each), one at 128.
//
// Every mbarrier wait is bounded; if one runs out the kernel raises bit 4 of the error flag and
// winds down.  No cluster launch, no multicast.
#include <cuda.h>
#include <string.h>

#include "common.cuh"

using namespace kvf;

namespace {

// D: head size, 64 or 128.  A [rows][128] tile lies in shared memory as two [rows][64] halves of 128-byte
// swizzled rows; S = Q K^T then walks D/16 k-steps over the halves, and O += P V is one MMA of 64
// output columns per half of V.
constexpr int BM = 128;  // rows per CTA
constexpr int BN = 64;   // keys per tile
constexpr int SOFTMAX_WARPS = 8;                    // two groups of four: even and odd key tiles
constexpr int LOADER_WARP = SOFTMAX_WARPS, MMA_WARP = SOFTMAX_WARPS + 1;
constexpr int THREADS = (SOFTMAX_WARPS + 2) * 32;
template <int D> struct Shape {
  static constexpr int HALVES = D / 64;
  static constexpr int KV_STAGES = D == 64 ? 4 : 5;
  static constexpr int CTAS_PER_SM = D == 64 ? 2 : 1;  // 112 KB and 256 tensor-memory columns, or 224 KB and 512
  static constexpr uint32_t Q_BYTES = HALVES * 128 * 128;     // [128 rows][D] bfloat16
  static constexpr uint32_t KV_BYTES = HALVES * 64 * 128;     // a [64 keys][D] bfloat16 tile
  static constexpr uint32_t TMEM_COLS = D == 64 ? 256u : 512u;  // S: 2 x 64, O: 2 x D
  static constexpr size_t SMEM_BYTES = (size_t)Q_BYTES + (size_t)KV_STAGES * 2 * KV_BYTES + 2 * 128 * 128 + 256;
};
constexpr int LOOKAHEAD = 2;                 // tiles in flight behind the one being handed over
constexpr uint32_t Q_HALF = BM * 128;        // [128 rows][64] bfloat16
constexpr uint32_t KV_HALF = BN * 128;       // [64 keys][64] bfloat16
constexpr uint32_t P_BYTES = BM * 128;       // [128 rows][64 keys] bfloat16
constexpr uint32_t SPIN_LIMIT = 1u << 20;
constexpr float RESCALE_STEP = 8.f;          // log2 units

struct TcAttnParams {
  const bf16* q;
  bf16* out;
  const bf16* kcache;
  const bf16* vcache;
  const int* block_tables;
  const int* qsl;
  const int* ctx_lens;
  const int* work;  // n_work pairs (sequence or -1, first query of the tile), or null: the grid's y and z say which
  int* err;
  int num_seqs;  // a list entry that names a sequence beyond these is a dead tile
  int q_stride, out_stride, bt_stride;
  int nh, nkv, block_size, bs_shift;
  int window;
  float scale_log2;
  int use_tma;     // pages are multiples of 16 keys: K and V tiles come as tensor-map boxes of [box_rows][64]
  int box_rows;    // 16, 32 or 64: the largest of them that divides the page
  int total_rows;  // rows of the cache seen as [rows][64]: a box from this row reads zeros
};

__device__ __forceinline__ uint32_t sm32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
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
    if (done) return true;  // (try_wait itself suspends the thread for a while: no sleep between tries)
  }
  if (err) atomicOr(err, 4);
  return false;
}
__device__ __forceinline__ void cpa16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
// writes made through the generic proxy (cp.async, st.shared) become visible to the tensor core
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 16-byte chunk `c` (0..7) of row `row` of a [rows][64] bfloat16 tile with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int c) { return (uint32_t)(row * 128 + ((c ^ (row & 7)) << 4)); }

// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart (the same
// fields serve a K-major tile and an MN-major tile that is one swizzle row wide).
__device__ __forceinline__ uint64_t sdesc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}
// kind::f16 instruction descriptor: float accumulator, bfloat16 operands, A K-major, B K-major
// or MN-major (bit 16), N >> 3 in [17,23), M >> 4 in [24,29).
__host__ __device__ constexpr uint32_t idesc(int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t id, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(id), "r"(accumulate)
      : "memory");
}
// The same with the accumulate flag known when compiling (no predicate to set up at run time).
template <int ACC>
__device__ __forceinline__ void umma_c(uint32_t tmem_d, uint64_t a, uint64_t b, uint32_t id) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(a), "l"(b), "r"(id), "n"(ACC)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// Waits for the thread's tensor-memory loads; naming the registers as operands keeps the
// compiler from using them before the wait.
__device__ __forceinline__ void tmem_wait(uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]), "+r"(r[8]),
        "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]), "+r"(r[16]),
        "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]),
        "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
      :
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pk(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// One tile of the softmax for the thread's row.  v: the 64 raw scores (in place: not kept).
// MASK: some key of the tile may be hidden from some row of the warp.  Returns the tile's sum of
// P and stores P (bfloat16) into the row of the A-operand tile at p_row (a shared address of
// the row's first byte; chunk c of the row lies at p_row + ((c ^ (r & 7)) << 4)).
// Two floats side by side in a 64-bit register, for the packed fma and add of sm_100.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) { asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

template <bool MASK>
__device__ __forceinline__ float softmax_tile(uint32_t (&va)[32], uint32_t (&vb)[32], float& m_ref, float& corr,
                                              float scale_log2, int first, int last, uint32_t p_row, int r7) {
  // first/last: the tile-local range of visible keys of this row (MASK only)
  float mx = -INFINITY;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const float a = (!MASK || (j >= first && j <= last)) ? __uint_as_float(va[j]) : -INFINITY;
    const float b = (!MASK || (j + 32 >= first && j + 32 <= last)) ? __uint_as_float(vb[j]) : -INFINITY;
    mx = fmaxf(mx, fmaxf(a, b));  // (a three-input maximum)
  }
  mx *= scale_log2;  // scale > 0
  corr = 1.f;
  if (mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx > -INFINITY)) {
    corr = ex2(m_ref - mx);  // 0 the first time
    m_ref = mx;
  }
  const float m_use = (m_ref == -INFINITY) ? 0.f : m_ref;
  const uint64_t scale2 = pack2(scale_log2, scale_log2), neg_m2 = pack2(-m_use, -m_use);
  uint64_t sum_a = pack2(0.f, 0.f), sum_b = sum_a;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint32_t(&v)[32] = half ? vb : va;
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 32; j += 2) {
      const int c = half * 32 + j;
      float x0, x1;
      unpack2(fma2(pack2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), scale2, neg_m2), x0, x1);
      float e0 = ex2(x0), e1 = ex2(x1);
      if (MASK) {
        if (c < first || c > last) e0 = 0.f;
        if (c + 1 < first || c + 1 > last) e1 = 0.f;
      }
      if (j & 2)
        sum_b = add2(sum_b, pack2(e0, e1));
      else
        sum_a = add2(sum_a, pack2(e0, e1));
      w[j >> 1] = pk(e0, e1);
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const uint32_t dst = p_row + (uint32_t)(((half * 4 + q4) ^ r7) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(w[4 * q4]), "r"(w[4 * q4 + 1]),
                   "r"(w[4 * q4 + 2]), "r"(w[4 * q4 + 3])
                   : "memory");
    }
  }
  float s0, s1;
  unpack2(add2(sum_a, sum_b), s0, s1);
  return s0 + s1;
}

template <int D>
__global__ void __launch_bounds__(THREADS, Shape<D>::CTAS_PER_SM)
attn_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v, const TcAttnParams p) {
  constexpr int HALVES = Shape<D>::HALVES, KV_STAGES = Shape<D>::KV_STAGES;
  constexpr uint32_t Q_BYTES = Shape<D>::Q_BYTES, KV_BYTES = Shape<D>::KV_BYTES;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // no slack for rounding up (two CTAs have to fit an SM): the base must be 1024-byte aligned
  // as declared, else the kernel refuses (bit 8 of the error flag) rather than compute garbage
  const uint32_t base = sm32(smem_raw);
  const uint32_t q_s = base;                                    // [128 rows][64]
  const uint32_t kv_s = q_s + Q_BYTES;                          // per stage: K [64 keys][64], V [64 keys][64]
  const uint32_t p_s = kv_s + KV_STAGES * 2 * KV_BYTES;         // two [128 rows][64 keys] buffers
  const uint32_t bars = p_s + 2 * P_BYTES;
  const uint32_t q_full = bars, kv_full0 = bars + 8, kv_empty0 = kv_full0 + 8 * KV_STAGES;
  const uint32_t s_full0 = kv_empty0 + 8 * KV_STAGES, p_full0 = s_full0 + 16, pv_done0 = p_full0 + 16;
  const uint32_t tmem_slot = pv_done0 + 16;
  volatile uint32_t* tmem_slot_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - base));

  pdl_launch();
  if (base & 1023u) {
    if (threadIdx.x == 0 && p.err) atomicOr(p.err, 8);
    pdl_wait();
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid (kv heads, sequences, row blocks): CTAs start in the order of their index with x
  // fastest, so all heads of the longest walk start first, then the next longest, ...
  const int kvh = blockIdx.x;
  const int g = p.nh / p.nkv;
  const int tq = BM / g;
  // which tile of queries: from the list (made on the host, longest walk first), else from the grid
  int b = p.work ? p.work[2 * blockIdx.y] : (int)blockIdx.y;
  const int q0 = p.work ? p.work[2 * blockIdx.y + 1] : (int)(gridDim.z - 1 - blockIdx.z) * tq;  // the longest walks first
  if (b >= p.num_seqs) b = -1;  // whatever a list holds, nothing outside the step's arrays is read
  const int q_begin = b >= 0 ? p.qsl[b] : 0, q_len = b >= 0 ? p.qsl[b + 1] - q_begin : 0;
  const int ctx = b >= 0 ? p.ctx_lens[b] : 0;
  const bool live = q_len > 0 && ctx > 0 && q0 >= 0 && q0 < q_len;  // uniform over the CTA
  // A CTA without a tile leaves at once; the grid's first CTA stays for the dependency wait, so
  // the grid does not complete before its predecessor.
  if (!live && (blockIdx.x | blockIdx.y | blockIdx.z) != 0) return;
  const int n_tok = live ? min(tq, q_len - q0) : 0;
  const int p_first = ctx - q_len + q0;
  const int kv_hi = p_first + n_tok;
  const int kv_lo = p.window > 0 ? (max(0, p_first - p.window + 1) / BN) * BN : 0;
  const int n_tiles = live ? (kv_hi - kv_lo + BN - 1) / BN : 0;

  if (threadIdx.x == 0) {
    bar_init(q_full, 1);
    for (int s = 0; s < KV_STAGES; ++s) {
      bar_init(kv_full0 + 8 * s, 1);
      bar_init(kv_empty0 + 8 * s, 1);
    }
    for (int s = 0; s < 2; ++s) {
      bar_init(s_full0 + 8 * s, 1);
      bar_init(p_full0 + 8 * s, BM);
      bar_init(pv_done0 + 8 * s, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(Shape<D>::TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_ptr;
  // S of even and odd tiles: columns 0..63, 64..127; their O accumulators: 128..191, 192..255
  const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 2 * BN;

  pdl_wait();

  if (live && warp == LOADER_WARP) {
    // ---- loader: Q, then a K and a V tile per stage; 16-byte chunks into the swizzled layout
    const bf16* qg = p.q + (size_t)(q_begin + q0) * p.q_stride + (size_t)(kvh * g) * D;
    for (int idx = lane; idx < BM * (D / 8); idx += 32) {
      const int r = idx / (D / 8), c = idx % (D / 8);
      const int tok = r / g, hh = r - tok * g;
      const bool valid = tok < n_tok;
      cpa16(q_s + (c >> 3) * Q_HALF + sw128(r, c & 7), qg + (valid ? (size_t)tok * p.q_stride + (size_t)hh * D + c * 8 : 0), valid);
    }
    const int* bt = p.block_tables + (size_t)b * p.bt_stride;
    // A tile's 64 keys sit in up to 64 pages: lane l looks up keys l and l+32 (independent table
    // reads), and the copy loop, in which 8 lanes share a key, gets each key's row from the lane
    // that holds it.
    auto issue_tile = [&](int t) {
      const int s = t % KV_STAGES;
      const uint32_t ks = kv_s + s * 2 * KV_BYTES, vs = ks + KV_BYTES;
      const int t0 = kv_lo + t * BN;
      long long row[2];  // element offset of the key's row in the cache, or -1
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int kp = t0 + lane + 32 * j;
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
        row[j] = blk >= 0 ? (((long long)blk * p.nkv + kvh) * p.block_size + off) * D : -1;
      }
      const int c = lane & 7, sub = lane >> 3;
#pragma unroll
      for (int i = 0; i < BN / 4; ++i) {
        const int key = 4 * i + sub;  // held by lane key % 32 in slot key / 32 = i / 8
        const long long src = __shfl_sync(0xffffffffu, row[i >> 3], 4 * (i & 7) + sub);
        const bool valid = src >= 0;
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          const long long at = valid ? src + h * 64 + c * 8 : 0;
          cpa16(ks + h * KV_HALF + sw128(key, c), p.kcache + at, valid);
          cpa16(vs + h * KV_HALF + sw128(key, c), p.vcache + at, valid);
        }
      }
    };
    if (p.use_tma) {
      // A tile is 64 / box_rows boxes of K and as many of V, one pair per lane, which the copy
      // engine lands in the swizzled layout and counts on the stage's barrier.  Only a tile that
      // reaches past the context inside a live page (whatever lies there must not be read: the
      // last tile of the sequence, at most) goes the slow way, which zero-fills by key.
      cpa_commit();  // Q
      bool ok = true, q_handed = false;
      for (int t = 0; t < n_tiles && ok; ++t) {
        const int s = t % KV_STAGES;
        if (t >= KV_STAGES) ok = __all_sync(0xffffffffu, bar_wait(kv_empty0 + 8 * s, ((t / KV_STAGES) - 1) & 1, p.err));
        if (!ok) break;
        const int t0 = kv_lo + t * BN;
        const bool ragged = t0 + BN > ctx && (ctx & (p.box_rows - 1)) != 0;
        if (!ragged) {
          // lane j brings box j of the tile (box_rows keys of one page: a K box and a V box)
          const uint32_t bar = kv_full0 + 8 * s, ks = kv_s + s * 2 * KV_BYTES, vs = ks + KV_BYTES;
          if (lane == 0) bar_expect_tx(bar, 2 * KV_BYTES);
          __syncwarp();
          if (lane < BN / p.box_rows) {
            const int key0 = t0 + p.box_rows * lane;
            int blk = -1, off = 0;
            if (key0 < ctx) {
              if (p.bs_shift >= 0) {
                blk = bt[key0 >> p.bs_shift];
                off = key0 & (p.block_size - 1);
              } else {
                blk = bt[key0 / p.block_size];
                off = key0 % p.block_size;
              }
            }
            const int row = blk >= 0 ? (blk * p.nkv + kvh) * p.block_size + off : p.total_rows;
#pragma unroll
            for (int h = 0; h < HALVES; ++h) {
              tma_load_2d(ks + h * KV_HALF + lane * p.box_rows * 128, &map_k, 64 * h, row, bar);
              tma_load_2d(vs + h * KV_HALF + lane * p.box_rows * 128, &map_v, 64 * h, row, bar);
            }
          }
        } else {
          issue_tile(t);
          cpa_commit();
          cpa_wait<0>();
          fence_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (!q_handed) bar_arrive(q_full);
            bar_arrive(kv_full0 + 8 * s);
          }
          q_handed = true;
        }
        if (!q_handed && (t + 1 >= KV_STAGES || t + 1 == n_tiles)) {
          // the first tiles are on their way: now wait for Q
          cpa_wait<0>();
          fence_async_smem();
          __syncwarp();
          if (lane == 0) bar_arrive(q_full);
          q_handed = true;
        }
      }
    } else {
    // groups: {Q, tile 0}, {tile 1}, ...; an empty group stands for a tile past the end
#pragma unroll
      for (int t = 0; t < LOOKAHEAD; ++t) {
        if (t < n_tiles) issue_tile(t);
        cpa_commit();
      }
      bool ok = true;
      for (int t = 0; t < n_tiles && ok; ++t) {
        // tile t (and, the first time, Q) has landed: hand it to the tensor core
        cpa_wait<LOOKAHEAD - 1>();
        fence_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (t == 0) bar_arrive(q_full);
          bar_arrive(kv_full0 + 8 * (t % KV_STAGES));
        }
        const int nx = t + LOOKAHEAD;
        if (nx < n_tiles) {
          if (nx >= KV_STAGES) ok = bar_wait(kv_empty0 + 8 * (nx % KV_STAGES), ((nx / KV_STAGES) - 1) & 1, p.err);
          if (ok) issue_tile(nx);
        }
        cpa_commit();
      }
      cpa_wait<0>();
    }
  } else if (live && warp == MMA_WARP) {
    if (lane == 0) {
      // ---- MMA issuer.  When P(t) arrives its group waits for S(t+2) and for nothing else, so S(t+2)
      // goes out first (its buffer was read before P(t) was written) and P(t) V(t) after it; whether
      // K(t+2) has landed is asked while the softmax of tile t still runs.  Descriptors are made
      // once; a tile's differ from them by its stage and k-step (the address field counts 16-byte
      // units and cannot carry out of its 14 bits: shared memory ends below 256 KB).
      constexpr uint32_t id_s = idesc(BN, 0), id_o = idesc(64, 1);
      constexpr uint32_t STAGE_UNITS = (2 * KV_BYTES) >> 4;
      const uint64_t q_d = sdesc(q_s), k_d = sdesc(kv_s), v_d = sdesc(kv_s + KV_BYTES), p_d = sdesc(p_s);
      auto issue_s = [&](int t, int stage) {
        const uint32_t dst = tmem_s + (uint32_t)((t & 1) * BN);
        const uint64_t kd = k_d + (uint32_t)stage * STAGE_UNITS;
        umma_c<0>(dst, q_d, kd, id_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk)  // k-steps 0..3 in the first half of the tiles, 4..7 in the second
          umma_c<1>(dst, q_d + (((kk >> 2) * Q_HALF) >> 4) + 2 * (kk & 3), kd + (((kk >> 2) * KV_HALF) >> 4) + 2 * (kk & 3), id_s);
        umma_commit(s_full0 + 8 * (t & 1));
      };
      bool ok = bar_wait(q_full, 0, p.err);
      if (ok) ok = bar_wait(kv_full0, 0, p.err);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(0, 0);
      }
      if (ok && n_tiles > 1) {
        ok = bar_wait(kv_full0 + 8, 0, p.err);
        if (ok) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(1, 1);
        }
      }
      int st_s = 2 % KV_STAGES, st_pv = 0;  // the stages of tile t+2 and of tile t
      for (int t = 0; t < n_tiles && ok; ++t) {
        const bool more = t + 2 < n_tiles;
        if (more) ok = bar_wait(kv_full0 + 8 * st_s, ((t + 2) / KV_STAGES) & 1, p.err);
        if (ok) ok = bar_wait(p_full0 + 8 * (t & 1), (t >> 1) & 1, p.err);  // P(t) is in shared memory, O has been rescaled
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (more) {
          issue_s(t + 2, st_s);
          st_s = st_s + 1 == KV_STAGES ? 0 : st_s + 1;
        }
        const uint64_t vd = v_d + (uint32_t)st_pv * STAGE_UNITS, pd = p_d + (uint32_t)(t & 1) * (P_BYTES >> 4);
        const uint32_t od = tmem_o + (uint32_t)((t & 1) * D);
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {  // 64 output dims per half of V
          // A: 16 keys of P = 32 bytes along the row; B: 16 keys of V = 16 rows of 128 bytes
          umma(od + 64 * h, pd, vd + ((h * KV_HALF) >> 4), id_o, t > 1 ? 1u : 0u);
#pragma unroll
          for (int kk = 1; kk < BN / 16; ++kk) umma_c<1>(od + 64 * h, pd + 2 * kk, vd + ((h * KV_HALF + kk * 16 * 128) >> 4), id_o);
        }
        umma_commit(pv_done0 + 8 * (t & 1));  // O[t&1] holds tiles t&1, .., t; P buffer t&1 may be rewritten
        umma_commit(kv_empty0 + 8 * st_pv);   // and the stage may be refilled
        st_pv = st_pv + 1 == KV_STAGES ? 0 : st_pv + 1;
      }
    }
  } else if (live && warp < SOFTMAX_WARPS) {
    // ---- softmax and output: thread r of each group owns row r; group 0 takes the even key tiles,
    // group 1 the odd ones, each with its S buffer, P buffer, O accumulator, maximum and sum
    const int grp = warp >> 2;
    const int r = threadIdx.x & 127;
    const int tok = r / g, hh = r - tok * g;
    const bool valid = tok < n_tok;
    const int pos = valid ? p_first + tok : -1;
    const int lo = p.window > 0 ? pos - p.window + 1 : 0;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t my_s = tmem_s + lane_addr + (uint32_t)(grp * BN), my_o = tmem_o + lane_addr + (uint32_t)(grp * D);
    const uint32_t s_bar = s_full0 + 8 * grp, p_bar = p_full0 + 8 * grp, pv_bar = pv_done0 + 8 * grp;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    int i = 0;  // index among this group's tiles
    for (int t = grp; t < n_tiles && ok; t += 2, ++i) {
      const int key0 = kv_lo + t * BN;
      // (tcgen05.ld and st are warp-wide: the lanes of a warp leave the loop together)
      ok = __all_sync(0xffffffffu, bar_wait(s_bar, i & 1, p.err));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t va[32], vb[32];
      tmem_ld32(my_s, va);
      tmem_ld32(my_s + 32, vb);
      // the group's last P V is done: its P buffer may be rewritten and its O may be rescaled
      if (i >= 1) ok = bar_wait(pv_bar, (i - 1) & 1, p.err);
      tmem_wait(va);
      tmem_wait(vb);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const bool need_mask = (key0 + BN - 1 > pos) || (key0 < lo);
      const uint32_t p_row = p_s + (uint32_t)grp * P_BYTES + (uint32_t)r * 128u;
      float corr, sum;
      if (__any_sync(0xffffffffu, need_mask))
        sum = softmax_tile<true>(va, vb, m_ref, corr, p.scale_log2, max(lo, key0) - key0, min(pos, key0 + BN - 1) - key0, p_row, r & 7);
      else
        sum = softmax_tile<false>(va, vb, m_ref, corr, p.scale_log2, 0, BN - 1, p_row, r & 7);
      l = l * corr + sum;
      if (i > 0 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
        for (int c0 = 0; c0 < D; c0 += 32) {
          uint32_t v[32];
          tmem_ld32(my_o + (uint32_t)c0, v);
          tmem_wait(v);
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * corr);
          tmem_st32(my_o + (uint32_t)c0, v);
        }
        tmem_wait_st();
      }
      fence_async_smem();
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      bar_arrive(p_bar);
    }
    if (ok && i > 0) ok = __all_sync(0xffffffffu, bar_wait(pv_bar, (i - 1) & 1, p.err));
    // ---- the two groups' results become one: group 1 hands its maximum and sum over (through its P
    // buffer, which its last P V has read), group 0 reads both accumulators
    float2* xch = reinterpret_cast<float2*>(smem_raw + (p_s + P_BYTES - base));
    if (grp == 1) xch[r] = make_float2(ok ? m_ref : -INFINITY, ok ? l : 0.f);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    asm volatile("bar.sync 1, %0;" ::"n"(SOFTMAX_WARPS * 32) : "memory");
    if (grp == 0 && ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float2 other = xch[r];
      const float m_all = fmaxf(m_ref, other.x);
      const float w0 = (m_ref == -INFINITY) ? 0.f : ex2(m_ref - m_all), w1 = (other.x == -INFINITY) ? 0.f : ex2(other.x - m_all);
      const float l_all = l * w0 + other.y * w1;
      const float f0 = l_all > 0.f ? w0 / l_all : 0.f, f1 = l_all > 0.f ? w1 / l_all : 0.f;
      const bool use1 = __any_sync(0xffffffffu, other.y > 0.f);  // group 1 saw a tile (else its accumulator was never written)
      bf16* dst = p.out + (size_t)(q_begin + q0 + (valid ? tok : 0)) * p.out_stride + (size_t)(kvh * g + hh) * D;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t v[32], u[32];
        tmem_ld32(my_o + (uint32_t)c0, v);
        tmem_wait(v);
        if (use1) {
          tmem_ld32(my_o + (uint32_t)(D + c0), u);
          tmem_wait(u);
        }
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            f[e] = __uint_as_float(v[j + e]) * f0;
            if (use1 && f1 != 0.f) f[e] += __uint_as_float(u[j + e]) * f1;
          }
          if (valid)
            *reinterpret_cast<uint4*>(dst + c0 + j) = make_uint4(pk(f[0], f[1]), pk(f[2], f[3]), pk(f[4], f[5]), pk(f[6], f[7]));
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Shape<D>::TMEM_COLS) : "memory");
  }
}

}  // namespace

namespace {

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

// The cache as [rows][d] bfloat16; boxes of [box_rows][64], 128-byte swizzle, zeros past the end.
int cache_map(CUtensorMap* map, const void* ptr, long long rows, int d, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)d, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)d * 2};
  const cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int D>
int launch_tc_attn(const CUtensorMap& mk, const CUtensorMap& mv, const TcAttnParams& p, dim3 grid, cudaStream_t st) {
  cudaError_t e = cudaFuncSetAttribute(attn_tcgen05_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Shape<D>::SMEM_BYTES);
  if (e != cudaSuccess) return (int)e;
  return launch(attn_tcgen05_kernel<D>, grid, dim3(THREADS), Shape<D>::SMEM_BYTES, st, mk, mv, p);
}

}  // namespace

// bfloat16, head size 64 or 128, nh/nkv <= 128; out rows and q rows 16-byte aligned.  err: device flag.
// kcache/vcache: [num_blocks][nkv][block_size][d].
KVF_API int kvf_paged_attention_tcgen05_bf16(const void* q, void* out, const void* kcache, const void* vcache,
                                             const int* block_tables, const int* qsl, const int* ctx_lens, int B,
                                             int max_q_len, int q_stride, int out_stride, int bt_stride, int nh,
                                             int nkv, int d, int block_size, long long num_blocks, float scale,
                                             int window, const int* work, int n_work, int* err, cudaStream_t st) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if ((d != 64 && d != 128) || nkv <= 0 || nh % nkv != 0 || nh / nkv > BM || block_size <= 0 || num_blocks <= 0) return (int)cudaErrorInvalidValue;
  if ((q_stride & 7) || (out_stride & 7) || ((((uintptr_t)q) | ((uintptr_t)out)) & 15)) return (int)cudaErrorInvalidValue;
  if ((unsigned)B > 65535u || (max_q_len + (BM / (nh / nkv)) - 1) / (BM / (nh / nkv)) > 65535) return (int)cudaErrorInvalidValue;
  TcAttnParams p;
  p.q = (const bf16*)q; p.out = (bf16*)out; p.kcache = (const bf16*)kcache; p.vcache = (const bf16*)vcache;
  p.block_tables = block_tables; p.qsl = qsl; p.ctx_lens = ctx_lens; p.err = err;
  p.work = work;
  p.num_seqs = B;
  p.q_stride = q_stride; p.out_stride = out_stride; p.bt_stride = bt_stride;
  p.nh = nh; p.nkv = nkv; p.block_size = block_size; p.window = window;
  p.bs_shift = -1;
  for (int sh = 0; sh < 31; ++sh)
    if ((1 << sh) == block_size) p.bs_shift = sh;
  p.scale_log2 = scale * 1.4426950408889634f;
  // pages of a multiple of 16 keys come in as tensor-map boxes; other page sizes key by key
  const long long rows = num_blocks * nkv * block_size;
  p.use_tma = (block_size % 16 == 0) && rows < (1ll << 31) - 64 && ((((uintptr_t)kcache) | ((uintptr_t)vcache)) & 15) == 0;
  p.total_rows = (int)(p.use_tma ? rows : 0);
  p.box_rows = block_size % 64 == 0 ? 64 : block_size % 32 == 0 ? 32 : 16;
  CUtensorMap mk, mv;
  memset(&mk, 0, sizeof(mk));
  memset(&mv, 0, sizeof(mv));
  if (p.use_tma) {
    if (cache_map(&mk, kcache, rows, d, p.box_rows) || cache_map(&mv, vcache, rows, d, p.box_rows)) p.use_tma = 0;
  }
  const int g = nh / nkv, tq = BM / g;
  if (work && (n_work <= 0 || n_work > 65535)) return (int)cudaErrorInvalidValue;
  const dim3 grid(nkv, work ? n_work : B, work ? 1 : (max_q_len + tq - 1) / tq);
  return d == 64 ? launch_tc_attn<64>(mk, mv, p, grid, st) : launch_tc_attn<128>(mk, mv, p, grid, st);
}
