// Skinny bfloat16 matrix product for decoding:  y[M, N] = x[M, K] * W[N, K]^T  with M <= 64.
//
// With so few tokens the product is bound by streaming W from HBM once.  So W rides the
// MMA's 16-row side (mma.sync m16n8k16, W tile as the A operand) and the tokens its 8-column
// side; a CTA owns 64 rows of W and, when N alone gives too few CTAs to pull the full
// bandwidth, a slice of K (grid.y); W and x tiles come in through a deep cp.async pipeline
// (16-byte chunks, XOR-swizzled rows) so that tens of KB per SM are in flight.
//
// Outputs (mode):
//   0  bfloat16 y[M, N]
//   1  float    y[M, N]                       (logits)
//   2  float    partial[ky][M, N]             one slice of K per grid.y; the consumer sums them
//                                             in slice order, so the result is reproducible
//   3  bfloat16 act[M, N/2] = silu(g) * u     W holds gate and up rows interleaved in blocks
//                                             of 8 ([g0..7, u0..7, g8..15, ...]), so a thread
//                                             finds g_i and u_i in its own accumulators
// Any N; K a multiple of 8; rows and chunks past the edges are zero-filled.
#include "common.cuh"

using namespace kvf;

namespace {

constexpr int BN = 64;   // rows of W per CTA
constexpr int BK = 64;   // k per stage
constexpr int THREADS = 128;

struct SkinnyParams {
  const bf16* x;
  const bf16* w;
  void* out;
  int M, N, K;
  int ldx, ldw, ldo;
  int k_per_split;  // multiple of BK
  int mode;
  long long split_stride;  // elements between partial slices
};

__device__ __forceinline__ uint32_t s_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cpa16(uint32_t dst, const void* src, bool valid) {
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cpa_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cpa_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 16-byte chunk `chunk` (0..7) of row `row` in a swizzled tile of 128-byte rows
__device__ __forceinline__ uint32_t toff(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

// NT: token n-tiles of 8 (M <= 8*NT).  STAGES: pipeline depth.
template <int NT, int STAGES>
__global__ void __launch_bounds__(THREADS) gemm_skinny_kernel(const SkinnyParams p) {
  extern __shared__ __align__(128) unsigned char smem_raw[];
  constexpr int W_BYTES = BN * 128;
  constexpr int X_ROWS = NT * 8;
  constexpr int X_BYTES = X_ROWS * 128;
  constexpr int STAGE_BYTES = W_BYTES + X_BYTES;
  const uint32_t smem = s_u32(smem_raw);

  const int n0 = blockIdx.x * BN;
  const int k_begin = blockIdx.y * p.k_per_split;
  const int k_end = min(p.K, k_begin + p.k_per_split);
  const int n_iters = (k_end - k_begin + BK - 1) / BK;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // W does not depend on the kernel before this one; x does.
  auto load_w = [&](int stage, int it) {
    const int k0 = k_begin + it * BK;
    const uint32_t ws = smem + stage * STAGE_BYTES;
#pragma unroll
    for (int i = 0; i < (BN * 8) / THREADS; ++i) {
      const int idx = threadIdx.x + i * THREADS;
      const int row = idx >> 3, c = idx & 7;
      const int k = k0 + c * 8;
      const bool valid = (n0 + row < p.N) && (k < k_end);
      cpa16(ws + toff(row, c), p.w + (valid ? (size_t)(n0 + row) * p.ldw + k : 0), valid);
    }
  };
  auto load_x = [&](int stage, int it) {
    const int k0 = k_begin + it * BK;
    const uint32_t xs = smem + stage * STAGE_BYTES + W_BYTES;
    for (int idx = threadIdx.x; idx < X_ROWS * 8; idx += THREADS) {
      const int row = idx >> 3, c = idx & 7;
      const int k = k0 + c * 8;
      const bool valid = (row < p.M) && (k < k_end);
      cpa16(xs + toff(row, c), p.x + (valid ? (size_t)row * p.ldx + k : 0), valid);
    }
  };

  float acc[NT][4];
#pragma unroll
  for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;

  // Weight tiles of the first stages start streaming before the kernel ahead of this one in
  // the stream has finished; the activations are fetched once it has.  Group order is
  // W_0..W_{S-2}, x_0..x_{S-2}, then one group per later stage: "all but the newest S-2
  // groups are done" then means that both halves of the current stage have landed.
  pdl_launch();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_iters) load_w(s, s);
    cpa_commit();
  }
  pdl_wait();
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_iters) load_x(s, s);
    cpa_commit();
  }
  for (int it = 0; it < n_iters; ++it) {
    cpa_wait<STAGES - 2>();
    __syncthreads();  // stage `it` has landed for every thread; stage `it-1` has been consumed
    if (it + STAGES - 1 < n_iters) {
      load_w((it + STAGES - 1) % STAGES, it + STAGES - 1);
      load_x((it + STAGES - 1) % STAGES, it + STAGES - 1);
    }
    cpa_commit();
    const uint32_t ws = smem + (it % STAGES) * STAGE_BYTES, xs = ws + W_BYTES;
#pragma unroll
    for (int kk = 0; kk < BK / 16; ++kk) {
      uint32_t a[4];
      ldsm_x4(a, ws + toff(warp * 16 + (lane & 7) + (((lane >> 3) & 1) << 3), 2 * kk + (lane >> 4)));
#pragma unroll
      for (int j = 0; j < NT; j += 2) {
        uint32_t b[4];
        // tokens j*8 .. j*8+15 (for NT == 1 the second half re-reads the first and is unused)
        const int trow = (NT == 1) ? (lane & 7) : (j * 8 + ((lane >> 4) << 3) + (lane & 7));
        ldsm_x4(b, xs + toff(trow, 2 * kk + ((lane >> 3) & 1)));
        mma16816(acc[j], a, b[0], b[1]);
        if (NT > 1) mma16816(acc[j + 1 < NT ? j + 1 : j], a, b[2], b[3]);
      }
    }
  }
  cpa_wait<0>();

  // ---- epilogue.  acc[j]: c0,c1 -> feature f0 = warp*16 + lane/4, tokens t, t+1; c2,c3 -> f0 + 8
  const int f0 = n0 + warp * 16 + (lane >> 2);
#pragma unroll
  for (int j = 0; j < NT; ++j) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int t = j * 8 + ((lane & 3) << 1) + e;
      if (t >= p.M) continue;
      if (p.mode == 3) {
        // rows f0 (gate) and f0 + 8 (up) of the interleaved W are gate_i and up_i, i = n0/2 + warp*8 + lane/4
        const int i = (n0 >> 1) + warp * 8 + (lane >> 2);
        if (2 * i < p.N) {
          const float gv = acc[j][e], uv = acc[j][2 + e];
          reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + i] = __float2bfloat16_rn(gv / (1.f + expf(-gv)) * uv);
        }
      } else {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int f = f0 + 8 * h;
          if (f >= p.N) continue;
          const float v = acc[j][2 * h + e];
          if (p.mode == 0)
            reinterpret_cast<bf16*>(p.out)[(size_t)t * p.ldo + f] = __float2bfloat16_rn(v);
          else
            reinterpret_cast<float*>(p.out)[(size_t)blockIdx.y * p.split_stride + (size_t)t * p.ldo + f] = v;
        }
      }
    }
  }
}

template <int NT, int STAGES>
int launch_skinny(const SkinnyParams& p, int ksplit, cudaStream_t st) {
  const size_t smem = (size_t)STAGES * (BN * 128 + NT * 8 * 128);
  auto kern = gemm_skinny_kernel<NT, STAGES>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  dim3 grid((p.N + BN - 1) / BN, ksplit);
  return launch(kern, grid, dim3(THREADS), smem, st, p);
}

}  // namespace

// x: [M, K] (row stride ldx), w: [N, K] (row stride ldw), both bfloat16, 16-byte aligned rows.
// mode as at the top of this file; ldo = row stride of the output in elements; for mode 2
// `ksplit` slices of K are written split_stride elements apart.  M <= 64, K % 8 == 0.
KVF_API int kvf_gemm_skinny_bf16(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw,
                                 int ldo, int mode, int ksplit, long long split_stride, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (M > 64 || K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || mode < 0 || mode > 3 || ksplit < 1)
    return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)x) & 15) || (((uintptr_t)w) & 15)) return (int)cudaErrorInvalidValue;
  if (mode != 2 && ksplit != 1) return (int)cudaErrorInvalidValue;
  if (mode == 3 && (N & 15)) return (int)cudaErrorInvalidValue;
  SkinnyParams p;
  p.x = (const bf16*)x; p.w = (const bf16*)w; p.out = out;
  p.M = M; p.N = N; p.K = K; p.ldx = ldx; p.ldw = ldw; p.ldo = ldo;
  p.mode = mode; p.split_stride = split_stride;
  const int k_iters = (K + BK - 1) / BK;
  p.k_per_split = ((k_iters + ksplit - 1) / ksplit) * BK;
  if ((long long)(ksplit - 1) * p.k_per_split >= K) return (int)cudaErrorInvalidValue;  // an empty slice
  if (M <= 8) return launch_skinny<1, 8>(p, ksplit, st);
  if (M <= 16) return launch_skinny<2, 8>(p, ksplit, st);
  if (M <= 32) return launch_skinny<4, 6>(p, ksplit, st);
  return launch_skinny<8, 6>(p, ksplit, st);
}
