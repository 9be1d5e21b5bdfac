// True 32-bit matrix product on the FP32 pipes:  C[M,N] = A[M,K] * W[N,K]^T.
//
// No tensor cores and no reduced-precision mode: every product is an FFMA.  Each output
// element is accumulated by one thread over k = 0..K-1 in order, so its value does not
// depend on M, on the tile it falls in or on the rest of the batch.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

__global__ void __launch_bounds__(256)
sgemm_nt_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int M,
                int N, int K, int lda, int ldw, int ldc, int vec_ok) {
  __shared__ __align__(16) float As[BK][BM + PAD];
  __shared__ __align__(16) float Ws[BK][BN + PAD];
  const int t = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int lrow = t >> 2, lk = (t & 3) * 4;  // loader: 64 rows x 4 quads of k
  const int ty = t >> 4, tx = t & 15;         // compute: 16 x 16 threads, 4 x 4 each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  for (int k0 = 0; k0 < K; k0 += BK) {
    float a[4] = {0.f, 0.f, 0.f, 0.f}, w[4] = {0.f, 0.f, 0.f, 0.f};
    const int gm = m0 + lrow, gn = n0 + lrow, gk = k0 + lk;
    if (gm < M) {
      const float* p = A + (size_t)gm * lda + gk;
      if (vec_ok && gk + 3 < K) {
        float4 v = *reinterpret_cast<const float4*>(p);
        a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (gk + i < K) a[i] = p[i];
      }
    }
    if (gn < N) {
      const float* p = W + (size_t)gn * ldw + gk;
      if (vec_ok && gk + 3 < K) {
        float4 v = *reinterpret_cast<const float4*>(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (gk + i < K) w[i] = p[i];
      }
    }
    __syncthreads();  // the previous tile has been consumed
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      As[lk + i][lrow] = a[i];
      Ws[lk + i][lrow] = w[i];
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 wv = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float ar[4] = {av.x, av.y, av.z, av.w};
      const float wr[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
    }
  }
}

// The same sums for many rows (prompts): tiles of 128 x 128 outputs, 8 x 8 per thread (as four blocks
// of 4 x 4, so that a thread's reads of shared memory are whole float4s), the next tile's operands
// fetched into registers while this one is multiplied, two buffers in shared memory.  An output is
// still one accumulator that walks k = 0..K-1 in order: the same bits as from the kernels above and below.
constexpr int LM = 128, LN = 128, LK = 16, LPAD = 4;

__global__ void __launch_bounds__(256, 2)
sgemm_nt_large_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int M,
                      int N, int K, int lda, int ldw, int ldc, int vec_ok) {
  __shared__ __align__(16) float As[2][LK][LM + LPAD];
  __shared__ __align__(16) float Ws[2][LK][LN + LPAD];
  const int t = threadIdx.x;
  const int m0 = blockIdx.y * LM, n0 = blockIdx.x * LN;
  const int ty = t >> 4, tx = t & 15;  // 16 x 16 threads; rows ty*4.. and 64 + ty*4.., columns likewise
  // loader: 128 rows x 4 quads of k, two rows per thread (row, row + 64)
  const int lrow = t >> 2, lk = (t & 3) * 4;
  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
  float ra[2][4], rw[2][4];
  auto fetch = [&](int k0) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int gm = m0 + lrow + 64 * h, gn = n0 + lrow + 64 * h, gk = k0 + lk;
#pragma unroll
      for (int i = 0; i < 4; ++i) ra[h][i] = rw[h][i] = 0.f;
      if (gm < M) {
        const float* p = A + (size_t)gm * lda + gk;
        if (vec_ok && gk + 3 < K) {
          const float4 v = *reinterpret_cast<const float4*>(p);
          ra[h][0] = v.x; ra[h][1] = v.y; ra[h][2] = v.z; ra[h][3] = v.w;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (gk + i < K) ra[h][i] = p[i];
        }
      }
      if (gn < N) {
        const float* p = W + (size_t)gn * ldw + gk;
        if (vec_ok && gk + 3 < K) {
          const float4 v = *reinterpret_cast<const float4*>(p);
          rw[h][0] = v.x; rw[h][1] = v.y; rw[h][2] = v.z; rw[h][3] = v.w;
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            if (gk + i < K) rw[h][i] = p[i];
        }
      }
    }
  };
  auto stash = [&](int buf) {
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        As[buf][lk + i][lrow + 64 * h] = ra[h][i];
        Ws[buf][lk + i][lrow + 64 * h] = rw[h][i];
      }
  };
  fetch(0);
  stash(0);
  __syncthreads();
  int buf = 0;
  for (int k0 = 0; k0 < K; k0 += LK) {
    const bool more = k0 + LK < K;
    if (more) fetch(k0 + LK);  // on its way while this tile is multiplied
#pragma unroll
    for (int k = 0; k < LK; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + ty * 4]);
      const float4 w0 = *reinterpret_cast<const float4*>(&Ws[buf][k][tx * 4]);
      const float4 w1 = *reinterpret_cast<const float4*>(&Ws[buf][k][64 + tx * 4]);
      const float ar[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float wr[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(ar[i], wr[j], acc[i][j]);
    }
    if (more) {
      stash(buf ^ 1);  // the other buffer: its last readers passed the barrier below one tile ago
      __syncthreads();
      buf ^= 1;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int gm = m0 + (i < 4 ? ty * 4 + i : 64 + ty * 4 + i - 4);
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int gn = n0 + (j < 4 ? tx * 4 + j : 64 + tx * 4 + j - 4);
      if (gn < N) C[(size_t)gm * ldc + gn] = acc[i][j];
    }
  }
}

// The same sums for a handful of rows (decoding): with M <= 16 the tiles above are nearly empty and
// a product with a narrow output (N = 2,048: 32 CTAs) leaves most SMs idle.  Here a CTA of 64
// threads takes MR rows of A (8 or 16) and 256 / MR rows of W, four outputs per thread (two rows of
// A by two rows of W); W and A come in through a cp.async pipeline, k contiguous in shared memory,
// and each output is one accumulator that walks k = 0..K-1 in order, exactly as above: the bits are
// the same whichever of the two kernels runs.  (Entries past K are filled with zeros and add
// nothing.)  What bounds a warp is its chains of dependent FMAs, so a thread has four of them.
// Needs K % 4 == 0 and 16-byte aligned rows.
constexpr int SBK = 64, SSTAGES = 6, SLD = SBK + 4, STHREADS = 64;

template <int MR>
__global__ void __launch_bounds__(STHREADS)
sgemm_nt_small_kernel(const float* __restrict__ A, const float* __restrict__ W, float* __restrict__ C, int M,
                      int N, int K, int lda, int ldw, int ldc) {
  constexpr int SBN = 256 / MR, HN = SBN / 2, HM = MR / 2;
  constexpr int STAGE = (SBN + MR) * SLD;  // floats: the rows of W, then the rows of A
  extern __shared__ __align__(16) float small_smem[];
  const int t = threadIdx.x;
  const int n0 = blockIdx.x * SBN;
  const int nl = t % HN, mr = t / HN;  // outputs: rows mr and mr + HM, columns n0 + nl and n0 + nl + HN
  const int n_tiles = (K + SBK - 1) / SBK;
  auto load = [&](int stage, int tile) {
    const int k0 = tile * SBK;
    float* ws = small_smem + stage * STAGE;
    float* as = ws + SBN * SLD;
#pragma unroll
    for (int i = t; i < SBN * 16; i += STHREADS) {  // rows of W x 16 chunks of 4 floats
      const int row = i >> 4, c = (i & 15) * 4;
      const bool ok = n0 + row < N && k0 + c < K;
      const float* src = ok ? W + (size_t)(n0 + row) * ldw + k0 + c : W;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(ws + row * SLD + c);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0));
    }
#pragma unroll
    for (int i = t; i < MR * 16; i += STHREADS) {
      const int row = i >> 4, c = (i & 15) * 4;
      const bool ok = row < M && k0 + c < K;
      const float* src = ok ? A + (size_t)row * lda + k0 + c : A;
      const unsigned dst = (unsigned)__cvta_generic_to_shared(as + row * SLD + c);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(ok ? 16 : 0));
    }
  };
#pragma unroll
  for (int s = 0; s < SSTAGES - 1; ++s) {
    if (s < n_tiles) load(s, s);
    asm volatile("cp.async.commit_group;" ::);
  }
  float c00 = 0.f, c01 = 0.f, c10 = 0.f, c11 = 0.f;  // c[row][column]
  for (int tile = 0; tile < n_tiles; ++tile) {
    asm volatile("cp.async.wait_group %0;" ::"n"(SSTAGES - 2));
    __syncthreads();  // tile `tile` has landed for every thread; tile - 1 has been consumed
    if (tile + SSTAGES - 1 < n_tiles) load((tile + SSTAGES - 1) % SSTAGES, tile + SSTAGES - 1);
    asm volatile("cp.async.commit_group;" ::);
    const float* ws = small_smem + (tile % SSTAGES) * STAGE;
    const float* a0 = ws + SBN * SLD + mr * SLD;
    const float* a1 = a0 + HM * SLD;
    const float* w0 = ws + nl * SLD;
    const float* w1 = w0 + HN * SLD;
#pragma unroll
    for (int k = 0; k < SBK; k += 4) {
      const float4 p = *reinterpret_cast<const float4*>(a0 + k);
      const float4 q = *reinterpret_cast<const float4*>(a1 + k);
      const float4 u = *reinterpret_cast<const float4*>(w0 + k);
      const float4 v = *reinterpret_cast<const float4*>(w1 + k);
      c00 = fmaf(p.x, u.x, c00); c01 = fmaf(p.x, v.x, c01); c10 = fmaf(q.x, u.x, c10); c11 = fmaf(q.x, v.x, c11);
      c00 = fmaf(p.y, u.y, c00); c01 = fmaf(p.y, v.y, c01); c10 = fmaf(q.y, u.y, c10); c11 = fmaf(q.y, v.y, c11);
      c00 = fmaf(p.z, u.z, c00); c01 = fmaf(p.z, v.z, c01); c10 = fmaf(q.z, u.z, c10); c11 = fmaf(q.z, v.z, c11);
      c00 = fmaf(p.w, u.w, c00); c01 = fmaf(p.w, v.w, c01); c10 = fmaf(q.w, u.w, c10); c11 = fmaf(q.w, v.w, c11);
    }
  }
  asm volatile("cp.async.wait_group 0;" ::);
  const int col0 = n0 + nl, col1 = n0 + nl + HN;
  if (mr < M) {
    if (col0 < N) C[(size_t)mr * ldc + col0] = c00;
    if (col1 < N) C[(size_t)mr * ldc + col1] = c01;
  }
  if (mr + HM < M) {
    if (col0 < N) C[(size_t)(mr + HM) * ldc + col0] = c10;
    if (col1 < N) C[(size_t)(mr + HM) * ldc + col1] = c11;
  }
}

template <int MR>
int launch_small(const float* A, const float* W, float* C, int M, int N, int K, int lda, int ldw, int ldc, cudaStream_t st) {
  constexpr int SBN = 256 / MR;
  const size_t smem = (size_t)SSTAGES * (SBN + MR) * SLD * sizeof(float);
  cudaError_t e = cudaFuncSetAttribute(sgemm_nt_small_kernel<MR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  sgemm_nt_small_kernel<MR><<<dim3((N + SBN - 1) / SBN), STHREADS, smem, st>>>(A, W, C, M, N, K, lda, ldw, ldc);
  return KVF_LAUNCH_STATUS();
}

}  // namespace

// A: [M,K] row stride lda; W: [N,K] row stride ldw; C: [M,N] row stride ldc; all float.
KVF_API int kvf_gemm_nt_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda,
                            int ldw, int ldc, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  const int vec_ok = ((lda & 3) == 0) && ((ldw & 3) == 0) && ((((uintptr_t)A) & 15) == 0) &&
                     ((((uintptr_t)W) & 15) == 0);
  if (M <= 16 && vec_ok && (K & 3) == 0) {
    if (M <= 8) return launch_small<8>(A, W, C, M, N, K, lda, ldw, ldc, st);
    return launch_small<16>(A, W, C, M, N, K, lda, ldw, ldc, st);
  }
  if (M > 64 && N > 64) {
    dim3 large((N + LN - 1) / LN, (M + LM - 1) / LM);
    if (large.y > 65535) return (int)cudaErrorInvalidValue;
    sgemm_nt_large_kernel<<<large, 256, 0, st>>>(A, W, C, M, N, K, lda, ldw, ldc, vec_ok);
    return KVF_LAUNCH_STATUS();
  }
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
  sgemm_nt_kernel<<<grid, 256, 0, st>>>(A, W, C, M, N, K, lda, ldw, ldc, vec_ok);
  return KVF_LAUNCH_STATUS();
}
