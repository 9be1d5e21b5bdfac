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

}  // namespace

// A: [M,K] row stride lda; W: [N,K] row stride ldw; C: [M,N] row stride ldc; all float.
KVF_API int kvf_gemm_nt_f32(const float* A, const float* W, float* C, int M, int N, int K, int lda,
                            int ldw, int ldc, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0) return (int)cudaErrorInvalidValue;
  const int vec_ok = ((lda & 3) == 0) && ((ldw & 3) == 0) && ((((uintptr_t)A) & 15) == 0) &&
                     ((((uintptr_t)W) & 15) == 0);
  dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
  if (grid.y > 65535) return (int)cudaErrorInvalidValue;
  sgemm_nt_kernel<<<grid, 256, 0, st>>>(A, W, C, M, N, K, lda, ldw, ldc, vec_ok);
  return KVF_LAUNCH_STATUS();
}
