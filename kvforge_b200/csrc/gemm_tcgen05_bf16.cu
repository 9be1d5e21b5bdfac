// bfloat16 matrix product for many tokens (prefill) on the 5th-generation tensor cores:
//   y[M, N] = x[M, K] * W[N, K]^T,  float accumulation in tensor memory.
//
// A CTA computes 128 x BN tiles of y, one after the other (persistent, one CTA per SM), with
// two accumulators in tensor memory so that a tile's epilogue runs under the next tile's MMAs.
// Roles by warp:
//   warp 0   one thread issues TMA loads (cp.async.bulk.tensor) of the x tile [128 x 64] and the
//            W tile [BN x 64] of each stage into 128-byte-swizzled shared memory and arms the
//            stage's "full" mbarrier with the byte count;
//   warp 1   allocates 2*BN columns of tensor memory, then one thread waits for "full", issues
//            four tcgen05.mma (128 x BN x 16 each) per stage from shared-memory descriptors, and
//            commits them to the stage's "empty" mbarrier (the producer may refill the stage
//            when they have read it); after the last stage it commits to the "accumulator
//            ready" mbarrier;
//   warps 2-5  wait for the accumulator, read it with tcgen05.ld (each warp its quarter of the
//            128 rows, 32 columns at a time), apply the epilogue and store.
// Epilogues: bfloat16 y; or act[M, N/2] = silu(g) * u for W with gate and up rows interleaved
// in blocks of 8 (a thread holds 32 consecutive columns of a row, so g_i and u_i meet in it).
//
// Rows of x past M, rows of W past N and k past K are zero-filled by TMA, so any M and N and
// any K that is a multiple of 8 work; stores are guarded.  Every wait on an mbarrier is
// bounded: if one runs out, the kernel raises bit 4 of the error flag and winds down (tensor
// memory is freed) instead of hanging.  No cluster launch and no multicast.
#include <cuda.h>

#include "common.cuh"

using namespace kvf;

namespace {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bfloat16 = one 128-byte swizzle row
constexpr int THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 20;  // polls of try_wait, each followed by a short sleep: about a second in all

struct TcParams {
  void* out;
  int M, N, K;
  int ldo;
  int mode;  // 0: bfloat16 y; 3: bfloat16 silu(g)*u
  int* err;
};

__device__ __forceinline__ uint32_t sm_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns false (and raises the flag) when
// the limit runs out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err) {
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

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// Shared-memory matrix descriptor for a K-major tile of 128-byte rows with the 128-byte
// swizzle: start address >> 4 in bits [0,14); leading byte offset (unused for this layout)
// = 1 in [16,30); stride between 8-row groups = 1024 bytes >> 4 in [32,46); descriptor
// version 1 in [46,48); layout type 2 (128-byte swizzle) in [61,64).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
  return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) |
         ((uint64_t)2 << 61);
}

// Instruction descriptor of kind::f16: float accumulator (1 in [4,6)), bfloat16 A and B
// (1 in [7,10) and [10,13)), both K-major (0 in bits 15 and 16), N >> 3 in [17,23), M >> 4 in [24,29).
template <int BN> __host__ __device__ constexpr uint32_t instr_desc() {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
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

__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Persistent: a CTA walks tiles t = blockIdx.x, blockIdx.x + gridDim.x, ... (tiles that share a
// W tile are neighbours, so the CTAs that run together read the same weights from L2).  Two
// accumulators of BN columns each alternate, so the epilogue of one tile runs under the MMAs
// of the next.
template <int BN, int STAGES>
__global__ void __launch_bounds__(THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                    const TcParams p) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: a power of two
  // tiles first (each 1024-byte aligned, as the swizzle wants), then the barriers
  const uint32_t smem = (sm_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = smem + STAGES * STAGE_BYTES;
  const uint32_t full0 = bars, empty0 = bars + 8 * STAGES;           // per stage
  const uint32_t acc_full0 = bars + 16 * STAGES, acc_empty0 = acc_full0 + 16;  // per accumulator
  const uint32_t tmem_slot = acc_empty0 + 16;
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - sm_u32(smem_raw)));

  pdl_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m_tiles = (p.M + BM - 1) / BM, n_tiles = (p.N + BN - 1) / BN;
  const int num_tiles = m_tiles * n_tiles;
  const int n_k = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full0 + 8 * b, 1);
      mbar_init(acc_empty0 + 8 * b, 4);  // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot_ptr;

  pdl_wait();  // x comes from the kernel before this one

  if (warp == 0) {
    if (lane == 0) {
      // ---- producer: one running count of stages over all tiles of this CTA
      int g = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
        for (int it = 0; it < n_k; ++it, ++g) {
          const int s = g % STAGES;
          if (g >= STAGES && !mbar_wait(empty0 + 8 * s, ((g / STAGES) - 1) & 1, p.err)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem + s * STAGE_BYTES, b_dst = a_dst + A_BYTES;
          mbar_expect_tx(full0 + 8 * s, STAGE_BYTES);
          tma_load_2d(a_dst, &map_x, it * BK, m0, full0 + 8 * s);
          tma_load_2d(b_dst, &map_w, it * BK, n0, full0 + 8 * s);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- MMA issuer
      constexpr uint32_t idesc = instr_desc<BN>();
      int g = 0, j = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++j) {
        const int b = j & 1;
        // the epilogue must have drained this accumulator's previous tile
        if (j >= 2 && !mbar_wait(acc_empty0 + 8 * b, ((j >> 1) - 1) & 1, p.err)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_d = tmem_base + (uint32_t)(b * BN);
        for (int it = 0; it < n_k; ++it, ++g) {
          const int s = g % STAGES;
          ok = mbar_wait(full0 + 8 * s, (g / STAGES) & 1, p.err);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t adesc = smem_desc(smem + s * STAGE_BYTES), bdesc = smem_desc(smem + s * STAGE_BYTES + A_BYTES);
#pragma unroll
          for (int kk = 0; kk < BK / 16; ++kk)  // 16 k = 32 bytes = 2 units of the descriptor's address field
            umma_bf16(tmem_d, adesc + 2 * kk, bdesc + 2 * kk, idesc, (it > 0 || kk > 0) ? 1u : 0u);
          umma_commit(empty0 + 8 * s);  // arrives when these MMAs have read the stage
        }
        if (ok) umma_commit(acc_full0 + 8 * b);  // arrives when the tile's MMAs have written the accumulator
      }
    }
  } else {
    // ---- epilogue: warp w may touch the 32 lanes (rows) w % 4 of tensor memory
    const int q = warp & 3;
    int j = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++j) {
      const int b = j & 1;
      const int m0 = (t % m_tiles) * BM, n0 = (t / m_tiles) * BN;
      const int row = m0 + q * 32 + lane;
      if (!mbar_wait(acc_full0 + 8 * b, (j >> 1) & 1, p.err)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN + c0), r);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col = n0 + c0;
        if (row >= p.M || col >= p.N) continue;
        if (p.mode == 3) {
          // columns are weight rows [g0..7, u0..7, g8..15, u8..15]: 16 outputs from 32 columns
          bf16* dst = reinterpret_cast<bf16*>(p.out) + (size_t)row * p.ldo + (col >> 1);
          uint32_t o[8];
#pragma unroll
          for (int h = 0; h < 2; ++h)
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
              const float g0 = __uint_as_float(r[16 * h + i]), g1 = __uint_as_float(r[16 * h + i + 1]);
              const float u0 = __uint_as_float(r[16 * h + 8 + i]), u1 = __uint_as_float(r[16 * h + 8 + i + 1]);
              o[4 * h + (i >> 1)] = pack2(__fdividef(g0, 1.f + __expf(-g0)) * u0, __fdividef(g1, 1.f + __expf(-g1)) * u1);
            }
          if (col + 32 <= p.N) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(dst + 8) = make_uint4(o[4], o[5], o[6], o[7]);
          } else {
            const bf16* ob = reinterpret_cast<const bf16*>(o);
            for (int i = 0; i < 16; ++i)
              if (col + 16 * (i >> 3) < p.N) dst[i] = ob[i];  // N is a multiple of 16: whole blocks of [8 g | 8 u]
          }
        } else {
          bf16* dst = reinterpret_cast<bf16*>(p.out) + (size_t)row * p.ldo + col;
          if (col + 32 <= p.N) {
#pragma unroll
            for (int i = 0; i < 32; i += 8)
              *reinterpret_cast<uint4*>(dst + i) =
                  make_uint4(pack2(__uint_as_float(r[i]), __uint_as_float(r[i + 1])),
                             pack2(__uint_as_float(r[i + 2]), __uint_as_float(r[i + 3])),
                             pack2(__uint_as_float(r[i + 4]), __uint_as_float(r[i + 5])),
                             pack2(__uint_as_float(r[i + 6]), __uint_as_float(r[i + 7])));
          } else {
            for (int i = 0; i < 32; ++i)
              if (col + i < p.N) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
          }
        }
      }
      // this warp has read its part of the accumulator: the MMA warp may overwrite it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty0 + 8 * b);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
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

// A [rows x k] bfloat16 matrix with row stride ld elements; boxes of [box_rows x 64], 128-byte
// swizzle, zeros outside the matrix.
int make_map(CUtensorMap* map, const void* ptr, int rows, int k, int ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn) return (int)cudaErrorNotSupported;
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)cudaErrorInvalidValue;
}

template <int BN, int STAGES>
int launch_tc(const CUtensorMap& mx, const CUtensorMap& mw, const TcParams& p, cudaStream_t st) {
  constexpr size_t smem = 1024 + (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 16 * STAGES + 64;
  auto kern = gemm_tcgen05_kernel<BN, STAGES>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return (int)e;
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  dim3 grid(tiles < sms ? tiles : sms);
  return launch(kern, grid, dim3(THREADS), smem, st, mx, mw, p);
}

}  // namespace

// x: [M, K] (row stride ldx), w: [N, K] (row stride ldw), bfloat16, 16-byte aligned, K % 8 == 0,
// strides multiples of 8.  mode 0: out bfloat16 [M, N]; mode 3: out bfloat16 [M, N/2] =
// silu(gate) * up for w in the interleaved gate/up layout (N % 16 == 0).  err: device flag
// (bit 4 is raised if a wait inside the kernel ran out).
KVF_API int kvf_gemm_tcgen05_bf16(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw,
                                  int ldo, int mode, int* err, cudaStream_t st) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K & 7) || (ldx & 7) || (ldw & 7) || (ldo & 7) || (mode != 0 && mode != 3))
    return (int)cudaErrorInvalidValue;
  if ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)out)) & 15) return (int)cudaErrorInvalidValue;
  if (mode == 3 && (N & 15)) return (int)cudaErrorInvalidValue;
  TcParams p;
  p.out = out; p.M = M; p.N = N; p.K = K; p.ldo = ldo; p.mode = mode; p.err = err;
  CUtensorMap mx, mw;
  int rc = make_map(&mx, x, M, K, ldx, BM);
  if (rc) return rc;
  if (N >= 256) {
    rc = make_map(&mw, w, N, K, ldw, 256);
    if (rc) return rc;
    return launch_tc<256, 4>(mx, mw, p, st);
  }
  rc = make_map(&mw, w, N, K, ldw, 128);
  if (rc) return rc;
  return launch_tc<128, 4>(mx, mw, p, st);
}
