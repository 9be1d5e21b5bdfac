// Shared device helpers for the kvforge_b200 kernels (sm_100a).
//
// Storage type T is float (the true 32-bit path) or __nv_bfloat16 (the serving path).
// All arithmetic that the numerics rules name (norms, rotation, softmax, residual sum)
// is done in float whatever T is.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define KVF_API extern "C" __attribute__((visibility("default")))

// Launchers return the launch status so that Python can raise with the kernel's name.
#define KVF_LAUNCH_STATUS() ((int)cudaPeekAtLastError())

namespace kvf {

typedef __nv_bfloat16 bf16;

// ---- programmatic dependent launch: a kernel may be scheduled while the kernel before it in
// the stream is still running, do what does not depend on that kernel (set-up, prefetching
// weights), and wait where it first touches that kernel's results.
//   pdl_launch(): "the next kernel in the stream may be scheduled now".
//   pdl_wait():   returns once every kernel before this one has finished and its writes are
//                 visible.  Nothing that an earlier kernel wrote may be read, and nothing that
//                 an earlier kernel reads may be written, before it.
// Both do nothing when the launch carries no such dependency.
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Whether launches of this library ask for programmatic dependent launch (one flag per
// shared library; off unless the host turns it on).
inline int g_pdl_enabled = 0;

template <typename... KArgs, typename... Args>
inline int launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_pdl_enabled ? 1 : 0;
  return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum with a fixed reduction tree (the result does not depend on the grid).
// `scratch` holds at least 32 floats of shared memory.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : 0.f;
  r = warp_sum(r);
  return r;
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
  r = warp_max(r);
  return r;
}

// 8 bfloat16 values (one 16-byte load) to floats.
__device__ __forceinline__ void bf16x8_to_float(const uint4& u, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}

// One pair of a rotary encoding: (x1, x2) turned by the angle whose cosine and sine are given.
// The roundings are spelled out (a product, then a fused multiply-add) so that every kernel
// that rotates gives the same bits, whichever of them a step's token count selects.
__device__ __forceinline__ void rotate_pair(float x1, float x2, float cs, float sn, float& y1, float& y2) {
  y1 = __fmaf_rn(x1, cs, -__fmul_rn(x2, sn));
  y2 = __fmaf_rn(x2, cs, __fmul_rn(x1, sn));
}

}  // namespace kvf
