// The last step of the decode form of paged attention, shared by its kernels: the partial
// results of the key ranges of one (sequence, head) become one output row.
#pragma once

#include "common.cuh"

namespace kvf {

__device__ __forceinline__ uint32_t kvf_pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// The merge of the key ranges of one (sequence, head) by one warp, in range order whichever
// CTA runs it: lanes over the ranges for the weights, then lanes over the output dims.
// wgt: ns floats of shared memory of this warp.  The sums of the first ranges are requested
// before the weights are worked out, so that both reads wait for memory at the same time.
template <int D>
__device__ __forceinline__ void merge_ranges_warp(const float* part_acc, const float* part_ml, size_t base, int ns,
                                                  float* wgt, bf16* o, int lane) {
  constexpr int PRE = 8;     // ranges read ahead
  constexpr int JN = D / 64; // float2 per lane and range
  float2 pre[PRE][JN];
#pragma unroll
  for (int s = 0; s < PRE; ++s) {
#pragma unroll
    for (int jj = 0; jj < JN; ++jj)
      pre[s][jj] = s < ns ? __ldcg(reinterpret_cast<const float2*>(part_acc + (base + s) * D + 2 * lane + 64 * jj)) : make_float2(0.f, 0.f);
  }
  float mx = -INFINITY;
  for (int s = lane; s < ns; s += 32) {
    const float ms = __ldcg(part_ml + (base + s) * 2);
    wgt[s] = ms;
    mx = fmaxf(mx, ms);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
  float lsum = 0.f;
  for (int s = lane; s < ns; s += 32) {
    const float ms = wgt[s];
    const float w = (ms == -INFINITY) ? 0.f : __expf(ms - mx);
    wgt[s] = w;
    lsum += w * __ldcg(part_ml + (base + s) * 2 + 1);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, off);
  __syncwarp();
  const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
  float2 acc[JN];
#pragma unroll
  for (int jj = 0; jj < JN; ++jj) acc[jj] = make_float2(0.f, 0.f);
#pragma unroll
  for (int s = 0; s < PRE; ++s) {
    const float w = s < ns ? wgt[s] : 0.f;
    if (w != 0.f) {  // an empty range wrote no sums: whatever was read for it is dropped
#pragma unroll
      for (int jj = 0; jj < JN; ++jj) {
        acc[jj].x += w * pre[s][jj].x;
        acc[jj].y += w * pre[s][jj].y;
      }
    }
  }
  for (int s = PRE; s < ns; ++s) {
    const float w = wgt[s];
    if (w != 0.f) {
#pragma unroll
      for (int jj = 0; jj < JN; ++jj) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(part_acc + (base + s) * D + 2 * lane + 64 * jj));
        acc[jj].x += w * v.x;
        acc[jj].y += w * v.y;
      }
    }
  }
#pragma unroll
  for (int jj = 0; jj < JN; ++jj) *reinterpret_cast<uint32_t*>(o + 2 * lane + 64 * jj) = kvf_pack_bf16x2(acc[jj].x * inv, acc[jj].y * inv);
  __syncwarp();
}

// The CTA-wide hand-over before that merge: every CTA of a (sequence, kv head) has written its
// partial results; the one that draws the last of `ns` tickets merges (and leaves the counter
// at zero for the next launch).  Returns whether this CTA is that one.  s_flag: one int of
// shared memory.
__device__ __forceinline__ bool last_of_ranges(int* ticket, int ns, int* s_flag) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int t = atomicAdd(ticket, 1);
    *s_flag = (t == ns - 1);
    if (t == ns - 1) *ticket = 0;
  }
  __syncthreads();
  const bool last = *s_flag != 0;
  if (last) __threadfence();
  return last;
}

}  // namespace kvf
