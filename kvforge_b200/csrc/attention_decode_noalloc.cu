// The allocation-free variant of the split-KV decode attention (see kvforge_noalloc.h for
// who needs it and the rules of use).  It runs the very kernels of attention_mma.cu; what
// differs is where the partial results of the key ranges go: into the fixed array below
// instead of a buffer that the caller allocated.
//
// In host code the name of a __device__ array is a stand-in that lives in host memory, not a
// device address: handing it to a kernel would make the kernel fault, or, on a machine whose
// GPU can reach host memory, quietly scribble over the wrong place.  The device address is
// asked for once per device with cudaGetSymbolAddress, with that device current, and that
// pointer is what the kernels get.
#include <stdio.h>

#include "attention_mma.cu"  // the kernels themselves (they have internal linkage)
#include "kvforge_noalloc.h"

namespace {

constexpr size_t SCRATCH_FLOATS = KVF_NOALLOC_SCRATCH_BYTES / sizeof(float);
static __device__ __align__(256) float g_noalloc_scratch[SCRATCH_FLOATS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};  // device address of the array, per device ordinal

thread_local char g_last_error[256] = "";

int refuse(int code, const char* fmt, long long a = 0, long long b = 0) {
  snprintf(g_last_error, sizeof(g_last_error), fmt, a, b);
  return code;
}

// The array's device address on the current device; looked up on the first call there.
int scratch_on_current_device(float** ptr) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return refuse((int)e, "cudaGetDevice failed (%lld)", (long long)e);
  if (dev < 0 || dev >= MAX_DEVICES) return refuse(KVF_NOALLOC_BAD_ARGUMENT, "device ordinal %lld is out of range", dev);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p) return refuse((int)e, "cudaGetSymbolAddress failed (%lld)", (long long)e);
    g_scratch_addr[dev] = p;
  }
  *ptr = g_scratch_addr[dev];
  return 0;
}

}  // namespace

KVF_API const char* kvf_noalloc_last_error(void) { return g_last_error; }

KVF_API int kvf_paged_attention_decode_noalloc_bf16(const void* q, void* out, const void* kcache,
                                                    const void* vcache, const int* block_tables, const int* qsl,
                                                    const int* ctx_lens, int B, int q_stride, int out_stride,
                                                    int bt_stride, int nh, int nkv, int d, int block_size,
                                                    float scale, int window, int split_size, int max_context,
                                                    cudaStream_t stream) {
  g_last_error[0] = 0;
  if (B <= 0) return 0;
  if (!q || !out || !kcache || !vcache || !block_tables || !qsl || !ctx_lens)
    return refuse(KVF_NOALLOC_BAD_ARGUMENT, "a null pointer was passed");
  if ((d != 64 && d != 128) || nkv <= 0 || nh <= 0 || nh % nkv != 0 || nh / nkv > 16)
    return refuse(KVF_NOALLOC_BAD_ARGUMENT, "needs head size 64 or 128 and at most 16 query heads per kv head (got d=%lld, nh/nkv=%lld)",
                  d, nkv > 0 ? nh / nkv : 0);
  if (split_size <= 0 || split_size % 64 != 0 || max_context <= 0)
    return refuse(KVF_NOALLOC_BAD_ARGUMENT, "split_size must be a positive multiple of 64 and max_context positive (got %lld, %lld)",
                  split_size, max_context);
  const long long splits = ((long long)max_context + split_size - 1) / split_size;
  if (splits > 1024) return refuse(KVF_NOALLOC_TOO_LARGE, "%lld key ranges exceed the limit of 1024: use a larger split_size", splits);
  // layout inside the array: sums [B][nh][splits][d], then (maximum, sum) pairs [B][nh][splits][2]
  const long long acc_floats = (long long)B * nh * splits * d;
  const long long ml_floats = (long long)B * nh * splits * 2;
  if (acc_floats + ml_floats > (long long)SCRATCH_FLOATS)
    return refuse(KVF_NOALLOC_TOO_LARGE, "the partial results need %lld bytes; the built-in scratch holds %lld",
                  (acc_floats + ml_floats) * (long long)sizeof(float), (long long)KVF_NOALLOC_SCRATCH_BYTES);
  float* scratch = nullptr;
  int rc = scratch_on_current_device(&scratch);
  if (rc) return rc;
  rc = kvf_paged_attention_mma_bf16(q, out, kcache, vcache, block_tables, qsl, ctx_lens, B, /*max_q_len=*/1, q_stride,
                                    out_stride, bt_stride, nh, nkv, d, block_size, scale, window, split_size,
                                    (int)splits, (int)splits, scratch, scratch + acc_floats, stream);
  if (rc) return refuse(rc, "the kernels could not be launched (cudaError %lld)", rc);
  return 0;
}
