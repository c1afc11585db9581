// See no_alloc.h: split-KV flash-decode whose scratch lives in a fixed device array.
#include "no_alloc.h"

#include "attention.h"
#include "common.cuh"

namespace {

// The split-KV partials (normalised partial outputs followed by their log-sum-exp).
// In host code this name is only a handle for cudaGetSymbolAddress, never a pointer.
static __device__ __align__(256) unsigned char g_noalloc_scratch[B200_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};   // device address of the array, per device

// Device address of the array on the current device; looked up once per device.
int scratch_address(void** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return B200_NOALLOC_NO_SYMBOL;
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!ptr) return B200_NOALLOC_NO_SYMBOL;
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

B200_API long b200_paged_decode_noalloc_bytes(int B, int Hq, int D, int num_splits) {
  if (num_splits <= 1) return 0;
  return (long)B * Hq * num_splits * (long)(D + 1) * (long)sizeof(float);
}

B200_API int b200_paged_decode_noalloc(const void* q, long q_stride, const void* k_cache,
                                       const void* v_cache, const void* block_table,
                                       int max_blocks, const void* seq_lens, int B, int Hq,
                                       int Hkv, int D, int block_size, float scale, int window,
                                       int num_splits, void* out, long out_stride,
                                       long num_blocks_total, int* status,
                                       cudaStream_t stream) {
  if (B <= 0) return 0;
  if (num_splits < 1) num_splits = 1;
  const long need = b200_paged_decode_noalloc_bytes(B, Hq, D, num_splits);
  if (need > (long)B200_NOALLOC_SCRATCH_BYTES) return B200_NOALLOC_TOO_LARGE;
  float* partial_o = nullptr;
  float* partial_lse = nullptr;
  if (num_splits > 1) {
    void* base = nullptr;
    const int rc = scratch_address(&base);
    if (rc) return rc;
    partial_o = (float*)base;
    partial_lse = partial_o + (long)B * Hq * num_splits * D;
  }
  return b200::launch_paged_decode(q, q_stride, k_cache, v_cache, (const int*)block_table,
                                   max_blocks, (const int*)seq_lens, B, Hq, Hkv, D, block_size,
                                   scale, window, num_splits, out, out_stride, partial_o,
                                   partial_lse, num_blocks_total, status, stream);
}
