// KV-cache block movement.
//   * kv_block_copy: gather/scatter of paged KV blocks between two caches (same GPU, or a
//     peer GPU's cache mapped through CUDA IPC: the loads then cross NVLink from inside the
//     kernel).  One launch moves any number of (src block -> dst block) pairs of every
//     layer, optionally re-slicing KV heads when prefill and decode use different TP sizes.
//     It is the worker side of the disaggregated-prefill connector: the reference builds
//     (src, dst, len) lists per layer and hands them to a transfer engine, then fixes the
//     layout with transpose_kv_cache_by_block
//     (vllm_ascend/distributed/kv_transfer/kv_p2p/mooncake_connector.py:775-1028, 1271-1296);
//     here the copy writes straight into the destination block table layout.
//   * swap/copy blocks inside one cache (attention/attention_v1.py:119-145).
#include "common.cuh"
#include <cstdio>
#include <cuda_bf16.h>

namespace b200 {

struct KvCopyParams {
  const void* const* src_tensors;   // [num_tensors] device array of cache base pointers (K and V of every layer)
  void* const* dst_tensors;         // [num_tensors]
  const int* src_blocks;            // [num_pairs]
  const int* dst_blocks;            // [num_pairs]
  int num_pairs, num_tensors;
  int block_size, head_dim_bytes;   // bytes of one (token, head) vector
  int num_heads;                    // heads to copy
  int src_head0, dst_head0;         // first head on each side
  // element strides in bytes: block, token, head
  long src_sb, src_st, src_sh;
  long dst_sb, dst_st, dst_sh;
  long src_num_blocks, dst_num_blocks;
  int* status;
};

__global__ void kv_block_copy_kernel(const KvCopyParams p) {
  const int pair = blockIdx.x, tensor = blockIdx.y;
  const int sb = p.src_blocks[pair], db = p.dst_blocks[pair];
  if (sb < 0 || sb >= p.src_num_blocks || db < 0 || db >= p.dst_num_blocks) {
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, B200_BAD_INDEX);
    return;
  }
  const uint8_t* src = (const uint8_t*)p.src_tensors[tensor] + (long)sb * p.src_sb;
  uint8_t* dst = (uint8_t*)p.dst_tensors[tensor] + (long)db * p.dst_sb;
  const int vecs = p.head_dim_bytes >> 4;
  const int total = p.block_size * p.num_heads * vecs;
  for (int i = threadIdx.x; i < total; i += blockDim.x) {
    const int v = i % vecs;
    const int rest = i / vecs;
    const int tok = rest % p.block_size;
    const int h = rest / p.block_size;
    const uint4 val = *reinterpret_cast<const uint4*>(
        src + (long)tok * p.src_st + (long)(p.src_head0 + h) * p.src_sh + (v << 4));
    *reinterpret_cast<uint4*>(dst + (long)tok * p.dst_st + (long)(p.dst_head0 + h) * p.dst_sh +
                              (v << 4)) = val;
  }
}

// pairs [n, 2] (src, dst) inside one cache tensor; block_bytes contiguous per block
__global__ void copy_blocks_kernel(uint8_t* cache, const long* pairs, long block_bytes) {
  const long s = pairs[2 * blockIdx.x], d = pairs[2 * blockIdx.x + 1];
  const uint4* src = reinterpret_cast<const uint4*>(cache + s * block_bytes);
  uint4* dst = reinterpret_cast<uint4*>(cache + d * block_bytes);
  for (long i = threadIdx.x; i < (block_bytes >> 4); i += blockDim.x) dst[i] = src[i];
}

}  // namespace b200

using namespace b200;

// src_tensors / dst_tensors: DEVICE arrays of num_tensors base pointers.
// strides in bytes (block, token, head).  head_dim_bytes multiple of 16.
B200_API int b200_kv_block_copy(const void* src_tensors, const void* dst_tensors,
                                const void* src_blocks, const void* dst_blocks, int num_pairs,
                                int num_tensors, int block_size, int head_dim_bytes,
                                int num_heads, int src_head0, int dst_head0, long src_sb,
                                long src_st, long src_sh, long dst_sb, long dst_st, long dst_sh,
                                long src_num_blocks, long dst_num_blocks, int* status,
                                cudaStream_t stream) {
  if (num_pairs <= 0 || num_tensors <= 0) return 0;
  if (head_dim_bytes & 15) return 9100;
  KvCopyParams p;
  p.src_tensors = (const void* const*)src_tensors;
  p.dst_tensors = (void* const*)dst_tensors;
  p.src_blocks = (const int*)src_blocks;
  p.dst_blocks = (const int*)dst_blocks;
  p.num_pairs = num_pairs; p.num_tensors = num_tensors;
  p.block_size = block_size; p.head_dim_bytes = head_dim_bytes;
  p.num_heads = num_heads; p.src_head0 = src_head0; p.dst_head0 = dst_head0;
  p.src_sb = src_sb; p.src_st = src_st; p.src_sh = src_sh;
  p.dst_sb = dst_sb; p.dst_st = dst_st; p.dst_sh = dst_sh;
  p.src_num_blocks = src_num_blocks; p.dst_num_blocks = dst_num_blocks;
  p.status = status;
  dim3 grid((unsigned)num_pairs, (unsigned)num_tensors);
  kv_block_copy_kernel<<<grid, 256, 0, stream>>>(p);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_copy_blocks(void* cache, const void* pairs, int num_pairs, long block_bytes,
                              cudaStream_t stream) {
  if (num_pairs <= 0) return 0;
  if (block_bytes & 15) return 9100;
  copy_blocks_kernel<<<num_pairs, 256, 0, stream>>>((uint8_t*)cache, (const long*)pairs,
                                                    block_bytes);
  return B200_CHECK_LAUNCH();
}

// ---------------------------------------------------------------- block zeroing / debug print
namespace b200 {

// Zero whole KV blocks of every cache tensor: freshly allocated blocks must not carry bit
// patterns of earlier requests into masked positions (the reference zeroes new blocks with
// a small kernel of its own, vllm_ascend/worker/utils.py:15-184).
__global__ void zero_blocks_kernel(void* const* tensors, const int* blocks, long block_stride_bytes,
                                   long block_bytes) {
  uint8_t* base = (uint8_t*)tensors[blockIdx.y] + (long)blocks[blockIdx.x] * block_stride_bytes;
  uint4* p = reinterpret_cast<uint4*>(base);
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (long i = threadIdx.x; i < (block_bytes >> 4); i += blockDim.x) p[i] = z;
}

// Graph-safe debug print: runs as a kernel in stream order, so it also shows values inside
// captured graphs (role of the reference's device_print / device_print_tensor ops).
__global__ void device_print_kernel(const float* f32, const __nv_bfloat16* bf16, long n, int tag) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  printf("[device_print %d]", tag);
  for (long i = 0; i < n; i++) printf(" %g", f32 ? f32[i] : __bfloat162float(bf16[i]));
  printf("\n");
}

}  // namespace b200

// tensors: device array of num_tensors base pointers of DENSE per-block storage (block b of
// tensor i starts at base + b * block_stride_bytes); blocks: device int32 [num_blocks].
B200_API int b200_zero_blocks(const void* tensors, int num_tensors, const void* blocks, int num_blocks,
                              long block_stride_bytes, long block_bytes, cudaStream_t stream) {
  if (num_blocks <= 0 || num_tensors <= 0) return 0;
  if ((block_bytes & 15) || (block_stride_bytes & 15)) return 9100;
  zero_blocks_kernel<<<dim3(num_blocks, num_tensors), 256, 0, stream>>>(
      (void* const*)tensors, (const int*)blocks, block_stride_bytes, block_bytes);
  return B200_CHECK_LAUNCH();
}

// dtype 0: fp32, 1: bf16; prints the first n values
B200_API int b200_device_print(const void* data, int dtype, long n, int tag, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n > 64) n = 64;
  device_print_kernel<<<1, 32, 0, stream>>>(dtype == 0 ? (const float*)data : nullptr,
                                            dtype == 1 ? (const __nv_bfloat16*)data : nullptr, n, tag);
  return B200_CHECK_LAUNCH();
}

// ---------------------------------------------------------------- wait budget (all kernels)
namespace b200 {
namespace {
constexpr int kMaxWaitSetters = 64;
b200_wait_setter_t g_wait_setters[kMaxWaitSetters];     // zero-initialised before any dynamic initialiser runs
int g_num_wait_setters = 0;
}  // namespace

int b200_register_wait_setter(b200_wait_setter_t fn) {
  if (g_num_wait_setters < kMaxWaitSetters) g_wait_setters[g_num_wait_setters++] = fn;
  return g_num_wait_setters;
}
}  // namespace b200

// Sets, for the current device, how long any in-kernel wait (mbarrier, peer flag) may last before
// the kernel gives up, records B200_TIMEOUT in its status word and returns.  cycles <= 0 restores
// the default.  Returns 0 or the first CUDA error.
B200_API int b200_set_wait_budget_cycles(long long cycles) {
  if (cycles <= 0) cycles = B200_WAIT_CYCLES_DEFAULT;
  for (int i = 0; i < b200::g_num_wait_setters; i++) {
    const int rc = b200::g_wait_setters[i](cycles);
    if (rc) return rc;
  }
  return 0;
}
