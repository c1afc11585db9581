// Small device-side bookkeeping ops: slot mapping from block tables, kernel-block expansion of a
// block table, token-id histogram, row scatter by N-d index, sign-bit packing.
//
// These run once per step next to much larger kernels; what matters is that they run on the device
// in stream order (inside CUDA graphs, without a host round trip), not their bandwidth.
#include "common.cuh"

namespace b200 {

// slot[t] = block_table[req[t], pos[t] / block_size] * block_size + pos[t] % block_size.
// Tokens with req < 0 (padding of a captured graph) get slot -1, which the KV-write kernels skip.
// A position beyond the table or a block id outside [0, num_blocks) records B200_BAD_INDEX and
// yields -1 instead of an address (the reference computes the mapping with a device kernel per
// KV group, vllm_ascend/worker/block_table.py:28-358).
__global__ void slot_mapping_kernel(const int* __restrict__ block_table, long table_stride,
                                    int max_blocks_per_req, const int* __restrict__ req,
                                    const long* __restrict__ pos, int num_tokens, int block_size,
                                    long num_blocks, long* __restrict__ slots, int* status) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= num_tokens) return;
  const int r = req[t];
  if (r < 0) { slots[t] = -1; return; }
  const long p = pos[t];
  const long bi = p / block_size;
  if (p < 0 || bi >= max_blocks_per_req) {
    if (status) atomicCAS(status, 0, B200_BAD_INDEX);
    slots[t] = -1;
    return;
  }
  const long b = block_table[(long)r * table_stride + bi];
  if (b < 0 || b >= num_blocks) {
    if (status) atomicCAS(status, 0, B200_BAD_INDEX);
    slots[t] = -1;
    return;
  }
  slots[t] = b * block_size + (p - bi * block_size);
}

// A KV group whose memory-manager block holds `ratio` attention-kernel blocks (hybrid models:
// the manager's block is sized so that every group's page has the same byte size, the attention
// kernel keeps its own page length): out[r, i * ratio + j] = in[r, i] * ratio + j.
__global__ void expand_block_table_kernel(const int* __restrict__ in, long in_stride,
                                          int* __restrict__ out, long out_stride, int num_reqs,
                                          int blocks_per_req, int ratio) {
  const long n = (long)num_reqs * blocks_per_req * ratio;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const int j = (int)(i % ratio);
    const long bi = (i / ratio) % blocks_per_req;
    const long r = i / ((long)ratio * blocks_per_req);
    const int b = in[r * in_stride + bi];
    out[r * out_stride + bi * ratio + j] = b < 0 ? -1 : b * ratio + j;
  }
}

// counts[row[t], id[t]] += 1 (counts int32 [rows, vocab]); ids outside [0, vocab) are skipped.
// Used for the output-token histograms of the frequency / presence penalties
// (vllm_ascend/ops/triton/penalty.py:35-139 takes precomputed bin counts).
__global__ void bincount_kernel(const long* __restrict__ ids, const int* __restrict__ rows, long n,
                                int* __restrict__ counts, int num_rows, int vocab) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long v = ids[i];
    const int r = rows ? rows[i] : 0;
    if (v < 0 || v >= vocab || r < 0 || r >= num_rows) continue;
    atomicAdd(&counts[(long)r * vocab + v], 1);
  }
}

// var[idx[i, 0], ..., idx[i, k-1], :] = upd[i, :] with the trailing `row_bytes` bytes as one row.
// dims: the k leading extents of var.  Rows whose index falls outside are skipped and recorded.
// Duplicate indices: one of the writers wins (as in the reference's op,
// csrc/moe/scatter_nd_update_v2/op_kernel/scatter_nd_update_v2.cpp).
struct ScatterDims { long d[4]; };

__global__ void scatter_nd_update_kernel(uint8_t* __restrict__ var, const long* __restrict__ idx,
                                         const uint8_t* __restrict__ upd, long n, int k,
                                         ScatterDims dims, long row_bytes, int* status) {
  const long i = blockIdx.x;
  if (i >= n) return;
  long lin = 0;
  bool ok = true;
  for (int a = 0; a < k; a++) {
    const long v = idx[i * k + a];
    ok = ok && v >= 0 && v < dims.d[a];
    lin = lin * dims.d[a] + v;
  }
  if (!ok) {
    if (status && threadIdx.x == 0) atomicCAS(status, 0, B200_BAD_INDEX);
    return;
  }
  uint8_t* dst = var + lin * row_bytes;
  const uint8_t* src = upd + i * row_bytes;
  if (((row_bytes | (long)(uintptr_t)dst | (long)(uintptr_t)src) & 15) == 0) {
    for (long j = threadIdx.x; j < (row_bytes >> 4); j += blockDim.x)
      reinterpret_cast<uint4*>(dst)[j] = reinterpret_cast<const uint4*>(src)[j];
  } else {
    for (long j = threadIdx.x; j < row_bytes; j += blockDim.x) dst[j] = src[j];
  }
}

// out[j] bit b = sign bit of x[8 j + b] (first element in the lowest bit); n multiple of 8 is not
// required: missing elements read as positive.  T is a 16- or 32-bit float pattern.
template <typename T>
__global__ void sign_bits_pack_kernel(const T* __restrict__ x, long n, uint8_t* __restrict__ out) {
  const long nb = (n + 7) >> 3;
  constexpr int SHIFT = sizeof(T) * 8 - 1;
  for (long j = blockIdx.x * (long)blockDim.x + threadIdx.x; j < nb; j += (long)gridDim.x * blockDim.x) {
    unsigned byte = 0;
#pragma unroll
    for (int b = 0; b < 8; b++) {
      const long e = j * 8 + b;
      if (e < n) byte |= (unsigned)((x[e] >> SHIFT) & 1) << b;
    }
    out[j] = (uint8_t)byte;
  }
}

// y[e] = bit ? -1 : +1 scaled by `scale` (bf16 or fp32 output).
template <typename T>
__global__ void sign_bits_unpack_kernel(const uint8_t* __restrict__ in, long n, float scale,
                                        T* __restrict__ y) {
  for (long e = blockIdx.x * (long)blockDim.x + threadIdx.x; e < n; e += (long)gridDim.x * blockDim.x) {
    const float v = ((in[e >> 3] >> (e & 7)) & 1) ? -scale : scale;
    if constexpr (sizeof(T) == 2) y[e] = __float2bfloat16(v); else y[e] = v;
  }
}

static inline int grid_for(long n, int block = 256, int cap = 148 * 8) {
  long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace b200

using namespace b200;

B200_API int b200_slot_mapping(const void* block_table, long table_stride, int max_blocks_per_req,
                               const void* req, const void* pos, int num_tokens, int block_size,
                               long num_blocks, void* slots, int* status, cudaStream_t stream) {
  if (num_tokens <= 0) return 0;
  if (block_size <= 0) return 9300;
  slot_mapping_kernel<<<(num_tokens + 255) / 256, 256, 0, stream>>>(
      (const int*)block_table, table_stride, max_blocks_per_req, (const int*)req, (const long*)pos,
      num_tokens, block_size, num_blocks, (long*)slots, status);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_expand_block_table(const void* in, long in_stride, void* out, long out_stride,
                                     int num_reqs, int blocks_per_req, int ratio, cudaStream_t stream) {
  if (num_reqs <= 0 || blocks_per_req <= 0) return 0;
  if (ratio <= 0) return 9300;
  const long n = (long)num_reqs * blocks_per_req * ratio;
  expand_block_table_kernel<<<grid_for(n), 256, 0, stream>>>((const int*)in, in_stride, (int*)out,
                                                             out_stride, num_reqs, blocks_per_req, ratio);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_bincount(const void* ids, const void* rows, long n, void* counts, int num_rows,
                           int vocab, cudaStream_t stream) {
  if (n <= 0) return 0;
  bincount_kernel<<<grid_for(n), 256, 0, stream>>>((const long*)ids, (const int*)rows, n, (int*)counts,
                                                   num_rows, vocab);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_scatter_nd_update(void* var, const void* idx, const void* upd, long n, int k,
                                    const long* dims, long row_bytes, int* status, cudaStream_t stream) {
  if (n <= 0 || row_bytes <= 0) return 0;
  if (k < 1 || k > 4) return 9301;
  ScatterDims d;
  for (int a = 0; a < 4; a++) d.d[a] = a < k ? dims[a] : 1;
  scatter_nd_update_kernel<<<(unsigned)n, 128, 0, stream>>>((uint8_t*)var, (const long*)idx,
                                                            (const uint8_t*)upd, n, k, d, row_bytes, status);
  return B200_CHECK_LAUNCH();
}

// elem_bytes: 2 (bf16 / fp16) or 4 (fp32)
B200_API int b200_sign_bits_pack(const void* x, long n, int elem_bytes, void* out, cudaStream_t stream) {
  if (n <= 0) return 0;
  const long nb = (n + 7) >> 3;
  if (elem_bytes == 2)
    sign_bits_pack_kernel<uint16_t><<<grid_for(nb), 256, 0, stream>>>((const uint16_t*)x, n, (uint8_t*)out);
  else if (elem_bytes == 4)
    sign_bits_pack_kernel<uint32_t><<<grid_for(nb), 256, 0, stream>>>((const uint32_t*)x, n, (uint8_t*)out);
  else
    return 9302;
  return B200_CHECK_LAUNCH();
}

B200_API int b200_sign_bits_unpack(const void* in, long n, float scale, int out_elem_bytes, void* y,
                                   cudaStream_t stream) {
  if (n <= 0) return 0;
  if (out_elem_bytes == 2)
    sign_bits_unpack_kernel<__nv_bfloat16><<<grid_for(n), 256, 0, stream>>>((const uint8_t*)in, n, scale,
                                                                             (__nv_bfloat16*)y);
  else if (out_elem_bytes == 4)
    sign_bits_unpack_kernel<float><<<grid_for(n), 256, 0, stream>>>((const uint8_t*)in, n, scale, (float*)y);
  else
    return 9302;
  return B200_CHECK_LAUNCH();
}
