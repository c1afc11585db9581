// LoRA gather-matvec kernels.
//   shrink: v[t, j]   = scale * sum_k A[slot(t), j, k] * x[t, k]          (j < R rows of the stacked A)
//   expand: y[t, off + n] += sum_j B[slot(t), n, j] * v[t, v_off + j]      (n < N)
// bgmv takes one adapter slot per token (decode batches); sgmv takes segments of consecutive
// tokens that share a slot (prefill) and reuses each adapter row across a tile of tokens.
// slot < 0 means "no adapter": the token is skipped.  Same op set as the reference's
// bgmv_shrink / bgmv_expand / sgmv_shrink / sgmv_expand (csrc/kernels/bgmv_shrink.cpp,
// bgmv_expand.cpp, sgmv_shrink.cpp, sgmv_expand.cpp; Python side lora/lora_ops.py:19-122).
#include "common.cuh"
#include <cuda_bf16.h>

namespace b200 {

__device__ __forceinline__ float dot8(const uint4& a, const uint4& b) {
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
    s = fmaf(fa.x, fb.x, s);
    s = fmaf(fa.y, fb.y, s);
  }
  return s;
}

// grid (T, ceil(R / 8)); block 256 = 8 warps, one adapter row per warp.
__global__ void bgmv_shrink_kernel(const __nv_bfloat16* __restrict__ x, long x_stride,
                                   const __nv_bfloat16* __restrict__ A, long a_slot_stride,
                                   const int* __restrict__ slots, float* __restrict__ v,
                                   int v_stride, int R, int K, float scale, int num_slots,
                                   int* status) {
  const int t = blockIdx.x;
  const int slot = slots[t];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.y * 8 + warp;
  if (j >= R) return;
  if (slot < 0) { if (lane == 0) v[(long)t * v_stride + j] = 0.f; return; }
  if (slot >= num_slots) { if (lane == 0 && status) atomicExch(status, B200_BAD_INDEX); return; }
  const uint4* xr = reinterpret_cast<const uint4*>(x + (long)t * x_stride);
  const uint4* ar = reinterpret_cast<const uint4*>(A + (long)slot * a_slot_stride + (long)j * K);
  float s = 0.f;
  for (int k = lane; k < (K >> 3); k += 32) s += dot8(ar[k], xr[k]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) v[(long)t * v_stride + j] = s * scale;
}

// grid (T, ceil(N / 256)); one output column per thread, R <= 128 values of B per thread.
__global__ void bgmv_expand_kernel(const float* __restrict__ v, int v_stride, int v_off,
                                   const __nv_bfloat16* __restrict__ B, long b_slot_stride,
                                   const int* __restrict__ slots, __nv_bfloat16* __restrict__ y,
                                   long y_stride, int y_off, int N, int R, int num_slots,
                                   int add, int* status) {
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  if (slot >= num_slots) { if (threadIdx.x == 0 && status) atomicExch(status, B200_BAD_INDEX); return; }
  __shared__ float sv[128];
  for (int j = threadIdx.x; j < R; j += blockDim.x) sv[j] = v[(long)t * v_stride + v_off + j];
  __syncthreads();
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  if (n >= N) return;
  const uint4* br = reinterpret_cast<const uint4*>(B + (long)slot * b_slot_stride + (long)n * R);
  float s = 0.f;
  for (int j8 = 0; j8 < (R >> 3); ++j8) {
    const uint4 w = br[j8];
    const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(pw[i]);
      s = fmaf(f.x, sv[j8 * 8 + 2 * i], s);
      s = fmaf(f.y, sv[j8 * 8 + 2 * i + 1], s);
    }
  }
  __nv_bfloat16* out = y + (long)t * y_stride + y_off + n;
  *out = __float2bfloat16(add ? __bfloat162float(*out) + s : s);
}

constexpr int SG_TOK = 8;   // tokens per tile

// grid (num_tiles, ceil(R / 8)); tile_seg/tile_tok0 give each tile's segment and first token.
__global__ void sgmv_shrink_kernel(const __nv_bfloat16* __restrict__ x, long x_stride,
                                   const __nv_bfloat16* __restrict__ A, long a_slot_stride,
                                   const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                                   const int* __restrict__ seg_slot, const int* __restrict__ tile_seg,
                                   const int* __restrict__ tile_tok0, float* __restrict__ v,
                                   int v_stride, int R, int K, float scale, int num_slots,
                                   int* status) {
  const int seg = tile_seg[blockIdx.x];
  const int slot = seg_slot[seg];
  const int t0 = tile_tok0[blockIdx.x];
  const int nt = min(SG_TOK, seg_start[seg] + seg_len[seg] - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.y * 8 + warp;
  if (j >= R || nt <= 0) return;
  if (slot < 0) {
    if (lane < nt) v[(long)(t0 + lane) * v_stride + j] = 0.f;
    return;
  }
  if (slot >= num_slots) { if (lane == 0 && status) atomicExch(status, B200_BAD_INDEX); return; }
  const uint4* ar = reinterpret_cast<const uint4*>(A + (long)slot * a_slot_stride + (long)j * K);
  float s[SG_TOK];
#pragma unroll
  for (int i = 0; i < SG_TOK; ++i) s[i] = 0.f;
  for (int k = lane; k < (K >> 3); k += 32) {
    const uint4 a = ar[k];
#pragma unroll
    for (int i = 0; i < SG_TOK; ++i)
      if (i < nt) s[i] += dot8(a, reinterpret_cast<const uint4*>(x + (long)(t0 + i) * x_stride)[k]);
  }
#pragma unroll
  for (int i = 0; i < SG_TOK; ++i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s[i] += __shfl_xor_sync(0xffffffffu, s[i], o);
    if (lane == 0 && i < nt) v[(long)(t0 + i) * v_stride + j] = s[i] * scale;
  }
}

// grid (num_tiles, ceil(N / 256))
__global__ void sgmv_expand_kernel(const float* __restrict__ v, int v_stride, int v_off,
                                   const __nv_bfloat16* __restrict__ B, long b_slot_stride,
                                   const int* __restrict__ seg_start, const int* __restrict__ seg_len,
                                   const int* __restrict__ seg_slot, const int* __restrict__ tile_seg,
                                   const int* __restrict__ tile_tok0, __nv_bfloat16* __restrict__ y,
                                   long y_stride, int y_off, int N, int R, int num_slots, int add,
                                   int* status) {
  const int seg = tile_seg[blockIdx.x];
  const int slot = seg_slot[seg];
  if (slot < 0) return;
  if (slot >= num_slots) { if (threadIdx.x == 0 && status) atomicExch(status, B200_BAD_INDEX); return; }
  const int t0 = tile_tok0[blockIdx.x];
  const int nt = min(SG_TOK, seg_start[seg] + seg_len[seg] - t0);
  __shared__ float sv[SG_TOK][128];
  for (int i = threadIdx.x; i < nt * R; i += blockDim.x)
    sv[i / R][i % R] = v[(long)(t0 + i / R) * v_stride + v_off + i % R];
  __syncthreads();
  const int n = blockIdx.y * blockDim.x + threadIdx.x;
  if (n >= N || nt <= 0) return;
  const uint4* br = reinterpret_cast<const uint4*>(B + (long)slot * b_slot_stride + (long)n * R);
  float s[SG_TOK];
#pragma unroll
  for (int i = 0; i < SG_TOK; ++i) s[i] = 0.f;
  for (int j8 = 0; j8 < (R >> 3); ++j8) {
    const uint4 w = br[j8];
    const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = __bfloat1622float2(pw[q]);
#pragma unroll
      for (int i = 0; i < SG_TOK; ++i) {
        s[i] = fmaf(f.x, sv[i][j8 * 8 + 2 * q], s[i]);
        s[i] = fmaf(f.y, sv[i][j8 * 8 + 2 * q + 1], s[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < SG_TOK; ++i) {
    if (i < nt) {
      __nv_bfloat16* out = y + (long)(t0 + i) * y_stride + y_off + n;
      *out = __float2bfloat16(add ? __bfloat162float(*out) + s[i] : s[i]);
    }
  }
}

}  // namespace b200

using namespace b200;

static int lora_check(int R, int K_or_N, bool shrink) {
  if (R <= 0 || R > 128 * 8) return 9300;             // stacked rows (slices * rank) for shrink
  if (shrink && (K_or_N & 7)) return 9301;            // 16-byte rows
  if (!shrink && ((R & 7) || R > 128)) return 9302;   // expand keeps one rank vector in smem
  return 0;
}

B200_API int b200_bgmv_shrink(const void* x, long x_stride, const void* A, long a_slot_stride,
                              const void* slots, void* v, int v_stride, int T, int R, int K,
                              float scale, int num_slots, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (int e = lora_check(R, K, true)) return e;
  bgmv_shrink_kernel<<<dim3(T, (R + 7) / 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)A, a_slot_stride, (const int*)slots,
      (float*)v, v_stride, R, K, scale, num_slots, status);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_bgmv_expand(const void* v, int v_stride, int v_off, const void* B,
                              long b_slot_stride, const void* slots, void* y, long y_stride,
                              int y_off, int T, int N, int R, int num_slots, int add, int* status,
                              cudaStream_t stream) {
  if (T <= 0 || N <= 0) return 0;
  if (int e = lora_check(R, N, false)) return e;
  bgmv_expand_kernel<<<dim3(T, (N + 255) / 256), 256, 0, stream>>>(
      (const float*)v, v_stride, v_off, (const __nv_bfloat16*)B, b_slot_stride, (const int*)slots,
      (__nv_bfloat16*)y, y_stride, y_off, N, R, num_slots, add, status);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_sgmv_shrink(const void* x, long x_stride, const void* A, long a_slot_stride,
                              const void* seg_start, const void* seg_len, const void* seg_slot,
                              const void* tile_seg, const void* tile_tok0, int num_tiles, void* v,
                              int v_stride, int R, int K, float scale, int num_slots, int* status,
                              cudaStream_t stream) {
  if (num_tiles <= 0) return 0;
  if (int e = lora_check(R, K, true)) return e;
  sgmv_shrink_kernel<<<dim3(num_tiles, (R + 7) / 8), 256, 0, stream>>>(
      (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)A, a_slot_stride,
      (const int*)seg_start, (const int*)seg_len, (const int*)seg_slot, (const int*)tile_seg,
      (const int*)tile_tok0, (float*)v, v_stride, R, K, scale, num_slots, status);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_sgmv_expand(const void* v, int v_stride, int v_off, const void* B,
                              long b_slot_stride, const void* seg_start, const void* seg_len,
                              const void* seg_slot, const void* tile_seg, const void* tile_tok0,
                              int num_tiles, void* y, long y_stride, int y_off, int N, int R,
                              int num_slots, int add, int* status, cudaStream_t stream) {
  if (num_tiles <= 0 || N <= 0) return 0;
  if (int e = lora_check(R, N, false)) return e;
  sgmv_expand_kernel<<<dim3(num_tiles, (N + 255) / 256), 256, 0, stream>>>(
      (const float*)v, v_stride, v_off, (const __nv_bfloat16*)B, b_slot_stride,
      (const int*)seg_start, (const int*)seg_len, (const int*)seg_slot, (const int*)tile_seg,
      (const int*)tile_tok0, (__nv_bfloat16*)y, y_stride, y_off, N, R, num_slots, add, status);
  return B200_CHECK_LAUNCH();
}
