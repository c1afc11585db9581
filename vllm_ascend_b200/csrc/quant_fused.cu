// Producers of block-scaled fp8 activations fused with the op in front of the GEMM:
//   add + RMSNorm  -> e4m3 values + one fp32 scale per 128 columns   (and the updated residual)
//   SiLU(gate)*up  -> e4m3 values + one fp32 scale per 128 columns
// They replace norm -> quant and activation -> quant pairs, saving one bf16 round trip of the
// activations through HBM each.  Same fusions as the reference's rms_norm_dynamic_quant and
// dequant_swiglu_quant / swiglu_group_quant ops (csrc/attention/rms_norm_dynamic_quant,
// csrc/moe/swiglu_group_quant), with 1x128 group scales instead of per-token scales.
// Values are rounded to bf16 before quantisation, exactly as the unfused sequence does.
#include "common.cuh"
#include <cuda_bf16.h>
#include <cuda_fp8.h>

namespace b200 {

// amax over the 16 lanes that share one 128-column group (lanes 16g .. 16g+15)
__device__ __forceinline__ float group16_max(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint2 quant8(const float* v, float inv) {
  __nv_fp8_e4m3 o[8];
#pragma unroll
  for (int j = 0; j < 8; j++) o[j] = __nv_fp8_e4m3(v[j] * inv);
  return *reinterpret_cast<uint2*>(o);
}

template <int VEC_PER_THREAD>
__global__ void rms_norm_quant_fp8_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* res,
                                          const __nv_bfloat16* __restrict__ w,
                                          __nv_fp8_e4m3* __restrict__ q, float* __restrict__ scales,
                                          int H, float eps, int gemma, long x_stride) {
  const long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
  uint4* rr = res ? reinterpret_cast<uint4*>(res + row * (long)H) : nullptr;
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const int nvec = H >> 3;
  float vals[VEC_PER_THREAD][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; i++) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      uint4 a = xr[v];
      uint32_t aw[4] = {a.x, a.y, a.z, a.w};
      if (rr) {
        uint4 b = rr[v];
        uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float2 fa = unpack_bf16x2(aw[j]), fb = unpack_bf16x2(bw[j]);
          aw[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
        }
        rr[v] = make_uint4(aw[0], aw[1], aw[2], aw[3]);
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 f = unpack_bf16x2(aw[j]);
        vals[i][2 * j] = f.x;
        vals[i][2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) vals[i][j] = 0.f;
    }
  }
  __shared__ float red[32];
  ss = warp_reduce_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
    t = warp_reduce_sum(t);
    if (threadIdx.x == 0) red[0] = rsqrtf(t / (float)H + eps);
  }
  __syncthreads();
  const float inv_rms = red[0];
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; i++) {
    const int v = threadIdx.x + i * blockDim.x;       // uniform per 16-lane group: blockDim % 32 == 0
    float y[8];
    float amax = 0.f;
    if (v < nvec) {
      uint4 ww = wr[v];
      uint32_t w4[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 fw = unpack_bf16x2(w4[j]);
        if (gemma) { fw.x += 1.f; fw.y += 1.f; }
        const float2 r = unpack_bf16x2(pack_bf16x2(vals[i][2 * j] * inv_rms * fw.x,
                                                    vals[i][2 * j + 1] * inv_rms * fw.y));
        y[2 * j] = r.x;
        y[2 * j + 1] = r.y;
        amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
      }
    }
    amax = group16_max(amax);
    if (v < nvec) {
      const float scale = fmaxf(amax, 1e-10f) / 448.f;
      reinterpret_cast<uint2*>(q + row * (long)H)[v] = quant8(y, 1.f / scale);
      if ((v & 15) == 0) scales[row * (long)(H >> 7) + (v >> 4)] = scale;
    }
  }
}

// x [T, 2I] (gate | up) -> q [T, I] e4m3, scales [T, I/128]
__global__ void silu_mul_quant_fp8_kernel(const __nv_bfloat16* __restrict__ x,
                                          __nv_fp8_e4m3* __restrict__ q, float* __restrict__ scales,
                                          int I, float limit) {
  const long row = blockIdx.x;
  const uint4* g = reinterpret_cast<const uint4*>(x + row * 2L * I);
  const uint4* u = reinterpret_cast<const uint4*>(x + row * 2L * I + I);
  const int nvec = I >> 3;
  for (int v0 = 0; v0 < nvec; v0 += blockDim.x) {
    const int v = v0 + threadIdx.x;
    float y[8];
    float amax = 0.f;
    if (v < nvec) {
      const uint4 a = g[v], b = u[v];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 fg = unpack_bf16x2(aw[j]), fu = unpack_bf16x2(bw[j]);
        if (limit > 0.f) {
          fg.x = fminf(fg.x, limit); fg.y = fminf(fg.y, limit);
          fu.x = fminf(fmaxf(fu.x, -limit), limit); fu.y = fminf(fmaxf(fu.y, -limit), limit);
        }
        const float2 r = unpack_bf16x2(pack_bf16x2(fg.x / (1.f + __expf(-fg.x)) * fu.x,
                                                    fg.y / (1.f + __expf(-fg.y)) * fu.y));
        y[2 * j] = r.x;
        y[2 * j + 1] = r.y;
        amax = fmaxf(amax, fmaxf(fabsf(r.x), fabsf(r.y)));
      }
    }
    amax = group16_max(amax);
    if (v < nvec) {
      const float scale = fmaxf(amax, 1e-10f) / 448.f;
      reinterpret_cast<uint2*>(q + row * (long)I)[v] = quant8(y, 1.f / scale);
      if ((v & 15) == 0) scales[row * (long)(I >> 7) + (v >> 4)] = scale;
    }
  }
}

}  // namespace b200

using namespace b200;

// H multiple of 128.  residual (may be null) is updated in place with x + residual.
B200_API int b200_rms_norm_quant_fp8(const void* x, void* residual, const void* w, void* q,
                                     void* scales, long T, int H, float eps, int gemma,
                                     long x_stride, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 128) return 9100;
  const int nvec = H >> 3;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  const int per = (nvec + threads - 1) / threads;
#define LAUNCH_RNQ(V)                                                                        \
  rms_norm_quant_fp8_kernel<V><<<(unsigned)T, threads, 0, stream>>>(                           \
      (const __nv_bfloat16*)x, (__nv_bfloat16*)residual, (const __nv_bfloat16*)w,             \
      (__nv_fp8_e4m3*)q, (float*)scales, H, eps, gemma, x_stride)
  if (per <= 1) LAUNCH_RNQ(1);
  else if (per <= 2) LAUNCH_RNQ(2);
  else if (per <= 4) LAUNCH_RNQ(4);
  else return 9101;
#undef LAUNCH_RNQ
  return B200_CHECK_LAUNCH();
}

B200_API int b200_silu_mul_quant_fp8(const void* x, void* q, void* scales, long T, int I, float limit,
                                     cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I % 128) return 9100;
  int threads = ((I >> 3) + 31) / 32 * 32;
  if (threads > 512) threads = 512;
  silu_mul_quant_fp8_kernel<<<(unsigned)T, threads, 0, stream>>>(
      (const __nv_bfloat16*)x, (__nv_fp8_e4m3*)q, (float*)scales, I, limit);
  return B200_CHECK_LAUNCH();
}
