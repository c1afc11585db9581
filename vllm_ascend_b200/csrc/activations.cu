// Activation family beside SiLU-mul, and the gated RMSNorm:
//   act_and_mul : out = act(gate) * up for act in {gelu (erf), gelu (tanh), swiglu-oai}
//   act         : out = act(x) for act in {quick_gelu, gelu, gelu_tanh}
//   rms_norm_gated : out = rmsnorm(x) * w * silu(z)         (gate after the norm)
// The reference routes these through vendor ops and small Triton kernels
// (vllm_ascend/ops/activation.py:35-86, ops/layernorm.py:110-197).
#include "common.cuh"
#include <cuda_bf16.h>

namespace b200 {

enum : int { ACT_GELU = 1, ACT_GELU_TANH = 2, ACT_QUICK_GELU = 3, ACT_SWIGLU_OAI = 4 };

__device__ __forceinline__ float act_fn(float x, int kind) {
  switch (kind) {
    case ACT_GELU: return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
    case ACT_GELU_TANH: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.f + tanhf(u));
    }
    case ACT_QUICK_GELU: return x / (1.f + __expf(-1.702f * x));
    default: return x / (1.f + __expf(-x));
  }
}

// gated == 1: x is [T, 2I] (gate | up); else x is [T, I]
__global__ void act_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, long T,
                           int I, int kind, int gated, float alpha, float limit) {
  const int nvec = I >> 3;
  const long total = T * nvec;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long row = i / nvec;
    const int v = (int)(i - row * nvec);
    const long in_row = gated ? 2L * I : I;
    const uint4 a = reinterpret_cast<const uint4*>(x + row * in_row)[v];
    uint4 b = make_uint4(0, 0, 0, 0);
    if (gated) b = reinterpret_cast<const uint4*>(x + row * in_row + I)[v];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float2 fa = unpack_bf16x2(aw[j]);
      float r0, r1;
      if (kind == ACT_SWIGLU_OAI) {
        // gate clamped above, up clamped both ways; gate * sigmoid(alpha * gate) * (up + 1)
        float2 fu = unpack_bf16x2(bw[j]);
        fa.x = fminf(fa.x, limit); fa.y = fminf(fa.y, limit);
        fu.x = fminf(fmaxf(fu.x, -limit), limit); fu.y = fminf(fmaxf(fu.y, -limit), limit);
        r0 = fa.x / (1.f + __expf(-alpha * fa.x)) * (fu.x + 1.f);
        r1 = fa.y / (1.f + __expf(-alpha * fa.y)) * (fu.y + 1.f);
      } else {
        r0 = act_fn(fa.x, kind);
        r1 = act_fn(fa.y, kind);
        if (gated) {
          const float2 fu = unpack_bf16x2(bw[j]);
          r0 *= fu.x;
          r1 *= fu.y;
        }
      }
      o[j] = pack_bf16x2(r0, r1);
    }
    reinterpret_cast<uint4*>(out + row * (long)I)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// one warp per row group of `group` columns (group = H for a plain gated norm, or the per-head
// size when the norm is applied per head); H % group == 0, group % 8 == 0
__global__ void rms_norm_gated_kernel(const __nv_bfloat16* __restrict__ x,
                                      const __nv_bfloat16* __restrict__ z,
                                      const __nv_bfloat16* __restrict__ w,
                                      __nv_bfloat16* __restrict__ out, long rows, int group, float eps,
                                      int norm_before_gate) {
  const long r = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const __nv_bfloat16* xr = x + r * (long)group;
  const __nv_bfloat16* zr = z + r * (long)group;
  float ss = 0.f;
  for (int c = lane; c < group; c += 32) {
    float v = __bfloat162float(xr[c]);
    if (!norm_before_gate) {
      const float g = __bfloat162float(zr[c]);
      v *= g / (1.f + __expf(-g));
    }
    ss += v * v;
  }
  ss = warp_reduce_sum(ss);
  const float inv = rsqrtf(ss / (float)group + eps);
  for (int c = lane; c < group; c += 32) {
    float v = __bfloat162float(xr[c]);
    const float g = __bfloat162float(zr[c]);
    const float sg = g / (1.f + __expf(-g));
    if (!norm_before_gate) v *= sg;
    v = v * inv * __bfloat162float(w[c]);
    if (norm_before_gate) v *= sg;
    out[r * (long)group + c] = __float2bfloat16(v);
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_activation(const void* x, void* out, long T, int I, int kind, int gated, float alpha,
                             float limit, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I & 7) return 9100;
  if (kind < ACT_GELU || kind > ACT_SWIGLU_OAI || (kind == ACT_SWIGLU_OAI && !gated)) return 9600;
  const long total = T * (I >> 3);
  long blocks = (total + 255) / 256;
  const long cap = (long)num_sms() * 16;
  if (blocks > cap) blocks = cap;
  act_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, T, I, kind,
                                                   gated, alpha, limit);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_rms_norm_gated(const void* x, const void* z, const void* w, void* out, long rows,
                                 int group, float eps, int norm_before_gate, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (group <= 0) return 9100;
  const long blocks = (rows + 7) / 8;
  rms_norm_gated_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
      (const __nv_bfloat16*)x, (const __nv_bfloat16*)z, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, rows,
      group, eps, norm_before_gate);
  return B200_CHECK_LAUNCH();
}
