// MLA pre-processing of one step, fused: what lies between the down-projections and the attention
// kernel of a multi-head-latent-attention layer.
//
//   kv  [T, dc + dr]  (output of the joint KV down-projection)
//     latent = RMSNorm(kv[:, :dc]) * w          -> latent cache slot of the token (and an optional copy)
//     k_pe   = RoPE(kv[:, dc:])                  -> rope-key cache slot of the token (and an optional copy)
//   q   [T, H, dn + dr]
//     q[..., dn:] = RoPE(q[..., dn:])            in place
//
// RoPE is the interleaved (GPT-J) pairing (2j, 2j+1) of DeepSeek's rope slice, angles from a
// [max_pos, dr] fp32 table (cos in the first half of a row, sin in the second).  One CTA per
// token; values are computed in fp32 and rounded to bf16 once, like the separate norm / rope /
// scatter steps they replace.  Tokens with slot < 0 (padding, or tokens another rank stores) do the
// q rotation only.  The reference runs this stage as one fused op as well (csrc/mla_preprocess/,
// registered as npu_mla_process in csrc/torch_binding.cpp:1987-1997), there together with the
// projections.
#include "common.cuh"
#include <cuda_bf16.h>

namespace b200 {

struct MlaPreParams {
  __nv_bfloat16* q;
  long q_stride;           // elements between tokens
  int H, dn, dr;
  const __nv_bfloat16* kv;
  long kv_stride;
  int dc;
  const __nv_bfloat16* norm_w;
  float eps;
  const long* positions;
  const float* cos_sin;    // [max_pos, dr]
  long max_pos;
  const long* slot_mapping;
  __nv_bfloat16* lat_cache;   // [num_slots, dc]
  __nv_bfloat16* pe_cache;    // [num_slots, dr]
  long num_slots;
  __nv_bfloat16* latent_out;  // optional [T, dc]
  __nv_bfloat16* kpe_out;     // optional [T, dr]
  int* status;
};

__global__ void __launch_bounds__(256) mla_preprocess_kernel(const MlaPreParams p) {
  __shared__ float red[8];
  __shared__ float s_inv;
  const long t = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long pos = p.positions[t];
  bool bad = pos < 0 || pos >= p.max_pos;
  if (bad) pos = 0;
  long slot = p.slot_mapping ? p.slot_mapping[t] : -1;
  if (slot >= p.num_slots) {
    bad = true;
    slot = -1;
  }
  if (bad && tid == 0 && p.status) atomicCAS(p.status, 0, B200_BAD_INDEX);
  const float* cs = p.cos_sin + pos * (long)p.dr;
  const int half = p.dr >> 1;

  // ---- latent: RMSNorm over dc
  const __nv_bfloat16* kvrow = p.kv + t * p.kv_stride;
  const bool want_latent = slot >= 0 || p.latent_out != nullptr;
  if (want_latent) {
    float ss = 0.f;
    for (int i = tid; i < p.dc; i += blockDim.x) {
      const float v = __bfloat162float(kvrow[i]);
      ss += v * v;
    }
    ss = warp_reduce_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (warp == 0) {
      float v = lane < (int)(blockDim.x >> 5) ? red[lane] : 0.f;
      v = warp_reduce_sum(v);
      if (lane == 0) s_inv = rsqrtf(v / (float)p.dc + p.eps);
    }
    __syncthreads();
    const float inv = s_inv;
    for (int i = tid; i < p.dc; i += blockDim.x) {
      const __nv_bfloat16 o =
          __float2bfloat16(__bfloat162float(kvrow[i]) * inv * __bfloat162float(p.norm_w[i]));
      if (slot >= 0) p.lat_cache[slot * p.dc + i] = o;
      if (p.latent_out) p.latent_out[t * p.dc + i] = o;
    }
    // ---- rope key
    for (int j = tid; j < half; j += blockDim.x) {
      const float x1 = __bfloat162float(kvrow[p.dc + 2 * j]);
      const float x2 = __bfloat162float(kvrow[p.dc + 2 * j + 1]);
      const float c = cs[j], s = cs[half + j];
      const __nv_bfloat16 o1 = __float2bfloat16(x1 * c - x2 * s);
      const __nv_bfloat16 o2 = __float2bfloat16(x2 * c + x1 * s);
      if (slot >= 0) {
        p.pe_cache[slot * p.dr + 2 * j] = o1;
        p.pe_cache[slot * p.dr + 2 * j + 1] = o2;
      }
      if (p.kpe_out) {
        p.kpe_out[t * p.dr + 2 * j] = o1;
        p.kpe_out[t * p.dr + 2 * j + 1] = o2;
      }
    }
  }
  // ---- rope slice of every query head, in place (one bf16 pair = one 4-byte access)
  __nv_bfloat16* qrow = p.q + t * p.q_stride;
  const int D = p.dn + p.dr;
  const int pairs = p.H * half;
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int h = i / half, j = i - h * half;
    __nv_bfloat162* ptr = reinterpret_cast<__nv_bfloat162*>(qrow + (long)h * D + p.dn + 2 * j);
    const float2 x = __bfloat1622float2(*ptr);
    const float c = cs[j], s = cs[half + j];
    *ptr = __floats2bfloat162_rn(x.x * c - x.y * s, x.y * c + x.x * s);
  }
}

}  // namespace b200

using namespace b200;

// dn, dr, q_stride and the q base must keep every (head, pair) 4-byte aligned: dn and dr even,
// q_stride even.  kv_stride is free.  lat_cache / pe_cache: dense [num_slots, dc] / [num_slots, dr].
B200_API int b200_mla_preprocess(void* q, long q_stride, int T, int H, int dn, int dr, const void* kv,
                                 long kv_stride, int dc, const void* norm_w, float eps,
                                 const void* positions, const void* cos_sin, long max_pos,
                                 const void* slot_mapping, void* lat_cache, void* pe_cache,
                                 long num_slots, void* latent_out, void* kpe_out, int* status,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((dn & 1) || (dr & 1) || (q_stride & 1) || dr <= 0 || dc <= 0 || H <= 0) return 9400;
  if ((reinterpret_cast<uintptr_t>(q) & 3) != 0) return 9401;
  if (slot_mapping && (!lat_cache || !pe_cache)) return 9402;
  MlaPreParams p;
  p.q = (__nv_bfloat16*)q; p.q_stride = q_stride; p.H = H; p.dn = dn; p.dr = dr;
  p.kv = (const __nv_bfloat16*)kv; p.kv_stride = kv_stride; p.dc = dc;
  p.norm_w = (const __nv_bfloat16*)norm_w; p.eps = eps;
  p.positions = (const long*)positions; p.cos_sin = (const float*)cos_sin; p.max_pos = max_pos;
  p.slot_mapping = (const long*)slot_mapping;
  p.lat_cache = (__nv_bfloat16*)lat_cache; p.pe_cache = (__nv_bfloat16*)pe_cache;
  p.num_slots = num_slots;
  p.latent_out = (__nv_bfloat16*)latent_out; p.kpe_out = (__nv_bfloat16*)kpe_out;
  p.status = status;
  mla_preprocess_kernel<<<T, 256, 0, stream>>>(p);
  return B200_CHECK_LAUNCH();
}
