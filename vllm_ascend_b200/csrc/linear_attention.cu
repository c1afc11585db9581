// Linear-attention building blocks of Gated DeltaNet layers (Qwen3-Next style hybrids):
//   causal_conv1d     depthwise short convolution over the token axis of variable-length
//                     sequences with a per-sequence state of the last K-1 inputs, + SiLU
//   gated_delta_rule  the recurrence  S <- S * exp(g_t);  d = beta_t * (v_t - S^T k_t);
//                     S <- S + k_t d^T;  o_t = S^T q_t   with S in registers (one thread per
//                     value column), for prefill chunks and single-token decode alike
// Counterparts of the reference's causal_conv1d and recurrent / chunked gated-delta-rule ops
// (csrc/moe/causal_conv1d*, csrc/attention/recurrent_gated_delta_rule*, ops/triton/fla/*).
#include "common.cuh"
#include <cuda_bf16.h>

namespace b200 {

// x [T, C] bf16 (row stride x_stride) -> y [T, C]; weight [C, K] bf16; bias [C] or null.
// state [slots, K-1, C] bf16: the last K-1 inputs of the sequence, read when has_init[b],
// always written back.  One thread per channel, sequential over the sequence's tokens.
template <int K>
__global__ void causal_conv1d_kernel(const __nv_bfloat16* __restrict__ x, long x_stride,
                                     const __nv_bfloat16* __restrict__ w,
                                     const __nv_bfloat16* __restrict__ bias,
                                     __nv_bfloat16* __restrict__ state, const int* __restrict__ cu,
                                     const int* __restrict__ slots, const int* __restrict__ has_init,
                                     __nv_bfloat16* __restrict__ y, long y_stride, int C, int act,
                                     long num_slots, int* status) {
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int t0 = cu[b], t1 = cu[b + 1];
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (status) atomicExch(status, B200_BAD_INDEX);
    return;
  }
  float wk[K];
#pragma unroll
  for (int j = 0; j < K; j++) wk[j] = __bfloat162float(w[(long)c * K + j]);
  const float bs = bias ? __bfloat162float(bias[c]) : 0.f;
  __nv_bfloat16* st = state + (long)slot * (K - 1) * C + c;
  float hist[K];      // hist[K-1] is the current input
#pragma unroll
  for (int j = 0; j < K - 1; j++) hist[j] = has_init[b] ? __bfloat162float(st[(long)j * C]) : 0.f;
  for (int t = t0; t < t1; t++) {
    hist[K - 1] = __bfloat162float(x[(long)t * x_stride + c]);
    float acc = bs;
#pragma unroll
    for (int j = 0; j < K; j++) acc = fmaf(wk[j], hist[j], acc);
    if (act) acc = acc / (1.f + __expf(-acc));
    y[(long)t * y_stride + c] = __float2bfloat16(acc);
#pragma unroll
    for (int j = 0; j < K - 1; j++) hist[j] = hist[j + 1];
  }
#pragma unroll
  for (int j = 0; j < K - 1; j++) st[(long)j * C] = __float2bfloat16(hist[j]);
}

// q, k [T, Hk, DK], v [T, Hv, DV] bf16 (token strides given), g, beta [T, Hv] fp32,
// state [slots, Hv, DK, DV] fp32, out [T, Hv, DV] bf16.  Hv % Hk == 0 (value heads share keys).
// Block = (sequence, value head), DV threads; thread j owns column j of S (DK registers).
template <int DK, int DV>
__global__ void __launch_bounds__(DV)
gated_delta_rule_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                        const __nv_bfloat16* __restrict__ v, long qk_stride, long v_stride,
                        const float* __restrict__ g, const float* __restrict__ beta,
                        float* __restrict__ state, const int* __restrict__ cu,
                        const int* __restrict__ slots, const int* __restrict__ has_init,
                        __nv_bfloat16* __restrict__ out, long out_stride, int Hk, int Hv,
                        float scale, int l2norm, long num_slots, int* status) {
  const int b = blockIdx.x, hv = blockIdx.y;
  const int hk = hv / (Hv / Hk);
  const int j = threadIdx.x;
  const int slot = slots[b];
  if (slot < 0 || slot >= num_slots) {
    if (j == 0 && status) atomicExch(status, B200_BAD_INDEX);
    return;
  }
  __shared__ float ks[DK], qs[DK];
  __shared__ float red[2][DV / 32];
  float S[DK];
  float* sp = state + (((long)slot * Hv + hv) * DK) * DV + j;
  if (has_init[b]) {
#pragma unroll
    for (int i = 0; i < DK; i++) S[i] = sp[(long)i * DV];
  } else {
#pragma unroll
    for (int i = 0; i < DK; i++) S[i] = 0.f;
  }
  const int t0 = cu[b], t1 = cu[b + 1];
  // inputs of token t + 1 are fetched while token t is processed: the recurrence is sequential,
  // so the global-load latency would otherwise sit on every step
  float n_k = 0.f, n_q = 0.f, n_v = 0.f, n_g = 0.f, n_b = 0.f;
  auto fetch = [&](int t) {
    if (j < DK) {
      n_k = __bfloat162float(k[(long)t * qk_stride + (long)hk * DK + j]);
      n_q = __bfloat162float(q[(long)t * qk_stride + (long)hk * DK + j]);
    }
    n_v = __bfloat162float(v[(long)t * v_stride + (long)hv * DV + j]);
    n_g = g[(long)t * Hv + hv];
    n_b = beta[(long)t * Hv + hv];
  };
  if (t0 < t1) fetch(t0);
  for (int t = t0; t < t1; t++) {
    float kval = n_k, qval = n_q;
    const float vt = n_v, decay = __expf(n_g), bt = n_b;
    if (t + 1 < t1) fetch(t + 1);
    __syncthreads();                    // previous token's reads of ks / qs are done
    // DV >= DK: the first DK threads stage k_t and q_t (optionally L2-normalised)
    float kq = kval * kval, qq = qval * qval;
    if (l2norm) {
      kq = warp_reduce_sum(kq);
      qq = warp_reduce_sum(qq);
      if ((j & 31) == 0) { red[0][j >> 5] = kq; red[1][j >> 5] = qq; }
      __syncthreads();
      float ksum = 0.f, qsum = 0.f;
#pragma unroll
      for (int w = 0; w < DV / 32; w++) { ksum += red[0][w]; qsum += red[1][w]; }
      kval *= rsqrtf(ksum + 1e-6f);
      qval *= rsqrtf(qsum + 1e-6f);
    }
    if (j < DK) {
      ks[j] = kval;
      qs[j] = qval * scale;
    }
    __syncthreads();
    float mem = 0.f;
#pragma unroll
    for (int i = 0; i < DK; i++) {
      S[i] *= decay;
      mem = fmaf(S[i], ks[i], mem);
    }
    const float delta = (vt - mem) * bt;
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DK; i++) {
      S[i] = fmaf(ks[i], delta, S[i]);
      o = fmaf(S[i], qs[i], o);
    }
    out[(long)t * out_stride + (long)hv * DV + j] = __float2bfloat16(o);
  }
#pragma unroll
  for (int i = 0; i < DK; i++) sp[(long)i * DV] = S[i];
}

}  // namespace b200

using namespace b200;

// cu: int32 [B + 1] token offsets, slots: int32 [B] state rows, has_init: int32 [B].
B200_API int b200_causal_conv1d(const void* x, long x_stride, const void* w, const void* bias, void* state,
                                const void* cu, const void* slots, const void* has_init, void* y,
                                long y_stride, int B, int C, int K, int act, long num_slots, int* status,
                                cudaStream_t stream) {
  if (B <= 0 || C <= 0) return 0;
  dim3 grid((unsigned)((C + 127) / 128), (unsigned)B);
#define LAUNCH_CONV(KK)                                                                             \
  causal_conv1d_kernel<KK><<<grid, 128, 0, stream>>>(                                               \
      (const __nv_bfloat16*)x, x_stride, (const __nv_bfloat16*)w, (const __nv_bfloat16*)bias,       \
      (__nv_bfloat16*)state, (const int*)cu, (const int*)slots, (const int*)has_init,               \
      (__nv_bfloat16*)y, y_stride, C, act, num_slots, status)
  if (K == 4) LAUNCH_CONV(4);
  else if (K == 3) LAUNCH_CONV(3);
  else if (K == 2) LAUNCH_CONV(2);
  else return 9800;
#undef LAUNCH_CONV
  return B200_CHECK_LAUNCH();
}

B200_API int b200_gated_delta_rule(const void* q, const void* k, const void* v, long qk_stride,
                                   long v_stride, const void* g, const void* beta, void* state,
                                   const void* cu, const void* slots, const void* has_init, void* out,
                                   long out_stride, int B, int Hk, int Hv, int DK, int DV, float scale,
                                   int l2norm, long num_slots, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (Hk <= 0 || Hv % Hk) return 9801;
  dim3 grid((unsigned)B, (unsigned)Hv);
#define LAUNCH_GDR(A, Bv)                                                                           \
  gated_delta_rule_kernel<A, Bv><<<grid, Bv, 0, stream>>>(                                          \
      (const __nv_bfloat16*)q, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, qk_stride, v_stride, \
      (const float*)g, (const float*)beta, (float*)state, (const int*)cu, (const int*)slots,        \
      (const int*)has_init, (__nv_bfloat16*)out, out_stride, Hk, Hv, scale, l2norm, num_slots, status)
  if (DK == 128 && DV == 128) LAUNCH_GDR(128, 128);
  else if (DK == 64 && DV == 64) LAUNCH_GDR(64, 64);
  else if (DK == 64 && DV == 128) LAUNCH_GDR(64, 128);
  else if (DK == 32 && DV == 32) LAUNCH_GDR(32, 32);
  else return 9802;
#undef LAUNCH_GDR
  return B200_CHECK_LAUNCH();
}
