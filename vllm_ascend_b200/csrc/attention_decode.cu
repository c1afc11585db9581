// Paged GQA flash-decode on CUDA cores (one query token per sequence) with
// split-KV partials in caller-provided scratch, plus the split merge kernel that
// the tensor-core attention kernel shares.
//
// Semantics follow the reference's pure-decode path (_npu_paged_attention,
// vllm_ascend/attention/attention_v1.py:1555-1574): softmax(q k^T * scale) v over
// the first seq_len tokens of the sequence's block table.
//
// Scratch layout (fp32): partial_o [B, Hq, S, D] (each split normalised by its
// own sum), partial_lse [B, Hq, S] (natural-log sum-exp, -inf for empty splits).
#include "common.cuh"
#include "attention.h"

namespace b200 {

template <int D, int G>
__global__ void __launch_bounds__(128)
paged_decode_kernel(const __nv_bfloat16* __restrict__ q, long q_stride,
                    const __nv_bfloat16* __restrict__ k_cache,
                    const __nv_bfloat16* __restrict__ v_cache,
                    const int* __restrict__ block_table, int max_blocks,
                    const int* __restrict__ seq_lens, int block_size, int Hkv, float scale_log2,
                    int window, int num_splits, __nv_bfloat16* __restrict__ out, long out_stride,
                    float* __restrict__ partial_o, float* __restrict__ partial_lse,
                    long num_blocks_total, int* status) {
  constexpr int LPK = D / 8;        // lanes per key (16-byte loads)
  constexpr int KPI = 32 / LPK;     // keys per warp iteration
  constexpr int NGRP = 4 * KPI;     // independent accumulator groups in the CTA
  const int b = blockIdx.x, h = blockIdx.y, split = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK;       // which key of the iteration
  const int dl = lane % LPK;        // which 8-dim slice
  const int seq_len = seq_lens[b];
  int kv_begin = 0;
  if (window > 0 && seq_len > window) kv_begin = seq_len - window;
  const int span = seq_len - kv_begin;
  int per = (span + num_splits - 1) / num_splits;
  per = ((per + 31) / 32) * 32;
  const int k0 = kv_begin + split * per;
  const int k1 = min(seq_len, k0 + per);

  __shared__ float sm_m[NGRP][G], sm_l[NGRP][G];
  __shared__ float sm_o[NGRP][G][D];

  float qf[G][8];
#pragma unroll
  for (int g = 0; g < G; g++) {
    const uint4 raw =
        *reinterpret_cast<const uint4*>(q + (long)b * q_stride + (long)(h * G + g) * D + dl * 8);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 f = unpack_bf16x2(w[j]);
      qf[g][2 * j] = f.x * scale_log2;
      qf[g][2 * j + 1] = f.y * scale_log2;
    }
  }
  float m[G], l[G], o[G][8];
#pragma unroll
  for (int g = 0; g < G; g++) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) o[g][j] = 0.f;
  }
  const int* bt = block_table + (long)b * max_blocks;
  const long row_elems = (long)Hkv * D;

  for (int kb = k0 + warp * KPI; kb < k1; kb += 4 * KPI) {
    const int key = kb + sub;
    const bool valid = key < k1;
    float kf[8], vf[8];
    if (valid) {
      const int blk = bt[key / block_size];
      if (blk < 0 || blk >= num_blocks_total) {
        if (status) atomicExch(status, B200_BAD_INDEX);
#pragma unroll
        for (int j = 0; j < 8; j++) { kf[j] = 0.f; vf[j] = 0.f; }
      } else {
        const long off = ((long)blk * block_size + key % block_size) * row_elems + (long)h * D + dl * 8;
        const uint4 kr = __ldg(reinterpret_cast<const uint4*>(k_cache + off));
        const uint4 vr = __ldg(reinterpret_cast<const uint4*>(v_cache + off));
        const uint32_t kw[4] = {kr.x, kr.y, kr.z, kr.w}, vw[4] = {vr.x, vr.y, vr.z, vr.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const float2 a = unpack_bf16x2(kw[j]), c = unpack_bf16x2(vw[j]);
          kf[2 * j] = a.x; kf[2 * j + 1] = a.y;
          vf[2 * j] = c.x; vf[2 * j + 1] = c.y;
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; j++) { kf[j] = 0.f; vf[j] = 0.f; }
    }
#pragma unroll
    for (int g = 0; g < G; g++) {
      float s = 0.f;
#pragma unroll
      for (int j = 0; j < 8; j++) s += qf[g][j] * kf[j];
#pragma unroll
      for (int off = LPK / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
      if (!valid) s = -INFINITY;
      const float mn = fmaxf(m[g], s);
      const float ms = (mn == -INFINITY) ? 0.f : mn;
      const float alpha = exp2f(m[g] - ms);
      const float pv = exp2f(s - ms);
      l[g] = l[g] * alpha + pv;
#pragma unroll
      for (int j = 0; j < 8; j++) o[g][j] = o[g][j] * alpha + pv * vf[j];
      m[g] = mn;
    }
  }
  // ---- combine the NGRP partial states of this CTA
  const int grp = warp * KPI + sub;
#pragma unroll
  for (int g = 0; g < G; g++) {
    if (dl == 0) { sm_m[grp][g] = m[g]; sm_l[grp][g] = l[g]; }
#pragma unroll
    for (int j = 0; j < 8; j++) sm_o[grp][g][dl * 8 + j] = o[g][j];
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int i = 0; i < NGRP; i++) M = fmaxf(M, sm_m[i][g]);
    float L = 0.f, acc = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int i = 0; i < NGRP; i++) {
        const float w = exp2f(sm_m[i][g] - M);
        L += w * sm_l[i][g];
        acc += w * sm_o[i][g][d];
      }
    }
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int hq = h * G + g;
    if (num_splits == 1) {
      out[(long)b * out_stride + (long)hq * D + d] = __float2bfloat16(acc * inv);
    } else {
      const long pidx = ((long)b * (Hkv * G) + hq) * num_splits + split;
      partial_o[pidx * D + d] = acc * inv;
      if (d == 0)
        partial_lse[pidx] = (L > 0.f) ? (M * 0.6931471805599453f + logf(L)) : -INFINITY;
    }
  }
}

// out[t, hq, :] = sum_s softmax_s(lse)[s] * partial_o[t, hq, s, :]
__global__ void merge_splits_kernel(const float* __restrict__ partial_o,
                                    const float* __restrict__ partial_lse, int num_splits, int D,
                                    int Hq, __nv_bfloat16* __restrict__ out, long out_stride,
                                    float* __restrict__ lse_out) {
  const long t = blockIdx.x;
  const int hq = blockIdx.y;
  const long base = (t * Hq + hq) * num_splits;
  float M = -INFINITY;
  for (int s = 0; s < num_splits; s++) M = fmaxf(M, partial_lse[base + s]);
  if (lse_out && threadIdx.x == 0) {
    float L = 0.f;
    if (M != -INFINITY)
      for (int s = 0; s < num_splits; s++) L += __expf(partial_lse[base + s] - M);
    lse_out[t * Hq + hq] = L > 0.f ? M + logf(L) : -INFINITY;
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f, L = 0.f;
    if (M != -INFINITY) {
      for (int s = 0; s < num_splits; s++) {
        const float w = __expf(partial_lse[base + s] - M);
        L += w;
        acc += w * partial_o[(base + s) * D + d];
      }
    }
    out[t * out_stride + (long)hq * D + d] = __float2bfloat16(L > 0.f ? acc / L : 0.f);
  }
}

int launch_merge_splits(const float* partial_o, const float* partial_lse, long T, int Hq,
                        int num_splits, int D, void* out, long out_stride, cudaStream_t stream,
                        float* lse_out) {
  if (T <= 0) return 0;
  dim3 grid((unsigned)T, (unsigned)Hq);
  merge_splits_kernel<<<grid, D >= 128 ? 128 : 64, 0, stream>>>(
      partial_o, partial_lse, num_splits, D, Hq, (__nv_bfloat16*)out, out_stride, lse_out);
  return B200_CHECK_LAUNCH();
}

int launch_paged_decode(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                        const int* block_table, int max_blocks, const int* seq_lens, int B,
                        int Hq, int Hkv, int D, int block_size, float scale, int window,
                        int num_splits, void* out, long out_stride, float* partial_o,
                        float* partial_lse, long num_blocks_total, int* status,
                        cudaStream_t stream) {
  if (B <= 0) return 0;
  const int G = Hq / Hkv;
  if (G * Hkv != Hq) return 9110;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && (!partial_o || !partial_lse)) return 9111;
  const float scale_log2 = scale * 1.4426950408889634f;
  dim3 grid((unsigned)B, (unsigned)Hkv, (unsigned)num_splits);
#define LAUNCH_DEC(DD, GG)                                                                   \
  paged_decode_kernel<DD, GG><<<grid, 128, 0, stream>>>(                                     \
      (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_cache,                      \
      (const __nv_bfloat16*)v_cache, block_table, max_blocks, seq_lens, block_size, Hkv,     \
      scale_log2, window, num_splits, (__nv_bfloat16*)out, out_stride, partial_o,            \
      partial_lse, num_blocks_total, status)
#define DISPATCH_G(DD)                                   \
  switch (G) {                                           \
    case 1: LAUNCH_DEC(DD, 1); break;                    \
    case 2: LAUNCH_DEC(DD, 2); break;                    \
    case 4: LAUNCH_DEC(DD, 4); break;                    \
    case 8: LAUNCH_DEC(DD, 8); break;                    \
    default: return 9112;                                \
  }
  if (D == 128) { DISPATCH_G(128) }
  else if (D == 64) { DISPATCH_G(64) }
  else return 9113;
#undef DISPATCH_G
#undef LAUNCH_DEC
  int rc = B200_CHECK_LAUNCH();
  if (rc) return rc;
  if (num_splits > 1)
    return launch_merge_splits(partial_o, partial_lse, B, Hq, num_splits, D, out, out_stride,
                               stream);
  return 0;
}

}  // namespace b200

// Scratch sizes in bytes for a decode call with the given split count.
B200_API long b200_paged_decode_scratch_bytes(int B, int Hq, int D, int num_splits) {
  if (num_splits <= 1) return 0;
  return (long)B * Hq * num_splits * (D + 1) * (long)sizeof(float);
}

// q: [B, Hq, D] (token stride q_stride elements), caches [NB, block_size, Hkv, D],
// block_table int32 [B, max_blocks], seq_lens int32 [B], out [B, Hq, D].
// scratch: b200_paged_decode_scratch_bytes() bytes when num_splits > 1.
B200_API int b200_paged_decode(const void* q, long q_stride, const void* k_cache,
                               const void* v_cache, const void* block_table, int max_blocks,
                               const void* seq_lens, int B, int Hq, int Hkv, int D,
                               int block_size, float scale, int window, int num_splits,
                               void* out, long out_stride, void* scratch, long num_blocks_total,
                               int* status, cudaStream_t stream) {
  float* po = (float*)scratch;
  float* pl = po ? po + (long)B * Hq * num_splits * D : nullptr;
  return b200::launch_paged_decode(q, q_stride, k_cache, v_cache, (const int*)block_table,
                                   max_blocks, (const int*)seq_lens, B, Hq, Hkv, D, block_size,
                                   scale, window, num_splits, out, out_stride, po, pl,
                                   num_blocks_total, status, stream);
}

// Merge attention results computed over disjoint key sets (KV splits of one call, or the ranks of
// a context-parallel group): partial_o fp32 [T, Hq, S, D] (each normalised by its own denominator),
// partial_lse fp32 [T, Hq, S] -> out bf16 [T, Hq, D] (row stride out_stride elements), optional
// merged lse_out [T, Hq].
B200_API int b200_merge_attn_partials(const void* partial_o, const void* partial_lse, long T, int Hq,
                                      int S, int D, void* out, long out_stride, void* lse_out,
                                      cudaStream_t stream) {
  if (S < 1 || D < 1 || Hq < 1) return 9114;
  return b200::launch_merge_splits((const float*)partial_o, (const float*)partial_lse, T, Hq, S, D,
                                   out, out_stride, stream, (float*)lse_out);
}
