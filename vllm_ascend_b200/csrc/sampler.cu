// Sampling kernels.  Semantics follow the reference sampler
// (vllm_ascend/sample/sampler.py:20-271): penalties -> temperature -> top-k ->
// top-p (-> min-p) -> exponential-race sampling argmax(p / Exp(1)); greedy rows
// take argmax of the raw logits.  Instead of the reference's full sort, the
// top-k and top-p cut-offs are found with a 3-pass radix select over the float
// bit patterns (count histograms for top-k, mass histograms for top-p), so a row
// costs a handful of streaming passes over the vocabulary.
#include "common.cuh"

namespace b200 {

constexpr int SAMP_THREADS = 1024;

// ---------------------------------------------------------------- Philox4x32-10
__device__ __forceinline__ uint4 philox4x32(uint4 ctr, uint2 key) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int i = 0; i < 10; i++) {
    const uint32_t hi0 = __umulhi(M0, ctr.x), lo0 = M0 * ctr.x;
    const uint32_t hi1 = __umulhi(M1, ctr.z), lo1 = M1 * ctr.z;
    ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
    key.x += W0;
    key.y += W1;
  }
  return ctr;
}
__device__ __forceinline__ float u32_to_unit(uint32_t x) {  // (0, 1]
  return ((float)(x >> 8) + 1.0f) * (1.0f / 16777216.0f);
}

template <typename T>
__device__ __forceinline__ float ld_logit(const T* p, long i);
template <>
__device__ __forceinline__ float ld_logit<float>(const float* p, long i) { return p[i]; }
template <>
__device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, long i) {
  return __bfloat162float(p[i]);
}

// block-wide argmax helper: (value, index) with lowest index on ties
__device__ __forceinline__ void block_argmax(float& v, int& idx, float* sv, int* si) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { sv[warp] = v; si[warp] = idx; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    v = lane < nw ? sv[lane] : -INFINITY;
    idx = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
    }
    if (lane == 0) { sv[0] = v; si[0] = idx; }
  }
  __syncthreads();
  v = sv[0];
  idx = si[0];
  __syncthreads();
}

template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, long ld, int V,
                              long* __restrict__ out) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const T* row = logits + (long)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  int done = 0;                        // elements [0, done) are covered by the vector loop
  if constexpr (sizeof(T) == 2) {
    // 16-byte loads (8 logits) when the row starts on a 16-byte boundary; a thread walks its
    // chunks in ascending index order, so "first maximum wins" still holds per thread
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
      const int nvec = V >> 3;
      const uint4* rv = reinterpret_cast<const uint4*>(row);
      for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
        const uint4 q = rv[c];
        const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
          const float lo = __uint_as_float(w4[k] << 16);
          const float hi = __uint_as_float(w4[k] & 0xffff0000u);
          if (lo > best) { best = lo; bi = c * 8 + 2 * k; }
          if (hi > best) { best = hi; bi = c * 8 + 2 * k + 1; }
        }
      }
      done = nvec << 3;
    }
  }
  for (int i = done + threadIdx.x; i < V; i += blockDim.x) {
    const float v = ld_logit<T>(row, i);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
  block_argmax(best, bi, sv, si);
  if (threadIdx.x == 0) out[blockIdx.x] = bi;
}

// ---------------------------------------------------------------- penalties
// logits fp32 [B, V] in place. prompt_ids [B, Lp], output_ids [B, Lo] int64, padded with
// values >= V. rep/freq/pres: [B].  Dynamic smem: 2 bitmaps of ceil(V/32) words.
__global__ void penalties_kernel(float* logits, long ld, int V, const long* prompt_ids, int Lp,
                                 const long* output_ids, int Lo, const float* rep,
                                 const float* freq, const float* pres) {
  extern __shared__ uint32_t bm[];
  const int words = (V + 31) / 32;
  uint32_t* seen_all = bm;
  uint32_t* seen_out = bm + words;
  const int b = blockIdx.x;
  float* row = logits + (long)b * ld;
  const float rp = rep ? rep[b] : 1.f, fp = freq ? freq[b] : 0.f, pp = pres ? pres[b] : 0.f;
  if (rp == 1.f && fp == 0.f && pp == 0.f) return;
  for (int i = threadIdx.x; i < 2 * words; i += blockDim.x) bm[i] = 0;
  __syncthreads();
  if (rp != 1.f) {
    for (int i = threadIdx.x; i < Lp + Lo; i += blockDim.x) {
      const long id = i < Lp ? prompt_ids[(long)b * Lp + i] : output_ids[(long)b * Lo + (i - Lp)];
      if (id < 0 || id >= V) continue;
      const uint32_t bit = 1u << (id & 31);
      const uint32_t old = atomicOr(&seen_all[id >> 5], bit);
      if (!(old & bit)) {
        const float x = row[id];
        row[id] = x > 0.f ? x / rp : x * rp;
      }
    }
  }
  __syncthreads();
  if (fp != 0.f || pp != 0.f) {
    for (int i = threadIdx.x; i < Lo; i += blockDim.x) {
      const long id = output_ids[(long)b * Lo + i];
      if (id < 0 || id >= V) continue;
      const uint32_t bit = 1u << (id & 31);
      const uint32_t old = atomicOr(&seen_out[id >> 5], bit);
      float d = -fp;
      if (!(old & bit)) d -= pp;
      atomicAdd(&row[id], d);
    }
  }
}

// ---------------------------------------------------------------- top-k/top-p sampling
// Radix select helper state lives in shared memory.
struct RadixSmem {
  float hist[2048];
  float red[32];
  int redi[32];
  uint32_t prefix;      // selected high bits so far
  float remaining;      // remaining count / mass to find inside the selected bin
  float total;
};

// One pass: histogram (count or mass) of the `bits`-wide digit at `shift` over elements
// whose higher bits equal `prefix` and which pass the `floor_key` filter, then walk
// bins from the top to find where the cumulative quantity reaches `remaining`.
__device__ void radix_pass(const float* __restrict__ e, int V, RadixSmem* s, int shift, int bits,
                           uint32_t hi_mask, bool by_mass, uint32_t floor_key) {
  const int nb = 1 << bits;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) s->hist[i] = 0.f;
  __syncthreads();
  const uint32_t prefix = s->prefix;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = e[i];
    const uint32_t k = __float_as_uint(v);
    if (k < floor_key) continue;
    if ((k & hi_mask) != prefix) continue;
    atomicAdd(&s->hist[(k >> shift) & (nb - 1)], by_mass ? v : 1.f);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float rem = s->remaining;
    int sel = 0;
    for (int bin = nb - 1; bin >= 0; bin--) {
      const float hval = s->hist[bin];
      if (hval >= rem || bin == 0) { sel = bin; break; }
      rem -= hval;
    }
    // fp rounding can leave every bin below rem: fall back to the lowest non-empty bin
    s->prefix = prefix | ((uint32_t)sel << shift);
    s->remaining = rem;
  }
  __syncthreads();
}

// logits: fp32 [B, V] (already penalised), overwritten with exp((x - max)/T).
// temperature/top_k/top_p/min_p: per row (top_k <= 0 or >= V: off; top_p >= 1: off).
// seeds: per-row uint64 seed, offsets: per-row counter (e.g. number of tokens generated).
__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(float* logits, long ld, int V, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const float* __restrict__ min_p, const unsigned long long* __restrict__ seeds,
              const long* __restrict__ offsets, long* __restrict__ out) {
  __shared__ RadixSmem s;
  const int b = blockIdx.x;
  float* row = logits + (long)b * ld;
  const float T = temperature ? temperature[b] : 1.f;
  // ---- max (also the greedy answer)
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = row[i];
    if (v > best) { best = v; bi = i; }
  }
  block_argmax(best, bi, s.red, s.redi);
  if (T < 1e-5f) {
    if (threadIdx.x == 0) out[b] = bi;
    return;
  }
  // ---- e = exp((x - max)/T), Z
  const float invT = 1.f / T;
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float ev = __expf((row[i] - best) * invT);
    row[i] = ev;
    z += ev;
  }
  z = warp_reduce_sum(z);
  if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = z;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s.red[threadIdx.x] : 0.f;
    t = warp_reduce_sum(t);
    if (threadIdx.x == 0) s.total = t;
  }
  __syncthreads();
  float mass = s.total;
  uint32_t thr_key = 0;  // keep elements with key >= thr_key

  const int k = top_k ? top_k[b] : 0;
  if (k > 0 && k < V) {
    if (threadIdx.x == 0) { s.prefix = 0; s.remaining = (float)k; }
    __syncthreads();
    radix_pass(row, V, &s, 21, 11, 0x00000000u, false, 0);
    radix_pass(row, V, &s, 10, 11, 0xFFE00000u, false, 0);
    radix_pass(row, V, &s, 0, 10, 0xFFFFFC00u, false, 0);
    thr_key = s.prefix;
    __syncthreads();
    // mass of the kept set
    float mk = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float v = row[i];
      if (__float_as_uint(v) >= thr_key) mk += v;
    }
    mk = warp_reduce_sum(mk);
    if ((threadIdx.x & 31) == 0) s.red[threadIdx.x >> 5] = mk;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? s.red[threadIdx.x] : 0.f;
      t = warp_reduce_sum(t);
      if (threadIdx.x == 0) s.total = t;
    }
    __syncthreads();
    mass = s.total;
  }
  const float pth = top_p ? top_p[b] : 1.f;
  if (pth < 1.f) {
    if (threadIdx.x == 0) { s.prefix = 0; s.remaining = pth * mass; }
    __syncthreads();
    radix_pass(row, V, &s, 21, 11, 0x00000000u, true, thr_key);
    radix_pass(row, V, &s, 10, 11, 0xFFE00000u, true, thr_key);
    radix_pass(row, V, &s, 0, 10, 0xFFFFFC00u, true, thr_key);
    const uint32_t tp = s.prefix;
    if (tp > thr_key) thr_key = tp;
    __syncthreads();
  }
  const float mp = min_p ? min_p[b] : 0.f;
  if (mp > 0.f) {
    const uint32_t tm = __float_as_uint(mp);  // max e is exactly 1
    if (tm > thr_key) thr_key = tm;
  }
  // ---- exponential race over the kept set
  const unsigned long long seed = seeds ? seeds[b] : 0ull;
  const long offset = offsets ? offsets[b] : 0;
  const uint2 key = make_uint2((uint32_t)seed, (uint32_t)(seed >> 32));
  float bestv = -INFINITY;
  int besti = bi;
  for (int i0 = threadIdx.x * 4; i0 < V; i0 += blockDim.x * 4) {
    const uint4 rnd = philox4x32(
        make_uint4((uint32_t)i0, (uint32_t)offset, (uint32_t)((unsigned long long)offset >> 32), 0u), key);
    const uint32_t rr[4] = {rnd.x, rnd.y, rnd.z, rnd.w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int i = i0 + j;
      if (i < V) {
        const float v = row[i];
        if (__float_as_uint(v) >= thr_key && v > 0.f) {
          const float ex = -__logf(u32_to_unit(rr[j]));  // Exp(1)
          const float sc = v / fmaxf(ex, 1e-20f);
          if (sc > bestv || (sc == bestv && i < besti)) { bestv = sc; besti = i; }
        }
      }
    }
  }
  block_argmax(bestv, besti, s.red, s.redi);
  if (threadIdx.x == 0) out[b] = besti;
}

__global__ void cast_bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, long ld_in,
                                        float* __restrict__ out, long ld_out, int V) {
  const __nv_bfloat16* r = in + (long)blockIdx.x * ld_in;
  float* o = out + (long)blockIdx.x * ld_out;
  for (int i = threadIdx.x; i < V; i += blockDim.x) o[i] = __bfloat162float(r[i]);
}

}  // namespace b200

using namespace b200;

// dtype: 0 = bf16, 1 = fp32.  out: int64 [B]
B200_API int b200_argmax(const void* logits, int dtype, long ld, int B, int V, void* out,
                         cudaStream_t stream) {
  if (B <= 0) return 0;
  if (dtype == 0)
    argmax_kernel<__nv_bfloat16><<<B, SAMP_THREADS, 0, stream>>>((const __nv_bfloat16*)logits, ld,
                                                                  V, (long*)out);
  else
    argmax_kernel<float><<<B, SAMP_THREADS, 0, stream>>>((const float*)logits, ld, V, (long*)out);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_cast_bf16_f32(const void* in, long ld_in, void* out, long ld_out, int B, int V,
                                cudaStream_t stream) {
  if (B <= 0) return 0;
  cast_bf16_to_f32_kernel<<<B, 1024, 0, stream>>>((const __nv_bfloat16*)in, ld_in, (float*)out,
                                                  ld_out, V);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_apply_penalties(void* logits, long ld, int B, int V, const void* prompt_ids,
                                  int Lp, const void* output_ids, int Lo, const void* rep,
                                  const void* freq, const void* pres, cudaStream_t stream) {
  if (B <= 0) return 0;
  const int words = (V + 31) / 32;
  const size_t smem = (size_t)2 * words * 4;
  static size_t smem_set = 0;
  if (smem > 48 * 1024 && smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(penalties_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    smem_set = smem;
  }
  penalties_kernel<<<B, 512, smem, stream>>>((float*)logits, ld, V, (const long*)prompt_ids, Lp,
                                             (const long*)output_ids, Lo, (const float*)rep,
                                             (const float*)freq, (const float*)pres);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_sample(void* logits_f32, long ld, int B, int V, const void* temperature,
                         const void* top_k, const void* top_p, const void* min_p,
                         const void* seeds, const void* offsets, void* out,
                         cudaStream_t stream) {
  if (B <= 0) return 0;
  sample_kernel<<<B, SAMP_THREADS, 0, stream>>>(
      (float*)logits_f32, ld, V, (const float*)temperature, (const int*)top_k,
      (const float*)top_p, (const float*)min_p, (const unsigned long long*)seeds,
      (const long*)offsets, (long*)out);
  return B200_CHECK_LAUNCH();
}
