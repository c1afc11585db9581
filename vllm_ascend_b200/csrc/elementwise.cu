// Memory-bound per-token ops of the decoder layer, bf16, 16-byte vector access:
//   * RMSNorm and residual-add + RMSNorm          (reference: vllm_ascend/ops/layernorm.py:63-107)
//   * SiLU-and-mul                                (reference: vllm_ascend/ops/activation.py:35-48)
//   * split-QKV + per-head q/k RMSNorm + RoPE + paged KV-cache write in one pass
//     (reference fuses the first three in ops/triton/linearnorm/split_qkv_rmsnorm_rope.py
//      and writes the cache in attention/attention_v1.py:1622-1652)
//   * embedding gather with vocab-shard masking   (reference: ops/vocab_parallel_embedding.py:229-257)
//   * per-token-group (1x128) fp8 e4m3 quantisation
#include "common.cuh"
#include <cuda_fp8.h>

namespace b200 {

// ---------------------------------------------------------------- RMSNorm
// One CTA per row. x,res,out: [T, H]; w: [H].  If res != null:
//   res <- bf16(x + res);  out <- rmsnorm(res) * w      (out may alias x)
// gemma: weight used as (1 + w).
template <int VEC_PER_THREAD>
__global__ void rms_norm_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* res,
                                const __nv_bfloat16* __restrict__ w, __nv_bfloat16* out, int H,
                                float eps, int gemma, long x_stride, long out_stride) {
  const long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
  uint4* rr = res ? reinterpret_cast<uint4*>(res + row * (long)H) : nullptr;
  uint4* orow = reinterpret_cast<uint4*>(out + row * out_stride);
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
        uint32_t zw[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
          float2 fa = unpack_bf16x2(aw[j]), fb = unpack_bf16x2(bw[j]);
          zw[j] = pack_bf16x2(fa.x + fb.x, fa.y + fb.y);
          aw[j] = zw[j];
        }
        rr[v] = make_uint4(zw[0], zw[1], zw[2], zw[3]);
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 f = unpack_bf16x2(aw[j]);
        vals[i][2 * j] = f.x;
        vals[i][2 * j + 1] = f.y;
        ss += f.x * f.x + f.y * f.y;
      }
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
  const float inv = red[0];
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; i++) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      uint4 ww = wr[v];
      uint32_t w4[4] = {ww.x, ww.y, ww.z, ww.w};
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 fw = unpack_bf16x2(w4[j]);
        if (gemma) { fw.x += 1.f; fw.y += 1.f; }
        o[j] = pack_bf16x2(vals[i][2 * j] * inv * fw.x, vals[i][2 * j + 1] * inv * fw.y);
      }
      orow[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

// ---------------------------------------------------------------- SiLU-mul
// x: [T, 2*I] (gate | up) -> out [T, I];  optional clamp (swiglu "limit").
__global__ void silu_and_mul_kernel(const __nv_bfloat16* __restrict__ x,
                                    __nv_bfloat16* __restrict__ out, long T, int I, float limit) {
  const int nvec = I >> 3;
  const long total = T * nvec;
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total;
       idx += (long)gridDim.x * blockDim.x) {
    const long t = idx / nvec;
    const int v = (int)(idx - t * nvec);
    const uint4 g = reinterpret_cast<const uint4*>(x + t * 2 * (long)I)[v];
    const uint4 u = reinterpret_cast<const uint4*>(x + t * 2 * (long)I + I)[v];
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
      float2 fg = unpack_bf16x2(gw[j]), fu = unpack_bf16x2(uw[j]);
      if (limit > 0.f) {
        fg.x = fminf(fg.x, limit); fg.y = fminf(fg.y, limit);
        fu.x = fminf(fmaxf(fu.x, -limit), limit); fu.y = fminf(fmaxf(fu.y, -limit), limit);
      }
      const float a = fg.x / (1.f + __expf(-fg.x)) * fu.x;
      const float b = fg.y / (1.f + __expf(-fg.y)) * fu.y;
      o[j] = pack_bf16x2(a, b);
    }
    reinterpret_cast<uint4*>(out + t * (long)I)[v] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// ---------------------------------------------------------------- embedding
// out[t] = (vocab_start <= id < vocab_end) ? weight[id - vocab_start] : 0
__global__ void embedding_kernel(const long* __restrict__ ids,
                                 const __nv_bfloat16* __restrict__ weight,
                                 __nv_bfloat16* __restrict__ out, int H, long vocab_start,
                                 long vocab_end) {
  const long t = blockIdx.x;
  const long id = ids[t];
  const int nvec = H >> 3;
  uint4* o = reinterpret_cast<uint4*>(out + t * (long)H);
  if (id < vocab_start || id >= vocab_end) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) o[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* wrow = reinterpret_cast<const uint4*>(weight + (id - vocab_start) * (long)H);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) o[v] = wrow[v];
}

// ---------------------------------------------------------------- QK-norm + RoPE + KV write
// qkv: [T, (Hq + 2*Hkv) * D] row stride qkv_stride.  One warp per (token, head).
// cos_sin: [max_pos, rot_dim] fp32, first half cos, second half sin (neox layout
// pairs element j with j + rot_dim/2).  q and k are updated in place; k and v are
// scattered to the paged caches [num_blocks, block_size, Hkv, D] at
// slot_mapping[t] (slot < 0: skipped).  Multimodal rotary (mrope_axis != null): positions is
// [3, pos_stride] (temporal, height, width) and rotary pair e takes its angle at the position of
// axis mrope_axis[e]; text tokens carry the same position on all three axes.
template <int D>
__global__ void qknorm_rope_kvwrite_kernel(__nv_bfloat16* qkv, long qkv_stride,
                                           const long* __restrict__ positions,
                                           const float* __restrict__ cos_sin, int rot_dim,
                                           const __nv_bfloat16* __restrict__ q_norm_w,
                                           const __nv_bfloat16* __restrict__ k_norm_w, float eps,
                                           __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                                           const long* __restrict__ slot_mapping, int T, int Hq,
                                           int Hkv, long num_slots, int block_size,
                                           int kv_layout, int* status,
                                           const int* __restrict__ mrope_axis, long pos_stride) {
  constexpr int PER = D / 32;
  const int warps_per_block = blockDim.x >> 5;
  const int heads_total = Hq + 2 * Hkv;
  const long gw = (long)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (gw >= (long)T * heads_total) return;
  const int t = (int)(gw / heads_total);
  const int h = (int)(gw - (long)t * heads_total);
  const int lane = threadIdx.x & 31;
  __nv_bfloat16* src = qkv + (long)t * qkv_stride + (long)h * D;
  float v[PER];
#pragma unroll
  for (int i = 0; i < PER; i++) v[i] = __bfloat162float(src[lane + 32 * i]);

  const bool is_q = h < Hq;
  const bool is_k = !is_q && h < Hq + Hkv;
  if (is_q || is_k) {
    const __nv_bfloat16* nw = is_q ? q_norm_w : k_norm_w;
    if (nw) {
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < PER; i++) ss += v[i] * v[i];
      ss = warp_reduce_sum(ss);
      const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
      for (int i = 0; i < PER; i++) {
        // round to bf16 like the unfused norm -> rope sequence does
        v[i] = __bfloat162float(
            __float2bfloat16(v[i] * inv * __bfloat162float(nw[lane + 32 * i])));
      }
    }
    if (rot_dim > 0) {
      const long pos = positions[t];
      const float* cs = cos_sin + pos * (long)rot_dim;
      const int half = rot_dim >> 1;      // multiple of 32
      const int hp = half >> 5;           // register distance between partners
      // hp is 1, 2 or 4; the static loop keeps v[] in registers
#pragma unroll
      for (int hh = 1; hh <= (PER > 1 ? PER / 2 : 1); hh <<= 1) {
        if (hp == hh) {
#pragma unroll
          for (int i = 0; i < hh; i++) {
            if (i + hh < PER) {
              const int e = lane + 32 * i;
              const float* ce = cs;
              if (mrope_axis) ce = cos_sin + positions[mrope_axis[e] * pos_stride + t] * (long)rot_dim;
              const float c = ce[e], s = ce[half + e];
              const float x1 = v[i], x2 = v[i + hh];
              v[i] = x1 * c - x2 * s;
              v[i + hh] = x2 * c + x1 * s;
            }
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < PER; i++) src[lane + 32 * i] = __float2bfloat16(v[i]);
  }
  if (!is_q && k_cache) {
    const long slot = slot_mapping[t];
    if (slot < 0) return;
    if (slot >= num_slots) {
      if (status) atomicExch(status, B200_BAD_INDEX);
      return;
    }
    const int kvh = is_k ? (h - Hq) : (h - Hq - Hkv);
    long row = slot * Hkv + kvh;                     // [blocks, tokens, heads, D]
    if (kv_layout == 1) {                            // [blocks, heads, tokens, D]
      const long blk = slot / block_size, off = slot - blk * block_size;
      row = (blk * Hkv + kvh) * block_size + off;
    }
    __nv_bfloat16* dst = (is_k ? k_cache : v_cache) + row * (long)D;
#pragma unroll
    for (int i = 0; i < PER; i++) dst[lane + 32 * i] = __float2bfloat16(v[i]);
  }
}

// Fast path for D = 128 with full rotary (rot_dim = 128).  The op moves ~27 KB per token and is
// limited by instruction issue as much as by bytes, so: a half-warp owns one (token, head) row and
// lane l holds elements [4l, 4l+4) AND their rotation partners [64+4l, 64+4l+4) (two 8-byte
// accesses, each half-warp access covers 128 contiguous bytes), which makes the rotation
// shuffle-free; a warp walks QKN_ROWS_PER_WARP rows and issues all row loads up front.
constexpr int QKN_ROWS_PER_WARP = 8;     // 4 rows per half-warp

__global__ void __launch_bounds__(256)
qknorm_rope_kvwrite_d128_kernel(__nv_bfloat16* qkv, long qkv_stride,
                                const long* __restrict__ positions,
                                const float* __restrict__ cos_sin,
                                const __nv_bfloat16* __restrict__ q_norm_w,
                                const __nv_bfloat16* __restrict__ k_norm_w, float eps,
                                __nv_bfloat16* k_cache, __nv_bfloat16* v_cache,
                                const long* __restrict__ slot_mapping, int T, int Hq, int Hkv,
                                long num_slots, int block_size, int kv_layout, int* status) {
  constexpr int D = 128;
  constexpr int RPT = QKN_ROWS_PER_WARP / 2;          // rows per thread
  const int heads_total = Hq + 2 * Hkv;
  const long total_rows = (long)T * heads_total;
  const long gw = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int hl = lane & 15;                            // lane inside the half-warp
  const long row0 = gw * QKN_ROWS_PER_WARP + (lane >> 4);
  if (gw * QKN_ROWS_PER_WARP >= total_rows) return;

  uint2 lo[RPT], hi[RPT];                              // elements 4hl.. and 64+4hl..
  int tt[RPT], hh[RPT];
  bool ok[RPT];
#pragma unroll
  for (int i = 0; i < RPT; i++) {
    const long r = row0 + 2 * i;
    ok[i] = r < total_rows;
    const long rc = ok[i] ? r : 0;
    tt[i] = (int)(rc / heads_total);
    hh[i] = (int)(rc - (long)tt[i] * heads_total);
    const uint2* src = reinterpret_cast<const uint2*>(qkv + (long)tt[i] * qkv_stride + (long)hh[i] * D);
    lo[i] = ok[i] ? src[hl] : make_uint2(0u, 0u);
    hi[i] = ok[i] ? src[16 + hl] : make_uint2(0u, 0u);
  }
  // norm weights of this thread's 8 columns (q and k), shared by all of its rows
  float wq[8], wk[8];
  {
    const uint2 z = make_uint2(0u, 0u);
    const uint2 a0 = q_norm_w ? reinterpret_cast<const uint2*>(q_norm_w)[hl] : z;
    const uint2 a1 = q_norm_w ? reinterpret_cast<const uint2*>(q_norm_w)[16 + hl] : z;
    const uint2 b0 = k_norm_w ? reinterpret_cast<const uint2*>(k_norm_w)[hl] : z;
    const uint2 b1 = k_norm_w ? reinterpret_cast<const uint2*>(k_norm_w)[16 + hl] : z;
    const uint32_t aw[4] = {a0.x, a0.y, a1.x, a1.y}, bw[4] = {b0.x, b0.y, b1.x, b1.y};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float2 fa = unpack_bf16x2(aw[j]), fb = unpack_bf16x2(bw[j]);
      wq[2 * j] = fa.x; wq[2 * j + 1] = fa.y;
      wk[2 * j] = fb.x; wk[2 * j + 1] = fb.y;
    }
  }
  // rotary angles of the token the previous row belonged to: a thread's rows are heads of one token
  // most of the time, so the table is read once per token instead of once per (token, head)
  int t_cs = -1;
  float cc[4] = {1.f, 1.f, 1.f, 1.f}, sv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < RPT; i++) {
    const int t = tt[i], h = hh[i];
    const bool is_q = h < Hq;
    const bool is_k = !is_q && h < Hq + Hkv;
    const bool rot = is_q || is_k;
    uint2 olo = lo[i], ohi = hi[i];
    // every lane takes part in the reduction shuffles; rows past the end carry zeros
    float v[8];                                          // v[0..3] first half, v[4..7] partners
    {
      const uint32_t w32[4] = {lo[i].x, lo[i].y, hi[i].x, hi[i].y};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 f = unpack_bf16x2(w32[j]);
        v[2 * j] = f.x; v[2 * j + 1] = f.y;
      }
    }
    const bool has_norm = is_q ? (q_norm_w != nullptr) : (is_k && k_norm_w != nullptr);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 8; j++) ss += v[j] * v[j];
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (rot) {
      if (has_norm) {
        const float inv = rsqrtf(ss / (float)D + eps);
#pragma unroll
        for (int j = 0; j < 8; j++)      // rounded to bf16 like the unfused norm -> rope sequence
          v[j] = __bfloat162float(__float2bfloat16(v[j] * inv * (is_q ? wq[j] : wk[j])));
      }
      if (t != t_cs) {
        const float* cs = cos_sin + positions[t] * (long)D + hl * 4;
        const float4 c = *reinterpret_cast<const float4*>(cs);
        const float4 sn = *reinterpret_cast<const float4*>(cs + 64);
        cc[0] = c.x; cc[1] = c.y; cc[2] = c.z; cc[3] = c.w;
        sv[0] = sn.x; sv[1] = sn.y; sv[2] = sn.z; sv[3] = sn.w;
        t_cs = t;
      }
      float x1[4], x2[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        x1[j] = v[j] * cc[j] - v[4 + j] * sv[j];
        x2[j] = v[4 + j] * cc[j] + v[j] * sv[j];
      }
      olo = make_uint2(pack_bf16x2(x1[0], x1[1]), pack_bf16x2(x1[2], x1[3]));
      ohi = make_uint2(pack_bf16x2(x2[0], x2[1]), pack_bf16x2(x2[2], x2[3]));
    }
    if (!ok[i]) continue;
    if (rot) {
      uint2* dst = reinterpret_cast<uint2*>(qkv + (long)t * qkv_stride + (long)h * D);
      dst[hl] = olo;
      dst[16 + hl] = ohi;
    }
    if (!is_q && k_cache) {
      const long slot = slot_mapping[t];
      if (slot < 0) continue;
      if (slot >= num_slots) {
        if (hl == 0 && status) atomicExch(status, B200_BAD_INDEX);
        continue;
      }
      const int kvh = is_k ? (h - Hq) : (h - Hq - Hkv);
      long row = slot * Hkv + kvh;
      if (kv_layout == 1) {
        const long blk = slot / block_size, off = slot - blk * block_size;
        row = (blk * Hkv + kvh) * block_size + off;
      }
      uint2* dst = reinterpret_cast<uint2*>((is_k ? k_cache : v_cache) + row * (long)D);
      dst[hl] = olo;
      dst[16 + hl] = ohi;
    }
  }
}

// Rotary embedding from per-token angle tables (vision encoders: the angle of a pair depends on
// the patch's row for one half of the pairs and on its column for the other, so the host builds
// cos / sin [N, half] once per image batch).  x: [N, H, D] with token stride x_stride, pairs
// (e, e + half) for e < half, in place.  One warp per (token, head).
__global__ void rope_table_kernel(__nv_bfloat16* x, long x_stride, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, long N, int H, int D, int half) {
  const long gw = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (gw >= N * H) return;
  const long t = gw / H;
  const int h = (int)(gw - t * H);
  __nv_bfloat16* row = x + t * x_stride + (long)h * D;
  const float* c = cos_t + t * half;
  const float* sn = sin_t + t * half;
  for (int e = threadIdx.x & 31; e < half; e += 32) {
    const float x1 = __bfloat162float(row[e]), x2 = __bfloat162float(row[e + half]);
    row[e] = __float2bfloat16(x1 * c[e] - x2 * sn[e]);
    row[e + half] = __float2bfloat16(x2 * c[e] + x1 * sn[e]);
  }
}

// ---------------------------------------------------------------- fp8 1x128 group quant
// x: [T, H] bf16 -> q: [T, H] e4m3, scales: [T, H/128] fp32 (scale = amax/448).
// One warp per group of 128 elements.
__global__ void quant_fp8_group128_kernel(const __nv_bfloat16* __restrict__ x,
                                          __nv_fp8_e4m3* __restrict__ q,
                                          float* __restrict__ scales, long num_groups,
                                          int pow2_scale) {
  const long g = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (g >= num_groups) return;
  const int lane = threadIdx.x & 31;
  const uint2 raw = reinterpret_cast<const uint2*>(x + g * 128)[lane];
  const float2 a = unpack_bf16x2(raw.x), b = unpack_bf16x2(raw.y);
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
  amax = warp_reduce_max(amax);
  float scale = fmaxf(amax, 1e-10f) / 448.f;
  if (pow2_scale) scale = exp2f(ceilf(log2f(scale)));
  const float inv = 1.f / scale;
  __nv_fp8_e4m3 o[4] = {__nv_fp8_e4m3(a.x * inv), __nv_fp8_e4m3(a.y * inv),
                        __nv_fp8_e4m3(b.x * inv), __nv_fp8_e4m3(b.y * inv)};
  reinterpret_cast<uint32_t*>(q + g * 128)[lane] = *reinterpret_cast<uint32_t*>(o);
  if (lane == 0) scales[g] = scale;
}


// ---------------------------------------------------------------- fp8 per-token quant
// x: [T, H] bf16 (row stride x_stride) -> q: [T, H] e4m3, scales: [T] fp32 (amax / 448).
// One CTA per row, the row stays in registers between the amax pass and the store.
template <int VEC_PER_THREAD>
__global__ void quant_fp8_per_token_kernel(const __nv_bfloat16* __restrict__ x, long x_stride,
                                           __nv_fp8_e4m3* __restrict__ q, float* __restrict__ scales,
                                           int H) {
  const long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
  const int nvec = H >> 3;
  float vals[VEC_PER_THREAD][8];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; i++) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      const uint4 a = xr[v];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 f = unpack_bf16x2(aw[j]);
        vals[i][2 * j] = f.x;
        vals[i][2 * j + 1] = f.y;
        amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
      }
    }
  }
  __shared__ float red[33];
  amax = warp_reduce_max(amax);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
    t = warp_reduce_max(t);
    if (threadIdx.x == 0) red[32] = fmaxf(t, 1e-10f) / 448.f;
  }
  __syncthreads();
  const float scale = red[32];
  if (threadIdx.x == 0) scales[row] = scale;
  uint2* qr = reinterpret_cast<uint2*>(q + row * (long)H);
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; i++) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      __nv_fp8_e4m3 o[8];
#pragma unroll
      for (int j = 0; j < 8; j++) o[j] = __nv_fp8_e4m3(__fdiv_rn(vals[i][j], scale));   // as x / scale in fp32
      qr[v] = *reinterpret_cast<uint2*>(o);
    }
  }
}

// ---------------------------------------------------------------- LayerNorm
// One CTA per row, row held in registers: mean, then the variance around it, then
// out <- (x - mean) * rstd * w + b.  Used by vision-tower blocks and mergers.
template <int VEC_PER_THREAD>
__global__ void layer_norm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                  const __nv_bfloat16* __restrict__ b, __nv_bfloat16* __restrict__ out,
                                  int H, float eps, long x_stride, long out_stride) {
  const long row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + row * x_stride);
  uint4* orow = reinterpret_cast<uint4*>(out + row * out_stride);
  const int nvec = H >> 3;
  float vals[VEC_PER_THREAD][8];
  __shared__ float red[33];
  auto block_sum = [&](float v) {
    v = warp_reduce_sum(v);
    __syncthreads();                       // previous use of red is over
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
      t = warp_reduce_sum(t);
      if (threadIdx.x == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
  };
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; i++) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      uint4 a = xr[v];
      uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 f = unpack_bf16x2(aw[j]);
        vals[i][2 * j] = f.x;
        vals[i][2 * j + 1] = f.y;
        s += f.x + f.y;
      }
    }
  }
  const float mean = block_sum(s) / (float)H;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; i++) {
    if (threadIdx.x + i * blockDim.x < nvec) {
#pragma unroll
      for (int j = 0; j < 8; j++) {
        const float d = vals[i][j] - mean;
        ss = fmaf(d, d, ss);
      }
    }
  }
  const float rstd = rsqrtf(block_sum(ss) / (float)H + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
  const uint4* br = reinterpret_cast<const uint4*>(b);
#pragma unroll
  for (int i = 0; i < VEC_PER_THREAD; i++) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      uint4 ww = wr[v];
      uint32_t w4[4] = {ww.x, ww.y, ww.z, ww.w};
      uint32_t b4[4] = {0u, 0u, 0u, 0u};
      if (b) {
        uint4 bb = br[v];
        b4[0] = bb.x; b4[1] = bb.y; b4[2] = bb.z; b4[3] = bb.w;
      }
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 fw = unpack_bf16x2(w4[j]), fb = unpack_bf16x2(b4[j]);
        o[j] = pack_bf16x2(fmaf((vals[i][2 * j] - mean) * rstd, fw.x, fb.x),
                           fmaf((vals[i][2 * j + 1] - mean) * rstd, fw.y, fb.y));
      }
      orow[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_rms_norm(const void* x, void* residual, const void* w, void* out, long T, int H,
                           float eps, int gemma, long x_stride, long out_stride,
                           cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return 9100;
  const int nvec = H >> 3;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  const int per = (nvec + threads - 1) / threads;
  auto X = (const __nv_bfloat16*)x;
  auto R = (__nv_bfloat16*)residual;
  auto W = (const __nv_bfloat16*)w;
  auto O = (__nv_bfloat16*)out;
  if (per <= 1)
    rms_norm_kernel<1><<<(unsigned)T, threads, 0, stream>>>(X, R, W, O, H, eps, gemma, x_stride,
                                                            out_stride);
  else if (per <= 2)
    rms_norm_kernel<2><<<(unsigned)T, threads, 0, stream>>>(X, R, W, O, H, eps, gemma, x_stride,
                                                            out_stride);
  else if (per <= 4)
    rms_norm_kernel<4><<<(unsigned)T, threads, 0, stream>>>(X, R, W, O, H, eps, gemma, x_stride,
                                                            out_stride);
  else
    return 9101;  // hidden size above 32768 not supported
  return B200_CHECK_LAUNCH();
}

B200_API int b200_layer_norm(const void* x, const void* w, const void* b, void* out, long T, int H,
                             float eps, long x_stride, long out_stride, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || (x_stride & 7) || (out_stride & 7)) return 9110;
  const int nvec = H >> 3;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  const int per = (nvec + threads - 1) / threads;
  auto X = (const __nv_bfloat16*)x;
  auto W = (const __nv_bfloat16*)w;
  auto Bp = (const __nv_bfloat16*)b;
  auto O = (__nv_bfloat16*)out;
  if (per <= 1)
    layer_norm_kernel<1><<<(unsigned)T, threads, 0, stream>>>(X, W, Bp, O, H, eps, x_stride, out_stride);
  else if (per <= 2)
    layer_norm_kernel<2><<<(unsigned)T, threads, 0, stream>>>(X, W, Bp, O, H, eps, x_stride, out_stride);
  else if (per <= 4)
    layer_norm_kernel<4><<<(unsigned)T, threads, 0, stream>>>(X, W, Bp, O, H, eps, x_stride, out_stride);
  else
    return 9111;
  return B200_CHECK_LAUNCH();
}

B200_API int b200_silu_and_mul(const void* x, void* out, long T, int I, float limit,
                               cudaStream_t stream) {
  if (T <= 0) return 0;
  if (I & 7) return 9100;
  const long total = T * (I >> 3);
  long blocks = (total + 255) / 256;
  const long cap = (long)num_sms() * 16;
  if (blocks > cap) blocks = cap;
  silu_and_mul_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const __nv_bfloat16*)x,
                                                            (__nv_bfloat16*)out, T, I, limit);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_embedding(const void* ids, const void* weight, void* out, long T, int H,
                            long vocab_start, long vocab_end, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return 9100;
  embedding_kernel<<<(unsigned)T, 128, 0, stream>>>((const long*)ids,
                                                    (const __nv_bfloat16*)weight,
                                                    (__nv_bfloat16*)out, H, vocab_start,
                                                    vocab_end);
  return B200_CHECK_LAUNCH();
}

static int qknorm_rope_impl(void* qkv, long qkv_stride, const void* positions,
                            const void* cos_sin, int rot_dim, const void* q_norm_w,
                            const void* k_norm_w, float eps, void* k_cache,
                            void* v_cache, const void* slot_mapping, int T, int Hq,
                            int Hkv, int D, long num_slots, int block_size,
                            int kv_layout, int* status, const void* mrope_axis, long pos_stride,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (rot_dim > D || (rot_dim > 0 && ((rot_dim >> 1) & 31))) return 9102;
  const long warps = (long)T * (Hq + 2 * Hkv);
  const int wpb = 8;
  const unsigned blocks = (unsigned)((warps + wpb - 1) / wpb);
#define LAUNCH_ROPE(DD)                                                                       \
  qknorm_rope_kvwrite_kernel<DD><<<blocks, wpb * 32, 0, stream>>>(                            \
      (__nv_bfloat16*)qkv, qkv_stride, (const long*)positions, (const float*)cos_sin, rot_dim, \
      (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w, eps,                    \
      (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (const long*)slot_mapping, T, Hq, Hkv, \
      num_slots, block_size, kv_layout, status, (const int*)mrope_axis, pos_stride)
  if (D == 128 && rot_dim == 128 && (qkv_stride & 3) == 0 && !mrope_axis &&
      (((uintptr_t)qkv | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)q_norm_w |
        (uintptr_t)k_norm_w) & 7) == 0) {
    const long w8 = (warps + QKN_ROWS_PER_WARP - 1) / QKN_ROWS_PER_WARP;
    const unsigned blocks8 = (unsigned)((w8 + wpb - 1) / wpb);
    qknorm_rope_kvwrite_d128_kernel<<<blocks8, wpb * 32, 0, stream>>>(
        (__nv_bfloat16*)qkv, qkv_stride, (const long*)positions, (const float*)cos_sin,
        (const __nv_bfloat16*)q_norm_w, (const __nv_bfloat16*)k_norm_w, eps,
        (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, (const long*)slot_mapping, T, Hq, Hkv,
        num_slots, block_size, kv_layout, status);
    return B200_CHECK_LAUNCH();
  }
  if (D == 128) LAUNCH_ROPE(128);
  else if (D == 64) LAUNCH_ROPE(64);
  else if (D == 256) LAUNCH_ROPE(256);
  else if (D == 96) LAUNCH_ROPE(96);
  else if (D == 32) LAUNCH_ROPE(32);
  else return 9103;
#undef LAUNCH_ROPE
  return B200_CHECK_LAUNCH();
}

B200_API int b200_qknorm_rope_kvwrite(void* qkv, long qkv_stride, const void* positions,
                                      const void* cos_sin, int rot_dim, const void* q_norm_w,
                                      const void* k_norm_w, float eps, void* k_cache,
                                      void* v_cache, const void* slot_mapping, int T, int Hq,
                                      int Hkv, int D, long num_slots, int block_size,
                                      int kv_layout, int* status, cudaStream_t stream) {
  return qknorm_rope_impl(qkv, qkv_stride, positions, cos_sin, rot_dim, q_norm_w, k_norm_w, eps,
                          k_cache, v_cache, slot_mapping, T, Hq, Hkv, D, num_slots, block_size,
                          kv_layout, status, nullptr, 0, stream);
}

// positions: int64 [3, pos_stride]; mrope_axis: int32 [rot_dim / 2] with values 0..2.
B200_API int b200_qknorm_mrope_kvwrite(void* qkv, long qkv_stride, const void* positions,
                                       long pos_stride, const void* mrope_axis,
                                       const void* cos_sin, int rot_dim, const void* q_norm_w,
                                       const void* k_norm_w, float eps, void* k_cache,
                                       void* v_cache, const void* slot_mapping, int T, int Hq,
                                       int Hkv, int D, long num_slots, int block_size,
                                       int kv_layout, int* status, cudaStream_t stream) {
  if (!mrope_axis) return 9104;
  return qknorm_rope_impl(qkv, qkv_stride, positions, cos_sin, rot_dim, q_norm_w, k_norm_w, eps,
                          k_cache, v_cache, slot_mapping, T, Hq, Hkv, D, num_slots, block_size,
                          kv_layout, status, mrope_axis, pos_stride, stream);
}

B200_API int b200_rope_table(void* x, long x_stride, const void* cos_t, const void* sin_t, long N,
                             int H, int D, int half, cudaStream_t stream) {
  if (N <= 0 || H <= 0) return 0;
  if (half <= 0 || 2 * half > D) return 9105;
  const long warps = N * H;
  rope_table_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(
      (__nv_bfloat16*)x, x_stride, (const float*)cos_t, (const float*)sin_t, N, H, D, half);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_quant_fp8_per_token(const void* x, long x_stride, void* q, void* scales, long T,
                                      int H, cudaStream_t stream) {
  if (T <= 0) return 0;
  if ((H & 7) || (x_stride & 7)) return 9120;
  const int nvec = H >> 3;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  const int per = (nvec + threads - 1) / threads;
  auto X = (const __nv_bfloat16*)x;
  auto Q = (__nv_fp8_e4m3*)q;
  auto S = (float*)scales;
  if (per <= 1) quant_fp8_per_token_kernel<1><<<(unsigned)T, threads, 0, stream>>>(X, x_stride, Q, S, H);
  else if (per <= 2) quant_fp8_per_token_kernel<2><<<(unsigned)T, threads, 0, stream>>>(X, x_stride, Q, S, H);
  else if (per <= 4) quant_fp8_per_token_kernel<4><<<(unsigned)T, threads, 0, stream>>>(X, x_stride, Q, S, H);
  else return 9121;
  return B200_CHECK_LAUNCH();
}

B200_API int b200_quant_fp8_group128(const void* x, void* q, void* scales, long T, int H,
                                     int pow2_scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H % 128) return 9100;
  const long groups = T * (H / 128);
  const unsigned blocks = (unsigned)((groups + 7) / 8);
  quant_fp8_group128_kernel<<<blocks, 256, 0, stream>>>((const __nv_bfloat16*)x,
                                                        (__nv_fp8_e4m3*)q, (float*)scales,
                                                        groups, pow2_scale);
  return B200_CHECK_LAUNCH();
}
