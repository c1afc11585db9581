// Paged GQA attention on tcgen05 tensor cores with TMEM accumulators, fed by TMA.
// One kernel serves chunked prefill, decode (optionally split-KV) and
// speculative-decode verification: every query token attends to the first
// (context + its own position + 1) tokens of its sequence's paged KV cache.
//
// Behavioural parity: the reference's fused-infer-attention path over the paged
// cache in TND layout with causal / sliding-window masking
// (vllm_ascend/attention/attention_v1.py:1341-1472) and its paged decode path
// (:1555-1574); the K/V of the new tokens are already in the cache (written by
// the RoPE+KV-write kernel).
//
// Tile = 128 query rows x 128 keys.  Query rows pack the G = Hq/Hkv heads that
// share one KV head: row r = token (r / G), head (r % G), so each K/V page is
// loaded once per 128 (token, head) rows.
//   warp 0     TMA producer (Q once; K and V pages per tile, 128-byte swizzle)
//   warp 1     tcgen05.mma issuer:  S = Q K^T  (K-major x K-major, f32 in TMEM, double-buffered)
//                                   O += P V   (P from shared memory, V MN-major)
//   warps 2-5  softmax: tcgen05.ld S row -> mask -> online max/sum -> P (bf16, swizzled
//              shared memory); rescale O in TMEM only when the running max moved by
//              more than a threshold; final normalise + store (or split partials)
// All waits are bounded; on timeout the CTA aborts cleanly and reports a status.
#include "common.cuh"
#include "attention.h"

#include <mutex>
#include <string.h>
#include <unordered_map>
#include <string>

namespace b200 {

constexpr int ATT_THREADS = 192;
constexpr int ATT_HALF_BYTES = 128 * 128;  // 128 rows x 64 bf16

struct AttnParams {
  const int* query_start_loc;  // [B+1]
  const int* seq_lens;         // [B]
  const int* block_table;      // [B, max_blocks]
  const int* tile_seq;         // [tiles] or null: tile i <-> sequence i, token offset 0
  const int* tile_qoff;        // [tiles] first query token of the tile inside its sequence
  int max_blocks, block_size, rows_per_load;
  int G, Hkv, Hq, tok_per_tile;
  float scale_log2;
  int causal, window, num_splits;
  __nv_bfloat16* out;
  long out_stride;
  float* partial_o;
  float* partial_lse;
  long num_blocks_total;
  int* status;
  uint32_t v_lbo, v_sbo;
  float rescale_threshold;
};

__device__ __forceinline__ float att_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int D>
struct AttCfg {
  static constexpr int NH = D / 64;
  static constexpr int KS = (D == 64) ? 4 : 2;
  static constexpr int TILE_BYTES = NH * ATT_HALF_BYTES;
  static constexpr int P_BYTES = 2 * ATT_HALF_BYTES;   // one P buffer (two 64-key halves)
  static constexpr int P_BUFS = 2;                     // P(j+1) is written while PV(j) runs
  static constexpr int SMEM_BYTES = TILE_BYTES * (1 + 2 * KS) + P_BUFS * P_BYTES + 1024 + 512;
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = 256;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap tmap_q,
                   const __grid_constant__ CUtensorMap tmap_k,
                   const __grid_constant__ CUtensorMap tmap_v, AttnParams p) {
  using Cfg = AttCfg<D>;
  constexpr int NH = Cfg::NH, KS = Cfg::KS;

  // ---------------- work decode (uniform over the CTA)
  const int h = blockIdx.x, wi = blockIdx.y, split = blockIdx.z;
  const int seq = p.tile_seq ? p.tile_seq[wi] : wi;
  const int tok0 = p.tile_qoff ? p.tile_qoff[wi] : 0;
  const int q_start = p.query_start_loc[seq];
  const int q_len = p.query_start_loc[seq + 1] - q_start;
  const int seq_len = p.seq_lens[seq];
  const int ctx = seq_len - q_len;
  const int G = p.G;
  const int ntok = min(p.tok_per_tile, q_len - tok0);
  if (ntok <= 0) return;
  const int kv_end = p.causal ? min(seq_len, ctx + tok0 + ntok) : seq_len;
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, ctx + tok0 - p.window + 1);
  const int tile_lo = kv_lo >> 7, tile_hi = (kv_end + 127) >> 7;
  const int n_all = tile_hi - tile_lo;
  const int per_split = (n_all + p.num_splits - 1) / p.num_splits;
  const int t0 = tile_lo + split * per_split;
  const int t1 = min(tile_hi, t0 + per_split);
  const int n = t1 - t0;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (n <= 0) {  // empty split: neutral partial
    if (p.num_splits > 1 && threadIdx.x < 128) {
      const int row = threadIdx.x, tok = row / G, g = row % G;
      if (tok < ntok) {
        const long pidx =
            ((long)(q_start + tok0 + tok) * p.Hq + (h * G + g)) * p.num_splits + split;
        p.partial_lse[pidx] = -INFINITY;
        for (int d = 0; d < D; d++) p.partial_o[pidx * D + d] = 0.f;
      }
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* Qs = smem;
  uint8_t* Ks = Qs + Cfg::TILE_BYTES;
  uint8_t* Vs = Ks + KS * Cfg::TILE_BYTES;
  uint8_t* Ps = Vs + KS * Cfg::TILE_BYTES;
  uint64_t* bars = (uint64_t*)(Ps + Cfg::P_BUFS * Cfg::P_BYTES);
  uint64_t* q_full = bars;              // 1
  uint64_t* k_full = bars + 1;          // KS
  uint64_t* k_empty = k_full + KS;      // KS
  uint64_t* v_full = k_empty + KS;      // KS
  uint64_t* v_empty = v_full + KS;      // KS
  uint64_t* s_ready = v_empty + KS;     // 2
  uint64_t* s_free = s_ready + 2;       // 2
  uint64_t* p_ready = s_free + 2;       // 2 (per P buffer)
  uint64_t* pv_done = p_ready + 2;      // 2 (per P buffer)
  uint32_t* tmem_ptr = (uint32_t*)(pv_done + 2);
  volatile int* abort_word = (volatile int*)(tmem_ptr + 1);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < KS; s++) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&s_ready[b], 1);
      mbar_init(&s_free[b], 4);
      mbar_init(&p_ready[b], 4);
      mbar_init(&pv_done[b], 1);
    }
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    const int* bt = p.block_table + (long)seq * p.max_blocks;
    const int rpl = p.rows_per_load;
    const int parts = 128 / rpl;
    if (lane == 0) {
      mbar_expect_tx(q_full, Cfg::TILE_BYTES);
#pragma unroll
      for (int hf = 0; hf < NH; hf++)
        tma_load_4d(Qs + hf * ATT_HALF_BYTES, &tmap_q, q_full, hf * 64, 0, h, q_start + tok0);
    }
    // Block ids are fetched one tile ahead (lane p holds the id of part p), so the
    // dependent global load never sits between a freed stage and the next TMA issue.
    auto load_blk = [&](int j) -> int {
      if (j >= n || lane >= parts) return 0;
      const int key0 = ((t0 + j) << 7) + lane * rpl;
      return bt[min(key0, seq_len - 1) / p.block_size];
    };
    int blk_cur = load_blk(0);
    for (int j = 0; j < n; j++) {
      const int ks = j % KS;
      const uint32_t ph = (uint32_t)(j / KS) & 1u;
      const int key_base = (t0 + j) << 7;
      const int blk_next = load_blk(j + 1);
      bool bad = blk_cur < 0 || blk_cur >= p.num_blocks_total;
      bad = __any_sync(0xffffffffu, bad && lane < parts);
#pragma unroll 1
      for (int kv = 0; kv < 2; kv++) {
        uint64_t* fullb = kv == 0 ? &k_full[ks] : &v_full[ks];
        uint64_t* emptyb = kv == 0 ? &k_empty[ks] : &v_empty[ks];
        if (!mbar_wait(emptyb, ph ^ 1u, abort_word)) goto done;
        if (bad) {
          *abort_word = B200_BAD_INDEX;
          goto done;
        }
        for (int part = 0; part < parts; part++) {
          const int blk = __shfl_sync(0xffffffffu, blk_cur, part);
          if (lane == 0) {
            uint8_t* dst = (kv == 0 ? Ks : Vs) + ks * Cfg::TILE_BYTES;
            const CUtensorMap* tm = kv == 0 ? &tmap_k : &tmap_v;
            if (part == 0) mbar_expect_tx(fullb, Cfg::TILE_BYTES);
            const int off = (key_base + part * rpl) % p.block_size;
#pragma unroll
            for (int hf = 0; hf < NH; hf++)
              tma_load_4d(dst + hf * ATT_HALF_BYTES + part * rpl * 128, tm, fullb, hf * 64, h, off, blk);
          }
        }
        __syncwarp();
      }
      blk_cur = blk_next;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc_f16(128, 128, true, false, false);
    constexpr uint32_t idesc_o = make_idesc_f16(128, D, true, false, true);
    const uint32_t q_addr = smem_u32(Qs), k_addr = smem_u32(Ks), v_addr = smem_u32(Vs),
                   p_addr = smem_u32(Ps);
    if (!mbar_wait(q_full, 0, abort_word)) goto done;
    auto issue_s = [&](int j) -> bool {
      const int ks = j % KS;
      const uint32_t ph = (uint32_t)(j / KS) & 1u;
      const int b = j & 1;
      if (!mbar_wait(&k_full[ks], ph, abort_word)) return false;
      if (!mbar_wait(&s_free[b], (((uint32_t)j >> 1) & 1u) ^ 1u, abort_word)) return false;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < D / 16; kk++) {
          const uint32_t o = (kk >> 2) * ATT_HALF_BYTES + (kk & 3) * 32;
          const uint64_t da = make_smem_desc(q_addr + o, 16, 1024, kLayoutSw128);
          const uint64_t db =
              make_smem_desc(k_addr + ks * Cfg::TILE_BYTES + o, 16, 1024, kLayoutSw128);
          umma_f16_ss(tmem_base + b * 128, da, db, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[ks]);
        umma_commit(&s_ready[b]);
      }
      __syncwarp();
      return true;
    };
    if (!issue_s(0)) goto done;
    for (int j = 0; j < n; j++) {
      if (j + 1 < n) {
        if (!issue_s(j + 1)) goto done;
      }
      const int vs = j % KS;
      const uint32_t ph = (uint32_t)(j / KS) & 1u;
      if (!mbar_wait(&v_full[vs], ph, abort_word)) goto done;
      const int pb = j & 1;
      if (!mbar_wait(&p_ready[pb], ((uint32_t)j >> 1) & 1u, abort_word)) goto done;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < 8; kk++) {
          const uint32_t po = (kk >> 2) * ATT_HALF_BYTES + (kk & 3) * 32;
          const uint64_t da =
              make_smem_desc(p_addr + pb * Cfg::P_BYTES + po, 16, 1024, kLayoutSw128);
          const uint64_t db = make_smem_desc(v_addr + vs * Cfg::TILE_BYTES + kk * 2048, p.v_lbo,
                                             p.v_sbo, kLayoutSw128);
          umma_f16_ss(tmem_base + Cfg::O_COL, da, db, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[vs]);
        umma_commit(&pv_done[pb]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue
    const int qd = warp & 3;
    const int row = qd * 32 + lane;
    const int tok = row / G, g = row % G;
    const bool row_valid = tok < ntok;
    const int q_pos = ctx + tok0 + tok;
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl2 = p.scale_log2;
    int hi = seq_len;                      // keys [lo, hi) are visible to this row
    if (p.causal) hi = min(hi, q_pos + 1);
    int lo = 0;
    if (p.window > 0) lo = max(0, q_pos - p.window + 1);
    float m = -INFINITY, l = 0.f;
    uint8_t* prow = Ps + row * 128;

    for (int j = 0; j < n; j++) {
      const int b = j & 1;
      if (!mbar_wait(&s_ready[b], ((uint32_t)j >> 1) & 1u, abort_word)) goto done;
      tc_fence_after();
      const int tile_base = (t0 + j) << 7;
      // mask needed when the tile is not entirely inside every row's window
      const bool need_mask = (tile_base + 128 > min(seq_len, p.causal ? ctx + tok0 + 1 : seq_len)) ||
                             (p.window > 0);
      // ---- the whole score row lives in registers: one TMEM read, no second pass
      uint32_t sreg[128];
      tmem_ld_32x32b_x32(t_lane + b * 128, sreg);
      tmem_ld_32x32b_x32(t_lane + b * 128 + 32, sreg + 32);
      tmem_ld_32x32b_x32(t_lane + b * 128 + 64, sreg + 64);
      tmem_ld_32x32b_x32(t_lane + b * 128 + 96, sreg + 96);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[b]);
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < 128; i++) {
          const int key = tile_base + i;
          if (!(key >= lo && key < hi)) sreg[i] = 0xff800000u;   // -inf
        }
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < 128; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(sreg[i]));
        mx1 = fmaxf(mx1, __uint_as_float(sreg[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(sreg[i + 2]));
        mx3 = fmaxf(mx3, __uint_as_float(sreg[i + 3]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      float alpha = 1.f;
      bool need = false;
      if (mx > m) {
        if (j == 0 || m == -INFINITY || (mx - m) * sl2 > p.rescale_threshold) {
          alpha = (m == -INFINITY) ? 0.f : att_exp2((m - mx) * sl2);
          need = (j > 0) && (m != -INFINITY);   // an all-masked row has accumulated zeros only
          m = mx;
        }
      }
      l *= alpha;
      const bool warp_need = __any_sync(0xffffffffu, need && row_valid);
      // P buffer j&1 was last read by PV(j-2); O must be quiescent only for a rescale
      if (j >= 2) {
        if (!mbar_wait(&pv_done[j & 1], (((uint32_t)j - 2) >> 1) & 1u, abort_word)) goto done;
      }
      if (warp_need) {
        if (!mbar_wait(&pv_done[(j - 1) & 1], (((uint32_t)j - 1) >> 1) & 1u, abort_word)) goto done;
        tc_fence_after();
        const float a = need ? alpha : 1.f;
#pragma unroll 1
        for (int c = 0; c < D / 32; c++) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(t_lane + Cfg::O_COL + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i++) r[i] = __float_as_uint(__uint_as_float(r[i]) * a);
          tmem_st_32x32b_x32(t_lane + Cfg::O_COL + c * 32, r);
        }
        tmem_st_wait();
      }
      // ---- probabilities -> swizzled shared memory (A operand of P V)
      const float nmb = (m == -INFINITY) ? 0.f : -m * sl2;
      float rs0 = 0.f, rs1 = 0.f;
      uint8_t* pbuf = prow + (j & 1) * Cfg::P_BYTES;
#pragma unroll
      for (int c8 = 0; c8 < 16; c8++) {            // 16 chunks of 8 keys = one 16-byte store
        uint32_t pk[4];
#pragma unroll
        for (int q2 = 0; q2 < 4; q2++) {
          const int i = c8 * 8 + q2 * 2;
          const float p0 = att_exp2(fmaf(__uint_as_float(sreg[i]), sl2, nmb));
          const float p1 = att_exp2(fmaf(__uint_as_float(sreg[i + 1]), sl2, nmb));
          rs0 += p0;
          rs1 += p1;
          pk[q2] = pack_bf16x2(p0, p1);
        }
        const int chunk = c8 & 7;
        *reinterpret_cast<uint4*>(pbuf + (c8 >> 3) * ATT_HALF_BYTES + ((chunk ^ (row & 7)) << 4)) =
            make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
      l += rs0 + rs1;
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j & 1]);
    }
    // ---- epilogue
    if (!mbar_wait(&pv_done[(n - 1) & 1], (((uint32_t)n - 1) >> 1) & 1u, abort_word)) goto done;
    tc_fence_after();
    const float inv = l > 0.f ? 1.f / l : 0.f;
    const long tokidx = (long)q_start + tok0 + tok;
    const int hq = h * G + g;
#pragma unroll 1
    for (int c = 0; c < D / 32; c++) {
      uint32_t r[32];
      tmem_ld_32x32b_x32(t_lane + Cfg::O_COL + c * 32, r);
      tmem_ld_wait();
      if (row_valid) {
        if (p.num_splits == 1) {
          __nv_bfloat16* dst = p.out + tokidx * p.out_stride + (long)hq * D + c * 32;
#pragma unroll
          for (int q4 = 0; q4 < 4; q4++) {
            uint4 o;
            o.x = pack_bf16x2(__uint_as_float(r[q4 * 8 + 0]) * inv, __uint_as_float(r[q4 * 8 + 1]) * inv);
            o.y = pack_bf16x2(__uint_as_float(r[q4 * 8 + 2]) * inv, __uint_as_float(r[q4 * 8 + 3]) * inv);
            o.z = pack_bf16x2(__uint_as_float(r[q4 * 8 + 4]) * inv, __uint_as_float(r[q4 * 8 + 5]) * inv);
            o.w = pack_bf16x2(__uint_as_float(r[q4 * 8 + 6]) * inv, __uint_as_float(r[q4 * 8 + 7]) * inv);
            reinterpret_cast<uint4*>(dst)[q4] = o;
          }
        } else {
          const long pidx = (tokidx * p.Hq + hq) * p.num_splits + split;
          float* dst = p.partial_o + pidx * D + c * 32;
#pragma unroll
          for (int q4 = 0; q4 < 8; q4++) {
            float4 o = make_float4(__uint_as_float(r[q4 * 4 + 0]) * inv, __uint_as_float(r[q4 * 4 + 1]) * inv,
                                   __uint_as_float(r[q4 * 4 + 2]) * inv, __uint_as_float(r[q4 * 4 + 3]) * inv);
            reinterpret_cast<float4*>(dst)[q4] = o;
          }
          if (c == 0)
            p.partial_lse[pidx] =
                (l > 0.f) ? (m * sl2 * 0.6931471805599453f + logf(l)) : -INFINITY;
        }
      }
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    // let copies still in flight land before the CTA's shared memory is released
    const uint64_t t_start = globaltimer_ns();
    while (globaltimer_ns() - t_start < 50000ull) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, *abort_word);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ---------------------------------------------------------------- host
struct TmapCache {
  std::unordered_map<std::string, CUtensorMap> map;
  std::mutex mu;
  int get(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
          const uint64_t* strides, const uint32_t* box) {
    char key[200];
    memset(key, 0, sizeof(key));
    memcpy(key, &base, 8);
    memcpy(key + 8, dims, 8 * rank);
    memcpy(key + 48, strides, 8 * (rank - 1));
    memcpy(key + 88, box, 4 * rank);
    std::string k(key, 120);
    std::lock_guard<std::mutex> g(mu);
    auto it = map.find(k);
    if (it != map.end()) {
      *out = it->second;
      return 0;
    }
    int rc = make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, dims, strides, box,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (map.size() > 4096) map.clear();
    map.emplace(k, *out);
    return 0;
  }
};
static TmapCache g_att_tmaps;

template <int D>
static int launch_attn_tc(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                          const AttnParams& p, int num_tiles, cudaStream_t stream) {
  using Cfg = AttCfg<D>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_tc_kernel<D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (num_tiles > 65535) return 9125;
  dim3 grid((unsigned)p.Hkv, (unsigned)num_tiles, (unsigned)p.num_splits);
  attn_fwd_tc_kernel<D><<<grid, ATT_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, p);
  return B200_CHECK_LAUNCH();
}

}  // namespace b200

B200_API long b200_attn_scratch_bytes(long T, int Hq, int D, int num_splits) {
  if (num_splits <= 1) return 0;
  return T * Hq * num_splits * (long)(D + 1) * (long)sizeof(float);
}

// q: [T, Hq, D] bf16 with token stride q_stride (elements); caches
// [num_blocks, block_size, Hkv, D]; out [T, Hq, D] token stride out_stride.
// query_start_loc int32 [B+1], seq_lens int32 [B], block_table int32 [B, max_blocks].
// tile_seq / tile_qoff: int32 [num_tiles] work list (null => tile i is sequence
// i starting at its first query token; requires q_len <= 128/G).
// scratch: b200_attn_scratch_bytes() bytes when num_splits > 1.
// v_lbo / v_sbo = 0 selects the default V-operand descriptor offsets.
B200_API int b200_attn_fwd_tc(const void* q, long q_stride, long T, const void* k_cache,
                              const void* v_cache, long num_blocks, int block_size,
                              const void* query_start_loc, const void* seq_lens,
                              const void* block_table, int max_blocks, const void* tile_seq,
                              const void* tile_qoff, int num_tiles, int Hq, int Hkv, int D,
                              float scale, int causal, int window, int num_splits, void* out,
                              long out_stride, void* scratch, float rescale_threshold,
                              unsigned v_lbo, unsigned v_sbo, int kv_layout, int* status,
                              cudaStream_t stream) {
  using namespace b200;
  if (num_tiles <= 0 || T <= 0) return 0;
  const int G = Hq / Hkv;
  if (G * Hkv != Hq || G > 128 || (128 % G) != 0) return 9120;
  if (D != 128 && D != 64) return 9121;
  if (block_size < 8 || (block_size < 128 && (128 % block_size) != 0) ||
      (block_size > 128 && (block_size % 128) != 0))
    return 9122;
  if ((q_stride & 7) || (out_stride & 7)) return 9123;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && !scratch) return 9124;
  const int tok_per_tile = 128 / G;
  const int rpl = block_size < 128 ? block_size : 128;

  CUtensorMap tq, tk, tv;
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)G, (uint64_t)Hkv, (uint64_t)T};
    uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)G * D * 2, (uint64_t)q_stride * 2};
    uint32_t box[4] = {64, (uint32_t)G, 1, (uint32_t)tok_per_tile};
    int rc = g_att_tmaps.get(&tq, q, 4, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)block_size, (uint64_t)num_blocks};
    uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)Hkv * D * 2,
                       (uint64_t)block_size * Hkv * D * 2};
    if (kv_layout == 1) {   // [blocks, heads, tokens, D]
      str[0] = (uint64_t)block_size * D * 2;
      str[1] = (uint64_t)D * 2;
    }
    uint32_t box[4] = {64, 1, (uint32_t)rpl, 1};
    int rc = g_att_tmaps.get(&tk, k_cache, 4, dims, str, box);
    if (rc) return rc;
    rc = g_att_tmaps.get(&tv, v_cache, 4, dims, str, box);
    if (rc) return rc;
  }
  AttnParams p;
  p.query_start_loc = (const int*)query_start_loc;
  p.seq_lens = (const int*)seq_lens;
  p.block_table = (const int*)block_table;
  p.tile_seq = (const int*)tile_seq;
  p.tile_qoff = (const int*)tile_qoff;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.rows_per_load = rpl;
  p.G = G; p.Hkv = Hkv; p.Hq = Hq;
  p.tok_per_tile = tok_per_tile;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.causal = causal; p.window = window; p.num_splits = num_splits;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.partial_o = (float*)scratch;
  p.partial_lse = scratch ? (float*)scratch + T * Hq * (long)num_splits * D : nullptr;
  p.num_blocks_total = num_blocks;
  p.status = status;
  p.v_lbo = v_lbo ? v_lbo : (uint32_t)ATT_HALF_BYTES;
  p.v_sbo = v_sbo ? v_sbo : 1024u;
  p.rescale_threshold = rescale_threshold;
  int rc = (D == 128) ? launch_attn_tc<128>(tq, tk, tv, p, num_tiles, stream)
                      : launch_attn_tc<64>(tq, tk, tv, p, num_tiles, stream);
  if (rc) return rc;
  if (num_splits > 1)
    return launch_merge_splits(p.partial_o, p.partial_lse, T, Hq, num_splits, D, out,
                               out_stride, stream);
  return 0;
}
