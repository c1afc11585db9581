// Absorbed-weight MLA decode attention on tcgen05.
//
// Per token the cache holds one normalised latent (512) and one RoPE key slice (64); every
// head attends with a 576-wide query (q_nope absorbed through W_UK, plus q_pe) and reads the
// latent again as its value.  So this is MQA with one shared 576-wide key that is also the
// value, and the kernel keeps ONE copy of a 128-key tile in shared memory and uses it as
// both MMA operands, in "keys on the M axis" form:
//   S^T[128 keys, NQ heads]  = KV_tile[128, 576] . Q^T        (A = 9 slabs of 64 columns, K-major)
//   O^T[512, NQ heads]      += latent_tile^T[512, 128 keys] . P^T   (A = the same slabs, MN-major,
//                                                                   four M=128 blocks of d)
// A tile is 147 KB, so there is one tile buffer; it is refilled slab by slab: the two slabs of
// value block b are handed back to the TMA producer as soon as PV block b has been issued, so
// the next tile streams in behind the current tile's PV MMAs.  S^T and the four O^T blocks live
// in TMEM (6 * NQ columns).  One CTA serves NQ (16 or 32) heads of one query row; split-KV
// partials are merged by log-sum-exp.
//
// Parity: the decode branch of the reference's MLA backend (MQA over the latent cache with the
// rope side input, vllm_ascend/attention/mla_v1.py:1373-1577).  All waits are bounded.
#include "attention.h"
#include "common.cuh"

#include <mutex>
#include <string.h>
#include <string>
#include <unordered_map>

namespace b200 {

constexpr int MLA_THREADS = 192;
constexpr int MLA_DC = 512;
constexpr int MLA_DR = 64;
constexpr int MLA_SLABS = 9;               // 8 latent slabs + 1 rope slab of 64 columns
constexpr int MLA_SLAB = 128 * 128;        // 128 keys x 64 bf16
constexpr float kMlaRescaleLog2 = 8.f;

struct MlaParams {
  const int* row_seq;       // [R] block-table row of each query row
  const int* row_kv_len;    // [R] keys visible to the query row
  const int* block_table;
  int max_blocks, block_size, rows_per_load;
  int H;
  float scale_log2;
  int num_splits;
  __nv_bfloat16* out;       // [R, H, 512]
  long out_stride;          // elements between rows
  float* partial_o;
  float* partial_lse;
  long num_blocks_total;
  int* status;
};

template <int NQ>
struct MlaCfg {
  static constexpr int Q_SLAB = NQ * 128;
  static constexpr int Q_BYTES = MLA_SLABS * Q_SLAB;
  static constexpr int TILE_BYTES = MLA_SLABS * MLA_SLAB;
  static constexpr int P_HALF = NQ * 128;           // NQ rows x 64 keys
  static constexpr int P_BYTES = 2 * P_HALF;
  static constexpr int MISC_BYTES = 2048;           // barriers, tmem pointer, reduction scratch
  static constexpr int SMEM_BYTES = TILE_BYTES + Q_BYTES + 2 * P_BYTES + MISC_BYTES + 1024;
  static constexpr int TMEM_COLS = NQ == 16 ? 128 : 256;
  static constexpr int O_COL = 2 * NQ;
};

__device__ __forceinline__ float mla_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void mla_softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int NQ>
__device__ __forceinline__ void mla_tmem_ld(uint32_t addr, uint32_t* r) {
  if constexpr (NQ == 16) tmem_ld_32x32b_x16(addr, r); else tmem_ld_32x32b_x32(addr, r);
}
template <int NQ>
__device__ __forceinline__ void mla_tmem_st(uint32_t addr, const uint32_t* r) {
  if constexpr (NQ == 16) tmem_st_32x32b_x16(addr, r); else tmem_st_32x32b_x32(addr, r);
}

template <int NQ>
__global__ void __launch_bounds__(MLA_THREADS, 1)
mla_decode_kernel(const __grid_constant__ CUtensorMap tmap_q,
                  const __grid_constant__ CUtensorMap tmap_lat,
                  const __grid_constant__ CUtensorMap tmap_pe, const MlaParams p) {
  using Cfg = MlaCfg<NQ>;
  const int hb = blockIdx.x, row = blockIdx.y, split = blockIdx.z;
  const int kv_len = p.row_kv_len[row];
  const int seq = p.row_seq[row];
  const int n_all = (kv_len + 127) >> 7;
  const int per_split = (n_all + p.num_splits - 1) / p.num_splits;
  const int t0 = split * per_split;
  const int t1 = min(n_all, t0 + per_split);
  const int n = t1 - t0;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (n <= 0) {
    if (p.num_splits > 1) {
      for (int c = threadIdx.x; c < NQ; c += blockDim.x) {
        const long pidx = ((long)row * p.H + hb * NQ + c) * p.num_splits + split;
        p.partial_lse[pidx] = -INFINITY;
        for (int d = 0; d < MLA_DC; d++) p.partial_o[pidx * MLA_DC + d] = 0.f;
      }
    } else {
      for (int i = threadIdx.x; i < NQ * MLA_DC; i += blockDim.x)
        p.out[(long)row * p.out_stride + (long)(hb * NQ) * MLA_DC + i] = __float2bfloat16(0.f);
    }
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* KVs = smem;
  uint8_t* Qs = KVs + Cfg::TILE_BYTES;
  uint8_t* Ps = Qs + Cfg::Q_BYTES;
  uint64_t* bars = (uint64_t*)(Ps + 2 * Cfg::P_BYTES);
  uint64_t* q_full = bars;                 // 1
  uint64_t* h_full = bars + 1;             // 9
  uint64_t* h_empty = h_full + MLA_SLABS;  // 9
  uint64_t* s_ready = h_empty + MLA_SLABS; // 2
  uint64_t* s_free = s_ready + 2;          // 2
  uint64_t* p_ready = s_free + 2;          // 2
  uint64_t* pv_done = p_ready + 2;         // 2
  uint32_t* tmem_ptr = (uint32_t*)(pv_done + 2);
  volatile int* abort_word = (volatile int*)(tmem_ptr + 1);
  int* redi = (int*)(tmem_ptr + 4);        // [2 tiles][4 warps][NQ]
  float* redf = (float*)(redi + 2 * 4 * NQ);   // [4 warps][NQ]

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < MLA_SLABS; s++) {
      mbar_init(&h_full[s], 1);
      mbar_init(&h_empty[s], 1);
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
    tma_prefetch_desc(&tmap_lat);
    tma_prefetch_desc(&tmap_pe);
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
      mbar_expect_tx(q_full, Cfg::Q_BYTES);
#pragma unroll
      for (int s = 0; s < MLA_SLABS; s++)
        tma_load_3d(Qs + s * Cfg::Q_SLAB, &tmap_q, q_full, s * 64, hb * NQ, row);
    }
    for (int j = 0; j < n; j++) {
      const uint32_t ph = (uint32_t)j & 1u;
      const int key_base = (t0 + j) << 7;
      int blk = 0;
      if (lane < parts) blk = bt[min(key_base + lane * rpl, kv_len - 1) / p.block_size];
      bool bad = lane < parts && (blk < 0 || blk >= p.num_blocks_total);
      bad = __any_sync(0xffffffffu, bad);
      if (bad) {
        *abort_word = B200_BAD_INDEX;
        goto done;
      }
#pragma unroll 1
      for (int s = 0; s < MLA_SLABS; s++) {
        if (!mbar_wait(&h_empty[s], ph ^ 1u, abort_word)) goto done;
        for (int part = 0; part < parts; part++) {
          const int b = __shfl_sync(0xffffffffu, blk, part);
          if (lane == 0) {
            if (part == 0) mbar_expect_tx(&h_full[s], MLA_SLAB);
            const int off = (key_base + part * rpl) % p.block_size;
            uint8_t* dst = KVs + s * MLA_SLAB + part * rpl * 128;
            if (s < 8) tma_load_3d(dst, &tmap_lat, &h_full[s], s * 64, off, b);
            else tma_load_3d(dst, &tmap_pe, &h_full[s], 0, off, b);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc_f16(128, NQ, true, false, false);
    constexpr uint32_t idesc_o = make_idesc_f16(128, NQ, true, true, false);   // A = latent^T, MN-major
    const uint32_t q_addr = smem_u32(Qs), kv_addr = smem_u32(KVs), p_addr = smem_u32(Ps);
    if (!mbar_wait(q_full, 0, abort_word)) goto done;
    for (int j = 0; j < n; j++) {
      const uint32_t ph = (uint32_t)j & 1u;
      const int b = j & 1;
      if (!mbar_wait(&s_free[b], (((uint32_t)j >> 1) & 1u) ^ 1u, abort_word)) goto done;
#pragma unroll 1
      for (int s = 0; s < MLA_SLABS; s++) {
        if (!mbar_wait(&h_full[s], ph, abort_word)) goto done;
        tc_fence_after();
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < 4; kk++) {
            const uint64_t da = make_smem_desc(kv_addr + s * MLA_SLAB + kk * 32, 16, 1024, kLayoutSw128);
            const uint64_t db = make_smem_desc(q_addr + s * Cfg::Q_SLAB + kk * 32, 16, 1024, kLayoutSw128);
            umma_f16_ss(tmem_base + b * NQ, da, db, idesc_s, (s > 0 || kk > 0) ? 1u : 0u);
          }
          if (s == MLA_SLABS - 1) {
            umma_commit(&h_empty[s]);        // the rope slab is not a value operand
            umma_commit(&s_ready[b]);
          }
        }
        __syncwarp();
      }
      if (!mbar_wait(&p_ready[b], ((uint32_t)j >> 1) & 1u, abort_word)) goto done;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll 1
        for (int blk = 0; blk < 4; blk++) {
#pragma unroll
          for (int kk = 0; kk < 8; kk++) {
            // A: 16 keys of latent^T for d in [128 blk, 128 blk + 128): two 64-wide d atoms one
            // slab apart, 8-key groups 1024 B apart
            const uint64_t da = make_smem_desc(kv_addr + (2 * blk) * MLA_SLAB + kk * 2048, MLA_SLAB,
                                               1024, kLayoutSw128);
            const uint64_t db = make_smem_desc(
                p_addr + b * Cfg::P_BYTES + (kk >> 2) * Cfg::P_HALF + (kk & 3) * 32, 16, 1024,
                kLayoutSw128);
            umma_f16_ss(tmem_base + Cfg::O_COL + blk * NQ, da, db, idesc_o,
                        (j > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&h_empty[2 * blk]);
          umma_commit(&h_empty[2 * blk + 1]);
        }
        umma_commit(&pv_done[b]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue
    const int qd = warp & 3;
    const int tid = qd * 32 + lane;                 // key inside the tile; d inside a value block
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl2 = p.scale_log2;
    float m[NQ], lsum[NQ];
#pragma unroll
    for (int c = 0; c < NQ; c++) {
      m[c] = -INFINITY;
      lsum[c] = 0.f;
    }
    for (int j = 0; j < n; j++) {
      const int b = j & 1;
      if (!mbar_wait(&s_ready[b], ((uint32_t)j >> 1) & 1u, abort_word)) goto done;
      tc_fence_after();
      uint32_t r[NQ];
      mla_tmem_ld<NQ>(t_lane + b * NQ, r);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[b]);
      const int key = ((t0 + j) << 7) + tid;
      const bool visible = key < kv_len;
      float s[NQ];
      int* rj = redi + (j & 1) * 4 * NQ + qd * NQ;
#pragma unroll
      for (int c = 0; c < NQ; c++) {
        s[c] = visible ? __uint_as_float(r[c]) : -INFINITY;
        int ob = __float_as_int(s[c]);
        ob ^= (ob >> 31) & 0x7fffffff;              // order-preserving float -> int
        const int wm = __reduce_max_sync(0xffffffffu, ob);
        if (lane == 0) rj[c] = wm;
      }
      mla_softmax_bar();
      const int* ra = redi + (j & 1) * 4 * NQ;
      bool any_change = false;
      float alpha[NQ];
#pragma unroll
      for (int c = 0; c < NQ; c++) {
        int t = max(max(ra[c], ra[NQ + c]), max(ra[2 * NQ + c], ra[3 * NQ + c]));
        t ^= (t >> 31) & 0x7fffffff;
        const float mn = fmaxf(m[c], __int_as_float(t));
        alpha[c] = 1.f;
        if (mn > m[c] && (m[c] == -INFINITY || (mn - m[c]) * sl2 > kMlaRescaleLog2)) {
          alpha[c] = (m[c] == -INFINITY) ? 0.f : mla_exp2((m[c] - mn) * sl2);
          any_change = any_change || (m[c] != -INFINITY);
          m[c] = mn;
        }
        lsum[c] *= alpha[c];
      }
      if (j >= 2) {      // P buffer j&1 was last read by PV(j-2)
        if (!mbar_wait(&pv_done[j & 1], (((uint32_t)j - 2) >> 1) & 1u, abort_word)) goto done;
      }
      if (j > 0 && any_change) {    // uniform over the 128 threads: O^T must be quiescent
        if (!mbar_wait(&pv_done[(j - 1) & 1], (((uint32_t)j - 1) >> 1) & 1u, abort_word)) goto done;
        tc_fence_after();
#pragma unroll 1
        for (int blk = 0; blk < 4; blk++) {
          uint32_t o[NQ];
          mla_tmem_ld<NQ>(t_lane + Cfg::O_COL + blk * NQ, o);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < NQ; c++) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha[c]);
          mla_tmem_st<NQ>(t_lane + Cfg::O_COL + blk * NQ, o);
        }
        tmem_st_wait();
      }
      // probabilities of this key for every head -> P[head][key] (K-major, swizzled)
      uint8_t* pbase = Ps + (j & 1) * Cfg::P_BYTES + (tid >> 6) * Cfg::P_HALF;
      const int kin = tid & 63;
#pragma unroll
      for (int c = 0; c < NQ; c++) {
        const float mb = (m[c] == -INFINITY) ? 0.f : m[c] * sl2;
        const float pv = mla_exp2(s[c] * sl2 - mb);
        lsum[c] += pv;
        const int chunk = (kin >> 3) ^ (c & 7);
        *reinterpret_cast<__nv_bfloat16*>(pbase + c * 128 + (chunk << 4) + (kin & 7) * 2) =
            __float2bfloat16(pv);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[j & 1]);
    }
    // ---- epilogue
    if (!mbar_wait(&pv_done[(n - 1) & 1], (((uint32_t)n - 1) >> 1) & 1u, abort_word)) goto done;
    tc_fence_after();
    mla_softmax_bar();
#pragma unroll
    for (int c = 0; c < NQ; c++) {
      const float w = warp_reduce_sum(lsum[c]);
      if (lane == 0) redf[qd * NQ + c] = w;
    }
    mla_softmax_bar();
    float inv[NQ], lse[NQ];
#pragma unroll
    for (int c = 0; c < NQ; c++) {
      const float l = redf[c] + redf[NQ + c] + redf[2 * NQ + c] + redf[3 * NQ + c];
      inv[c] = l > 0.f ? 1.f / l : 0.f;
      lse[c] = l > 0.f ? (m[c] * sl2 * 0.6931471805599453f + logf(l)) : -INFINITY;
    }
#pragma unroll 1
    for (int blk = 0; blk < 4; blk++) {
      uint32_t o[NQ];
      mla_tmem_ld<NQ>(t_lane + Cfg::O_COL + blk * NQ, o);
      tmem_ld_wait();
      const int d = blk * 128 + tid;
#pragma unroll
      for (int c = 0; c < NQ; c++) {
        const int head = hb * NQ + c;
        const float val = __uint_as_float(o[c]) * inv[c];
        if (p.num_splits == 1) {
          p.out[(long)row * p.out_stride + (long)head * MLA_DC + d] = __float2bfloat16(val);
        } else {
          const long pidx = ((long)row * p.H + head) * p.num_splits + split;
          p.partial_o[pidx * MLA_DC + d] = val;
          if (d == 0) p.partial_lse[pidx] = lse[c];
        }
      }
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
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

struct MlaTmapCache {
  std::unordered_map<std::string, CUtensorMap> map;
  std::mutex mu;
  int get(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
          const uint64_t* strides, const uint32_t* box) {
    char key[96];
    memset(key, 0, sizeof(key));
    memcpy(key, &base, 8);
    memcpy(key + 8, dims, 8 * rank);
    memcpy(key + 40, strides, 8 * (rank - 1));
    memcpy(key + 64, box, 4 * rank);
    std::string k(key, 96);
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
static MlaTmapCache g_mla_tmaps;

template <int NQ>
static int launch_mla(const CUtensorMap& tq, const CUtensorMap& tl, const CUtensorMap& tp,
                      const MlaParams& p, dim3 grid, cudaStream_t stream) {
  using Cfg = MlaCfg<NQ>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(mla_decode_kernel<NQ>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  mla_decode_kernel<NQ><<<grid, MLA_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tl, tp, p);
  return B200_CHECK_LAUNCH();
}

}  // namespace b200

// q: [R, H, 576] bf16 (absorbed q_nope (512) then q_pe (64)), row stride q_stride elements.
// lat_cache [blocks, block_size, 512], pe_cache [blocks, block_size, 64] (bf16, dense).
// row_seq / row_kv_len: int32 [R]: block-table row and visible key count of every query row
// (a decode token sees all of its sequence; row t of a multi-token query sees ctx + t + 1).
// out: [R, H, 512].  scratch: R * H * num_splits * 513 floats when num_splits > 1.
// lse_out (optional, fp32 [R, H]): log-sum-exp of every (row, head) over the keys the row saw, for
// callers that merge the results of several calls (context-parallel ranks).  It is produced by the
// split merge, so a call that wants it runs with at least two KV splits.
B200_API int b200_mla_decode_lse(const void* q, long q_stride, long R, int H, const void* lat_cache,
                                 const void* pe_cache, long num_blocks, int block_size,
                                 const void* row_seq, const void* row_kv_len,
                                 const void* block_table, int max_blocks, float scale,
                                 int num_splits, void* out, long out_stride, void* scratch,
                                 void* lse_out, int* status, cudaStream_t stream) {
  using namespace b200;
  if (R <= 0) return 0;
  if (lse_out && num_splits < 2) num_splits = 2;
  if (H % 16) return 9500;
  if (block_size < 8 || (block_size < 128 && (128 % block_size) != 0) ||
      (block_size > 128 && (block_size % 128) != 0))
    return 9501;
  if ((q_stride & 7) || (out_stride & 7)) return 9502;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && !scratch) return 9503;
  if (R > 65535 || num_splits > 65535) return 9504;
  const int NQ = (H % 32 == 0) ? 32 : 16;
  const int rpl = block_size < 128 ? block_size : 128;
  CUtensorMap tq, tl, tp;
  {
    uint64_t dims[3] = {(uint64_t)(MLA_DC + MLA_DR), (uint64_t)H, (uint64_t)R};
    uint64_t str[2] = {(uint64_t)(MLA_DC + MLA_DR) * 2, (uint64_t)q_stride * 2};
    uint32_t box[3] = {64, (uint32_t)NQ, 1};
    int rc = g_mla_tmaps.get(&tq, q, 3, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)MLA_DC, (uint64_t)block_size, (uint64_t)num_blocks};
    uint64_t str[2] = {(uint64_t)MLA_DC * 2, (uint64_t)block_size * MLA_DC * 2};
    uint32_t box[3] = {64, (uint32_t)rpl, 1};
    int rc = g_mla_tmaps.get(&tl, lat_cache, 3, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)MLA_DR, (uint64_t)block_size, (uint64_t)num_blocks};
    uint64_t str[2] = {(uint64_t)MLA_DR * 2, (uint64_t)block_size * MLA_DR * 2};
    uint32_t box[3] = {64, (uint32_t)rpl, 1};
    int rc = g_mla_tmaps.get(&tp, pe_cache, 3, dims, str, box);
    if (rc) return rc;
  }
  MlaParams p;
  p.row_seq = (const int*)row_seq;
  p.row_kv_len = (const int*)row_kv_len;
  p.block_table = (const int*)block_table;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.rows_per_load = rpl;
  p.H = H;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.num_splits = num_splits;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.partial_o = (float*)scratch;
  p.partial_lse = scratch ? (float*)scratch + R * H * (long)num_splits * MLA_DC : nullptr;
  p.num_blocks_total = num_blocks;
  p.status = status;
  dim3 grid((unsigned)(H / NQ), (unsigned)R, (unsigned)num_splits);
  int rc = (NQ == 32) ? launch_mla<32>(tq, tl, tp, p, grid, stream)
                      : launch_mla<16>(tq, tl, tp, p, grid, stream);
  if (rc) return rc;
  if (num_splits > 1)
    return launch_merge_splits(p.partial_o, p.partial_lse, R, H, num_splits, MLA_DC, out,
                               out_stride, stream, (float*)lse_out);
  return 0;
}

B200_API int b200_mla_decode(const void* q, long q_stride, long R, int H, const void* lat_cache,
                             const void* pe_cache, long num_blocks, int block_size,
                             const void* row_seq, const void* row_kv_len, const void* block_table,
                             int max_blocks, float scale, int num_splits, void* out,
                             long out_stride, void* scratch, int* status, cudaStream_t stream) {
  return b200_mla_decode_lse(q, q_stride, R, H, lat_cache, pe_cache, num_blocks, block_size, row_seq,
                             row_kv_len, block_table, max_blocks, scale, num_splits, out,
                             out_stride, scratch, nullptr, status, stream);
}
