// Flash-decode on tcgen05 in "keys on the M axis" form, for sequences with at most
// 16 / G query tokens (decode and short speculative verification).
//
// Decode attention streams the whole KV cache once and is bound by HBM, so the
// kernel is organised around the K/V stream instead of around query rows:
//   S^T[128 keys, 16] = K_tile[128 keys, D] . Q^T          (A = K, K-major; B = Q, K-major)
//   O^T[D, 16]      += V_tile^T[D, 128 keys] . P^T         (A = V, MN-major; B = P, K-major)
// The 16 columns are the (token, head-of-group) rows that share this KV head.
// Every softmax thread owns one key of the tile (one TMEM lane): it masks and
// exponentiates only the valid columns, the per-column max is reduced across the
// 128 threads, and the running row sums stay thread-local until the end.  K and V
// pages arrive through a 3-stage TMA pipeline; accumulators live in TMEM
// (S^T double-buffered, 16 columns each; O^T 16 columns).
//
// Parity: the reference's paged decode path (_npu_paged_attention,
// vllm_ascend/attention/attention_v1.py:1555-1574) incl. split-KV partials merged
// by log-sum-exp (npu_attention_update).  All waits are bounded.
#include "attention.h"
#include "common.cuh"

#include <mutex>
#include <string.h>
#include <string>
#include <unordered_map>

namespace b200 {

constexpr int DEC_THREADS = 192;
constexpr int DEC_NQ = 16;                 // MMA N: query rows per CTA
constexpr int DEC_HALF = 128 * 128;        // 128 keys x 64 bf16
constexpr int DEC_QHALF = DEC_NQ * 128;    // 16 rows x 64 bf16
constexpr float kRescaleLog2 = 8.f;

struct DecParams {
  const int* query_start_loc;
  const int* seq_lens;
  const int* block_table;
  int max_blocks, block_size, rows_per_load;
  int G, Hkv, Hq;
  float scale_log2;
  int window, num_splits;
  __nv_bfloat16* out;
  long out_stride;
  float* partial_o;
  float* partial_lse;
  float* lse_out;            // optional [T, Hq] natural-log sum-exp of the scaled scores (-inf: no key)
  long num_blocks_total;
  int num_seqs, num_items;   // items = Hkv x sequences x splits
  int tail_loads;            // 1: the last tile of a sequence is loaded in 32-key pieces (pages >= 128 keys)
  int l2_prefetch;           // tiles the L2 prefetch of K / V runs ahead of the staged loads (0 = off)
  int* status;
  long long* timeline;   // optional [3 roles][64 tiles][8 stamps] of clock64, CTA 0 only
};

template <int D>
struct DecCfg {
  static constexpr int NH = D / 64;
  static constexpr int STAGES = 3;
  static constexpr int TILE_BYTES = NH * DEC_HALF;
  static constexpr int Q_BYTES = NH * DEC_QHALF;
  static constexpr int P_BYTES = 2 * DEC_QHALF;     // one P buffer (two 64-key halves)
  static constexpr int P_BUFS = 2;                  // double-buffered so P(j+1) overlaps PV(j)
  static constexpr int SMEM_BYTES =
      2 * STAGES * TILE_BYTES + 2 * Q_BYTES + P_BUFS * P_BYTES + 1024 + 1024;
  static constexpr int TMEM_COLS = 64;
  static constexpr int O_COL = 32;                  // two O^T accumulators: columns 32..47, 48..63
};

// Device-side timeline: stamp k of tile j for a role (0 producer, 1 MMA issuer, 2 softmax).
#define DEC_STAMP(role, j, k)                                                            \
  do {                                                                                 \
    if (tl && (j) < 64u) tl[((role) * 64 + (j)) * 8 + (k)] = clock64() - tl_t0;         \
  } while (0)

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ void softmax_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// One work item = (KV head, sequence, KV split).  The kernel is persistent: CTA b serves items
// b, b + gridDim.x, ... and the three roles keep running tile / item counters, so barrier
// initialisation, the TMEM allocation and the pipeline fill are paid once per CTA, the K/V
// stream of the next item is already in flight while the current item's epilogue runs, and
// a short item (a few tiles) costs no more than its bytes.
struct DecItem {
  int h, seq, split;
  int q_start, q_len, seq_len, ctx, t0, n;
};

// The three words of an item that live in global memory.  They are loaded one item ahead
// (dec_load) and turned into a DecItem (dec_make, arithmetic only) when the item starts, so no
// role waits for a dependent global load at an item boundary.
struct DecRaw {
  int q0, q1, seq_len;
};

__device__ __forceinline__ DecRaw dec_load(const DecParams& p, int item) {
  const int seq = (item / p.Hkv) % p.num_seqs;
  DecRaw r;
  r.q0 = p.query_start_loc[seq];
  r.q1 = p.query_start_loc[seq + 1];
  r.seq_len = p.seq_lens[seq];
  return r;
}

__device__ __forceinline__ DecItem dec_make(const DecParams& p, int item, const DecRaw& r) {
  DecItem w;
  w.h = item % p.Hkv;
  const int q = item / p.Hkv;
  w.seq = q % p.num_seqs;
  w.split = q / p.num_seqs;
  w.q_start = r.q0;
  w.q_len = r.q1 - r.q0;
  w.seq_len = r.seq_len;
  w.ctx = w.seq_len - w.q_len;
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, w.ctx - p.window + 1);
  const int tile_lo = kv_lo >> 7, tile_hi = (w.seq_len + 127) >> 7;
  const int n_all = tile_hi - tile_lo;
  const int per_split = (n_all + p.num_splits - 1) / p.num_splits;
  w.t0 = tile_lo + w.split * per_split;
  w.n = w.q_len > 0 ? max(0, min(tile_hi, w.t0 + per_split) - w.t0) : 0;
  return w;
}

__device__ __forceinline__ DecItem dec_item(const DecParams& p, int item) {
  return dec_make(p, item, dec_load(p, item));
}

template <int D, int NVT>
__global__ void __launch_bounds__(DEC_THREADS, 1)
attn_decode_tc_kernel(const __grid_constant__ CUtensorMap tmap_q,
                      const __grid_constant__ CUtensorMap tmap_k,
                      const __grid_constant__ CUtensorMap tmap_v,
                      const __grid_constant__ CUtensorMap tmap_k32,
                      const __grid_constant__ CUtensorMap tmap_v32, const DecParams p) {
  using Cfg = DecCfg<D>;
  constexpr int NH = Cfg::NH, ST = Cfg::STAGES;
  const int G = p.G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  long long* tl = (p.timeline && blockIdx.x == 0 && lane == 0) ? p.timeline : nullptr;
  const long long tl_t0 = clock64();

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* Ks = smem;
  uint8_t* Vs = Ks + ST * Cfg::TILE_BYTES;
  uint8_t* Qs = Vs + ST * Cfg::TILE_BYTES;          // two Q buffers
  uint8_t* Ps = Qs + 2 * Cfg::Q_BYTES;
  uint64_t* bars = (uint64_t*)(Ps + Cfg::P_BUFS * Cfg::P_BYTES);
  uint64_t* q_full = bars;            // 2
  uint64_t* q_empty = q_full + 2;     // 2
  uint64_t* k_full = q_empty + 2;     // ST
  uint64_t* k_empty = k_full + ST;    // ST
  uint64_t* v_full = k_empty + ST;    // ST
  uint64_t* v_empty = v_full + ST;    // ST
  uint64_t* s_ready = v_empty + ST;   // 2
  uint64_t* s_free = s_ready + 2;     // 2
  uint64_t* p_ready = s_free + 2;     // 2 (per P buffer)
  uint64_t* pv_done = p_ready + 2;    // 2 (per P buffer)
  uint64_t* o_free = pv_done + 2;     // 2 (per O accumulator)
  uint32_t* tmem_ptr = (uint32_t*)(o_free + 2);
  volatile int* abort_word = (volatile int*)(tmem_ptr + 1);
  float* red = (float*)(tmem_ptr + 2);            // [2 tiles][4 warps][16] maxima
  float* red_sum = red + 128;                     // [4 warps][16] row sums of the epilogue

  if (p.tail_loads) {
    // The last tile of a sequence is fetched in 32-key pieces up to its length; the rest of the
    // stage keeps what an earlier tile left there.  Those keys are masked (P = 0), so all that is
    // asked of the stale rows is that they are finite: start from zeros instead of whatever the
    // shared memory held.
    uint4* z = reinterpret_cast<uint4*>(Ks);
    for (int i = threadIdx.x; i < 2 * ST * Cfg::TILE_BYTES / 16; i += DEC_THREADS)
      z[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async_smem();
  }
  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; b++) {
      mbar_init(&q_full[b], 1);
      mbar_init(&q_empty[b], 1);
      mbar_init(&s_ready[b], 1);
      mbar_init(&s_free[b], 4);
      mbar_init(&p_ready[b], 4);
      mbar_init(&pv_done[b], 1);
      mbar_init(&o_free[b], 4);
    }
    for (int s = 0; s < ST; s++) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
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
    if (p.tail_loads) {
      tma_prefetch_desc(&tmap_k32);
      tma_prefetch_desc(&tmap_v32);
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const int num_items = p.num_items;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    const int rpl = p.rows_per_load;
    const int parts = 128 / rpl;
    uint32_t gt = 0, it = 0;             // tiles / items issued so far by this CTA
    // The description of an item (two dependent global loads) and the block ids of its first tile
    // (a third) are fetched while the previous item streams, so that the first TMA of an item
    // can follow the last TMA of its predecessor without a gap and the K/V pipeline stays full
    // across item boundaries.
    auto first_blk = [&](const DecItem& d) -> int {
      if (d.n <= 0 || lane >= parts) return 0;
      const int key0 = (d.t0 << 7) + lane * rpl;
      return p.block_table[(long)d.seq * p.max_blocks + min(key0, d.seq_len - 1) / p.block_size];
    };
    DecItem w_next;
    DecRaw raw_next = {0, 0, 0};          // words of the item after the next one
    int blk_first_next = 0;
    w_next.n = 0;
    if ((int)blockIdx.x < num_items) {
      w_next = dec_item(p, blockIdx.x);
      blk_first_next = first_blk(w_next);
      if ((int)(blockIdx.x + gridDim.x) < num_items) raw_next = dec_load(p, blockIdx.x + gridDim.x);
    }
    auto advance = [&](int item_after) {
      if (item_after < num_items) {
        w_next = dec_make(p, item_after, raw_next);
        blk_first_next = first_blk(w_next);
        if (item_after + (int)gridDim.x < num_items) raw_next = dec_load(p, item_after + gridDim.x);
      }
    };
    // The query rows of an item go into Q buffer (its index among the non-empty items) & 1; the
    // buffer of the item after the current one is free (its last reader was two items ago), so
    // that load is issued one item early as well and never sits in front of an item's first MMA.
    auto load_q = [&](uint32_t idx, const DecItem& d) -> bool {
      const int b = idx & 1;
      if (!mbar_wait(&q_empty[b], ((idx >> 1) & 1u) ^ 1u, abort_word)) return false;
      if (lane == 0) {
        mbar_expect_tx(&q_full[b], Cfg::Q_BYTES);
#pragma unroll
        for (int hf = 0; hf < NH; hf++)
          tma_load_4d(Qs + b * Cfg::Q_BYTES + hf * DEC_QHALF, &tmap_q, &q_full[b], hf * 64, 0, d.h, d.q_start);
      }
      __syncwarp();
      return true;
    };
    bool q_ahead = false;                // the next non-empty item's Q load was already issued
    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
      const DecItem w = w_next;
      int blk_cur = blk_first_next;
      const int item_after = item + gridDim.x;
      if (w.n <= 0) {
        advance(item_after);
        continue;
      }
      const int* bt = p.block_table + (long)w.seq * p.max_blocks;
      if (!q_ahead) {
        if (!load_q(it, w)) goto done;
      }
      q_ahead = false;
      // Block ids are fetched one tile ahead (lane p holds the id of part p), so the
      // dependent global load never sits between a freed stage and the next TMA issue.
      auto load_blk = [&](int j) -> int {
        if (j >= w.n || lane >= parts) return 0;
        const int key0 = ((w.t0 + j) << 7) + lane * rpl;
        return bt[min(key0, w.seq_len - 1) / p.block_size];
      };
      for (int j = 0; j < w.n; j++, gt++) {
        const int st = gt % ST;
        const uint32_t ph = (gt / ST) & 1u;
        const int key_base = (w.t0 + j) << 7;
        const int blk_next = load_blk(j + 1);
        if (p.l2_prefetch > 0 && j + p.l2_prefetch < w.n) {
          // ask for a later tile's pages in L2 now: the bytes in flight towards shared memory are
          // bounded by the stage ring, requests towards L2 are not
          const int jp = j + p.l2_prefetch;
          const int blk_pf = load_blk(jp);
          if (lane < parts && blk_pf >= 0 && blk_pf < p.num_blocks_total) {
            const int off = (((w.t0 + jp) << 7) + lane * rpl) % p.block_size;
#pragma unroll
            for (int hf = 0; hf < NH; hf++) {
              tma_prefetch_l2_4d(&tmap_k, hf * 64, w.h, off, blk_pf);
              tma_prefetch_l2_4d(&tmap_v, hf * 64, w.h, off, blk_pf);
            }
          }
        }
        bool bad = blk_cur < 0 || blk_cur >= p.num_blocks_total;
        bad = __any_sync(0xffffffffu, bad && lane < parts);
#pragma unroll 1
        for (int kv = 0; kv < 2; kv++) {
          uint64_t* fullb = kv == 0 ? &k_full[st] : &v_full[st];
          uint64_t* emptyb = kv == 0 ? &k_empty[st] : &v_empty[st];
          if (!mbar_wait(emptyb, ph ^ 1u, abort_word)) goto done;
          DEC_STAMP(0, gt, kv);
          if (bad) {
            *abort_word = B200_BAD_INDEX;
            goto done;
          }
          // 32-key pieces of the tile that hold keys of the sequence (4 = the whole tile)
          int nsub = 4;
          if (p.tail_loads) {
            const int valid = w.seq_len - key_base;
            if (valid < 128) nsub = (valid + 31) >> 5;
          }
          if (nsub < 4) {
            const int blk = __shfl_sync(0xffffffffu, blk_cur, 0);
            if (lane == 0) {
              uint8_t* dst = (kv == 0 ? Ks : Vs) + st * Cfg::TILE_BYTES;
              const CUtensorMap* tm = kv == 0 ? &tmap_k32 : &tmap_v32;
              mbar_expect_tx(fullb, nsub * NH * 32 * 128);
              const int off = key_base % p.block_size;
              for (int sub = 0; sub < nsub; sub++) {
#pragma unroll
                for (int hf = 0; hf < NH; hf++)
                  tma_load_4d(dst + hf * DEC_HALF + sub * 32 * 128, tm, fullb, hf * 64, w.h,
                              off + sub * 32, blk);
              }
            }
            __syncwarp();
            continue;
          }
          for (int part = 0; part < parts; part++) {
            const int blk = __shfl_sync(0xffffffffu, blk_cur, part);
            if (lane == 0) {
              uint8_t* dst = (kv == 0 ? Ks : Vs) + st * Cfg::TILE_BYTES;
              const CUtensorMap* tm = kv == 0 ? &tmap_k : &tmap_v;
              if (part == 0) mbar_expect_tx(fullb, Cfg::TILE_BYTES);
              const int off = (key_base + part * rpl) % p.block_size;
#pragma unroll
              for (int hf = 0; hf < NH; hf++)
                tma_load_4d(dst + hf * DEC_HALF + part * rpl * 128, tm, fullb, hf * 64, w.h, off, blk);
            }
          }
          __syncwarp();
        }
        blk_cur = blk_next;
        if (j == 0) advance(item_after);       // after this item's first tile is on its way
        // third tile: its stage was freed by the last S MMA of the previous item, so the Q buffer
        // of the next item (last read by that MMA) is free as well and load_q does not wait
        if (j == min(2, w.n - 1) && item_after < num_items && w_next.n > 0) {
          if (!load_q(it + 1, w_next)) goto done;
          q_ahead = true;
        }
      }
      it++;
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc_s = make_idesc_f16(128, DEC_NQ, true, false, false);
    constexpr uint32_t idesc_o = make_idesc_f16(D, DEC_NQ, true, true, false);   // A = V, MN-major
    const uint32_t q_addr0 = smem_u32(Qs), k_addr = smem_u32(Ks), v_addr = smem_u32(Vs),
                   p_addr = smem_u32(Ps);
    uint32_t gt = 0, it = 0;
    DecRaw raw_next = {0, 0, 0};
    if ((int)blockIdx.x < num_items) raw_next = dec_load(p, blockIdx.x);
    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
      const DecItem w = dec_make(p, item, raw_next);
      if (item + (int)gridDim.x < num_items) raw_next = dec_load(p, item + gridDim.x);
      if (w.n <= 0) continue;
      const int qb = it & 1;
      const uint32_t q_addr = q_addr0 + qb * Cfg::Q_BYTES;
      const uint32_t o_col = Cfg::O_COL + qb * DEC_NQ;
      if (!mbar_wait(&q_full[qb], (it >> 1) & 1u, abort_word)) goto done;
      // the accumulator of two items ago has been read out by its epilogue
      if (!mbar_wait(&o_free[qb], ((it >> 1) & 1u) ^ 1u, abort_word)) goto done;
      auto issue_s = [&](int j) -> bool {
        const uint32_t g = gt + (uint32_t)j;
        const int st = g % ST;
        const uint32_t ph = (g / ST) & 1u;
        const int b = g & 1;
        if (!mbar_wait(&k_full[st], ph, abort_word)) return false;
        DEC_STAMP(1, g, 0);
        if (!mbar_wait(&s_free[b], ((g >> 1) & 1u) ^ 1u, abort_word)) return false;
        tc_fence_after();
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < D / 16; kk++) {
            const uint64_t da = make_smem_desc(
                k_addr + st * Cfg::TILE_BYTES + (kk >> 2) * DEC_HALF + (kk & 3) * 32, 16, 1024,
                kLayoutSw128);
            const uint64_t db = make_smem_desc(q_addr + (kk >> 2) * DEC_QHALF + (kk & 3) * 32, 16,
                                               1024, kLayoutSw128);
            umma_f16_ss(tmem_base + b * DEC_NQ, da, db, idesc_s, kk > 0 ? 1u : 0u);
          }
          umma_commit(&k_empty[st]);
          umma_commit(&s_ready[b]);
          if (j == w.n - 1) umma_commit(&q_empty[qb]);     // last read of this item's Q
        }
        __syncwarp();
        return true;
      };
      if (!issue_s(0)) goto done;
      for (int j = 0; j < w.n; j++) {
        if (j + 1 < w.n) {
          if (!issue_s(j + 1)) goto done;
        }
        const uint32_t g = gt + (uint32_t)j;
        const int st = g % ST;
        const uint32_t ph = (g / ST) & 1u;
        const int pb = g & 1;
        if (!mbar_wait(&v_full[st], ph, abort_word)) goto done;
        DEC_STAMP(1, g, 1);
        if (!mbar_wait(&p_ready[pb], (g >> 1) & 1u, abort_word)) goto done;
        DEC_STAMP(1, g, 2);
        tc_fence_after();
        if (lane == 0) {
#pragma unroll
          for (int kk = 0; kk < 8; kk++) {
            // A: 16 keys of V^T (two 64-wide d atoms DEC_HALF apart, 8-key groups 1024 B apart)
            const uint64_t da = make_smem_desc(v_addr + st * Cfg::TILE_BYTES + kk * 2048, DEC_HALF,
                                               1024, kLayoutSw128);
            const uint64_t db = make_smem_desc(
                p_addr + pb * Cfg::P_BYTES + (kk >> 2) * DEC_QHALF + (kk & 3) * 32, 16, 1024,
                kLayoutSw128);
            umma_f16_ss(tmem_base + o_col, da, db, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&v_empty[st]);
          umma_commit(&pv_done[pb]);
        }
        __syncwarp();
      }
      gt += (uint32_t)w.n;
      it++;
    }
  } else {
    // ------------------------------------------------------------ softmax / epilogue
    // NVT = compile-time bound on the valid columns (query rows x heads of the group).
    const int qd = warp & 3;
    const int tid = qd * 32 + lane;                 // key inside the tile; d index for O^T
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
    const float sl2 = p.scale_log2;
    int* redi = reinterpret_cast<int*>(red);        // [2 tiles][4 warps][16]
    uint32_t gt = 0, it = 0;
    DecRaw raw_next = {0, 0, 0};
    if ((int)blockIdx.x < num_items) raw_next = dec_load(p, blockIdx.x);
    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
      const DecItem w = dec_make(p, item, raw_next);
      if (item + (int)gridDim.x < num_items) raw_next = dec_load(p, item + gridDim.x);
      const int nv = w.q_len * G;                   // valid columns (<= 16)
      if (w.n <= 0) {
        if (p.num_splits > 1 && w.q_len > 0) {      // an empty split still owns its partial slots
          for (int c = tid; c < nv; c += 128) {
            const long pidx =
                ((long)(w.q_start + c / G) * p.Hq + (w.h * G + c % G)) * p.num_splits + w.split;
            p.partial_lse[pidx] = -INFINITY;
            for (int d = 0; d < D; d++) p.partial_o[pidx * D + d] = 0.f;
          }
        } else if (p.num_splits == 1 && p.lse_out && w.q_len > 0) {
          // a caller that merges partial results of several ranks needs a defined (zero-weight)
          // result for a sequence none of whose keys live here
          for (int c = 0; c < nv; c++) {
            const long tok = w.q_start + c / G;
            const int hq = w.h * G + c % G;
            if (tid == 0) p.lse_out[tok * p.Hq + hq] = -INFINITY;
            if (tid < D) p.out[tok * p.out_stride + (long)hq * D + tid] = __float2bfloat16(0.f);
          }
        }
        continue;
      }
      const uint32_t o_col = Cfg::O_COL + (it & 1) * DEC_NQ;
      float m[NVT], lsum[NVT];
      int hi[NVT], lo[NVT];                           // keys [lo, hi) are visible to column c
      int hi_min = w.seq_len, lo_max = 0;
#pragma unroll
      for (int c = 0; c < NVT; c++) {
        m[c] = -INFINITY;
        lsum[c] = 0.f;
        const int q_pos = w.ctx + min(c / G, w.q_len - 1);
        hi[c] = min(w.seq_len, q_pos + 1);
        lo[c] = p.window > 0 ? max(0, q_pos - p.window + 1) : 0;
        hi_min = min(hi_min, hi[c]);
        lo_max = max(lo_max, lo[c]);
      }

      for (int j = 0; j < w.n; j++) {
        const uint32_t g = gt + (uint32_t)j;
        const int b = g & 1;
        if (warp == 2) DEC_STAMP(2, g, 0);
        if (!mbar_wait(&s_ready[b], (g >> 1) & 1u, abort_word)) goto done;
        if (warp == 2) DEC_STAMP(2, g, 1);
        tc_fence_after();
        uint32_t r[16];
        tmem_ld_32x32b_x16(t_lane + b * DEC_NQ, r);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[b]);
        const int tile_base = (w.t0 + j) << 7;
        const int key = tile_base + tid;
        // only tiles that straddle a visibility limit need per-key masking
        const bool need_mask = (tile_base + 128 > hi_min) || (tile_base < lo_max);
        float s[NVT];
        int* rj = redi + b * 64 + qd * 16;
#pragma unroll
        for (int c = 0; c < NVT; c++) {
          s[c] = __uint_as_float(r[c]);
          if (need_mask && !(key >= lo[c] && key < hi[c])) s[c] = -INFINITY;
          int ob = __float_as_int(s[c]);
          ob ^= (ob >> 31) & 0x7fffffff;              // order-preserving float -> int
          const int wm = __reduce_max_sync(0xffffffffu, ob);
          if (lane == 0) rj[c] = wm;
        }
        if (warp == 2) DEC_STAMP(2, g, 5);
        softmax_bar();
        if (warp == 2) DEC_STAMP(2, g, 6);
        const int* ra = redi + b * 64;
        bool any_change = false;
        float alpha[NVT];
#pragma unroll
        for (int c = 0; c < NVT; c++) {
          int t = max(max(ra[c], ra[16 + c]), max(ra[32 + c], ra[48 + c]));
          t ^= (t >> 31) & 0x7fffffff;
          const float mn = fmaxf(m[c], __int_as_float(t));
          alpha[c] = 1.f;
          // lazy rescaling: the reference max only moves when it would grow by more than
          // 2^kRescaleLog2, so most tiles never touch the O^T accumulator
          if (mn > m[c] && (m[c] == -INFINITY || (mn - m[c]) * sl2 > kRescaleLog2)) {
            alpha[c] = (m[c] == -INFINITY) ? 0.f : fast_exp2((m[c] - mn) * sl2);
            any_change = any_change || (m[c] != -INFINITY);
            m[c] = mn;
          }
          lsum[c] *= alpha[c];
        }
        if (warp == 2) DEC_STAMP(2, g, 7);
        // P buffer g&1 was last read by PV(g-2) (possibly of the previous item)
        if (g >= 2) {
          if (!mbar_wait(&pv_done[b], ((g - 2) >> 1) & 1u, abort_word)) goto done;
        }
        if (j > 0 && any_change) {    // uniform over the 128 threads: O^T must be quiescent
          if (!mbar_wait(&pv_done[(g - 1) & 1], ((g - 1) >> 1) & 1u, abort_word)) goto done;
          tc_fence_after();
          uint32_t o[16];
          tmem_ld_32x32b_x16(t_lane + o_col, o);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < NVT; c++) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha[c]);
          tmem_st_32x32b_x16(t_lane + o_col, o);
          tmem_st_wait();
        }
        if (warp == 2) DEC_STAMP(2, g, 2);
        // probabilities of this key for every column -> P[c][key] (K-major, swizzled)
        uint8_t* pbase = Ps + b * Cfg::P_BYTES + (tid >> 6) * DEC_QHALF;
        const int kin = tid & 63;
#pragma unroll
        for (int c = 0; c < NVT; c++) {
          const float mb = (m[c] == -INFINITY) ? 0.f : m[c] * sl2;
          const float pv = fast_exp2(s[c] * sl2 - mb);
          lsum[c] += pv;
          const int chunk = (kin >> 3) ^ (c & 7);
          *reinterpret_cast<__nv_bfloat16*>(pbase + c * 128 + (chunk << 4) + (kin & 7) * 2) =
              __float2bfloat16(pv);
        }
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready[b]);
        if (warp == 2) DEC_STAMP(2, g, 3);
      }
      gt += (uint32_t)w.n;
      // ---- epilogue of the item: total row sums, normalise, store
      {
        const uint32_t gl = gt - 1;
        if (!mbar_wait(&pv_done[gl & 1], (gl >> 1) & 1u, abort_word)) goto done;
      }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < NVT; c++) {
        const float ws = warp_reduce_sum(lsum[c]);
        if (lane == 0) red_sum[qd * DEC_NQ + c] = ws;
      }
      uint32_t o[16];
      tmem_ld_32x32b_x16(t_lane + o_col, o);
      tmem_ld_wait();
      tc_fence_before();
      softmax_bar();            // row sums visible; every thread holds its O^T row
      if (lane == 0) mbar_arrive(&o_free[it & 1]);
      if (tid < D) {
#pragma unroll
        for (int c = 0; c < NVT; c++) {
          if (c < nv) {
            const float l = red_sum[c] + red_sum[DEC_NQ + c] + red_sum[2 * DEC_NQ + c] +
                            red_sum[3 * DEC_NQ + c];
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const long tok = w.q_start + c / G;
            const int hq = w.h * G + c % G;
            const float val = __uint_as_float(o[c]) * inv;
            if (p.num_splits == 1) {
              p.out[tok * p.out_stride + (long)hq * D + tid] = __float2bfloat16(val);
              if (tid == 0 && p.lse_out)
                p.lse_out[tok * p.Hq + hq] =
                    (l > 0.f) ? (m[c] * sl2 * 0.6931471805599453f + logf(l)) : -INFINITY;
            } else {
              const long pidx = (tok * p.Hq + hq) * p.num_splits + w.split;
              p.partial_o[pidx * D + tid] = val;
              if (tid == 0)
                p.partial_lse[pidx] =
                    (l > 0.f) ? (m[c] * sl2 * 0.6931471805599453f + logf(l)) : -INFINITY;
            }
          }
        }
      }
      // the next item's epilogue overwrites red_sum only after a softmax_bar of its tile loop
      it++;
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

// ---------------------------------------------------------------- host
struct DecTmapCache {
  std::unordered_map<std::string, CUtensorMap> map;
  std::mutex mu;
  int get(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
          const uint64_t* strides, const uint32_t* box) {
    char key[128];
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
static DecTmapCache g_dec_tmaps;
static int g_dec_l2_prefetch = 0;      // tiles of L2 prefetch ahead of the staged K / V loads (0 = off)

}  // namespace b200

// Distance (128-key tiles) of the L2 prefetch of K / V pages for every following call; 0 = off.
B200_API int b200_attn_decode_set_l2_prefetch(int tiles) {
  b200::g_dec_l2_prefetch = tiles < 0 ? 0 : (tiles > 16 ? 16 : tiles);
  return 0;
}

// Decode / short-query attention: every sequence has q_len <= 16 / (Hq/Hkv) query
// tokens (query_start_loc gives their positions in q).  Arguments as b200_attn_fwd_tc;
// scratch needs b200_attn_scratch_bytes(T, Hq, D, num_splits) bytes when num_splits > 1.
// lse_out (optional, fp32 [T, Hq]): log-sum-exp of every (token, head) over the keys this call saw,
// for callers that merge the results of several calls (context-parallel ranks).
B200_API int b200_attn_decode_tc_lse(const void* q, long q_stride, long T, const void* k_cache,
                                     const void* v_cache, long num_blocks, int block_size,
                                     const void* query_start_loc, const void* seq_lens,
                                     const void* block_table, int max_blocks, int num_seqs, int Hq,
                                     int Hkv, int D, float scale, int window, int num_splits,
                                     int max_q_len, void* out, long out_stride, void* scratch,
                                     int kv_layout, void* lse_out,
                                     int* status, void* timeline, cudaStream_t stream) {
  using namespace b200;
  if (num_seqs <= 0 || T <= 0) return 0;
  const int G = Hq / Hkv;
  if (G * Hkv != Hq || G > DEC_NQ || (DEC_NQ % G) != 0) return 9120;
  if (D != 128) return 9121;
  if (block_size < 8 || (block_size < 128 && (128 % block_size) != 0) ||
      (block_size > 128 && (block_size % 128) != 0))
    return 9122;
  if ((q_stride & 7) || (out_stride & 7)) return 9123;
  if (num_splits < 1) num_splits = 1;
  if (num_splits > 1 && !scratch) return 9124;
  const int rpl = block_size < 128 ? block_size : 128;
  CUtensorMap tq, tk, tv, tk32, tv32;
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)G, (uint64_t)Hkv, (uint64_t)T};
    uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)G * D * 2, (uint64_t)q_stride * 2};
    uint32_t box[4] = {64, (uint32_t)G, 1, (uint32_t)(DEC_NQ / G)};
    int rc = g_dec_tmaps.get(&tq, q, 4, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)block_size, (uint64_t)num_blocks};
    // kv_layout 0: [blocks, tokens, heads, D]; 1: [blocks, heads, tokens, D]
    uint64_t str[3] = {(uint64_t)D * 2, (uint64_t)Hkv * D * 2,
                       (uint64_t)block_size * Hkv * D * 2};
    if (kv_layout == 1) {
      str[0] = (uint64_t)block_size * D * 2;
      str[1] = (uint64_t)D * 2;
    }
    uint32_t box[4] = {64, 1, (uint32_t)rpl, 1};
    int rc = g_dec_tmaps.get(&tk, k_cache, 4, dims, str, box);
    if (rc) return rc;
    rc = g_dec_tmaps.get(&tv, v_cache, 4, dims, str, box);
    if (rc) return rc;
    tk32 = tk;
    tv32 = tv;
    if (rpl == 128) {
      uint32_t box32[4] = {64, 1, 32, 1};
      rc = g_dec_tmaps.get(&tk32, k_cache, 4, dims, str, box32);
      if (rc) return rc;
      rc = g_dec_tmaps.get(&tv32, v_cache, 4, dims, str, box32);
      if (rc) return rc;
    }
  }
  DecParams p;
  p.query_start_loc = (const int*)query_start_loc;
  p.seq_lens = (const int*)seq_lens;
  p.block_table = (const int*)block_table;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.rows_per_load = rpl;
  p.G = G; p.Hkv = Hkv; p.Hq = Hq;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  p.num_splits = num_splits;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.partial_o = (float*)scratch;
  p.partial_lse = scratch ? (float*)scratch + T * Hq * (long)num_splits * D : nullptr;
  p.lse_out = (float*)lse_out;
  p.num_blocks_total = num_blocks;
  p.status = status;
  p.timeline = (long long*)timeline;
  using Cfg = DecCfg<128>;
  const long items = (long)Hkv * num_seqs * num_splits;
  if (items > 0x7fffffffL) return 9125;
  p.num_seqs = num_seqs;
  p.tail_loads = rpl == 128 ? 1 : 0;
  p.l2_prefetch = g_dec_l2_prefetch;
  p.num_items = (int)items;
  static int sm_count[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 9127;
  if (sm_count[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      return 9127;
    sm_count[dev] = n;
  }
  dim3 grid((unsigned)(items < sm_count[dev] ? items : sm_count[dev]));
  // columns that can be valid: query tokens per sequence x heads per group
  if (max_q_len < 1) max_q_len = 1;
  const int ncols = max_q_len * G;
  if (ncols > DEC_NQ) return 9126;
#define LAUNCH_DEC_TC(NV)                                                                   \
  do {                                                                                      \
    static bool attr_set = false;                                                           \
    if (!attr_set) {                                                                        \
      cudaError_t e = cudaFuncSetAttribute(attn_decode_tc_kernel<128, NV>,                  \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                           Cfg::SMEM_BYTES);                                \
      if (e != cudaSuccess) return (int)e;                                                  \
      attr_set = true;                                                                      \
    }                                                                                       \
    attn_decode_tc_kernel<128, NV><<<grid, DEC_THREADS, Cfg::SMEM_BYTES, stream>>>(tq, tk, tv, tk32,  \
                                                                                    tv32, p); \
  } while (0)
  if (ncols <= 1) LAUNCH_DEC_TC(1);
  else if (ncols <= 2) LAUNCH_DEC_TC(2);
  else if (ncols <= 4) LAUNCH_DEC_TC(4);
  else if (ncols <= 8) LAUNCH_DEC_TC(8);
  else LAUNCH_DEC_TC(16);
#undef LAUNCH_DEC_TC
  int rc = B200_CHECK_LAUNCH();
  if (rc) return rc;
  if (num_splits > 1)
    return launch_merge_splits(p.partial_o, p.partial_lse, T, Hq, num_splits, D, out,
                               out_stride, stream, (float*)lse_out);
  return 0;
}

B200_API int b200_attn_decode_tc(const void* q, long q_stride, long T, const void* k_cache,
                                 const void* v_cache, long num_blocks, int block_size,
                                 const void* query_start_loc, const void* seq_lens,
                                 const void* block_table, int max_blocks, int num_seqs, int Hq,
                                 int Hkv, int D, float scale, int window, int num_splits,
                                 int max_q_len, void* out, long out_stride, void* scratch,
                                 int kv_layout,
                                 int* status, void* timeline, cudaStream_t stream) {
  return b200_attn_decode_tc_lse(q, q_stride, T, k_cache, v_cache, num_blocks, block_size,
                                 query_start_loc, seq_lens, block_table, max_blocks, num_seqs, Hq,
                                 Hkv, D, scale, window, num_splits, max_q_len, out, out_stride,
                                 scratch, kv_layout, nullptr, status, timeline, stream);
}
