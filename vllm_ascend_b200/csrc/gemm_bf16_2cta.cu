// bf16 GEMM with paired-CTA tensor-core instructions (tcgen05 cta_group::2):
//   C[M,N] = A[M,K] * W[N,K]^T (+bias) (+residual)   or   silu(A Wg^T) * (A Wu^T)
//
// Two CTAs of a cluster (two neighbouring SMs) work on one 256 x 256 output tile.
// Each CTA stages its own 128 rows of A and HALF of the W tile (128 rows), so a
// stage costs 32 KB per CTA instead of 48 KB and the pipeline is 6 deep.  The
// leader CTA issues `tcgen05.mma.cta_group::2` (M = 256): the hardware reads A
// from both CTAs' shared memory and the two halves of W, and writes each CTA's
// 128 x 256 half of the accumulator into that CTA's own TMEM.  Completion is
// broadcast to both CTAs with `tcgen05.commit ... multicast::cluster`.
// TMA loads are plain `cta_group::2` loads (no multicast): each CTA fetches its
// own tiles and reports the bytes to the leader's barrier.
//
//   warp 0      TMA producer (both CTAs)
//   warp 1      MMA issuer (leader CTA only) + TMEM alloc/dealloc (both)
//   warps 2..5  epilogue (both CTAs, each for its own 128 rows)
// All waits are bounded (common.cuh); the cluster barriers at start and end are
// reached by every thread on every path.
#include "comm.cuh"

#include <mutex>
#include <unordered_map>

namespace b200 {

constexpr int G2_BM = 256;          // per CTA pair
constexpr int G2_BN = 256;
constexpr int G2_BK = 64;
constexpr int G2_THREADS = 192;
constexpr int G2_STAGES = 6;
constexpr int G2_A_BYTES = 128 * G2_BK * 2;        // 16 KB: this CTA's rows of A
constexpr int G2_B_BYTES = 128 * G2_BK * 2;        // 16 KB: this CTA's half of the W tile
constexpr int G2_STAGE_BYTES = G2_A_BYTES + G2_B_BYTES;
// reduce-scatter epilogue: every epilogue warp stages 32 rows x 64 columns (128 B per row, 16 B pad)
// so that rows leave for their owner's GPU as 128-byte segments instead of one 16-byte store per row
constexpr int G2_RS_ROW_BYTES = 144;
constexpr int G2_RS_STAGE_BYTES = 4 * 32 * G2_RS_ROW_BYTES;
constexpr int G2_SMEM_BYTES = G2_STAGES * G2_STAGE_BYTES + 1024 + 256 + G2_RS_STAGE_BYTES;
constexpr uint32_t kPeerBitMask = 0xFEFFFFFFu;     // clears the CTA-rank bit of a shared address

struct Gemm2Params {
  int M, N, K, ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  __nv_bfloat16* C;
  int* status;
  int tiles_m, tiles_n;
  int swiglu;          // W = [gate; up]: tile pairs 128 gate + 128 up columns
  int up_row_offset;
  // ---- fused collectives (same protocol as the single-CTA kernel's AG / RS modes)
  int mode;                           // 0, G2_AG or G2_RS
  const uint32_t* ag_flags;           // local CommCtl.ag_flag
  const uint32_t* ag_epoch;
  int rows_per_src, my_rank, num_ranks;
  __nv_bfloat16* rs_dst[kMaxRanks];   // staging on owner o: [num_ranks][rows_per_owner][N]
  uint32_t* rs_flag_dst[kMaxRanks];
  CommCtl* ctl;
  int rows_per_owner;
  int raster;                         // M-tiles per raster group (0/1: column-major order)
  int bn;                             // tile width: 128..256 in steps of 16 (32 with the reduce-scatter
                                      // epilogue, whose staging flushes 64-column pairs; SwiGLU tiles: 256)
  // ---- RMSNorm folded into the GEMMs around it (the norm weight lives in W of the consumer)
  // Row statistics travel as per-column-tile partial sums so that their total does not depend on
  // the order in which tiles finish: buffer [ss_parts_max][ss_stride] fp32 followed by one int32
  // (the number of partials the producer wrote).
  const float* row_ss_in;             // sum of squares of the rows of A: accumulators are scaled by
  float inv_dim, eps;                 //     rsqrt(sum_i row_ss_in[i][row] * inv_dim + eps) before bias / SwiGLU
  float* row_ss_out;                  // [tile_n][row] = sum of squares of the bf16 output row within that column tile
  long ss_stride;
  int ss_parts_max;
  int l2_prefetch;                    // k-blocks the L2 prefetch of W (and A) runs ahead of the staged loads; 0 = off
};
// G2_PUB: the last CTA publishes this rank's reduce-scatter epoch to every peer (set with G2_RS;
// alone it is the NVLS form: rows stay in the local multicast-bound buffer C)
enum : int { G2_AG = 1, G2_RS = 2, G2_PUB = 4 };

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;"
               ::: "memory");
}
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ void tma_load_2d_2sm(void* dst, const CUtensorMap* map,
                                                uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(map), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_2sm(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_2sm() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_2sm(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void umma_f16_ss_2sm(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                                uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at the same shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_2sm(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64"
      " [%0], %1;" ::"r"(smem_u32(bar)),
      "h"(mask)
      : "memory");
}

// Tile order: groups of `raster` M-tiles are walked column by column, so the clusters that run
// at the same time share a few A row-blocks and a few W column-blocks (both stay in L2)
// instead of streaming all of A against one W block.
__device__ __forceinline__ void tile_of(const Gemm2Params& p, int t, int& tm, int& tn) {
  const int gm_full = p.raster;
  if (gm_full <= 1 || gm_full >= p.tiles_m) {
    tm = t % p.tiles_m;
    tn = t / p.tiles_m;
    return;
  }
  const int per_group = gm_full * p.tiles_n;
  const int g = t / per_group, r = t - g * per_group;
  const int first = g * gm_full;
  const int gm = min(gm_full, p.tiles_m - first);
  tm = first + r % gm;
  tn = r / gm;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(G2_THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b, const Gemm2Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles = smem;
  uint64_t* full_bar = (uint64_t*)(smem + G2_STAGES * G2_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + G2_STAGES;
  uint64_t* tmem_full = empty_bar + G2_STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;          // [2] (the leader's copy is the one in use)
  uint32_t* tmem_ptr = (uint32_t*)(tmem_empty + 2);
  volatile int* abort_word = (volatile int*)(tmem_ptr + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int num_kb = (p.K + G2_BK - 1) / G2_BK;
  const int num_tiles = p.tiles_m * p.tiles_n;
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < G2_STAGES; s++) {
      mbar_init(&full_bar[s], 1);     // leader's expect_tx arrival; bytes come from both CTAs
      mbar_init(&empty_bar[s], 1);    // one commit from the leader's MMA warp
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 8);   // 4 epilogue warps of each CTA
    }
    *abort_word = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc_2sm(tmem_ptr, 512);
    tmem_relinquish_2sm();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();       // both CTAs' barriers exist before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    int stage = 0;
    uint32_t phase = 0;
    uint32_t ag_epoch = 0;
    if (p.mode & G2_AG) ag_epoch = *((volatile const uint32_t*)p.ag_epoch);
    for (int t = cluster_id; t < num_tiles; t += num_clusters) {
      int tm, tn;
      tile_of(p, t, tm, tn);
      if (p.mode & G2_AG) tm = (tm + (p.my_rank * p.rows_per_src) / G2_BM) % p.tiles_m;   // local rows first
      const int a_row = tm * G2_BM + (int)rank * 128;
      if (p.mode & G2_AG) {
        // this CTA's 128 rows come from source ranks s0..s1: wait for their pushes
        if (lane == 0 && a_row < p.M) {
          const int last_row = min(a_row + 128, p.M) - 1;
          const int s0 = a_row / p.rows_per_src, s1 = last_row / p.rows_per_src;
          for (int s = s0; s <= s1; s++) {
            if (s == p.my_rank) continue;
            if (!wait_flag_ge(&p.ag_flags[s], ag_epoch, p.status)) *abort_word = B200_TIMEOUT;
          }
          fence_proxy_async_global();
        }
        __syncwarp();
        if (*abort_word) goto done;
      }
      // plain: this CTA's 128 of the tile's 256 W rows.  SwiGLU: the leader stages the 128
      // gate rows, the peer the matching 128 up rows.
      const int w_row = p.swiglu ? tn * 128 + (int)rank * p.up_row_offset
                                 : tn * p.bn + (int)rank * (p.bn >> 1);
      // Few row tiles (decode batches): every weight byte is read from DRAM once and nothing else
      // hides that latency but the depth of the stage ring, so the boxes of later k-blocks are
      // requested into L2 ahead of time.  One row tile asks for W, one column tile for A.
      const bool pf_w = p.l2_prefetch > 0 && tm == 0;
      const bool pf_a = p.l2_prefetch > 0 && p.mode == 0 && tn == 0 && a_row < p.M;
      if (lane == 0 && (pf_w || pf_a)) {
        for (int kb = 0; kb < p.l2_prefetch && kb < num_kb; kb++) {
          if (pf_w) tma_prefetch_l2_2d(&tmap_b, kb * G2_BK, w_row);
          if (pf_a) tma_prefetch_l2_2d(&tmap_a, kb * G2_BK, a_row);
        }
      }
      for (int kb = 0; kb < num_kb; kb++) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word)) goto done;
        if (lane == 0) {
          const int kpf = kb + p.l2_prefetch;
          if (kpf < num_kb) {
            if (pf_w) tma_prefetch_l2_2d(&tmap_b, kpf * G2_BK, w_row);
            if (pf_a) tma_prefetch_l2_2d(&tmap_a, kpf * G2_BK, a_row);
          }
          uint8_t* sa = tiles + stage * G2_STAGE_BYTES;
          uint8_t* sb = sa + G2_A_BYTES;
          const uint32_t lbar = smem_u32(&full_bar[stage]) & kPeerBitMask;
          if (leader) mbar_expect_tx(&full_bar[stage], 2 * (G2_A_BYTES + (p.bn >> 1) * G2_BK * 2));
          tma_load_2d_2sm(sa, &tmap_a, lbar, kb * G2_BK, a_row);
          tma_load_2d_2sm(sb, &tmap_b, lbar, kb * G2_BK, w_row);
        }
        __syncwarp();
        if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (leader) {
      const uint32_t idesc = make_idesc_f16(G2_BM, p.bn, true, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      for (int t = cluster_id; t < num_tiles; t += num_clusters, it++) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word)) goto done;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * G2_BN;
        for (int kb = 0; kb < num_kb; kb++) {
          if (!mbar_wait(&full_bar[stage], phase, abort_word)) goto done;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t sa = smem_u32(tiles + stage * G2_STAGE_BYTES);
            const uint32_t sb = sa + G2_A_BYTES;
#pragma unroll
            for (int kk = 0; kk < G2_BK / 16; kk++) {
              const uint64_t da = make_smem_desc(sa + kk * 32, 16, 1024, kLayoutSw128);
              const uint64_t db = make_smem_desc(sb + kk * 32, 16, 1024, kLayoutSw128);
              umma_f16_ss_2sm(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
            }
            umma_commit_2sm(&empty_bar[stage]);
            if (kb == num_kb - 1) umma_commit_2sm(&tmem_full[acc]);
          }
          __syncwarp();
          if (++stage == G2_STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    const int out_per_tile = p.swiglu ? 128 : p.bn;
    uint8_t* rs_stage = smem + G2_STAGES * G2_STAGE_BYTES + 256 + q * (32 * G2_RS_ROW_BYTES);
    int it = 0;
    for (int t = cluster_id; t < num_tiles; t += num_clusters, it++) {
      int tm, tn;
      tile_of(p, t, tm, tn);
      if (p.mode & G2_AG) tm = (tm + (p.my_rank * p.rows_per_src) / G2_BM) % p.tiles_m;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_word)) goto done;
      tc_fence_after();
      const int row = tm * G2_BM + (int)rank * 128 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * G2_BN;
      __nv_bfloat16* crow;
      if (p.mode & G2_RS) {
        // partial-sum row goes straight into its owner's staging buffer over NVLink
        const int owner = row_ok ? row / p.rows_per_owner : 0;
        const int local = row - owner * p.rows_per_owner;
        crow = p.rs_dst[owner] + ((size_t)p.my_rank * p.rows_per_owner + local) * p.ldc;
      } else {
        crow = p.C + (size_t)row * p.ldc;
      }
      const __nv_bfloat16* rrow = p.residual ? p.residual + (size_t)row * p.ldc : nullptr;
      float rstd = 1.f, ss_acc = 0.f;
      if (p.row_ss_in && row_ok) {
        int parts = *reinterpret_cast<const int*>(p.row_ss_in + (long)p.ss_parts_max * p.ss_stride);
        parts = parts < 0 ? 0 : (parts > p.ss_parts_max ? p.ss_parts_max : parts);
        float ss = 0.f;
        for (int i = 0; i < parts; i++) ss += p.row_ss_in[(long)i * p.ss_stride + row];   // fixed order
        rstd = rsqrtf(ss * p.inv_dim + p.eps);
      }
      if (p.row_ss_out && t == 0 && rank == 0 && q == 0 && lane == 0)
        *reinterpret_cast<int*>(p.row_ss_out + (long)p.ss_parts_max * p.ss_stride) = p.tiles_n;
#pragma unroll 1
      for (int c0 = 0; c0 < out_per_tile; c0 += 32) {
        const int col0 = tn * out_per_tile + c0;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c0, r);
        if (p.swiglu) {
          uint32_t u[32];
          tmem_ld_32x32b_x32(t_row + 128 + c0, u);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const float g = __uint_as_float(r[j]) * rstd;
            r[j] = __float_as_uint(g / (1.f + __expf(-g)) * (__uint_as_float(u[j]) * rstd));
          }
        } else {
          tmem_ld_wait();
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const int col = col0 + g * 8;
            if (col < p.N && c0 + g * 8 < out_per_tile) {     // tile widths are multiples of 16
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; j++) v[j] = __uint_as_float(r[g * 8 + j]);
              if (p.row_ss_in && !p.swiglu) {
#pragma unroll
                for (int j = 0; j < 8; j++) v[j] *= rstd;
              }
              if (p.bias) {
                const uint4 bv = *reinterpret_cast<const uint4*>(p.bias + col);
                const uint32_t bw[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  const float2 f = unpack_bf16x2(bw[j]);
                  v[2 * j] += f.x;
                  v[2 * j + 1] += f.y;
                }
              }
              if (rrow) {
                const uint4 rv = *reinterpret_cast<const uint4*>(rrow + col);
                const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  const float2 f = unpack_bf16x2(rw[j]);
                  v[2 * j] += f.x;
                  v[2 * j + 1] += f.y;
                }
              }
              uint4 o;
              o.x = pack_bf16x2(v[0], v[1]);
              o.y = pack_bf16x2(v[2], v[3]);
              o.z = pack_bf16x2(v[4], v[5]);
              o.w = pack_bf16x2(v[6], v[7]);
              if (p.row_ss_out) {       // of the values as stored (bf16), like a norm that reads them back
                const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                  const float2 f = unpack_bf16x2(ow[j]);
                  ss_acc += f.x * f.x + f.y * f.y;
                }
              }
              if (p.mode & G2_RS)
                *reinterpret_cast<uint4*>(rs_stage + lane * G2_RS_ROW_BYTES + ((c0 & 32) + g * 8) * 2) = o;
              else
                *reinterpret_cast<uint4*>(crow + col) = o;
            }
          }
        }
        if (p.mode & G2_RS) {
          // flush after two 32-column chunks (or at the tile's / matrix's last chunk): lanes regroup so
          // one store instruction covers 4 rows x 128 contiguous bytes (8 rows x 64 bytes for a lone chunk)
          const bool last = (col0 + 32 >= p.N) || (c0 + 32 >= out_per_tile);
          if ((c0 & 32) || last) {
            __syncwarp();
            const int staged = (c0 & 32) ? 64 : 32;
            const int colbase = col0 - (c0 & 32);
            const int segs = staged >> 3;                 // 16-byte segments per row: 8 or 4
            const int rows_per_inst = 32 / segs;
            const unsigned long long my_ptr = (unsigned long long)crow;
            for (int r0 = 0; r0 < 32; r0 += rows_per_inst) {
              const int rr = r0 + lane / segs, sg = lane % segs;
              const unsigned long long ptr = __shfl_sync(0xffffffffu, my_ptr, rr);
              const int ok = __shfl_sync(0xffffffffu, (int)row_ok, rr);
              const int col = colbase + sg * 8;
              if (ok && col < p.N)
                *reinterpret_cast<uint4*>((__nv_bfloat16*)ptr + col) =
                    *reinterpret_cast<const uint4*>(rs_stage + rr * G2_RS_ROW_BYTES + sg * 16);
            }
            __syncwarp();
          }
        }
      }
      if (p.row_ss_out && row_ok) p.row_ss_out[(long)tn * p.ss_stride + row] = ss_acc;
      tc_fence_before();
      __syncwarp();
      // accumulator buffer drained: tell the leader's MMA warp (local or remote arrive)
      if (lane == 0) mbar_arrive_cluster(mapa_shared(smem_u32(&tmem_empty[acc]), 0));
    }
    if (p.mode & G2_PUB) __threadfence_system();   // partial rows visible to their owners
  }
done:
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    const uint64_t t_start = globaltimer_ns();
    while (globaltimer_ns() - t_start < 50000ull) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, *abort_word);
  } else if ((p.mode & G2_PUB) && threadIdx.x == 0) {
    // the last CTA of the grid publishes this rank's reduce-scatter epoch to every owner
    const uint32_t prev = atomicAdd(&p.ctl->done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      const uint32_t epoch = p.ctl->rs_epoch + 1;
      for (int o = 0; o < p.num_ranks; o++) st_release_sys(p.rs_flag_dst[o], epoch);
      p.ctl->rs_epoch = epoch;
      p.ctl->done_ctr = 0;
      __threadfence();
    }
  }
  // neither CTA may free TMEM or leave while its partner can still signal it or read its tiles
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_2sm(tmem_base, 512);
  }
}

// ---------------------------------------------------------------- host
struct Tmap2Key {
  const void* ptr;
  uint64_t rows, cols, ld;
  bool operator==(const Tmap2Key& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld;
  }
};
struct Tmap2Hash {
  size_t operator()(const Tmap2Key& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    return h;
  }
};

// row-major bf16 [rows, cols], box = 128 rows x 64 columns, 128-byte swizzle
static int get_tmap_128x64(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                           uint64_t ld, uint32_t box_rows = 128) {
  static std::unordered_map<Tmap2Key, CUtensorMap, Tmap2Hash> cache;
  static std::mutex mu;
  Tmap2Key key{ptr, rows, cols, ld | ((uint64_t)box_rows << 48)};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld * 2};
  uint32_t box[2] = {64, box_rows};
  int rc = make_tmap(out, ptr, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

}  // namespace b200

using namespace b200;

static int g_raster = 16;
static int g_force_bn = 0;      // 0: choose per problem; 128..256: fixed tile width (benchmarks)
static int g_l2_prefetch = 0;   // prefetch distance in k-blocks (0 = off)

static int launch_2cta(const void* A, const void* W, Gemm2Params& p, int lda, int ldw, long a_rows,
                       cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_2cta_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         G2_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int max_clusters = num_sms() / 2;
  p.tiles_m = (p.M + G2_BM - 1) / G2_BM;
  // Tile width.  256 columns make the best use of the tensor cores, but whole waves of tiles
  // over the CTA pairs matter more when there are only a few tiles: a decode batch of 768 rows
  // against N = 4096 is 48 tiles of 256 columns on 74 pairs (35% of the GPU idle), or 66 tiles
  // of 192 columns in the same single wave.  Cost model: waves x tile width; a narrower tile
  // must win by 8% to be taken.  M = 768, N = 4096 ends at 176 columns: 72 tiles on 74 pairs.
  const int bn_step = (p.mode & G2_RS) ? 32 : 16;
  if (p.swiglu) {
    p.bn = G2_BN;
  } else if (g_force_bn >= 128 && g_force_bn <= 256 && (g_force_bn % bn_step) == 0) {
    p.bn = g_force_bn;
  } else {
    auto cost = [&](int bn) {
      const long tiles = (long)p.tiles_m * ((p.N + bn - 1) / bn);
      return ((tiles + max_clusters - 1) / max_clusters) * bn;
    };
    p.bn = G2_BN;
    long best = cost(G2_BN);
    for (int bn = G2_BN - bn_step; bn >= 128; bn -= bn_step) {
      const long c = cost(bn);
      if (c * 100 < best * 92) {
        best = c;
        p.bn = bn;
      }
    }
  }
  CUtensorMap ta, tb;
  int rc = get_tmap_128x64(&ta, A, (uint64_t)a_rows, (uint64_t)p.K, (uint64_t)lda);
  if (rc) return rc;
  rc = get_tmap_128x64(&tb, W, (uint64_t)(p.swiglu ? 2L * p.N : p.N), (uint64_t)p.K, (uint64_t)ldw,
                       p.swiglu ? 128u : (uint32_t)(p.bn >> 1));
  if (rc) return rc;
  p.up_row_offset = p.N;
  const int out_per_tile = p.swiglu ? 128 : p.bn;
  p.tiles_n = (p.N + out_per_tile - 1) / out_per_tile;
  int clusters = p.tiles_m * p.tiles_n;
  if (clusters > max_clusters) clusters = max_clusters;
  p.raster = g_raster;
  // L2 prefetch of the streamed operands ahead of the staged loads: measured neutral to slightly
  // negative on decode-sized problems (768 x 4096 x 12288: 0.0799 ms off, 0.0799 / 0.0810 / 0.0819 ms
  // at 8 / 16 / 32 k-blocks), so it is off unless asked for
  p.l2_prefetch = g_l2_prefetch > 0 ? g_l2_prefetch : 0;
  gemm_bf16_2cta_kernel<<<2 * clusters, G2_THREADS, G2_SMEM_BYTES, stream>>>(ta, tb, p);
  return B200_CHECK_LAUNCH();
}

// All-gather -> GEMM with the paired-CTA kernel (contract of b200_gemm_ag_bf16; swiglu != 0
// additionally fuses silu(gate) * up, W = [gate (N rows); up (N rows)]).
B200_API int b200_gemm_ag_bf16_2cta(const void* A, const void* W, void* C, const void* bias, int M,
                                    int N, int K, int lda, int ldw, int ldc, void* ctl,
                                    int my_rank, int num_ranks, int rows_per_src, int swiglu,
                                    int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  if (num_ranks > kMaxRanks || rows_per_src <= 0) return 9130;
  if (swiglu && (N % 128)) return 9132;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.swiglu = swiglu;
  p.mode = G2_AG;
  CommCtl* c = (CommCtl*)ctl;
  p.ag_flags = c->ag_flag;
  p.ag_epoch = &c->ag_epoch;
  p.ctl = c;
  p.rows_per_src = rows_per_src;
  p.my_rank = my_rank;
  p.num_ranks = num_ranks;
  return launch_2cta(A, W, p, lda, ldw, M, stream);
}

// GEMM -> reduce-scatter with the paired-CTA kernel (contract of b200_gemm_rs_bf16).
B200_API int b200_gemm_rs_bf16_2cta(const void* A, const void* W, const void* bias, int M, int N,
                                    int K, int lda, int ldw, void* const* rs_staging,
                                    void* const* peer_ctl, int my_rank, int num_ranks,
                                    int rows_per_owner, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7)) return 9100;
  if (num_ranks > kMaxRanks || (long)rows_per_owner * num_ranks < M) return 9130;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = N;
  p.bias = (const __nv_bfloat16*)bias;
  p.status = status;
  p.mode = G2_RS | G2_PUB;
  p.my_rank = my_rank;
  p.num_ranks = num_ranks;
  p.rows_per_owner = rows_per_owner;
  for (int o = 0; o < num_ranks; o++) {
    p.rs_dst[o] = (__nv_bfloat16*)rs_staging[o];
    p.rs_flag_dst[o] = &((CommCtl*)peer_ctl[o])->rs_flag[my_rank];
  }
  p.ctl = (CommCtl*)peer_ctl[my_rank];
  return launch_2cta(A, W, p, lda, ldw, M, stream);
}

// GEMM whose output stays in this rank's own buffer C [M, N] (a multicast-bound partial-sum buffer)
// and whose completion is published to every peer's rs_flag: the producer side of the NVLS
// reduce (b200_nvls_reduce_add_norm_push sums the ranks' buffers inside the switch).
B200_API int b200_gemm_pub_bf16_2cta(const void* A, const void* W, void* C, const void* bias, int M,
                                     int N, int K, int lda, int ldw, int ldc, void* const* peer_ctl,
                                     int my_rank, int num_ranks, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  if (num_ranks > kMaxRanks) return 9130;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.mode = G2_PUB;
  p.my_rank = my_rank;
  p.num_ranks = num_ranks;
  for (int o = 0; o < num_ranks; o++) p.rs_flag_dst[o] = &((CommCtl*)peer_ctl[o])->rs_flag[my_rank];
  p.ctl = (CommCtl*)peer_ctl[my_rank];
  return launch_2cta(A, W, p, lda, ldw, M, stream);
}

// Same contract as b200_gemm_bf16; with swiglu != 0, W is [gate (N rows); up (N rows)]
// (N a multiple of 128) and C[M, N] = silu(A Wg^T) * (A Wu^T).
B200_API int b200_gemm_bf16_2cta(const void* A, const void* W, void* C, const void* bias,
                                 const void* residual, int M, int N, int K, int lda, int ldw,
                                 int ldc, int swiglu, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  if (swiglu && (N % 128)) return 9132;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.swiglu = swiglu;
  return launch_2cta(A, W, p, lda, ldw, M, stream);
}

// Distance (k-blocks) of the L2 prefetch for every following call; 0 or negative = off (the default).
B200_API int b200_gemm_2cta_set_l2_prefetch(int kblocks) {
  g_l2_prefetch = kblocks;
  return 0;
}

// Fixed tile width of the paired-CTA kernel for every following call (0 = choose per problem).
B200_API int b200_gemm_2cta_set_bn(int bn) {
  g_force_bn = bn;
  return 0;
}

// b200_gemm_bf16_2cta with the RMSNorm around it folded in (either side optional):
// Statistics buffers: fp32 [ss_parts_max][ss_stride] (ss_stride >= M) followed by one int32.
//   row_ss_in : accumulators are scaled by rsqrt(sum of the row's partials / norm_dim + eps) (the
//               normalisation of A's rows; the norm weight is expected inside W); the trailing int
//               says how many partials the producer wrote,
//   row_ss_out: partial [column tile][row] = sum of squares of the stored output row (+bias
//               +residual, bf16) inside that column tile, and the tile count in the trailing int.
// Partials instead of atomic adds: the total is summed in a fixed order, so a step repeats bit for
// bit.  The output must have at most ss_parts_max column tiles of the narrowest tile width (128).
B200_API int b200_gemm_bf16_2cta_norm(const void* A, const void* W, void* C, const void* bias,
                                      const void* residual, int M, int N, int K, int lda, int ldw,
                                      int ldc, int swiglu, const void* row_ss_in, int norm_dim,
                                      float eps, void* row_ss_out, long ss_stride, int ss_parts_max,
                                      int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  if (swiglu && (N % 128)) return 9132;
  if (row_ss_in && norm_dim <= 0) return 9133;
  if ((row_ss_in || row_ss_out) && (ss_stride < M || ss_parts_max < 1)) return 9134;
  if (row_ss_out && (long)ss_parts_max * 128 < N) return 9135;
  Gemm2Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.swiglu = swiglu;
  p.row_ss_in = (const float*)row_ss_in;
  p.inv_dim = norm_dim > 0 ? 1.f / (float)norm_dim : 0.f;
  p.eps = eps;
  p.row_ss_out = (float*)row_ss_out;
  p.ss_stride = ss_stride;
  p.ss_parts_max = ss_parts_max;
  return launch_2cta(A, W, p, lda, ldw, M, stream);
}

// Tile order of the paired-CTA kernel: M-tiles per raster group (1 = plain column-major).
B200_API int b200_gemm_2cta_set_raster(int m_tiles_per_group) {
  g_raster = m_tiles_per_group < 1 ? 1 : m_tiles_per_group;
  return 0;
}
