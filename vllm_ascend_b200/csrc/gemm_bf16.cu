// bf16 GEMM family for sm_100a:  C[M,N] = A[M,K] * W[N,K]^T  with fused variants.
//
// Both operands are K-major (row-major activations, nn.Linear weights) — the
// layout of every linear layer of the decoder (parity: the reference's
// unquantized GEMM op, vllm_ascend/ops/linear.py:53-110, and its communication-
// fused linear ops, vllm_ascend/ops/linear_op.py:152-273).
//
// One persistent, warp-specialised kernel (one CTA per SM):
//   warp 0      TMA producer: 128x64 A tile + BNx64 W tile per stage, 128B swizzle
//   warp 1      MMA issuer: tcgen05.mma cta_group::1, M=128, N=BN, K=16, f32 accum in TMEM
//   warps 2..5  epilogue: tcgen05.ld 32x32b -> bf16 -> 16-byte stores
// Two TMEM accumulator buffers let the epilogue of tile i overlap the main
// loop of tile i+1.  Mode bits select the fused behaviour:
//   AG     all-gather -> GEMM: rows of A are pushed into this GPU's memory by its
//          peers; the producer waits for the source rank's epoch flag before
//          loading a tile and starts with the locally produced rows.
//   RS     GEMM -> reduce-scatter: the epilogue stores each bf16 partial row
//          straight into the owning rank's staging buffer over NVLink (peer
//          pointers), and the last CTA publishes this rank's epoch flag.
//   SWIGLU W holds [gate; up]; the tile pairs 128 gate with 128 up columns and the
//          epilogue writes silu(gate) * up.
//   GROUPED rows of A are grouped by expert (prefix offsets on the device) and
//          each group multiplies its own weight matrix (MoE grouped GEMM).
// All waits are bounded (see common.cuh / comm.cuh).
#include "comm.cuh"
#include "common.cuh"

#include <mutex>
#include <unordered_map>

namespace b200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_MAX_GROUPS = 512;

enum : int { GEMM_AG = 1, GEMM_RS = 2, GEMM_SWIGLU = 4, GEMM_GROUPED = 8,
              GEMM_WAITFLAGS = 16,   // producer waits for every rank's flag before the first load
              GEMM_SCATTER = 32,     // epilogue stores row i to peer (row_meta[i] >> 24), row (row_meta[i] & 0xffffff)
              GEMM_PUB = 64 };       // last CTA publishes the reduce-scatter epoch (with GEMM_RS, or alone: rows stay local)

template <int BN>
struct GemmCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = GEMM_BM * GEMM_BK * 2;
  static constexpr int kBBytes = BN * GEMM_BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;  // 256 or 512 (power of two)
  // tiles + barriers + tmem pointer + abort word + group table, plus alignment slack
  // epilogues that store rows into another GPU's memory (reduce-scatter, MoE scatter) stage 32 rows x
  // 64 columns per warp (128 B per row + 16 B pad) and send 128-byte row segments
  static constexpr int kRsRowBytes = 144;
  static constexpr int kRsStageOff = (kStages * kStageBytes + 256 + (GEMM_MAX_GROUPS + 1) * 4 + 15) / 16 * 16;
  static constexpr int kSmemBytes = kRsStageOff + 4 * 32 * kRsRowBytes + 1024;
};

struct GemmParams {
  int M, N, K;         // N = output columns (after SwiGLU pairing: columns of the product / 2)
  int ldc;             // row stride of C (elements)
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldc] or null
  __nv_bfloat16* C;
  int* status;         // device status word (may be null)
  int tiles_m, tiles_n;
  int mode;
  // ---- AG
  const uint32_t* ag_flags;   // local CommCtl.ag_flag
  const uint32_t* ag_epoch;   // local CommCtl.ag_epoch (epoch to wait for)
  int rows_per_src;
  int my_rank, num_ranks;
  // ---- RS
  __nv_bfloat16* rs_dst[kMaxRanks];   // staging on owner o: [num_ranks][rows_per_owner][N]
  uint32_t* rs_flag_dst[kMaxRanks];   // &ctl(o)->rs_flag[my_rank]
  CommCtl* ctl;
  int rows_per_owner;
  // ---- SWIGLU
  int up_row_offset;          // row of W where the "up" half starts (I), per group
  // ---- GROUPED
  const int* group_offsets;   // [num_groups + 1] row offsets into A / C
  int num_groups;
  int w_rows_per_group;       // rows of W per group
  // ---- WAITFLAGS / SCATTER (fused MoE): rs_dst[] = peers' combine buffers
  const uint32_t* wait_flags;   // [num_ranks] local flags
  const uint32_t* wait_epoch;   // wait for *wait_epoch + 1
  const int* row_meta;          // [rows] (dst rank << 24) | dst row
  MoeCtl* moe_ctl;              // local control block (epoch, done counter)
  uint32_t* moe_flag_dst[kMaxRanks];   // &moe_ctl(o)->comb_flag[my_rank]
};

struct TileCoord {
  int row0;      // first row of the tile in A / C
  int row_end;   // rows >= row_end are not stored
  int tn;        // N tile index
  int w_row0;    // first row of W for the (gate) part of the tile
};

template <int BN>
__device__ __forceinline__ bool tile_coord(const GemmParams& p, const int* grp_tiles, int t,
                                           TileCoord& c) {
  constexpr int BN_OUT = BN;  // columns of W consumed per tile
  if (p.mode & GEMM_GROUPED) {
    // grp_tiles[e] = first tile (in units of M tiles) of group e
    int lo = 0, hi = p.num_groups;
    const int tm_global = t % grp_tiles[p.num_groups];
    const int tn = t / grp_tiles[p.num_groups];
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (grp_tiles[mid] <= tm_global) lo = mid; else hi = mid;
    }
    const int e = lo;
    const int g0 = p.group_offsets[e], g1 = p.group_offsets[e + 1];
    c.row0 = g0 + (tm_global - grp_tiles[e]) * GEMM_BM;
    c.row_end = g1;
    c.tn = tn;
    const int ncols = (p.mode & GEMM_SWIGLU) ? BN_OUT / 2 : BN_OUT;
    c.w_row0 = e * p.w_rows_per_group + tn * ncols;
    return true;
  }
  int tm = t % p.tiles_m;
  const int tn = t / p.tiles_m;
  if (p.mode & GEMM_AG) {
    const int rot = (p.my_rank * p.rows_per_src) / GEMM_BM;
    tm = (tm + rot) % p.tiles_m;
  }
  c.row0 = tm * GEMM_BM;
  c.row_end = p.M;
  c.tn = tn;
  const int ncols = (p.mode & GEMM_SWIGLU) ? BN_OUT / 2 : BN_OUT;
  c.w_row0 = tn * ncols;
  return true;
}

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
  using Cfg = GemmCfg<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles = smem;
  uint64_t* full_bar = (uint64_t*)(smem + Cfg::kStages * Cfg::kStageBytes);
  uint64_t* empty_bar = full_bar + Cfg::kStages;
  uint64_t* tmem_full = empty_bar + Cfg::kStages;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;             // [2]
  uint32_t* tmem_ptr = (uint32_t*)(tmem_empty + 2);
  volatile int* abort_word = (volatile int*)(tmem_ptr + 1);
  int* grp_tiles = (int*)(tmem_ptr + 2);            // [num_groups + 1] (GROUPED only)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
  const bool swiglu = (p.mode & GEMM_SWIGLU) != 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);  // one arrival per epilogue warp
    }
    *abort_word = 0;
    mbar_fence_init();
    if (p.mode & GEMM_GROUPED) {
      // offsets come from device memory the caller filled: a table that is not ascending inside
      // [0, M] (stale or overwritten) is reported and yields no tiles instead of addresses
      int acc = 0;
      bool ok = p.group_offsets[0] >= 0;
      for (int e = 0; e < p.num_groups; e++) {
        grp_tiles[e] = acc;
        const int g0 = p.group_offsets[e], g1 = p.group_offsets[e + 1];
        if (g1 < g0 || g1 > p.M) ok = false;
        const int cnt = ok ? g1 - g0 : 0;
        acc += (cnt + GEMM_BM - 1) / GEMM_BM;
      }
      if (!ok) {
        for (int e = 0; e <= p.num_groups; e++) grp_tiles[e] = 0;
        acc = 0;
        if (p.status) atomicCAS(p.status, 0, B200_BAD_INDEX);
      }
      grp_tiles[p.num_groups] = acc;
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, Cfg::kTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_ptr;
  const int num_tiles = (p.mode & GEMM_GROUPED) ? grp_tiles[p.num_groups] * p.tiles_n
                                                : p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    uint32_t ag_epoch = 0;
    if (p.mode & GEMM_AG) ag_epoch = *((volatile const uint32_t*)p.ag_epoch);
    if ((p.mode & GEMM_WAITFLAGS) && blockIdx.x < num_tiles) {
      // rows of A are written by peers: wait until every rank has published this call's epoch
      if (lane == 0) {
        const uint32_t e = *((volatile const uint32_t*)p.wait_epoch) + 1;
        for (int s = 0; s < p.num_ranks; s++)
          if (!wait_flag_ge(&p.wait_flags[s], e, p.status)) { *abort_word = B200_TIMEOUT; break; }
        fence_proxy_async_global();
      }
      __syncwarp();
      if (*abort_word) goto done;
    }
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      TileCoord c;
      tile_coord<BN>(p, grp_tiles, t, c);
      if (p.mode & GEMM_AG) {
        // rows of this tile come from source ranks s0..s1: wait for their pushes
        if (lane == 0) {
          const int last_row = min(c.row0 + GEMM_BM, p.M) - 1;
          const int s0 = c.row0 / p.rows_per_src, s1 = last_row / p.rows_per_src;
          for (int s = s0; s <= s1; s++) {
            if (s == p.my_rank) continue;
            if (!wait_flag_ge(&p.ag_flags[s], ag_epoch, p.status)) *abort_word = B200_TIMEOUT;
          }
          fence_proxy_async_global();
        }
        __syncwarp();
        if (*abort_word) goto done;
      }
      for (int kb = 0; kb < num_kb; kb++) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word)) goto done;
        if (lane == 0) {
          uint8_t* sa = tiles + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * GEMM_BK, c.row0);
          if (swiglu) {
            // 128 gate rows then 128 up rows (the W tensor map has a 128-row box)
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * GEMM_BK, c.w_row0);
            tma_load_2d(sb + Cfg::kBBytes / 2, &tmap_b, &full_bar[stage], kb * GEMM_BK,
                        c.w_row0 + p.up_row_offset);
          } else {
            tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * GEMM_BK, c.w_row0);
          }
        }
        __syncwarp();
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_f16(GEMM_BM, BN, true, false, false);
    int stage = 0;
    uint32_t phase = 0;
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, it++) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_word)) goto done;
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + acc * BN;
      for (int kb = 0; kb < num_kb; kb++) {
        if (!mbar_wait(&full_bar[stage], phase, abort_word)) goto done;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(tiles + stage * Cfg::kStageBytes);
          const uint32_t sb = sa + Cfg::kABytes;
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; kk++) {
            const uint64_t da = make_smem_desc(sa + kk * 32, 16, 1024, kLayoutSw128);
            const uint64_t db = make_smem_desc(sb + kk * 32, 16, 1024, kLayoutSw128);
            umma_f16_ss(d_tmem, da, db, idesc, (kb > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (kb == num_kb - 1) umma_commit(&tmem_full[acc]);
        }
        __syncwarp();
        if (++stage == Cfg::kStages) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    constexpr int OUT_COLS = BN;             // accumulator columns per tile
    const bool remote_rows = (p.mode & (GEMM_RS | GEMM_SCATTER)) != 0;
    uint8_t* rs_stage = smem + Cfg::kRsStageOff + q * (32 * Cfg::kRsRowBytes);
    const int out_per_tile = swiglu ? OUT_COLS / 2 : OUT_COLS;
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, it++) {
      TileCoord c;
      tile_coord<BN>(p, grp_tiles, t, c);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_word)) goto done;
      tc_fence_after();
      const int row = c.row0 + q * 32 + lane;
      const bool row_ok = row < c.row_end;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      __nv_bfloat16* crow;
      if (p.mode & GEMM_RS) {
        const int owner = row_ok ? row / p.rows_per_owner : 0;
        const int local = row - owner * p.rows_per_owner;
        crow = p.rs_dst[owner] + ((size_t)p.my_rank * p.rows_per_owner + local) * p.ldc;
      } else if (p.mode & GEMM_SCATTER) {
        const int meta = row_ok ? p.row_meta[row] : 0;
        crow = p.rs_dst[(meta >> 24) & (kMaxRanks - 1)] + (size_t)(meta & 0xffffff) * p.ldc;
      } else {
        crow = p.C + (size_t)row * p.ldc;
      }
      const __nv_bfloat16* rrow = p.residual ? p.residual + (size_t)row * p.ldc : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < out_per_tile; c0 += 32) {
        const int col0 = c.tn * out_per_tile + c0;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c0, r);
        if (swiglu) {
          uint32_t u[32];
          tmem_ld_32x32b_x32(t_row + OUT_COLS / 2 + c0, u);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; j++) {
            const float g = __uint_as_float(r[j]);
            r[j] = __float_as_uint(g / (1.f + __expf(-g)) * __uint_as_float(u[j]));
          }
        } else {
          tmem_ld_wait();
        }
        if (row_ok) {
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const int col = col0 + g * 8;
            if (col < p.N) {  // N is a multiple of 8
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; j++) v[j] = __uint_as_float(r[g * 8 + j]);
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
              if (remote_rows)
                *reinterpret_cast<uint4*>(rs_stage + lane * Cfg::kRsRowBytes + ((c0 & 32) + g * 8) * 2) = o;
              else
                *reinterpret_cast<uint4*>(crow + col) = o;
            }
          }
        }
        if (remote_rows) {
          // flush after two 32-column chunks (or at the last chunk): lanes regroup so one store
          // instruction covers 4 rows x 128 contiguous bytes (8 rows x 64 bytes for a lone chunk)
          const bool last = (col0 + 32 >= p.N) || (c0 + 32 >= out_per_tile);
          if ((c0 & 32) || last) {
            __syncwarp();
            const int staged = (c0 & 32) ? 64 : 32;
            const int colbase = col0 - (c0 & 32);
            const int segs = staged >> 3;
            const int rows_per_inst = 32 / segs;
            const unsigned long long my_ptr = (unsigned long long)crow;
            for (int r0 = 0; r0 < 32; r0 += rows_per_inst) {
              const int rr = r0 + lane / segs, sg = lane % segs;
              const unsigned long long ptr = __shfl_sync(0xffffffffu, my_ptr, rr);
              const int ok = __shfl_sync(0xffffffffu, (int)row_ok, rr);
              const int col = colbase + sg * 8;
              if (ok && col < p.N)
                *reinterpret_cast<uint4*>((__nv_bfloat16*)ptr + col) =
                    *reinterpret_cast<const uint4*>(rs_stage + rr * Cfg::kRsRowBytes + sg * 16);
            }
            __syncwarp();
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
    if (p.mode & (GEMM_RS | GEMM_SCATTER | GEMM_PUB)) __threadfence_system();   // rows visible to their owners
  }
done:
  tc_fence_before();
  __syncthreads();
  if (*abort_word != 0) {
    const uint64_t t_start = globaltimer_ns();
    while (globaltimer_ns() - t_start < 50000ull) __nanosleep(1000);
    if (threadIdx.x == 0 && p.status) atomicExch(p.status, *abort_word);
    __syncthreads();
  } else if ((p.mode & GEMM_PUB) && threadIdx.x == 0) {
    // last CTA of the grid publishes this rank's reduce-scatter epoch to every owner
    const uint32_t prev = atomicAdd(&p.ctl->done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      const uint32_t epoch = p.ctl->rs_epoch + 1;
      for (int o = 0; o < p.num_ranks; o++) st_release_sys(p.rs_flag_dst[o], epoch);
      p.ctl->rs_epoch = epoch;
      p.ctl->done_ctr = 0;
      __threadfence();
    }
  } else if ((p.mode & GEMM_SCATTER) && threadIdx.x == 0) {
    // last CTA tells every token owner that this rank's expert outputs are in its buffer
    const uint32_t prev = atomicAdd(&p.moe_ctl->done_ctr2, 1u);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      const uint32_t epoch = *((volatile uint32_t*)&p.moe_ctl->epoch) + 1;
      for (int o = 0; o < p.num_ranks; o++) st_release_sys(p.moe_flag_dst[o], epoch);
      p.moe_ctl->done_ctr2 = 0;
      __threadfence();
    }
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ---------------------------------------------------------------- host
struct TmapKey {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows;
  bool operator==(const TmapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ k.box_rows;
    return h;
  }
};

// Tensor map of a row-major bf16 [rows, cols] matrix with row stride ld, box
// = [box_rows, 64 cols], 128-byte swizzle.  Cached: encoding costs a few us.
static int get_tmap_2d_bf16(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                            uint64_t ld, uint32_t box_rows) {
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  static std::mutex mu;
  TmapKey key{ptr, rows, cols, ld, box_rows};
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

template <int BN>
static int launch_gemm(const void* A, const void* W, GemmParams& p, int lda, int ldw,
                       long a_rows, long w_rows, int max_ctas, cudaStream_t stream) {
  using Cfg = GemmCfg<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_bf16_kernel<BN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  CUtensorMap ta, tb;
  int rc = get_tmap_2d_bf16(&ta, A, (uint64_t)a_rows, (uint64_t)p.K, (uint64_t)lda, GEMM_BM);
  if (rc) return rc;
  const uint32_t b_box = (p.mode & GEMM_SWIGLU) ? BN / 2 : BN;
  rc = get_tmap_2d_bf16(&tb, W, (uint64_t)w_rows, (uint64_t)p.K, (uint64_t)ldw, b_box);
  if (rc) return rc;
  const int out_per_tile = (p.mode & GEMM_SWIGLU) ? BN / 2 : BN;
  p.tiles_m = (p.M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (p.N + out_per_tile - 1) / out_per_tile;
  int sms = num_sms();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  int grid;
  if (p.mode & GEMM_GROUPED) {
    grid = sms;   // tile count is only known on the device
  } else {
    grid = p.tiles_m * p.tiles_n;
    if (grid > sms) grid = sms;
  }
  gemm_bf16_kernel<BN><<<grid, GEMM_THREADS, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return B200_CHECK_LAUNCH();
}

static int pick_bn(int M, int N, int bn) {
  if (bn == 128 || bn == 256) return bn;
  // 256-wide tiles halve A re-reads; use them when they still fill the GPU.
  const long tiles256 = (long)((M + 127) / 128) * ((N + 255) / 256);
  bn = (N >= 256 && tiles256 >= num_sms()) ? 256 : 128;
  if (N % 256 != 0 && N % 128 == 0) bn = 128;
  return bn;
}

static void init_params(GemmParams& p) { memset(&p, 0, sizeof(p)); }

}  // namespace b200

using namespace b200;

// C[M,N] (row stride ldc) = A[M,K] (row stride lda) * W[N,K]^T (row stride ldw)
// (+bias[N]) (+residual[M,N] with row stride ldc).  Requirements: K, N, lda,
// ldw, ldc multiples of 8; all base pointers 16-byte aligned.  bn selects the
// N tile (128 or 256; 0 = choose).  Returns 0 or a CUDA / encode error code.
B200_API int b200_gemm_bf16(const void* A, const void* W, void* C, const void* bias,
                            const void* residual, int M, int N, int K, int lda, int ldw,
                            int ldc, int bn, int* status, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  GemmParams p;
  init_params(p);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  if (pick_bn(M, N, bn) == 256) return launch_gemm<256>(A, W, p, lda, ldw, M, N, max_ctas, stream);
  return launch_gemm<128>(A, W, p, lda, ldw, M, N, max_ctas, stream);
}

// out[M, I] = silu(A W_gate^T) * (A W_up^T) with W = [gate (I rows); up (I rows)] of row
// stride ldw.  I must be a multiple of 128.
B200_API int b200_gemm_swiglu_bf16(const void* A, const void* W, void* out, int M, int I, int K,
                                   int lda, int ldw, int ldo, int* status,
                                   cudaStream_t stream) {
  if (M <= 0 || I <= 0) return 0;
  if ((K & 7) || (I % 128) || (lda & 7) || (ldw & 7) || (ldo & 7)) return 9100;
  GemmParams p;
  init_params(p);
  p.M = M; p.N = I; p.K = K; p.ldc = ldo;
  p.C = (__nv_bfloat16*)out;
  p.status = status;
  p.mode = GEMM_SWIGLU;
  p.up_row_offset = I;
  return launch_gemm<256>(A, W, p, lda, ldw, M, 2L * I, 0, stream);
}

// All-gather -> GEMM.  A [M, K] lives in this rank's gather buffer; rows
// [s*rows_per_src, (s+1)*rows_per_src) are pushed by rank s, which then raises
// ctl->ag_flag[s] to the current epoch (ctl->ag_epoch).
B200_API int b200_gemm_ag_bf16(const void* A, const void* W, void* C, const void* bias, int M,
                               int N, int K, int lda, int ldw, int ldc, void* ctl, int my_rank,
                               int num_ranks, int rows_per_src, int bn, int* status,
                               cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  if (num_ranks > kMaxRanks || rows_per_src <= 0) return 9130;
  GemmParams p;
  init_params(p);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.mode = GEMM_AG;
  CommCtl* c = (CommCtl*)ctl;
  p.ag_flags = c->ag_flag;
  p.ag_epoch = &c->ag_epoch;
  p.ctl = c;
  p.rows_per_src = rows_per_src;
  p.my_rank = my_rank;
  p.num_ranks = num_ranks;
  if (pick_bn(M, N, bn) == 256) return launch_gemm<256>(A, W, p, lda, ldw, M, N, 0, stream);
  return launch_gemm<128>(A, W, p, lda, ldw, M, N, 0, stream);
}

// GEMM -> reduce-scatter.  Row r of the bf16 partial product goes to rank
// o = r / rows_per_owner, at rs_staging[o][my_rank][r % rows_per_owner][0..N).
// rs_staging / peer_ctl: host arrays of num_ranks device pointers (peer-mapped).
B200_API int b200_gemm_rs_bf16(const void* A, const void* W, const void* bias, int M, int N,
                               int K, int lda, int ldw, void* const* rs_staging,
                               void* const* peer_ctl, int my_rank, int num_ranks,
                               int rows_per_owner, int bn, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7)) return 9100;
  if (num_ranks > kMaxRanks || rows_per_owner * num_ranks < M) return 9130;
  GemmParams p;
  init_params(p);
  p.M = M; p.N = N; p.K = K; p.ldc = N;
  p.bias = (const __nv_bfloat16*)bias;
  p.status = status;
  p.mode = GEMM_RS | GEMM_PUB;
  p.my_rank = my_rank;
  p.num_ranks = num_ranks;
  p.rows_per_owner = rows_per_owner;
  for (int o = 0; o < num_ranks; o++) {
    p.rs_dst[o] = (__nv_bfloat16*)rs_staging[o];
    p.rs_flag_dst[o] = &((CommCtl*)peer_ctl[o])->rs_flag[my_rank];
  }
  p.ctl = (CommCtl*)peer_ctl[my_rank];
  if (pick_bn(M, N, bn) == 256) return launch_gemm<256>(A, W, p, lda, ldw, M, N, 0, stream);
  return launch_gemm<128>(A, W, p, lda, ldw, M, N, 0, stream);
}

// GEMM into this rank's own buffer C (a multicast-bound partial-sum buffer) that publishes its
// completion to every peer's rs_flag: producer side of b200_nvls_reduce_add_norm_push.
B200_API int b200_gemm_pub_bf16(const void* A, const void* W, void* C, const void* bias, int M, int N,
                                int K, int lda, int ldw, int ldc, void* const* peer_ctl, int my_rank,
                                int num_ranks, int bn, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  if (num_ranks > kMaxRanks) return 9130;
  GemmParams p;
  init_params(p);
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.mode = GEMM_PUB;
  p.my_rank = my_rank;
  p.num_ranks = num_ranks;
  for (int o = 0; o < num_ranks; o++) p.rs_flag_dst[o] = &((CommCtl*)peer_ctl[o])->rs_flag[my_rank];
  p.ctl = (CommCtl*)peer_ctl[my_rank];
  if (pick_bn(M, N, bn) == 256) return launch_gemm<256>(A, W, p, lda, ldw, M, N, 0, stream);
  return launch_gemm<128>(A, W, p, lda, ldw, M, N, 0, stream);
}

// Grouped GEMM (MoE): rows [offsets[e], offsets[e+1]) of A multiply W[e] ([n_per_group, K]);
// with swiglu != 0, W[e] = [gate (I); up (I)] and C has I columns.  total_rows bounds the
// rows of A / C; offsets is a device int32 array of num_groups + 1 entries.
B200_API int b200_grouped_gemm_bf16(const void* A, const void* W, void* C, const void* offsets,
                                    int num_groups, long total_rows, int N, int K, int lda,
                                    int ldw, int ldc, int swiglu, int* status,
                                    cudaStream_t stream) {
  if (total_rows <= 0 || N <= 0 || num_groups <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  if (num_groups > GEMM_MAX_GROUPS) return 9131;
  if (swiglu && (N % 128)) return 9132;
  GemmParams p;
  init_params(p);
  p.M = (int)total_rows; p.N = N; p.K = K; p.ldc = ldc;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.mode = GEMM_GROUPED | (swiglu ? GEMM_SWIGLU : 0);
  p.group_offsets = (const int*)offsets;
  p.num_groups = num_groups;
  p.w_rows_per_group = swiglu ? 2 * N : N;
  p.up_row_offset = N;
  const long w_rows = (long)num_groups * p.w_rows_per_group;
  if (swiglu || N % 256 == 0)
    return launch_gemm<256>(A, W, p, lda, ldw, total_rows, w_rows, 0, stream);
  return launch_gemm<128>(A, W, p, lda, ldw, total_rows, w_rows, 0, stream);
}

// Fused-MoE expert GEMMs over the packed receive pool of this rank.
//   gemm1: act[r, :I] = silu(X W1g^T) * (X W1u^T) for the rows of every local expert; the
//          producer first waits until every rank's dispatch flag reached epoch + 1.
//   gemm2: row r of act W2^T is stored straight into the token owner's combine buffer over
//          peer memory (owner and row from row_meta), then the owners are flagged.
// offsets: device int32 [num_groups + 1]; pool_rows: capacity of the pool (rows of X / act).
B200_API int b200_moe_gemm1_bf16(const void* X, const void* W13, void* act, const void* offsets,
                                 int num_groups, long pool_rows, int I, int K, void* moe_ctl,
                                 int num_ranks, int* status, cudaStream_t stream) {
  if ((K & 7) || (I % 128) || num_groups > GEMM_MAX_GROUPS || num_ranks > kMaxRanks) return 9100;
  GemmParams p;
  init_params(p);
  p.M = (int)pool_rows; p.N = I; p.K = K; p.ldc = I;
  p.C = (__nv_bfloat16*)act;
  p.status = status;
  p.mode = GEMM_GROUPED | GEMM_SWIGLU | GEMM_WAITFLAGS;
  p.group_offsets = (const int*)offsets;
  p.num_groups = num_groups;
  p.w_rows_per_group = 2 * I;
  p.up_row_offset = I;
  MoeCtl* c = (MoeCtl*)moe_ctl;
  p.wait_flags = c->disp_flag;
  p.wait_epoch = &c->epoch;
  p.num_ranks = num_ranks;
  return launch_gemm<256>(X, W13, p, K, K, pool_rows, (long)num_groups * 2 * I, 0, stream);
}

B200_API int b200_moe_gemm2_scatter_bf16(const void* act, const void* W2, const void* offsets,
                                         const void* row_meta, int num_groups, long pool_rows,
                                         int H, int I, void* const* comb_bufs,
                                         void* const* peer_moe_ctl, int my_rank, int num_ranks,
                                         int* status, cudaStream_t stream) {
  if ((I & 7) || (H & 7) || num_groups > GEMM_MAX_GROUPS || num_ranks > kMaxRanks) return 9100;
  GemmParams p;
  init_params(p);
  p.M = (int)pool_rows; p.N = H; p.K = I; p.ldc = H;
  p.status = status;
  p.mode = GEMM_GROUPED | GEMM_SCATTER;
  p.group_offsets = (const int*)offsets;
  p.num_groups = num_groups;
  p.w_rows_per_group = H;
  p.row_meta = (const int*)row_meta;
  p.my_rank = my_rank;
  p.num_ranks = num_ranks;
  for (int o = 0; o < num_ranks; o++) {
    p.rs_dst[o] = (__nv_bfloat16*)comb_bufs[o];
    p.moe_flag_dst[o] = &((MoeCtl*)peer_moe_ctl[o])->comb_flag[my_rank];
  }
  p.moe_ctl = (MoeCtl*)peer_moe_ctl[my_rank];
  if (H % 256 == 0)
    return launch_gemm<256>(act, W2, p, I, I, pool_rows, (long)num_groups * H, 0, stream);
  return launch_gemm<128>(act, W2, p, I, I, pool_rows, (long)num_groups * H, 0, stream);
}
