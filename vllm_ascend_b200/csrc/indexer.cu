// "Lightning indexer" scores for sparse attention on tcgen05:
//   score[r, s] = sum_g w[r, g] * relu( q_idx[r, g, :] . k_idx[s, :] )      for s < kv_len[r]
// computed with keys on the MMA M axis: S^T[128 keys, G] = K_tile[128, 128] . Q^T, then every
// epilogue thread owns one key and folds its G columns into one number.  Key pages stream
// through a 3-stage TMA pipeline; tiles are independent, so the grid covers (row, tile chunk).
// Top-k over the scores is taken by the caller.  Same math as the reference's
// npu_lightning_indexer (csrc/attention/lightning_indexer/README.md).
#include "common.cuh"

#include <mutex>
#include <string.h>
#include <string>
#include <unordered_map>

namespace b200 {

constexpr int IDX_THREADS = 192;
constexpr int IDX_D = 128;
constexpr int IDX_HALF = 128 * 128;        // 128 keys x 64 bf16
constexpr int IDX_STAGES = 3;
constexpr int IDX_TILE_BYTES = 2 * IDX_HALF;

struct IdxParams {
  const int* row_seq;
  const int* row_kv_len;
  const int* block_table;
  const float* weights;     // [R, G]
  float* scores;            // [R, score_stride]
  long score_stride;
  int max_blocks, block_size, rows_per_load;
  int G, tiles_per_cta;
  long num_blocks_total;
  int* status;
};

template <int NG>
__global__ void __launch_bounds__(IDX_THREADS, 1)
indexer_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
               const IdxParams p) {
  constexpr int Q_HALF = NG * 128;
  constexpr int Q_BYTES = 2 * Q_HALF;
  const int row = blockIdx.x;
  const int kv_len = p.row_kv_len[row];
  const int n_all = (kv_len + 127) >> 7;
  const int t0 = blockIdx.y * p.tiles_per_cta;
  const int n = min(n_all, t0 + p.tiles_per_cta) - t0;
  if (n <= 0) return;
  const int seq = p.row_seq[row];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* Ks = smem;
  uint8_t* Qs = Ks + IDX_STAGES * IDX_TILE_BYTES;
  uint64_t* bars = (uint64_t*)(Qs + Q_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = k_full + IDX_STAGES;
  uint64_t* s_ready = k_empty + IDX_STAGES;   // 2
  uint64_t* s_free = s_ready + 2;             // 2
  uint32_t* tmem_ptr = (uint32_t*)(s_free + 2);
  volatile int* abort_word = (volatile int*)(tmem_ptr + 1);
  float* w_s = (float*)(tmem_ptr + 2);        // [NG]

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < IDX_STAGES; s++) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&s_ready[b], 1);
      mbar_init(&s_free[b], 4);
    }
    *abort_word = 0;
    mbar_fence_init();
  }
  if (threadIdx.x >= 64 && threadIdx.x - 64 < NG)
    w_s[threadIdx.x - 64] = (int)(threadIdx.x - 64) < p.G ? p.weights[(long)row * p.G + threadIdx.x - 64] : 0.f;
  if (warp == 1) {
    tmem_alloc(tmem_ptr, 128);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
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
      mbar_expect_tx(q_full, Q_BYTES);
      tma_load_3d(Qs, &tmap_q, q_full, 0, 0, row);
      tma_load_3d(Qs + Q_HALF, &tmap_q, q_full, 64, 0, row);
    }
    for (int j = 0; j < n; j++) {
      const int st = j % IDX_STAGES;
      const uint32_t ph = (uint32_t)(j / IDX_STAGES) & 1u;
      const int key_base = (t0 + j) << 7;
      int blk = 0;
      if (lane < parts) blk = bt[min(key_base + lane * rpl, kv_len - 1) / p.block_size];
      bool bad = lane < parts && (blk < 0 || blk >= p.num_blocks_total);
      bad = __any_sync(0xffffffffu, bad);
      if (bad) {
        *abort_word = B200_BAD_INDEX;
        goto done;
      }
      if (!mbar_wait(&k_empty[st], ph ^ 1u, abort_word)) goto done;
      for (int part = 0; part < parts; part++) {
        const int b = __shfl_sync(0xffffffffu, blk, part);
        if (lane == 0) {
          if (part == 0) mbar_expect_tx(&k_full[st], IDX_TILE_BYTES);
          const int off = (key_base + part * rpl) % p.block_size;
          uint8_t* dst = Ks + st * IDX_TILE_BYTES + part * rpl * 128;
          tma_load_3d(dst, &tmap_k, &k_full[st], 0, off, b);
          tma_load_3d(dst + IDX_HALF, &tmap_k, &k_full[st], 64, off, b);
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_f16(128, NG, true, false, false);
    const uint32_t q_addr = smem_u32(Qs), k_addr = smem_u32(Ks);
    if (!mbar_wait(q_full, 0, abort_word)) goto done;
    for (int j = 0; j < n; j++) {
      const int st = j % IDX_STAGES;
      const uint32_t ph = (uint32_t)(j / IDX_STAGES) & 1u;
      const int b = j & 1;
      if (!mbar_wait(&k_full[st], ph, abort_word)) goto done;
      if (!mbar_wait(&s_free[b], (((uint32_t)j >> 1) & 1u) ^ 1u, abort_word)) goto done;
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < IDX_D / 16; kk++) {
          const uint64_t da = make_smem_desc(k_addr + st * IDX_TILE_BYTES + (kk >> 2) * IDX_HALF + (kk & 3) * 32,
                                             16, 1024, kLayoutSw128);
          const uint64_t db = make_smem_desc(q_addr + (kk >> 2) * Q_HALF + (kk & 3) * 32, 16, 1024, kLayoutSw128);
          umma_f16_ss(tmem_base + b * NG, da, db, idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_ready[b]);
      }
      __syncwarp();
    }
  } else {
    // ------------------------------------------------------------ score reduction
    const int qd = warp & 3;
    const int tid = qd * 32 + lane;
    const uint32_t t_lane = tmem_base + ((uint32_t)(qd * 32) << 16);
    float* out = p.scores + (long)row * p.score_stride;
    for (int j = 0; j < n; j++) {
      const int b = j & 1;
      if (!mbar_wait(&s_ready[b], ((uint32_t)j >> 1) & 1u, abort_word)) goto done;
      tc_fence_after();
      float acc = 0.f;
#pragma unroll
      for (int c0 = 0; c0 < NG; c0 += 16) {
        uint32_t r[16];
        tmem_ld_32x32b_x16(t_lane + b * NG + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 16; c++) acc = fmaf(w_s[c0 + c], fmaxf(__uint_as_float(r[c]), 0.f), acc);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[b]);
      const int key = ((t0 + j) << 7) + tid;
      if (key < p.score_stride) out[key] = key < kv_len ? acc : -INFINITY;
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
    tmem_dealloc(tmem_base, 128);
  }
}

struct IdxTmapCache {
  std::unordered_map<std::string, CUtensorMap> map;
  std::mutex mu;
  int get(CUtensorMap* out, const void* base, const uint64_t* dims, const uint64_t* strides,
          const uint32_t* box) {
    char key[72];
    memset(key, 0, sizeof(key));
    memcpy(key, &base, 8);
    memcpy(key + 8, dims, 24);
    memcpy(key + 32, strides, 16);
    memcpy(key + 48, box, 12);
    std::string k(key, 72);
    std::lock_guard<std::mutex> g(mu);
    auto it = map.find(k);
    if (it != map.end()) {
      *out = it->second;
      return 0;
    }
    int rc = make_tmap(out, base, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, dims, strides, box,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    if (map.size() > 4096) map.clear();
    map.emplace(k, *out);
    return 0;
  }
};
static IdxTmapCache g_idx_tmaps;

template <int NG>
static int launch_indexer(const CUtensorMap& tq, const CUtensorMap& tk, const IdxParams& p, dim3 grid,
                          cudaStream_t stream) {
  constexpr int SMEM = IDX_STAGES * IDX_TILE_BYTES + 2 * NG * 128 + 1024 + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(indexer_kernel<NG>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  indexer_kernel<NG><<<grid, IDX_THREADS, SMEM, stream>>>(tq, tk, p);
  return B200_CHECK_LAUNCH();
}

// Gather rows of paged caches: out[r, j, :] = cache[block_table[row_seq[r], idx / bs], idx % bs, :]
// for idx = indices[r, j] (idx < 0: zeros).  width_bytes multiple of 16.
__global__ void gather_paged_rows_kernel(const uint8_t* __restrict__ cache, const int* __restrict__ indices,
                                         const int* __restrict__ row_seq, const int* __restrict__ block_table,
                                         int max_blocks, int block_size, int topk, int width_bytes,
                                         long num_blocks_total, uint8_t* __restrict__ out, int* status) {
  const long r = blockIdx.y;
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int j = blockIdx.x * warps + warp;
  if (j >= topk) return;
  const int idx = indices[r * topk + j];
  uint4* dst = reinterpret_cast<uint4*>(out + (r * topk + j) * (long)width_bytes);
  const int nvec = width_bytes >> 4;
  if (idx < 0) {
    for (int v = lane; v < nvec; v += 32) dst[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const int blk = block_table[(long)row_seq[r] * max_blocks + idx / block_size];
  if (blk < 0 || blk >= num_blocks_total) {
    if (lane == 0 && status) atomicExch(status, B200_BAD_INDEX);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(cache + ((long)blk * block_size + idx % block_size) * width_bytes);
  for (int v = lane; v < nvec; v += 32) dst[v] = src[v];
}

}  // namespace b200

// q_idx [R, G, 128] bf16 (row stride q_stride elements), weights [R, G] fp32,
// k_cache [blocks, block_size, 128] bf16; scores [R, score_stride] fp32 (filled for keys
// < ceil(kv_len / 128) * 128, -inf from kv_len on; the caller pre-fills the rest with -inf).
B200_API int b200_lightning_indexer(const void* q_idx, long q_stride, long R, int G, const void* weights,
                                    const void* k_cache, long num_blocks, int block_size,
                                    const void* row_seq, const void* row_kv_len, const void* block_table,
                                    int max_blocks, int max_kv_len, void* scores, long score_stride,
                                    int* status, cudaStream_t stream) {
  using namespace b200;
  if (R <= 0 || max_kv_len <= 0) return 0;
  if (G < 1 || G > 64) return 9700;
  if (block_size < 8 || (block_size < 128 && (128 % block_size) != 0) ||
      (block_size > 128 && (block_size % 128) != 0))
    return 9701;
  if ((q_stride & 7) || R > 65535) return 9702;
  const int NG = G <= 16 ? 16 : (G <= 32 ? 32 : 64);
  const int rpl = block_size < 128 ? block_size : 128;
  CUtensorMap tq, tk;
  {
    uint64_t dims[3] = {(uint64_t)IDX_D, (uint64_t)G, (uint64_t)R};
    uint64_t str[2] = {(uint64_t)IDX_D * 2, (uint64_t)q_stride * 2};
    uint32_t box[3] = {64, (uint32_t)NG, 1};       // rows beyond G read as zeros (weight 0 anyway)
    int rc = g_idx_tmaps.get(&tq, q_idx, dims, str, box);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)IDX_D, (uint64_t)block_size, (uint64_t)num_blocks};
    uint64_t str[2] = {(uint64_t)IDX_D * 2, (uint64_t)block_size * IDX_D * 2};
    uint32_t box[3] = {64, (uint32_t)rpl, 1};
    int rc = g_idx_tmaps.get(&tk, k_cache, dims, str, box);
    if (rc) return rc;
  }
  IdxParams p;
  p.row_seq = (const int*)row_seq;
  p.row_kv_len = (const int*)row_kv_len;
  p.block_table = (const int*)block_table;
  p.weights = (const float*)weights;
  p.scores = (float*)scores;
  p.score_stride = score_stride;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.rows_per_load = rpl;
  p.G = G;
  p.num_blocks_total = num_blocks;
  p.status = status;
  const int tiles = (max_kv_len + 127) / 128;
  // enough CTAs to fill the GPU, but several tiles per CTA so the Q load is amortised
  int chunks = (2 * num_sms() + (int)R - 1) / (int)R;
  if (chunks < 1) chunks = 1;
  if (chunks > tiles) chunks = tiles;
  p.tiles_per_cta = (tiles + chunks - 1) / chunks;
  chunks = (tiles + p.tiles_per_cta - 1) / p.tiles_per_cta;
  dim3 grid((unsigned)R, (unsigned)chunks);
  if (NG == 16) return launch_indexer<16>(tq, tk, p, grid, stream);
  if (NG == 32) return launch_indexer<32>(tq, tk, p, grid, stream);
  return launch_indexer<64>(tq, tk, p, grid, stream);
}

B200_API int b200_gather_paged_rows(const void* cache, const void* indices, const void* row_seq,
                                    const void* block_table, int max_blocks, int block_size, long R,
                                    int topk, int width_bytes, long num_blocks, void* out, int* status,
                                    cudaStream_t stream) {
  using namespace b200;
  if (R <= 0 || topk <= 0) return 0;
  if ((width_bytes & 15) || R > 65535) return 9100;
  dim3 grid((unsigned)((topk + 7) / 8), (unsigned)R);
  gather_paged_rows_kernel<<<grid, 256, 0, stream>>>((const uint8_t*)cache, (const int*)indices,
                                                     (const int*)row_seq, (const int*)block_table, max_blocks,
                                                     block_size, topk, width_bytes, num_blocks, (uint8_t*)out,
                                                     status);
  return B200_CHECK_LAUNCH();
}
