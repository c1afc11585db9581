// Block-scaled FP8 GEMM for sm_100a (the W8A8 serving format of DeepSeek-V3 style
// checkpoints):
//   C[M,N] (bf16) = sum_kb  a_scale[m, kb] * w_scale[n/128, kb] * (A8[m, kb] . W8[n, kb]^T)
// A8 [M,K] e4m3 with one fp32 scale per (row, 128 columns); W8 [N,K] e4m3 with one
// fp32 scale per 128 x 128 block.  Reference scheme: vllm_ascend/quantization/methods/fp8.py
// (block-scaled weights) + w8a8_dynamic.py (per-token activation scales).
//
// The scales change every 128 columns of K, so products of different K blocks cannot
// be summed inside the tensor core.  Two-level accumulation:
//   warp 0      TMA producer: 128 x 128 e4m3 tiles of A and W (one 128-byte swizzle row each)
//   warp 1      tcgen05.mma kind::f8f6f4 (M=128, N=128, K=32 x 4) per K block into one of two
//               TMEM partial buffers (fresh accumulator every block)
//   warps 2..9  read the partial with tcgen05.ld, scale it by a_scale * w_scale and add it to
//               fp32 accumulators held in registers; store bf16 at the end.  Two warpgroups
//               split the tile's 128 columns (64 accumulators per thread, both TMEM loads of a
//               K block in flight before the one wait): the promotion of a block has to keep up
//               with its MMA, which four warps with 128 accumulators each did not
// The MMA of block kb+1 overlaps the promotion of block kb.  Grouped mode (MoE experts)
// uses per-group row offsets and per-expert weight / scale matrices.  Bounded waits.
#include "common.cuh"

#include <mutex>
#include <unordered_map>

namespace b200 {

constexpr int F8_BM = 128, F8_BN = 128, F8_BK = 128;
constexpr int F8_THREADS = 320;            // producer, MMA issuer, 2 x 4 promotion warps
constexpr int F8_HALF = F8_BN / 2;         // columns per promotion warpgroup
constexpr int F8_STAGES = 6;
constexpr int F8_TILE_BYTES = 128 * 128;                 // 16 KB per operand tile
constexpr int F8_STAGE_BYTES = 2 * F8_TILE_BYTES;
constexpr int F8_MAX_GROUPS = 512;
constexpr int F8_SMEM_BYTES = F8_STAGES * F8_STAGE_BYTES + 1024 + 256 + (F8_MAX_GROUPS + 1) * 4;

struct Fp8Params {
  int M, N, K, ldc;
  const float* a_scale;     // [M, K/128]
  const float* w_scale;     // [groups][ceil(N/128), K/128]
  __nv_bfloat16* C;
  const __nv_bfloat16* bias;
  int* status;
  int tiles_m, tiles_n;
  int num_kb;
  // per-channel mode (dynamic per-token x per-output-channel scales, constant along K):
  // row_scale [M], col_scale [groups][N]; the K blocks are summed unscaled and the product of
  // the two scales is applied once in the epilogue
  const float* row_scale;
  const float* col_scale;
  // grouped
  const int* group_offsets;
  int num_groups;
  int w_rows_per_group;
};

struct F8Tile {
  int row0, row_end, tn, w_row0, group;
};

__device__ __forceinline__ void f8_tile(const Fp8Params& p, const int* grp_tiles, int t, F8Tile& c) {
  if (p.num_groups > 0) {
    const int total_m = grp_tiles[p.num_groups];
    const int tm_global = t % total_m;
    const int tn = t / total_m;
    int lo = 0, hi = p.num_groups;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (grp_tiles[mid] <= tm_global) lo = mid; else hi = mid;
    }
    c.group = lo;
    c.row0 = p.group_offsets[lo] + (tm_global - grp_tiles[lo]) * F8_BM;
    c.row_end = p.group_offsets[lo + 1];
    c.tn = tn;
    c.w_row0 = lo * p.w_rows_per_group + tn * F8_BN;
  } else {
    c.group = 0;
    c.row0 = (t % p.tiles_m) * F8_BM;
    c.row_end = p.M;
    c.tn = t / p.tiles_m;
    c.w_row0 = c.tn * F8_BN;
  }
}

__global__ void __launch_bounds__(F8_THREADS, 1)
gemm_fp8_block_kernel(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b, const Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* tiles = smem;
  uint64_t* full_bar = (uint64_t*)(smem + F8_STAGES * F8_STAGE_BYTES);
  uint64_t* empty_bar = full_bar + F8_STAGES;
  uint64_t* part_full = empty_bar + F8_STAGES;    // [2]
  uint64_t* part_empty = part_full + 2;           // [2]
  uint32_t* tmem_ptr = (uint32_t*)(part_empty + 2);
  volatile int* abort_word = (volatile int*)(tmem_ptr + 1);
  int* grp_tiles = (int*)(tmem_ptr + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = p.num_kb;

  if (threadIdx.x == 0) {
    for (int s = 0; s < F8_STAGES; s++) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; b++) {
      mbar_init(&part_full[b], 1);
      mbar_init(&part_empty[b], 8);
    }
    *abort_word = 0;
    mbar_fence_init();
    if (p.num_groups > 0) {
      // a table that is not ascending inside [0, M] is reported and yields no tiles
      int acc = 0;
      bool ok = p.group_offsets[0] >= 0;
      for (int e = 0; e < p.num_groups; e++) {
        grp_tiles[e] = acc;
        const int g0 = p.group_offsets[e], g1 = p.group_offsets[e + 1];
        if (g1 < g0 || g1 > p.M) ok = false;
        acc += ok ? (g1 - g0 + F8_BM - 1) / F8_BM : 0;
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
    tmem_alloc(tmem_ptr, 256);
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
  const int num_tiles = (p.num_groups > 0 ? grp_tiles[p.num_groups] : p.tiles_m) * p.tiles_n;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      F8Tile c;
      f8_tile(p, grp_tiles, t, c);
      for (int kb = 0; kb < num_kb; kb++) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word)) goto done;
        if (lane == 0) {
          uint8_t* sa = tiles + stage * F8_STAGE_BYTES;
          mbar_expect_tx(&full_bar[stage], F8_STAGE_BYTES);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * F8_BK, c.row0);
          tma_load_2d(sa + F8_TILE_BYTES, &tmap_b, &full_bar[stage], kb * F8_BK, c.w_row0);
        }
        __syncwarp();
        if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    constexpr uint32_t idesc = make_idesc_e4m3(F8_BM, F8_BN);
    int stage = 0;
    uint32_t phase = 0;
    uint32_t it = 0;          // K blocks issued so far (selects the partial buffer)
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      for (int kb = 0; kb < num_kb; kb++, it++) {
        const int b = it & 1;
        if (!mbar_wait(&part_empty[b], ((it >> 1) & 1u) ^ 1u, abort_word)) goto done;
        if (!mbar_wait(&full_bar[stage], phase, abort_word)) goto done;
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = smem_u32(tiles + stage * F8_STAGE_BYTES);
          const uint32_t sb = sa + F8_TILE_BYTES;
#pragma unroll
          for (int kk = 0; kk < F8_BK / 32; kk++) {       // 32 e4m3 = 32 bytes per MMA
            const uint64_t da = make_smem_desc(sa + kk * 32, 16, 1024, kLayoutSw128);
            const uint64_t db = make_smem_desc(sb + kk * 32, 16, 1024, kLayoutSw128);
            umma_f8_ss(tmem_base + b * F8_BN, da, db, idesc, kk > 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          umma_commit(&part_full[b]);
        }
        __syncwarp();
        if (++stage == F8_STAGES) { stage = 0; phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ promotion + epilogue
    const int q = warp & 3;                              // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;                    // which 64 columns of the tile
    const int kblocks = p.K / F8_BK;                     // columns of the scale matrices
    const int n_blocks = (p.N + F8_BN - 1) / F8_BN;
    uint32_t it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      F8Tile c;
      f8_tile(p, grp_tiles, t, c);
      const int row = c.row0 + q * 32 + lane;
      const bool row_ok = row < c.row_end;
      const bool per_channel = p.row_scale != nullptr;
      const float* as_row = per_channel ? nullptr : p.a_scale + (size_t)(row_ok ? row : 0) * kblocks;
      const float* ws_row = per_channel ? nullptr : p.w_scale + ((size_t)c.group * n_blocks + c.tn) * kblocks;
      float acc[F8_HALF];
#pragma unroll
      for (int i = 0; i < F8_HALF; i++) acc[i] = 0.f;
      float sc_next = per_channel ? 1.f : as_row[0] * ws_row[0];
      for (int kb = 0; kb < num_kb; kb++, it++) {
        const int b = it & 1;
        const float sc = sc_next;
        if (!per_channel && kb + 1 < num_kb) sc_next = as_row[kb + 1] * ws_row[kb + 1];
        if (!mbar_wait(&part_full[b], (it >> 1) & 1u, abort_word)) goto done;
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + b * F8_BN + half * F8_HALF;
        uint32_t r0[32], r1[32];
        tmem_ld_32x32b_x32(t_row, r0);
        tmem_ld_32x32b_x32(t_row + 32, r1);
        tmem_ld_wait();
        // the partial is in registers: the MMA warp may overwrite the buffer
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&part_empty[b]);
#pragma unroll
        for (int i = 0; i < 32; i++) acc[i] = fmaf(__uint_as_float(r0[i]), sc, acc[i]);
#pragma unroll
        for (int i = 0; i < 32; i++) acc[32 + i] = fmaf(__uint_as_float(r1[i]), sc, acc[32 + i]);
      }
      if (row_ok) {
        __nv_bfloat16* crow = p.C + (size_t)row * p.ldc;
        const float rs = per_channel ? p.row_scale[row] : 1.f;
        const float* cs = per_channel ? p.col_scale + (size_t)c.group * p.N : nullptr;
#pragma unroll
        for (int g = 0; g < F8_HALF / 8; g++) {
          const int col = c.tn * F8_BN + half * F8_HALF + g * 8;
          if (col < p.N) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; j++) v[j] = acc[g * 8 + j];
            if (per_channel) {
              const float4 c0 = *reinterpret_cast<const float4*>(cs + col);
              const float4 c1 = *reinterpret_cast<const float4*>(cs + col + 4);
              const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
#pragma unroll
              for (int j = 0; j < 8; j++) v[j] *= rs * cv[j];
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
            *reinterpret_cast<uint4*>(crow + col) =
                make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                           pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
          }
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
    tmem_dealloc(tmem_base, 256);
  }
}

// ---------------------------------------------------------------- host
struct F8Key {
  const void* ptr;
  uint64_t rows, cols, ld;
  bool operator==(const F8Key& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld;
  }
};
struct F8Hash {
  size_t operator()(const F8Key& k) const {
    size_t h = (size_t)k.ptr;
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    return h;
  }
};

// row-major 8-bit [rows, cols] (row stride ld bytes), box 128 rows x 128 bytes, 128B swizzle
static int get_tmap_u8(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                       uint64_t ld) {
  static std::unordered_map<F8Key, CUtensorMap, F8Hash> cache;
  static std::mutex mu;
  F8Key key{ptr, rows, cols, ld};
  std::lock_guard<std::mutex> g(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  uint64_t dims[2] = {cols, rows};
  uint64_t strides[1] = {ld};
  uint32_t box[2] = {128, 128};
  int rc = make_tmap(out, ptr, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, dims, strides, box,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc) return rc;
  if (cache.size() > 8192) cache.clear();
  cache.emplace(key, *out);
  return 0;
}

static int launch_fp8(const void* A, const void* W, Fp8Params& p, int lda, int ldw, long a_rows,
                      long w_rows, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_block_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         F8_SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  CUtensorMap ta, tb;
  int rc = get_tmap_u8(&ta, A, (uint64_t)a_rows, (uint64_t)p.K, (uint64_t)lda);
  if (rc) return rc;
  rc = get_tmap_u8(&tb, W, (uint64_t)w_rows, (uint64_t)p.K, (uint64_t)ldw);
  if (rc) return rc;
  p.tiles_m = (p.M + F8_BM - 1) / F8_BM;
  p.tiles_n = (p.N + F8_BN - 1) / F8_BN;
  p.num_kb = p.K / F8_BK;
  int grid = num_sms();
  if (p.num_groups == 0 && p.tiles_m * p.tiles_n < grid) grid = p.tiles_m * p.tiles_n;
  gemm_fp8_block_kernel<<<grid, F8_THREADS, F8_SMEM_BYTES, stream>>>(ta, tb, p);
  return B200_CHECK_LAUNCH();
}

}  // namespace b200

using namespace b200;

// C[M,N] bf16 = block-scaled product of A8 [M,K] e4m3 (a_scale [M, K/128] fp32) and
// W8 [N,K] e4m3 (w_scale [ceil(N/128), K/128] fp32).  K multiple of 128, N multiple of 8.
B200_API int b200_gemm_fp8_block(const void* A8, const void* a_scale, const void* W8,
                                 const void* w_scale, void* C, const void* bias, int M, int N,
                                 int K, int lda, int ldw, int ldc, int* status,
                                 cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 128) || (N & 7) || (lda & 15) || (ldw & 15) || (ldc & 7)) return 9100;
  Fp8Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.a_scale = (const float*)a_scale;
  p.w_scale = (const float*)w_scale;
  p.C = (__nv_bfloat16*)C;
  p.bias = (const __nv_bfloat16*)bias;
  p.status = status;
  return launch_fp8(A8, W8, p, lda, ldw, M, N, stream);
}

// Grouped variant: rows [offsets[e], offsets[e+1]) of A8 use expert e's W8[e] ([N,K]) and
// w_scale[e] ([ceil(N/128), K/128]).
B200_API int b200_grouped_gemm_fp8_block(const void* A8, const void* a_scale, const void* W8,
                                         const void* w_scale, void* C, const void* offsets,
                                         int num_groups, long total_rows, int N, int K, int lda,
                                         int ldw, int ldc, int* status, cudaStream_t stream) {
  if (total_rows <= 0 || N <= 0 || num_groups <= 0) return 0;
  if ((K % 128) || (N & 7) || (lda & 15) || (ldw & 15) || (ldc & 7)) return 9100;
  if (num_groups > F8_MAX_GROUPS) return 9131;
  Fp8Params p;
  memset(&p, 0, sizeof(p));
  p.M = (int)total_rows; p.N = N; p.K = K; p.ldc = ldc;
  p.a_scale = (const float*)a_scale;
  p.w_scale = (const float*)w_scale;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.group_offsets = (const int*)offsets;
  p.num_groups = num_groups;
  p.w_rows_per_group = N;
  return launch_fp8(A8, W8, p, lda, ldw, total_rows, (long)num_groups * N, stream);
}

// Per-token x per-channel form (dynamic W8A8 in e4m3): C = row_scale[m] * col_scale[n] * (A8 . W8^T).
// row_scale [M] fp32, col_scale [N] fp32 (16-byte aligned, N multiple of 8).
B200_API int b200_gemm_fp8_channel(const void* A8, const void* row_scale, const void* W8,
                                   const void* col_scale, void* C, const void* bias, int M, int N,
                                   int K, int lda, int ldw, int ldc, int* status,
                                   cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if ((K % 128) || (N & 7) || (lda & 15) || (ldw & 15) || (ldc & 7) || ((uintptr_t)col_scale & 15))
    return 9100;
  Fp8Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.row_scale = (const float*)row_scale;
  p.col_scale = (const float*)col_scale;
  p.C = (__nv_bfloat16*)C;
  p.bias = (const __nv_bfloat16*)bias;
  p.status = status;
  return launch_fp8(A8, W8, p, lda, ldw, M, N, stream);
}

// Grouped per-channel form: expert e's W8[e] [N,K] with col_scale[e] [N].
B200_API int b200_grouped_gemm_fp8_channel(const void* A8, const void* row_scale, const void* W8,
                                           const void* col_scale, void* C, const void* offsets,
                                           int num_groups, long total_rows, int N, int K, int lda,
                                           int ldw, int ldc, int* status, cudaStream_t stream) {
  if (total_rows <= 0 || N <= 0 || num_groups <= 0) return 0;
  if ((K % 128) || (N & 7) || (lda & 15) || (ldw & 15) || (ldc & 7) || ((uintptr_t)col_scale & 15))
    return 9100;
  if (num_groups > F8_MAX_GROUPS) return 9131;
  Fp8Params p;
  memset(&p, 0, sizeof(p));
  p.M = (int)total_rows; p.N = N; p.K = K; p.ldc = ldc;
  p.row_scale = (const float*)row_scale;
  p.col_scale = (const float*)col_scale;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.group_offsets = (const int*)offsets;
  p.num_groups = num_groups;
  p.w_rows_per_group = N;
  return launch_fp8(A8, W8, p, lda, ldw, total_rows, (long)num_groups * N, stream);
}
