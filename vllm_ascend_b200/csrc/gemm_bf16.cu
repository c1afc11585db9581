// bf16 GEMM for sm_100a:  C[M,N] = A[M,K] * W[N,K]^T (+ bias[N]) (+ residual[M,N])
//
// Both operands are K-major (row-major activations, nn.Linear weights), which
// is the layout every linear layer of the decoder uses (parity with the
// reference's unquantized GEMM custom op, vllm_ascend/ops/linear.py:53-110).
//
// Structure: persistent CTAs (one per SM), warp-specialised:
//   warp 0      TMA producer: 128x64 A tile + BNx64 W tile per stage, 128B swizzle
//   warp 1      MMA issuer: tcgen05.mma cta_group::1, M=128, N=BN, K=16, f32 accum in TMEM
//   warps 2..5  epilogue: tcgen05.ld 32x32b -> bf16 -> 16-byte global stores
// Two TMEM accumulator buffers let the epilogue of tile i overlap the main
// loop of tile i+1.  All waits are bounded (see common.cuh).
#include "common.cuh"

#include <mutex>
#include <unordered_map>

namespace b200 {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;

template <int BN>
struct GemmCfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = GEMM_BM * GEMM_BK * 2;
  static constexpr int kBBytes = BN * GEMM_BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;  // 256 or 512 (power of two)
  // tiles + barriers + tmem pointer + abort word, plus 1 KB alignment slack
  static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

struct GemmParams {
  int M, N, K;
  int ldc;             // row stride of C (elements)
  const __nv_bfloat16* bias;      // [N] or null
  const __nv_bfloat16* residual;  // [M, ldc] or null
  __nv_bfloat16* C;
  int* status;         // device status word (may be null)
  int tiles_m, tiles_n;
};

template <int BN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, GemmParams p) {
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

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_kb = (p.K + GEMM_BK - 1) / GEMM_BK;
  const int num_tiles = p.tiles_m * p.tiles_n;

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

  // Tile order: consecutive CTAs take consecutive M tiles of the same N tile so
  // the W tile is shared through L2.
  if (warp == 0) {
    // ------------------------------------------------------------ producer
    int stage = 0;
    uint32_t phase = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      for (int kb = 0; kb < num_kb; kb++) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_word)) goto done;
        if (lane == 0) {
          uint8_t* sa = tiles + stage * Cfg::kStageBytes;
          uint8_t* sb = sa + Cfg::kABytes;
          mbar_expect_tx(&full_bar[stage], Cfg::kStageBytes);
          tma_load_2d(sa, &tmap_a, &full_bar[stage], kb * GEMM_BK, tm * GEMM_BM);
          tma_load_2d(sb, &tmap_b, &full_bar[stage], kb * GEMM_BK, tn * BN);
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
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, it++) {
      const int tm = t % p.tiles_m, tn = t / p.tiles_m;
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_word)) goto done;
      tc_fence_after();
      const int row = tm * GEMM_BM + q * 32 + lane;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      __nv_bfloat16* crow = p.C + (size_t)row * p.ldc;
      const __nv_bfloat16* rrow = p.residual ? p.residual + (size_t)row * p.ldc : nullptr;
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += 32) {
        const int col0 = tn * BN + c0;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c0, r);
        tmem_ld_wait();
        if (row < p.M) {
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
              *reinterpret_cast<uint4*>(crow + col) = o;
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }
done:
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_word != 0 && p.status) atomicExch(p.status, *abort_word);
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
static int launch_gemm(const void* A, const void* W, void* C, const void* bias,
                       const void* residual, int M, int N, int K, int lda, int ldw, int ldc,
                       int* status, int max_ctas, cudaStream_t stream) {
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
  int rc = get_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, GEMM_BM);
  if (rc) return rc;
  rc = get_tmap_2d_bf16(&tb, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, BN);
  if (rc) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.bias = (const __nv_bfloat16*)bias;
  p.residual = (const __nv_bfloat16*)residual;
  p.C = (__nv_bfloat16*)C;
  p.status = status;
  p.tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (N + BN - 1) / BN;
  int grid = p.tiles_m * p.tiles_n;
  int sms = num_sms();
  if (max_ctas > 0 && max_ctas < sms) sms = max_ctas;
  if (grid > sms) grid = sms;
  gemm_bf16_kernel<BN><<<grid, GEMM_THREADS, Cfg::kSmemBytes, stream>>>(ta, tb, p);
  return B200_CHECK_LAUNCH();
}

}  // namespace b200

// C[M,N] (row stride ldc) = A[M,K] (row stride lda) * W[N,K]^T (row stride ldw)
// (+bias[N]) (+residual[M,N] with row stride ldc).  Requirements: K, N, lda,
// ldw, ldc multiples of 8; all base pointers 16-byte aligned.  bn selects the
// N tile (128 or 256; 0 = choose).  Returns 0 or a CUDA / encode error code.
B200_API int b200_gemm_bf16(const void* A, const void* W, void* C, const void* bias,
                            const void* residual, int M, int N, int K, int lda, int ldw,
                            int ldc, int bn, int* status, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((K & 7) || (N & 7) || (lda & 7) || (ldw & 7) || (ldc & 7)) return 9100;
  if (bn == 0) {
    // 256-wide tiles halve A re-reads; use them when they still fill the GPU.
    const long tiles256 = (long)((M + 127) / 128) * ((N + 255) / 256);
    bn = (N >= 256 && tiles256 >= b200::num_sms()) ? 256 : 128;
    if (N % 256 != 0 && N % 128 == 0) bn = 128;
  }
  if (bn == 256)
    return b200::launch_gemm<256>(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, status,
                                  max_ctas, stream);
  return b200::launch_gemm<128>(A, W, C, bias, residual, M, N, K, lda, ldw, ldc, status,
                                max_ctas, stream);
}
