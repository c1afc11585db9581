// MoE routing and token movement kernels.
//   * gating top-k: softmax / sigmoid scores, correction bias, group-limited selection,
//     renormalisation and scaling in one warp-per-token kernel (the reference's
//     moe_gating_top_k op, csrc/moe/moe_gating_top_k; signature torch_binding.cpp:2135-2150)
//   * permute: histogram of tokens per local expert, exclusive offsets, and the gather of
//     token rows into expert-major order (npu_moe_init_routing_v2 / npu_moe_token_permute)
//   * combine: weighted sum of the k expert outputs of every token (npu_moe_token_unpermute)
// The grouped GEMMs in between are csrc/gemm_bf16.cu (GROUPED mode) and
// csrc/gemm_fp8_block.cu.
#include "common.cuh"

namespace b200 {

constexpr int GATE_MAX_PER_LANE = 16;   // experts <= 512

// logits [T, E] fp32 -> weights [T, k] fp32, ids [T, k] int32
// scoring: 0 softmax, 1 sigmoid.  Group-limited: experts are split into n_group groups, the
// topk_group groups with the best group score stay eligible (group score = max, or the sum
// of the top two when a correction bias is given).  Selection uses score + bias, the
// returned weight is the unbiased score.
__global__ void moe_gating_topk_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                       float* __restrict__ weights, int* __restrict__ ids, int T,
                                       int E, int k, int scoring, int renorm, int n_group,
                                       int topk_group, float scale) {
  const int warps = blockDim.x >> 5;
  const int t = blockIdx.x * warps + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  const int per = (E + 31) / 32;
  float score[GATE_MAX_PER_LANE], choice[GATE_MAX_PER_LANE];
  const float* row = logits + (size_t)t * E;
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < GATE_MAX_PER_LANE; i++) {
    const int e = lane + 32 * i;
    score[i] = (i < per && e < E) ? row[e] : -INFINITY;
    mx = fmaxf(mx, score[i]);
  }
  if (scoring == 0) {
    mx = warp_reduce_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < GATE_MAX_PER_LANE; i++) {
      const int e = lane + 32 * i;
      score[i] = (i < per && e < E) ? __expf(score[i] - mx) : 0.f;
      sum += score[i];
    }
    sum = warp_reduce_sum(sum);
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < GATE_MAX_PER_LANE; i++) score[i] *= inv;
  } else {
#pragma unroll
    for (int i = 0; i < GATE_MAX_PER_LANE; i++) {
      const int e = lane + 32 * i;
      score[i] = (i < per && e < E) ? 1.f / (1.f + __expf(-score[i])) : 0.f;
    }
  }
#pragma unroll
  for (int i = 0; i < GATE_MAX_PER_LANE; i++) {
    const int e = lane + 32 * i;
    choice[i] = (i < per && e < E) ? score[i] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  if (n_group > 1) {
    // group scores; every lane ends up with the eligibility of all groups (n_group <= 32)
    const int gsz = E / n_group;
    float my_gscore = -INFINITY;                 // lane g holds the score of group g
    for (int g = 0; g < n_group; g++) {
      float b1 = -INFINITY, b2 = -INFINITY;      // best two inside the group among my experts
#pragma unroll
      for (int i = 0; i < GATE_MAX_PER_LANE; i++) {
        const int e = lane + 32 * i;
        if (i < per && e < E && e / gsz == g) {
          const float v = choice[i];
          if (v > b1) { b2 = b1; b1 = v; } else if (v > b2) { b2 = v; }
        }
      }
      // merge the per-lane (best, second) pairs across the warp
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float o1 = __shfl_xor_sync(0xffffffffu, b1, o);
        const float o2 = __shfl_xor_sync(0xffffffffu, b2, o);
        const float n1 = fmaxf(b1, o1);
        const float n2 = fmaxf(fminf(b1, o1), fmaxf(b2, o2));
        b1 = n1;
        b2 = n2;
      }
      const float gs = bias ? (b1 + b2) : b1;
      if (lane == g) my_gscore = gs;
    }
    // pick topk_group groups
    unsigned keep = 0;
    for (int r = 0; r < topk_group; r++) {
      float v = my_gscore;
      int idx = lane;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
      }
      keep |= 1u << idx;
      if (lane == idx) my_gscore = -INFINITY;
    }
#pragma unroll
    for (int i = 0; i < GATE_MAX_PER_LANE; i++) {
      const int e = lane + 32 * i;
      if (i < per && e < E && !((keep >> (e / gsz)) & 1u)) choice[i] = -INFINITY;
    }
  }
  // iterative top-k (lowest index wins ties)
  float wsum = 0.f;
  float my_w = 0.f;
  int my_id = 0;
  for (int r = 0; r < k; r++) {
    float v = -INFINITY;
    int idx = 0x7fffffff;
    float sc = 0.f;
#pragma unroll
    for (int i = 0; i < GATE_MAX_PER_LANE; i++) {
      const int e = lane + 32 * i;
      if (i < per && e < E && (choice[i] > v || (choice[i] == v && e < idx))) {
        v = choice[i]; idx = e; sc = score[i];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      const float os = __shfl_xor_sync(0xffffffffu, sc, o);
      if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; sc = os; }
    }
    if ((idx & 31) == lane) {
#pragma unroll
      for (int i = 0; i < GATE_MAX_PER_LANE; i++)
        if (lane + 32 * i == idx) choice[i] = -INFINITY;
    }
    wsum += sc;
    if (lane == r) { my_w = sc; my_id = idx; }
  }
  if (lane < k) {
    float w = my_w;
    if (renorm) w /= fmaxf(wsum, 1e-20f);
    weights[(size_t)t * k + lane] = w * scale;
    ids[(size_t)t * k + lane] = my_id;
  }
}

// ---------------------------------------------------------------- permute
// local_ids [T*k] int32 (expert on this rank, or -1).  counts/cursor [E] zeroed by the caller.
__global__ void moe_count_kernel(const int* __restrict__ local_ids, int n, int E, int* counts) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int e = local_ids[i];
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
}
// offsets[E+1] = exclusive prefix sum of counts (single block)
__global__ void moe_scan_kernel(const int* __restrict__ counts, int E, int* offsets) {
  __shared__ int s[1024];
  const int t = threadIdx.x;
  int v = t < E ? counts[t] : 0;
  s[t] = v;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int add = t >= o ? s[t - o] : 0;
    __syncthreads();
    s[t] += add;
    __syncthreads();
  }
  if (t < E) offsets[t + 1] = s[t];
  if (t == 0) offsets[0] = 0;
}
// pos[i] = destination row of pair i (or -1); src_token[row] = token of that row
__global__ void moe_assign_kernel(const int* __restrict__ local_ids, int n, int k, int E,
                                  const int* __restrict__ offsets, int* cursor, int* pos,
                                  int* src_token) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int e = local_ids[i];
  if (e < 0 || e >= E) {
    pos[i] = -1;
    return;
  }
  const int r = offsets[e] + atomicAdd(&cursor[e], 1);
  pos[i] = r;
  src_token[r] = i / k;
}
// out[row] = x[src_token[row]] for row < offsets[E]
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                       const int* __restrict__ src_token,
                                       const int* __restrict__ offsets, int E, int H,
                                       __nv_bfloat16* __restrict__ out) {
  const int row = blockIdx.x;
  if (row >= offsets[E]) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)src_token[row] * H);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * H);
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) dst[v] = src[v];
}
// out[t] = sum_s w[t,s] * y[pos[t,s]]
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                                   const float* __restrict__ w, int k, int H,
                                   __nv_bfloat16* __restrict__ out, int accumulate) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < (H >> 3); v += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (accumulate) {
      const uint4 o = reinterpret_cast<const uint4*>(out + (size_t)t * H)[v];
      const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 f = unpack_bf16x2(ow[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    }
    for (int s = 0; s < k; s++) {
      const int r = pos[t * k + s];
      if (r < 0) continue;
      const float ws = w[t * k + s];
      const uint4 a = reinterpret_cast<const uint4*>(y + (size_t)r * H)[v];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float2 f = unpack_bf16x2(aw[j]);
        acc[2 * j] += ws * f.x;
        acc[2 * j + 1] += ws * f.y;
      }
    }
    reinterpret_cast<uint4*>(out + (size_t)t * H)[v] =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                   pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_moe_gating_topk(const void* logits, const void* bias, void* weights, void* ids,
                                  int T, int E, int k, int scoring, int renorm, int n_group,
                                  int topk_group, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (E > 32 * GATE_MAX_PER_LANE || k > 32 || k > E) return 9150;
  if (n_group > 1 && (n_group > 32 || E % n_group || topk_group > n_group)) return 9151;
  const int wpb = 4;
  moe_gating_topk_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, stream>>>(
      (const float*)logits, (const float*)bias, (float*)weights, (int*)ids, T, E, k, scoring,
      renorm, n_group, topk_group, scale);
  return B200_CHECK_LAUNCH();
}

// Builds expert-major order for the (token, slot) pairs whose expert lives on this rank.
// workspace ints: counts[E] | cursor[E] | offsets[E+1]; all written here.
B200_API int b200_moe_permute(const void* local_ids, int T, int k, int E, void* counts,
                              void* cursor, void* offsets, void* pos, void* src_token,
                              cudaStream_t stream) {
  if (E > 1024) return 9152;
  const int n = T * k;
  cudaMemsetAsync(counts, 0, sizeof(int) * E, stream);
  cudaMemsetAsync(cursor, 0, sizeof(int) * E, stream);
  if (n > 0) {
    moe_count_kernel<<<(n + 255) / 256, 256, 0, stream>>>((const int*)local_ids, n, E, (int*)counts);
  }
  moe_scan_kernel<<<1, 1024, 0, stream>>>((const int*)counts, E, (int*)offsets);
  if (n > 0) {
    moe_assign_kernel<<<(n + 255) / 256, 256, 0, stream>>>((const int*)local_ids, n, k, E,
                                                           (const int*)offsets, (int*)cursor,
                                                           (int*)pos, (int*)src_token);
  }
  return B200_CHECK_LAUNCH();
}

B200_API int b200_moe_gather_rows(const void* x, const void* src_token, const void* offsets, int E,
                                  int H, int max_rows, void* out, cudaStream_t stream) {
  if (max_rows <= 0) return 0;
  if (H & 7) return 9100;
  moe_gather_rows_kernel<<<max_rows, 128, 0, stream>>>((const __nv_bfloat16*)x,
                                                       (const int*)src_token,
                                                       (const int*)offsets, E, H,
                                                       (__nv_bfloat16*)out);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_moe_combine(const void* y, const void* pos, const void* w, int T, int k, int H,
                              void* out, int accumulate, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H & 7) return 9100;
  moe_combine_kernel<<<T, 128, 0, stream>>>((const __nv_bfloat16*)y, (const int*)pos,
                                            (const float*)w, k, H, (__nv_bfloat16*)out, accumulate);
  return B200_CHECK_LAUNCH();
}
