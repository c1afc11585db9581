// Fused expert-parallel MoE over peer memory: token dispatch and result combine without a
// collective library call and without a host round trip.
//
//   moe_dispatch_kernel   histogram of this rank's routing -> every peer (peer stores + flag);
//                         wait for all histograms; every rank derives the same packed layout
//                         [expert-major, source-rank-major] of each owner's receive pool and
//                         stores its token rows (+ origin tag) straight into the owners' pools.
//   grouped GEMM1+SwiGLU  (gemm_bf16.cu, WAITFLAGS) starts when every source's rows have landed.
//   grouped GEMM2         (gemm_bf16.cu, SCATTER) stores each output row into the token
//                         owner's combine buffer from the epilogue, then flags the owners.
//   moe_reduce_kernel     waits for every expert owner, out[t] = sum_k w[t,k] * comb[t,k].
//
// Counterpart of the reference's dispatch_ffn_combine kernel
// (csrc/mc2/dispatch_ffn_combine/op_kernel/dispatch_ffn_combine_kernel.hpp:842-1022: count
// all-gather, per-expert pull, GMM1/SwiGLU/GMM2, write-back into the owner's peer buffer,
// weighted unpermute).  Every wait is bounded and reports B200_TIMEOUT instead of hanging.
#include "comm.cuh"
#include <cuda_bf16.h>

namespace b200 {

constexpr int kMoeMaxExperts = 512;

struct MoeDispatchParams {
  const __nv_bfloat16* x;      // [T, H]
  long x_stride;
  const int* topk_ids;         // [T, topk] global (physical) expert ids, < 0 = no expert
  int T, topk, H, E, E_local, my_rank, num_ranks;
  int* hist;                   // local [num_ranks][E], row s written by rank s
  int* peer_hist[kMaxRanks];
  __nv_bfloat16* peer_recv_x[kMaxRanks];
  int* peer_recv_meta[kMaxRanks];
  MoeCtl* peer_ctl[kMaxRanks];
  int* cursor;                 // local [E], zero on entry, zeroed again on exit
  int* group_offsets;          // local out [E_local + 1]
  long pool_rows;
  int* status;
};

__global__ void __launch_bounds__(256)
moe_dispatch_kernel(const MoeDispatchParams p) {
  __shared__ int s_a[kMoeMaxExperts];     // block 0: my histogram; then: base row of expert e
  __shared__ int s_abort, s_last;
  MoeCtl* ctl = p.peer_ctl[p.my_rank];
  const uint32_t epoch = *((volatile uint32_t*)&ctl->epoch) + 1;
  const int tid = threadIdx.x;
  const int npairs = p.T * p.topk;
  if (tid == 0) { s_abort = 0; s_last = 0; }

  if (blockIdx.x == 0) {
    for (int e = tid; e < p.E; e += blockDim.x) s_a[e] = 0;
    __syncthreads();
    for (int i = tid; i < npairs; i += blockDim.x) {
      const int e = p.topk_ids[i];
      if (e >= 0 && e < p.E) atomicAdd(&s_a[e], 1);
      else if (e >= p.E && p.status) atomicExch(p.status, B200_BAD_INDEX);
    }
    __syncthreads();
    for (int o = 0; o < p.num_ranks; o++)
      for (int e = tid; e < p.E; e += blockDim.x)
        p.peer_hist[o][(long)p.my_rank * p.E + e] = s_a[e];
    __threadfence_system();
    __syncthreads();
    if (tid < p.num_ranks) st_release_sys(&p.peer_ctl[tid]->hist_flag[p.my_rank], epoch);
  }
  __syncthreads();
  if (tid < p.num_ranks) {
    if (!wait_flag_ge(&ctl->hist_flag[tid], epoch, p.status)) s_abort = 1;
  }
  __syncthreads();
  if (s_abort) return;

  // packed layout of owner d's pool: experts of d in order, inside an expert the source ranks
  // in order.  base(e) = rows before my rows of expert e in its owner's pool.
  for (int e = tid; e < p.E; e += blockDim.x) {
    const int first = (e / p.E_local) * p.E_local;
    int base = 0;
    for (int e2 = first; e2 < e; e2++)
      for (int s = 0; s < p.num_ranks; s++) base += __ldcg(&p.hist[(long)s * p.E + e2]);
    for (int s = 0; s < p.my_rank; s++) base += __ldcg(&p.hist[(long)s * p.E + e]);
    s_a[e] = base;
  }
  if (blockIdx.x == 0 && tid == 0) {
    int acc = 0;
    const int first = p.my_rank * p.E_local;
    for (int j = 0; j < p.E_local; j++) {
      p.group_offsets[j] = acc;
      for (int s = 0; s < p.num_ranks; s++) acc += __ldcg(&p.hist[(long)s * p.E + first + j]);
    }
    if (acc > p.pool_rows) {       // cannot happen while every rank sends <= capacity tokens
      if (p.status) atomicExch(p.status, B200_OVERFLOW);
      acc = (int)p.pool_rows;
    }
    p.group_offsets[p.E_local] = acc;
  }
  __syncthreads();

  const int warp = tid >> 5, lane = tid & 31;
  const int warps_total = gridDim.x * (blockDim.x >> 5);
  const int vec_per_row = p.H >> 3;
  for (int i = blockIdx.x * (blockDim.x >> 5) + warp; i < npairs; i += warps_total) {
    const int e = p.topk_ids[i];
    if (e < 0 || e >= p.E) continue;
    int pos = 0;
    if (lane == 0) pos = s_a[e] + atomicAdd(&p.cursor[e], 1);
    pos = __shfl_sync(0xffffffffu, pos, 0);
    if (pos >= p.pool_rows) {
      if (lane == 0 && p.status) atomicExch(p.status, B200_OVERFLOW);
      continue;
    }
    const int d = e / p.E_local;
    const uint4* src = reinterpret_cast<const uint4*>(p.x + (long)(i / p.topk) * p.x_stride);
    uint4* dst = reinterpret_cast<uint4*>(p.peer_recv_x[d] + (long)pos * p.H);
    for (int v = lane; v < vec_per_row; v += 32) dst[v] = src[v];
    if (lane == 0) p.peer_recv_meta[d][pos] = (p.my_rank << 24) | i;
  }
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const uint32_t prev = atomicAdd(&ctl->done_ctr, 1u);
    s_last = (prev == gridDim.x - 1);
  }
  __syncthreads();
  if (s_last) {
    for (int e = tid; e < p.E; e += blockDim.x) p.cursor[e] = 0;
    __threadfence_system();
    __syncthreads();
    if (tid < p.num_ranks) st_release_sys(&p.peer_ctl[tid]->disp_flag[p.my_rank], epoch);
    if (tid == 0) { ctl->done_ctr = 0; __threadfence(); }
  }
}

struct MoeReduceParams {
  const __nv_bfloat16* comb;   // local [T * topk, H], written by the expert owners
  const float* topk_w;         // [T, topk]
  const int* topk_ids;         // [T, topk]
  __nv_bfloat16* out;          // [T, H]
  long out_stride;
  int T, topk, H, num_ranks;
  MoeCtl* ctl;
  int* status;
};

__global__ void __launch_bounds__(256)
moe_reduce_kernel(const MoeReduceParams p) {
  __shared__ int s_abort;
  const int tid = threadIdx.x;
  const uint32_t epoch = *((volatile uint32_t*)&p.ctl->epoch) + 1;
  if (tid == 0) s_abort = 0;
  __syncthreads();
  if (tid < p.num_ranks) {
    if (!wait_flag_ge(&p.ctl->comb_flag[tid], epoch, p.status)) s_abort = 1;
  }
  __syncthreads();
  if (!s_abort) {
    const int vec_per_row = p.H >> 3;
    for (int t = blockIdx.x; t < p.T; t += gridDim.x) {
      for (int v = tid; v < vec_per_row; v += blockDim.x) {
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; j++) acc[j] = 0.f;
        for (int k = 0; k < p.topk; k++) {
          if (p.topk_ids[t * p.topk + k] < 0) continue;
          const float w = p.topk_w[t * p.topk + k];
          const uint4 r = __ldcg(reinterpret_cast<const uint4*>(p.comb + (long)(t * p.topk + k) * p.H) + v);
          const uint32_t rw[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float2 f = unpack_bf16x2(rw[j]);
            acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
            acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
          }
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        reinterpret_cast<uint4*>(p.out + (long)t * p.out_stride)[v] = o;
      }
    }
  }
  __syncthreads();
  // the call is over on this rank (also after a timeout, so the epochs stay aligned)
  if (tid == 0) {
    const uint32_t prev = atomicAdd(&p.ctl->done_ctr3, 1u);
    if (prev == gridDim.x - 1) {
      p.ctl->epoch = epoch;
      p.ctl->done_ctr3 = 0;
      __threadfence();
    }
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_moe_ctl_bytes() { return (int)sizeof(MoeCtl); }

// peer_* : host arrays of num_ranks device pointers (peer-mapped); hist/cursor/group_offsets local.
B200_API int b200_moe_dispatch(const void* x, long x_stride, const void* topk_ids, int T, int topk,
                               int H, int E, int E_local, int my_rank, int num_ranks,
                               void* const* peer_hist, void* const* peer_recv_x,
                               void* const* peer_recv_meta, void* const* peer_ctl, void* cursor,
                               void* group_offsets, long pool_rows, int* status,
                               cudaStream_t stream) {
  if (E > kMoeMaxExperts || num_ranks > kMaxRanks || (H & 7) || E_local * num_ranks != E) return 9400;
  if ((long)T * topk >= (1 << 24)) return 9401;
  MoeDispatchParams p;
  p.x = (const __nv_bfloat16*)x; p.x_stride = x_stride; p.topk_ids = (const int*)topk_ids;
  p.T = T; p.topk = topk; p.H = H; p.E = E; p.E_local = E_local;
  p.my_rank = my_rank; p.num_ranks = num_ranks;
  for (int o = 0; o < num_ranks; o++) {
    p.peer_hist[o] = (int*)peer_hist[o];
    p.peer_recv_x[o] = (__nv_bfloat16*)peer_recv_x[o];
    p.peer_recv_meta[o] = (int*)peer_recv_meta[o];
    p.peer_ctl[o] = (MoeCtl*)peer_ctl[o];
  }
  p.hist = (int*)peer_hist[my_rank];
  p.cursor = (int*)cursor;
  p.group_offsets = (int*)group_offsets;
  p.pool_rows = pool_rows;
  p.status = status;
  // every block must be resident at once: block 0 publishes what the others wait for
  int grid = (T * topk + 7) / 8;
  if (grid < 1) grid = 1;
  if (grid > num_sms()) grid = num_sms();
  moe_dispatch_kernel<<<grid, 256, 0, stream>>>(p);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_moe_reduce(const void* comb, const void* topk_w, const void* topk_ids, void* out,
                             long out_stride, int T, int topk, int H, int num_ranks, void* moe_ctl,
                             int* status, cudaStream_t stream) {
  if ((H & 7) || num_ranks > kMaxRanks) return 9400;
  MoeReduceParams p;
  p.comb = (const __nv_bfloat16*)comb; p.topk_w = (const float*)topk_w;
  p.topk_ids = (const int*)topk_ids; p.out = (__nv_bfloat16*)out; p.out_stride = out_stride;
  p.T = T; p.topk = topk; p.H = H; p.num_ranks = num_ranks;
  p.ctl = (MoeCtl*)moe_ctl; p.status = status;
  int grid = T < 1 ? 1 : (T > 4 * num_sms() ? 4 * num_sms() : T);
  moe_reduce_kernel<<<grid, 256, 0, stream>>>(p);
  return B200_CHECK_LAUNCH();
}
