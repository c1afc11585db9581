// Peer-memory communication kernels for tensor parallelism over NVLink/NVSwitch.
//
//   * symmetric buffers: cudaMalloc + CUDA IPC handles, mapped by every peer
//   * barrier / one-shot all-reduce for small messages (decode-sized activations)
//   * reduce + residual-add + RMSNorm + all-gather push: the consumer of a
//     GEMM->reduce-scatter and the producer of the next all-gather->GEMM in ONE
//     kernel: it sums the bf16 partial rows that the peers' GEMM epilogues stored
//     into this rank's staging buffer, adds the (sequence-sharded) residual,
//     normalises, and stores the normalised rows into every peer's gather buffer.
//
// Replaces the reference's TP collectives around row/column-parallel linears
// (vllm_ascend/ops/linear_op.py:152-191; npu_mm_reduce_scatter_base,
// vllm_ascend/device/device_op.py:164-190).  Every wait is bounded.
#include "comm.cuh"

namespace b200 {

// ---------------------------------------------------------------- barrier
__global__ void barrier_kernel(CommCtl* ctl, uint32_t* const* peer_bar_flags, int my_rank,
                               int num_ranks) {
  // peer_bar_flags[o] = &ctl(o)->bar_flag[my_rank]
  const uint32_t epoch = ctl->bar_epoch + 1;
  if (threadIdx.x < num_ranks) {
    __threadfence_system();
    st_release_sys(peer_bar_flags[threadIdx.x], epoch);
    wait_flag_ge(&ctl->bar_flag[threadIdx.x], epoch, &ctl->status);
  }
  __syncthreads();
  if (threadIdx.x == 0) ctl->bar_epoch = epoch;
}

struct PeerPtrs {
  void* p[kMaxRanks];
};
struct PeerFlags {
  uint32_t* p[kMaxRanks];
};

// ---------------------------------------------------------------- one-shot all-reduce
// Every rank has copied its input into its own symmetric buffer `bufs.p[my_rank]`.
// After a barrier each rank sums all peers' buffers (fixed rank order, so every
// rank gets bit-identical results) into `out`.
__global__ void allreduce_oneshot_kernel(PeerPtrs bufs, PeerFlags bar_flags, CommCtl* ctl,
                                         __nv_bfloat16* out, long n_vec8, int my_rank,
                                         int num_ranks) {
  __shared__ uint32_t s_epoch;
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    s_epoch = ctl->bar_epoch + 1;
    s_ok = 1;
  }
  __syncthreads();
  const uint32_t epoch = s_epoch;
  // one CTA publishes; every CTA waits on the local flags
  if (blockIdx.x == 0 && threadIdx.x < num_ranks) {
    __threadfence_system();
    st_release_sys(bar_flags.p[threadIdx.x], epoch);
  }
  if (threadIdx.x < num_ranks) {
    if (!wait_flag_ge(&ctl->bar_flag[threadIdx.x], epoch, &ctl->status)) s_ok = 0;
  }
  __syncthreads();
  if (s_ok) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n_vec8;
         i += (long)gridDim.x * blockDim.x) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < num_ranks; r++) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(bufs.p[r]) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const float2 f = unpack_bf16x2(w[j]);
          acc[2 * j] += f.x;
          acc[2 * j + 1] += f.y;
        }
      }
      reinterpret_cast<uint4*>(out)[i] =
          make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                     pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
  }
  // the epoch advances once per launch; the last CTA to finish records it, and a
  // second barrier phase keeps a fast rank from overwriting its buffer while a slow
  // peer is still reading it
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(&ctl->done_ctr2, 1u);
    if (prev == gridDim.x - 1) {
      ctl->done_ctr2 = 0;
      const uint32_t e2 = epoch + 1;
      __threadfence_system();
      for (int r = 0; r < num_ranks; r++) st_release_sys(bar_flags.p[r], e2);
      for (int r = 0; r < num_ranks; r++) wait_flag_ge(&ctl->bar_flag[r], e2, &ctl->status);
      ctl->bar_epoch = e2;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------- reduce + add + norm + push
// CTAs walk the local rows (rows_local rows of H columns) with a grid stride: the peers' flags are
// checked, and the system-scope fence after the remote stores is paid, once per CTA instead of once
// per row.
//   staging : [num_src][rows_local][H] bf16 partial sums written by the peers' GEMM
//             epilogues (num_src = 0: no reduction, `x_local` is the input instead)
//   residual: [rows_local][H] bf16, updated in place (may be null when num_src == 0
//             and the input itself is the residual)
//   ag_dst  : peer gather buffers, this rank's rows land at row my_rank*rows_local + i
// NVSwitch multicast accesses (address = multicast mapping of a symmetric buffer)
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc)
      : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_b128(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

template <int VEC_PER_THREAD>
__global__ void reduce_add_norm_push_kernel(const __nv_bfloat16* staging, int num_src,
                                            const __nv_bfloat16* x_local,
                                            __nv_bfloat16* residual,
                                            const __nv_bfloat16* __restrict__ weight, float eps,
                                            PeerPtrs ag_dst, PeerFlags ag_flag_dst, CommCtl* ctl,
                                            int rows_local, int H, int my_rank, int num_ranks,
                                            int skip_norm, __nv_bfloat16* mc_gather) {
  __shared__ float red[32];
  __shared__ int s_ok;
  const int nvec = H >> 3;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (num_src > 0) {
    const uint32_t epoch = ctl->rs_epoch;      // published by this rank's own GEMM-RS launch
    if (threadIdx.x < num_ranks && threadIdx.x != my_rank) {
      if (!wait_flag_ge(&ctl->rs_flag[threadIdx.x], epoch, &ctl->status)) s_ok = 0;
    }
    __syncthreads();
  }
  float vals[VEC_PER_THREAD][8];
  if (s_ok) {
   for (int row = blockIdx.x; row < rows_local; row += gridDim.x) {
    float ss = 0.f;
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; i++) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (num_src > 0) {
          for (int s = 0; s < num_src; s++) {
            const uint4 pv = __ldcg(reinterpret_cast<const uint4*>(
                                        staging + ((size_t)s * rows_local + row) * H) + v);
            const uint32_t w[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const float2 f = unpack_bf16x2(w[j]);
              acc[2 * j] += f.x;
              acc[2 * j + 1] += f.y;
            }
          }
        } else {
          const uint4 pv = reinterpret_cast<const uint4*>(x_local + (size_t)row * H)[v];
          const uint32_t w[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float2 f = unpack_bf16x2(w[j]);
            acc[2 * j] = f.x;
            acc[2 * j + 1] = f.y;
          }
        }
        uint32_t zw[4];
        if (residual && num_src > 0) {
          // the reduced GEMM output is rounded to bf16 before the residual add, as the
          // unfused all-reduce -> add sequence does
          uint4* rr = reinterpret_cast<uint4*>(residual + (size_t)row * H) + v;
          const uint4 rv = *rr;
          const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float2 f = unpack_bf16x2(rw[j]);
            const float2 g = unpack_bf16x2(pack_bf16x2(acc[2 * j], acc[2 * j + 1]));
            zw[j] = pack_bf16x2(g.x + f.x, g.y + f.y);
          }
          *rr = make_uint4(zw[0], zw[1], zw[2], zw[3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; j++) zw[j] = pack_bf16x2(acc[2 * j], acc[2 * j + 1]);
          if (residual)
            reinterpret_cast<uint4*>(residual + (size_t)row * H)[v] =
                make_uint4(zw[0], zw[1], zw[2], zw[3]);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
          const float2 f = unpack_bf16x2(zw[j]);
          vals[i][2 * j] = f.x;
          vals[i][2 * j + 1] = f.y;
          ss += f.x * f.x + f.y * f.y;
        }
      }
    }
    ss = warp_reduce_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
      t = warp_reduce_sum(t);
      if (threadIdx.x == 0) red[0] = skip_norm ? 1.f : rsqrtf(t / (float)H + eps);
    }
    __syncthreads();
    const float inv = red[0];
    const size_t dst_row = (size_t)my_rank * rows_local + row;
#pragma unroll
    for (int i = 0; i < VEC_PER_THREAD; i++) {
      const int v = threadIdx.x + i * blockDim.x;
      if (v < nvec) {
        uint32_t o[4];
        if (skip_norm) {
#pragma unroll
          for (int j = 0; j < 4; j++) o[j] = pack_bf16x2(vals[i][2 * j], vals[i][2 * j + 1]);
        } else {
          const uint4 ww = reinterpret_cast<const uint4*>(weight)[v];
          const uint32_t w4[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float2 fw = unpack_bf16x2(w4[j]);
            o[j] = pack_bf16x2(vals[i][2 * j] * inv * fw.x, vals[i][2 * j + 1] * inv * fw.y);
          }
        }
        const uint4 ov = make_uint4(o[0], o[1], o[2], o[3]);
        if (mc_gather) {
          // one store leaves this GPU; the switch replicates it into every rank's gather buffer
          multimem_st_b128(mc_gather + dst_row * H + (size_t)v * 8, ov);
        } else {
          for (int r = 0; r < num_ranks; r++) {
            const int peer = (my_rank + r) % num_ranks;     // spread traffic over the links
            reinterpret_cast<uint4*>((__nv_bfloat16*)ag_dst.p[peer] + dst_row * H)[v] = ov;
          }
        }
      }
    }
    __syncthreads();          // red[] is reused by the next row
   }
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&ctl->done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      const uint32_t epoch = ctl->ag_epoch + 1;
      if (ctl->status == 0)
        for (int r = 0; r < num_ranks; r++) st_release_sys(ag_flag_dst.p[r], epoch);
      ctl->ag_epoch = epoch;
      ctl->done_ctr = 0;
      __threadfence();
    }
  }
}

// ---------------------------------------------------------------- NVLS (multimem) variant
// The same step through NVSwitch multicast memory: every rank's GEMM wrote its bf16 partial
// [T, H] into ITS OWN copy of a multicast-bound buffer; the owner of a row shard fetches the sum
// over all ranks with one `multimem.ld_reduce` per 16 bytes (the switch adds the N copies in
// fp32, 1/N of the bytes arrive here) and publishes the normalised rows with `multimem.st`
// (one store leaves this GPU, the switch replicates it into every rank's gather buffer).
// Flags and epochs are the ones of the peer-store variant.
template <int VEC_PER_THREAD>
__global__ void nvls_reduce_add_norm_push_kernel(const __nv_bfloat16* mc_partial, int reduce,
                                                 const __nv_bfloat16* x_local,
                                                 __nv_bfloat16* residual,
                                                 const __nv_bfloat16* __restrict__ weight, float eps,
                                                 __nv_bfloat16* mc_gather, PeerFlags ag_flag_dst,
                                                 CommCtl* ctl, int rows_local, int H, int my_rank,
                                                 int num_ranks, int skip_norm) {
  __shared__ float red[32];
  __shared__ int s_ok;
  const int nvec = H >> 3;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (reduce) {
    const uint32_t epoch = ctl->rs_epoch;      // published by this rank's own GEMM launch
    if (threadIdx.x < num_ranks && threadIdx.x != my_rank) {
      if (!wait_flag_ge(&ctl->rs_flag[threadIdx.x], epoch, &ctl->status)) s_ok = 0;
    }
    __syncthreads();
  }
  float vals[VEC_PER_THREAD][8];
  if (s_ok) {
    for (int row = blockIdx.x; row < rows_local; row += gridDim.x) {
      const size_t grow = (size_t)my_rank * rows_local + row;
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < VEC_PER_THREAD; i++) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
          uint32_t zw[4];
          if (reduce) {
            const uint4 pv = multimem_ld_reduce_bf16x8(mc_partial + grow * H + (size_t)v * 8);
            const uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w};
            uint4* rr = reinterpret_cast<uint4*>(residual + (size_t)row * H) + v;
            const uint4 rv = *rr;
            const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const float2 f = unpack_bf16x2(rw[j]);
              const float2 g = unpack_bf16x2(pw[j]);     // the reduced GEMM output, rounded to bf16
              zw[j] = pack_bf16x2(g.x + f.x, g.y + f.y);
            }
            *rr = make_uint4(zw[0], zw[1], zw[2], zw[3]);
          } else {
            const uint4 pv = reinterpret_cast<const uint4*>(x_local + (size_t)row * H)[v];
            zw[0] = pv.x; zw[1] = pv.y; zw[2] = pv.z; zw[3] = pv.w;
          }
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const float2 f = unpack_bf16x2(zw[j]);
            vals[i][2 * j] = f.x;
            vals[i][2 * j + 1] = f.y;
            ss += f.x * f.x + f.y * f.y;
          }
        }
      }
      ss = warp_reduce_sum(ss);
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
      __syncthreads();
      if (threadIdx.x < 32) {
        float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
        t = warp_reduce_sum(t);
        if (threadIdx.x == 0) red[0] = skip_norm ? 1.f : rsqrtf(t / (float)H + eps);
      }
      __syncthreads();
      const float inv = red[0];
#pragma unroll
      for (int i = 0; i < VEC_PER_THREAD; i++) {
        const int v = threadIdx.x + i * blockDim.x;
        if (v < nvec) {
          uint32_t o[4];
          if (skip_norm) {
#pragma unroll
            for (int j = 0; j < 4; j++) o[j] = pack_bf16x2(vals[i][2 * j], vals[i][2 * j + 1]);
          } else {
            const uint4 ww = reinterpret_cast<const uint4*>(weight)[v];
            const uint32_t w4[4] = {ww.x, ww.y, ww.z, ww.w};
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const float2 fw = unpack_bf16x2(w4[j]);
              o[j] = pack_bf16x2(vals[i][2 * j] * inv * fw.x, vals[i][2 * j + 1] * inv * fw.y);
            }
          }
          multimem_st_b128(mc_gather + grow * H + (size_t)v * 8, make_uint4(o[0], o[1], o[2], o[3]));
        }
      }
      __syncthreads();          // red[] is reused by the next row
    }
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t prev = atomicAdd(&ctl->done_ctr, 1u);
    if (prev == gridDim.x - 1) {
      __threadfence_system();
      const uint32_t epoch = ctl->ag_epoch + 1;
      if (ctl->status == 0)
        for (int r = 0; r < num_ranks; r++) st_release_sys(ag_flag_dst.p[r], epoch);
      ctl->ag_epoch = epoch;
      ctl->done_ctr = 0;
      __threadfence();
    }
  }
}

// Wait until every source rank's all-gather rows of the current epoch have landed.
__global__ void ag_wait_kernel(CommCtl* ctl, int my_rank, int num_ranks) {
  if (threadIdx.x < num_ranks && threadIdx.x != my_rank)
    wait_flag_ge(&ctl->ag_flag[threadIdx.x], ctl->ag_epoch, &ctl->status);
}

__global__ void memset_ctl_kernel(CommCtl* ctl) {
  if (threadIdx.x == 0) {
    CommCtl z = {};
    *ctl = z;
  }
}

}  // namespace b200

using namespace b200;

// ---------------------------------------------------------------- symmetric memory (host)
B200_API int b200_symm_alloc(long bytes, void** out) {
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) return (int)e;
  *out = p;
  return 0;
}
B200_API int b200_symm_free(void* p) { return (int)cudaFree(p); }
B200_API int b200_ipc_get_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  memcpy(handle64, &h, sizeof(h));
  return 0;
}
B200_API int b200_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
B200_API int b200_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }
B200_API int b200_comm_ctl_bytes() { return (int)sizeof(CommCtl); }

B200_API int b200_comm_read_status(void* ctl, int* out, cudaStream_t stream) {
  cudaError_t e = cudaMemcpyAsync(out, &((CommCtl*)ctl)->status, sizeof(int),
                                  cudaMemcpyDeviceToHost, stream);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaStreamSynchronize(stream);
}

B200_API int b200_comm_barrier(void* const* peer_ctl, int my_rank, int num_ranks,
                               cudaStream_t stream) {
  // device array of flag pointers is passed through a small managed struct
  static thread_local uint32_t** d_flags = nullptr;
  static thread_local int d_n = 0;
  if (!d_flags || d_n != num_ranks) {
    if (d_flags) cudaFree(d_flags);
    if (cudaMalloc(&d_flags, sizeof(uint32_t*) * kMaxRanks) != cudaSuccess) return 9140;
    d_n = num_ranks;
    uint32_t* h[kMaxRanks];
    for (int o = 0; o < num_ranks; o++) h[o] = &((CommCtl*)peer_ctl[o])->bar_flag[my_rank];
    cudaMemcpy(d_flags, h, sizeof(uint32_t*) * num_ranks, cudaMemcpyHostToDevice);
  }
  barrier_kernel<<<1, 32, 0, stream>>>((CommCtl*)peer_ctl[my_rank], d_flags, my_rank, num_ranks);
  return B200_CHECK_LAUNCH();
}

// in: this rank's symmetric buffer (already holding the input); peers: all ranks' buffers
B200_API int b200_allreduce_oneshot(void* const* peer_bufs, void* const* peer_ctl, void* out,
                                    long numel, int my_rank, int num_ranks,
                                    cudaStream_t stream) {
  if (numel <= 0) return 0;
  if (numel & 7) return 9100;
  PeerPtrs b;
  PeerFlags f;
  for (int r = 0; r < num_ranks; r++) {
    b.p[r] = peer_bufs[r];
    f.p[r] = &((CommCtl*)peer_ctl[r])->bar_flag[my_rank];
  }
  const long nvec = numel >> 3;
  long blocks = (nvec + 255) / 256;
  if (blocks > 4 * 148) blocks = 4 * 148;
  allreduce_oneshot_kernel<<<(unsigned)blocks, 256, 0, stream>>>(
      b, f, (CommCtl*)peer_ctl[my_rank], (__nv_bfloat16*)out, nvec, my_rank, num_ranks);
  return B200_CHECK_LAUNCH();
}

// staging: local [num_src][rows_local][H] (num_src = num_ranks, or 0 to normalise x_local);
// ag_bufs / peer_ctl: host arrays of peer-mapped pointers.
// mc_gather (optional): multicast address of the gather buffer; the push then uses multimem.st.
B200_API int b200_reduce_add_norm_push_mc(const void* staging, int num_src, const void* x_local,
                                          void* residual, const void* weight, float eps,
                                          void* const* ag_bufs, void* const* peer_ctl,
                                          int rows_local, int H, int my_rank, int num_ranks,
                                          int skip_norm, void* mc_gather, cudaStream_t stream);

B200_API int b200_reduce_add_norm_push(const void* staging, int num_src, const void* x_local,
                                       void* residual, const void* weight, float eps,
                                       void* const* ag_bufs, void* const* peer_ctl,
                                       int rows_local, int H, int my_rank, int num_ranks,
                                       int skip_norm, cudaStream_t stream) {
  return b200_reduce_add_norm_push_mc(staging, num_src, x_local, residual, weight, eps, ag_bufs,
                                      peer_ctl, rows_local, H, my_rank, num_ranks, skip_norm, nullptr,
                                      stream);
}

B200_API int b200_reduce_add_norm_push_mc(const void* staging, int num_src, const void* x_local,
                                          void* residual, const void* weight, float eps,
                                          void* const* ag_bufs, void* const* peer_ctl,
                                          int rows_local, int H, int my_rank, int num_ranks,
                                          int skip_norm, void* mc_gather, cudaStream_t stream) {
  if (rows_local <= 0) return 0;
  if (H & 7) return 9100;
  PeerPtrs a;
  PeerFlags f;
  for (int r = 0; r < num_ranks; r++) {
    a.p[r] = ag_bufs[r];
    f.p[r] = &((CommCtl*)peer_ctl[r])->ag_flag[my_rank];
  }
  const int nvec = H >> 3;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32 * ((num_ranks + 31) / 32)) threads = 32 * ((num_ranks + 31) / 32);
  const int per = (nvec + threads - 1) / threads;
  CommCtl* ctl = (CommCtl*)peer_ctl[my_rank];
  const int grid = rows_local < 148 * 4 ? rows_local : 148 * 4;
#define LAUNCH_RANP(V)                                                                       \
  reduce_add_norm_push_kernel<V><<<grid, threads, 0, stream>>>(                              \
      (const __nv_bfloat16*)staging, num_src, (const __nv_bfloat16*)x_local,                 \
      (__nv_bfloat16*)residual, (const __nv_bfloat16*)weight, eps, a, f, ctl, rows_local, H, \
      my_rank, num_ranks, skip_norm, (__nv_bfloat16*)mc_gather)
  if (per <= 1) LAUNCH_RANP(1);
  else if (per <= 2) LAUNCH_RANP(2);
  else if (per <= 4) LAUNCH_RANP(4);
  else return 9101;
#undef LAUNCH_RANP
  return B200_CHECK_LAUNCH();
}

// NVLS form of b200_reduce_add_norm_push.  mc_partial / mc_gather: multicast addresses of the
// partial-sum buffer [T, H] and of the gather buffer [T, H] (T = num_ranks * rows_local);
// reduce = 0 normalises x_local (first layer) instead of summing partials.
B200_API int b200_nvls_reduce_add_norm_push(const void* mc_partial, int reduce, const void* x_local,
                                            void* residual, const void* weight, float eps,
                                            void* mc_gather, void* const* peer_ctl, int rows_local,
                                            int H, int my_rank, int num_ranks, int skip_norm,
                                            cudaStream_t stream) {
  if (rows_local <= 0) return 0;
  if (H & 7) return 9100;
  if (!mc_gather || (reduce && (!mc_partial || !residual))) return 9141;
  PeerFlags f;
  for (int r = 0; r < num_ranks; r++) f.p[r] = &((CommCtl*)peer_ctl[r])->ag_flag[my_rank];
  const int nvec = H >> 3;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32 * ((num_ranks + 31) / 32)) threads = 32 * ((num_ranks + 31) / 32);
  const int per = (nvec + threads - 1) / threads;
  CommCtl* ctl = (CommCtl*)peer_ctl[my_rank];
  const int grid = rows_local < 148 * 4 ? rows_local : 148 * 4;
#define LAUNCH_NVLS(V)                                                                          \
  nvls_reduce_add_norm_push_kernel<V><<<grid, threads, 0, stream>>>(                            \
      (const __nv_bfloat16*)mc_partial, reduce, (const __nv_bfloat16*)x_local,                  \
      (__nv_bfloat16*)residual, (const __nv_bfloat16*)weight, eps, (__nv_bfloat16*)mc_gather, f, \
      ctl, rows_local, H, my_rank, num_ranks, skip_norm)
  if (per <= 1) LAUNCH_NVLS(1);
  else if (per <= 2) LAUNCH_NVLS(2);
  else if (per <= 4) LAUNCH_NVLS(4);
  else return 9101;
#undef LAUNCH_NVLS
  return B200_CHECK_LAUNCH();
}

B200_API int b200_ag_wait(void* ctl, int my_rank, int num_ranks, cudaStream_t stream) {
  ag_wait_kernel<<<1, 32, 0, stream>>>((CommCtl*)ctl, my_rank, num_ranks);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_comm_ctl_reset(void* ctl, cudaStream_t stream) {
  memset_ctl_kernel<<<1, 32, 0, stream>>>((CommCtl*)ctl);
  return B200_CHECK_LAUNCH();
}
