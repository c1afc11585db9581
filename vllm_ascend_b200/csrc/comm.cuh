// Cross-GPU signalling primitives over peer-mapped ("symmetric") memory.
//
// Flags carry monotonically increasing epochs, so nothing is ever reset and a
// flag that a peer never writes simply keeps an old epoch: the waiter gives up
// after a bounded time, records B200_TIMEOUT and the kernel returns normally.
// (The reference's equivalents spin without bound:
//  csrc/mc2/dispatch_ffn_combine/op_kernel/utils/hccl_shmem.hpp:45-79, 243-300.)
#pragma once
#include "common.cuh"

namespace b200 {

constexpr int kMaxRanks = 16;

// Layout of one rank's control block (lives inside its symmetric buffer).
struct CommCtl {
  uint32_t ag_flag[kMaxRanks];    // written by peer src: "my all-gather rows for epoch e are in your buffer"
  uint32_t rs_flag[kMaxRanks];    // written by peer src: "my reduce-scatter partials for epoch e are in your buffer"
  uint32_t bar_flag[kMaxRanks];   // generic barrier / all-reduce signals
  uint32_t ag_epoch;              // local: last epoch this rank published
  uint32_t rs_epoch;
  uint32_t bar_epoch;
  uint32_t done_ctr;              // local: CTAs finished in the current kernel ("last block" detection)
  uint32_t done_ctr2;
  int status;                     // local: B200_TIMEOUT etc.
  uint32_t pad[9];
};

// Control block of the fused MoE dispatch/GEMM/combine path (lives at the start of the MoE
// symmetric region of every rank).  All flags are epochs of the same monotonically
// increasing call counter.
struct MoeCtl {
  uint32_t hist_flag[kMaxRanks];   // peer src published its routing histogram for epoch e
  uint32_t disp_flag[kMaxRanks];   // peer src finished writing its token rows for epoch e
  uint32_t comb_flag[kMaxRanks];   // peer (expert owner) finished writing my result rows
  uint32_t epoch;                  // local: calls completed so far
  uint32_t done_ctr;               // "last block" detection, dispatch kernel
  uint32_t done_ctr2;              // same, scatter GEMM
  uint32_t done_ctr3;              // same, reduce kernel
  uint32_t pad[12];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}

// Bounded wait until *flag >= epoch (wrap-safe signed compare).  Returns false on
// timeout after recording it in *status.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* flag, uint32_t epoch, int* status,
                                             long long budget_cycles = B200_WAIT_CYCLES) {
  if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
  long long t0 = 0;
  uint32_t spins = 0;
  while (true) {
    if ((int32_t)(ld_acquire_sys(flag) - epoch) >= 0) return true;
    if ((++spins & 0x3f) == 0) {
      const long long now = clock64();
      if (t0 == 0) {
        t0 = now;
      } else if (now - t0 > budget_cycles) {
        if (status) atomicExch(status, B200_TIMEOUT);
        return false;
      }
      __nanosleep(64);
    }
  }
}

}  // namespace b200
