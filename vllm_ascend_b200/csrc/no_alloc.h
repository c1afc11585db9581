// Allocation-free entry point of the split-KV flash-decode kernel.
//
// This entry point has no counterpart in the reference project.  It exists for
// callers that must not allocate device memory at the time of the call: code that
// runs inside a memory pool it may not grow, plugins loaded into a host process
// that owns the allocator, and real-time loops where a cudaMalloc (which may
// synchronise the device) is not acceptable.  Such callers cannot provide the
// scratch buffer that b200_paged_decode() needs for its split-KV partial results,
// and must not trigger an allocation inside the library either.
//
// b200_paged_decode_noalloc() keeps that scratch in a fixed array in device global
// memory that is part of the library image (B200_NOALLOC_SCRATCH_BYTES per GPU that
// loads the library, held until the process exits).  The caller passes inputs and
// outputs only.
//
//   * Limit: the partials need  B * Hq * num_splits * (D + 1) * 4  bytes.  A call that
//     needs more than B200_NOALLOC_SCRATCH_BYTES is rejected with
//     B200_NOALLOC_TOO_LARGE and nothing is launched; use fewer splits or
//     b200_paged_decode() with your own buffer.
//   * First call on a device: the library looks up the device address of the array
//     (cudaGetSymbolAddress, with that device current) and remembers it.  Make the
//     first call on each device outside of any stream capture.  Host threads that make
//     their first calls at the same time may each do the look-up; they store the same value
//     into the same slot, which is harmless, so the slot is not locked.
//   * The array is shared by every call on the device and keeps the previous call's
//     contents.  Nothing in it has to start at zero: every partial that the merge step
//     reads is written earlier in the same call.  Two calls whose kernels overlap on
//     the GPU (different streams, no dependency) race on the array: serialise them.
//   * No cudaMalloc, cudaFree or other allocating routine is called on any path.
#pragma once
#include <cuda_runtime.h>

#define B200_NOALLOC_SCRATCH_BYTES (8u << 20)
#define B200_NOALLOC_TOO_LARGE 9200
#define B200_NOALLOC_NO_SYMBOL 9201

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments as b200_paged_decode() without the scratch pointer:
// q [B, Hq, D] bf16 (token stride q_stride elements), caches [blocks, block_size, Hkv, D],
// block_table int32 [B, max_blocks], seq_lens int32 [B], out [B, Hq, D].
// Returns 0, a CUDA error code, or one of the B200_NOALLOC_* codes above.
int b200_paged_decode_noalloc(const void* q, long q_stride, const void* k_cache,
                              const void* v_cache, const void* block_table, int max_blocks,
                              const void* seq_lens, int B, int Hq, int Hkv, int D,
                              int block_size, float scale, int window, int num_splits, void* out,
                              long out_stride, long num_blocks_total, int* status,
                              cudaStream_t stream);

// Bytes of the built-in scratch a call with these sizes would use (0 when num_splits <= 1).
long b200_paged_decode_noalloc_bytes(int B, int Hq, int D, int num_splits);

#ifdef __cplusplus
}
#endif
