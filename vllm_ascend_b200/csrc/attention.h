// Internal launchers shared between the attention translation units.
#pragma once
#include <cuda_runtime.h>

namespace b200 {

// lse_out (optional, [T, Hq]): log-sum-exp of the merged result
int launch_merge_splits(const float* partial_o, const float* partial_lse, long T, int Hq,
                        int num_splits, int D, void* out, long out_stride, cudaStream_t stream,
                        float* lse_out = nullptr);

int launch_paged_decode(const void* q, long q_stride, const void* k_cache, const void* v_cache,
                        const int* block_table, int max_blocks, const int* seq_lens, int B,
                        int Hq, int Hkv, int D, int block_size, float scale, int window,
                        int num_splits, void* out, long out_stride, float* partial_o,
                        float* partial_lse, long num_blocks_total, int* status,
                        cudaStream_t stream);

}  // namespace b200
