// Speculative-decoding kernels.
//   rejection_sample: one CTA per request walks its draft tokens in order.
//     greedy row : accept while draft[i] == target_argmax[i]; emit target_argmax at the
//                  first mismatch; all accepted -> emit the bonus token.
//     random row : accept x = draft[i] when u[i] < p_target(x) / p_draft(x) (p_draft = 1
//                  without draft probabilities, e.g. n-gram proposals); at the first
//                  rejection emit a recovered token ~ max(p_target - p_draft, 0), drawn by an
//                  exponential race over the vocabulary with caller-provided noise; bonus
//                  token only when every draft was accepted.
//     output [B, max_spec + 1] padded with -1, plus the number of emitted tokens per row.
//   Semantics of the reference's rejection sampler (vllm_ascend/sample/rejection_sampler.py:422-905,
//   1130-1310; kernels ops/triton/reject_sample.py:35-700).
//   expand_draft_inputs: scatter (last sampled token, draft tokens) of every request into the
//   flat input / position arrays of a verification step (the reference's
//   csrc/moe/copy_and_expand_eagle_inputs).
#include "common.cuh"

namespace b200 {

struct RejectParams {
  const int* draft_ids;        // [N] flattened
  const int* cu_draft;         // [B + 1]
  const int* target_argmax;    // [N] (greedy rows)
  const int* bonus_ids;        // [B]
  const float* target_probs;   // [N, V] or null when every row is greedy
  const float* draft_probs;    // [N, V] or null
  const float* uniform;        // [N]
  const float* race_noise;     // [B, V] exponential(1) samples
  const unsigned char* is_greedy;  // [B]
  int* out;                    // [B, max_spec + 1]
  int* num_out;                // [B]
  int B, V, max_spec;
  int* status;
};

__global__ void __launch_bounds__(256) rejection_sample_kernel(const RejectParams p) {
  const int b = blockIdx.x;
  const int tid = threadIdx.x;
  const int s0 = p.cu_draft[b], n = p.cu_draft[b + 1] - s0;
  int* out = p.out + (long)b * (p.max_spec + 1);
  __shared__ int s_stop;            // position of the first rejection, or n
  __shared__ float s_best[8];
  __shared__ int s_arg[8];
  for (int i = tid; i <= p.max_spec; i += blockDim.x) out[i] = -1;
  if (n < 0 || n > p.max_spec) {
    if (tid == 0) { if (p.status) atomicExch(p.status, B200_BAD_INDEX); p.num_out[b] = 0; }
    return;
  }
  __syncthreads();
  const bool greedy = p.is_greedy[b] != 0 || p.target_probs == nullptr;
  if (tid == 0) {
    int stop = n;
    for (int i = 0; i < n; i++) {
      const int x = p.draft_ids[s0 + i];
      bool accept;
      if (greedy) {
        accept = (x == p.target_argmax[s0 + i]);
      } else {
        const float pt = (x >= 0 && x < p.V) ? p.target_probs[(long)(s0 + i) * p.V + x] : 0.f;
        const float pd = p.draft_probs ? p.draft_probs[(long)(s0 + i) * p.V + x] : 1.f;
        accept = pd > 0.f && p.uniform[s0 + i] * pd < pt;
      }
      if (!accept) { stop = i; break; }
      out[i] = x;
    }
    s_stop = stop;
  }
  __syncthreads();
  const int stop = s_stop;
  if (stop == n) {                       // everything accepted: bonus token
    if (tid == 0) { out[n] = p.bonus_ids[b]; p.num_out[b] = n + 1; }
    return;
  }
  if (greedy) {
    if (tid == 0) { out[stop] = p.target_argmax[s0 + stop]; p.num_out[b] = stop + 1; }
    return;
  }
  // recovered token: argmax_v max(pt - pd, 0) / noise[v]
  const float* pt = p.target_probs + (long)(s0 + stop) * p.V;
  const float* pd = p.draft_probs ? p.draft_probs + (long)(s0 + stop) * p.V : nullptr;
  const float* nz = p.race_noise + (long)b * p.V;
  const int xd = p.draft_ids[s0 + stop];
  float best = -1.f;
  int arg = 0;
  for (int v = tid; v < p.V; v += blockDim.x) {
    float r = pd ? fmaxf(pt[v] - pd[v], 0.f) : (v == xd ? 0.f : pt[v]);
    r = r / fmaxf(nz[v], 1e-20f);
    if (r > best) { best = r; arg = v; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
    if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
  }
  if ((tid & 31) == 0) { s_best[tid >> 5] = best; s_arg[tid >> 5] = arg; }
  __syncthreads();
  if (tid == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); w++)
      if (s_best[w] > best || (s_best[w] == best && s_arg[w] < arg)) { best = s_best[w]; arg = s_arg[w]; }
    out[stop] = arg;
    p.num_out[b] = stop + 1;
  }
}

// one thread per (request, j): j = 0 is the request's last sampled token, j >= 1 draft j-1.
__global__ void expand_draft_inputs_kernel(const int* __restrict__ last_tokens,
                                           const int* __restrict__ draft_ids,
                                           const int* __restrict__ cu_draft,
                                           const int* __restrict__ start_pos,
                                           long* __restrict__ input_ids, long* __restrict__ positions,
                                           int* __restrict__ cu_out, int B, int max_spec) {
  const int b = blockIdx.x;
  if (b >= B) return;
  const int s0 = cu_draft[b], n = cu_draft[b + 1] - s0;
  const int o0 = s0 + b;                       // every earlier request contributed draft + 1 rows
  for (int j = threadIdx.x; j <= n && j <= max_spec; j += blockDim.x) {
    input_ids[o0 + j] = (j == 0) ? last_tokens[b] : draft_ids[s0 + j - 1];
    positions[o0 + j] = start_pos[b] + j;
  }
  if (threadIdx.x == 0) {
    cu_out[b] = o0;
    if (b == B - 1) cu_out[B] = o0 + n + 1;
  }
}

}  // namespace b200

using namespace b200;

B200_API int b200_rejection_sample(const void* draft_ids, const void* cu_draft,
                                   const void* target_argmax, const void* bonus_ids,
                                   const void* target_probs, const void* draft_probs,
                                   const void* uniform, const void* race_noise,
                                   const void* is_greedy, void* out, void* num_out, int B, int V,
                                   int max_spec, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  RejectParams p;
  p.draft_ids = (const int*)draft_ids; p.cu_draft = (const int*)cu_draft;
  p.target_argmax = (const int*)target_argmax; p.bonus_ids = (const int*)bonus_ids;
  p.target_probs = (const float*)target_probs; p.draft_probs = (const float*)draft_probs;
  p.uniform = (const float*)uniform; p.race_noise = (const float*)race_noise;
  p.is_greedy = (const unsigned char*)is_greedy;
  p.out = (int*)out; p.num_out = (int*)num_out;
  p.B = B; p.V = V; p.max_spec = max_spec; p.status = status;
  rejection_sample_kernel<<<B, 256, 0, stream>>>(p);
  return B200_CHECK_LAUNCH();
}

B200_API int b200_expand_draft_inputs(const void* last_tokens, const void* draft_ids,
                                      const void* cu_draft, const void* start_pos, void* input_ids,
                                      void* positions, void* cu_out, int B, int max_spec,
                                      cudaStream_t stream) {
  if (B <= 0) return 0;
  expand_draft_inputs_kernel<<<B, 32, 0, stream>>>((const int*)last_tokens, (const int*)draft_ids,
                                                   (const int*)cu_draft, (const int*)start_pos,
                                                   (long*)input_ids, (long*)positions, (int*)cu_out,
                                                   B, max_spec);
  return B200_CHECK_LAUNCH();
}
