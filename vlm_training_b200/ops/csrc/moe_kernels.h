// C entry points of the mixture-of-experts routing / permutation kernels (moe_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif
// softmax over E experts (E <= 512) -> top-k (ties to the lower id) -> optional renormalisation.
// logits [T, E] bf16 or fp32; weights [T, k] fp32; experts [T, k] int32; counts: optional [E] histogram (atomicAdd).
int vlmt_moe_route_fwd(const void* logits, int logits_fp32, int T, int E, int k, int renorm, float* weights, int* experts, int* counts,
                       cudaStream_t st);
int vlmt_moe_route_bwd(const void* logits, int logits_fp32, const int* experts, const float* weights, const float* dweights, int T, int E,
                       int k, int renorm, void* dlogits, cudaStream_t st);
// Stable counting sort of n_slots slots by expert into the padded row layout of the grouped GEMM (128-row tiles per expert).
// hist: scratch of vlmt_moe_plan_blocks(n_slots) * E ints; counts [E]; prefix [E + 1] (first tile of every expert, total);
// dest [n_slots] (row of every slot); slot_of_row [cap_rows] (slot of every row, -1 = padding).
int vlmt_moe_plan_blocks(long n_slots);
int vlmt_moe_plan(const int* experts, long n_slots, int E, int* hist, int* counts, int* prefix, int* dest, int* slot_of_row, long cap_rows,
                  cudaStream_t st);
// rows[r] = scale[slot] * src[slot / k] for the slot of row r (zeros for padding rows), rows of tiles in use only
int vlmt_moe_rows_from_tokens(const void* src, const int* slot_of_row, const int* prefix, int E, int k, int H, const float* scale, void* rows,
                              long cap_rows, cudaStream_t st);
// out[t] = sum_j w[t,j] * rows[dest[t,j]] (w null: plain sum; out null: skipped); dw[t,j] = <g[t], rows[dest[t,j]]> when g, dw given
int vlmt_moe_tokens_from_rows(const void* rows, const int* dest, const float* w, int T, int k, int H, void* out, const void* g, float* dw,
                              cudaStream_t st);
#ifdef __cplusplus
}
#endif
