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
// the two stages of vlmt_moe_plan on their own; row_base (optional, [E]): first row per expert given by the caller
int vlmt_moe_plan_count(const int* experts, long n_slots, int E, int* hist, int* counts, int* prefix, cudaStream_t st);
int vlmt_moe_plan_place(const int* experts, long n_slots, int E, const int* hist, const int* prefix, const int* row_base, int* dest,
                        int* slot_of_row, long cap_rows, cudaStream_t st);
// rows[r] = scale[slot] * src[slot / k] for the slot of row r (zeros for padding rows), rows of tiles in use only
int vlmt_moe_rows_from_tokens(const void* src, const int* slot_of_row, const int* prefix, int E, int k, int H, const float* scale, void* rows,
                              long cap_rows, cudaStream_t st);
// out[t] = sum_j w[t,j] * rows[dest[t,j]] (w null: plain sum; out null: skipped); dw[t,j] = <g[t], rows[dest[t,j]]> when g, dw given
int vlmt_moe_tokens_from_rows(const void* rows, const int* dest, const float* w, int T, int k, int H, void* out, const void* g, float* dw,
                              cudaStream_t st);
// ---- expert parallelism over peer memory (ep ranks; expert e lives on rank e / (E / ep); all buffers symmetric) ----
// this rank's counts [E] -> row `me` of every rank's [ep, E] count matrix (mats[r] = rank r's matrix)
int vlmt_ep_push_counts(const int* counts, int E, void* const* mats, int ep, int me, cudaStream_t st);
// from the complete count matrix: row_base [E] (first row of THIS rank's slots of every expert inside the owner's buffer),
// prefix_local [E/ep + 1] and tot_local [E/ep] of the experts this rank owns; status 200 when an owner's rows exceed cap_rows
int vlmt_ep_plan(const int* counts_all, int ep, int E, int me, int cap_rows, int* row_base, int* prefix_local, int* tot_local, int* status,
                 cudaStream_t st);
// rows[o][dest[slot]] = scale[slot] * src[slot / k]; srcs[o][dest[slot]] = me * n_slots + slot   (o = owner of experts[slot])
int vlmt_ep_dispatch(const void* src, const int* experts, const int* dest, const float* scale, long n_slots, int k, int H, int El, int me,
                     void* const* rows, void* const* srcs, int ep, cudaStream_t st);
// owner: zero the padding rows of every local expert's last tile and mark them src_of_row = -1
int vlmt_ep_zero_padding(void* rows, int* src_of_row, const int* prefix_local, const int* tot_local, int El, int H, long cap_rows,
                         cudaStream_t st);
// owner: backs[source rank][slot] = y[row] for every row that holds a slot
int vlmt_ep_return(const void* y, const int* src_of_row, const int* prefix_local, int El, long n_slots, int H, long cap_rows,
                   void* const* backs, int ep, cudaStream_t st);
#ifdef __cplusplus
}
#endif
