// Intra-chunk stages of the gated delta rule (prepare and output, forward and backward); see gdn_chunk_sm100.cu.
// All tile stacks are head-major: [H, N, rows, cols] bf16; q, k, v, do and the gradients are in token layout [T, H, 128].
// `chunks`: int32 [N, 2] on the device: first token and number of rows (1..64) of every chunk slot.
#pragma once
#include <cuda_runtime.h>

extern "C" {
int vlmt_gdn_prepare_fwd(const void* q, const void* k, const void* v, long ldq, long ldk, long ldv, const float* g, const float* beta,
                         const int* chunks, int T, int H, int N, float scale, float eps, void* w, void* u, void* kdec, void* qg, void* P,
                         void* Tm, float* gc, float* decay, int* status, cudaStream_t st);
int vlmt_gdn_output_fwd(const void* qg, const void* P, const void* states, const void* vnew, const int* chunks, int H, int N, void* o,
                        int* status, cudaStream_t st);
int vlmt_gdn_output_bwd(const void* dout, long ld_do, const void* qg, const void* P, const void* states, const void* vnew,
                        const int* chunks, int T, int H, int N, void* dqg, void* dP, void* dvn, void* dS, int* status, cudaStream_t st);
int vlmt_gdn_prepare_bwd(const void* q, const void* k, const void* v, long ldq, long ldk, long ldv, const float* beta, const float* gc,
                         const int* chunks, int T, int H, int N, float scale, float eps, const void* states, const void* adj,
                         const void* vnew, const void* du, const void* dqg, const void* dP, const void* P, const void* Tm, void* dq,
                         void* dk, void* dv, float* dg, float* dbeta, int* status, cudaStream_t st);
}
