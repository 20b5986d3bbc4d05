// C entry points of the cross-entropy and AdamW kernels (loss_optim.cu).
#pragma once
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif
// In place: logits[rows, V] -> grad_scale * (softmax - onehot); loss[row] = lse - logit[target] (0 if ignored).
void vlmt_ce_fwd_bwd(void* logits, long ld, const long* targets, float* loss, float grad_scale, int rows, int V, long ignore_index,
                     cudaStream_t st);
// m / v are fp32, or bf16 when state_bf16 != 0
// zero_grad != 0: the gradient range is cleared after it has been consumed
void vlmt_adamw(void* grad, int grad_fp32, float* master, void* m, void* v, int state_bf16, void* param, long n, float lr, float b1,
                float b2, float eps, float wd, float bc1, float bc2, float grad_scale, int zero_grad, cudaStream_t st);
// partial[slab, c] = sum of rows of the slab (512 rows each) of column c; cols must be even
void vlmt_sum_rows_f32(const float* partial, int rows, int cols, float* out, cudaStream_t st);
int vlmt_colsum_slabs(int rows);
void vlmt_colsum(const void* x, long ld, int rows, int cols, float* partial, float* out, cudaStream_t st);
void vlmt_sumsq(const void* x, int fp32, long n, float* out, cudaStream_t st);
#ifdef __cplusplus
}
#endif
