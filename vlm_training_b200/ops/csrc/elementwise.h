// C entry points of the bandwidth-bound fused kernels (elementwise.cu).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif
int vlmt_norm_blocks(int rows);
void vlmt_rmsnorm_fwd(const void* x, const void* res, const void* w, int w_fp32, void* y, void* r_out, float* rstd, int rows, int D, float eps, int offset, cudaStream_t st);
int vlmt_rmsnorm_bwd(const void* dy, const void* x, const void* w, int w_fp32, const float* rstd, const void* dres, void* dx, float* dw_partial, int rows, int D, int offset, cudaStream_t st);
void vlmt_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows, int D, float eps, cudaStream_t st);
int vlmt_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx, float* dw_partial, float* db_partial, int rows, int D, cudaStream_t st);
void vlmt_rmsnorm_gated_fwd(const void* x, const void* z, const void* w, void* y, float* rstd, int rows, int D, float eps, cudaStream_t st);
int vlmt_rmsnorm_gated_bwd(const void* dy, const void* x, const void* z, const void* w, const float* rstd, void* dx, void* dz, float* dw_partial, int rows, int D, cudaStream_t st);
void vlmt_swiglu_fwd(const void* gu, void* out, long rows, int I, cudaStream_t st);
void vlmt_swiglu_bwd(const void* dout, const void* gu, void* dgu, long rows, int I, cudaStream_t st);
void vlmt_sigmoid_mul_fwd(const void* x, const void* gate, void* out, long n, cudaStream_t st);
void vlmt_sigmoid_mul_bwd(const void* dout, const void* x, const void* gate, void* dx, void* dgate, long n, cudaStream_t st);
void vlmt_gelu_fwd(const void* x, void* y, long n, int tanh_approx, cudaStream_t st);
void vlmt_gelu_bwd(const void* dy, const void* x, void* dx, long n, int tanh_approx, cudaStream_t st);
int vlmt_qkv_blocks(long items);
int vlmt_qkv_norm_rope_fwd(const void* qkv, const void* qw, const void* kw, const float* cosv, const float* sinv, void* q, void* k, void* v, void* gate, float* rstd, int T, int n_q, int n_kv, int D, int R, float eps, int offset, int gated, int has_norm, cudaStream_t st);
int vlmt_qkv_norm_rope_bwd(const void* dq, const void* dk, const void* dv, const void* dgate, const void* qkv, const void* qw, const void* kw, const float* cosv, const float* sinv, const float* rstd, void* dqkv, float* dw_partial, int T, int n_q, int n_kv, int D, int R, int offset, int gated, int has_norm, cudaStream_t st);
void vlmt_rope_generic(const void* x, long ss, long hs, const float* cosv, const float* sinv, void* out, long oss, long ohs, int S, int H, int D, int transpose, cudaStream_t st);
void vlmt_gdn_gates_fwd(const void* a, const void* b, long row_stride, const float* A_log, const float* dt_bias, float* g, void* beta, long T, int H, cudaStream_t st);
int vlmt_gdn_gates_bwd(const float* dg, const void* dbeta, const void* a, const void* b, long row_stride, const float* A_log, const float* dt_bias, void* da, void* db, long out_stride, float* partial, long T, int H, cudaStream_t st);
int vlmt_conv1d_silu_fwd(const void* x, long xs, const void* w, const int* seq_idx, void* y, long ys, int T, int C, int K, cudaStream_t st);
int vlmt_conv1d_bwd_slabs(int T);
int vlmt_conv1d_silu_bwd(const void* dy, long dys, const void* x, long xs, const void* w, const int* seq_idx, void* dx, long dxs, float* dw_partial, int T, int C, int K, cudaStream_t st);
void vlmt_rows_update(void* out, const long* index, const void* src, long n_rows, int D, int add, cudaStream_t st);
void vlmt_rows_gather(void* dst, const long* index, const void* src, long n_rows, int D, cudaStream_t st);
#ifdef __cplusplus
}
#endif
