// Selected-key attention for DSA (see dsa_attention.cu).  q, o, d_o [B, Hkv * rep, D] bf16; k, v [L, Hkv, D] bf16;
// sel [B, kk] int32 key rows (-1 = unused slot); lse [B, Hkv * rep] fp32; dq [B, Hkv * rep, D], dk, dv [L, Hkv, D] fp32
// (dk / dv are accumulated into, so the caller zeroes them).  Return 0, or a negative code (-2: unsupported D / rep).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif
int vlmt_dsa_supported(int D, int rep);
int vlmt_dsa_fwd(const void* q, const void* k, const void* v, const int* sel, void* o, float* lse, int B, int Hkv, int rep, int D,
                 int kk, float scale, cudaStream_t st);
// forward on the tensor cores (dsa_attention_sm100.cu): D = 256, 8 query heads per kv head; `status`: the device status word
int vlmt_dsa_fwd_tc(const void* q, const void* k, const void* v, const int* sel, void* o, float* lse, int B, int Hkv, int kk, float scale,
                    int* status, cudaStream_t st);
int vlmt_dsa_bwd_tc(const void* q, const void* k, const void* v, const int* sel, const void* o, const float* lse, const void* d_o,
                    float* dq, float* dk, float* dv, int B, int Hkv, int kk, float scale, int* status, cudaStream_t st);
int vlmt_dsa_bwd(const void* q, const void* k, const void* v, const int* sel, const void* o, const float* lse, const void* d_o,
                 float* dq, float* dk, float* dv, int B, int Hkv, int rep, int D, int kk, float scale, cudaStream_t st);
// lightning indexer (dsa_indexer_sm100.cu): scores of one query block and the per-query top-k selection
int vlmt_dsa_index_scores(const void* iq, const void* ik, const float* w, int T, int q_tok0, int q_pos0, int k_tok0, int B, int n_keys,
                          float* scores, int ld, int* status, cudaStream_t st);
int vlmt_dsa_topk(const float* scores, int B, int ld, int q_pos0, int kk, int* sel, cudaStream_t st);
#ifdef __cplusplus
}
#endif
