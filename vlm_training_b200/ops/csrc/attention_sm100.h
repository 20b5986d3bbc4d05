// C entry points of the tcgen05 varlen attention kernels (attention_sm100.cu).
#pragma once
#include <cuda_runtime.h>

#include "gemm_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif
// q [T,Hq,D], k/v [T,Hkv,D] bf16 with token strides ldq/ldk/ldv (elements); o [T,Hq,D]; lse [Hq,T] (natural log).
// cu: int32 [n_docs+1] device pointer.  D in {64, 128, 256} (256: the single-tile kernels of attention256_sm100.cu; d_eff unused).  d_eff (<= D) says that channels >= d_eff are zero padding in
// q/k/v (head dims such as 72 are stored padded to D): the contractions over the head dim (Q.K^T, dO.V^T) skip the
// 16-channel steps that lie entirely in the padding; the MMAs whose N dimension is the head dim stay full width
// (narrower ones measured slower).
int vlmt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu, int n_docs, int T, int Hq, int Hkv,
                  int D, int d_eff, long ldq, long ldk, long ldv, float scale, int causal, int* status, cudaStream_t st);
// all tensors contiguous; delta is fp32 scratch [Hq,T]
int vlmt_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse, float* delta, void* dq,
                  void* dk, void* dv, const int* cu, int n_docs, int T, int Hq, int Hkv, int D, int d_eff, float scale, int causal, int* status,
                  cudaStream_t st);
#ifdef __cplusplus
}
#endif
