// C entry points of the tcgen05 varlen attention kernels (attention_sm100.cu).
#pragma once
#include <cuda_runtime.h>

#include "gemm_sm100.h"

#ifdef __cplusplus
extern "C" {
#endif
// q [T,Hq,d], k / v [T,Hkv,d] bf16, each with its own token stride (ld*) and head stride (hs*) in elements, so slices of a
// fused projection are read in place; d a multiple of 8 up to 128, or 256.  o [T,Hq,d] contiguous; lse [Hq,T] (natural log).
// cu: int32 [n_docs+1] device pointer.  The kernels work on 64- or 128-wide tiles: TMA zero-fills the channels between d
// and the tile width, the contractions over the head dim stop at the next multiple of 16 and the output-side products are
// only that wide.  d = 256: the single-tile kernels of attention256_sm100.cu (heads contiguous).
int vlmt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu, int n_docs, int T, int Hq, int Hkv,
                  int d, long ldq, long hsq, long ldk, long hsk, long ldv, long hsv, float scale, int causal, int* status, cudaStream_t st);
// dout, o, dq, dk, dv contiguous; delta is fp32 scratch [Hq,T]
int vlmt_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse, float* delta, void* dq,
                  void* dk, void* dv, const int* cu, int n_docs, int T, int Hq, int Hkv, int d, long ldq, long hsq, long ldk, long hsk,
                  long ldv, long hsv, float scale, int causal, int* status, cudaStream_t st);
#ifdef __cplusplus
}
#endif
