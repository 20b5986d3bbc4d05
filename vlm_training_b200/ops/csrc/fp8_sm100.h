// C entry points of the FP8 training path (fp8_sm100.cu): tensor-wise dynamic quantisation and the tcgen05 FP8 GEMM.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum Fp8Format { FP8_E4M3 = 0, FP8_E5M2 = 1 };

#ifdef __cplusplus
extern "C" {
#endif
// rec[0] = max |x| over the [rows, cols] bf16 matrix (row stride ld elements).  rec is two floats in device memory; the
// call clears it first (stream-ordered).
int vlmt_fp8_amax(const void* x, long ld, long rows, long cols, float* rec, cudaStream_t stream);
// q = saturate(x * s) with s = format_max / max(rec[0], 1e-12); rec[1] = 1 / s (the factor that undoes the scaling).
// out_rm: [rows, ld_rm] bytes, the matrix as it is; out_t: [cols, ld_t] bytes, its transpose; either may be null.
int vlmt_fp8_cast(const void* x, long ld, long rows, long cols, float* rec, int format, void* out_rm, long ld_rm, void* out_t,
                  long ld_t, cudaStream_t stream);
// D[M,N] (+)= rec_a[1] * rec_b[1] * A(M,K) * B(N,K)^T: A and B one byte per element in the given formats, both K-major
// (row strides lda / ldb bytes, multiples of 16); D bf16 with row stride ldd elements (a multiple of 8).  With
// `accumulate` the product is added into D by the memory system (TMA reduce-add) and a long K is cut into parts that fill
// the SMs.  Returns 0 or a CUDA / encode error code; device-side timeouts land in *status.
int vlmt_gemm_fp8(const void* A, const void* B, void* D, int M, int N, int K, long lda, long ldb, long ldd, int a_format, int b_format,
                  const float* rec_a, const float* rec_b, int accumulate, int* status, int num_sms, cudaStream_t stream);
#ifdef __cplusplus
}
#endif
