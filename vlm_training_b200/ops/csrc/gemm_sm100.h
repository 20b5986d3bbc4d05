// C entry points of the tcgen05 GEMM (gemm_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

enum GemmEpilogue { GEMM_EPI_NONE = 0, GEMM_EPI_GELU_TANH = 1, GEMM_EPI_GELU_ERF = 2 };

#ifdef __cplusplus
extern "C" {
#endif
// D[M,N] (+)= A(M,K) * B(N,K)^T (+ bias[N]) (-> GELU), bf16 in, fp32 accumulate.
// a_mn_major: A is stored [K, M] (lda = M-stride);  else [M, K].
// b_mn_major: B is stored [K, N];                    else [N, K].
// Dacc32 != null: write/accumulate fp32 results there instead of bf16 D.
// Returns 0 or a CUDA / encode error code; device-side timeouts land in *status.
int vlmt_gemm_bf16(const void* A, const void* B, void* D, float* Dacc32, const void* bias, int M, int N, int K, int lda,
                   int ldb, int ldd, int a_mn_major, int b_mn_major, int epilogue, int accumulate, int* status, int num_sms,
                   cudaStream_t stream);
// Same GEMM (A K-major; B K-major or MN-major) whose output rows go to `world` destinations: rows owned by rank o
// (blocks of rows_per_rank, a multiple of 128) are stored into dst[o], typically peer memory.
int vlmt_gemm_bf16_rs_push(const void* A, const void* B, void* const* dst, int world, int rows_per_rank, int M, int N, int K, int lda,
                           int ldb, int ldd, int b_mn_major, int* status, int num_sms, cudaStream_t stream);
// One launch for all groups (the experts of a MoE layer); `prefix` (device memory, groups + 1 ints) gives the first
// 128-row tile of every group in the padded row layout.  mode 1: forward / dgrad, groups partition the M dimension
// (M = row capacity) and every group has its own B (stacked along B's rows); mode 2: wgrad, groups partition the
// contraction over the rows (K = row capacity) and every group writes its own [M, N] block of D.
int vlmt_gemm_bf16_grouped(const void* A, const void* B, void* D, const int* prefix, int groups, int mode, int M, int N, int K, int lda,
                           int ldb, int ldd, int a_mn_major, int b_mn_major, int* status, int num_sms, cudaStream_t stream);
// All-gather fused into the GEMM (tensor-parallel column linear on sequence-sharded rows): D[world * rows, N] =
// gathered(A) x op(B).  The kernel copies this rank's rows `src` [rows, K] (contiguous) into block `rank` of
// gathered[r] for every rank r (peer stores; gathered[rank] == A_full is the local [world * rows, K] buffer), stores
// `epoch` into flag_dst[r][rank] of every peer when the copy is complete, computes the tiles of its own rows from `src`
// meanwhile and reads a peer's block of A_full once flags[peer] >= epoch (bounded wait -> status 100 + peer).
// counter: one zero-initialised unsigned in local device memory.  B K-major or MN-major; N > 128; rows % 128 == 0.
// parameter all-gather inside the consuming GEMM: Y = X W^T with W [N, K] at element w_lo of a flat parameter bucket that is
// sharded over `world` ranks (`shard` elements each, peer-readable at shard_ptrs[o]); see gemm_sm100.cu
int vlmt_gemm_bf16_wgather(const void* X, void* D, const void* bias, int M, int N, int K, int ldx, int ldd, void* bucket, long w_lo,
                           const void* const* shard_ptrs, long shard, int world, int rank, int* flags, unsigned* counters, int epoch,
                           int* status, int num_sms, cudaStream_t stream);
int vlmt_gemm_bf16_ag(const void* src, void* A_full, const void* B, void* D, void* const* gathered, void* const* flag_dst,
                      const int* flags, unsigned* counter, int epoch, int world, int rank, int rows, int N, int K, int ldb, int ldd,
                      int b_mn_major, int* status, int num_sms, cudaStream_t stream);
// bound of the in-GEMM wait for a peer's flag on the current device, in milliseconds (default 20 000)
int vlmt_gemm_set_flag_wait_ms(long ms);
// 2-D bf16 tensor map with 128-byte swizzle; `out_map` points at 128 bytes (CUtensorMap).
int vlmt_make_tmap_2d_bf16(void* out_map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                           uint32_t box_inner, uint32_t box_outer);
// the same for one-byte elements (fp8 operands)
int vlmt_make_tmap_2d_u8(void* out_map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                         uint32_t box_inner, uint32_t box_outer);
// [d2][d1][d0] bf16 (d0 contiguous) with byte strides for d1 and d2 (multiples of 16); boxes are zero-filled outside the tensor
int vlmt_make_tmap_3d_bf16(void* out_map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                           uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2);
#ifdef __cplusplus
}
#endif
