// C entry points of the fused collective kernels (comm_kernels.cu).
#pragma once
#include <cuda_runtime.h>
#ifdef __cplusplus
extern "C" {
#endif
// One kernel: reduce-scatter of bf16 grads + AdamW on the local fp32 shard + all-gather of bf16 params.
// grad_ptrs / param_ptrs: `world` device pointers (one per rank, this rank's own included) to the start of the
// bucket in each rank's flat buffer.  grad_mc / param_mc: multicast (NVLS) addresses of the same bucket or null.
// [lo, hi): this rank's shard in elements relative to the bucket start, multiples of 8.
// status: the device status word (or null); when it is non-zero at kernel start (a bounded wait ran out earlier, e.g. the
// wait for this bucket's "gradients final" flags) the kernel returns without reading or writing anything.
// m, v: the Adam moments of the shard, fp32 or (state_bf16 != 0) bf16; master: fp32.
// zero_own: with world == 1, clear the gradients after they have been consumed.
int vlmt_fused_rs_adamw_ag(void* const* grad_ptrs, void* const* param_ptrs, void* grad_mc, void* param_mc, int world, long lo, long hi,
                           float* master, void* m, void* v, int state_bf16, float lr, float b1, float b2, float eps, float wd, float bc1,
                           float bc2, float grad_scale, int zero_own, const int* status, cudaStream_t st);
// The same step split in two for gradient clipping.  Pass 1: red[0 : hi - lo] (fp32) = sum over ranks of the gradients of this
// rank's shard, *sumsq += sum red^2.  Pass 2 (after the ranks' partial sums of squares have been added up into *sumsq):
// AdamW from `red` with the gradients scaled by grad_scale * min(1, max_norm / (grad_scale * sqrt(*sumsq) + 1e-6)), new
// parameters stored to every rank.  Both return at once when *status is non-zero.
int vlmt_rs_reduce_sumsq(void* const* grad_ptrs, void* grad_mc, int world, long lo, long hi, float* red, float* sumsq, const int* status,
                         cudaStream_t st);
int vlmt_adamw_push(const float* red, const float* sumsq, float max_norm, void* const* param_ptrs, void* param_mc, int world, long lo,
                    long hi, float* master, void* m, void* v, int state_bf16, float lr, float b1, float b2, float eps, float wd, float bc1,
                    float bc2, float grad_scale, const int* status, cudaStream_t st);
// out[rows, D] = residual + sum over ranks of partial_r[row0 : row0 + rows, :]
int vlmt_peer_sum_rows(void* const* partial_ptrs, int world, long row0, long rows, int D, const void* residual, void* out, cudaStream_t st);
// Signalled peer-to-peer collectives over symmetric staging slots (protocol: comm_kernels.cu).
// flag_ptrs[r]: address of rank r's int32 flag array (length >= world); my_flags: this rank's own array.
// bound of every flag wait on the current device, in milliseconds (default 20 000)
int vlmt_set_flag_wait_ms(long ms);
int vlmt_signal_peers(void* const* flag_ptrs, int world, int my_rank, int epoch, cudaStream_t st);
// one-block kernel that returns once my_flags[r] >= epoch for every r < world except skip_rank (-1: none);
// bounded wait, status word on timeout
int vlmt_wait_flags(const int* my_flags, int world, int epoch, int skip_rank, int* status, cudaStream_t st);
// out[r*n:(r+1)*n] = rank r's slot (bf16 elements); waits (bounded) for every rank's signal `epoch`
int vlmt_pull_gather(void* const* slot_ptrs, void* out, long n_per_rank, int world, const int* my_flags, int epoch, int* status,
                     cudaStream_t st);
// the same for the elements [lo, hi) of the gathered array only (multiples of 8); no flags
int vlmt_pull_gather_range(void* const* slot_ptrs, void* out, long n_per_rank, int world, long lo, long hi, cudaStream_t st);
// out[0:n] = residual + sum_r slot_r[me*n:(me+1)*n]
int vlmt_pull_reduce(void* const* slot_ptrs, void* out, const void* residual, long n_per_rank, int world, int my_rank,
                     const int* my_flags, int epoch, int* status, cudaStream_t st);
#ifdef __cplusplus
}
#endif
