// Chunk-to-chunk scan of the gated delta rule (see gdn_scan_sm100.cu for the recurrence it runs).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// x1, x2 [n_chunks, H, 64, 128] bf16; e, y [n_chunks, H, 64, 128] bf16; decay [n_chunks, H] fp32;
// ext (may be null) and states [n_chunks, H, 128, 128] bf16; ranges: n_docs pairs (first chunk, chunk count).
// head_major = 1: every tensor is [H, n_chunks, ...] instead (the tile of chunk c, head h is h * n_chunks + c).
// reverse = 0: y = e - x1 z^T, z = decay z + y^T x2;  reverse = 1: chunks visited last to first,
// y = e + x1 z^T, z = ext + decay z - y^T x2.  Returns 0 or a negative / tensor-map error code.
int vlmt_gdn_scan(const void* x1, const void* x2, const void* e, const float* decay, const void* ext, void* y, void* states,
                  const int* ranges, int n_docs, int n_chunks, int H, int head_major, int reverse, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
