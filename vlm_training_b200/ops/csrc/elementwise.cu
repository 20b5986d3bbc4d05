// Bandwidth-bound fused kernels (bf16 I/O, fp32 math): RMSNorm (+residual, offset form),
// LayerNorm, gated RMSNorm, SwiGLU, sigmoid gating, GELU, fused per-head QK-norm + rotary +
// layout split of the fused qkv projection, ViT rotary, Gated-DeltaNet gate prep, depthwise
// causal conv1d + SiLU over packed rows, row scatter / row add for vision features.
//
// Conventions: one warp per row for the row-reduction kernels, 16-byte vector accesses,
// weight-gradient partial sums written per block (reduced by the caller) so results are
// bit-reproducible run to run.
#include "elementwise.h"
#include "no_alloc_entry.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const bf162* p = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(p[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  bf162* p = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float ldw(const bf16* w, int i) { return __bfloat162float(w[i]); }
__device__ __forceinline__ float ldw(const float* w, int i) { return w[i]; }

constexpr int kWarpsPerBlock = 8;
constexpr int kThreads = kWarpsPerBlock * 32;

// ----------------------------------------------------------------------------------- RMSNorm forward
// y = x * rstd * (w or 1+w);  optional residual: r = x + res is written out and normalised.
template <typename WT>
__global__ void rmsnorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res, const WT* __restrict__ w,
                                   bf16* __restrict__ y, bf16* __restrict__ r_out, float* __restrict__ rstd, int rows, int D,
                                   float eps, int offset) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;
  for (int row = blockIdx.x * kWarpsPerBlock + warp; row < rows; row += gridDim.x * kWarpsPerBlock) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
    const uint4* rr = res ? reinterpret_cast<const uint4*>(res + (size_t)row * D) : nullptr;
    uint4* ro = r_out ? reinterpret_cast<uint4*>(r_out + (size_t)row * D) : nullptr;
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      unpack8(xr[v], f);
      if (rr) {
        float g[8];
        unpack8(rr[v], g);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] += g[i];
        uint4 pk = pack8(f);
        ro[v] = pk;
        unpack8(pk, f);  // normalise the rounded residual stream, as the unfused sequence does
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / (float)D + eps);
    if (lane == 0 && rstd) rstd[row] = rs;
    const uint4* src = rr ? reinterpret_cast<const uint4*>(r_out + (size_t)row * D) : xr;
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * D);
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      unpack8(src[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float wv = ldw(w, v * 8 + i);
        f[i] = f[i] * rs * (offset ? 1.f + wv : wv);
      }
      yr[v] = pack8(f);
    }
  }
}

// ----------------------------------------------------------------------------------- RMSNorm backward
// dx = rstd * (g - xhat * mean(g * xhat)) (+ dres),  g = dy * w';   dw_partial[block] += dy * xhat
template <typename WT>
__global__ void rmsnorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const WT* __restrict__ w,
                                   const float* __restrict__ rstd, const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                   float* __restrict__ dw_partial, int rows, int D, int offset) {
  extern __shared__ float sm_dw[];  // [kWarpsPerBlock][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int nvec = D >> 3;
  float* my_dw = sm_dw + (size_t)warp * D;
  for (int i = lane; i < D; i += 32) my_dw[i] = 0.f;
  __syncwarp();
  for (int row = blockIdx.x * nwarps + warp; row < rows; row += gridDim.x * nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * D);
    const float rs = rstd[row];
    float dot = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float xf[8], gf[8];
      unpack8(xr[v], xf);
      unpack8(gr[v], gf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float wv = ldw(w, v * 8 + i);
        wv = offset ? 1.f + wv : wv;
        const float xh = xf[i] * rs;
        dot += gf[i] * wv * xh;
        my_dw[v * 8 + i] += gf[i] * xh;
      }
    }
    dot = warp_sum(dot) / (float)D;
    const uint4* dr = dres ? reinterpret_cast<const uint4*>(dres + (size_t)row * D) : nullptr;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * D);
    for (int v = lane; v < nvec; v += 32) {
      float xf[8], gf[8], o[8];
      unpack8(xr[v], xf);
      unpack8(gr[v], gf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float wv = ldw(w, v * 8 + i);
        wv = offset ? 1.f + wv : wv;
        o[i] = rs * (gf[i] * wv - xf[i] * rs * dot);
      }
      if (dr) {
        float e[8];
        unpack8(dr[v], e);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += e[i];
      }
      dxr[v] = pack8(o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = 0.f;
for (int wi = 0; wi < nwarps; ++wi) s += sm_dw[(size_t)wi * D + i];
    dw_partial[(size_t)blockIdx.x * D + i] = s;
  }
}

// ----------------------------------------------------------------------------------- LayerNorm
__global__ void layernorm_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, const bf16* __restrict__ b,
                                     bf16* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int rows, int D,
                                     float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = D >> 3;
  for (int row = blockIdx.x * kWarpsPerBlock + warp; row < rows; row += gridDim.x * kWarpsPerBlock) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
    float s = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      unpack8(xr[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += f[i];
    }
    const float mu = warp_sum(s) / (float)D;
    float ss = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      unpack8(xr[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) { const float d = f[i] - mu; ss += d * d; }
    }
    const float rs = rsqrtf(warp_sum(ss) / (float)D + eps);
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * D);
    for (int v = lane; v < nvec; v += 32) {
      float f[8];
      unpack8(xr[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = (f[i] - mu) * rs * ldw(w, v * 8 + i) + (b ? ldw(b, v * 8 + i) : 0.f);
      yr[v] = pack8(f);
    }
  }
}

// dx = rstd * (g - mean(g) - xhat * mean(g * xhat)), g = dy * w; partial dw, db per block
__global__ void layernorm_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ w,
                                     const float* __restrict__ mean, const float* __restrict__ rstd, bf16* __restrict__ dx,
                                     float* __restrict__ dw_partial, float* __restrict__ db_partial, int rows, int D) {
  extern __shared__ float sm_acc[];  // [kWarpsPerBlock][2][D]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  const int nvec = D >> 3;
  float* my_dw = sm_acc + (size_t)warp * 2 * D;
  float* my_db = my_dw + D;
  for (int i = lane; i < 2 * D; i += 32) my_dw[i] = 0.f;
  __syncwarp();
  for (int row = blockIdx.x * nwarps + warp; row < rows; row += gridDim.x * nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * D);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * D);
    const float mu = mean[row], rs = rstd[row];
    float s1 = 0.f, s2 = 0.f;
    for (int v = lane; v < nvec; v += 32) {
      float xf[8], gf[8];
      unpack8(xr[v], xf);
      unpack8(gr[v], gf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (xf[i] - mu) * rs;
        const float g = gf[i] * ldw(w, v * 8 + i);
        s1 += g;
        s2 += g * xh;
        my_dw[v * 8 + i] += gf[i] * xh;
        my_db[v * 8 + i] += gf[i];
      }
    }
    s1 = warp_sum(s1) / (float)D;
    s2 = warp_sum(s2) / (float)D;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * D);
    for (int v = lane; v < nvec; v += 32) {
      float xf[8], gf[8], o[8];
      unpack8(xr[v], xf);
      unpack8(gr[v], gf);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float xh = (xf[i] - mu) * rs;
        o[i] = rs * (gf[i] * ldw(w, v * 8 + i) - s1 - xh * s2);
      }
      dxr[v] = pack8(o);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float a = 0.f, c = 0.f;
for (int wi = 0; wi < nwarps; ++wi) { a += sm_acc[(size_t)wi * 2 * D + i]; c += sm_acc[(size_t)wi * 2 * D + D + i]; }
    dw_partial[(size_t)blockIdx.x * D + i] = a;
    db_partial[(size_t)blockIdx.x * D + i] = c;
  }
}

// ----------------------------------------------------------------------------------- row-tile norm kernels
// The kernels above give a warp a whole row (re-reading it for every pass and, in backward, accumulating the weight
// gradient through shared memory); they measured 16-40 % of copy bandwidth.  The row-tile forms below are used whenever
// D <= 8192: a block of up to 256 threads works on a group of rows at a time, every thread owns the same VPT 8-element
// column groups of every row, so the rows stay in registers between the passes, the weights are loaded once per thread,
// and the weight gradient of a thread's columns accumulates in its own registers (no shared memory, no cross-warp sum).
//
// The inputs stream through a ring of kPipe stages in shared memory.  A stage holds the rows of one group for every input
// tensor; a thread copies (cp.async) exactly the 16-byte vectors it will read itself, so the ring needs no barrier.  While
// a block sums, computes and stores group g, the copies of the next kPipe - 1 groups are in flight: a block keeps the
// memory system busy all the time instead of alternating between a load phase and a store phase (the version that loaded
// straight into registers reached 0.33-0.48 of copy bandwidth on 8192 x 4096).
constexpr int kRT = 256;   // threads per block
constexpr int kRR = 4;     // most rows per group (sizes the scratch of the block-wide sums)
constexpr int kPipe = 3;   // stages of the copy ring

// rows per group: four for narrow rows (one column group per thread), one where a thread owns several column groups of a row
template <int VPT> struct TileRows { static constexpr int value = VPT == 1 ? 4 : 1; };

__device__ __forceinline__ void cp16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// slot of (stage, tensor) inside the ring: RR rows of nvec vectors
template <int RR>
__device__ __forceinline__ uint4* ring_slot(uint4* ring, int stage, int tensor, int n_tensors, int nvec) {
  return ring + (size_t)(stage * n_tensors + tensor) * RR * nvec;
}
// start the copies of this thread's vectors of group g (nothing for rows or columns outside the matrix)
template <int RR, int VPT>
__device__ __forceinline__ void ring_issue(uint4* slot, const bf16* __restrict__ src, int g, int rows, int nvec) {
#pragma unroll
  for (int r = 0; r < RR; ++r) {
    const int row = g * RR + r;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * (int)blockDim.x;
      if (row < rows && v < nvec) cp16(slot + r * nvec + v, reinterpret_cast<const uint4*>(src) + (size_t)row * nvec + v);
    }
  }
}
// this thread's vectors of group g out of a finished stage; positions outside the matrix read as zeros
template <int RR, int VPT>
__device__ __forceinline__ void ring_read(const uint4* slot, int g, int rows, int nvec, uint4 (&dst)[RR][VPT]) {
#pragma unroll
  for (int r = 0; r < RR; ++r) {
    const int row = g * RR + r;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = threadIdx.x + k * (int)blockDim.x;
      dst[r][k] = (row < rows && v < nvec) ? slot[r * nvec + v] : make_uint4(0u, 0u, 0u, 0u);
    }
  }
}

// Sum K per-thread values over the block; every thread gets the totals.  `sm` holds 2 x K x 8 floats and is used
// alternately (`parity`), which makes one __syncthreads per call sufficient.
template <int K>
__device__ __forceinline__ void block_sum(float (&v)[K], float* sm, int& parity) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* buf = sm + parity * K * 8;
#pragma unroll
  for (int k = 0; k < K; ++k) v[k] = warp_sum(v[k]);
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < K; ++k) buf[k * 8 + warp] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < K; ++k) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += buf[k * 8 + w];   // blocks may be narrower than kRT
    v[k] = t;
  }
  parity ^= 1;
}
__device__ __forceinline__ void ld_w8(const bf16* w, int v, float (&f)[8]) { unpack8(reinterpret_cast<const uint4*>(w)[v], f); }
__device__ __forceinline__ void ld_w8(const float* w, int v, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(w)[2 * v], b = reinterpret_cast<const float4*>(w)[2 * v + 1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}

template <typename WT, int VPT>
__global__ void __launch_bounds__(kRT) rmsnorm_fwd_tile_kernel(const bf16* __restrict__ x, const bf16* __restrict__ res,
                                                              const WT* __restrict__ w, bf16* __restrict__ y, bf16* __restrict__ r_out,
                                                              float* __restrict__ rstd, int rows, int D, float eps, int offset) {
  constexpr int RR = TileRows<VPT>::value;
  extern __shared__ uint4 ring[];
  __shared__ float sm[2 * kRR * 8];
  const int nvec = D >> 3;
  const int nt = res ? 2 : 1;
  float wv[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * (int)blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) wv[k][i] = 0.f;
    if (v < nvec) {
      ld_w8(w, v, wv[k]);
      if (offset) {
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[k][i] += 1.f;
      }
    }
  }
  int parity = 0;
  const int n_groups = (rows + RR - 1) / RR;
  auto issue = [&](int g, int stage) {
    if (g < n_groups) {
      ring_issue<RR, VPT>(ring_slot<RR>(ring, stage, 0, nt, nvec), x, g, rows, nvec);
      if (res) ring_issue<RR, VPT>(ring_slot<RR>(ring, stage, 1, nt, nvec), res, g, rows, nvec);
    }
    cp_commit();   // one group per call, empty or not: the wait below counts groups
  };
#pragma unroll
  for (int s = 0; s < kPipe; ++s) issue(blockIdx.x + s * gridDim.x, s);
  int stage = 0;
  for (int g = blockIdx.x; g < n_groups; g += gridDim.x) {
    cp_wait<kPipe - 1>();
    uint4 xv[RR][VPT], ev[RR][VPT];
    ring_read<RR, VPT>(ring_slot<RR>(ring, stage, 0, nt, nvec), g, rows, nvec, xv);
    if (res) ring_read<RR, VPT>(ring_slot<RR>(ring, stage, 1, nt, nvec), g, rows, nvec, ev);
    float ss[RR];
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      ss[r] = 0.f;
      const int row = g * RR + r;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = threadIdx.x + k * (int)blockDim.x;
        float f[8];
        unpack8(xv[r][k], f);
        if (res) {
          float e[8];
          unpack8(ev[r][k], e);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] += e[i];
          xv[r][k] = pack8(f);
          if (row < rows && v < nvec) reinterpret_cast<uint4*>(r_out)[(size_t)row * nvec + v] = xv[r][k];
          unpack8(xv[r][k], f);  // normalise the rounded residual stream, as the unfused sequence does
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss[r] += f[i] * f[i];
      }
    }
    block_sum<RR>(ss, sm, parity);
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      const int row = g * RR + r;
      if (row >= rows) continue;
      const float rs = rsqrtf(ss[r] / (float)D + eps);
      if (threadIdx.x == 0 && rstd) rstd[row] = rs;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = threadIdx.x + k * (int)blockDim.x;
        if (v < nvec) {
          float f[8];
          unpack8(xv[r][k], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = f[i] * rs * wv[k][i];
          reinterpret_cast<uint4*>(y)[(size_t)row * nvec + v] = pack8(f);
        }
      }
    }
    issue(g + kPipe * gridDim.x, stage);   // the stage just read is free again (only this thread touches its slots)
    stage = stage + 1 == kPipe ? 0 : stage + 1;
  }
  cp_wait<0>();
}

template <typename WT, int VPT>
__global__ void __launch_bounds__(kRT) rmsnorm_bwd_tile_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                              const WT* __restrict__ w, const float* __restrict__ rstd,
                                                              const bf16* __restrict__ dres, bf16* __restrict__ dx,
                                                              float* __restrict__ dw_partial, int rows, int D, int offset) {
  constexpr int RR = TileRows<VPT>::value;
  extern __shared__ uint4 ring[];
  __shared__ float sm[2 * kRR * 8];
  const int nvec = D >> 3;
  const int nt = dres ? 3 : 2;
  float wv[VPT][8], dw[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * (int)blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) { dw[k][i] = 0.f; wv[k][i] = 0.f; }
    if (v < nvec) {
      ld_w8(w, v, wv[k]);
      if (offset) {
#pragma unroll
        for (int i = 0; i < 8; ++i) wv[k][i] += 1.f;
      }
    }
  }
  int parity = 0;
  const int n_groups = (rows + RR - 1) / RR;
  auto issue = [&](int g, int stage) {
    if (g < n_groups) {
      ring_issue<RR, VPT>(ring_slot<RR>(ring, stage, 0, nt, nvec), x, g, rows, nvec);
      ring_issue<RR, VPT>(ring_slot<RR>(ring, stage, 1, nt, nvec), dy, g, rows, nvec);
      if (dres) ring_issue<RR, VPT>(ring_slot<RR>(ring, stage, 2, nt, nvec), dres, g, rows, nvec);
    }
    cp_commit();
  };
#pragma unroll
  for (int s = 0; s < kPipe; ++s) issue(blockIdx.x + s * gridDim.x, s);
  int stage = 0;
  for (int g = blockIdx.x; g < n_groups; g += gridDim.x) {
    cp_wait<kPipe - 1>();
    uint4 xv[RR][VPT], gv[RR][VPT];
    ring_read<RR, VPT>(ring_slot<RR>(ring, stage, 0, nt, nvec), g, rows, nvec, xv);
    ring_read<RR, VPT>(ring_slot<RR>(ring, stage, 1, nt, nvec), g, rows, nvec, gv);
    float dot[RR], rs[RR];
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      dot[r] = 0.f;
      const int row = g * RR + r;
      rs[r] = row < rows ? rstd[row] : 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        float xf[8], gf[8];
        unpack8(xv[r][k], xf);
        unpack8(gv[r][k], gf);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = xf[i] * rs[r];
          dot[r] += gf[i] * wv[k][i] * xh;
          dw[k][i] += gf[i] * xh;
        }
      }
    }
    block_sum<RR>(dot, sm, parity);
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      const int row = g * RR + r;
      if (row >= rows) continue;
      const float dt = dot[r] / (float)D;
      const uint4* dslot = ring_slot<RR>(ring, stage, 2, nt, nvec);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = threadIdx.x + k * (int)blockDim.x;
        if (v < nvec) {
          float xf[8], gf[8], out[8];
          unpack8(xv[r][k], xf);
          unpack8(gv[r][k], gf);
#pragma unroll
          for (int i = 0; i < 8; ++i) out[i] = rs[r] * (gf[i] * wv[k][i] - xf[i] * rs[r] * dt);
          if (dres) {
            float e[8];
            unpack8(dslot[r * nvec + v], e);
#pragma unroll
            for (int i = 0; i < 8; ++i) out[i] += e[i];
          }
          reinterpret_cast<uint4*>(dx)[(size_t)row * nvec + v] = pack8(out);
        }
      }
    }
    issue(g + kPipe * gridDim.x, stage);
    stage = stage + 1 == kPipe ? 0 : stage + 1;
  }
  cp_wait<0>();
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * (int)blockDim.x;
    if (v < nvec) {
      float4* dst = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * D + (size_t)v * 8);
      dst[0] = make_float4(dw[k][0], dw[k][1], dw[k][2], dw[k][3]);
      dst[1] = make_float4(dw[k][4], dw[k][5], dw[k][6], dw[k][7]);
    }
  }
}

template <int VPT>
__global__ void __launch_bounds__(kRT) layernorm_fwd_tile_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                const bf16* __restrict__ b, bf16* __restrict__ y,
                                                                float* __restrict__ mean, float* __restrict__ rstd, int rows, int D,
                                                                float eps) {
  constexpr int RR = TileRows<VPT>::value;
  extern __shared__ uint4 ring[];
  __shared__ float sm[2 * kRR * 8];
  const int nvec = D >> 3;
  float wv[VPT][8], bv[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * (int)blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) { bv[k][i] = 0.f; wv[k][i] = 0.f; }
    if (v < nvec) {
      ld_w8(w, v, wv[k]);
      if (b) ld_w8(b, v, bv[k]);
    }
  }
  int parity = 0;
  const int n_groups = (rows + RR - 1) / RR;
  auto issue = [&](int g, int stage) {
    if (g < n_groups) ring_issue<RR, VPT>(ring_slot<RR>(ring, stage, 0, 1, nvec), x, g, rows, nvec);
    cp_commit();
  };
#pragma unroll
  for (int s = 0; s < kPipe; ++s) issue(blockIdx.x + s * gridDim.x, s);
  int stage = 0;
  for (int g = blockIdx.x; g < n_groups; g += gridDim.x) {
    cp_wait<kPipe - 1>();
    uint4 xv[RR][VPT];
    ring_read<RR, VPT>(ring_slot<RR>(ring, stage, 0, 1, nvec), g, rows, nvec, xv);
    float s[RR];
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      s[r] = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        float f[8];
        unpack8(xv[r][k], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) s[r] += f[i];
      }
    }
    block_sum<RR>(s, sm, parity);
    float ss[RR];
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      s[r] /= (float)D;  // mean
      ss[r] = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = threadIdx.x + k * (int)blockDim.x;
        if (v < nvec) {
          float f[8];
          unpack8(xv[r][k], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) { const float d = f[i] - s[r]; ss[r] += d * d; }
        }
      }
    }
    block_sum<RR>(ss, sm, parity);
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      const int row = g * RR + r;
      if (row >= rows) continue;
      const float mu = s[r], rs = rsqrtf(ss[r] / (float)D + eps);
      if (threadIdx.x == 0) { mean[row] = mu; rstd[row] = rs; }
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = threadIdx.x + k * (int)blockDim.x;
        if (v < nvec) {
          float f[8];
          unpack8(xv[r][k], f);
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = (f[i] - mu) * rs * wv[k][i] + bv[k][i];
          reinterpret_cast<uint4*>(y)[(size_t)row * nvec + v] = pack8(f);
        }
      }
    }
    issue(g + kPipe * gridDim.x, stage);
    stage = stage + 1 == kPipe ? 0 : stage + 1;
  }
  cp_wait<0>();
}

template <int VPT>
__global__ void __launch_bounds__(kRT) layernorm_bwd_tile_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x,
                                                                const bf16* __restrict__ w, const float* __restrict__ mean,
                                                                const float* __restrict__ rstd, bf16* __restrict__ dx,
                                                                float* __restrict__ dw_partial, float* __restrict__ db_partial, int rows,
                                                                int D) {
  constexpr int RR = TileRows<VPT>::value;
  extern __shared__ uint4 ring[];
  __shared__ float sm[2 * 2 * kRR * 8];
  const int nvec = D >> 3;
  float wv[VPT][8], dw[VPT][8], db[VPT][8];
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * (int)blockDim.x;
#pragma unroll
    for (int i = 0; i < 8; ++i) { dw[k][i] = 0.f; db[k][i] = 0.f; wv[k][i] = 0.f; }
    if (v < nvec) ld_w8(w, v, wv[k]);
  }
  int parity = 0;
  const int n_groups = (rows + RR - 1) / RR;
  auto issue = [&](int g, int stage) {
    if (g < n_groups) {
      ring_issue<RR, VPT>(ring_slot<RR>(ring, stage, 0, 2, nvec), x, g, rows, nvec);
      ring_issue<RR, VPT>(ring_slot<RR>(ring, stage, 1, 2, nvec), dy, g, rows, nvec);
    }
    cp_commit();
  };
#pragma unroll
  for (int s = 0; s < kPipe; ++s) issue(blockIdx.x + s * gridDim.x, s);
  int stage = 0;
  for (int g = blockIdx.x; g < n_groups; g += gridDim.x) {
    cp_wait<kPipe - 1>();
    uint4 xv[RR][VPT], gv[RR][VPT];
    ring_read<RR, VPT>(ring_slot<RR>(ring, stage, 0, 2, nvec), g, rows, nvec, xv);
    ring_read<RR, VPT>(ring_slot<RR>(ring, stage, 1, 2, nvec), g, rows, nvec, gv);
    float s12[2 * RR], mu[RR], rs[RR];
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      s12[2 * r] = s12[2 * r + 1] = 0.f;
      const int row = g * RR + r;
      mu[r] = row < rows ? mean[row] : 0.f;
      rs[r] = row < rows ? rstd[row] : 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = threadIdx.x + k * (int)blockDim.x;
        if (row < rows && v < nvec) {
          float xf[8], gf[8];
          unpack8(xv[r][k], xf);
          unpack8(gv[r][k], gf);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float xh = (xf[i] - mu[r]) * rs[r];
            const float gw = gf[i] * wv[k][i];
            s12[2 * r] += gw;
            s12[2 * r + 1] += gw * xh;
            dw[k][i] += gf[i] * xh;
            db[k][i] += gf[i];
          }
        }
      }
    }
    block_sum<2 * RR>(s12, sm, parity);
#pragma unroll
    for (int r = 0; r < RR; ++r) {
      const int row = g * RR + r;
      if (row >= rows) continue;
      const float s1 = s12[2 * r] / (float)D, s2 = s12[2 * r + 1] / (float)D;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = threadIdx.x + k * (int)blockDim.x;
        if (v < nvec) {
          float xf[8], gf[8], out[8];
          unpack8(xv[r][k], xf);
          unpack8(gv[r][k], gf);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float xh = (xf[i] - mu[r]) * rs[r];
            out[i] = rs[r] * (gf[i] * wv[k][i] - s1 - xh * s2);
          }
          reinterpret_cast<uint4*>(dx)[(size_t)row * nvec + v] = pack8(out);
        }
      }
    }
    issue(g + kPipe * gridDim.x, stage);
    stage = stage + 1 == kPipe ? 0 : stage + 1;
  }
  cp_wait<0>();
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int v = threadIdx.x + k * (int)blockDim.x;
    if (v < nvec) {
      float4* d1 = reinterpret_cast<float4*>(dw_partial + (size_t)blockIdx.x * D + (size_t)v * 8);
      float4* d2 = reinterpret_cast<float4*>(db_partial + (size_t)blockIdx.x * D + (size_t)v * 8);
      d1[0] = make_float4(dw[k][0], dw[k][1], dw[k][2], dw[k][3]);
      d1[1] = make_float4(dw[k][4], dw[k][5], dw[k][6], dw[k][7]);
      d2[0] = make_float4(db[k][0], db[k][1], db[k][2], db[k][3]);
      d2[1] = make_float4(db[k][4], db[k][5], db[k][6], db[k][7]);
    }
  }
}

// ----------------------------------------------------------------------------------- LayerNorm forward, one warp per row
// Rows of 776 to 1280 channels (the ViT's 1152).  The row-tile kernels spend about 200 instructions per thread and row
// on eight elements there (three conversions of the same vector, two block-wide sums with a barrier each) and are bound
// by instruction issue at a quarter of the memory bandwidth.  Here a warp owns a whole row: lane l holds the vectors
// l, l + 32, ... (VL of them) as floats, both sums are five shuffles, the weights are read from shared memory, and the
// rows arrive through the same kind of per-thread `cp.async` ring (every lane copies exactly the vectors it reads itself).
// 28672 x 1152: 0.0349 ms against 0.0451 ms.  The backward pass stays on the row-tile kernel: a warp-per-row form needs
// 2 x VL x 8 gradient accumulators per lane (184 registers, two blocks of four warps per SM) and measured 0.097 ms against
// 0.083 ms.
constexpr int kLnWarpsFwd = 8, kLnPipeFwd = 3;

template <int VL>
__global__ void __launch_bounds__(kLnWarpsFwd * 32) layernorm_fwd_warp_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w,
                                                                             const bf16* __restrict__ b, bf16* __restrict__ y,
                                                                             float* __restrict__ mean, float* __restrict__ rstd, int rows,
                                                                             int D, float eps) {
  extern __shared__ uint4 dyn[];
  float* sw = reinterpret_cast<float*>(dyn);        // weights and bias as floats, [D] each
  float* sb = sw + D;
  uint4* ring = reinterpret_cast<uint4*>(sb + D);   // [warp][stage][nvec]
  const int nvec = D >> 3, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    sw[i] = __bfloat162float(w[i]);
    sb[i] = b ? __bfloat162float(b[i]) : 0.f;
  }
  __syncthreads();
  uint4* my = ring + (size_t)warp * kLnPipeFwd * nvec;
  const int row_step = gridDim.x * kLnWarpsFwd;
  auto issue = [&](int row, int stage) {
    if (row < rows) {
#pragma unroll
      for (int k = 0; k < VL; ++k) {
        const int v = lane + 32 * k;
        if (v < nvec) cp16(my + stage * nvec + v, reinterpret_cast<const uint4*>(x) + (size_t)row * nvec + v);
      }
    }
    cp_commit();   // one group per call, empty or not: the wait below counts groups
  };
  const int row0 = blockIdx.x * kLnWarpsFwd + warp;
#pragma unroll
  for (int s = 0; s < kLnPipeFwd; ++s) issue(row0 + s * row_step, s);
  int stage = 0;
  for (int row = row0; row < rows; row += row_step) {
    cp_wait<kLnPipeFwd - 1>();
    float f[VL][8];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < VL; ++k) {
      const int v = lane + 32 * k;
      if (v < nvec) {
        unpack8(my[stage * nvec + v], f[k]);
#pragma unroll
        for (int i = 0; i < 8; ++i) s += f[k][i];
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[k][i] = 0.f;
      }
    }
    const float mu = warp_sum(s) / (float)D;
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VL; ++k) {
      if (lane + 32 * k < nvec) {
#pragma unroll
        for (int i = 0; i < 8; ++i) { f[k][i] -= mu; ss += f[k][i] * f[k][i]; }
      }
    }
    const float rs = rsqrtf(warp_sum(ss) / (float)D + eps);
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
#pragma unroll
    for (int k = 0; k < VL; ++k) {
      const int v = lane + 32 * k;
      if (v < nvec) {
        const float4 w0 = *reinterpret_cast<const float4*>(sw + v * 8), w1 = *reinterpret_cast<const float4*>(sw + v * 8 + 4);
        const float4 b0 = *reinterpret_cast<const float4*>(sb + v * 8), b1 = *reinterpret_cast<const float4*>(sb + v * 8 + 4);
        const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        const float bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
        float o[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = f[k][i] * rs * wv[i] + bv[i];
        reinterpret_cast<uint4*>(y)[(size_t)row * nvec + v] = pack8(o);
      }
    }
    issue(row + kLnPipeFwd * row_step, stage);   // the stage just read is free again (only this lane touches its slots)
    stage = stage + 1 == kLnPipeFwd ? 0 : stage + 1;
  }
  cp_wait<0>();
}

// ----------------------------------------------------------------------------------- gated RMSNorm (GDN output)
// y = x * rstd * w * z * sigmoid(z), rows of D (<= 256), one warp per row
__global__ void rmsnorm_gated_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ z, const bf16* __restrict__ w,
                                         bf16* __restrict__ y, float* __restrict__ rstd, int rows, int D, float eps) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row = blockIdx.x * kWarpsPerBlock + warp; row < rows; row += gridDim.x * kWarpsPerBlock) {
    float ss = 0.f;
    for (int i = lane; i < D; i += 32) { const float f = __bfloat162float(x[(size_t)row * D + i]); ss += f * f; }
    const float rs = rsqrtf(warp_sum(ss) / (float)D + eps);
    if (lane == 0) rstd[row] = rs;
    for (int i = lane; i < D; i += 32) {
      const float f = __bfloat162float(x[(size_t)row * D + i]);
      const float zz = __bfloat162float(z[(size_t)row * D + i]);
      y[(size_t)row * D + i] = __float2bfloat16(f * rs * ldw(w, i) * zz * sigmoidf_(zz));
    }
  }
}
__global__ void rmsnorm_gated_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, const bf16* __restrict__ z,
                                         const bf16* __restrict__ w, const float* __restrict__ rstd, bf16* __restrict__ dx,
                                         bf16* __restrict__ dz, float* __restrict__ dw_partial, int rows, int D) {
  extern __shared__ float sm_dw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nwarps = blockDim.x >> 5;
  float* my_dw = sm_dw + (size_t)warp * D;
  for (int i = lane; i < D; i += 32) my_dw[i] = 0.f;
  __syncwarp();
  for (int row = blockIdx.x * nwarps + warp; row < rows; row += gridDim.x * nwarps) {
    const float rs = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < D; i += 32) {
      const size_t o = (size_t)row * D + i;
      const float xh = __bfloat162float(x[o]) * rs, zz = __bfloat162float(z[o]), g = __bfloat162float(dy[o]);
      const float sg = sigmoidf_(zz), act = zz * sg;
      const float gn = g * act;  // grad wrt normalised*weight
      dot += gn * ldw(w, i) * xh;
      my_dw[i] += gn * xh;
      dz[o] = __float2bfloat16(g * xh * ldw(w, i) * (sg + act * (1.f - sg)));
    }
    dot = warp_sum(dot) / (float)D;
    for (int i = lane; i < D; i += 32) {
      const size_t o = (size_t)row * D + i;
      const float xh = __bfloat162float(x[o]) * rs, zz = __bfloat162float(z[o]), g = __bfloat162float(dy[o]);
      const float gn = g * zz * sigmoidf_(zz);
      dx[o] = __float2bfloat16(rs * (gn * ldw(w, i) - xh * dot));
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < D; i += blockDim.x) {
    float s = 0.f;
for (int wi = 0; wi < nwarps; ++wi) s += sm_dw[(size_t)wi * D + i];
    dw_partial[(size_t)blockIdx.x * D + i] = s;
  }
}

// ----------------------------------------------------------------------------------- SwiGLU
__global__ void swiglu_fwd_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, long rows, int I) {
  const long nvec = rows * (I >> 3);
  const int vper = I >> 3;
  for (long v = blockIdx.x * (long)blockDim.x + threadIdx.x; v < nvec; v += (long)gridDim.x * blockDim.x) {
    const long row = v / vper;
    const int c = (int)(v - row * vper);
    const uint4* base = reinterpret_cast<const uint4*>(gu + row * 2 * (long)I);
    float g[8], u[8], o[8];
    unpack8(base[c], g);
    unpack8(base[vper + c], u);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = g[i] * sigmoidf_(g[i]) * u[i];
    reinterpret_cast<uint4*>(out)[v] = pack8(o);
  }
}
__global__ void swiglu_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ gu, bf16* __restrict__ dgu, long rows,
                                  int I) {
  const long nvec = rows * (I >> 3);
  const int vper = I >> 3;
  for (long v = blockIdx.x * (long)blockDim.x + threadIdx.x; v < nvec; v += (long)gridDim.x * blockDim.x) {
    const long row = v / vper;
    const int c = (int)(v - row * vper);
    const uint4* base = reinterpret_cast<const uint4*>(gu + row * 2 * (long)I);
    uint4* obase = reinterpret_cast<uint4*>(dgu + row * 2 * (long)I);
    float g[8], u[8], d[8], dg[8], du[8];
    unpack8(base[c], g);
    unpack8(base[vper + c], u);
    unpack8(reinterpret_cast<const uint4*>(dout)[v], d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float s = sigmoidf_(g[i]);
      const float silu = g[i] * s;
      du[i] = d[i] * silu;
      dg[i] = d[i] * u[i] * (s + silu * (1.f - s));
    }
    obase[c] = pack8(dg);
    obase[vper + c] = pack8(du);
  }
}

// ----------------------------------------------------------------------------------- x * sigmoid(gate)
__global__ void sigmoid_mul_fwd_kernel(const bf16* __restrict__ x, const bf16* __restrict__ gate, bf16* __restrict__ out, long n8) {
  for (long v = blockIdx.x * (long)blockDim.x + threadIdx.x; v < n8; v += (long)gridDim.x * blockDim.x) {
    float a[8], g[8];
    unpack8(reinterpret_cast<const uint4*>(x)[v], a);
    unpack8(reinterpret_cast<const uint4*>(gate)[v], g);
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] *= sigmoidf_(g[i]);
    reinterpret_cast<uint4*>(out)[v] = pack8(a);
  }
}
__global__ void sigmoid_mul_bwd_kernel(const bf16* __restrict__ dout, const bf16* __restrict__ x, const bf16* __restrict__ gate,
                                       bf16* __restrict__ dx, bf16* __restrict__ dgate, long n8) {
  for (long v = blockIdx.x * (long)blockDim.x + threadIdx.x; v < n8; v += (long)gridDim.x * blockDim.x) {
    float a[8], g[8], d[8], o1[8], o2[8];
    unpack8(reinterpret_cast<const uint4*>(x)[v], a);
    unpack8(reinterpret_cast<const uint4*>(gate)[v], g);
    unpack8(reinterpret_cast<const uint4*>(dout)[v], d);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float s = sigmoidf_(g[i]);
      o1[i] = d[i] * s;
      o2[i] = d[i] * a[i] * s * (1.f - s);
    }
    reinterpret_cast<uint4*>(dx)[v] = pack8(o1);
    reinterpret_cast<uint4*>(dgate)[v] = pack8(o2);
  }
}

// ----------------------------------------------------------------------------------- GELU
__device__ __forceinline__ float gelu_f(float x, int tanh_approx) {
  if (tanh_approx) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}
__device__ __forceinline__ float gelu_grad_f(float x, int tanh_approx) {
  if (tanh_approx) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    const float t = tanhf(u);
    const float du = 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * du;
  }
  const float cdf = 0.5f * (1.f + erff(x * 0.7071067811865476f));
  return cdf + x * 0.3989422804014327f * __expf(-0.5f * x * x);
}
// four vectors per thread and iteration, all loads first: one 16-byte load in flight per thread leaves a streaming kernel
// at less than half of the memory bandwidth
__global__ void gelu_fwd_kernel(const bf16* __restrict__ x, bf16* __restrict__ y, long n8, int tanh_approx) {
  constexpr int U = 4;
  const long stride = (long)gridDim.x * blockDim.x;
  long v = blockIdx.x * (long)blockDim.x + threadIdx.x;
  for (; v + (U - 1) * stride < n8; v += U * stride) {
    uint4 r[U];
#pragma unroll
    for (int u = 0; u < U; ++u) r[u] = reinterpret_cast<const uint4*>(x)[v + u * stride];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float a[8];
      unpack8(r[u], a);
#pragma unroll
      for (int i = 0; i < 8; ++i) a[i] = gelu_f(a[i], tanh_approx);
      reinterpret_cast<uint4*>(y)[v + u * stride] = pack8(a);
    }
  }
  for (; v < n8; v += stride) {
    float a[8];
    unpack8(reinterpret_cast<const uint4*>(x)[v], a);
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = gelu_f(a[i], tanh_approx);
    reinterpret_cast<uint4*>(y)[v] = pack8(a);
  }
}
__global__ void gelu_bwd_kernel(const bf16* __restrict__ dy, const bf16* __restrict__ x, bf16* __restrict__ dx, long n8,
                                int tanh_approx) {
  constexpr int U = 4;
  const long stride = (long)gridDim.x * blockDim.x;
  long v = blockIdx.x * (long)blockDim.x + threadIdx.x;
  for (; v + (U - 1) * stride < n8; v += U * stride) {
    uint4 rx[U], rd[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      rx[u] = reinterpret_cast<const uint4*>(x)[v + u * stride];
      rd[u] = reinterpret_cast<const uint4*>(dy)[v + u * stride];
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float a[8], d[8];
      unpack8(rx[u], a);
      unpack8(rd[u], d);
#pragma unroll
      for (int i = 0; i < 8; ++i) d[i] *= gelu_grad_f(a[i], tanh_approx);
      reinterpret_cast<uint4*>(dx)[v + u * stride] = pack8(d);
    }
  }
  for (; v < n8; v += stride) {
    float a[8], d[8];
    unpack8(reinterpret_cast<const uint4*>(x)[v], a);
    unpack8(reinterpret_cast<const uint4*>(dy)[v], d);
#pragma unroll
    for (int i = 0; i < 8; ++i) d[i] *= gelu_grad_f(a[i], tanh_approx);
    reinterpret_cast<uint4*>(dx)[v] = pack8(d);
  }
}

// ----------------------------------------------------------------------------------- fused qkv split + QK-norm + rotary
// One warp per (token, head slot).  Head slots: [0, n_q) q heads, [n_q, n_q+n_kv) k heads,
// [n_q+n_kv, n_q+2 n_kv) v heads.  Lane owns E = D/32 consecutive channels; the rotate-half
// partner of channel j (< R/2) is j + R/2, held by lane + (R/2)/E.
// E consecutive bf16 (E = 1, 2, 4, 8; the address is E*2-byte aligned) <-> floats, as one memory access
template <int E> struct VecE;
template <> struct VecE<1> { using T = unsigned short; };
template <> struct VecE<2> { using T = uint32_t; };
template <> struct VecE<4> { using T = uint2; };
template <> struct VecE<8> { using T = uint4; };
template <int E>
__device__ __forceinline__ void ldE(const bf16* p, float (&f)[E]) {
  const typename VecE<E>::T raw = *reinterpret_cast<const typename VecE<E>::T*>(p);
  const bf16* h = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
  for (int i = 0; i < E; ++i) f[i] = __bfloat162float(h[i]);
}
template <int E>
__device__ __forceinline__ void stE(bf16* p, const float (&f)[E]) {
  typename VecE<E>::T raw;
  bf16* h = reinterpret_cast<bf16*>(&raw);
#pragma unroll
  for (int i = 0; i < E; ++i) h[i] = __float2bfloat16(f[i]);
  *reinterpret_cast<typename VecE<E>::T*>(p) = raw;
}
template <int E>
__device__ __forceinline__ void cpE(bf16* dst, const bf16* src) {
  *reinterpret_cast<typename VecE<E>::T*>(dst) = *reinterpret_cast<const typename VecE<E>::T*>(src);
}
// E consecutive floats starting at p[j] when the whole group lies below `limit`, else zeros (j, limit multiples of E
// when `vec`; element-wise otherwise)
template <int E>
__device__ __forceinline__ void ldF(const float* p, int j, int limit, bool vec, float (&f)[E]) {
  if (vec && E >= 2) {
    if (j < limit) {
      if constexpr (E == 2) { const float2 a = *reinterpret_cast<const float2*>(p + j); f[0] = a.x; f[1] = a.y; }
      else {
#pragma unroll
        for (int q4 = 0; q4 < E / 4; ++q4) {
          const float4 a = *reinterpret_cast<const float4*>(p + j + 4 * q4);
          f[4 * q4] = a.x; f[4 * q4 + 1] = a.y; f[4 * q4 + 2] = a.z; f[4 * q4 + 3] = a.w;
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < E; ++i) f[i] = 0.f;
    }
  } else {
#pragma unroll
    for (int i = 0; i < E; ++i) f[i] = (j + i < limit) ? p[j + i] : 0.f;
  }
}

constexpr int kQkvGroup = 12;   // heads of one token handled by one warp (the token's angles are loaded once per group)

template <int E>
__global__ void qkv_norm_rope_fwd_kernel(const bf16* __restrict__ qkv, const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                                         const float* __restrict__ cosv, const float* __restrict__ sinv, bf16* __restrict__ q,
                                         bf16* __restrict__ k, bf16* __restrict__ v, bf16* __restrict__ gate,
                                         float* __restrict__ rstd, int T, int n_q, int n_kv, int R, float eps, int offset,
                                         int gated, int has_norm) {
  constexpr int D = E * 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = n_q + 2 * n_kv;
  const int qstride = gated ? 2 * D : D;
  const int W = n_q * qstride + 2 * n_kv * D;
  const int groups = (slots + kQkvGroup - 1) / kQkvGroup;
  const long total = (long)T * groups;
  const int half = R >> 1;
  const int plane = half / E;  // partner lane distance
  const bool vec_cs = (R % E) == 0 && (R % 4) == 0;  // a lane's E angles are all inside or all outside [0, R), 16-byte aligned rows
  // A warp takes a group of heads of ONE token, so the token's angles are loaded once and stay in registers (they are four
  // times the bytes of a head); four heads per iteration, all loads first: a single 256-byte item in flight per warp leaves
  // the kernel latency-bound.
  constexpr int U = 4;
  using Raw = typename VecE<E>::T;
  for (long task = blockIdx.x * (long)kWarpsPerBlock + warp; task < total; task += (long)gridDim.x * kWarpsPerBlock) {
    const int t = (int)(task / groups);
    const int s_begin = (int)(task - (long)t * groups) * kQkvGroup, s_end = min(slots, s_begin + kQkvGroup);
    float c[E], sn[E];
    ldF<E>(cosv + (size_t)t * R, lane * E, R, vec_cs, c);
    ldF<E>(sinv + (size_t)t * R, lane * E, R, vec_cs, sn);
    const bf16* row = qkv + (size_t)t * W;
   for (int s0 = s_begin; s0 < s_end; s0 += U) {
    const bf16* src[U];
    bf16* dst[U];
    const bf16* wn[U];
    int tt[U], sl[U], kind[U];  // kind: 0 q, 1 k, 2 v, -1 none
    Raw raw[U], graw[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int s = s0 + u;
      kind[u] = -1;
      if (s >= s_end) continue;
      tt[u] = t; sl[u] = s; wn[u] = nullptr;
      if (s < n_q) { src[u] = row + s * qstride; dst[u] = q + ((size_t)t * n_q + s) * D; wn[u] = qw; kind[u] = 0; }
      else if (s < n_q + n_kv) { const int h = s - n_q; src[u] = row + n_q * qstride + h * D; dst[u] = k + ((size_t)t * n_kv + h) * D; wn[u] = kw; kind[u] = 1; }
      else { const int h = s - n_q - n_kv; src[u] = row + n_q * qstride + n_kv * D + h * D; dst[u] = v + ((size_t)t * n_kv + h) * D; kind[u] = 2; }
      raw[u] = *reinterpret_cast<const Raw*>(src[u] + lane * E);
      if (kind[u] == 0 && gated) graw[u] = *reinterpret_cast<const Raw*>(src[u] + D + lane * E);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (kind[u] < 0) continue;
      if (kind[u] == 2) {
        *reinterpret_cast<Raw*>(dst[u] + lane * E) = raw[u];
        continue;
      }
      const int t = tt[u], s = sl[u];
      if (kind[u] == 0 && gated) *reinterpret_cast<Raw*>(gate + ((size_t)t * n_q + s) * D + lane * E) = graw[u];
      float f[E];
      {
        const bf16* h = reinterpret_cast<const bf16*>(&raw[u]);
#pragma unroll
        for (int i = 0; i < E; ++i) f[i] = __bfloat162float(h[i]);
      }
      if (has_norm) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < E; ++i) ss += f[i] * f[i];
        const float rs = rsqrtf(warp_sum(ss) / (float)D + eps);
        if (lane == 0) rstd[(size_t)t * (n_q + n_kv) + s] = rs;
        float wv[E];
        ldE<E>(wn[u] + lane * E, wv);
#pragma unroll
        for (int i = 0; i < E; ++i) {
          // round to bf16 between norm and rotary like the unfused sequence of ops
          f[i] = __bfloat162float(__float2bfloat16(f[i] * rs * (offset ? 1.f + wv[i] : wv[i])));
        }
      }
      // rotary on channels [0, R)
      float o[E];
#pragma unroll
      for (int i = 0; i < E; ++i) {
        const int j = lane * E + i;
        const float partner = __shfl_xor_sync(0xffffffffu, f[i], plane);
        o[i] = j < R ? f[i] * c[i] + (j < half ? -partner : partner) * sn[i] : f[i];
      }
      stE<E>(dst[u] + lane * E, o);
    }
   }
  }
}

template <int E>
__global__ void qkv_norm_rope_bwd_kernel(const bf16* __restrict__ dq, const bf16* __restrict__ dk, const bf16* __restrict__ dv,
                                         const bf16* __restrict__ dgate, const bf16* __restrict__ qkv, const bf16* __restrict__ qw,
                                         const bf16* __restrict__ kw, const float* __restrict__ cosv, const float* __restrict__ sinv,
                                         const float* __restrict__ rstd, bf16* __restrict__ dqkv, float* __restrict__ dw_partial,
                                         int T, int n_q, int n_kv, int R, int offset, int gated, int has_norm) {
  constexpr int D = E * 32;
  __shared__ float sm_dw[kWarpsPerBlock][2][D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = n_q + 2 * n_kv;
  const int qstride = gated ? 2 * D : D;
  const int W = n_q * qstride + 2 * n_kv * D;
  const int groups = (slots + kQkvGroup - 1) / kQkvGroup;
  const long total = (long)T * groups;
  const int half = R >> 1;
  const int plane = half / E;
  const bool vec_cs = (R % E) == 0 && (R % 4) == 0;
  float acc_q[E], acc_k[E];
#pragma unroll
  for (int i = 0; i < E; ++i) acc_q[i] = acc_k[i] = 0.f;
  for (long task = blockIdx.x * (long)kWarpsPerBlock + warp; task < total; task += (long)gridDim.x * kWarpsPerBlock) {
    const int t = (int)(task / groups);
    const int s_begin = (int)(task - (long)t * groups) * kQkvGroup, s_end = min(slots, s_begin + kQkvGroup);
    float c[E], sn[E];   // the token's angles: once per group of heads
    ldF<E>(cosv + (size_t)t * R, lane * E, R, vec_cs, c);
    ldF<E>(sinv + (size_t)t * R, lane * E, R, vec_cs, sn);
    const bf16* row = qkv + (size_t)t * W;
    bf16* drow = dqkv + (size_t)t * W;
#pragma unroll 4
   for (int s = s_begin; s < s_end; ++s) {
    int kind, off;
    const bf16* g;
    const bf16* wn = nullptr;
    if (s < n_q) { kind = 0; off = s * qstride; g = dq + ((size_t)t * n_q + s) * D; wn = qw; }
    else if (s < n_q + n_kv) { kind = 1; const int h = s - n_q; off = n_q * qstride + h * D; g = dk + ((size_t)t * n_kv + h) * D; wn = kw; }
    else { kind = 2; const int h = s - n_q - n_kv; off = n_q * qstride + n_kv * D + h * D; g = dv + ((size_t)t * n_kv + h) * D; }
    if (kind == 2) {
      cpE<E>(drow + off + lane * E, g + lane * E);
      continue;
    }
    if (kind == 0 && gated) cpE<E>(drow + off + D + lane * E, dgate + ((size_t)t * n_q + s) * D + lane * E);
    // rotary transpose: dn[j] = do[j] c[j] + (j < half ? do[j+half] s[j+half] : -do[j-half] s[j-half])
    float d[E], dn[E];
    ldE<E>(g + lane * E, d);
#pragma unroll
    for (int i = 0; i < E; ++i) {
      const int j = lane * E + i;
      const float ds = d[i] * sn[i];  // sn is zero beyond R
      const float partner = __shfl_xor_sync(0xffffffffu, ds, plane);
      dn[i] = j < R ? d[i] * c[i] + (j < half ? partner : -partner) : d[i];
    }
    if (!has_norm) {
      stE<E>(drow + off + lane * E, dn);
      continue;
    }
    const float rs = rstd[(size_t)t * (n_q + n_kv) + s];
    float xh[E], wv[E], dot = 0.f;
    ldE<E>(row + off + lane * E, xh);
    ldE<E>(wn + lane * E, wv);
#pragma unroll
    for (int i = 0; i < E; ++i) {
      if (offset) wv[i] += 1.f;
      xh[i] *= rs;
      dot += dn[i] * wv[i] * xh[i];
      if (kind == 0) acc_q[i] += dn[i] * xh[i]; else acc_k[i] += dn[i] * xh[i];
    }
    dot = warp_sum(dot) / (float)D;
    float out[E];
#pragma unroll
    for (int i = 0; i < E; ++i) out[i] = rs * (dn[i] * wv[i] - xh[i] * dot);
    stE<E>(drow + off + lane * E, out);
   }
  }
#pragma unroll
  for (int i = 0; i < E; ++i) { sm_dw[warp][0][lane * E + i] = acc_q[i]; sm_dw[warp][1][lane * E + i] = acc_k[i]; }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) {
    float sacc = 0.f;
#pragma unroll
    for (int wi = 0; wi < kWarpsPerBlock; ++wi) sacc += sm_dw[wi][i / D][i % D];
    dw_partial[(size_t)blockIdx.x * 2 * D + i] = sacc;
  }
}

// ----------------------------------------------------------------------------------- ViT rotary (any even D, strided input)
// x [S, H, D] with strides (ss, hs, 1) -> contiguous out; cos/sin [S, D] fp32; transpose=1 gives the backward map.
// the same rotation on groups of 4 channels (8-byte bf16 accesses, 16-byte angle loads): needs D/2, every stride and
// every base address to be multiples of 4 elements
// IdxT: unsigned (the usual case: S * H * D / 8 items fit 32 bits, and the index arithmetic is three cheap 32-bit divisions
// instead of three 64-bit ones, which cost more than the rest of the loop body) or long
template <typename IdxT>
__global__ void rope_generic_vec4_kernel(const bf16* __restrict__ x, long ss, long hs, const float* __restrict__ cosv,
                                         const float* __restrict__ sinv, bf16* __restrict__ out, long oss, long ohs, int S, int H, int D,
                                         int transpose) {
  const int half = D >> 1;
  const IdxT hq = (IdxT)(half >> 2), nh = (IdxT)H;
  const IdxT total = (IdxT)S * nh * hq;
  for (IdxT idx = (IdxT)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (IdxT)gridDim.x * blockDim.x) {
    const int j = (int)(idx % hq) * 4;
    const IdxT sh = idx / hq;
    const int h = (int)(sh % nh);
    const long s = (long)(sh / nh);
    const bf16* p = x + s * ss + h * hs;
    float a[4], b[4], o0[4], o1[4];
    ldE<4>(p + j, a);
    ldE<4>(p + j + half, b);
    const float4 c0 = *reinterpret_cast<const float4*>(cosv + s * D + j), c1 = *reinterpret_cast<const float4*>(cosv + s * D + j + half);
    const float4 s0 = *reinterpret_cast<const float4*>(sinv + s * D + j), s1 = *reinterpret_cast<const float4*>(sinv + s * D + j + half);
    const float c0v[4] = {c0.x, c0.y, c0.z, c0.w}, c1v[4] = {c1.x, c1.y, c1.z, c1.w};
    const float s0v[4] = {s0.x, s0.y, s0.z, s0.w}, s1v[4] = {s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if (!transpose) { o0[i] = a[i] * c0v[i] - b[i] * s0v[i]; o1[i] = b[i] * c1v[i] + a[i] * s1v[i]; }
      else { o0[i] = a[i] * c0v[i] + b[i] * s1v[i]; o1[i] = b[i] * c1v[i] - a[i] * s0v[i]; }
    }
    bf16* q = out + s * oss + h * ohs;
    stE<4>(q + j, o0);
    stE<4>(q + j + half, o1);
  }
}
__global__ void rope_generic_kernel(const bf16* __restrict__ x, long ss, long hs, const float* __restrict__ cosv,
                                    const float* __restrict__ sinv, bf16* __restrict__ out, long oss, long ohs, int S, int H, int D,
                                    int transpose) {
  const int half = D >> 1;
  const long total = (long)S * H * half;
  for (long idx = blockIdx.x * (long)blockDim.x + threadIdx.x; idx < total; idx += (long)gridDim.x * blockDim.x) {
    const int j = (int)(idx % half);
    const long sh = idx / half;
    const int h = (int)(sh % H);
    const long s = sh / H;
    const bf16* p = x + s * ss + h * hs;
    const float a = __bfloat162float(p[j]), b = __bfloat162float(p[j + half]);
    const float c0 = cosv[s * D + j], c1 = cosv[s * D + j + half], s0 = sinv[s * D + j], s1 = sinv[s * D + j + half];
    float o0, o1;
    if (!transpose) { o0 = a * c0 - b * s0; o1 = b * c1 + a * s1; }
    else { o0 = a * c0 + b * s1; o1 = b * c1 - a * s0; }
    bf16* q = out + s * oss + h * ohs;
    q[j] = __float2bfloat16(o0);
    q[j + half] = __float2bfloat16(o1);
  }
}

// ----------------------------------------------------------------------------------- GDN gate prep
// g = -exp(A_log) * softplus(a + dt_bias) (fp32 out), beta = sigmoid(b) (bf16 out); a,b strided rows
__global__ void gdn_gates_fwd_kernel(const bf16* __restrict__ a, const bf16* __restrict__ b, long row_stride,
                                     const float* __restrict__ A_log, const float* __restrict__ dt_bias, float* __restrict__ g,
                                     bf16* __restrict__ beta, long T, int H) {
  const long n = T * H;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long t = i / H;
    const int h = (int)(i - t * H);
    const float av = __bfloat162float(a[t * row_stride + h]) + dt_bias[h];
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    g[i] = -__expf(A_log[h]) * sp;
    beta[i] = __float2bfloat16(sigmoidf_(__bfloat162float(b[t * row_stride + h])));
  }
}
// da = dg * (-exp(A_log)) * sigmoid(a + dt_bias); db = dbeta * beta (1-beta);
// dA_log[h] += dg * g ; ddt_bias[h] += da  (per-block partials, H <= 256)
__global__ void gdn_gates_bwd_kernel(const float* __restrict__ dg, const bf16* __restrict__ dbeta, const bf16* __restrict__ a,
                                     const bf16* __restrict__ b, long row_stride, const float* __restrict__ A_log,
                                     const float* __restrict__ dt_bias, bf16* __restrict__ da, bf16* __restrict__ db,
                                     long out_stride, float* __restrict__ partial, long T, int H) {
  extern __shared__ float sm[];  // [2][H]
  for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) sm[i] = 0.f;
  __syncthreads();
  const long n = T * H;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const long t = i / H;
    const int h = (int)(i - t * H);
    const float av = __bfloat162float(a[t * row_stride + h]) + dt_bias[h];
    const float sp = av > 20.f ? av : log1pf(__expf(av));
    const float eA = __expf(A_log[h]);
    const float dgi = dg[i];
    const float dav = dgi * (-eA) * sigmoidf_(av);
    const float bt = sigmoidf_(__bfloat162float(b[t * row_stride + h]));
    da[t * out_stride + h] = __float2bfloat16(dav);
    db[t * out_stride + h] = __float2bfloat16(__bfloat162float(dbeta[i]) * bt * (1.f - bt));
    atomicAdd(&sm[h], dgi * (-eA) * sp);
    atomicAdd(&sm[H + h], dav);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 2 * H; i += blockDim.x) partial[(size_t)blockIdx.x * 2 * H + i] = sm[i];
}

// ----------------------------------------------------------------------------------- depthwise causal conv1d + SiLU (packed rows)
// x [T, C] (row stride xs), w [C, K] fp32/bf16, seq_idx [T]; y[t,c] = silu(sum_j w[c,j] x[t-(K-1)+j, c]) within a document
// Sliding-window form: a thread owns 8 channels and walks `rows_per_thread` consecutive tokens, keeping the last K-1
// input rows and its K x 8 weights in registers, so every input row and weight is read once (plus K-1 rows of overlap
// per walk).  seq_idx is non-decreasing, so row t-k belongs to token t's document iff seq_idx[t-k] == seq_idx[t].
template <int K>
__global__ void conv1d_silu_fwd_kernel(const bf16* __restrict__ x, long xs, const bf16* __restrict__ w, const int* __restrict__ seq_idx,
                                       bf16* __restrict__ y, long ys, int T, int C, int rows_per_thread) {
  static_assert(K == 4, "window code below is written for K = 4");
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int t0 = blockIdx.y * rows_per_thread;
  const int t1 = min(T, t0 + rows_per_thread);
  float wv[K][8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint2 w4 = *reinterpret_cast<const uint2*>(w + (long)(c + i) * K);   // K = 4 bf16 = 8 bytes
    wv[0][i] = __uint_as_float(w4.x << 16); wv[1][i] = __uint_as_float(w4.x & 0xffff0000u);
    wv[2][i] = __uint_as_float(w4.y << 16); wv[3][i] = __uint_as_float(w4.y & 0xffff0000u);
  }
  float x1[8], x2[8], x3[8];   // rows t-1, t-2, t-3
  int d1 = -1, d2 = -1, d3 = -1;
#pragma unroll
  for (int i = 0; i < 8; ++i) x1[i] = x2[i] = x3[i] = 0.f;
  if (t0 - 1 >= 0) { d1 = seq_idx[t0 - 1]; unpack8(*reinterpret_cast<const uint4*>(x + (long)(t0 - 1) * xs + c), x1); }
  if (t0 - 2 >= 0) { d2 = seq_idx[t0 - 2]; unpack8(*reinterpret_cast<const uint4*>(x + (long)(t0 - 2) * xs + c), x2); }
  if (t0 - 3 >= 0) { d3 = seq_idx[t0 - 3]; unpack8(*reinterpret_cast<const uint4*>(x + (long)(t0 - 3) * xs + c), x3); }
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    float x0[8];
    unpack8(*reinterpret_cast<const uint4*>(x + (long)t * xs + c), x0);
    const int d0 = seq_idx[t];
    const float m1 = d1 == d0 ? 1.f : 0.f, m2 = d2 == d0 ? 1.f : 0.f, m3 = d3 == d0 ? 1.f : 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float a = x0[i] * wv[3][i];
      a = fmaf(m1 * x1[i], wv[2][i], a);
      a = fmaf(m2 * x2[i], wv[1][i], a);
      a = fmaf(m3 * x3[i], wv[0][i], a);
      acc[i] = a * sigmoidf_(a);
    }
    *reinterpret_cast<uint4*>(y + (long)t * ys + c) = pack8(acc);
#pragma unroll
    for (int i = 0; i < 8; ++i) { x3[i] = x2[i]; x2[i] = x1[i]; x1[i] = x0[i]; }
    d3 = d2; d2 = d1; d1 = d0;
  }
}
// dx[t,c] = sum_j w[c,j] * dpre[t+(K-1)-j, c] (same document), dpre = dy * silu'(pre), pre recomputed from x;
// dw[c,j] = sum_t dpre[t,c] x[t-(K-1)+j, c].  A thread owns 4 channels and walks one slab of tokens [t0, t1) plus K-1
// tokens of lookahead (their dpre is needed for the slab's last dx rows; they do not count toward dw): at token t it
// forms dpre[t] from the sliding input window and then emits dx[t-(K-1)] from the sliding dpre window.
template <int K>
__global__ void conv1d_silu_bwd_kernel(const bf16* __restrict__ dy, long dys, const bf16* __restrict__ x, long xs,
                                       const bf16* __restrict__ w, const int* __restrict__ seq_idx, bf16* __restrict__ dx, long dxs,
                                       float* __restrict__ dw_partial, int T, int C, int t_per_block) {
  static_assert(K == 4, "window code below is written for K = 4");
  constexpr int V = 4;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * V;
  if (c >= C) return;
  const int t0 = blockIdx.y * t_per_block;
  const int t1 = min(T, t0 + t_per_block);
  float wv[K][V], dwacc[K][V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const uint2 w4 = *reinterpret_cast<const uint2*>(w + (long)(c + i) * K);
    wv[0][i] = __uint_as_float(w4.x << 16); wv[1][i] = __uint_as_float(w4.x & 0xffff0000u);
    wv[2][i] = __uint_as_float(w4.y << 16); wv[3][i] = __uint_as_float(w4.y & 0xffff0000u);
#pragma unroll
    for (int j = 0; j < K; ++j) dwacc[j][i] = 0.f;
  }
  auto ld4 = [&](const bf16* ptr, float (&f)[V]) {
    const uint2 u = *reinterpret_cast<const uint2*>(ptr);
    f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
    f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
  };
  float x1[V], x2[V], x3[V];          // input rows t-1, t-2, t-3
  float p1[V], p2[V], p3[V];          // dpre of tokens t-1, t-2, t-3
  int d1 = -1, d2 = -1, d3 = -1;      // their documents (-1: no such token)
#pragma unroll
  for (int i = 0; i < V; ++i) x1[i] = x2[i] = x3[i] = p1[i] = p2[i] = p3[i] = 0.f;
  // input rows before the slab are needed for pre[t0 ...]; dpre of tokens before the slab is never needed (dx looks ahead)
  if (t0 - 1 >= 0) { d1 = seq_idx[t0 - 1]; ld4(x + (long)(t0 - 1) * xs + c, x1); }
  if (t0 - 2 >= 0) { d2 = seq_idx[t0 - 2]; ld4(x + (long)(t0 - 2) * xs + c, x2); }
  if (t0 - 3 >= 0) { d3 = seq_idx[t0 - 3]; ld4(x + (long)(t0 - 3) * xs + c, x3); }
  const int t_end = t1 + (K - 1);
#pragma unroll 2
  for (int t = t0; t < t_end; ++t) {
    float x0[V], p0[V];
    int d0 = -2;                       // beyond the last token: matches no document
    if (t < T) {
      float g[V];
      ld4(x + (long)t * xs + c, x0);
      ld4(dy + (long)t * dys + c, g);
      d0 = seq_idx[t];
      const float m1 = d1 == d0 ? 1.f : 0.f, m2 = d2 == d0 ? 1.f : 0.f, m3 = d3 == d0 ? 1.f : 0.f;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float a = x0[i] * wv[3][i];
        a = fmaf(m1 * x1[i], wv[2][i], a);
        a = fmaf(m2 * x2[i], wv[1][i], a);
        a = fmaf(m3 * x3[i], wv[0][i], a);
        const float sg = sigmoidf_(a);
        p0[i] = g[i] * (sg + a * sg * (1.f - sg));
      }
      if (t < t1) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          dwacc[3][i] = fmaf(p0[i], x0[i], dwacc[3][i]);
          dwacc[2][i] = fmaf(p0[i], m1 * x1[i], dwacc[2][i]);
          dwacc[1][i] = fmaf(p0[i], m2 * x2[i], dwacc[1][i]);
          dwacc[0][i] = fmaf(p0[i], m3 * x3[i], dwacc[0][i]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < V; ++i) { x0[i] = 0.f; p0[i] = 0.f; }
    }
    // dx of token s = t - 3: taps j = 3, 2, 1, 0 meet dpre of tokens s, s+1, s+2, s+3 = t-3, t-2, t-1, t
    const int sidx = t - (K - 1);
    if (sidx >= t0) {
      const float n2 = d2 == d3 ? 1.f : 0.f, n1 = d1 == d3 ? 1.f : 0.f, n0 = d0 == d3 ? 1.f : 0.f;
      float o[V];
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float a = wv[3][i] * p3[i];
        a = fmaf(n2 * wv[2][i], p2[i], a);
        a = fmaf(n1 * wv[1][i], p1[i], a);
        a = fmaf(n0 * wv[0][i], p0[i], a);
        o[i] = a;
      }
      uint2 pk;
      const __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
      pk.x = *reinterpret_cast<const uint32_t*>(&lo);
      pk.y = *reinterpret_cast<const uint32_t*>(&hi);
      *reinterpret_cast<uint2*>(dx + (long)sidx * dxs + c) = pk;
    }
#pragma unroll
    for (int i = 0; i < V; ++i) { x3[i] = x2[i]; x2[i] = x1[i]; x1[i] = x0[i]; p3[i] = p2[i]; p2[i] = p1[i]; p1[i] = p0[i]; }
    d3 = d2; d2 = d1; d1 = d0;
  }
#pragma unroll
  for (int i = 0; i < V; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) dw_partial[((size_t)blockIdx.y * C + c + i) * K + j] = dwacc[j][i];
}

// ----------------------------------------------------------------------------------- row scatter / row add
// out[index[i], :] (=|+=) src[i, :]   (index rows are unique)
__global__ void rows_update_kernel(bf16* __restrict__ out, const long* __restrict__ index, const bf16* __restrict__ src, long n_rows,
                                   int D, int add) {
  const int vper = D >> 3;
  const long total = n_rows * vper;
  for (long v = blockIdx.x * (long)blockDim.x + threadIdx.x; v < total; v += (long)gridDim.x * blockDim.x) {
    const long i = v / vper;
    const int c = (int)(v - i * vper);
    uint4* dst = reinterpret_cast<uint4*>(out + index[i] * (long)D) + c;
    uint4 s = reinterpret_cast<const uint4*>(src + i * (long)D)[c];
    if (add) {
      float a[8], b[8];
      unpack8(*dst, a);
      unpack8(s, b);
#pragma unroll
      for (int k = 0; k < 8; ++k) a[k] += b[k];
      s = pack8(a);
    }
    *dst = s;
  }
}
// dst[i, :] = src[index[i], :]
__global__ void rows_gather_kernel(bf16* __restrict__ dst, const long* __restrict__ index, const bf16* __restrict__ src, long n_rows,
                                   int D) {
  const int vper = D >> 3;
  const long total = n_rows * vper;
  for (long v = blockIdx.x * (long)blockDim.x + threadIdx.x; v < total; v += (long)gridDim.x * blockDim.x) {
    const long i = v / vper;
    const int c = (int)(v - i * vper);
    reinterpret_cast<uint4*>(dst + i * (long)D)[c] = reinterpret_cast<const uint4*>(src + index[i] * (long)D)[c];
  }
}

inline int grid_for(long work_items, int per_block, int cap) {
  long g = (work_items + per_block - 1) / per_block;
  if (g < 1) g = 1;
  return (int)(g < cap ? g : cap);
}

}  // namespace

// ===================================================================================== launchers
#define BF(p) reinterpret_cast<const bf16*>(p)
#define BFM(p) reinterpret_cast<bf16*>(p)

// bytes of the copy ring of a row-tile launch: kPipe stages of `tensors` inputs, `rr` rows each
static size_t ring_bytes(int D, int rr, int tensors) { return (size_t)kPipe * tensors * rr * (D >> 3) * sizeof(uint4); }
// a kernel whose ring plus its static scratch exceeds the default 48 KB of shared memory has to be told so
template <typename K>
static void allow_smem(K kernel, size_t bytes) {
  if (bytes > 40 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}
// grid of a forward row-tile kernel: one wave of resident blocks (a second, partly filled wave costs a whole pass)
template <typename K>
static int tile_grid(K kernel, int rows, int threads, int rr, size_t smem) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return grid_for(rows, rr, sms * per_sm);
}
extern "C" {

// three blocks per SM: what the backward row-tile kernels keep resident (registers and copy ring), so the grid is one wave
int vlmt_norm_blocks(int rows) { return grid_for(rows, kWarpsPerBlock, 148 * 3); }

// warps per block of the backward norm kernels: each warp owns `floats_per_warp` fp32 accumulators in smem
static int bwd_warps(size_t floats_per_warp) {
  int w = (int)((200 * 1024) / (floats_per_warp * sizeof(float)));
  if (w > kWarpsPerBlock) w = kWarpsPerBlock;
  return w < 1 ? 0 : w;
}

// column groups per thread of the row-tile kernels (0: D is too wide for them)
static int tile_vpt(int D) {
  const int nvec = D >> 3;
  if ((D & 7) || nvec > 4 * kRT) return 0;
  return nvec <= kRT ? 1 : (nvec <= 2 * kRT ? 2 : 4);
}
// threads per block of a row-tile launch: with one column group per thread a narrow row (1152 channels = 144 groups) gets a
// block of just enough warps instead of 256 threads of which 112 idle
static int tile_threads(int D, int vpt) {
  if (vpt != 1) return kRT;
  const int t = (((D >> 3) + 31) / 32) * 32;
  return t < 64 ? 64 : (t > kRT ? kRT : t);
}
// vectors per lane of the warp-per-row LayerNorm kernels (0: the width is outside their range)
static int ln_warp_vl(int D) {
  if ((D & 7) || D <= 768 || D > 1280) return 0;
  return ((D >> 3) + 31) / 32 <= 4 ? 4 : 5;
}
#define TILE_DISPATCH(VPT, CALL1, CALL2, CALL4) do { if ((VPT) == 1) { CALL1; } else if ((VPT) == 2) { CALL2; } else { CALL4; } } while (0)

void vlmt_rmsnorm_fwd(const void* x, const void* res, const void* w, int w_fp32, void* y, void* r_out, float* rstd, int rows, int D,
                      float eps, int offset, cudaStream_t st) {
  if (rows <= 0) return;
  const int vpt = tile_vpt(D);
  if (vpt) {
#define RF(WT, V) do { const size_t sb = ring_bytes(D, TileRows<V>::value, res ? 2 : 1); auto kf = rmsnorm_fwd_tile_kernel<WT, V>; allow_smem(kf, sb); \
    kf<<<tile_grid(kf, rows, tile_threads(D, vpt), TileRows<V>::value, sb), tile_threads(D, vpt), sb, st>>>(BF(x), BF(res), (const WT*)w, BFM(y), BFM(r_out), rstd, rows, D, eps, offset); } while (0)
    if (w_fp32) TILE_DISPATCH(vpt, RF(float, 1), RF(float, 2), RF(float, 4));
    else TILE_DISPATCH(vpt, RF(bf16, 1), RF(bf16, 2), RF(bf16, 4));
#undef RF
    return;
  }
  const int grid = grid_for(rows, kWarpsPerBlock, 148 * 8);
  if (w_fp32)
    rmsnorm_fwd_kernel<float><<<grid, kThreads, 0, st>>>(BF(x), BF(res), (const float*)w, BFM(y), BFM(r_out), rstd, rows, D, eps, offset);
  else
    rmsnorm_fwd_kernel<bf16><<<grid, kThreads, 0, st>>>(BF(x), BF(res), BF(w), BFM(y), BFM(r_out), rstd, rows, D, eps, offset);
}

// dw_partial has vlmt_norm_blocks(rows) rows; every one of them is written
int vlmt_rmsnorm_bwd(const void* dy, const void* x, const void* w, int w_fp32, const float* rstd, const void* dres, void* dx,
                     float* dw_partial, int rows, int D, int offset, cudaStream_t st) {
  const int grid = vlmt_norm_blocks(rows);
  const int vpt = tile_vpt(D);
  if (vpt) {
#define RB(WT, V) do { const size_t sb = ring_bytes(D, TileRows<V>::value, dres ? 3 : 2); auto kb = rmsnorm_bwd_tile_kernel<WT, V>; allow_smem(kb, sb); \
    kb<<<grid, tile_threads(D, vpt), sb, st>>>(BF(dy), BF(x), (const WT*)w, rstd, BF(dres), BFM(dx), dw_partial, rows, D, offset); } while (0)
    if (w_fp32) TILE_DISPATCH(vpt, RB(float, 1), RB(float, 2), RB(float, 4));
    else TILE_DISPATCH(vpt, RB(bf16, 1), RB(bf16, 2), RB(bf16, 4));
#undef RB
    return grid;
  }
  const int nw = bwd_warps(D);
  if (nw == 0) return -1;
  const size_t smem = (size_t)nw * D * sizeof(float);
  const int kThreadsDyn = nw * 32;
  if (w_fp32) {
    auto k = rmsnorm_bwd_kernel<float>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<grid, kThreadsDyn, smem, st>>>(BF(dy), BF(x), (const float*)w, rstd, BF(dres), BFM(dx), dw_partial, rows, D, offset);
  } else {
    auto k = rmsnorm_bwd_kernel<bf16>;
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    k<<<grid, kThreadsDyn, smem, st>>>(BF(dy), BF(x), BF(w), rstd, BF(dres), BFM(dx), dw_partial, rows, D, offset);
  }
  return grid;
}

void vlmt_layernorm_fwd(const void* x, const void* w, const void* b, void* y, float* mean, float* rstd, int rows, int D, float eps,
                        cudaStream_t st) {
  if (rows <= 0) return;
  const int vl = ln_warp_vl(D);
  if (vl) {
    const size_t sb = 2 * (size_t)D * sizeof(float) + (size_t)kLnWarpsFwd * kLnPipeFwd * (D >> 3) * sizeof(uint4);
#define LW(V) do { auto kf = layernorm_fwd_warp_kernel<V>; allow_smem(kf, sb); \
    kf<<<tile_grid(kf, rows, kLnWarpsFwd * 32, kLnWarpsFwd, sb), kLnWarpsFwd * 32, sb, st>>>(BF(x), BF(w), BF(b), BFM(y), mean, rstd, rows, D, eps); } while (0)
    if (vl == 4) LW(4); else LW(5);
#undef LW
    return;
  }
  const int vpt = tile_vpt(D);
  if (vpt) {
#define LF(V) do { const size_t sb = ring_bytes(D, TileRows<V>::value, 1); auto kf = layernorm_fwd_tile_kernel<V>; allow_smem(kf, sb); \
    kf<<<tile_grid(kf, rows, tile_threads(D, vpt), TileRows<V>::value, sb), tile_threads(D, vpt), sb, st>>>(BF(x), BF(w), BF(b), BFM(y), mean, rstd, rows, D, eps); } while (0)
    TILE_DISPATCH(vpt, LF(1), LF(2), LF(4));
#undef LF
    return;
  }
  layernorm_fwd_kernel<<<grid_for(rows, kWarpsPerBlock, 148 * 8), kThreads, 0, st>>>(BF(x), BF(w), BF(b), BFM(y), mean, rstd, rows, D, eps);
}
int vlmt_layernorm_bwd(const void* dy, const void* x, const void* w, const float* mean, const float* rstd, void* dx, float* dw_partial,
                       float* db_partial, int rows, int D, cudaStream_t st) {
  const int grid = vlmt_norm_blocks(rows);
  const int vpt = tile_vpt(D);
  if (vpt) {
#define LB(V) do { const size_t sb = ring_bytes(D, TileRows<V>::value, 2); auto kb = layernorm_bwd_tile_kernel<V>; allow_smem(kb, sb); \
    kb<<<grid, tile_threads(D, vpt), sb, st>>>(BF(dy), BF(x), BF(w), mean, rstd, BFM(dx), dw_partial, db_partial, rows, D); } while (0)
    TILE_DISPATCH(vpt, LB(1), LB(2), LB(4));
#undef LB
    return grid;
  }
  const int nw = bwd_warps(2 * (size_t)D);
  if (nw == 0) return -1;
  const size_t smem = (size_t)nw * 2 * D * sizeof(float);
  cudaFuncSetAttribute(layernorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  layernorm_bwd_kernel<<<grid, nw * 32, smem, st>>>(BF(dy), BF(x), BF(w), mean, rstd, BFM(dx), dw_partial, db_partial, rows, D);
  return grid;
}

void vlmt_rmsnorm_gated_fwd(const void* x, const void* z, const void* w, void* y, float* rstd, int rows, int D, float eps, cudaStream_t st) {
  rmsnorm_gated_fwd_kernel<<<grid_for(rows, kWarpsPerBlock, 148 * 16), kThreads, 0, st>>>(BF(x), BF(z), BF(w), BFM(y), rstd, rows, D, eps);
}
int vlmt_rmsnorm_gated_bwd(const void* dy, const void* x, const void* z, const void* w, const float* rstd, void* dx, void* dz,
                           float* dw_partial, int rows, int D, cudaStream_t st) {
  const int grid = vlmt_norm_blocks(rows);
  rmsnorm_gated_bwd_kernel<<<grid, kThreads, (size_t)kWarpsPerBlock * D * sizeof(float), st>>>(BF(dy), BF(x), BF(z), BF(w), rstd, BFM(dx),
                                                                                            BFM(dz), dw_partial, rows, D);
  return grid;
}

void vlmt_swiglu_fwd(const void* gu, void* out, long rows, int I, cudaStream_t st) {
  swiglu_fwd_kernel<<<grid_for(rows * (I >> 3), 256, 148 * 16), 256, 0, st>>>(BF(gu), BFM(out), rows, I);
}
void vlmt_swiglu_bwd(const void* dout, const void* gu, void* dgu, long rows, int I, cudaStream_t st) {
  swiglu_bwd_kernel<<<grid_for(rows * (I >> 3), 256, 148 * 16), 256, 0, st>>>(BF(dout), BF(gu), BFM(dgu), rows, I);
}
void vlmt_sigmoid_mul_fwd(const void* x, const void* gate, void* out, long n, cudaStream_t st) {
  sigmoid_mul_fwd_kernel<<<grid_for(n >> 3, 256, 148 * 16), 256, 0, st>>>(BF(x), BF(gate), BFM(out), n >> 3);
}
void vlmt_sigmoid_mul_bwd(const void* dout, const void* x, const void* gate, void* dx, void* dgate, long n, cudaStream_t st) {
  sigmoid_mul_bwd_kernel<<<grid_for(n >> 3, 256, 148 * 16), 256, 0, st>>>(BF(dout), BF(x), BF(gate), BFM(dx), BFM(dgate), n >> 3);
}
void vlmt_gelu_fwd(const void* x, void* y, long n, int tanh_approx, cudaStream_t st) {
  gelu_fwd_kernel<<<grid_for(n >> 3, 256, 148 * 16), 256, 0, st>>>(BF(x), BFM(y), n >> 3, tanh_approx);
}
void vlmt_gelu_bwd(const void* dy, const void* x, void* dx, long n, int tanh_approx, cudaStream_t st) {
  gelu_bwd_kernel<<<grid_for(n >> 3, 256, 148 * 16), 256, 0, st>>>(BF(dy), BF(x), BFM(dx), n >> 3, tanh_approx);
}

int vlmt_qkv_blocks(long items) { return grid_for(items, kWarpsPerBlock, 148 * 8); }

int vlmt_qkv_norm_rope_fwd(const void* qkv, const void* qw, const void* kw, const float* cosv, const float* sinv, void* q, void* k,
                           void* v, void* gate, float* rstd, int T, int n_q, int n_kv, int D, int R, float eps, int offset, int gated,
                           int has_norm, cudaStream_t st) {
  const int E = D / 32;
  if (D % 32 || R > D || (R / 2) % E || (((R / 2) / E) & ((R / 2) / E - 1)) || (R / 2) / E >= 32) return -1;
  const int grid = vlmt_qkv_blocks((long)T * ((n_q + 2 * n_kv + kQkvGroup - 1) / kQkvGroup));  // one warp per token and group of heads
#define LAUNCH(E_)                                                                                                              \
  qkv_norm_rope_fwd_kernel<E_><<<grid, kThreads, 0, st>>>(BF(qkv), BF(qw), BF(kw), cosv, sinv, BFM(q), BFM(k), BFM(v), BFM(gate), \
                                                          rstd, T, n_q, n_kv, R, eps, offset, gated, has_norm)
  switch (E) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 4: LAUNCH(4); break;
    case 8: LAUNCH(8); break;
    default: return -2;
  }
#undef LAUNCH
  return 0;
}
int vlmt_qkv_norm_rope_bwd(const void* dq, const void* dk, const void* dv, const void* dgate, const void* qkv, const void* qw,
                           const void* kw, const float* cosv, const float* sinv, const float* rstd, void* dqkv, float* dw_partial,
                           int T, int n_q, int n_kv, int D, int R, int offset, int gated, int has_norm, cudaStream_t st) {
  const int E = D / 32;
  const int grid = vlmt_qkv_blocks((long)T * (n_q + 2 * n_kv));
#define LAUNCH(E_)                                                                                                               \
  qkv_norm_rope_bwd_kernel<E_><<<grid, kThreads, 0, st>>>(BF(dq), BF(dk), BF(dv), BF(dgate), BF(qkv), BF(qw), BF(kw), cosv, sinv, \
                                                          rstd, BFM(dqkv), dw_partial, T, n_q, n_kv, R, offset, gated, has_norm)
  switch (E) {
    case 1: LAUNCH(1); break;
    case 2: LAUNCH(2); break;
    case 4: LAUNCH(4); break;
    case 8: LAUNCH(8); break;
    default: return -2;
  }
#undef LAUNCH
  return grid;
}

void vlmt_rope_generic(const void* x, long ss, long hs, const float* cosv, const float* sinv, void* out, long oss, long ohs, int S, int H,
                       int D, int transpose, cudaStream_t st) {
  const int half = D / 2;
  const bool vec4 = half % 4 == 0 && ss % 4 == 0 && hs % 4 == 0 && oss % 4 == 0 && ohs % 4 == 0 && ((uintptr_t)x & 7) == 0 &&
                    ((uintptr_t)out & 7) == 0 && ((uintptr_t)cosv & 15) == 0 && ((uintptr_t)sinv & 15) == 0;
  if (vec4) {
    const long items = (long)S * H * (half / 4);
    const int grid = grid_for(items, 256, 148 * 16);
    if (items + (long)grid * 256 < (1l << 32))   // the loop's last increment must not wrap
      rope_generic_vec4_kernel<unsigned><<<grid, 256, 0, st>>>(BF(x), ss, hs, cosv, sinv, BFM(out), oss, ohs, S, H, D, transpose);
    else
      rope_generic_vec4_kernel<long><<<grid, 256, 0, st>>>(BF(x), ss, hs, cosv, sinv, BFM(out), oss, ohs, S, H, D, transpose);
    return;
  }
  rope_generic_kernel<<<grid_for((long)S * H * (D / 2), 256, 148 * 16), 256, 0, st>>>(BF(x), ss, hs, cosv, sinv, BFM(out), oss, ohs, S, H, D,
                                                                                    transpose);
}

void vlmt_gdn_gates_fwd(const void* a, const void* b, long row_stride, const float* A_log, const float* dt_bias, float* g, void* beta,
                        long T, int H, cudaStream_t st) {
  gdn_gates_fwd_kernel<<<grid_for(T * H, 256, 148 * 8), 256, 0, st>>>(BF(a), BF(b), row_stride, A_log, dt_bias, g, BFM(beta), T, H);
}
int vlmt_gdn_gates_bwd(const float* dg, const void* dbeta, const void* a, const void* b, long row_stride, const float* A_log,
                       const float* dt_bias, void* da, void* db, long out_stride, float* partial, long T, int H, cudaStream_t st) {
  const int grid = grid_for(T * H, 256, 148 * 2);
  gdn_gates_bwd_kernel<<<grid, 256, 2 * H * sizeof(float), st>>>(dg, BF(dbeta), BF(a), BF(b), row_stride, A_log, dt_bias, BFM(da), BFM(db),
                                                               out_stride, partial, T, H);
  return grid;
}

int vlmt_conv1d_silu_fwd(const void* x, long xs, const void* w, const int* seq_idx, void* y, long ys, int T, int C, int K, cudaStream_t st) {
  if (K != 4 || (C & 7)) return -1;
  const int rows = 64;
  dim3 grid(((C >> 3) + 127) / 128, (T + rows - 1) / rows);
  conv1d_silu_fwd_kernel<4><<<grid, 128, 0, st>>>(BF(x), xs, BF(w), seq_idx, BFM(y), ys, T, C, rows);
  return 0;
}
int vlmt_conv1d_bwd_slabs(int T) { return (T + 255) / 256; }
int vlmt_conv1d_silu_bwd(const void* dy, long dys, const void* x, long xs, const void* w, const int* seq_idx, void* dx, long dxs,
                         float* dw_partial, int T, int C, int K, cudaStream_t st) {
  if (K != 4 || (C & 3)) return -1;
  dim3 grid(((C >> 2) + 127) / 128, vlmt_conv1d_bwd_slabs(T));
  conv1d_silu_bwd_kernel<4><<<grid, 128, 0, st>>>(BF(dy), dys, BF(x), xs, BF(w), seq_idx, BFM(dx), dxs, dw_partial, T, C, 256);
  return 0;
}

void vlmt_rows_update(void* out, const long* index, const void* src, long n_rows, int D, int add, cudaStream_t st) {
  if (n_rows == 0) return;
  rows_update_kernel<<<grid_for(n_rows * (D >> 3), 256, 148 * 16), 256, 0, st>>>(BFM(out), index, BF(src), n_rows, D, add);
}
void vlmt_rows_gather(void* dst, const long* index, const void* src, long n_rows, int D, cudaStream_t st) {
  if (n_rows == 0) return;
  rows_gather_kernel<<<grid_for(n_rows * (D >> 3), 256, 148 * 16), 256, 0, st>>>(BFM(dst), index, BF(src), n_rows, D);
}

}  // extern "C"


// ===================================================================================== allocation-free variant
// RMSNorm backward whose per-block partial weight gradients live in a fixed array of the library image instead of
// a caller-provided scratch tensor (contract: no_alloc_entry.h).  Nothing above this line is changed by it.
#include <mutex>
#include <stdio.h>

static __device__ __align__(256) float g_rmsnorm_bwd_scratch[VLMT_NOALLOC_MAX_BLOCKS * VLMT_NOALLOC_MAX_D];

namespace {
// dw[c] = sum over the `blocks` partial rows written by the backward kernel (every slot read here was written by it)
__global__ void static_scratch_colsum_kernel(const float* __restrict__ partial, float* __restrict__ dw, int blocks, int D) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= D) return;
  float s = 0.f;
  for (int b = 0; b < blocks; ++b) s += partial[(size_t)b * D + c];
  dw[c] = s;
}

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the CURRENT device (looked up once per device; in host code the array's name
// is only a handle for this lookup, never a pointer a kernel may use).
float* scratch_for_current_device(int* err) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) { *err = VLMT_NOALLOC_ERR_SYMBOL; return nullptr; }
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_rmsnorm_bwd_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      fprintf(stderr, "vlmt_rmsnorm_bwd_static: cudaGetSymbolAddress failed on device %d: %s\n", dev, cudaGetErrorString(e));
      *err = VLMT_NOALLOC_ERR_SYMBOL;
      return nullptr;
    }
    g_scratch_addr[dev] = ptr;
  }
  return g_scratch_addr[dev];
}
}  // namespace

extern "C" int vlmt_rmsnorm_bwd_static(const void* dy, const void* x, const void* w, int w_fp32, const float* rstd, const void* dres,
                                       void* dx, float* dw, int rows, int D, int offset, cudaStream_t st) {
  if (D <= 0 || (D & 7) || D > VLMT_NOALLOC_MAX_D) {
    fprintf(stderr, "vlmt_rmsnorm_bwd_static: D = %d is not supported (need a multiple of 8, at most %d: the built-in scratch "
                    "holds %d x %d floats)\n", D, VLMT_NOALLOC_MAX_D, VLMT_NOALLOC_MAX_BLOCKS, VLMT_NOALLOC_MAX_D);
    return VLMT_NOALLOC_ERR_SIZE;
  }
  int err = 0;
  float* scratch = scratch_for_current_device(&err);
  if (scratch == nullptr) return err;
  if (rows <= 0) {
    // no rows, no partial sums: the column-sum kernel over zero blocks still overwrites dw (an output) with zeros
    static_scratch_colsum_kernel<<<(D + 255) / 256, 256, 0, st>>>(scratch, dw, 0, D);
    return (int)cudaGetLastError();
  }
  const int nw = bwd_warps(D);
  if (nw == 0) return VLMT_NOALLOC_ERR_SIZE;
  int grid = (rows + nw - 1) / nw;
  if (grid > VLMT_NOALLOC_MAX_BLOCKS) grid = VLMT_NOALLOC_MAX_BLOCKS;
  const size_t smem = (size_t)nw * D * sizeof(float);
  cudaError_t e;
  if (w_fp32) {
    auto k = rmsnorm_bwd_kernel<float>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    k<<<grid, nw * 32, smem, st>>>(BF(dy), BF(x), (const float*)w, rstd, BF(dres), BFM(dx), scratch, rows, D, offset);
  } else {
    auto k = rmsnorm_bwd_kernel<bf16>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    k<<<grid, nw * 32, smem, st>>>(BF(dy), BF(x), BF(w), rstd, BF(dres), BFM(dx), scratch, rows, D, offset);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  static_scratch_colsum_kernel<<<(D + 255) / 256, 256, 0, st>>>(scratch, dw, grid, D);
  return (int)cudaGetLastError();
}
