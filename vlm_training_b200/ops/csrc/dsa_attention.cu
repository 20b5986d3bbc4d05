// Sparse (selected-key) attention for DSA: every query attends to its own list of up to `kk` key rows.
//
// One CTA per (query, kv head): the `REP` query heads that share the kv head are processed together, so every selected
// key / value row is read once per CTA.  Each query has its own key set, so there is no tile shared between queries to
// put on the tensor cores (M would be REP = 8); the kernel is a CUDA-core kernel bound by the gathered reads:
//   phase 1  thread <-> key:  s[j][h] = scale * q[h] . K[sel[j]]           (two keys per thread, q broadcast from smem)
//   phase 2  warp   <-> head: m[h], l[h], p = exp(s - m)                    (scores stay in shared memory)
//   phase 3  thread <-> dim:  o[h][d] = sum_j p[j][h] V[sel[j]][d] / l[h]   (coalesced value loads)
// The backward kernel recomputes p from the saved log-sum-exp, forms dS in phase 1 (thread <-> key, second pass over
// the value row for dP) and accumulates dQ in registers and dK / dV with float atomics in phase 2 (thread <-> dim).
// sel[j] < 0 marks an unused slot.  No waits on other CTAs anywhere.
#include "dsa_attention.h"

#include <cuda_bf16.h>
#include <math.h>
#include <stdint.h>

namespace {

constexpr int THREADS = 256;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// dot products of two key (or value) rows with the REP rows of `a_s` ([REP][D] floats in shared memory): every
// shared-memory read of `a_s` feeds both rows (the kernels are bound by the shared-memory pipe, so pairing the rows
// halves its load per key); 4 x 16 bytes of each row are loaded before they are used
template <int D, int REP>
__device__ __forceinline__ void row_dots2(const __nv_bfloat16* __restrict__ r0, const __nv_bfloat16* __restrict__ r1,
                                          const float* __restrict__ a_s, float (&acc0)[REP], float (&acc1)[REP]) {
#pragma unroll
  for (int h = 0; h < REP; ++h) { acc0[h] = 0.f; acc1[h] = 0.f; }
  for (int c0 = 0; c0 < D / 8; c0 += 4) {
    uint4 raw0[4], raw1[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      raw0[u] = *reinterpret_cast<const uint4*>(r0 + (c0 + u) * 8);
      raw1[u] = *reinterpret_cast<const uint4*>(r1 + (c0 + u) * 8);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float k0[8], k1[8];
      unpack8(raw0[u], k0);
      unpack8(raw1[u], k1);
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        const float4 a0 = *reinterpret_cast<const float4*>(a_s + h * D + (c0 + u) * 8);
        const float4 a1 = *reinterpret_cast<const float4*>(a_s + h * D + (c0 + u) * 8 + 4);
        acc0[h] += k0[0] * a0.x + k0[1] * a0.y + k0[2] * a0.z + k0[3] * a0.w + k0[4] * a1.x + k0[5] * a1.y + k0[6] * a1.z + k0[7] * a1.w;
        acc1[h] += k1[0] * a0.x + k1[1] * a0.y + k1[2] * a0.z + k1[3] * a0.w + k1[4] * a1.x + k1[5] * a1.y + k1[6] * a1.z + k1[7] * a1.w;
      }
    }
  }
}

struct Params {
  const __nv_bfloat16* q;    // [B, Hkv * REP, D]
  const __nv_bfloat16* k;    // [L, Hkv, D]
  const __nv_bfloat16* v;    // [L, Hkv, D]
  const int* sel;            // [B, kk], -1 = unused
  __nv_bfloat16* o;          // [B, Hkv * REP, D]
  float* lse;                // [B, Hkv * REP]  natural-log sum-exp of the scaled scores
  const __nv_bfloat16* d_o;  // backward only
  float* dq;                 // [B, Hkv * REP, D]
  float* dk;                 // [L, Hkv, D] accumulated with atomics
  float* dv;
  int B, Hkv, kk;
  float scale;
};

template <int D, int REP>
__global__ void __launch_bounds__(THREADS) dsa_fwd_kernel(Params p) {
  extern __shared__ float smem[];
  float* q_s = smem;                       // [REP][D]
  float* s_s = q_s + REP * D;              // [kk][REP]
  float* ml_s = s_s + (size_t)p.kk * REP;  // [2][REP]: max, 1 / sum
  int* sel_s = reinterpret_cast<int*>(ml_s + 2 * REP);  // [kk]
  const int b = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Hq = p.Hkv * REP;
  const __nv_bfloat16* qrow = p.q + ((size_t)b * Hq + g * REP) * D;
  for (int i = tid; i < REP * D; i += THREADS) q_s[i] = __bfloat162float(qrow[i]);
  for (int j = tid; j < p.kk; j += THREADS) sel_s[j] = p.sel[(size_t)b * p.kk + j];
  __syncthreads();
  // ---- phase 1: two keys per thread and pass (an unused or missing slot reads row 0 and is overwritten with -inf)
  for (int j = tid; j < p.kk; j += 2 * THREADS) {
    const int j1 = j + THREADS;
    const int i0 = sel_s[j], i1 = j1 < p.kk ? sel_s[j1] : -1;
    float a0[REP], a1[REP];
    row_dots2<D, REP>(p.k + ((size_t)max(i0, 0) * p.Hkv + g) * D, p.k + ((size_t)max(i1, 0) * p.Hkv + g) * D, q_s, a0, a1);
#pragma unroll
    for (int h = 0; h < REP; ++h) s_s[j * REP + h] = i0 >= 0 ? a0[h] * p.scale : -INFINITY;
    if (j1 < p.kk) {
#pragma unroll
      for (int h = 0; h < REP; ++h) s_s[j1 * REP + h] = i1 >= 0 ? a1[h] * p.scale : -INFINITY;
    }
  }
  __syncthreads();
  // ---- phase 2: warp h owns head h
  for (int h = warp; h < REP; h += THREADS / 32) {
    float m = -INFINITY;
    for (int j = lane; j < p.kk; j += 32) m = fmaxf(m, s_s[j * REP + h]);
    m = warp_max(m);
    const float mm = m == -INFINITY ? 0.f : m;
    float l = 0.f;
    for (int j = lane; j < p.kk; j += 32) {
      const float e = __expf(s_s[j * REP + h] - mm);
      s_s[j * REP + h] = e;
      l += e;
    }
    l = warp_sum(l);
    if (lane == 0) {
      ml_s[h] = mm;
      ml_s[REP + h] = l > 0.f ? 1.f / l : 0.f;
      p.lse[(size_t)b * Hq + g * REP + h] = l > 0.f ? mm + logf(l) : -INFINITY;
    }
  }
  __syncthreads();
  // ---- phase 3: thread <-> dim (threads beyond D idle for small heads)
  if (tid < D) {
    float acc[REP];
#pragma unroll
    for (int h = 0; h < REP; ++h) acc[h] = 0.f;
    // 8 value rows in flight per thread; an unused slot reads row 0 with probability 0
    constexpr int U = 8;
    for (int j0 = 0; j0 < p.kk; j0 += U) {
      float vv[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int j = j0 + u;
        const int idx = j < p.kk ? max(sel_s[j], 0) : 0;
        vv[u] = __bfloat162float(p.v[((size_t)idx * p.Hkv + g) * D + tid]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (j0 + u < p.kk) {
#pragma unroll
          for (int h = 0; h < REP; ++h) acc[h] = fmaf(s_s[(j0 + u) * REP + h], vv[u], acc[h]);
        }
      }
    }
#pragma unroll
    for (int h = 0; h < REP; ++h) p.o[((size_t)b * Hq + g * REP + h) * D + tid] = __float2bfloat16(acc[h] * ml_s[REP + h]);
  }
}

template <int D, int REP>
__global__ void __launch_bounds__(THREADS) dsa_bwd_kernel(Params p) {
  extern __shared__ float smem[];
  float* q_s = smem;                        // [REP][D]
  float* do_s = q_s + REP * D;              // [REP][D]
  float* p_s = do_s + REP * D;              // [kk][REP]  probabilities
  float* ds_s = p_s + (size_t)p.kk * REP;   // [kk][REP]  gradient of the raw (unscaled) scores
  float* st_s = ds_s + (size_t)p.kk * REP;  // [2][REP]: lse, delta
  int* sel_s = reinterpret_cast<int*>(st_s + 2 * REP);
  const int b = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Hq = p.Hkv * REP;
  const size_t row0 = ((size_t)b * Hq + g * REP) * D;
  for (int i = tid; i < REP * D; i += THREADS) {
    q_s[i] = __bfloat162float(p.q[row0 + i]);
    do_s[i] = __bfloat162float(p.d_o[row0 + i]);
  }
  for (int j = tid; j < p.kk; j += THREADS) sel_s[j] = p.sel[(size_t)b * p.kk + j];
  __syncthreads();
  // delta[h] = sum_d dO[h][d] O[h][d]
  for (int h = warp; h < REP; h += THREADS / 32) {
    float acc = 0.f;
    for (int d = lane; d < D; d += 32) acc += do_s[h * D + d] * __bfloat162float(p.o[row0 + (size_t)h * D + d]);
    acc = warp_sum(acc);
    if (lane == 0) {
      st_s[h] = p.lse[(size_t)b * Hq + g * REP + h];
      st_s[REP + h] = acc;
    }
  }
  __syncthreads();
  // ---- phase 1: thread <-> key (two keys per pass): p, dS
  for (int j = tid; j < p.kk; j += 2 * THREADS) {
    const int j1 = j + THREADS;
    const int i0 = sel_s[j], i1 = j1 < p.kk ? sel_s[j1] : -1;
    const size_t o0 = ((size_t)max(i0, 0) * p.Hkv + g) * D, o1 = ((size_t)max(i1, 0) * p.Hkv + g) * D;
    float sc0[REP], sc1[REP], dp0[REP], dp1[REP];
    row_dots2<D, REP>(p.k + o0, p.k + o1, q_s, sc0, sc1);
    row_dots2<D, REP>(p.v + o0, p.v + o1, do_s, dp0, dp1);
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      const float lse = st_s[h];
      const float pr = (i0 < 0 || lse == -INFINITY) ? 0.f : __expf(sc0[h] * p.scale - lse);
      p_s[j * REP + h] = pr;
      ds_s[j * REP + h] = pr * (dp0[h] - st_s[REP + h]) * p.scale;
    }
    if (j1 < p.kk) {
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        const float lse = st_s[h];
        const float pr = (i1 < 0 || lse == -INFINITY) ? 0.f : __expf(sc1[h] * p.scale - lse);
        p_s[j1 * REP + h] = pr;
        ds_s[j1 * REP + h] = pr * (dp1[h] - st_s[REP + h]) * p.scale;
      }
    }
  }
  __syncthreads();
  // ---- phase 2: thread <-> dim: dQ in registers, dK / dV with atomics
  if (tid < D) {
    float dq[REP], qv[REP], dov[REP];
#pragma unroll
    for (int h = 0; h < REP; ++h) { dq[h] = 0.f; qv[h] = q_s[h * D + tid]; dov[h] = do_s[h * D + tid]; }
    constexpr int U = 8;
    for (int j0 = 0; j0 < p.kk; j0 += U) {
      float kv[U];
      int idxs[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int j = j0 + u;
        idxs[u] = j < p.kk ? sel_s[j] : -1;
        kv[u] = __bfloat162float(p.k[((size_t)max(idxs[u], 0) * p.Hkv + g) * D + tid]);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (idxs[u] < 0) continue;
        const int j = j0 + u;
        float dk = 0.f, dv = 0.f;
#pragma unroll
        for (int h = 0; h < REP; ++h) {
          const float ds = ds_s[j * REP + h];
          dq[h] = fmaf(ds, kv[u], dq[h]);
          dk = fmaf(ds, qv[h], dk);
          dv = fmaf(p_s[j * REP + h], dov[h], dv);
        }
        const size_t off = ((size_t)idxs[u] * p.Hkv + g) * D + tid;
        atomicAdd(p.dk + off, dk);
        atomicAdd(p.dv + off, dv);
      }
    }
#pragma unroll
    for (int h = 0; h < REP; ++h) p.dq[row0 + (size_t)h * D + tid] = dq[h];
  }
}

template <int D, int REP>
int launch(const Params& p, bool backward, cudaStream_t st) {
  const size_t smem = backward ? sizeof(float) * (2 * REP * D + 2 * (size_t)p.kk * REP + 2 * REP) + sizeof(int) * p.kk
                               : sizeof(float) * (REP * D + (size_t)p.kk * REP + 2 * REP) + sizeof(int) * p.kk;
  if (smem > 200 * 1024) return -3;
  dim3 grid(p.B, p.Hkv);
  if (backward) {
    if (cudaFuncSetAttribute(dsa_bwd_kernel<D, REP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -4;
    dsa_bwd_kernel<D, REP><<<grid, THREADS, smem, st>>>(p);
  } else {
    if (cudaFuncSetAttribute(dsa_fwd_kernel<D, REP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) return -4;
    dsa_fwd_kernel<D, REP><<<grid, THREADS, smem, st>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int dispatch(const Params& p, int D, int rep, bool backward, cudaStream_t st) {
  if (D == 256 && rep == 8) return launch<256, 8>(p, backward, st);
  if (D == 128 && rep == 4) return launch<128, 4>(p, backward, st);
  if (D == 64 && rep == 2) return launch<64, 2>(p, backward, st);
  return -2;
}
}  // namespace

extern "C" int vlmt_dsa_supported(int D, int rep) { return (D == 256 && rep == 8) || (D == 128 && rep == 4) || (D == 64 && rep == 2); }

extern "C" int vlmt_dsa_fwd(const void* q, const void* k, const void* v, const int* sel, void* o, float* lse, int B, int Hkv, int rep,
                            int D, int kk, float scale, cudaStream_t st) {
  if (B <= 0 || kk <= 0) return 0;
  Params p{};
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.sel = sel;
  p.o = (__nv_bfloat16*)o; p.lse = lse; p.B = B; p.Hkv = Hkv; p.kk = kk; p.scale = scale;
  return dispatch(p, D, rep, false, st);
}

extern "C" int vlmt_dsa_bwd(const void* q, const void* k, const void* v, const int* sel, const void* o, const float* lse, const void* d_o,
                            float* dq, float* dk, float* dv, int B, int Hkv, int rep, int D, int kk, float scale, cudaStream_t st) {
  if (B <= 0 || kk <= 0) return 0;
  Params p{};
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.sel = sel;
  p.o = (__nv_bfloat16*)const_cast<void*>(o); p.lse = const_cast<float*>(lse); p.d_o = (const __nv_bfloat16*)d_o;
  p.dq = dq; p.dk = dk; p.dv = dv; p.B = B; p.Hkv = Hkv; p.kk = kk; p.scale = scale;
  return dispatch(p, D, rep, true, st);
}
