// Cross-entropy over one chunk of logits (forward loss + in-place gradient) and the fused
// AdamW update on flat fp32 master weights with a bf16 parameter write-back.
#include "loss_optim.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {
typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;

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

// One block per row.  Pass 1: online (max, sum-exp) over the row; pass 2: overwrite the row with
// grad_scale * (softmax - onehot) (zeros when the target is ignore_index).  loss[row] = lse - logit[target].
constexpr int CE_THREADS = 512;
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_bwd_kernel(bf16* __restrict__ logits, long ld, const long* __restrict__ targets, float* __restrict__ loss, float grad_scale,
                  int V, long ignore_index) {
  __shared__ float s_m[CE_THREADS / 32], s_s[CE_THREADS / 32];
  __shared__ float s_max, s_lse;
  const long row = blockIdx.x;
  bf16* lr = logits + row * ld;
  const long tgt = targets[row];
  const int nvec = V >> 3;
  const bool vec_ok = ((ld & 7) == 0) && ((V & 7) == 0);
  float m = -INFINITY, s = 0.f;
  auto upd = [&](float x) {
    if (x > m) { s = s * __expf(m - x) + 1.f; m = x; }
    else s += __expf(x - m);
  };
  if (vec_ok) {
    const uint4* lv = reinterpret_cast<const uint4*>(lr);
    for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
      float f[8];
      unpack8(lv[v], f);
      float lm = f[0];
#pragma unroll
      for (int i = 1; i < 8; ++i) lm = fmaxf(lm, f[i]);
      if (lm > m) { s *= __expf(m - lm); m = lm; }
#pragma unroll
      for (int i = 0; i < 8; ++i) s += __expf(f[i] - m);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += CE_THREADS) upd(__bfloat162float(lr[i]));
  }
  // warp then block reduction of (m, s)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if ((threadIdx.x & 31) == 0) { s_m[threadIdx.x >> 5] = m; s_s[threadIdx.x >> 5] = s; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float M = s_m[0], S = s_s[0];
    for (int w = 1; w < CE_THREADS / 32; ++w) {
      const float nm = fmaxf(M, s_m[w]);
      S = (M == -INFINITY ? 0.f : S * __expf(M - nm)) + (s_m[w] == -INFINITY ? 0.f : s_s[w] * __expf(s_m[w] - nm));
      M = nm;
    }
    s_max = M;
    s_lse = M + logf(S);
    const bool valid = tgt != ignore_index && tgt >= 0 && tgt < V;
    loss[row] = valid ? (s_lse - __bfloat162float(lr[tgt])) : 0.f;
  }
  __syncthreads();
  const float lse = s_lse;
  const bool valid = tgt != ignore_index && tgt >= 0 && tgt < V;
  const float sc = valid ? grad_scale : 0.f;
  if (vec_ok) {
    uint4* lv = reinterpret_cast<uint4*>(lr);
    for (int v = threadIdx.x; v < nvec; v += CE_THREADS) {
      float f[8];
      unpack8(lv[v], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float p = __expf(f[i] - lse);
        f[i] = sc * (p - ((long)(v * 8 + i) == tgt ? 1.f : 0.f));
      }
      lv[v] = pack8(f);
    }
  } else {
    for (int i = threadIdx.x; i < V; i += CE_THREADS) {
      const float p = __expf(__bfloat162float(lr[i]) - lse);
      lr[i] = __float2bfloat16(sc * (p - ((long)i == tgt ? 1.f : 0.f)));
    }
  }
}

// AdamW on a flat range: grads bf16 (or fp32), master/m/v fp32, bf16 parameter written back.
//   m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2 ; p = p (1 - lr wd) - lr * (m / bc1) / (sqrt(v / bc2) + eps)
__device__ __forceinline__ float ld_state(const float* p, long i) { return p[i]; }
__device__ __forceinline__ float ld_state(const bf16* p, long i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void st_state(float* p, long i, float x) { p[i] = x; }
__device__ __forceinline__ void st_state(bf16* p, long i, float x) { p[i] = __float2bfloat16(x); }

// GT: gradient type (bf16 / float); MT: moment storage type (float, or bf16 to halve the optimizer state).
// ZERO: also clear the gradient (saves the separate memset of the gradient buffer before the next step).
template <typename GT, typename MT, bool ZERO>
__global__ void adamw_kernel(GT* __restrict__ grad, float* __restrict__ master, MT* __restrict__ m, MT* __restrict__ v,
                             bf16* __restrict__ param, long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                             float grad_scale) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float g;
    if constexpr (sizeof(GT) == 2) g = __bfloat162float(grad[i]) * grad_scale; else g = (float)grad[i] * grad_scale;
    float mi = b1 * ld_state(m, i) + (1.f - b1) * g;
    float vi = b2 * ld_state(v, i) + (1.f - b2) * g * g;
    float p = master[i] * (1.f - lr * wd);
    p -= lr * (mi / bc1) / (sqrtf(vi / bc2) + eps);
    st_state(m, i, mi); st_state(v, i, vi); master[i] = p;
    if (param) param[i] = __float2bfloat16(p);
    if constexpr (ZERO) grad[i] = GT(0.f);
  }
}

// 8 consecutive values as floats <-> memory (16-byte accesses)
struct F8 { float x[8]; };
__device__ __forceinline__ F8 ld8(const float* p) {
  F8 r;
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  r.x[0] = a.x; r.x[1] = a.y; r.x[2] = a.z; r.x[3] = a.w; r.x[4] = b.x; r.x[5] = b.y; r.x[6] = b.z; r.x[7] = b.w;
  return r;
}
__device__ __forceinline__ F8 ld8(const bf16* p) {
  F8 r;
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const bf162* h = reinterpret_cast<const bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); r.x[2 * i] = f.x; r.x[2 * i + 1] = f.y; }
  return r;
}
__device__ __forceinline__ void st8(float* p, const F8& r) {
  reinterpret_cast<float4*>(p)[0] = make_float4(r.x[0], r.x[1], r.x[2], r.x[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(r.x[4], r.x[5], r.x[6], r.x[7]);
}
__device__ __forceinline__ void st8(bf16* p, const F8& r) {
  uint4 u;
  bf162* h = reinterpret_cast<bf162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(r.x[2 * i], r.x[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// The same update on groups of 8 elements with 16-byte loads and stores (all pointers 16-byte aligned, n8 groups).
template <typename GT, typename MT, bool ZERO>
__global__ void adamw_vec8_kernel(GT* __restrict__ grad, float* __restrict__ master, MT* __restrict__ m, MT* __restrict__ v,
                                  bf16* __restrict__ param, long n8, float lr, float b1, float b2, float eps, float wd, float rbc1,
                                  float rbc2, float grad_scale) {
  const float decay = 1.f - lr * wd;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long o = i * 8;
    const F8 g = ld8(grad + o);
    F8 mm = ld8(m + o), vv = ld8(v + o), pp = ld8(master + o);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g.x[k] * grad_scale;
      mm.x[k] = b1 * mm.x[k] + (1.f - b1) * gk;
      vv.x[k] = b2 * vv.x[k] + (1.f - b2) * gk * gk;
      pp.x[k] = pp.x[k] * decay - lr * (mm.x[k] * rbc1) / (sqrtf(vv.x[k] * rbc2) + eps);
    }
    st8(m + o, mm); st8(v + o, vv); st8(master + o, pp);
    if (param) st8(param + o, pp);
    if constexpr (ZERO) {
      F8 z;
#pragma unroll
      for (int k = 0; k < 8; ++k) z.x[k] = 0.f;
      st8(grad + o, z);
    }
  }
}

// out[c] = sum_r x[r, c]  (bf16 in, fp32 accumulate): one thread per column pair inside a row slab, partials per slab
__global__ void __launch_bounds__(256) colsum_kernel(const bf16* __restrict__ x, long ld, int rows, int cols, float* __restrict__ partial,
                                                      int rows_per_slab) {
  // block = 8 warps on the same 256 columns (lane <-> 8 columns, one 16-byte load per row); warp w takes rows w, w + 8, ...
  // of the slab, eight loads in flight; the warps' sums meet in shared memory
  __shared__ float red[8][256];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 256 + lane * 8;
  const int r0 = blockIdx.y * rows_per_slab;
  const int r1 = min(rows, r0 + rows_per_slab);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (c < cols) {   // cols is a multiple of 8: a thread's 8 columns are all inside or all outside
    int r = r0 + warp;
    for (; r + 56 < r1; r += 64) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = *reinterpret_cast<const uint4*>(x + (long)(r + 8 * u) * ld + c);
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const uint32_t w4[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[2 * j] += __uint_as_float(w4[j] << 16);
          acc[2 * j + 1] += __uint_as_float(w4[j] & 0xffff0000u);
        }
      }
    }
    for (; r < r1; r += 8) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + (long)r * ld + c);
      const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __uint_as_float(w4[j] << 16);
        acc[2 * j + 1] += __uint_as_float(w4[j] & 0xffff0000u);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[warp][lane * 8 + i] = acc[i];
  __syncthreads();
  const int cc = blockIdx.x * 256 + threadIdx.x;
  if (cc < cols) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w][threadIdx.x];
    partial[(long)blockIdx.y * cols + cc] = t;
  }
}

// out[c] = sum of the slabs' partial sums
__global__ void colsum_finish_kernel(const float* __restrict__ partial, int slabs, int cols, float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float t = 0.f;
  for (int sl = 0; sl < slabs; ++sl) t += partial[(long)sl * cols + c];
  out[c] = t;
}

// out[c] = sum over many partial rows (the per-block weight-gradient sums of the norm kernels: a few hundred rows).
// A block owns 16 columns; its 256 threads are 16 row lanes x 16 columns, lane j adds rows j, j + 16, ... and the 16 lane
// sums are added in lane order, so the result does not depend on timing.
__global__ void __launch_bounds__(256) sum_rows_kernel(const float* __restrict__ partial, int rows, int cols, float* __restrict__ out) {
  __shared__ float sm[16][17];
  const int cl = threadIdx.x & 15, lane = threadIdx.x >> 4;
  const int c = blockIdx.x * 16 + cl;
  float t0 = 0.f, t1 = 0.f, t2 = 0.f, t3 = 0.f;
  if (c < cols) {
    int r = lane;
    for (; r + 48 < rows; r += 64) {   // four independent loads in flight per thread
      t0 += partial[(long)r * cols + c];
      t1 += partial[(long)(r + 16) * cols + c];
      t2 += partial[(long)(r + 32) * cols + c];
      t3 += partial[(long)(r + 48) * cols + c];
    }
    for (; r < rows; r += 16) t0 += partial[(long)r * cols + c];
  }
  sm[lane][cl] = (t0 + t1) + (t2 + t3);
  __syncthreads();
  if (lane == 0 && c < cols) {
    float t = 0.f;
#pragma unroll
    for (int j = 0; j < 16; ++j) t += sm[j][cl];
    out[c] = t;
  }
}

// sum of squares of a flat bf16/fp32 range -> out[0] (atomic; used for gradient clipping)
template <typename GT>
__global__ void sumsq_kernel(const GT* __restrict__ x, long n, float* __restrict__ out) {
  float acc = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float f;
    if constexpr (sizeof(GT) == 2) f = __bfloat162float(x[i]); else f = (float)x[i];
    acc += f * f;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float sm[32];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += sm[w];
    atomicAdd(out, t);
  }
}
}  // namespace

extern "C" {
void vlmt_ce_fwd_bwd(void* logits, long ld, const long* targets, float* loss, float grad_scale, int rows, int V, long ignore_index,
                     cudaStream_t st) {
  if (rows <= 0) return;
  ce_fwd_bwd_kernel<<<rows, CE_THREADS, 0, st>>>(reinterpret_cast<bf16*>(logits), ld, targets, loss, grad_scale, V, ignore_index);
}
void vlmt_adamw(void* grad, int grad_fp32, float* master, void* m, void* v, int state_bf16, void* param, long n, float lr, float b1,
                float b2, float eps, float wd, float bc1, float bc2, float grad_scale, int zero_grad, cudaStream_t st) {
  if (n <= 0) return;
  bf16* pp = reinterpret_cast<bf16*>(param);
  const uintptr_t bits = (uintptr_t)grad | (uintptr_t)master | (uintptr_t)m | (uintptr_t)v | (uintptr_t)param;
  const long n8 = (bits & 15) == 0 ? n / 8 : 0;   // groups of 8 handled with 16-byte accesses
  const long done = n8 * 8;
#define LAUNCH(GT, MT, Z)                                                                                                         \
  do {                                                                                                                            \
    if (n8 > 0) {                                                                                                                 \
      long blocks = (n8 + 255) / 256;                                                                                             \
      if (blocks > 148 * 8) blocks = 148 * 8;                                                                                     \
      adamw_vec8_kernel<GT, MT, Z><<<(int)blocks, 256, 0, st>>>((GT*)grad, master, (MT*)m, (MT*)v, pp, n8, lr, b1, b2, eps, wd,   \
                                                                 1.f / bc1, 1.f / bc2, grad_scale);                                \
    }                                                                                                                             \
    if (done < n) {                                                                                                               \
      long blocks = (n - done + 255) / 256;                                                                                       \
      if (blocks > 148 * 16) blocks = 148 * 16;                                                                                   \
      adamw_kernel<GT, MT, Z><<<(int)blocks, 256, 0, st>>>((GT*)grad + done, master + done, (MT*)m + done, (MT*)v + done,         \
                                                            pp ? pp + done : nullptr, n - done, lr, b1, b2, eps, wd, bc1, bc2,     \
                                                            grad_scale);                                                           \
    }                                                                                                                             \
  } while (0)
#define PICK(GT, MT) do { if (zero_grad) LAUNCH(GT, MT, true); else LAUNCH(GT, MT, false); } while (0)
  if (grad_fp32) { if (state_bf16) PICK(float, bf16); else PICK(float, float); }
  else { if (state_bf16) PICK(bf16, bf16); else PICK(bf16, float); }
#undef PICK
#undef LAUNCH
}
int vlmt_colsum_slabs(int rows) { int s = (rows + 255) / 256; return s < 1 ? 1 : s; }
// column sums of x [rows, cols] (cols a multiple of 8, 16-byte aligned rows): `partial` holds vlmt_colsum_slabs(rows) x cols floats
void vlmt_colsum(const void* x, long ld, int rows, int cols, float* partial, float* out, cudaStream_t st) {
  if (cols <= 0) return;
  const int slabs = rows > 0 ? vlmt_colsum_slabs(rows) : 0;
  if (slabs > 0) {
    dim3 grid((cols + 255) / 256, slabs);
    colsum_kernel<<<grid, 256, 0, st>>>(reinterpret_cast<const bf16*>(x), ld, rows, cols, partial, 256);
  }
  colsum_finish_kernel<<<(cols + 255) / 256, 256, 0, st>>>(partial, slabs, cols, out);
}
// out[c] = sum over `rows` partial rows (the per-block weight-gradient sums of the norm kernels)
void vlmt_sum_rows_f32(const float* partial, int rows, int cols, float* out, cudaStream_t st) {
  if (cols <= 0) return;
  sum_rows_kernel<<<(cols + 15) / 16, 256, 0, st>>>(partial, rows, cols, out);
}
void vlmt_sumsq(const void* x, int fp32, long n, float* out, cudaStream_t st) {
  if (n <= 0) return;
  long blocks = (n + 1023) / 1024;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (fp32) sumsq_kernel<float><<<(int)blocks, 256, 0, st>>>((const float*)x, n, out);
  else sumsq_kernel<bf16><<<(int)blocks, 256, 0, st>>>((const bf16*)x, n, out);
}
}
