// Collectives fused with their adjacent compute, over NVLink / NVSwitch peer memory.
//
// fused_rs_adamw_ag: ONE kernel per bucket does gradient reduce-scatter + fp32 AdamW + parameter
// all-gather.  Every rank owns a contiguous shard [lo, hi) of the bucket.  For its shard it
//   1. reads the bf16 gradients of ALL ranks (plain 16-byte peer loads, or one multimem.ld_reduce
//      through the switch when a multicast mapping is available) and sums them in fp32,
//   2. updates its fp32 master weights and Adam moments (local HBM),
//   3. stores the new bf16 parameters into the flat parameter buffer of EVERY rank
//      (peer stores, or one multimem.st).
// Gradient bytes cross NVLink once, parameter bytes once; nothing is staged.  The kernel contains
// no waits: the caller orders it behind a one-block wait kernel on the same stream that returns once every
// peer's "gradients of this bucket are final" flag has arrived (signal_peers / wait_flags below).  If that
// wait, or any earlier bounded wait, ran out, the device status word is non-zero and the kernel returns
// without touching the optimizer state, so a lost peer can never corrupt master weights or moments.
//
// peer_sum_rows: out[r, :] = sum over ranks of partial_rank[r, :] for the rows a rank owns
// (tensor-parallel reduce-scatter), optionally fused with a residual add.
#include "comm_kernels.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {
typedef __nv_bfloat16 bf16;
typedef __nv_bfloat162 bf162;
constexpr int MAX_PEERS = 16;

struct PeerPtrs {
  void* p[MAX_PEERS];
};

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
__device__ __forceinline__ uint4 ld_peer_16B(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// sum of 8 bf16 over all devices of the multicast group, accumulated in fp32 inside the switch
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_ptr) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_ptr) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_st_16B(void* mc_ptr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

struct AdamArgs {
  float lr, b1, b2, eps, wd, bc1, bc2, grad_scale;
};

// 8 consecutive Adam moments, stored as fp32 or bf16
__device__ __forceinline__ void load_state8(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load_state8(const bf16* p, float (&f)[8]) { unpack8(*reinterpret_cast<const uint4*>(p), f); }
__device__ __forceinline__ void store_state8(float* p, const float (&f)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ void store_state8(bf16* p, const float (&f)[8]) { *reinterpret_cast<uint4*>(p) = pack8(f); }

// elements [lo, hi) of the bucket-relative flat buffers; lo, hi multiples of 8.  ST: storage type of the Adam moments
// (fp32, or bf16 to save 4 bytes per parameter; master weights are fp32 either way).  zero_own: also clear this rank's
// copy of the gradients it consumed (world 1: every gradient, so the next step needs no separate clearing pass).
template <bool MULTIMEM, typename ST>
__global__ void fused_rs_adamw_ag_kernel(PeerPtrs grads, PeerPtrs params, void* grad_mc, void* param_mc, int world, long lo, long hi,
                                         float* __restrict__ master, ST* __restrict__ m, ST* __restrict__ v, AdamArgs a,
                                         const int* __restrict__ status, int zero_own) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;  // an earlier wait gave up
  const long nvec = (hi - lo) >> 3;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long e = lo + (i << 3);
    float g[8];
    if (MULTIMEM) {
      unpack8(multimem_ld_reduce_bf16x8(reinterpret_cast<const bf16*>(grad_mc) + e), g);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = 0.f;
      for (int r = 0; r < world; ++r) {
        float t[8];
        unpack8(ld_peer_16B(reinterpret_cast<const bf16*>(grads.p[r]) + e), t);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] += t[k];
      }
      if (zero_own && world == 1) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(grads.p[0]) + e) = make_uint4(0u, 0u, 0u, 0u);
    }
    const long s = i << 3;  // offset into the local shard state
    float pm[8], mm[8], vv[8];
    load_state8(master + s, pm);
    load_state8(m + s, mm);
    load_state8(v + s, vv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g[k] * a.grad_scale;
      mm[k] = a.b1 * mm[k] + (1.f - a.b1) * gk;
      vv[k] = a.b2 * vv[k] + (1.f - a.b2) * gk * gk;
      float p = pm[k] * (1.f - a.lr * a.wd);
      p -= a.lr * (mm[k] / a.bc1) / (sqrtf(vv[k] / a.bc2) + a.eps);
      pm[k] = p;
    }
    store_state8(master + s, pm);
    store_state8(m + s, mm);
    store_state8(v + s, vv);
    const uint4 packed = pack8(pm);
    if (MULTIMEM) {
      multimem_st_16B(reinterpret_cast<bf16*>(param_mc) + e, packed);
    } else {
      for (int r = 0; r < world; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(params.p[r]) + e) = packed;
    }
  }
}

// ---- the same step in two kernels, for gradient clipping (the global norm must be known before the first update) ----
// reduce: red[i] = sum over ranks of grad_r[lo + i] (kept in fp32), sumsq += sum red[i]^2 (one atomicAdd per block)
template <bool MULTIMEM>
__global__ void rs_reduce_sumsq_kernel(PeerPtrs grads, void* grad_mc, int world, long lo, long hi, float* __restrict__ red,
                                       float* __restrict__ sumsq, const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  const long nvec = (hi - lo) >> 3;
  float local = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long e = lo + (i << 3);
    float g[8];
    if (MULTIMEM) {
      unpack8(multimem_ld_reduce_bf16x8(reinterpret_cast<const bf16*>(grad_mc) + e), g);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = 0.f;
      for (int r = 0; r < world; ++r) {
        float t[8];
        unpack8(ld_peer_16B(reinterpret_cast<const bf16*>(grads.p[r]) + e), t);
#pragma unroll
        for (int k = 0; k < 8; ++k) g[k] += t[k];
      }
    }
    store_state8(red + (i << 3), g);
#pragma unroll
    for (int k = 0; k < 8; ++k) local += g[k] * g[k];
  }
  __shared__ float warp_part[8];
#pragma unroll
  for (int o = 16; o; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0) warp_part[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += warp_part[w];
    atomicAdd(sumsq, t);
  }
}

// update: AdamW on the shard from the reduced gradient `red`, scaled by grad_scale and by the clip factor
// min(1, max_norm / (grad_scale * sqrt(*sumsq) + 1e-6)) read from device memory; new parameters go to every rank
template <bool MULTIMEM, typename ST>
__global__ void adamw_push_kernel(const float* __restrict__ red, const float* __restrict__ sumsq, float max_norm, PeerPtrs params,
                                  void* param_mc, int world, long lo, long hi, float* __restrict__ master, ST* __restrict__ m,
                                  ST* __restrict__ v, AdamArgs a, const int* __restrict__ status) {
  if (status != nullptr && *reinterpret_cast<const volatile int*>(status) != 0) return;
  const float norm = a.grad_scale * sqrtf(*sumsq);
  const float clip = fminf(1.f, max_norm / (norm + 1e-6f));
  const float gs = a.grad_scale * clip;
  const long nvec = (hi - lo) >> 3;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long e = lo + (i << 3);
    const long s = i << 3;
    float g[8], pm[8], mm[8], vv[8];
    load_state8(red + s, g);
    load_state8(master + s, pm);
    load_state8(m + s, mm);
    load_state8(v + s, vv);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g[k] * gs;
      mm[k] = a.b1 * mm[k] + (1.f - a.b1) * gk;
      vv[k] = a.b2 * vv[k] + (1.f - a.b2) * gk * gk;
      float p = pm[k] * (1.f - a.lr * a.wd);
      p -= a.lr * (mm[k] / a.bc1) / (sqrtf(vv[k] / a.bc2) + a.eps);
      pm[k] = p;
    }
    store_state8(master + s, pm);
    store_state8(m + s, mm);
    store_state8(v + s, vv);
    const uint4 packed = pack8(pm);
    if (MULTIMEM) {
      multimem_st_16B(reinterpret_cast<bf16*>(param_mc) + e, packed);
    } else {
      for (int r = 0; r < world; ++r) *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(params.p[r]) + e) = packed;
    }
  }
}

// out[row, :] = (residual ? residual[row, :] : 0) + sum_r partial_r[row0 + row, :]   (bf16, fp32 accumulation)
__global__ void peer_sum_rows_kernel(PeerPtrs partials, int world, long row0, long rows, int D, const bf16* __restrict__ residual,
                                     bf16* __restrict__ out) {
  const int vper = D >> 3;
  const long nvec = rows * vper;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    const long row = i / vper;
    const int c = (int)(i - row * vper);
    float acc[8];
    if (residual) unpack8(reinterpret_cast<const uint4*>(residual + row * D)[c], acc);
    else {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    }
    for (int r = 0; r < world; ++r) {
      float t[8];
      unpack8(ld_peer_16B(reinterpret_cast<const bf16*>(partials.p[r]) + (row0 + row) * D + c * 8), t);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += t[k];
    }
    reinterpret_cast<uint4*>(out + row * D)[c] = pack8(acc);
  }
}
// ------------------------------------------------------------------------------------ signalled P2P collectives
// Protocol (per process group, collectives numbered 1, 2, ... in program order, identical on every rank):
//   every rank copies its contribution into slot (e % n_slots) of its symmetric staging buffer, then `signal`
//   stores e into flag[my_rank] on EVERY rank (release, system scope); the pull kernel of collective e first
//   waits (bounded, see g_flag_wait_ns) until all of its own flag[r] >= e, then reads the peers' slots directly over NVLink.
// A slot is reused n_slots collectives later, by which time every peer has issued (in stream order, after its
// pull) the signals of the collectives in between, so no extra "done" handshake is needed.
// Wall-clock bound of a flag wait.  Long enough for an ordinary straggler (a rank that saves a checkpoint, a slow data
// batch, first-step allocation), short enough that a rank that is gone shows up as an error and not as a hung job.
// Set once per process from the host (environment variable VLMT_FLAG_WAIT_MS, default 20 s).
__device__ unsigned long long g_flag_wait_ns = 20000000000ull;

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned long long gtimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// block-wide: returns false (and records status 100 + rank of the missing peer) when a peer's signal did not arrive in time
// `skip` (a rank or -1): that rank's flag is not waited for.  A rank must not wait in one kernel for a signal that a
// SEPARATE launch on the same GPU still has to store (nothing guarantees that the two launches run concurrently);
// its own readiness is established by stream order instead.
__device__ bool wait_all_flags(const int* my_flags, int world, int epoch, int* status, int skip = -1) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const unsigned long long t0 = gtimer_ns();
    for (int r = 0; r < world && ok; ++r) {
      if (r == skip) continue;
      unsigned spins = 0;
      while (ld_acquire_sys(my_flags + r) < epoch) {
        if ((++spins & 0xff) == 0 && gtimer_ns() - t0 > g_flag_wait_ns) {
          atomicCAS(status, 0, 100 + r);
          ok = 0;
          break;
        }
      }
    }
  }
  __syncthreads();
  return ok != 0;
}

__global__ void signal_peers_kernel(PeerPtrs flag_ptrs, int world, int my_rank, int epoch) {
  if ((int)threadIdx.x < world) {
    __threadfence_system();  // everything this stream wrote before (the staging copy) is visible system-wide first
    st_release_sys(reinterpret_cast<int*>(flag_ptrs.p[threadIdx.x]) + my_rank, epoch);
  }
}

// stand-alone wait: later kernels of the stream start only after every rank stored `epoch` (or the wait timed out)
__global__ void wait_flags_kernel(const int* my_flags, int world, int epoch, int* status, int skip) {
  wait_all_flags(my_flags, world, epoch, status, skip);
}

// all-gather: out[r * n : (r + 1) * n] = slot of rank r   (n elements per rank, multiple of 8)
__global__ void pull_gather_kernel(PeerPtrs slots, bf16* __restrict__ out, long n, int world, const int* my_flags, int epoch,
                                   int* status) {
  if (!wait_all_flags(my_flags, world, epoch, status)) return;
  // Few blocks (two per SM) with four 16-byte loads in flight per thread: enough bytes in flight to fill NVLink, and few
  // enough registers and threads that the blocks share the SMs with a GEMM running on another stream.
  const long nvec = n >> 3;
  const long stride = (long)gridDim.x * blockDim.x;
  for (int r = 0; r < world; ++r) {
    const uint4* src = reinterpret_cast<const uint4*>(slots.p[r]);
    uint4* dst = reinterpret_cast<uint4*>(out) + (long)r * nvec;
    long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      const uint4 a = ld_peer_16B(src + i), b = ld_peer_16B(src + i + stride), c = ld_peer_16B(src + i + 2 * stride),
                  d = ld_peer_16B(src + i + 3 * stride);
      dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
    }
    for (; i < nvec; i += stride) dst[i] = ld_peer_16B(src + i);
  }
}

// the elements [lo, hi) of the gathered array only (out[r * n + j] = slot_r[j]); no flags: the slots do not change meanwhile
__global__ void pull_gather_range_kernel(PeerPtrs slots, bf16* __restrict__ out, long n, int world, long lo, long hi) {
  const long stride = (long)gridDim.x * blockDim.x;
  for (int r = 0; r < world; ++r) {
    const long a = max(lo, (long)r * n), b = min(hi, (long)(r + 1) * n);
    if (b <= a) continue;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const bf16*>(slots.p[r]) + (a - (long)r * n));
    uint4* dst = reinterpret_cast<uint4*>(out + a);
    const long nvec = (b - a) >> 3;
    long i = blockIdx.x * (long)blockDim.x + threadIdx.x;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      const uint4 v0 = ld_peer_16B(src + i), v1 = ld_peer_16B(src + i + stride), v2 = ld_peer_16B(src + i + 2 * stride),
                  v3 = ld_peer_16B(src + i + 3 * stride);
      dst[i] = v0; dst[i + stride] = v1; dst[i + 2 * stride] = v2; dst[i + 3 * stride] = v3;
    }
    for (; i < nvec; i += stride) dst[i] = ld_peer_16B(src + i);
  }
}

// reduce-scatter: out[0:n] = (residual) + sum_r slot_r[me * n : (me + 1) * n]   (own slot included; fp32 accumulation)
// With `pushed` the producers already stored their blocks into THIS rank's slot (block r from rank r): slots.p[r] then
// points at local memory and the reads stay on this GPU.
__global__ void pull_reduce_kernel(PeerPtrs slots, bf16* __restrict__ out, const bf16* __restrict__ residual, long n, int world,
                                   int my_rank, const int* my_flags, int epoch, int* status) {
  if (!wait_all_flags(my_flags, world, epoch, status)) return;
  const long nvec = n >> 3;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += (long)gridDim.x * blockDim.x) {
    float acc[8];
    if (residual) unpack8(reinterpret_cast<const uint4*>(residual)[i], acc);
    else {
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] = 0.f;
    }
    for (int r = 0; r < world; ++r) {
      float t[8];
      unpack8(ld_peer_16B(reinterpret_cast<const uint4*>(slots.p[r]) + (long)my_rank * nvec + i), t);
#pragma unroll
      for (int k = 0; k < 8; ++k) acc[k] += t[k];
    }
    reinterpret_cast<uint4*>(out)[i] = pack8(acc);
  }
}
}  // namespace

extern "C" {
int vlmt_set_flag_wait_ms(long ms) {
  const unsigned long long ns = (unsigned long long)(ms < 1 ? 1 : ms) * 1000000ull;
  return (int)cudaMemcpyToSymbol(g_flag_wait_ns, &ns, sizeof(ns));
}
int vlmt_signal_peers(void* const* flag_ptrs, int world, int my_rank, int epoch, cudaStream_t st) {
  if (world > MAX_PEERS) return -1;
  PeerPtrs f;
  for (int r = 0; r < world; ++r) f.p[r] = flag_ptrs[r];
  signal_peers_kernel<<<1, 32, 0, st>>>(f, world, my_rank, epoch);
  return (int)cudaGetLastError();
}
int vlmt_wait_flags(const int* my_flags, int world, int epoch, int skip_rank, int* status, cudaStream_t st) {
  wait_flags_kernel<<<1, 32, 0, st>>>(my_flags, world, epoch, status, skip_rank);
  return (int)cudaGetLastError();
}
int vlmt_pull_gather(void* const* slot_ptrs, void* out, long n_per_rank, int world, const int* my_flags, int epoch, int* status,
                     cudaStream_t st) {
  if (world > MAX_PEERS || (n_per_rank & 7)) return -1;
  PeerPtrs s;
  for (int r = 0; r < world; ++r) s.p[r] = slot_ptrs[r];
  long blocks = ((n_per_rank >> 3) + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;
  pull_gather_kernel<<<(int)blocks, 256, 0, st>>>(s, reinterpret_cast<bf16*>(out), n_per_rank, world, my_flags, epoch, status);
  return (int)cudaGetLastError();
}
int vlmt_pull_gather_range(void* const* slot_ptrs, void* out, long n_per_rank, int world, long lo, long hi, cudaStream_t st) {
  if (world > MAX_PEERS || (n_per_rank & 7) || (lo & 7) || (hi & 7)) return -1;
  if (hi <= lo) return 0;
  PeerPtrs s;
  for (int r = 0; r < world; ++r) s.p[r] = slot_ptrs[r];
  long blocks = (((hi - lo) >> 3) + 255) / 256;
  if (blocks > 148 * 2) blocks = 148 * 2;
  pull_gather_range_kernel<<<(int)blocks, 256, 0, st>>>(s, reinterpret_cast<bf16*>(out), n_per_rank, world, lo, hi);
  return (int)cudaGetLastError();
}
int vlmt_pull_reduce(void* const* slot_ptrs, void* out, const void* residual, long n_per_rank, int world, int my_rank,
                     const int* my_flags, int epoch, int* status, cudaStream_t st) {
  if (world > MAX_PEERS || (n_per_rank & 7)) return -1;
  PeerPtrs s;
  for (int r = 0; r < world; ++r) s.p[r] = slot_ptrs[r];
  long blocks = ((n_per_rank >> 3) + 255) / 256;
  if (blocks > 148 * 4) blocks = 148 * 4;
  pull_reduce_kernel<<<(int)blocks, 256, 0, st>>>(s, reinterpret_cast<bf16*>(out), reinterpret_cast<const bf16*>(residual), n_per_rank,
                                                  world, my_rank, my_flags, epoch, status);
  return (int)cudaGetLastError();
}
int vlmt_fused_rs_adamw_ag(void* const* grad_ptrs, void* const* param_ptrs, void* grad_mc, void* param_mc, int world, long lo, long hi,
                           float* master, void* m, void* v, int state_bf16, float lr, float b1, float b2, float eps, float wd, float bc1,
                           float bc2, float grad_scale, int zero_own, const int* status, cudaStream_t st) {
  if (world > MAX_PEERS) return -1;
  if ((lo & 7) || (hi & 7)) return -2;
  if (hi <= lo) return 0;
  PeerPtrs g, p;
  for (int r = 0; r < world; ++r) { g.p[r] = grad_ptrs[r]; p.p[r] = param_ptrs[r]; }
  AdamArgs a{lr, b1, b2, eps, wd, bc1, bc2, grad_scale};
  long blocks = (((hi - lo) >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  const bool mc = grad_mc && param_mc;
#define LAUNCH(MC, ST)                                                                                                          \
  fused_rs_adamw_ag_kernel<MC, ST><<<(int)blocks, 256, 0, st>>>(g, p, mc ? grad_mc : nullptr, mc ? param_mc : nullptr, world, lo, hi, \
                                                                master, reinterpret_cast<ST*>(m), reinterpret_cast<ST*>(v), a, status, zero_own)
  if (state_bf16) { if (mc) LAUNCH(true, bf16); else LAUNCH(false, bf16); }
  else { if (mc) LAUNCH(true, float); else LAUNCH(false, float); }
#undef LAUNCH
  return (int)cudaGetLastError();
}
int vlmt_rs_reduce_sumsq(void* const* grad_ptrs, void* grad_mc, int world, long lo, long hi, float* red, float* sumsq, const int* status,
                         cudaStream_t st) {
  if (world > MAX_PEERS) return -1;
  if ((lo & 7) || (hi & 7)) return -2;
  if (hi <= lo) return 0;
  PeerPtrs g;
  for (int r = 0; r < world; ++r) g.p[r] = grad_ptrs[r];
  long blocks = (((hi - lo) >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  if (grad_mc) rs_reduce_sumsq_kernel<true><<<(int)blocks, 256, 0, st>>>(g, grad_mc, world, lo, hi, red, sumsq, status);
  else rs_reduce_sumsq_kernel<false><<<(int)blocks, 256, 0, st>>>(g, nullptr, world, lo, hi, red, sumsq, status);
  return (int)cudaGetLastError();
}
int vlmt_adamw_push(const float* red, const float* sumsq, float max_norm, void* const* param_ptrs, void* param_mc, int world, long lo,
                    long hi, float* master, void* m, void* v, int state_bf16, float lr, float b1, float b2, float eps, float wd, float bc1,
                    float bc2, float grad_scale, const int* status, cudaStream_t st) {
  if (world > MAX_PEERS) return -1;
  if ((lo & 7) || (hi & 7)) return -2;
  if (hi <= lo) return 0;
  PeerPtrs p;
  for (int r = 0; r < world; ++r) p.p[r] = param_ptrs[r];
  AdamArgs a{lr, b1, b2, eps, wd, bc1, bc2, grad_scale};
  long blocks = (((hi - lo) >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
#define LAUNCH(MC, ST)                                                                                                   \
  adamw_push_kernel<MC, ST><<<(int)blocks, 256, 0, st>>>(red, sumsq, max_norm, p, MC ? param_mc : nullptr, world, lo, hi, master, \
                                                         reinterpret_cast<ST*>(m), reinterpret_cast<ST*>(v), a, status)
  if (state_bf16) { if (param_mc) LAUNCH(true, bf16); else LAUNCH(false, bf16); }
  else { if (param_mc) LAUNCH(true, float); else LAUNCH(false, float); }
#undef LAUNCH
  return (int)cudaGetLastError();
}
int vlmt_peer_sum_rows(void* const* partial_ptrs, int world, long row0, long rows, int D, const void* residual, void* out, cudaStream_t st) {
  if (world > MAX_PEERS || (D & 7)) return -1;
  if (rows <= 0) return 0;
  PeerPtrs p;
  for (int r = 0; r < world; ++r) p.p[r] = partial_ptrs[r];
  long blocks = (rows * (D >> 3) + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  peer_sum_rows_kernel<<<(int)blocks, 256, 0, st>>>(p, world, row0, rows, D, reinterpret_cast<const bf16*>(residual),
                                                    reinterpret_cast<bf16*>(out));
  return (int)cudaGetLastError();
}
}
