// Selected-key attention for DSA on the tensor cores (sm_100a), head size 256 with 8 query heads per kv head.
//
// Every query attends to its own list of key rows, so the only matrix a query shares with anything is its own
// [8 heads x 256] block of q.  Putting that on tcgen05 means turning the products around: the 128 gathered key rows of a
// tile are the M dimension, the query heads the (small) N dimension:
//
//     S^T [128 keys, 16]  = K_sel [128, 256] . Q^T        A = gathered key tile (K-major), B = q block, N = 16 (8 real heads)
//     O^T [256, 16]      += V_sel^T [256, 128] . P         A = gathered value tile read MN-major (two M = 128 halves), B = P^T
//
// One CTA per (query, kv head), 256 threads.  All warps gather: every selected row is 512 contiguous bytes, copied with
// 16-byte cp.async into the 128-byte-swizzle layout the MMA descriptors expect (one warp per row and instruction).  The
// key tile has two buffers and the value tile one, so a gather is always in flight: K(t+1) streams in from the moment
// tile t starts, V(t+1) while S(t+1) and its softmax are computed.  Warps 0-3 own the TMEM lanes:
// they read S^T (lane = key), keep a running maximum per head across the CTA (online softmax; the accumulator O^T has
// only 16 columns, so rescaling it costs 32 values per thread), write P^T as the next B operand and, at the end, divide
// O^T (lane = channel) by the row sums.  Rows 8-15 of both B operands are whatever follows in shared memory: they only
// reach accumulator columns that nobody reads.
//
// Every wait is bounded; a wait that runs out sets the status word and the CTA leaves through the common teardown.
#include "dsa_attention.h"
#include "sm100.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace {
using namespace sm100;

constexpr int D = 256, REP = 8, TK = 128, THREADS = 256;
constexpr int kRowBlk = TK * 128;        // one 64-channel block of a gathered tile: 128 rows x 128 bytes
constexpr int kTile = 4 * kRowBlk;       // [128 x 256] bf16
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]) : "r"(taddr));
}
__device__ __forceinline__ void bar_sync_128() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct Params {
  const __nv_bfloat16* q;    // [B, Hkv * 8, 256]
  const __nv_bfloat16* k;    // [L, Hkv, 256]
  const __nv_bfloat16* v;
  const int* sel;            // [B, kk], -1 = unused
  __nv_bfloat16* o;
  float* lse;                // natural-log sum-exp of the scaled scores
  int B, Hkv, kk;
  float scale;
  int* status;
};

struct Smem {
  // two key buffers (the next tile's keys stream in while this tile's scores are computed), one value buffer
  static constexpr int offK = 0, offV = offK + 2 * kTile, offQ = offV + kTile;   // q block: 4 channel blocks x [8 rows x 128 B]
  static constexpr int offP = offQ + 4 * 1024;                                  // P^T: 2 key blocks x [8 rows x 128 B]
  static constexpr int offF = offP + 2 * 1024 + 1024;                           // floats: wm [4][8], m_run [8], alpha [8], lsum [8]
  static constexpr int offCtl = offF + (32 + 24) * 4;
  static constexpr int offSel = offCtl + 64;
};

__global__ void __launch_bounds__(THREADS, 1) dsa_tc_fwd_kernel(Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* wm = reinterpret_cast<float*>(smem + Smem::offF);
  float* m_run = wm + 32;
  float* alpha_s = m_run + 8;
  float* lsum = alpha_s + 8;
  uint64_t* bar_s = reinterpret_cast<uint64_t*>(smem + Smem::offCtl);
  uint64_t* bar_o = bar_s + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_s + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* sel_s = reinterpret_cast<int*>(smem + Smem::offSel);

  const int b = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Hq = p.Hkv * REP;
  const int nt = (p.kk + TK - 1) / TK;
  constexpr int TMEM_COLS = 64, S_COL = 0, O_COL = 16;

  if (tid == 0) {
    mbar_init(bar_s, 1);
    mbar_init(bar_o, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc<TMEM_COLS>(tmem_slot);
  for (int j = tid; j < nt * TK; j += THREADS) sel_s[j] = j < p.kk ? p.sel[(size_t)b * p.kk + j] : -1;
  {  // q block as a K-major B operand: row = head, 16-byte group c of the 512-byte row
    const int h = tid >> 5, c = tid & 31;
    const uint4 val = *reinterpret_cast<const uint4*>(p.q + ((size_t)b * Hq + g * REP + h) * D + c * 8);
    *reinterpret_cast<uint4*>(smem + Smem::offQ + (c >> 3) * 1024 + h * 128 + (((c & 7) ^ h) << 4)) = val;
  }
  if (tid < 8) { m_run[tid] = -INFINITY; lsum[tid] = 0.f; }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // one warp copies one 512-byte row per instruction; an unused slot is zero-filled
  auto gather = [&](const __nv_bfloat16* src, uint8_t* dst, int t) {
#pragma unroll 4
    for (int i = 0; i < TK / 8; ++i) {
      const int r = i * 8 + warp;
      const int idx = sel_s[t * TK + r];
      const __nv_bfloat16* row = src + ((size_t)max(idx, 0) * p.Hkv + g) * D + lane * 8;
      cp_async16(dst + (lane >> 3) * kRowBlk + r * 128 + (((lane & 7) ^ (r & 7)) << 4), row, idx >= 0 ? 16 : 0);
    }
    cp_async_commit();
  };

  const float scale_log2 = p.scale * kLog2e;
  float l_thread[REP];
#pragma unroll
  for (int h = 0; h < REP; ++h) l_thread[h] = 0.f;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t idesc_s = make_idesc_bf16(128, 16, false, false), idesc_o = make_idesc_bf16(128, 16, true, false);

  gather(p.k, smem + Smem::offK, 0);
  gather(p.v, smem + Smem::offV, 0);
  bool ok = true;
  for (int t = 0; t < nt && ok; ++t) {
    // K(t+1) goes into the other key buffer, last read by the scores of tile t-1 (complete: their barrier was waited for)
    if (t + 1 < nt) gather(p.k, smem + Smem::offK + ((t + 1) & 1) * kTile, t + 1); else cp_async_commit();
    cp_async_wait<2>();          // K(t) has landed; V(t) and K(t+1) may still be in flight
    fence_async_proxy();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const SmemDesc a0 = make_desc(smem_u32(smem + Smem::offK + (t & 1) * kTile), 16, 1024), b0 = make_desc(smem_u32(smem + Smem::offQ), 16, 1024);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const SmemDesc a = desc_off(a0, (kk >> 2) * kRowBlk + (kk & 3) * 32), bb = desc_off(b0, (kk >> 2) * 1024 + (kk & 3) * 32);
        if (kk == 0) umma_ss<0>(tmem_base + S_COL, a, bb, idesc_s); else umma_ss<1>(tmem_base + S_COL, a, bb, idesc_s);
      }
      umma_commit(bar_s);
    }
    ok = mbar_wait(bar_s, t & 1, abort_flag, p.status, kErrTimeoutTmemFull);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after();
    if (warp < 4) {
      // ---- online softmax of this tile: thread <-> key
      const int r = tid;
      const bool valid = sel_s[t * TK + r] >= 0;
      uint32_t x[8];
      tmem_ld_32x8(tmem_base + lane_addr + S_COL, x);
      tmem_ld_wait();
      float s[REP], mx[REP];
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        s[h] = valid ? __uint_as_float(x[h]) * scale_log2 : -INFINITY;
        mx[h] = s[h];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int h = 0; h < REP; ++h) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], o));
      if (lane == 0) {
#pragma unroll
        for (int h = 0; h < REP; ++h) wm[warp * 8 + h] = mx[h];
      }
      bar_sync_128();
      float alpha[REP];
      bool any = false;
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        const float mt = fmaxf(fmaxf(wm[h], wm[8 + h]), fmaxf(wm[16 + h], wm[24 + h]));
        const float mo = m_run[h];
        const float mn = fmaxf(mo, mt);
        alpha[h] = (mn == mo) ? 1.f : ex2_approx(mo - mn);      // mo = -inf gives 0: nothing was accumulated yet
        any = any || (mn != mo);
        const float mm = mn == -INFINITY ? 0.f : mn;
        const float e = ex2_approx(s[h] - mm);
        l_thread[h] = l_thread[h] * alpha[h] + e;
        s[h] = e;
        mx[h] = mn;
      }
      // P^T as a K-major B operand: row = head, column = key of the tile
      {
        uint8_t* pb = smem + Smem::offP + (r >> 6) * 1024 + (r & 7) * 2;
        const int c16 = (r & 63) >> 3;
#pragma unroll
        for (int h = 0; h < REP; ++h) *reinterpret_cast<__nv_bfloat16*>(pb + h * 128 + ((c16 ^ h) << 4)) = __float2bfloat16(s[h]);
      }
      if (any && t > 0) {   // CTA-uniform: every thread computed the same maxima
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t ov[8];
          tmem_ld_32x8(tmem_base + lane_addr + O_COL + half * 16, ov);
          tmem_ld_wait();
#pragma unroll
          for (int h = 0; h < REP; ++h) ov[h] = __float_as_uint(__uint_as_float(ov[h]) * alpha[h]);
          tmem_st_32x8(tmem_base + lane_addr + O_COL + half * 16, ov);
        }
        tmem_st_wait();
      }
      bar_sync_128();   // every thread has read m_run before it changes
      if (tid < 8) m_run[tid] = mx[tid];
    }
    cp_async_wait<1>();          // V(t) has landed; K(t+1) may be in flight
    fence_async_proxy();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const SmemDesc b0 = make_desc(smem_u32(smem + Smem::offP), 16, 1024);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const SmemDesc a0 = make_desc(smem_u32(smem + Smem::offV + half * 2 * kRowBlk), kRowBlk, 1024);
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk) {
          const SmemDesc bb = desc_off(b0, (kk >> 2) * 1024 + (kk & 3) * 32);
          umma_ss<2>(tmem_base + O_COL + half * 16, desc_off(a0, kk * 2048), bb, idesc_o, (t > 0 || kk > 0) ? 1u : 0u);
        }
      }
      umma_commit(bar_o);
    }
    ok = mbar_wait(bar_o, t & 1, abort_flag, p.status, kErrTimeoutTmemFull);
    ok = __syncthreads_and(ok);
    if (!ok) break;
    tc_fence_after();
    if (t + 1 < nt) gather(p.v, smem + Smem::offV, t + 1); else cp_async_commit();
  }
  cp_async_wait<0>();
  if (ok && warp < 4) {
    // ---- row sums over the CTA, then O = O^T / l (thread <-> channel)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
      for (int h = 0; h < REP; ++h) l_thread[h] += __shfl_xor_sync(0xffffffffu, l_thread[h], o);
    if (lane == 0) {   // the four warps' sums meet in a fixed order: the result is bit-reproducible
#pragma unroll
      for (int h = 0; h < REP; ++h) wm[warp * 8 + h] = l_thread[h];
    }
    bar_sync_128();
    float inv[REP];
#pragma unroll
    for (int h = 0; h < REP; ++h) {
      const float l = (wm[h] + wm[8 + h]) + (wm[16 + h] + wm[24 + h]);
      inv[h] = l > 0.f ? 1.f / l : 0.f;
      if (tid == h) p.lse[(size_t)b * Hq + g * REP + h] = l > 0.f ? (m_run[h] + log2f(l)) * kLn2 : -INFINITY;
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t ov[8];
      tmem_ld_32x8(tmem_base + lane_addr + O_COL + half * 16, ov);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < REP; ++h)
        p.o[((size_t)b * Hq + g * REP + h) * D + half * 128 + tid] = __float2bfloat16(nt > 0 ? __uint_as_float(ov[h]) * inv[h] : 0.f);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// ================================================================================================ backward
// Same tiling.  Per 128-key tile:
//     S^T = K_sel Q^T, dP^T = V_sel dO^T                 (N = 16, as in the forward pass)
//     p = exp2(s - lse), dS = p (dP - delta) scale        threads <-> keys; written three ways:
//         dS^T [heads x keys]  B operand of  dQ^T [256, 16] += K_sel^T dS
//         dS   [keys x 16]     A operand of  dK_sel [128, 256] = dS Q      (one MMA: K = 16 heads, N = 256)
//         P    [keys x 16]     A operand of  dV_sel [128, 256] = P dO
// dK_sel / dV_sel leave through a shared-memory staging buffer, 32 columns at a time, as vector float reductions into
// the rows sel[j] of dk / dv (a warp instruction adds 4 rows x 128 contiguous bytes).  The q and dO blocks are stored once
// as [16 rows x 256]: rows 8-15 are zeros, because the dK / dV products contract over the 16 rows.
struct BwdParams {
  const __nv_bfloat16 *q, *k, *v, *o, *d_o;
  const int* sel;
  const float* lse;
  float *dq, *dk, *dv;       // dq [B, Hq, 256]; dk, dv [L, Hkv, 256] accumulated into
  int B, Hkv, kk;
  float scale;
  int* status;
};

struct BwdSmem {
  static constexpr int offK = 0, offV = offK + kTile;
  static constexpr int offQ = offV + kTile;              // 4 channel blocks x [16 rows x 128 B]
  static constexpr int offDO = offQ + 4 * 2048;
  static constexpr int offDS = offDO + 4 * 2048;         // [128 rows x 128 B], 32 bytes of every row in use
  static constexpr int offPA = offDS + TK * 128;
  static constexpr int offDST = offPA + TK * 128;        // dS^T: 2 key blocks x [8 rows x 128 B] (+ 1 KB that row group 1 reads)
  static constexpr int offStage = offDST + 3 * 1024;     // fp32 [128][36]
  static constexpr int kStageStride = 36;
  static constexpr int offF = offStage + TK * kStageStride * 4;   // lse2 [8], delta [8]
  static constexpr int offCtl = offF + 16 * 4;
  static constexpr int offSel = offCtl + 64;
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1) dsa_tc_bwd_kernel(BwdParams p) {
  using L = BwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* lse2 = reinterpret_cast<float*>(smem + L::offF);
  float* delta = lse2 + 8;
  float* stage = reinterpret_cast<float*>(smem + L::offStage);
  uint64_t* bar = reinterpret_cast<uint64_t*>(smem + L::offCtl);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* sel_s = reinterpret_cast<int*>(smem + L::offSel);

  const int b = blockIdx.x, g = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Hq = p.Hkv * REP;
  const int nt = (p.kk + TK - 1) / TK;
  constexpr int TMEM_COLS = 512, S_COL = 0, DP_COL = 16, DQ_COL = 32, ACC_COL = 256;
  const size_t row0 = ((size_t)b * Hq + g * REP) * D;

  if (tid == 0) {
    mbar_init(bar, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc<TMEM_COLS>(tmem_slot);
  for (int j = tid; j < nt * TK; j += THREADS) sel_s[j] = j < p.kk ? p.sel[(size_t)b * p.kk + j] : -1;
  {  // q and dO blocks: row = head (rows 8-15 zero), 16-byte group c of the 512-byte row
    const int h = tid >> 5, c = tid & 31;
    const uint32_t off = (c >> 3) * 2048 + h * 128 + (((c & 7) ^ h) << 4);
    *reinterpret_cast<uint4*>(smem + L::offQ + off) = *reinterpret_cast<const uint4*>(p.q + row0 + (size_t)h * D + c * 8);
    *reinterpret_cast<uint4*>(smem + L::offDO + off) = *reinterpret_cast<const uint4*>(p.d_o + row0 + (size_t)h * D + c * 8);
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    *reinterpret_cast<uint4*>(smem + L::offQ + (c >> 3) * 2048 + 1024 + h * 128 + ((c & 7) << 4)) = z;
    *reinterpret_cast<uint4*>(smem + L::offDO + (c >> 3) * 2048 + 1024 + h * 128 + ((c & 7) << 4)) = z;
  }
  // delta[h] = sum_d dO[h][d] O[h][d]: warp h
  {
    const int h = warp;
    float acc = 0.f;
    for (int d = lane; d < D; d += 32)
      acc += __bfloat162float(p.d_o[row0 + (size_t)h * D + d]) * __bfloat162float(p.o[row0 + (size_t)h * D + d]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (lane == 0) {
      delta[h] = acc;
      lse2[h] = p.lse[(size_t)b * Hq + g * REP + h] * kLog2e;
    }
  }
  // the A tiles of dK / dV use 32 bytes of every 128-byte row; the MMA reads only those
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  auto gather = [&](const __nv_bfloat16* src, uint8_t* dst, int t) {
#pragma unroll 4
    for (int i = 0; i < TK / 8; ++i) {
      const int r = i * 8 + warp;
      const int idx = sel_s[t * TK + r];
      const __nv_bfloat16* row = src + ((size_t)max(idx, 0) * p.Hkv + g) * D + lane * 8;
      cp_async16(dst + (lane >> 3) * kRowBlk + r * 128 + (((lane & 7) ^ (r & 7)) << 4), row, idx >= 0 ? 16 : 0);
    }
    cp_async_commit();
  };
  uint32_t phase = 0;
  auto mma_wait = [&]() -> bool {
    if (tid == 0) umma_commit(bar);
    bool ok = mbar_wait(bar, phase, abort_flag, p.status, kErrTimeoutTmemFull);
    phase ^= 1;
    ok = __syncthreads_and(ok);
    tc_fence_after();
    return ok;
  };
  // accumulator tile [128 keys x 256] -> vector reductions into the selected rows of `dst`
  auto scatter_acc = [&](float* dst, int t) {
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
#pragma unroll 1
    for (int c = 0; c < 8; ++c) {
      if (warp < 4) {
        uint32_t x[32];
        tmem_ld_32x32(tmem_base + lane_addr + ACC_COL + c * 32, x);
        tmem_ld_wait();
        float4* srow = reinterpret_cast<float4*>(stage + tid * L::kStageStride);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          srow[u] = make_float4(__uint_as_float(x[4 * u]), __uint_as_float(x[4 * u + 1]), __uint_as_float(x[4 * u + 2]), __uint_as_float(x[4 * u + 3]));
      }
      __syncthreads();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = warp * 16 + i * 4 + (lane >> 3);
        const int idx = sel_s[t * TK + r];
        if (idx >= 0) {
          const float4 v4 = *reinterpret_cast<const float4*>(stage + r * L::kStageStride + (lane & 7) * 4);
          red_add_v4(dst + ((size_t)idx * p.Hkv + g) * D + c * 32 + (lane & 7) * 4, v4.x, v4.y, v4.z, v4.w);
        }
      }
      __syncthreads();
    }
  };

  const float scale_log2 = p.scale * kLog2e;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
  const uint32_t idesc_s = make_idesc_bf16(128, 16, false, false), idesc_q = make_idesc_bf16(128, 16, true, false);
  const uint32_t idesc_kv = make_idesc_bf16(128, 256, false, true);

  gather(p.k, smem + L::offK, 0);
  gather(p.v, smem + L::offV, 0);
  bool ok = true;
  for (int t = 0; t < nt && ok; ++t) {
    cp_async_wait<0>();
    fence_async_proxy();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const SmemDesc ak = make_desc(smem_u32(smem + L::offK), 16, 1024), av = make_desc(smem_u32(smem + L::offV), 16, 1024);
      const SmemDesc bq = make_desc(smem_u32(smem + L::offQ), 16, 1024), bo = make_desc(smem_u32(smem + L::offDO), 16, 1024);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t oa = (kk >> 2) * kRowBlk + (kk & 3) * 32, ob = (kk >> 2) * 2048 + (kk & 3) * 32;
        umma_ss<2>(tmem_base + S_COL, desc_off(ak, oa), desc_off(bq, ob), idesc_s, kk > 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint32_t oa = (kk >> 2) * kRowBlk + (kk & 3) * 32, ob = (kk >> 2) * 2048 + (kk & 3) * 32;
        umma_ss<2>(tmem_base + DP_COL, desc_off(av, oa), desc_off(bo, ob), idesc_s, kk > 0 ? 1u : 0u);
      }
    }
    ok = mma_wait();
    if (!ok) break;
    if (t + 1 < nt) gather(p.v, smem + L::offV, t + 1);   // the value tile is only read by dP^T
    if (warp < 4) {
      const int r = tid;
      const bool valid = sel_s[t * TK + r] >= 0;
      uint32_t xs[8], xd[8];
      tmem_ld_32x8(tmem_base + lane_addr + S_COL, xs);
      tmem_ld_32x8(tmem_base + lane_addr + DP_COL, xd);
      tmem_ld_wait();
      float pr[8], ds[8];
#pragma unroll
      for (int h = 0; h < REP; ++h) {
        const float l2 = lse2[h];
        pr[h] = (valid && l2 != -INFINITY) ? ex2_approx(__uint_as_float(xs[h]) * scale_log2 - l2) : 0.f;
        ds[h] = pr[h] * (__uint_as_float(xd[h]) - delta[h]) * p.scale;
      }
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
      const uint4 dsv = make_uint4(pack_bf16x2(ds[0], ds[1]), pack_bf16x2(ds[2], ds[3]), pack_bf16x2(ds[4], ds[5]), pack_bf16x2(ds[6], ds[7]));
      const uint4 pv = make_uint4(pack_bf16x2(pr[0], pr[1]), pack_bf16x2(pr[2], pr[3]), pack_bf16x2(pr[4], pr[5]), pack_bf16x2(pr[6], pr[7]));
      *reinterpret_cast<uint4*>(smem + L::offDS + r * 128 + ((0 ^ (r & 7)) << 4)) = dsv;
      *reinterpret_cast<uint4*>(smem + L::offDS + r * 128 + ((1 ^ (r & 7)) << 4)) = z;
      *reinterpret_cast<uint4*>(smem + L::offPA + r * 128 + ((0 ^ (r & 7)) << 4)) = pv;
      *reinterpret_cast<uint4*>(smem + L::offPA + r * 128 + ((1 ^ (r & 7)) << 4)) = z;
      uint8_t* pb = smem + L::offDST + (r >> 6) * 1024 + (r & 7) * 2;
      const int c16 = (r & 63) >> 3;
#pragma unroll
      for (int h = 0; h < REP; ++h) *reinterpret_cast<__nv_bfloat16*>(pb + h * 128 + ((c16 ^ h) << 4)) = __float2bfloat16(ds[h]);
    }
    fence_async_proxy();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      const SmemDesc bt = make_desc(smem_u32(smem + L::offDST), 16, 1024);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const SmemDesc a0 = make_desc(smem_u32(smem + L::offK + half * 2 * kRowBlk), kRowBlk, 1024);
#pragma unroll
        for (int kk = 0; kk < TK / 16; ++kk)
          umma_ss<2>(tmem_base + DQ_COL + half * 16, desc_off(a0, kk * 2048), desc_off(bt, (kk >> 2) * 1024 + (kk & 3) * 32), idesc_q,
                     (t > 0 || kk > 0) ? 1u : 0u);
      }
      // dK_sel = dS Q: A [128 keys x 16 heads] K-major, B = the q block read MN-major (k-lines = heads, N = 256 channels)
      umma_ss<0>(tmem_base + ACC_COL, make_desc(smem_u32(smem + L::offDS), 16, 1024), make_desc(smem_u32(smem + L::offQ), 2048, 1024), idesc_kv);
    }
    ok = mma_wait();
    if (!ok) break;
    if (t + 1 < nt) gather(p.k, smem + L::offK, t + 1);   // the key tile was last read by dQ^T
    scatter_acc(p.dk, t);
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
      umma_ss<0>(tmem_base + ACC_COL, make_desc(smem_u32(smem + L::offPA), 16, 1024), make_desc(smem_u32(smem + L::offDO), 2048, 1024), idesc_kv);
    }
    ok = mma_wait();
    if (!ok) break;
    scatter_acc(p.dv, t);
    tc_fence_before();
  }
  cp_async_wait<0>();
  if (ok && warp < 4) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      uint32_t x[8];
      tmem_ld_32x8(tmem_base + lane_addr + DQ_COL + half * 16, x);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < REP; ++h) p.dq[row0 + (size_t)h * D + half * 128 + tid] = nt > 0 ? __uint_as_float(x[h]) : 0.f;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}
}  // namespace

extern "C" int vlmt_dsa_fwd_tc(const void* q, const void* k, const void* v, const int* sel, void* o, float* lse, int B, int Hkv, int kk,
                               float scale, int* status, cudaStream_t st) {
  if (B <= 0 || kk <= 0) return 0;
  Params p;
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.sel = sel;
  p.o = (__nv_bfloat16*)o; p.lse = lse; p.B = B; p.Hkv = Hkv; p.kk = kk; p.scale = scale; p.status = status;
  const int nt = (kk + TK - 1) / TK;
  const int smem = Smem::offSel + nt * TK * 4 + 1024;
  if (smem > 227 * 1024) return -3;
  if (cudaFuncSetAttribute(dsa_tc_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
  dsa_tc_fwd_kernel<<<dim3(B, Hkv), THREADS, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

extern "C" int vlmt_dsa_bwd_tc(const void* q, const void* k, const void* v, const int* sel, const void* o, const float* lse, const void* d_o,
                               float* dq, float* dk, float* dv, int B, int Hkv, int kk, float scale, int* status, cudaStream_t st) {
  if (B <= 0 || kk <= 0) return 0;
  BwdParams p;
  p.q = (const __nv_bfloat16*)q; p.k = (const __nv_bfloat16*)k; p.v = (const __nv_bfloat16*)v; p.o = (const __nv_bfloat16*)o;
  p.d_o = (const __nv_bfloat16*)d_o; p.sel = sel; p.lse = lse; p.dq = dq; p.dk = dk; p.dv = dv;
  p.B = B; p.Hkv = Hkv; p.kk = kk; p.scale = scale; p.status = status;
  const int nt = (kk + TK - 1) / TK;
  const int smem = BwdSmem::offSel + nt * TK * 4 + 1024;
  if (smem > 227 * 1024) return -3;
  if (cudaFuncSetAttribute(dsa_tc_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
  dsa_tc_bwd_kernel<<<dim3(B, Hkv), THREADS, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
