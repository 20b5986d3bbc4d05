// Varlen (packed-row) flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// All three kernels use ten warps: warp 0 issues TMA loads, one thread of warp 1 issues every MMA, warps 2..9 do
// the CUDA-core work between the MMAs (two warps per scheduler, so one warp's latencies hide behind the other).
// Probabilities and score gradients go back to the tensor core through tensor memory (they overwrite the fp32
// scores they were computed from and are read as the A operand of the next MMA), never through shared memory.
// Every MMA has N = 128 (or N = head dim): narrower MMAs occupy the tensor core for about 70 cycles whatever
// their size (measured), so they would waste it.
//
// Forward: one CTA per (256 queries of one document = two 128-row tiles, query head).  Warps 2..5 own tile 0 and
//   warps 6..9 tile 1, one query row per thread (tcgen05.ld gives a thread its whole row: row max and row sum need
//   no shuffles).  The MMA thread alternates between the tiles - P0.V, S0', P1.V, S1' - so the tensor core works
//   on one tile while the softmax of the other runs.  O accumulates in TMEM; it is rescaled only when a row's
//   running max grows by more than 2^8 (the stale max is used meanwhile, which only changes the common scale
//   of P and l).
// Backward: `attn_bwd_dkdv` (one CTA per 128-key tile and kv head; loops over 128-query tiles and the query heads
//   of the GQA group) and `attn_bwd_dq` (one CTA per 128-query tile and head; loops over 128-key tiles) recompute
//   S and dP = dO V^T on the tensor cores; each compute thread handles half of a 128-wide row in two phases
//   (P = exp2(S - lse), then dS = P (dP - delta)) so that the exp2 phase overlaps the dP and accumulation MMAs.
//   No atomics: results are bit-reproducible.
//
// Documents are [cu_seqlens[i], cu_seqlens[i+1]); tiles never mix documents: keys past the end of the document
// (and, with `causal`, keys after the query) are masked before the softmax.
//
// Building with -DVLMT_ATTN_TRACE records clock64 stamps of the MMA thread and of one compute warp of CTA (0,0) of
// the dQ kernel and prints them after the third backward call (a timeline tool; no effect on regular builds).
#include "attention_sm100.h"
#include "sm100.cuh"

#include <cuda_bf16.h>
#include <math.h>

#include <cstdio>
#include <cstdlib>
#include <type_traits>

namespace {
using namespace sm100;

constexpr int BM = 128, BN = 128;
constexpr int ATT_THREADS = 320;  // TMA warp, MMA warp, 8 compute warps
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.f;  // log2 units

struct TileInfo {
  int doc_start, doc_len, q0;  // q0: first row of the tile, local to the document
  bool valid;
};

// Linear tile id -> (document, block of `block_rows` rows).  Tiles are numbered document by document.
__device__ __forceinline__ TileInfo find_tile(const int* __restrict__ cu, int n_docs, int tile, int block_rows) {
  TileInfo ti;
  ti.valid = false;
  ti.doc_start = ti.doc_len = ti.q0 = 0;
  int acc = 0;
  for (int d = 0; d < n_docs; ++d) {
    const int s = cu[d], e = cu[d + 1];
    const int nb = (e - s + block_rows - 1) / block_rows;
    if (tile < acc + nb) {
      ti.doc_start = s;
      ti.doc_len = e - s;
      ti.q0 = (nb - 1 - (tile - acc)) * block_rows;  // longest-running (last) blocks first
      ti.valid = true;
      return ti;
    }
    acc += nb;
  }
  return ti;
}

__device__ __forceinline__ uint32_t (&as32(uint32_t* p))[32] { return *reinterpret_cast<uint32_t(*)[32]>(p); }

struct FwdParams {
  __nv_bfloat16* O;   // [T, Hq, D]
  float* LSE;         // [Hq, T]
  const int* cu;
  int n_docs, T, Hq, Hkv;
  float scale_log2;   // softmax scale * log2(e)
  int causal;
  int k_steps;        // 16-channel steps of the Q.K contraction and width of the P.V product (channels beyond 16 * k_steps are zero padding)
  int d_mem;          // head size in memory (<= D): TMA zero-fills the tile's channels beyond it, the output has this width
  int* status;
};

template <int D>
struct FwdSmem {
  static constexpr int kQ = BM * D * 2;    // one query tile
  static constexpr int kKV = BN * D * 2;
  static constexpr int offQ = 0;               // 2 tiles
  static constexpr int offK = offQ + 2 * kQ;   // 2 stages
  static constexpr int offV = offK + 2 * kKV;  // 2 stages
  static constexpr int offBar = offV + 2 * kKV;
  static constexpr int kTotal = offBar + 256 + 1024;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, FwdParams p) {
  using L = FwdSmem<D>;
  constexpr int DB = D / 64;  // 64-column blocks along the head dim
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* q_full = bars;            // 1
  uint64_t* k_full = bars + 1;        // 2 stages
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // per query tile
  uint64_t* p_full = bars + 11;       // per query tile (4 warps)
  uint64_t* o_done = bars + 13;       // per query tile: last P.V finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, 2 * BM);
  if (!ti.valid) return;  // uniform for the whole CTA
  const int hq = blockIdx.y;
  const int hkv = hq / (p.Hq / p.Hkv);
  // key tiles visible to query tile t (rows q0 + 128 t ...): none if the tile starts beyond the document
  int Jt[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int qs = ti.q0 + t * BM;
    const int kv_end = qs >= ti.doc_len ? 0 : (p.causal ? min(ti.doc_len, qs + BM) : ti.doc_len);
    Jt[t] = (kv_end + BN - 1) / BN;
  }
  const int J = max(Jt[0], Jt[1]);
  constexpr int TMEM_COLS = 512;
  constexpr int S_COL = 0, O_COL = 256;  // S_t at 128 t, O_t at 256 + D t

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4); mbar_init(&o_done[i], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) tmem_alloc<TMEM_COLS>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int row0 = ti.doc_start + ti.q0;
      mbar_expect_tx(q_full, 2 * L::kQ);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_3d(smem + L::offQ + t * L::kQ + b * 16384, &tmQ, q_full, 64 * b, hq, row0 + t * BM);
      for (int j = 0; j < J; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        const int krow = ti.doc_start + j * BN;
        if (!mbar_wait(&k_empty[s], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&k_full[s], L::kKV);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_3d(smem + L::offK + s * L::kKV + b * 16384, &tmK, &k_full[s], 64 * b, hkv, krow);
        if (!mbar_wait(&v_empty[s], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&v_full[s], L::kKV);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_3d(smem + L::offV + s * L::kKV + b * 16384, &tmV, &v_full[s], 64 * b, hkv, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, false, false);
      const uint32_t idesc_pv = make_idesc_bf16(BM, 16 * p.k_steps, false, true);   // only the channels that are not padding
      // S_t(j) = Q_t K_j^T.  It overwrites P_t(j-1), whose consumer P_t(j-1).V was issued earlier by this thread.
      const SmemDesc dQ0 = make_desc(smem_u32(smem + L::offQ), 16, 1024);
      const SmemDesc dK0 = make_desc(smem_u32(smem + L::offK), 16, 1024);
      const SmemDesc dV0 = make_desc(smem_u32(smem + L::offV), 16384, 1024);
      auto issue_S = [&](int t, int j) {
        const SmemDesc a = desc_off(dQ0, t * L::kQ), b = desc_off(dK0, (j & 1) * L::kKV);
        const uint32_t d = tmem_base + S_COL + t * BN;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk >= p.k_steps) break;
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          if (kk == 0) umma_ss<0>(d, a, b, idesc_s); else umma_ss<1>(d, desc_off(a, off), desc_off(b, off), idesc_s);
        }
        umma_commit(&s_full[t]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kErrTimeoutFull);
      if (ok && J > 0) {
        ok = mbar_wait(&k_full[0], 0, abort_flag, p.status, kErrTimeoutFull);
        if (ok) {
          tc_fence_after();
#pragma unroll
          for (int t = 0; t < 2; ++t) if (Jt[t] > 0) issue_S(t, 0);
          umma_commit(&k_empty[0]);
        }
      }
      for (int j = 0; j < J && ok; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&v_full[s], ph, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
        if (j + 1 < J && !mbar_wait(&k_full[s ^ 1], ((j + 1) >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
        const SmemDesc dV = desc_off(dV0, s * L::kKV);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= Jt[t]) continue;
          if (!mbar_wait(&p_full[t], j & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
          tc_fence_after();
          const uint32_t dO = tmem_base + O_COL + t * D, aP = tmem_base + S_COL + t * BN;
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {  // A = P_t: 128 lanes x 8 columns of packed bf16 pairs per 16 keys
            if (kk == 0) umma_ts<2>(dO, aP, dV, idesc_pv, (uint32_t)j); else umma_ts<1>(dO, aP + kk * 8, desc_off(dV, kk * 2048), idesc_pv);
          }
          if (j + 1 < Jt[t]) issue_S(t, j + 1);
          else umma_commit(&o_done[t]);
        }
        if (!ok) break;
        umma_commit(&v_empty[s]);
        if (j + 1 < J) umma_commit(&k_empty[s ^ 1]);  // K_{j+1} is free once every S_t(j+1) issued above has run
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warps
    const int t = (warp - 2) >> 2;         // query tile of this warp
    const int q = warp & 3;                // TMEM lane quarter this warp may access
    const int r = q * 32 + lane;           // row of the tile owned by this thread
    const int qi = ti.q0 + t * BM + r;     // query index local to the document
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t s_addr = tmem_base + S_COL + t * BN + lane_addr;
    const uint32_t o_addr = tmem_base + O_COL + t * D + lane_addr;
    const int Jm = Jt[t];
    float m_used = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < Jm && ok; ++j) {
      if (!mbar_wait(&s_full[t], j & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      uint32_t s[BN];
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) tmem_ld_32x32(s_addr + c * 32, as32(&s[c * 32]));
      tmem_ld_wait();
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN > ti.doc_len) || (p.causal && kv0 + BN - 1 > ti.q0 + t * BM);
      if (need_mask) {
        const int limit = (p.causal ? min(ti.doc_len - 1, qi) : ti.doc_len - 1) - kv0;  // last visible column of this tile
#pragma unroll
        for (int i = 0; i < BN; ++i) if (i > limit) s[i] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BN; i += 8) {
        mx0 = fmax3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
        mx2 = fmax3(mx2, __uint_as_float(s[i + 4]), __uint_as_float(s[i + 5]));
        mx3 = fmax3(mx3, __uint_as_float(s[i + 6]), __uint_as_float(s[i + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * p.scale_log2;  // the scale is positive: it commutes with max
      if (j == 0) {
        m_used = (mx == -INFINITY) ? 0.f : mx;
      } else {
        // S_t(j) was issued after P_t(j-1).V, so O_t is complete here and the tensor core does not touch it
        // before this warp publishes P_t(j).
        const bool grow = mx > m_used + kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = grow ? ex2_approx(m_used - mx) : 1.f;
          if (grow) m_used = mx;
          l *= alpha;
#pragma unroll
          for (int c = 0; c < D / 32; ++c) {
            if (c * 2 >= p.k_steps) break;   // channels beyond 16 * k_steps are never accumulated
            uint32_t o[32];
            tmem_ld_32x32(o_addr + c * 32, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_addr + c * 32, o);
          }
        }
      }
      const float neg_m = -m_used;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float e0 = ex2_approx(fmaf(__uint_as_float(s[c * 32 + 2 * i]), p.scale_log2, neg_m));
          const float e1 = ex2_approx(fmaf(__uint_as_float(s[c * 32 + 2 * i + 1]), p.scale_log2, neg_m));
          sum0 += e0;
          sum1 += e1;
          pk[i] = pack_bf16x2(e0, e1);
        }
        tmem_st_32x16(s_addr + c * 16, pk);  // P_t over the first 64 columns of S_t (every score is in registers already)
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      l += sum0 + sum1;
    }
    if (ok && Jm > 0 && mbar_wait(&o_done[t], 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const size_t tok = (size_t)(ti.doc_start + qi);
      __nv_bfloat16* dst = p.O + (tok * p.Hq + hq) * p.d_mem;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        if (c * 32 >= p.d_mem) break;
        uint32_t o[32];
        tmem_ld_32x32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (qi < ti.doc_len) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (c * 32 + u * 8 >= p.d_mem) break;   // channels beyond the head size exist only in the tile
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]) * inv, __uint_as_float(o[u * 8 + 1]) * inv);
            pk.y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]) * inv, __uint_as_float(o[u * 8 + 3]) * inv);
            pk.z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]) * inv, __uint_as_float(o[u * 8 + 5]) * inv);
            pk.w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]) * inv, __uint_as_float(o[u * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + u * 8) = pk;
          }
        }
      }
      if (qi < ti.doc_len) p.LSE[(size_t)hq * p.T + tok] = l > 0.f ? (m_used + log2f(l)) * kLn2 : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// ------------------------------------------------------------------------------------ backward helpers
// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O, float* __restrict__ delta,
                                  int T, int H, int D) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int total = T * H;
  if (warp >= total) return;
  const int t = warp / H, h = warp - t * H;
  const __nv_bfloat16* a = dO + ((size_t)t * H + h) * D;
  const __nv_bfloat16* b = O + ((size_t)t * H + h) * D;
  float acc = 0.f;
  for (int i = lane; i < D; i += 32) acc += __bfloat162float(a[i]) * __bfloat162float(b[i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) delta[(size_t)h * T + t] = acc;
}

struct BwdParams {
  __nv_bfloat16 *dQ, *dK, *dV;  // [T,Hq,D], [T,Hkv,D], [T,Hkv,D]
  const float* LSE;             // [Hq, T]
  const float* delta;           // [Hq, T]
  const int* cu;
  int n_docs, T, Hq, Hkv;
  float scale, scale_log2;
  int causal;
  int k_steps;        // 16-channel steps of the contractions over the head dim (Q.K and dO.V) and width of dQ / dK / dV; the rest is zero padding
  int d_mem;          // head size in memory (<= D)
  int* status;
  long long* trace;  // timeline dump of CTA (0,0) (only with -DVLMT_ATTN_TRACE; nullptr otherwise)
};

#ifdef VLMT_ATTN_TRACE
#define TRACE(slot, j) do { if (p.trace && blockIdx.x == 0 && blockIdx.y == 0 && (j) < 256) p.trace[(j) * 16 + (slot)] = clock64(); } while (0)
#else
#define TRACE(slot, j) do { } while (0)
#endif

// Backward.  Measured on B200 (in-kernel clock64 timeline, build with -DVLMT_ATTN_TRACE): one tcgen05.mma of shape
// 128 x N x 16 occupies the tensor core for about max(N / 2, 70) cycles whether its A operand comes from shared or from
// tensor memory, so MMAs narrower than N = 128 waste the pipe.  Both kernels therefore work on 128 x 128 score tiles
// (every MMA has N = 128 or N = D) and hide the CUDA-core work by splitting it in two phases per tile:
//   phase a:  P  = exp2(S * scale - lse)          (special-function-unit bound: 16 ex2 per clock per SM)
//   phase b:  dS = P * (dP - delta)               (needs dP, short)
// so that the tensor core computes dP (and the accumulations of the previous tile) while phase a runs.  P / dS are
// written as packed bf16 over the fp32 scores and are read from tensor memory as the A operand of the next MMA.
constexpr int NCW = 8;       // compute warps; a thread owns one row of the 128-row tile and 64 of its 128 columns
constexpr int CPT = 64;      // columns per thread

// A-operand column of k-step kk (16 streamed rows) inside a 128-column buffer: the warps that own columns
// [64 g, 64 g + 64) write their 64 values as 32 packed words at column 64 g, so no warp overwrites scores that the
// other group has not read yet.
__device__ __forceinline__ constexpr int packed_col(int kk) { return (kk >> 2) * 64 + (kk & 3) * 8; }

// Shared memory: two stationary [128 x D] tiles and two TMA rings for the streamed tiles.  The ring whose tiles are
// needed until the END of a step (Q for dK, K for dQ) has three stages, the other (dO / V, free after the first half of
// the step) two: a load is then issued about one whole step before its first use, which hides the TMA latency
// (about 1600 cycles for a 32 KB tile; with two stages each the tensor core idled on the loads).
template <int D>
struct BwdSmem {
  static constexpr int kTile = 128 * D * 2;    // one [128 x D] tile
  static constexpr int offA = 0;                     // dkdv: K_j   | dq: Q_i
  static constexpr int offB = offA + kTile;          // dkdv: V_j   | dq: dO_i
  static constexpr int offC = offB + kTile;          // 3 stages: dkdv Q_i  | dq K_j
  static constexpr int offD = offC + 3 * kTile;      // 2 stages: dkdv dO_i | dq V_j
  static constexpr int offStat = offD + 2 * kTile;   // dkdv: per column group and step parity: -lse2[64], -delta[64]
  static constexpr int offBar = offStat + 2 * 2 * 128 * 4;
  static constexpr int kSlack = 512;                 // room for rounding the dynamic shared memory base up to 1024 bytes
  static constexpr int kTotal = offBar + 256 + kSlack;
};

// Round the dynamic shared memory base up to 1024 bytes (TMA 128-byte swizzle atoms); returns nullptr if that needs more
// than the slack the launch reserved (the base is 1024-aligned in practice, so this does not happen).
template <int kSlack>
__device__ __forceinline__ uint8_t* align_smem(uint8_t* raw) {
  uint8_t* a = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  return (a - raw) <= kSlack ? a : nullptr;
}

// ------------------------------------------------------------------------------------------------ dK / dV
// One CTA per 128-key tile and kv head; loops over 128-query tiles and the query heads of the GQA group.
// Everything is computed transposed (rows = keys):
//   S^T = K Q^T -> X,  dP^T = V dO^T -> Y        (M = 128 keys, N = 128 queries)
//   dV += P^T dO (A = X),  dK += dS^T Q (A = Y)   (B = the [128 x D] query-side tile read MN-major)
// TMEM columns: X 0, Y 128, dV 256, dK 256 + D.  Tensor-core order: dV(i), S^T(i+1), dK(i), dP^T(i+1).
template <int D>
__global__ void __launch_bounds__(64 + 32 * NCW, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int DB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_smem<L::kSlack>(smem_raw);
  if (smem == nullptr) { if (threadIdx.x == 0) atomicCAS(p.status, 0, kErrTimeoutOther); return; }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* kv_full = bars;          // 1
  uint64_t* acc_done = bars + 1;     // 1
  uint64_t* q_full = bars + 2;       // 3
  uint64_t* q_empty = bars + 5;      // 3
  uint64_t* do_full = bars + 8;      // 2
  uint64_t* do_empty = bars + 10;    // 2
  uint64_t* s_full = bars + 12;      // S^T(i) is in X
  uint64_t* dp_full = bars + 13;     // dP^T(i) is in Y
  uint64_t* p_full = bars + 14;      // NCW warps: P^T(i) is in X
  uint64_t* ds_full = bars + 15;     // NCW warps: dS^T(i) is in Y
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat = reinterpret_cast<float*>(smem + L::offStat);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, 128);
  if (!ti.valid) return;
  const int hkv = blockIdx.y;
  const int group = p.Hq / p.Hkv;
  const int k0 = ti.q0;  // first key row of the tile (local to the document)
  const int n_qblk = (ti.doc_len + 127) / 128;
  const int i_first = p.causal ? k0 / 128 : 0;
  const int n_iter = (n_qblk - i_first) * group;
  constexpr int TMEM_COLS = 512;
  constexpr int X_COL = 0, Y_COL = 128, DV_COL = 256, DK_COL = 256 + D;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(acc_done, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&do_full[i], 1); mbar_init(&do_empty[i], 1); }
    mbar_init(s_full, 1); mbar_init(dp_full, 1); mbar_init(p_full, NCW); mbar_init(ds_full, NCW);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc<TMEM_COLS>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int krow = ti.doc_start + k0;
      mbar_expect_tx(kv_full, 2 * L::kTile);
#pragma unroll
      for (int b = 0; b < DB; ++b) {
        tma_load_3d(smem + L::offA + b * 16384, &tmK, kv_full, 64 * b, hkv, krow);
        tma_load_3d(smem + L::offB + b * 16384, &tmV, kv_full, 64 * b, hkv, krow);
      }
      int qs = 0;             // stage / phase of the Q ring (3 stages) ; the dO ring (2 stages) follows `it`
      uint32_t qph = 1;
      for (int it = 0; it < n_iter; ++it) {
        const int ds = it & 1;
        const int i = i_first + it / group, hq = hkv * group + it % group;
        const int qrow = ti.doc_start + i * 128;
        if (!mbar_wait(&q_empty[qs], qph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&q_full[qs], L::kTile);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_3d(smem + L::offC + qs * L::kTile + b * 16384, &tmQ, &q_full[qs], 64 * b, hq, qrow);
        if (!mbar_wait(&do_empty[ds], ((it >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&do_full[ds], L::kTile);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_3d(smem + L::offD + ds * L::kTile + b * 16384, &tmdO, &do_full[ds], 64 * b, hq, qrow);
        if (++qs == 3) { qs = 0; qph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);   // [128 keys] x [128 queries], contraction over d
      const uint32_t idesc_g = make_idesc_bf16(128, 16 * p.k_steps, false, true);  // [128 keys] x [channels], contraction over 128 queries
      const SmemDesc dK = make_desc(smem_u32(smem + L::offA), 16, 1024), dV = make_desc(smem_u32(smem + L::offB), 16, 1024);
      const SmemDesc dQk = make_desc(smem_u32(smem + L::offC), 16, 1024), dOk = make_desc(smem_u32(smem + L::offD), 16, 1024);         // K-major views
      const SmemDesc dQm = make_desc(smem_u32(smem + L::offC), 16384, 1024), dOm = make_desc(smem_u32(smem + L::offD), 16384, 1024);   // MN-major views
      const uint32_t tX = tmem_base + X_COL, tY = tmem_base + Y_COL;
      auto issue_score = [&](uint32_t dst, SmemDesc a, SmemDesc bq) {  // dst = a (stationary) x bq^T (streamed), both K-major
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk >= p.k_steps) break;
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          if (kk == 0) umma_ss<0>(dst, a, bq, idesc_s); else umma_ss<1>(dst, desc_off(a, off), desc_off(bq, off), idesc_s);
        }
      };
      auto issue_acc = [&](uint32_t dst, uint32_t a_tmem, SmemDesc bm, uint32_t acc) {  // dst += a_tmem [128 x 128] x bm [128 x D]
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          if (kk == 0) umma_ts<2>(dst, a_tmem, bm, idesc_g, acc); else umma_ts<1>(dst, a_tmem + packed_col(kk), desc_off(bm, kk * 2048), idesc_g);
        }
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kErrTimeoutFull);
      if (ok && n_iter > 0) {
        ok = mbar_wait(&q_full[0], 0, abort_flag, p.status, kErrTimeoutFull);
        if (ok) {
          tc_fence_after();
          issue_score(tX, dK, dQk);
          umma_commit(s_full);
          ok = mbar_wait(&do_full[0], 0, abort_flag, p.status, kErrTimeoutFull);
        }
        if (ok) {
          tc_fence_after();
          issue_score(tY, dV, dOk);
          umma_commit(dp_full);
        }
      }
      int qs = 0, qn = 1;     // Q-ring stage of step `it` and of step `it + 1`
      uint32_t qn_ph = 0;     // phase of q_full[qn] for step it + 1
      for (int it = 0; it < n_iter && ok; ++it) {
        const int ds = it & 1, dn = ds ^ 1;
        const bool more = it + 1 < n_iter;
        if (!mbar_wait(p_full, it & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        issue_acc(tmem_base + DV_COL, tX, desc_off(dOm, ds * L::kTile), (uint32_t)it);
        umma_commit(&do_empty[ds]);                          // dO_i was last read by dV(i)
        if (more) {
          if (!mbar_wait(&q_full[qn], qn_ph, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          issue_score(tX, dK, desc_off(dQk, qn * L::kTile));   // runs after dV(it), which read X
          umma_commit(s_full);
        }
        if (!mbar_wait(ds_full, it & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        issue_acc(tmem_base + DK_COL, tY, desc_off(dQm, qs * L::kTile), (uint32_t)it);
        umma_commit(&q_empty[qs]);                           // Q_i was last read by dK(i)
        if (more) {
          if (!mbar_wait(&do_full[dn], ((it + 1) >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          issue_score(tY, dV, desc_off(dOk, dn * L::kTile));   // runs after dK(it), which read Y
          umma_commit(dp_full);
        }
        qs = qn;
        if (++qn == 3) { qn = 0; qn_ph ^= 1; }
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int cw = warp - 2;
    const int cq = cw >> 2;                // column group: queries [64 cq, 64 cq + 64) of the streamed tile
    const int q = warp & 3;                // TMEM lane quarter this warp may access
    const int r = q * 32 + lane;           // key row of the tile owned by this thread
    const int kvi = k0 + r;                // key index local to the document
    const bool key_ok = kvi < ti.doc_len;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t tX = tmem_base + X_COL + cq * CPT + lane_addr, tY = tmem_base + Y_COL + cq * CPT + lane_addr;
    // every warp of a column group writes the same values into the group's area (no cross-warp ordering needed);
    // two areas alternate by step parity so that a warp one phase ahead never overwrites what a slower warp still reads
    // per-query statistics: lane l fetches those of queries 64 cq + l and 64 cq + 32 + l one step ahead
    auto fetch = [&](int it, float (&v)[4]) {
      const int i = i_first + it / group, hq = hkv * group + it % group;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int qq = i * 128 + cq * CPT + h * 32 + lane;
        const bool qok = qq < ti.doc_len;
        const size_t idx = (size_t)hq * p.T + ti.doc_start + (qok ? qq : 0);
        v[h] = qok ? -p.LSE[idx] * kLog2e : -INFINITY;  // -inf -> exp2(-inf) = 0 for queries beyond the document
        v[2 + h] = qok ? -p.delta[idx] : 0.f;
      }
    };
    float nxt[4] = {0.f, 0.f, 0.f, 0.f};
    if (n_iter > 0) fetch(0, nxt);
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2);
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int q0 = (i_first + it / group) * 128 + cq * CPT;   // first query of this thread's columns
      float* wstat = stat + (cq * 2 + (it & 1)) * 128;
      wstat[lane] = nxt[0]; wstat[32 + lane] = nxt[1]; wstat[64 + lane] = nxt[2]; wstat[96 + lane] = nxt[3];
      __syncwarp();
      if (it + 1 < n_iter) fetch(it + 1, nxt);
      // ---- phase a: P^T = exp2(S^T * scale - lse)
      if (!mbar_wait(s_full, it & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      // masked: keys beyond the document, or (causal) keys after the query.  Column c is visible iff c >= cmin.
      const bool need_mask = (k0 + 128 > ti.doc_len) || (p.causal && k0 + 127 > q0);
      const int cmin = !key_ok ? (1 << 30) : (p.causal ? kvi - q0 : -(1 << 30));
      float pr[CPT];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sr[32];
        tmem_ld_32x32(tX + c * 32, sr);
        tmem_ld_wait();
        auto body = [&](auto masked) {
#pragma unroll
          for (int u = 0; u < 32; u += 2) {
            const float2 l2 = *reinterpret_cast<const float2*>(wstat + c * 32 + u);
            float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[u]), __uint_as_float(sr[u + 1])), sc2, l2);
            if (decltype(masked)::value) {
              if (c * 32 + u < cmin) x.x = -INFINITY;
              if (c * 32 + u + 1 < cmin) x.y = -INFINITY;
            }
            pr[c * 32 + u] = ex2_approx(x.x);
            pr[c * 32 + u + 1] = ex2_approx(x.y);
          }
        };
        if (need_mask) body(std::true_type{}); else body(std::false_type{});
        uint32_t pk[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) pk[u] = pack_bf16x2(pr[c * 32 + 2 * u], pr[c * 32 + 2 * u + 1]);
        tmem_st_32x16(tX + c * 16, pk);   // packed P^T over this thread's own columns
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
      // ---- phase b: dS^T = P^T * (dP^T - delta)
      if (!mbar_wait(dp_full, it & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t dr[32];
        tmem_ld_32x32(tY + c * 32, dr);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int u = 0; u < 32; u += 2) {
          const float2 d2 = *reinterpret_cast<const float2*>(wstat + 64 + c * 32 + u);
          const float2 ds = __fmul2_rn(make_float2(pr[c * 32 + u], pr[c * 32 + u + 1]),
                                       __fadd2_rn(make_float2(__uint_as_float(dr[u]), __uint_as_float(dr[u + 1])), d2));
          pk[u >> 1] = pack_bf16x2(ds.x, ds.y);
        }
        tmem_st_32x16(tY + c * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    // epilogue: thread (r, cq) owns D / 2 channels of key row k0 + r of dV and dK (dK carries the softmax scale)
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      if (n_iter > 0) {
        constexpr int CH = D / 2;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* base = which == 0 ? p.dV : p.dK;
          const int col = which == 0 ? DV_COL : DK_COL;
          const float f = which == 0 ? 1.f : p.scale;
#pragma unroll 1
          for (int c = 0; c < CH / 16; ++c) {
            const int c0 = cq * CH + c * 16;
            uint32_t rr[16];
            tmem_ld_32x16(tmem_base + col + lane_addr + c0, rr);
            tmem_ld_wait();
            if (key_ok) {
              __nv_bfloat16* dst = base + ((size_t)(ti.doc_start + kvi) * p.Hkv + hkv) * p.d_mem + c0;
#pragma unroll
              for (int t = 0; t < 2; ++t) {
                if (c0 + t * 8 >= p.d_mem) break;
                uint4 pk;
                pk.x = pack_bf16x2(__uint_as_float(rr[t * 8 + 0]) * f, __uint_as_float(rr[t * 8 + 1]) * f);
                pk.y = pack_bf16x2(__uint_as_float(rr[t * 8 + 2]) * f, __uint_as_float(rr[t * 8 + 3]) * f);
                pk.z = pack_bf16x2(__uint_as_float(rr[t * 8 + 4]) * f, __uint_as_float(rr[t * 8 + 5]) * f);
                pk.w = pack_bf16x2(__uint_as_float(rr[t * 8 + 6]) * f, __uint_as_float(rr[t * 8 + 7]) * f);
                *reinterpret_cast<uint4*>(dst + t * 8) = pk;
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// ------------------------------------------------------------------------------------------------ dQ
// One CTA per 128-query tile and head, streaming 128-key tiles.
// TMEM: S[2] 0/128 (double-buffered, so phase a of step j+1 can start while step j finishes), dP 256, dQ 384.
// Tensor-core order: S(j+1), dQ(j), dP(j+1).
template <int D>
__global__ void __launch_bounds__(64 + 32 * NCW, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int DB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_smem<L::kSlack>(smem_raw);
  if (smem == nullptr) { if (threadIdx.x == 0) atomicCAS(p.status, 0, kErrTimeoutOther); return; }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* qdo_full = bars;         // 1
  uint64_t* acc_done = bars + 1;     // 1
  uint64_t* k_full = bars + 2;       // 3
  uint64_t* k_empty = bars + 5;      // 3
  uint64_t* v_full = bars + 8;       // 2
  uint64_t* v_empty = bars + 10;     // 2
  uint64_t* s_full = bars + 12;      // 2
  uint64_t* s_free = bars + 14;      // 2 (NCW warps): the scores of this buffer are in registers
  uint64_t* dp_full = bars + 16;     // 1
  uint64_t* ds_full = bars + 17;     // 1 (NCW warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, BM);
  if (!ti.valid) return;
  const int hq = blockIdx.y;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? min(ti.doc_len, ti.q0 + BM) : ti.doc_len;
  const int J = (kv_end + BN - 1) / BN;
  constexpr int TMEM_COLS = 512;
  constexpr int S_COL = 0, DP_COL = 256, DQ_COL = 384;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1); mbar_init(acc_done, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&s_free[i], NCW);
    }
    mbar_init(dp_full, 1); mbar_init(ds_full, NCW);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc<TMEM_COLS>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int qrow = ti.doc_start + ti.q0;
      mbar_expect_tx(qdo_full, 2 * L::kTile);
#pragma unroll
      for (int b = 0; b < DB; ++b) {
        tma_load_3d(smem + L::offA + b * 16384, &tmQ, qdo_full, 64 * b, hq, qrow);
        tma_load_3d(smem + L::offB + b * 16384, &tmdO, qdo_full, 64 * b, hq, qrow);
      }
      int ks = 0;             // stage / phase of the K ring (3 stages); the V ring (2 stages) follows j
      uint32_t kph = 1;
      for (int j = 0; j < J; ++j) {
        const int vs = j & 1;
        const int krow = ti.doc_start + j * BN;
        if (!mbar_wait(&k_empty[ks], kph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&k_full[ks], L::kTile);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_3d(smem + L::offC + ks * L::kTile + b * 16384, &tmK, &k_full[ks], 64 * b, hkv, krow);
        if (!mbar_wait(&v_empty[vs], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&v_full[vs], L::kTile);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_3d(smem + L::offD + vs * L::kTile + b * 16384, &tmV, &v_full[vs], 64 * b, hkv, krow);
        if (++ks == 3) { ks = 0; kph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      const uint32_t idesc_q = make_idesc_bf16(128, 16 * p.k_steps, false, true);  // dQ = dS K: A [128 q x 128 kv] from TMEM, B = K_j [128 kv x channels] MN-major
      const SmemDesc dQ = make_desc(smem_u32(smem + L::offA), 16, 1024), dO = make_desc(smem_u32(smem + L::offB), 16, 1024);
      const SmemDesc dKk = make_desc(smem_u32(smem + L::offC), 16, 1024), dVk = make_desc(smem_u32(smem + L::offD), 16, 1024);   // K-major views
      const SmemDesc dKm = make_desc(smem_u32(smem + L::offC), 16384, 1024);                                                     // MN-major view
      auto issue_score = [&](uint32_t dst, SmemDesc a, SmemDesc bk) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk >= p.k_steps) break;
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          if (kk == 0) umma_ss<0>(dst, a, bk, idesc_s); else umma_ss<1>(dst, desc_off(a, off), desc_off(bk, off), idesc_s);
        }
      };
      bool ok = mbar_wait(qdo_full, 0, abort_flag, p.status, kErrTimeoutFull);
      if (ok && J > 0) {
        ok = mbar_wait(&k_full[0], 0, abort_flag, p.status, kErrTimeoutFull);
        if (ok) {
          tc_fence_after();
          issue_score(tmem_base + S_COL, dQ, dKk);
          umma_commit(&s_full[0]);
          ok = mbar_wait(&v_full[0], 0, abort_flag, p.status, kErrTimeoutFull);
        }
        if (ok) {
          tc_fence_after();
          issue_score(tmem_base + DP_COL, dO, dVk);
          umma_commit(dp_full);
          umma_commit(&v_empty[0]);
        }
      }
      int ks = 0, kn = 1;     // K-ring stage of step j and of step j + 1
      uint32_t kn_ph = 0;     // phase of k_full[kn] for step j + 1
      for (int j = 0; j < J && ok; ++j) {
        TRACE(0, j);
        const int nb = (j + 1) & 1;
        const bool more = j + 1 < J;
        if (more) {
          if (!mbar_wait(&k_full[kn], kn_ph, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
          if (!mbar_wait(&s_free[nb], (((j + 1) >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty)) { ok = false; break; }
          tc_fence_after();
          issue_score(tmem_base + S_COL + nb * BN, dQ, desc_off(dKk, kn * L::kTile));
          umma_commit(&s_full[nb]);
        }
        TRACE(1, j);
        if (!mbar_wait(ds_full, j & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        TRACE(2, j);
        tc_fence_after();
        const SmemDesc k = desc_off(dKm, ks * L::kTile);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          if (kk == 0) umma_ts<2>(tmem_base + DQ_COL, tmem_base + DP_COL, k, idesc_q, (uint32_t)j);
          else umma_ts<1>(tmem_base + DQ_COL, tmem_base + DP_COL + packed_col(kk), desc_off(k, kk * 2048), idesc_q);
        }
        umma_commit(&k_empty[ks]);                          // K_j was last read by dQ(j)
        if (more) {
          if (!mbar_wait(&v_full[nb], ((j + 1) >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          issue_score(tmem_base + DP_COL, dO, desc_off(dVk, nb * L::kTile));   // runs after dQ(j), which read the dP buffer
          umma_commit(dp_full);
          umma_commit(&v_empty[nb]);                        // V_{j+1} is only read by dP(j+1)
        }
        ks = kn;
        if (++kn == 3) { kn = 0; kn_ph ^= 1; }
        TRACE(3, j);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int cq = (warp - 2) >> 2;        // column group: keys [64 cq, 64 cq + 64) of the streamed tile
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int qi = ti.q0 + r;
    const bool row_ok = qi < ti.doc_len;
    const size_t tok = (size_t)ti.doc_start + (row_ok ? qi : 0);
    const float neg_lse2 = row_ok ? -p.LSE[(size_t)hq * p.T + tok] * kLog2e : 0.f;
    const float neg_dl = row_ok ? -p.delta[(size_t)hq * p.T + tok] : 0.f;
    const float2 sc2 = make_float2(p.scale_log2, p.scale_log2), nl2 = make_float2(neg_lse2, neg_lse2), nd2 = make_float2(neg_dl, neg_dl);
    // last visible key (local index) of this row; -1 for rows beyond the document
    const int last = !row_ok ? -1 : (p.causal ? min(ti.doc_len - 1, qi) : ti.doc_len - 1);
    const uint32_t tDP = tmem_base + DP_COL + cq * CPT + lane_addr;
    bool ok = true;
    for (int j = 0; j < J && ok; ++j) {
      const int b = j & 1;
      // ---- phase a: P = exp2(S * scale - lse), kept in registers
      if (threadIdx.x == 64) TRACE(8, j);
      if (!mbar_wait(&s_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      if (threadIdx.x == 64) TRACE(9, j);
      tc_fence_after();
      const bool need_mask = (j * BN + BN > ti.doc_len) || (ti.q0 + BM > ti.doc_len) || (p.causal && j * BN + BN - 1 > ti.q0);
      const int umax = last - (j * BN + cq * CPT);   // columns u <= umax are visible
      float pr[CPT];
      uint32_t sr[CPT];
      tmem_ld_32x32(tmem_base + S_COL + b * BN + cq * CPT + lane_addr, as32(&sr[0]));
      tmem_ld_32x32(tmem_base + S_COL + b * BN + cq * CPT + 32 + lane_addr, as32(&sr[32]));
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free[b]);
      if (threadIdx.x == 64) TRACE(10, j);
      auto body = [&](auto masked) {
#pragma unroll
        for (int u = 0; u < CPT; u += 2) {
          float2 x = __ffma2_rn(make_float2(__uint_as_float(sr[u]), __uint_as_float(sr[u + 1])), sc2, nl2);
          if (decltype(masked)::value) {
            if (u > umax) x.x = -INFINITY;
            if (u + 1 > umax) x.y = -INFINITY;
          }
          pr[u] = ex2_approx(x.x);
          pr[u + 1] = ex2_approx(x.y);
        }
      };
      if (need_mask) body(std::true_type{}); else body(std::false_type{});
      if (threadIdx.x == 64) TRACE(11, j);
      // ---- phase b: dS = P * (dP - delta)
      if (!mbar_wait(dp_full, j & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      if (threadIdx.x == 64) TRACE(12, j);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t dr[32];
        tmem_ld_32x32(tDP + c * 32, dr);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int u = 0; u < 32; u += 2) {
          const float2 ds = __fmul2_rn(make_float2(pr[c * 32 + u], pr[c * 32 + u + 1]),
                                       __fadd2_rn(make_float2(__uint_as_float(dr[u]), __uint_as_float(dr[u + 1])), nd2));
          pk[u >> 1] = pack_bf16x2(ds.x, ds.y);
        }
        tmem_st_32x16(tDP + c * 16, pk);   // packed dS over this thread's own (already read) columns
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
      if (threadIdx.x == 64) TRACE(13, j);
    }
    // epilogue: thread (r, cq) owns D / 2 channels of query row q0 + r (dQ carries the softmax scale)
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      constexpr int CH = D / 2;
#pragma unroll 1
      for (int c = 0; c < CH / 16; ++c) {
        const int c0 = cq * CH + c * 16;
        uint32_t rr[16];
        tmem_ld_32x16(tmem_base + DQ_COL + lane_addr + c0, rr);
        tmem_ld_wait();
        if (row_ok && J > 0) {
          __nv_bfloat16* dst = p.dQ + (tok * p.Hq + hq) * p.d_mem + c0;
          const float f = p.scale;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (c0 + t * 8 >= p.d_mem) break;
            uint4 pk;
            pk.x = pack_bf16x2(__uint_as_float(rr[t * 8 + 0]) * f, __uint_as_float(rr[t * 8 + 1]) * f);
            pk.y = pack_bf16x2(__uint_as_float(rr[t * 8 + 2]) * f, __uint_as_float(rr[t * 8 + 3]) * f);
            pk.z = pack_bf16x2(__uint_as_float(rr[t * 8 + 4]) * f, __uint_as_float(rr[t * 8 + 5]) * f);
            pk.w = pack_bf16x2(__uint_as_float(rr[t * 8 + 6]) * f, __uint_as_float(rr[t * 8 + 7]) * f);
            *reinterpret_cast<uint4*>(dst + t * 8) = pk;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// tensor map over a [T, H, d] bf16 activation with token stride `ld` and head stride `hs` (elements), boxes of
// {64 channels, 1 head, 128 tokens}; channels of a box beyond d read as zeros
int make_act_tmap(CUtensorMap* m, const void* base, int T, int H, int d, long ld, long hs) {
  return vlmt_make_tmap_3d_bf16(m, base, (uint64_t)d, (uint64_t)H, (uint64_t)T, (uint64_t)hs * 2, (uint64_t)ld * 2, 64, 1, 128);
}

template <typename K>
int set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace

// head size 256: the single-tile kernels of attention256_sm100.cu
extern "C" int vlmt_attn256_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu, int n_docs, int T, int Hq,
                                int Hkv, long ldq, long ldk, long ldv, float scale, int causal, int* status, cudaStream_t st);
extern "C" int vlmt_attn256_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse, float* delta,
                                void* dq, void* dk, void* dv, const int* cu, int n_docs, int T, int Hq, int Hkv, float scale, int causal,
                                int* status, cudaStream_t st);

extern "C" int vlmt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu, int n_docs, int T, int Hq,
                             int Hkv, int d, long ldq, long hsq, long ldk, long hsk, long ldv, long hsv, float scale, int causal, int* status,
                             cudaStream_t st) {
  if (T <= 0 || n_docs <= 0) return 0;
  if (d == 256) {
    if (hsq != 256 || hsk != 256 || hsv != 256) return -11;
    return vlmt_attn256_fwd(q, k, v, o, lse, cu, n_docs, T, Hq, Hkv, ldq, ldk, ldv, scale, causal, status, st);
  }
  if (d <= 0 || d > 128 || (d & 7)) return -10;
  const int D = d <= 64 ? 64 : 128;   // tile width; TMA zero-fills the channels between d and D
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_act_tmap(&tq, q, T, Hq, d, ldq, hsq))) return 1000 + r;
  if ((r = make_act_tmap(&tk, k, T, Hkv, d, ldk, hsk))) return 2000 + r;
  if ((r = make_act_tmap(&tv, v, T, Hkv, d, ldv, hsv))) return 3000 + r;
  FwdParams p;
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.LSE = lse; p.cu = cu; p.n_docs = n_docs; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale_log2 = scale * kLog2e; p.causal = causal; p.status = status;
  p.k_steps = (d + 15) / 16;
  p.d_mem = d;
  dim3 grid(T / (2 * BM) + n_docs + 1, Hq);
  if (D == 128) {
    if ((r = set_smem(attn_fwd_kernel<128>, FwdSmem<128>::kTotal))) return r;
    attn_fwd_kernel<128><<<grid, ATT_THREADS, FwdSmem<128>::kTotal, st>>>(tq, tk, tv, p);
  } else {
    if ((r = set_smem(attn_fwd_kernel<64>, FwdSmem<64>::kTotal))) return r;
    attn_fwd_kernel<64><<<grid, ATT_THREADS, FwdSmem<64>::kTotal, st>>>(tq, tk, tv, p);
  }
  return (int)cudaGetLastError();
}

extern "C" int vlmt_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse, float* delta,
                             void* dq, void* dk, void* dv, const int* cu, int n_docs, int T, int Hq, int Hkv, int d, long ldq, long hsq,
                             long ldk, long hsk, long ldv, long hsv, float scale, int causal, int* status, cudaStream_t st) {
  if (T <= 0 || n_docs <= 0) return 0;
  if (d == 256) {
    if (hsq != 256 || hsk != 256 || hsv != 256 || ldq != (long)Hq * 256 || ldk != (long)Hkv * 256 || ldv != (long)Hkv * 256) return -11;
    return vlmt_attn256_bwd(dout, q, k, v, o, lse, delta, dq, dk, dv, cu, n_docs, T, Hq, Hkv, scale, causal, status, st);
  }
  if (d <= 0 || d > 128 || (d & 7)) return -10;
  const int D = d <= 64 ? 64 : 128;
  {
    const int warps = T * Hq;
    attn_delta_kernel<<<(warps * 32 + 255) / 256, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
                                                                reinterpret_cast<const __nv_bfloat16*>(o), delta, T, Hq, d);
  }
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_act_tmap(&tq, q, T, Hq, d, ldq, hsq))) return 1000 + r;
  if ((r = make_act_tmap(&tk, k, T, Hkv, d, ldk, hsk))) return 2000 + r;
  if ((r = make_act_tmap(&tv, v, T, Hkv, d, ldv, hsv))) return 3000 + r;
  if ((r = make_act_tmap(&tdo, dout, T, Hq, d, (long)Hq * d, d))) return 4000 + r;
  BwdParams p;
  p.dQ = reinterpret_cast<__nv_bfloat16*>(dq); p.dK = reinterpret_cast<__nv_bfloat16*>(dk); p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.LSE = lse; p.delta = delta; p.cu = cu; p.n_docs = n_docs; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * kLog2e; p.causal = causal; p.status = status;
  p.trace = nullptr;
  p.k_steps = (d + 15) / 16;
  p.d_mem = d;
#ifdef VLMT_ATTN_TRACE
  static long long* trace_buf = nullptr;
  if (!trace_buf) cudaMalloc(&trace_buf, 256 * 16 * sizeof(long long));
  cudaMemset(trace_buf, 0, 256 * 16 * sizeof(long long));
  p.trace = trace_buf;
#endif
  dim3 grid_kv(T / BN + n_docs + 1, Hkv), grid_q(T / BM + n_docs + 1, Hq);
  auto launch = [&](auto dtag) -> int {
    constexpr int Dh = decltype(dtag)::value;
    int rr;
    if ((rr = set_smem(attn_bwd_dkdv_kernel<Dh>, BwdSmem<Dh>::kTotal))) return rr;
    if ((rr = set_smem(attn_bwd_dq_kernel<Dh>, BwdSmem<Dh>::kTotal))) return rr;
    attn_bwd_dkdv_kernel<Dh><<<grid_kv, 64 + 32 * NCW, BwdSmem<Dh>::kTotal, st>>>(tq, tk, tv, tdo, p);
    attn_bwd_dq_kernel<Dh><<<grid_q, 64 + 32 * NCW, BwdSmem<Dh>::kTotal, st>>>(tq, tk, tv, tdo, p);
    return 0;
  };
  if (D == 128) r = launch(std::integral_constant<int, 128>{});
  else if (D == 64) r = launch(std::integral_constant<int, 64>{});
  else return -10;
  if (r) return r;
#ifdef VLMT_ATTN_TRACE
  {
    static int dumps = 0;
    cudaStreamSynchronize(st);
    static long long host[256 * 16];
    cudaMemcpy(host, p.trace, sizeof(host), cudaMemcpyDeviceToHost);
    if (dumps++ == 2) {
      const long long t0 = host[0];
      for (int j = 0; j < 256 && host[j * 16]; ++j) {
        fprintf(stderr, "TRACE j=%d mma:", j);
        for (int k = 0; k < 4; ++k) fprintf(stderr, " %lld", host[j * 16 + k] - t0);
        fprintf(stderr, " | cw:");
        for (int k = 8; k < 14; ++k) fprintf(stderr, " %lld", host[j * 16 + k] - t0);
        fprintf(stderr, "\n");
      }
    }
  }
#endif
  return (int)cudaGetLastError();
}
