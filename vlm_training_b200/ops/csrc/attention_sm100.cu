// Varlen (packed-row) flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// All three kernels use ten warps: warp 0 issues TMA loads, one thread of warp 1 issues every MMA, warps 2..9 do
// the CUDA-core work between the MMAs (two warps per scheduler, so one warp's latencies hide behind the other).
// Probabilities and score gradients go back to the tensor core through tensor memory (they overwrite the fp32
// scores they were computed from and are read as the A operand of the next MMA), never through shared memory.
//
// Forward: one CTA per (256 queries of one document = two 128-row tiles, query head).  Warps 2..5 own tile 0 and
//   warps 6..9 tile 1, one query row per thread (tcgen05.ld gives a thread its whole row: row max and row sum need
//   no shuffles).  The MMA thread alternates between the tiles - P0.V, S0', P1.V, S1' - so the tensor core works
//   on one tile while the softmax of the other runs.  O accumulates in TMEM; it is rescaled only when a row's
//   running max grows by more than 2^8 (the stale max is used meanwhile, which only changes the common scale
//   of P and l).
// Backward: `attn_bwd_dkdv` (one CTA per 128-key tile and kv head; loops over 64-query tiles and the query heads of
//   the GQA group) and `attn_bwd_dq` (one CTA per 128-query tile and head; loops over 64-key tiles) recompute
//   S and dP = dO V^T on the tensor cores; each compute thread handles half of a 64-wide row.  No atomics:
//   results are bit-reproducible.
//
// Documents are [cu_seqlens[i], cu_seqlens[i+1]); tiles never mix documents: keys past the end of the document
// (and, with `causal`, keys after the query) are masked before the softmax.
#include "attention_sm100.h"
#include "sm100.cuh"

#include <cuda_bf16.h>
#include <math.h>

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
        for (int b = 0; b < DB; ++b) tma_load_2d(smem + L::offQ + t * L::kQ + b * 16384, &tmQ, q_full, hq * D + 64 * b, row0 + t * BM);
      for (int j = 0; j < J; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        const int krow = ti.doc_start + j * BN;
        if (!mbar_wait(&k_empty[s], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&k_full[s], L::kKV);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_2d(smem + L::offK + s * L::kKV + b * 16384, &tmK, &k_full[s], hkv * D + 64 * b, krow);
        if (!mbar_wait(&v_empty[s], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&v_full[s], L::kKV);
#pragma unroll
        for (int b = 0; b < DB; ++b) tma_load_2d(smem + L::offV + s * L::kKV + b * 16384, &tmV, &v_full[s], hkv * D + 64 * b, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BM, BN, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BM, D, false, true);
      // S_t(j) = Q_t K_j^T.  It overwrites P_t(j-1), whose consumer P_t(j-1).V was issued earlier by this thread.
      auto issue_S = [&](int t, int j) {
        const uint32_t sQ = smem_u32(smem + L::offQ + t * L::kQ);
        const uint32_t sK = smem_u32(smem + L::offK + (j & 1) * L::kKV);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + S_COL + t * BN, make_smem_desc(sQ + off, 16, 1024), make_smem_desc(sK + off, 16, 1024), idesc_s, kk != 0);
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
        const uint32_t sV = smem_u32(smem + L::offV + s * L::kKV);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= Jt[t]) continue;
          if (!mbar_wait(&p_full[t], j & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk)  // A = P_t: 128 lanes x 8 columns of packed bf16 pairs per 16 keys
            umma_bf16_ts(tmem_base + O_COL + t * D, tmem_base + S_COL + t * BN + kk * 8, make_smem_desc(sV + kk * 2048, 16384, 1024),
                         idesc_pv, (j | kk) != 0);
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
      for (int i = 0; i < BN; i += 4) {
        mx0 = fmaxf(mx0, __uint_as_float(s[i]));     mx1 = fmaxf(mx1, __uint_as_float(s[i + 1]));
        mx2 = fmaxf(mx2, __uint_as_float(s[i + 2])); mx3 = fmaxf(mx3, __uint_as_float(s[i + 3]));
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
      __nv_bfloat16* dst = p.O + (tok * p.Hq + hq) * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(o_addr + c * 32, o);
        tmem_ld_wait();
        if (qi < ti.doc_len) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
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
  int* status;
};

// Backward tiles.  Both kernels keep a 128-row "stationary" tile (keys for dK/dV, queries for dQ) in shared memory and
// stream 64-row tiles of the other operand through a 3-stage ring, so that S and dP take 64 TMEM columns each and are
// double-buffered: the tensor core computes S/dP of step i+1 while the compute warps turn step i into P / dS, and the
// accumulation MMAs of step i overlap the CUDA-core work of step i+1.  P / dS are written as packed bf16 over the
// fp32 scores they came from and are read from tensor memory as the A operand.
constexpr int BS = 64;   // rows of the streamed tile
constexpr int NST = 3;   // stages of the streamed ring

template <int D>
struct BwdSmem {
  static constexpr int kBig = 128 * D * 2;     // stationary [128 x D] tile
  static constexpr int kSmall = BS * D * 2;    // streamed [64 x D] tile
  static constexpr int offA = 0;                        // dkdv: K_j   | dq: Q_i
  static constexpr int offB = offA + kBig;              // dkdv: V_j   | dq: dO_i
  static constexpr int offC = offB + kBig;              // NST stages: dkdv Q_i  | dq K_j
  static constexpr int offD = offC + NST * kSmall;      // NST stages: dkdv dO_i | dq V_j
  static constexpr int offStat = offD + NST * kSmall;   // per compute warp: lse2[32], delta[32] floats
  static constexpr int offBar = offStat + 8 * 64 * 4;
  static constexpr int kTotal = offBar + 256 + 1024;
};

// Column of the packed-bf16 A operand inside a 64-column fp32 buffer for k-step kk (16 rows of the streamed tile):
// the warps of column half h write their 32 values as 16 packed words at column 32 h, so no warp overwrites scores
// that the other half has not read yet.
__device__ __forceinline__ constexpr int packed_col(int kk) { return (kk >> 1) * 32 + (kk & 1) * 8; }

// dK_j, dV_j for one 128-key tile and one kv head.  Everything is computed transposed (rows = keys):
//   S^T = K Q^T, dP^T = V dO^T  (M = 128 keys, N = 64 queries)   ->  P^T, dS^T (thread = key row, half of the queries)
//   dV += P^T dO,  dK += dS^T Q  (A = [128 keys x 64 queries] from TMEM, B = the [64 x D] query-side tile read MN-major)
// TMEM columns: S^T[2] 0/64, dP^T[2] 128/192, dV 256, dK 256 + D.
template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int DB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* kv_full = bars;          // 1
  uint64_t* acc_done = bars + 1;     // 1
  uint64_t* qdo_full = bars + 2;     // NST
  uint64_t* qdo_empty = bars + 5;    // NST
  uint64_t* sdp_full = bars + 8;     // 2
  uint64_t* pds_full = bars + 10;    // 2 (8 warps)
  uint64_t* buf_free = bars + 12;    // 2: the accumulation MMAs that read P^T / dS^T of this buffer have finished
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat = reinterpret_cast<float*>(smem + L::offStat);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, 128);
  if (!ti.valid) return;
  const int hkv = blockIdx.y;
  const int group = p.Hq / p.Hkv;
  const int k0 = ti.q0;  // first key row of the tile (local to the document)
  const int n_qblk = (ti.doc_len + BS - 1) / BS;
  const int i_first = p.causal ? k0 / BS : 0;
  const int n_iter = (n_qblk - i_first) * group;
  constexpr int TMEM_COLS = 512;
  constexpr int ST_COL = 0, DPT_COL = 128, DV_COL = 256, DK_COL = 256 + D;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(acc_done, 1);
    for (int i = 0; i < NST; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sdp_full[i], 1); mbar_init(&pds_full[i], 8); mbar_init(&buf_free[i], 1); }
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
      mbar_expect_tx(kv_full, 2 * L::kBig);
#pragma unroll
      for (int b = 0; b < DB; ++b) {
        tma_load_2d(smem + L::offA + b * 16384, &tmK, kv_full, hkv * D + 64 * b, krow);
        tma_load_2d(smem + L::offB + b * 16384, &tmV, kv_full, hkv * D + 64 * b, krow);
      }
      int sg = 0;
      uint32_t ph = 1;
      for (int it = 0; it < n_iter; ++it) {
        const int i = i_first + it / group, hq = hkv * group + it % group;
        if (!mbar_wait(&qdo_empty[sg], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        const int qrow = ti.doc_start + i * BS;
        mbar_expect_tx(&qdo_full[sg], 2 * L::kSmall);
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_2d(smem + L::offC + sg * L::kSmall + b * 8192, &tmQ, &qdo_full[sg], hq * D + 64 * b, qrow);
          tma_load_2d(smem + L::offD + sg * L::kSmall + b * 8192, &tmdO, &qdo_full[sg], hq * D + 64 * b, qrow);
        }
        if (++sg == NST) { sg = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, BS, false, false);   // [128 keys] x [64 queries], contraction over d
      constexpr uint32_t idesc_g = make_idesc_bf16(128, D, false, true);      // [128 keys] x [D], contraction over 64 queries
      const uint32_t sK = smem_u32(smem + L::offA), sV = smem_u32(smem + L::offB);
      auto issue_sdp = [&](int it) -> bool {
        const int sg = it % NST, b = it & 1;
        if (!mbar_wait(&qdo_full[sg], (it / NST) & 1, abort_flag, p.status, kErrTimeoutFull)) return false;
        if (!mbar_wait(&buf_free[b], ((it >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + L::offC + sg * L::kSmall), sdO = smem_u32(smem + L::offD + sg * L::kSmall);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offk = (kk >> 2) * 16384 + (kk & 3) * 32, offq = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + ST_COL + b * BS, make_smem_desc(sK + offk, 16, 1024), make_smem_desc(sQ + offq, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offk = (kk >> 2) * 16384 + (kk & 3) * 32, offq = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + DPT_COL + b * BS, make_smem_desc(sV + offk, 16, 1024), make_smem_desc(sdO + offq, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&sdp_full[b]);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kErrTimeoutFull);
      if (ok && n_iter > 0) ok = issue_sdp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it + 1 < n_iter) { ok = issue_sdp(it + 1); if (!ok) break; }
        const int sg = it % NST, b = it & 1;
        if (!mbar_wait(&pds_full[b], (it >> 1) & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + L::offC + sg * L::kSmall), sdO = smem_u32(smem + L::offD + sg * L::kSmall);
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          umma_bf16_ts(tmem_base + DV_COL, tmem_base + ST_COL + b * BS + packed_col(kk), make_smem_desc(sdO + kk * 2048, 8192, 1024), idesc_g,
                       (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          umma_bf16_ts(tmem_base + DK_COL, tmem_base + DPT_COL + b * BS + packed_col(kk), make_smem_desc(sQ + kk * 2048, 8192, 1024), idesc_g,
                       (it | kk) != 0);
        umma_commit(&qdo_empty[sg]);
        umma_commit(&buf_free[b]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int cw = warp - 2;
    const int ch = cw >> 2;                // column half: queries [32 ch, 32 ch + 32) of the streamed tile
    const int q = warp & 3;                // TMEM lane quarter this warp may access
    const int r = q * 32 + lane;           // key row of the tile owned by this thread
    const int kvi = k0 + r;                // key index local to the document
    const bool key_ok = kvi < ti.doc_len;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float* wstat = stat + cw * 64;
    // per-query statistics: lane l fetches those of query 32 ch + l one step ahead
    auto fetch = [&](int it, float& l2, float& dl) {
      const int i = i_first + it / group, hq = hkv * group + it % group;
      const int qq = i * BS + ch * 32 + lane;
      const bool qok = qq < ti.doc_len;
      const size_t idx = (size_t)hq * p.T + ti.doc_start + (qok ? qq : 0);
      l2 = qok ? p.LSE[idx] * kLog2e : INFINITY;  // +inf -> exp2(-inf) = 0 for queries beyond the document
      dl = qok ? p.delta[idx] : 0.f;
    };
    float nl2 = 0.f, ndl = 0.f;
    if (n_iter > 0) fetch(0, nl2, ndl);
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int b = it & 1;
      const int q0 = (i_first + it / group) * BS + ch * 32;   // first query of this thread's columns
      __syncwarp();
      wstat[lane] = nl2;
      wstat[32 + lane] = ndl;
      __syncwarp();
      if (it + 1 < n_iter) fetch(it + 1, nl2, ndl);
      if (!mbar_wait(&sdp_full[b], (it >> 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[32], dr[32];
      tmem_ld_32x32(tmem_base + ST_COL + b * BS + ch * 32 + lane_addr, sr);
      tmem_ld_32x32(tmem_base + DPT_COL + b * BS + ch * 32 + lane_addr, dr);
      tmem_ld_wait();
      // masked: keys beyond the document, or (causal) keys after the query
      const bool need_mask = (k0 + 128 > ti.doc_len) || (p.causal && k0 + 127 > q0);
      uint32_t pp[16], dd[16];
#pragma unroll
      for (int u4 = 0; u4 < 8; ++u4) {
        const float4 l4 = reinterpret_cast<const float4*>(wstat)[u4];
        const float4 d4 = reinterpret_cast<const float4*>(wstat + 32)[u4];
        const float ls[4] = {l4.x, l4.y, l4.z, l4.w}, dls[4] = {d4.x, d4.y, d4.z, d4.w};
        float pv[4], dsv[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int u = u4 * 4 + e;
          float x = fmaf(__uint_as_float(sr[u]), p.scale_log2, -ls[e]);
          if (need_mask && !(key_ok && (!p.causal || kvi <= q0 + u))) x = -INFINITY;
          pv[e] = ex2_approx(x);
          dsv[e] = pv[e] * (__uint_as_float(dr[u]) - dls[e]);
        }
        pp[u4 * 2] = pack_bf16x2(pv[0], pv[1]);  pp[u4 * 2 + 1] = pack_bf16x2(pv[2], pv[3]);
        dd[u4 * 2] = pack_bf16x2(dsv[0], dsv[1]); dd[u4 * 2 + 1] = pack_bf16x2(dsv[2], dsv[3]);
      }
      tmem_st_32x16(tmem_base + ST_COL + b * BS + ch * 32 + lane_addr, pp);
      tmem_st_32x16(tmem_base + DPT_COL + b * BS + ch * 32 + lane_addr, dd);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[b]);
    }
    // epilogue: thread (r, ch) owns channels [ch D/2, (ch+1) D/2) of key row k0 + r of dV and dK (dK carries the softmax scale)
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      if (n_iter > 0) {
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* base = which == 0 ? p.dV : p.dK;
          const int col = which == 0 ? DV_COL : DK_COL;
          const float f = which == 0 ? 1.f : p.scale;
#pragma unroll 1
          for (int c = 0; c < D / 64; ++c) {
            const int c0 = ch * (D / 2) + c * 32;
            uint32_t rr[32];
            tmem_ld_32x32(tmem_base + col + lane_addr + c0, rr);
            tmem_ld_wait();
            if (key_ok) {
              __nv_bfloat16* dst = base + ((size_t)(ti.doc_start + kvi) * p.Hkv + hkv) * D + c0;
#pragma unroll
              for (int t = 0; t < 4; ++t) {
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

// dQ_i for one 128-query tile and head, streaming 64-key tiles.  TMEM: S[2] 0/64, dP[2] 128/192, dQ 256.
template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int DB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* qdo_full = bars;         // 1
  uint64_t* acc_done = bars + 1;     // 1
  uint64_t* kv_full = bars + 2;      // NST
  uint64_t* kv_empty = bars + 5;     // NST
  uint64_t* sdp_full = bars + 8;     // 2
  uint64_t* ds_full = bars + 10;     // 2 (8 warps)
  uint64_t* buf_free = bars + 12;    // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, BM);
  if (!ti.valid) return;
  const int hq = blockIdx.y;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? min(ti.doc_len, ti.q0 + BM) : ti.doc_len;
  const int J = (kv_end + BS - 1) / BS;
  constexpr int TMEM_COLS = 512;
  constexpr int S_COL = 0, DP_COL = 128, DQ_COL = 256;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1); mbar_init(acc_done, 1);
    for (int i = 0; i < NST; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(&sdp_full[i], 1); mbar_init(&ds_full[i], 8); mbar_init(&buf_free[i], 1); }
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
      mbar_expect_tx(qdo_full, 2 * L::kBig);
#pragma unroll
      for (int b = 0; b < DB; ++b) {
        tma_load_2d(smem + L::offA + b * 16384, &tmQ, qdo_full, hq * D + 64 * b, qrow);
        tma_load_2d(smem + L::offB + b * 16384, &tmdO, qdo_full, hq * D + 64 * b, qrow);
      }
      int sg = 0;
      uint32_t ph = 1;
      for (int j = 0; j < J; ++j) {
        if (!mbar_wait(&kv_empty[sg], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        const int krow = ti.doc_start + j * BS;
        mbar_expect_tx(&kv_full[sg], 2 * L::kSmall);
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_2d(smem + L::offC + sg * L::kSmall + b * 8192, &tmK, &kv_full[sg], hkv * D + 64 * b, krow);
          tma_load_2d(smem + L::offD + sg * L::kSmall + b * 8192, &tmV, &kv_full[sg], hkv * D + 64 * b, krow);
        }
        if (++sg == NST) { sg = 0; ph ^= 1; }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, BS, false, false);
      constexpr uint32_t idesc_q = make_idesc_bf16(128, D, false, true);  // dQ = dS K: A [128 q x 64 kv] from TMEM, B = K_j [64 kv x D] MN-major
      const uint32_t sQ = smem_u32(smem + L::offA), sdO = smem_u32(smem + L::offB);
      auto issue_sdp = [&](int j) -> bool {
        const int sg = j % NST, b = j & 1;
        if (!mbar_wait(&kv_full[sg], (j / NST) & 1, abort_flag, p.status, kErrTimeoutFull)) return false;
        if (!mbar_wait(&buf_free[b], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + L::offC + sg * L::kSmall), sV = smem_u32(smem + L::offD + sg * L::kSmall);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offq = (kk >> 2) * 16384 + (kk & 3) * 32, offk = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + S_COL + b * BS, make_smem_desc(sQ + offq, 16, 1024), make_smem_desc(sK + offk, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offq = (kk >> 2) * 16384 + (kk & 3) * 32, offk = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + DP_COL + b * BS, make_smem_desc(sdO + offq, 16, 1024), make_smem_desc(sV + offk, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&sdp_full[b]);
        return true;
      };
      bool ok = mbar_wait(qdo_full, 0, abort_flag, p.status, kErrTimeoutFull);
      if (ok && J > 0) ok = issue_sdp(0);
      for (int j = 0; j < J && ok; ++j) {
        if (j + 1 < J) { ok = issue_sdp(j + 1); if (!ok) break; }
        const int sg = j % NST, b = j & 1;
        if (!mbar_wait(&ds_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + L::offC + sg * L::kSmall);
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          umma_bf16_ts(tmem_base + DQ_COL, tmem_base + DP_COL + b * BS + packed_col(kk), make_smem_desc(sK + kk * 2048, 8192, 1024), idesc_q,
                       (j | kk) != 0);
        umma_commit(&kv_empty[sg]);
        umma_commit(&buf_free[b]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int ch = (warp - 2) >> 2;        // column half: keys [32 ch, 32 ch + 32) of the streamed tile
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int qi = ti.q0 + r;
    const bool row_ok = qi < ti.doc_len;
    const size_t tok = (size_t)ti.doc_start + (row_ok ? qi : 0);
    const float neg_lse2 = row_ok ? -p.LSE[(size_t)hq * p.T + tok] * kLog2e : 0.f;
    const float dl = row_ok ? p.delta[(size_t)hq * p.T + tok] : 0.f;
    bool ok = true;
    for (int j = 0; j < J && ok; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&sdp_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      uint32_t sr[32], dr[32];
      tmem_ld_32x32(tmem_base + S_COL + b * BS + ch * 32 + lane_addr, sr);
      tmem_ld_32x32(tmem_base + DP_COL + b * BS + ch * 32 + lane_addr, dr);
      tmem_ld_wait();
      const int kv0 = j * BS + ch * 32;
      const bool need_mask = (j * BS + BS > ti.doc_len) || (ti.q0 + BM > ti.doc_len) || (p.causal && j * BS + BS - 1 > ti.q0);
      uint32_t dd[16];
#pragma unroll
      for (int u2 = 0; u2 < 16; ++u2) {
        float dsv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int u = u2 * 2 + e;
          float x = fmaf(__uint_as_float(sr[u]), p.scale_log2, neg_lse2);
          if (need_mask && !(row_ok && kv0 + u < ti.doc_len && (!p.causal || kv0 + u <= qi))) x = -INFINITY;
          dsv[e] = ex2_approx(x) * (__uint_as_float(dr[u]) - dl);
        }
        dd[u2] = pack_bf16x2(dsv[0], dsv[1]);
      }
      tmem_st_32x16(tmem_base + DP_COL + b * BS + ch * 32 + lane_addr, dd);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[b]);
    }
    // epilogue: thread (r, ch) owns channels [ch D/2, (ch+1) D/2) of query row q0 + r (dQ carries the softmax scale)
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < D / 64; ++c) {
        const int c0 = ch * (D / 2) + c * 32;
        uint32_t rr[32];
        tmem_ld_32x32(tmem_base + DQ_COL + lane_addr + c0, rr);
        tmem_ld_wait();
        if (row_ok && J > 0) {
          __nv_bfloat16* dst = p.dQ + (tok * p.Hq + hq) * D + c0;
          const float f = p.scale;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
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

// tensor map over a [T, H*D] bf16 activation with row stride `ld` elements, boxes of {64 channels, 128 tokens}
int make_act_tmap(CUtensorMap* m, const void* base, int T, int HD, long ld, int box_rows = 128) {
  return vlmt_make_tmap_2d_bf16(m, base, (uint64_t)HD, (uint64_t)T, (uint64_t)ld * 2, 64, (uint32_t)box_rows);
}

template <typename K>
int set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

}  // namespace

extern "C" int vlmt_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu, int n_docs, int T, int Hq,
                             int Hkv, int D, int d_eff, long ldq, long ldk, long ldv, float scale, int causal, int* status, cudaStream_t st) {
  if (T <= 0 || n_docs <= 0) return 0;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_act_tmap(&tq, q, T, Hq * D, ldq))) return 1000 + r;
  if ((r = make_act_tmap(&tk, k, T, Hkv * D, ldk))) return 2000 + r;
  if ((r = make_act_tmap(&tv, v, T, Hkv * D, ldv))) return 3000 + r;
  FwdParams p;
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.LSE = lse; p.cu = cu; p.n_docs = n_docs; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale_log2 = scale * kLog2e; p.causal = causal; p.status = status;
  (void)d_eff;
  dim3 grid(T / (2 * BM) + n_docs + 1, Hq);
  if (D == 128) {
    if ((r = set_smem(attn_fwd_kernel<128>, FwdSmem<128>::kTotal))) return r;
    attn_fwd_kernel<128><<<grid, ATT_THREADS, FwdSmem<128>::kTotal, st>>>(tq, tk, tv, p);
  } else if (D == 64) {
    if ((r = set_smem(attn_fwd_kernel<64>, FwdSmem<64>::kTotal))) return r;
    attn_fwd_kernel<64><<<grid, ATT_THREADS, FwdSmem<64>::kTotal, st>>>(tq, tk, tv, p);
  } else {
    return -10;
  }
  return (int)cudaGetLastError();
}

extern "C" int vlmt_attn_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse, float* delta,
                             void* dq, void* dk, void* dv, const int* cu, int n_docs, int T, int Hq, int Hkv, int D, int d_eff, float scale,
                             int causal, int* status, cudaStream_t st) {
  if (T <= 0 || n_docs <= 0) return 0;
  {
    const int warps = T * Hq;
    attn_delta_kernel<<<(warps * 32 + 255) / 256, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
                                                                reinterpret_cast<const __nv_bfloat16*>(o), delta, T, Hq, D);
  }
  // 128-row boxes for the stationary tiles, 64-row boxes for the streamed ones
  CUtensorMap tq, tk, tv, tdo, tq64, tk64, tv64, tdo64;
  int r;
  if ((r = make_act_tmap(&tq, q, T, Hq * D, (long)Hq * D))) return 1000 + r;
  if ((r = make_act_tmap(&tk, k, T, Hkv * D, (long)Hkv * D))) return 2000 + r;
  if ((r = make_act_tmap(&tv, v, T, Hkv * D, (long)Hkv * D))) return 3000 + r;
  if ((r = make_act_tmap(&tdo, dout, T, Hq * D, (long)Hq * D))) return 4000 + r;
  if ((r = make_act_tmap(&tq64, q, T, Hq * D, (long)Hq * D, 64))) return 5000 + r;
  if ((r = make_act_tmap(&tk64, k, T, Hkv * D, (long)Hkv * D, 64))) return 6000 + r;
  if ((r = make_act_tmap(&tv64, v, T, Hkv * D, (long)Hkv * D, 64))) return 7000 + r;
  if ((r = make_act_tmap(&tdo64, dout, T, Hq * D, (long)Hq * D, 64))) return 8000 + r;
  BwdParams p;
  p.dQ = reinterpret_cast<__nv_bfloat16*>(dq); p.dK = reinterpret_cast<__nv_bfloat16*>(dk); p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.LSE = lse; p.delta = delta; p.cu = cu; p.n_docs = n_docs; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * kLog2e; p.causal = causal; p.status = status;
  (void)d_eff;
  dim3 grid_kv(T / BN + n_docs + 1, Hkv), grid_q(T / BM + n_docs + 1, Hq);
  if (D == 128) {
    if ((r = set_smem(attn_bwd_dkdv_kernel<128>, BwdSmem<128>::kTotal))) return r;
    if ((r = set_smem(attn_bwd_dq_kernel<128>, BwdSmem<128>::kTotal))) return r;
    attn_bwd_dkdv_kernel<128><<<grid_kv, ATT_THREADS, BwdSmem<128>::kTotal, st>>>(tq64, tk, tv, tdo64, p);
    attn_bwd_dq_kernel<128><<<grid_q, ATT_THREADS, BwdSmem<128>::kTotal, st>>>(tq, tk64, tv64, tdo, p);
  } else if (D == 64) {
    if ((r = set_smem(attn_bwd_dkdv_kernel<64>, BwdSmem<64>::kTotal))) return r;
    if ((r = set_smem(attn_bwd_dq_kernel<64>, BwdSmem<64>::kTotal))) return r;
    attn_bwd_dkdv_kernel<64><<<grid_kv, ATT_THREADS, BwdSmem<64>::kTotal, st>>>(tq64, tk, tv, tdo64, p);
    attn_bwd_dq_kernel<64><<<grid_q, ATT_THREADS, BwdSmem<64>::kTotal, st>>>(tq, tk64, tv64, tdo, p);
  } else {
    return -10;
  }
  return (int)cudaGetLastError();
}
