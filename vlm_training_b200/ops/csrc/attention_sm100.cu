// Varlen (packed-row) flash attention for sm_100a on tcgen05 tensor cores with TMEM accumulators.
//
// Forward: one CTA per (128-query tile of one document, query head).
//   warp 0      TMA: Q once, then K_j / V_j tiles through 2-stage rings
//   warp 1      MMA issuer: S_j = Q K_j^T into one of two TMEM S buffers (issued one tile ahead),
//               PV_j = P_j V_j into one of two TMEM PV buffers
//   warps 2..5  softmax: one query row per thread (tcgen05.ld gives a thread its whole row, so
//               row max / row sum need no shuffles), P_j written as bf16 into swizzled smem for
//               the second MMA, running output kept in registers and rescaled as PV tiles arrive
// Backward: `attn_bwd_dkdv` (one CTA per key tile and kv head, loops over the query tiles and the
// query heads of the GQA group) and `attn_bwd_dq` (one CTA per query tile and head) recompute
// S and dP = dO V^T on the tensor cores; no atomics, results are bit-reproducible.
//
// Documents are [cu_seqlens[i], cu_seqlens[i+1]); tiles never mix documents: keys past the end of
// the document (and, with `causal`, keys after the query) are masked to -inf before the softmax.
#include "attention_sm100.h"
#include "sm100.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace {
using namespace sm100;

constexpr int BM = 128, BN = 128;
constexpr int ATT_THREADS = 192;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct TileInfo {
  int doc_start, doc_len, q0;  // q0: first query row of the tile, local to the document
  bool valid;
};

// Linear tile id -> (document, query block).  Tiles are numbered document by document.
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

struct FwdParams {
  __nv_bfloat16* O;   // [T, Hq, D]
  float* LSE;         // [Hq, T]
  const int* cu;
  int n_docs, T, Hq, Hkv;
  float scale_log2;   // softmax scale * log2(e)
  int causal;
  int d_eff;          // channels that can be non-zero (multiple of 16, <= D): MMAs skip the zero padding beyond it
  int* status;
};

template <int D>
struct FwdSmem {
  static constexpr int kQ = BM * D * 2;
  static constexpr int kKV = BN * D * 2;
  static constexpr int kP = BM * BN * 2;
  static constexpr int offQ = 0;
  static constexpr int offK = offQ + kQ;          // 2 stages
  static constexpr int offV = offK + 2 * kKV;     // 2 stages
  static constexpr int offP = offV + 2 * kKV;     // 2 buffers
  static constexpr int offBar = offP + 2 * kP;
  static constexpr int kTotal = offBar + 256 + 1024;
};

// write 8 packed bf16 (16 B) of row r, logical column col (multiple of 8) into a [128 x 128] bf16 tile stored
// as two 64-column blocks of [128 rows][128 B] with the 128-byte swizzle
__device__ __forceinline__ void st_swizzled_16B(uint8_t* tile, int r, int col, uint4 v) {
  const int block = col >> 6;
  const int ci = (col & 63) >> 3;
  *reinterpret_cast<uint4*>(tile + block * 16384 + r * 128 + ((ci ^ (r & 7)) << 4)) = v;
}

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
  uint64_t* k_full = bars + 1;        // 2
  uint64_t* k_empty = bars + 3;       // 2
  uint64_t* v_full = bars + 5;        // 2
  uint64_t* v_empty = bars + 7;       // 2
  uint64_t* s_full = bars + 9;        // 2
  uint64_t* s_empty = bars + 11;      // 2
  uint64_t* p_full = bars + 13;       // 2
  uint64_t* p_empty = bars + 15;      // 2
  uint64_t* pv_full = bars + 17;      // 2
  uint64_t* pv_empty = bars + 19;     // 2
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, BM);
  if (!ti.valid) return;  // uniform for the whole CTA
  const int hq = blockIdx.y;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? min(ti.doc_len, ti.q0 + BM) : ti.doc_len;
  const int J = (kv_end + BN - 1) / BN;
  constexpr int TMEM_COLS = 512;
  constexpr int S_COL = 0, PV_COL = 256;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_empty[i], 4); mbar_init(&p_full[i], 4); mbar_init(&p_empty[i], 1);
      mbar_init(&pv_full[i], 1); mbar_init(&pv_empty[i], 4);
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
      mbar_expect_tx(q_full, L::kQ);
#pragma unroll
      for (int b = 0; b < DB; ++b) tma_load_2d(smem + L::offQ + b * 16384, &tmQ, q_full, hq * D + 64 * b, row0);
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
      const uint32_t idesc_pv = make_idesc_bf16(BM, p.d_eff, false, true);
      const uint32_t sQ = smem_u32(smem + L::offQ);
      auto issue_S = [&](int j) -> bool {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[s], ph, abort_flag, p.status, kErrTimeoutFull)) return false;
        if (!mbar_wait(&s_empty[s], ph ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + L::offK + s * L::kKV);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk * 16 >= p.d_eff) break;
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + S_COL + s * BN, make_smem_desc(sQ + off, 16, 1024), make_smem_desc(sK + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&s_full[s]);
        umma_commit(&k_empty[s]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kErrTimeoutFull);
      if (ok && J > 0) ok = issue_S(0);
      for (int j = 0; j < J && ok; ++j) {
        if (j + 1 < J) { ok = issue_S(j + 1); if (!ok) break; }
        const int b = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&p_full[b], ph, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        if (!mbar_wait(&v_full[b], ph, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
        if (!mbar_wait(&pv_empty[b], ph ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sP = smem_u32(smem + L::offP + b * L::kP);
        const uint32_t sV = smem_u32(smem + L::offV + b * L::kKV);
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t adesc = make_smem_desc(sP + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(sV + kk * 2048, 16384, 1024);
          umma_bf16(tmem_base + PV_COL + b * D, adesc, bdesc, idesc_pv, kk != 0);
        }
        umma_commit(&pv_full[b]);
        umma_commit(&v_empty[b]);
        umma_commit(&p_empty[b]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax / output warps
    const int q = warp & 3;
    const int r = q * 32 + lane;           // row of the tile owned by this thread
    const int qi = ti.q0 + r;              // query index local to the document
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float m = -INFINITY, l = 0.f, alpha_pending = 1.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < J && ok; ++j) {
      const int b = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&s_full[b], ph, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem_base + S_COL + b * BN + lane_addr;
      const int kv0 = j * BN;
      const bool need_mask = (kv0 + BN > ti.doc_len) || (p.causal && kv0 + BN - 1 > ti.q0);
      const int limit = p.causal ? min(ti.doc_len - 1, qi) : ti.doc_len - 1;  // last visible key (local index)
      // pass 1: row max of the raw scores (the softmax scale is positive, so it commutes with max)
      float mx_raw = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(s_addr + c * 32, rr);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) if (kv0 + c * 32 + i <= limit) mx_raw = fmaxf(mx_raw, __uint_as_float(rr[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx_raw = fmaxf(mx_raw, __uint_as_float(rr[i]));
        }
      }
      const float mx = fmaxf(m, mx_raw * p.scale_log2);
      const float m_use = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_use);
      m = mx;
      if (!mbar_wait(&p_empty[b], ph ^ 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
      // pass 2: probabilities -> smem (bf16), row sum
      uint8_t* sP = smem + L::offP + b * L::kP;
      float rowsum = 0.f;
      const float neg_m = -m_use;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(s_addr + c * 32, rr);
        tmem_ld_wait();
        float pr[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = exp2f(fmaf(__uint_as_float(rr[i]), p.scale_log2, neg_m));
          if (need_mask && kv0 + c * 32 + i > limit) e = 0.f;
          pr[i] = e;
          rowsum += e;
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint4 pk;
          __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int u = 0; u < 4; ++u) p2[u] = __floats2bfloat162_rn(pr[t * 8 + 2 * u], pr[t * 8 + 2 * u + 1]);
          st_swizzled_16B(sP, r, c * 32 + t * 8, pk);
        }
      }
      tc_fence_before();
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) { mbar_arrive(&s_empty[b]); mbar_arrive(&p_full[b]); }
      l = l * alpha + rowsum;
      // fold in the previous tile's P.V while the tensor core works on this one
      if (j > 0) {
        const int pb = (j - 1) & 1;
        const uint32_t pph = ((j - 1) >> 1) & 1;
        if (!mbar_wait(&pv_full[pb], pph, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
        const uint32_t pv_addr = tmem_base + PV_COL + pb * D + lane_addr;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          if (c * 32 < p.d_eff) {  // columns at and beyond d_eff were never written by the MMA: leave those outputs at zero
            uint32_t rr[32];
            tmem_ld_32x32(pv_addr + c * 32, rr);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < p.d_eff) o[c * 32 + i] = o[c * 32 + i] * alpha_pending + __uint_as_float(rr[i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&pv_empty[pb]);
      }
      alpha_pending = alpha;
    }
    if (ok && J > 0) {
      const int pb = (J - 1) & 1;
      const uint32_t pph = ((J - 1) >> 1) & 1;
      if (mbar_wait(&pv_full[pb], pph, abort_flag, p.status, kErrTimeoutTmemFull)) {
        tc_fence_after();
        const uint32_t pv_addr = tmem_base + PV_COL + pb * D + lane_addr;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          if (c * 32 < p.d_eff) {  // columns at and beyond d_eff were never written by the MMA: leave those outputs at zero
            uint32_t rr[32];
            tmem_ld_32x32(pv_addr + c * 32, rr);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i < p.d_eff) o[c * 32 + i] = o[c * 32 + i] * alpha_pending + __uint_as_float(rr[i]);
          }
        }
      } else {
        ok = false;
      }
    }
    if (ok && qi < ti.doc_len) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const size_t tok = (size_t)(ti.doc_start + qi);
      __nv_bfloat16* dst = p.O + (tok * p.Hq + hq) * D;
#pragma unroll
      for (int i = 0; i < D; i += 8) {
        uint4 pk;
        __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
        for (int u = 0; u < 4; ++u) p2[u] = __floats2bfloat162_rn(o[i + 2 * u] * inv, o[i + 2 * u + 1] * inv);
        *reinterpret_cast<uint4*>(dst + i) = pk;
      }
      p.LSE[(size_t)hq * p.T + tok] = l > 0.f ? (m + log2f(l)) * kLn2 : -INFINITY;
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
  int d_eff;
  int* status;
};

// Backward tiles.  Both kernels work on a 128-row "stationary" tile (keys for dK/dV, queries for dQ) and stream
// 64-row tiles of the other operand, so that S and dP take only 64 TMEM columns each and can be double-buffered:
// the tensor core computes S/dP of step i+1 while the CUDA cores turn step i into P / dS, and the accumulation MMAs
// of step i overlap the CUDA-core work of step i+1.
constexpr int BS = 64;  // rows of the streamed tile

template <int D>
struct BwdSmem {
  static constexpr int kBig = 128 * D * 2;     // stationary [128 x D] tile
  static constexpr int kSmall = BS * D * 2;    // streamed [64 x D] tile
  static constexpr int kSq = 128 * BS * 2;     // [128 x 64] bf16 tile (P^T / dS^T / dS)
  static constexpr int offA = 0;                       // dkdv: K_j   | dq: Q_i
  static constexpr int offB = offA + kBig;             // dkdv: V_j   | dq: dO_i
  static constexpr int offC = offB + kBig;             // 2 stages: dkdv Q_i  | dq K_j
  static constexpr int offD = offC + 2 * kSmall;       // 2 stages: dkdv dO_i | dq V_j
  static constexpr int offP = offD + 2 * kSmall;       // 2 buffers (dkdv: P^T)
  static constexpr int offDS = offP + 2 * kSq;         // 2 buffers (dS^T / dS)
  static constexpr int offStat = offDS + 2 * kSq;      // per compute warp: (lse2[64], delta[64]) floats
  static constexpr int offBar = offStat + 4 * 128 * 4;
  static constexpr int kTotal = offBar + 256 + 1024;
};

// 16 bytes of row r, column col (multiple of 8, < 64) of a [rows x 64] bf16 tile with 128-byte rows and 128-byte swizzle
__device__ __forceinline__ void st_sw64_16B(uint8_t* tile, int r, int col, uint4 v) {
  *reinterpret_cast<uint4*>(tile + r * 128 + (((col >> 3) ^ (r & 7)) << 4)) = v;
}

// dK_j, dV_j for one 128-key tile and one kv head.  Everything is computed transposed (rows = keys):
//   S^T = K Q^T, dP^T = V dO^T  (M = 128 keys, N = 64 queries)   ->  P^T, dS^T (thread = key row)
//   dV += P^T dO,  dK += dS^T Q  (A = [128 keys x 64 queries] K-major, B = the [64 x D] query-side tile read MN-major)
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
  uint64_t* qdo_full = bars + 1;     // 2
  uint64_t* qdo_empty = bars + 3;    // 2
  uint64_t* sdp_full = bars + 5;     // 2
  uint64_t* sdp_empty = bars + 7;    // 2 (4 warps)
  uint64_t* pds_full = bars + 9;     // 2 (4 warps)
  uint64_t* pds_empty = bars + 11;   // 2
  uint64_t* acc_done = bars + 13;    // 1
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); mbar_init(&sdp_full[i], 1); mbar_init(&sdp_empty[i], 4);
      mbar_init(&pds_full[i], 4); mbar_init(&pds_empty[i], 1);
    }
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
      for (int it = 0; it < n_iter; ++it) {
        const int st = it & 1;
        const int i = i_first + it / group, hq = hkv * group + it % group;
        if (!mbar_wait(&qdo_empty[st], ((it >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        const int qrow = ti.doc_start + i * BS;
        mbar_expect_tx(&qdo_full[st], 2 * L::kSmall);
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_2d(smem + L::offC + st * L::kSmall + b * 8192, &tmQ, &qdo_full[st], hq * D + 64 * b, qrow);
          tma_load_2d(smem + L::offD + st * L::kSmall + b * 8192, &tmdO, &qdo_full[st], hq * D + 64 * b, qrow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, BS, false, false);   // [128 keys] x [64 queries], contraction over d
      constexpr uint32_t idesc_g = make_idesc_bf16(128, D, false, true);      // [128 keys] x [D], contraction over 64 queries
      const uint32_t sK = smem_u32(smem + L::offA), sV = smem_u32(smem + L::offB);
      auto issue_sdp = [&](int it) -> bool {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&qdo_full[st], ph, abort_flag, p.status, kErrTimeoutFull)) return false;
        if (!mbar_wait(&sdp_empty[st], ph ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + L::offC + st * L::kSmall), sdO = smem_u32(smem + L::offD + st * L::kSmall);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offk = (kk >> 2) * 16384 + (kk & 3) * 32, offq = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + ST_COL + st * BS, make_smem_desc(sK + offk, 16, 1024), make_smem_desc(sQ + offq, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offk = (kk >> 2) * 16384 + (kk & 3) * 32, offq = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + DPT_COL + st * BS, make_smem_desc(sV + offk, 16, 1024), make_smem_desc(sdO + offq, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&sdp_full[st]);
        return true;
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kErrTimeoutFull);
      if (ok && n_iter > 0) ok = issue_sdp(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        if (it + 1 < n_iter) { ok = issue_sdp(it + 1); if (!ok) break; }
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!mbar_wait(&pds_full[st], ph, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sQ = smem_u32(smem + L::offC + st * L::kSmall), sdO = smem_u32(smem + L::offD + st * L::kSmall);
        const uint32_t sPT = smem_u32(smem + L::offP + st * L::kSq), sDST = smem_u32(smem + L::offDS + st * L::kSq);
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          umma_bf16(tmem_base + DV_COL, make_smem_desc(sPT + kk * 32, 16, 1024), make_smem_desc(sdO + kk * 2048, 8192, 1024), idesc_g,
                    (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          umma_bf16(tmem_base + DK_COL, make_smem_desc(sDST + kk * 32, 16, 1024), make_smem_desc(sQ + kk * 2048, 8192, 1024), idesc_g,
                    (it | kk) != 0);
        umma_commit(&qdo_empty[st]);
        umma_commit(&pds_empty[st]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;           // key row of the tile owned by this thread
    const int kvi = k0 + r;                // key index local to the document
    const bool key_ok = kvi < ti.doc_len;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int st = it & 1;
      const uint32_t ph = (it >> 1) & 1;
      const int i = i_first + it / group, hq = hkv * group + it % group;
      const int q0 = i * BS;
      // per-query statistics of this step -> this warp's own smem copy (warp-local, so no block barrier is involved)
      float* wstat = stat + q * 128;
      __syncwarp();
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int qc = lane + 32 * h;
        const int qq = q0 + qc;
        const bool qok = qq < ti.doc_len;
        const size_t tok = (size_t)ti.doc_start + (qok ? qq : 0);
        wstat[qc] = qok ? p.LSE[(size_t)hq * p.T + tok] * kLog2e : INFINITY;  // +inf -> exp2(-inf) = 0 for padded queries
        wstat[64 + qc] = qok ? p.delta[(size_t)hq * p.T + tok] : 0.f;
      }
      __syncwarp();
      if (!mbar_wait(&sdp_full[st], ph, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const float* lse2 = wstat;
      const float* dl = wstat + 64;
      float pr[BS], ds[BS];
#pragma unroll
      for (int c = 0; c < BS / 32; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld_32x32(tmem_base + ST_COL + st * BS + lane_addr + c * 32, sr);
        tmem_ld_32x32(tmem_base + DPT_COL + st * BS + lane_addr + c * 32, dr);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const int qc = c * 32 + u;
          const bool vis = key_ok && (!p.causal || kvi <= q0 + qc);
          const float pv = vis ? exp2f(fmaf(__uint_as_float(sr[u]), p.scale_log2, -lse2[qc])) : 0.f;
          pr[qc] = pv;
          ds[qc] = pv * (__uint_as_float(dr[u]) - dl[qc]) * p.scale;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sdp_empty[st]);
      if (!mbar_wait(&pds_empty[st], ph ^ 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
      uint8_t* sPT = smem + L::offP + st * L::kSq;
      uint8_t* sDST = smem + L::offDS + st * L::kSq;
#pragma unroll
      for (int t = 0; t < BS / 8; ++t) {
        uint4 a, b;
        __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&a);
        __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          a2[u] = __floats2bfloat162_rn(pr[t * 8 + 2 * u], pr[t * 8 + 2 * u + 1]);
          b2[u] = __floats2bfloat162_rn(ds[t * 8 + 2 * u], ds[t * 8 + 2 * u + 1]);
        }
        st_sw64_16B(sPT, r, t * 8, a);
        st_sw64_16B(sDST, r, t * 8, b);
      }
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[st]);
    }
    // epilogue: thread r owns key row k0 + r of dV and dK
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      if (n_iter > 0) {
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* base = which == 0 ? p.dV : p.dK;
          const int col = which == 0 ? DV_COL : DK_COL;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t rr[32];
            tmem_ld_32x32(tmem_base + col + lane_addr + c * 32, rr);
            tmem_ld_wait();
            if (key_ok) {
              __nv_bfloat16* dst = base + ((size_t)(ti.doc_start + kvi) * p.Hkv + hkv) * D + c * 32;
#pragma unroll
              for (int t = 0; t < 4; ++t) {
                uint4 pk;
                __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                  p2[u] = __floats2bfloat162_rn(__uint_as_float(rr[t * 8 + 2 * u]), __uint_as_float(rr[t * 8 + 2 * u + 1]));
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
  uint64_t* kv_full = bars + 1;      // 2
  uint64_t* kv_empty = bars + 3;     // 2
  uint64_t* sdp_full = bars + 5;     // 2
  uint64_t* sdp_empty = bars + 7;    // 2 (4 warps)
  uint64_t* ds_full = bars + 9;      // 2 (4 warps)
  uint64_t* ds_empty = bars + 11;    // 2
  uint64_t* acc_done = bars + 13;
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&sdp_full[i], 1); mbar_init(&sdp_empty[i], 4);
      mbar_init(&ds_full[i], 4); mbar_init(&ds_empty[i], 1);
    }
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
      for (int j = 0; j < J; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        const int krow = ti.doc_start + j * BS;
        mbar_expect_tx(&kv_full[st], 2 * L::kSmall);
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_2d(smem + L::offC + st * L::kSmall + b * 8192, &tmK, &kv_full[st], hkv * D + 64 * b, krow);
          tma_load_2d(smem + L::offD + st * L::kSmall + b * 8192, &tmV, &kv_full[st], hkv * D + 64 * b, krow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, BS, false, false);
      constexpr uint32_t idesc_q = make_idesc_bf16(128, D, false, true);  // dQ = dS K: A [128 q x 64 kv] K-major, B = K_j [64 kv x D] MN-major
      const uint32_t sQ = smem_u32(smem + L::offA), sdO = smem_u32(smem + L::offB);
      auto issue_sdp = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&kv_full[st], ph, abort_flag, p.status, kErrTimeoutFull)) return false;
        if (!mbar_wait(&sdp_empty[st], ph ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty)) return false;
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + L::offC + st * L::kSmall), sV = smem_u32(smem + L::offD + st * L::kSmall);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offq = (kk >> 2) * 16384 + (kk & 3) * 32, offk = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + S_COL + st * BS, make_smem_desc(sQ + offq, 16, 1024), make_smem_desc(sK + offk, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t offq = (kk >> 2) * 16384 + (kk & 3) * 32, offk = (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + DP_COL + st * BS, make_smem_desc(sdO + offq, 16, 1024), make_smem_desc(sV + offk, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(&sdp_full[st]);
        return true;
      };
      bool ok = mbar_wait(qdo_full, 0, abort_flag, p.status, kErrTimeoutFull);
      if (ok && J > 0) ok = issue_sdp(0);
      for (int j = 0; j < J && ok; ++j) {
        if (j + 1 < J) { ok = issue_sdp(j + 1); if (!ok) break; }
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&ds_full[st], ph, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        const uint32_t sK = smem_u32(smem + L::offC + st * L::kSmall);
        const uint32_t sDS = smem_u32(smem + L::offDS + st * L::kSq);
#pragma unroll
        for (int kk = 0; kk < BS / 16; ++kk)
          umma_bf16(tmem_base + DQ_COL, make_smem_desc(sDS + kk * 32, 16, 1024), make_smem_desc(sK + kk * 2048, 8192, 1024), idesc_q,
                    (j | kk) != 0);
        umma_commit(&kv_empty[st]);
        umma_commit(&ds_empty[st]);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const int qi = ti.q0 + r;
    const bool row_ok = qi < ti.doc_len;
    const size_t tok = (size_t)ti.doc_start + (row_ok ? qi : 0);
    const float lse2 = row_ok ? p.LSE[(size_t)hq * p.T + tok] * kLog2e : 0.f;
    const float dl = row_ok ? p.delta[(size_t)hq * p.T + tok] : 0.f;
    bool ok = true;
    for (int j = 0; j < J && ok; ++j) {
      const int st = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      if (!mbar_wait(&sdp_full[st], ph, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BS;
      float ds[BS];
#pragma unroll
      for (int c = 0; c < BS / 32; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld_32x32(tmem_base + S_COL + st * BS + lane_addr + c * 32, sr);
        tmem_ld_32x32(tmem_base + DP_COL + st * BS + lane_addr + c * 32, dr);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const int kv = kv0 + c * 32 + u;
          const bool vis = row_ok && kv < ti.doc_len && (!p.causal || kv <= qi);
          const float pv = vis ? exp2f(fmaf(__uint_as_float(sr[u]), p.scale_log2, -lse2)) : 0.f;
          ds[c * 32 + u] = pv * (__uint_as_float(dr[u]) - dl) * p.scale;
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sdp_empty[st]);
      if (!mbar_wait(&ds_empty[st], ph ^ 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
      uint8_t* sDS = smem + L::offDS + st * L::kSq;
#pragma unroll
      for (int t = 0; t < BS / 8; ++t) {
        uint4 b;
        __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
        for (int u = 0; u < 4; ++u) b2[u] = __floats2bfloat162_rn(ds[t * 8 + 2 * u], ds[t * 8 + 2 * u + 1]);
        st_sw64_16B(sDS, r, t * 8, b);
      }
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[st]);
    }
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(tmem_base + DQ_COL + lane_addr + c * 32, rr);
        tmem_ld_wait();
        if (row_ok && J > 0) {
          __nv_bfloat16* dst = p.dQ + (tok * p.Hq + hq) * D + c * 32;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint4 pk;
            __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
            for (int u = 0; u < 4; ++u)
              p2[u] = __floats2bfloat162_rn(__uint_as_float(rr[t * 8 + 2 * u]), __uint_as_float(rr[t * 8 + 2 * u + 1]));
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
  p.d_eff = (d_eff <= 0 || d_eff > D) ? D : ((d_eff + 15) / 16) * 16;
  dim3 grid(T / BM + n_docs + 1, Hq);
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
  p.d_eff = (d_eff <= 0 || d_eff > D) ? D : ((d_eff + 15) / 16) * 16;
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
