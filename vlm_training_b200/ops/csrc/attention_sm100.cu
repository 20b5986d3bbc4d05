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
      // pass 1: row max
      float mx = m;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(s_addr + c * 32, rr);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) { const float x = __uint_as_float(rr[i]) * p.scale_log2; if (kv0 + c * 32 + i <= limit) mx = fmaxf(mx, x); }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(rr[i]) * p.scale_log2);
        }
      }
      const float m_use = (mx == -INFINITY) ? 0.f : mx;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f(m - m_use);
      m = mx;
      if (!mbar_wait(&p_empty[b], ph ^ 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
      // pass 2: probabilities -> smem (bf16), row sum
      uint8_t* sP = smem + L::offP + b * L::kP;
      float rowsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t rr[32];
        tmem_ld_32x32(s_addr + c * 32, rr);
        tmem_ld_wait();
        float pr[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = exp2f(__uint_as_float(rr[i]) * p.scale_log2 - m_use);
          if (need_mask && kv0 + c * 32 + i > limit) e = 0.f;
          pr[i] = e;
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint4 pk;
          __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            p2[u] = __floats2bfloat162_rn(pr[t * 8 + 2 * u], pr[t * 8 + 2 * u + 1]);
            // sum what the tensor core will actually see (bf16-rounded), keeps O / l consistent
            const float2 back = __bfloat1622float2(p2[u]);
            rowsum += back.x + back.y;
          }
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

// Shared layout of both backward kernels: four [128 x D] operand tiles + two [128 x 128] bf16 tiles (P, dS)
template <int D>
struct BwdSmem {
  static constexpr int kTile = 128 * D * 2;
  static constexpr int kSq = 128 * 128 * 2;
  static constexpr int offA = 0;              // dkdv: K_j   | dq: Q_i
  static constexpr int offB = offA + kTile;   // dkdv: V_j   | dq: dO_i
  static constexpr int offC = offB + kTile;   // dkdv: Q_i   | dq: K_j
  static constexpr int offD = offC + kTile;   // dkdv: dO_i  | dq: V_j
  static constexpr int offP = offD + kTile;
  static constexpr int offDS = offP + kSq;
  static constexpr int offBar = offDS + kSq;
  static constexpr int kTotal = offBar + 256 + 1024;
};

// dK_j, dV_j for one key tile and one kv head: loop over the GQA group's query heads and the query tiles
// that can see this key tile.  TMEM: S | dP | dV | dK (4 x 128 columns for D = 128).
template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int DB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* kv_full = bars;        // K_j and V_j landed
  uint64_t* qdo_full = bars + 1;   // Q_i and dO_i landed
  uint64_t* qdo_empty = bars + 2;  // all MMAs reading Q_i / dO_i done
  uint64_t* sdp_full = bars + 3;   // S and dP computed
  uint64_t* pds_full = bars + 4;   // P and dS written to smem (4 warps)
  uint64_t* acc_done = bars + 5;   // final dV/dK accumulation done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, BN);
  if (!ti.valid) return;
  const int hkv = blockIdx.y;
  const int group = p.Hq / p.Hkv;
  const int k0 = ti.q0;  // first key row of the tile (local)
  const int n_qblk = (ti.doc_len + BM - 1) / BM;
  const int i_first = p.causal ? k0 / BM : 0;
  const int n_iter = (n_qblk - i_first) * group;
  constexpr int TMEM_COLS = 512;
  constexpr int S_COL = 0, DP_COL = 128, DV_COL = 256, DK_COL = 256 + D;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(qdo_empty, 1); mbar_init(sdp_full, 1);
    mbar_init(pds_full, 4); mbar_init(acc_done, 1);
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
        tma_load_2d(smem + L::offA + b * 16384, &tmK, kv_full, hkv * D + 64 * b, krow);
        tma_load_2d(smem + L::offB + b * 16384, &tmV, kv_full, hkv * D + 64 * b, krow);
      }
      for (int it = 0; it < n_iter; ++it) {
        const int i = i_first + it / group, hq = hkv * group + it % group;
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        const int qrow = ti.doc_start + i * BM;
        mbar_expect_tx(qdo_full, 2 * L::kTile);
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_2d(smem + L::offC + b * 16384, &tmQ, qdo_full, hq * D + 64 * b, qrow);
          tma_load_2d(smem + L::offD + b * 16384, &tmdO, qdo_full, hq * D + 64 * b, qrow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);   // S = Q K^T, dP = dO V^T
      const uint32_t idesc_g = make_idesc_bf16(128, p.d_eff, true, true);     // dV = P^T dO, dK = dS^T Q
      const uint32_t sK = smem_u32(smem + L::offA), sV = smem_u32(smem + L::offB);
      const uint32_t sQ = smem_u32(smem + L::offC), sdO = smem_u32(smem + L::offD);
      const uint32_t sP = smem_u32(smem + L::offP), sDS = smem_u32(smem + L::offDS);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kErrTimeoutFull);
      for (int it = 0; it < n_iter && ok; ++it) {
        const uint32_t ph = it & 1;
        if (!mbar_wait(qdo_full, ph, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk * 16 >= p.d_eff) break;
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + S_COL, make_smem_desc(sQ + off, 16, 1024), make_smem_desc(sK + off, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk * 16 >= p.d_eff) break;
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + DP_COL, make_smem_desc(sdO + off, 16, 1024), make_smem_desc(sV + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(sdp_full);
        if (!mbar_wait(pds_full, ph, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        // contraction over the 128 query rows: P / dS are [q][kv] tiles read as MN-major A (M = kv),
        // dO / Q are [q][d] tiles read as MN-major B (N = d)
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {
          umma_bf16(tmem_base + DV_COL, make_smem_desc(sP + kk * 2048, 16384, 1024), make_smem_desc(sdO + kk * 2048, 16384, 1024),
                    idesc_g, (it | kk) != 0);
        }
#pragma unroll
        for (int kk = 0; kk < BM / 16; ++kk) {
          umma_bf16(tmem_base + DK_COL, make_smem_desc(sDS + kk * 2048, 16384, 1024), make_smem_desc(sQ + kk * 2048, 16384, 1024),
                    idesc_g, (it | kk) != 0);
        }
        umma_commit(qdo_empty);
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;  // query row within the tile
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int i = i_first + it / group, hq = hkv * group + it % group;
      const uint32_t ph = it & 1;
      const int qi = i * BM + r;
      const bool row_ok = qi < ti.doc_len;
      const size_t tok = (size_t)ti.doc_start + (row_ok ? qi : 0);
      const float lse2 = row_ok ? p.LSE[(size_t)hq * p.T + tok] * kLog2e : 0.f;
      const float dl = row_ok ? p.delta[(size_t)hq * p.T + tok] : 0.f;
      if (!mbar_wait(sdp_full, ph, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      // the previous iteration's dV/dK MMAs (which read sP / sDS) completed before S/dP of this one were
      // committed: tcgen05 MMAs of one CTA execute in issue order, so the buffers are free to overwrite
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld_32x32(tmem_base + S_COL + lane_addr + c * 32, sr);
        tmem_ld_32x32(tmem_base + DP_COL + lane_addr + c * 32, dr);
        tmem_ld_wait();
        float pr[32], ds[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const int kv = k0 + c * 32 + u;
          const bool vis = row_ok && kv < ti.doc_len && (!p.causal || kv <= qi);
          const float pv = vis ? exp2f(__uint_as_float(sr[u]) * p.scale_log2 - lse2) : 0.f;
          pr[u] = pv;
          ds[u] = pv * (__uint_as_float(dr[u]) - dl) * p.scale;
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint4 a, b;
          __nv_bfloat162* a2 = reinterpret_cast<__nv_bfloat162*>(&a);
          __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            a2[u] = __floats2bfloat162_rn(pr[t * 8 + 2 * u], pr[t * 8 + 2 * u + 1]);
            b2[u] = __floats2bfloat162_rn(ds[t * 8 + 2 * u], ds[t * 8 + 2 * u + 1]);
          }
          st_swizzled_16B(smem + L::offP, r, c * 32 + t * 8, a);
          st_swizzled_16B(smem + L::offDS, r, c * 32 + t * 8, b);
        }
      }
      tc_fence_before();
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    // epilogue: thread r owns key row k0 + r of dV and dK
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      const int kvi = k0 + r;
      if (n_iter > 0) {
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* base = which == 0 ? p.dV : p.dK;
          const int col = which == 0 ? DV_COL : DK_COL;
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t rr[32];
            if (c * 32 < p.d_eff) {
              tmem_ld_32x32(tmem_base + col + lane_addr + c * 32, rr);
              tmem_ld_wait();
            }
#pragma unroll
            for (int u = 0; u < 32; ++u) if (c * 32 + u >= p.d_eff) rr[u] = 0u;
            if (kvi < ti.doc_len) {
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

// dQ_i for one query tile and head: loop over the key tiles it can see.  TMEM: S | dP | dQ.
template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, BwdParams p) {
  using L = BwdSmem<D>;
  constexpr int DB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* qdo_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* ds_full = bars + 4;
  uint64_t* acc_done = bars + 5;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, BM);
  if (!ti.valid) return;
  const int hq = blockIdx.y;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? min(ti.doc_len, ti.q0 + BM) : ti.doc_len;
  const int J = (kv_end + BN - 1) / BN;
  constexpr int TMEM_COLS = 512;
  constexpr int S_COL = 0, DP_COL = 128, DQ_COL = 256;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1); mbar_init(kv_full, 1); mbar_init(kv_empty, 1); mbar_init(sdp_full, 1);
    mbar_init(ds_full, 4); mbar_init(acc_done, 1);
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
        tma_load_2d(smem + L::offA + b * 16384, &tmQ, qdo_full, hq * D + 64 * b, qrow);
        tma_load_2d(smem + L::offB + b * 16384, &tmdO, qdo_full, hq * D + 64 * b, qrow);
      }
      for (int j = 0; j < J; ++j) {
        if (!mbar_wait(kv_empty, (j & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        const int krow = ti.doc_start + j * BN;
        mbar_expect_tx(kv_full, 2 * L::kTile);
#pragma unroll
        for (int b = 0; b < DB; ++b) {
          tma_load_2d(smem + L::offC + b * 16384, &tmK, kv_full, hkv * D + 64 * b, krow);
          tma_load_2d(smem + L::offD + b * 16384, &tmV, kv_full, hkv * D + 64 * b, krow);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
      const uint32_t idesc_q = make_idesc_bf16(128, p.d_eff, false, true);  // dQ = dS K : A K-major [q][kv], B = K [kv][d] MN-major
      const uint32_t sQ = smem_u32(smem + L::offA), sdO = smem_u32(smem + L::offB);
      const uint32_t sK = smem_u32(smem + L::offC), sV = smem_u32(smem + L::offD);
      const uint32_t sDS = smem_u32(smem + L::offDS);
      bool ok = mbar_wait(qdo_full, 0, abort_flag, p.status, kErrTimeoutFull);
      for (int j = 0; j < J && ok; ++j) {
        const uint32_t ph = j & 1;
        if (!mbar_wait(kv_full, ph, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk * 16 >= p.d_eff) break;
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + S_COL, make_smem_desc(sQ + off, 16, 1024), make_smem_desc(sK + off, 16, 1024), idesc_s, kk != 0);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          if (kk * 16 >= p.d_eff) break;
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + DP_COL, make_smem_desc(sdO + off, 16, 1024), make_smem_desc(sV + off, 16, 1024), idesc_s, kk != 0);
        }
        umma_commit(sdp_full);
        if (!mbar_wait(ds_full, ph, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
          const uint64_t adesc = make_smem_desc(sDS + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024);
          const uint64_t bdesc = make_smem_desc(sK + kk * 2048, 16384, 1024);
          umma_bf16(tmem_base + DQ_COL, adesc, bdesc, idesc_q, (j | kk) != 0);
        }
        umma_commit(kv_empty);
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
      const uint32_t ph = j & 1;
      if (!mbar_wait(sdp_full, ph, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const int kv0 = j * BN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld_32x32(tmem_base + S_COL + lane_addr + c * 32, sr);
        tmem_ld_32x32(tmem_base + DP_COL + lane_addr + c * 32, dr);
        tmem_ld_wait();
        float ds[32];
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const int kv = kv0 + c * 32 + u;
          const bool vis = row_ok && kv < ti.doc_len && (!p.causal || kv <= qi);
          const float pv = vis ? exp2f(__uint_as_float(sr[u]) * p.scale_log2 - lse2) : 0.f;
          ds[u] = pv * (__uint_as_float(dr[u]) - dl) * p.scale;
        }
#pragma unroll
        for (int t = 0; t < 4; ++t) {
          uint4 b;
          __nv_bfloat162* b2 = reinterpret_cast<__nv_bfloat162*>(&b);
#pragma unroll
          for (int u = 0; u < 4; ++u) b2[u] = __floats2bfloat162_rn(ds[t * 8 + 2 * u], ds[t * 8 + 2 * u + 1]);
          st_swizzled_16B(smem + L::offDS, r, c * 32 + t * 8, b);
        }
      }
      tc_fence_before();
      fence_async_proxy();
      __syncwarp();
      if (lane == 0) mbar_arrive(ds_full);
    }
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t rr[32];
        if (c * 32 < p.d_eff) {
          tmem_ld_32x32(tmem_base + DQ_COL + lane_addr + c * 32, rr);
          tmem_ld_wait();
        }
#pragma unroll
        for (int u = 0; u < 32; ++u) if (c * 32 + u >= p.d_eff) rr[u] = 0u;
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
int make_act_tmap(CUtensorMap* m, const void* base, int T, int HD, long ld) {
  return vlmt_make_tmap_2d_bf16(m, base, (uint64_t)HD, (uint64_t)T, (uint64_t)ld * 2, 64, 128);
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
  CUtensorMap tq, tk, tv, tdo;
  int r;
  if ((r = make_act_tmap(&tq, q, T, Hq * D, (long)Hq * D))) return 1000 + r;
  if ((r = make_act_tmap(&tk, k, T, Hkv * D, (long)Hkv * D))) return 2000 + r;
  if ((r = make_act_tmap(&tv, v, T, Hkv * D, (long)Hkv * D))) return 3000 + r;
  if ((r = make_act_tmap(&tdo, dout, T, Hq * D, (long)Hq * D))) return 4000 + r;
  BwdParams p;
  p.dQ = reinterpret_cast<__nv_bfloat16*>(dq); p.dK = reinterpret_cast<__nv_bfloat16*>(dk); p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.LSE = lse; p.delta = delta; p.cu = cu; p.n_docs = n_docs; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * kLog2e; p.causal = causal; p.status = status;
  p.d_eff = (d_eff <= 0 || d_eff > D) ? D : ((d_eff + 15) / 16) * 16;
  dim3 grid_kv(T / BN + n_docs + 1, Hkv), grid_q(T / BM + n_docs + 1, Hq);
  if (D == 128) {
    if ((r = set_smem(attn_bwd_dkdv_kernel<128>, BwdSmem<128>::kTotal))) return r;
    if ((r = set_smem(attn_bwd_dq_kernel<128>, BwdSmem<128>::kTotal))) return r;
    attn_bwd_dkdv_kernel<128><<<grid_kv, ATT_THREADS, BwdSmem<128>::kTotal, st>>>(tq, tk, tv, tdo, p);
    attn_bwd_dq_kernel<128><<<grid_q, ATT_THREADS, BwdSmem<128>::kTotal, st>>>(tq, tk, tv, tdo, p);
  } else if (D == 64) {
    if ((r = set_smem(attn_bwd_dkdv_kernel<64>, BwdSmem<64>::kTotal))) return r;
    if ((r = set_smem(attn_bwd_dq_kernel<64>, BwdSmem<64>::kTotal))) return r;
    attn_bwd_dkdv_kernel<64><<<grid_kv, ATT_THREADS, BwdSmem<64>::kTotal, st>>>(tq, tk, tv, tdo, p);
    attn_bwd_dq_kernel<64><<<grid_q, ATT_THREADS, BwdSmem<64>::kTotal, st>>>(tq, tk, tv, tdo, p);
  } else {
    return -10;
  }
  return (int)cudaGetLastError();
}
