// Varlen flash attention for head size 256 (the gated full-attention layers of Qwen3.5) on tcgen05 / TMEM.
//
// Head size 256 does not fit the two-query-tile layout of attention_sm100.cu (two [128 x 256] query tiles, two score
// tiles and two output accumulators exceed both shared and tensor memory), so these kernels work on ONE 128-row tile per
// CTA against streamed 64-row tiles of the other side, with the score buffers double-buffered in tensor memory so that
// the tensor core computes the scores of tile j + 1 while the CUDA cores work on tile j:
//
//   forward   CTA = (128 queries, query head).  S(j) = Q K_j^T (N = 64), online softmax with lazy rescale of the
//             [128 x 256] fp32 output accumulator in TMEM, O += P(j) V_j with P read from TMEM.
//   dQ        CTA = (128 queries, query head).  S(j), dP(j) = dO V_j^T, dS = P (dP - delta), dQ += dS(j) K_j.
//   dK / dV   CTA = (128 keys, kv head), everything transposed (rows = keys), looping over 64-query tiles and the
//             query heads of the GQA group.  The two accumulators ([128 x 256] fp32 each) plus double-buffered scores
//             exceed the 512 TMEM columns, so dV and dK are two passes of one templated kernel; each recomputes S^T.
//
// Roles per CTA (192 threads): warp 0 issues TMA loads, one thread of warp 1 issues every MMA, warps 2..5 own one row
// of the 128-row tile per thread.  Every wait is bounded (sm100::mbar_wait).  No atomics: results are bit-reproducible.
#include "attention_sm100.h"
#include "sm100.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace {
using namespace sm100;

constexpr int HD = 256;            // head size
constexpr int BR = 128;            // rows of the stationary tile
constexpr int BC = 64;             // rows of a streamed tile
constexpr int THREADS = 192;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.f;
constexpr int kBigTile = BR * HD * 2;     // 65536: a [128 x 256] tile = 4 blocks of [128 rows x 64 channels]
constexpr int kSmallTile = BC * HD * 2;   // 32768: a [64 x 256] tile = 4 blocks of [64 rows x 64 channels]
constexpr int kBigBlock = BR * 128, kSmallBlock = BC * 128;   // bytes of one 64-channel block

struct TileInfo {
  int doc_start, doc_len, q0;
  bool valid;
};
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

template <int kSlack>
__device__ __forceinline__ uint8_t* align_smem(uint8_t* raw) {
  uint8_t* a = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
  return (a - raw) <= kSlack ? a : nullptr;
}

// k-step kk (16 channels) of a K-major [rows x 256] tile stored as 64-channel blocks of `block_bytes`
__device__ __forceinline__ uint32_t kmajor_off(int kk, int block_bytes) { return (kk >> 2) * block_bytes + (kk & 3) * 32; }

// D[128 x 64] = A[128 x 256] (K-major, big tile) x B[64 x 256]^T (K-major, small tile): 16 MMAs
__device__ __forceinline__ void issue_scores(uint32_t dst, SmemDesc a_big, SmemDesc b_small, uint32_t idesc) {
#pragma unroll
  for (int kk = 0; kk < HD / 16; ++kk) {
    const SmemDesc a = desc_off(a_big, kmajor_off(kk, kBigBlock)), b = desc_off(b_small, kmajor_off(kk, kSmallBlock));
    if (kk == 0) umma_ss<0>(dst, a, b, idesc); else umma_ss<1>(dst, a, b, idesc);
  }
}
// D[128 x 256] (+)= A[128 x 64] (packed bf16 in TMEM at a_tmem) x B[64 x 256] (small tile read MN-major): 4 MMAs
__device__ __forceinline__ void issue_accumulate(uint32_t dst, uint32_t a_tmem, SmemDesc b_mn, uint32_t idesc, uint32_t acc) {
#pragma unroll
  for (int kk = 0; kk < BC / 16; ++kk) {
    if (kk == 0) umma_ts<2>(dst, a_tmem, b_mn, idesc, acc); else umma_ts<1>(dst, a_tmem + kk * 8, desc_off(b_mn, kk * 2048), idesc);
  }
}

struct Params {
  __nv_bfloat16 *O, *dQ, *dK, *dV;
  float* LSE;            // [Hq, T], natural log (written by forward, read by backward)
  const float* delta;    // [Hq, T]
  const int* cu;
  int n_docs, T, Hq, Hkv;
  float scale, scale_log2;
  int causal;
  int* status;
};

__device__ __forceinline__ void load_big(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int col0, int row0) {
#pragma unroll
  for (int b = 0; b < HD / 64; ++b) tma_load_2d(dst + b * kBigBlock, m, bar, col0 + 64 * b, row0);
}
__device__ __forceinline__ void load_small(uint8_t* dst, const CUtensorMap* m, uint64_t* bar, int col0, int row0) {
#pragma unroll
  for (int b = 0; b < HD / 64; ++b) tma_load_2d(dst + b * kSmallBlock, m, bar, col0 + 64 * b, row0);
}

__device__ __forceinline__ void teardown(volatile int* abort_flag, int warp, uint32_t tmem_base) {
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {   // give copies that are still in flight time to land before the smem goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<512>(tmem_base);
  }
}

// ------------------------------------------------------------------------------------------------ forward
struct FwdSmem {
  static constexpr int offQ = 0;
  static constexpr int offK = kBigTile;                 // 2 stages
  static constexpr int offV = offK + 2 * kSmallTile;    // 2 stages
  static constexpr int offBar = offV + 2 * kSmallTile;  // 196608
  static constexpr int kSlack = 1024;
  static constexpr int kTotal = offBar + 256 + kSlack;
};

__global__ void __launch_bounds__(THREADS, 1)
attn256_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, Params p) {
  using L = FwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_smem<L::kSlack>(smem_raw);
  if (smem == nullptr) { if (threadIdx.x == 0) atomicCAS(p.status, 0, kErrTimeoutOther); return; }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* q_full = bars;        // 1
  uint64_t* k_full = bars + 1;    // 2
  uint64_t* k_empty = bars + 3;   // 2
  uint64_t* v_full = bars + 5;    // 2
  uint64_t* v_empty = bars + 7;   // 2
  uint64_t* s_full = bars + 9;    // 2: S(j) is in score buffer j & 1
  uint64_t* p_full = bars + 11;   // 2 (4 warps): P(j) is in score buffer j & 1
  uint64_t* pv_done = bars + 13;  // 1: O holds the contributions of tiles 0..j
  uint64_t* o_done = bars + 14;   // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, BR);
  if (!ti.valid) return;  // uniform for the whole CTA
  const int hq = blockIdx.y;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? min(ti.doc_len, ti.q0 + BR) : ti.doc_len;
  const int J = (kv_end + BC - 1) / BC;
  constexpr int S_COL = 0, O_COL = 128;   // score buffers at 0 and 64, output accumulator at 128..383

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 4);
    }
    mbar_init(pv_done, 1); mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
  }
  if (warp == 1) tmem_alloc<512>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(q_full, kBigTile);
      load_big(smem + L::offQ, &tmQ, q_full, hq * HD, ti.doc_start + ti.q0);
      for (int j = 0; j < J; ++j) {
        const int s = j & 1;
        const uint32_t ph = ((j >> 1) & 1) ^ 1;
        const int krow = ti.doc_start + j * BC;
        if (!mbar_wait(&k_empty[s], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&k_full[s], kSmallTile);
        load_small(smem + L::offK + s * kSmallTile, &tmK, &k_full[s], hkv * HD, krow);
        if (!mbar_wait(&v_empty[s], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&v_full[s], kSmallTile);
        load_small(smem + L::offV + s * kSmallTile, &tmV, &v_full[s], hkv * HD, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BR, BC, false, false);
      constexpr uint32_t idesc_pv = make_idesc_bf16(BR, HD, false, true);
      const SmemDesc dQ = make_desc(smem_u32(smem + L::offQ), 16, 1024);
      const SmemDesc dK0 = make_desc(smem_u32(smem + L::offK), 16, 1024);
      const SmemDesc dV0 = make_desc(smem_u32(smem + L::offV), kSmallBlock, 1024);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kErrTimeoutFull);
      auto issue_S = [&](int j) -> bool {
        const int b = j & 1;
        if (!mbar_wait(&k_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) return false;
        tc_fence_after();
        issue_scores(tmem_base + S_COL + b * BC, dQ, desc_off(dK0, b * kSmallTile), idesc_s);
        umma_commit(&s_full[b]);
        umma_commit(&k_empty[b]);
        return true;
      };
      if (ok && J > 0) ok = issue_S(0);
      for (int j = 0; j < J && ok; ++j) {
        const int b = j & 1;
        // S(j + 1) overwrites the buffer of P(j - 1), whose consumer P(j - 1) V was issued earlier by this thread
        if (j + 1 < J && !issue_S(j + 1)) { ok = false; break; }
        if (!mbar_wait(&v_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
        if (!mbar_wait(&p_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        issue_accumulate(tmem_base + O_COL, tmem_base + S_COL + b * BC, desc_off(dV0, b * kSmallTile), idesc_pv, (uint32_t)j);
        umma_commit(&v_empty[b]);
        umma_commit(pv_done);
      }
      if (ok) umma_commit(o_done);
    }
  } else {
    const int q = warp & 3;                // TMEM lane quarter this warp may access
    const int r = q * 32 + lane;           // query row of the tile owned by this thread
    const int qi = ti.q0 + r;              // query index local to the document
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t o_addr = tmem_base + O_COL + lane_addr;
    float m_used = 0.f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < J && ok; ++j) {
      const int b = j & 1;
      const uint32_t s_addr = tmem_base + S_COL + b * BC + lane_addr;
      if (!mbar_wait(&s_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      uint32_t s[BC];
      tmem_ld_32x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld_32x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld_wait();
      const int kv0 = j * BC;
      const bool need_mask = (kv0 + BC > ti.doc_len) || (p.causal && kv0 + BC - 1 > ti.q0);
      if (need_mask) {
        const int limit = (p.causal ? min(ti.doc_len - 1, qi) : ti.doc_len - 1) - kv0;  // last visible column of this tile
#pragma unroll
        for (int i = 0; i < BC; ++i) if (i > limit) s[i] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int i = 0; i < BC; i += 4) {
        mx0 = fmax3(mx0, __uint_as_float(s[i]), __uint_as_float(s[i + 1]));
        mx1 = fmax3(mx1, __uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
      }
      const float mx = fmaxf(mx0, mx1) * p.scale_log2;   // the scale is positive: it commutes with max
      if (j == 0) {
        m_used = (mx == -INFINITY) ? 0.f : mx;
      } else {
        const bool grow = mx > m_used + kRescaleThreshold;
        if (__any_sync(0xffffffffu, grow)) {
          // O must hold every earlier tile and the tensor core must not touch it: P(j - 1) V has completed, P(j) V is not
          // issued before this warp publishes P(j)
          if (!mbar_wait(pv_done, (j - 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
          tc_fence_after();
          const float alpha = grow ? ex2_approx(m_used - mx) : 1.f;
          if (grow) m_used = mx;
          l *= alpha;
#pragma unroll 1
          for (int c = 0; c < HD / 32; ++c) {
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
      for (int c = 0; c < BC / 32; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float e0 = ex2_approx(fmaf(__uint_as_float(s[c * 32 + 2 * i]), p.scale_log2, neg_m));
          const float e1 = ex2_approx(fmaf(__uint_as_float(s[c * 32 + 2 * i + 1]), p.scale_log2, neg_m));
          sum0 += e0;
          sum1 += e1;
          pk[i] = pack_bf16x2(e0, e1);
        }
        tmem_st_32x16(s_addr + c * 16, pk);   // P(j) over the first 32 columns of its score buffer
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
      l += sum0 + sum1;
    }
    if (ok && J > 0 && mbar_wait(o_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const size_t tok = (size_t)(ti.doc_start + qi);
      __nv_bfloat16* dst = p.O + (tok * p.Hq + hq) * HD;
#pragma unroll 1
      for (int c = 0; c < HD / 32; ++c) {
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
  teardown(abort_flag, warp, tmem_base);
}

// ------------------------------------------------------------------------------------------------ backward
// Shared memory of both backward kernels: two stationary [128 x 256] tiles, a two-stage ring of [64 x 256] tiles for the
// streamed operand that is needed until the end of a step, one buffer for the one that is free after the step's first half.
struct BwdSmem {
  static constexpr int offA = 0;                        // dq: Q_i      | dk/dv: K_j
  static constexpr int offB = kBigTile;                 // dq: dO_i     | dk/dv: V_j (dK pass only)
  static constexpr int offC = 2 * kBigTile;             // 2 stages: dq K_j | dk/dv Q_i
  static constexpr int offD = offC + 2 * kSmallTile;    // 1 stage:  dq V_j | dk/dv dO_i
  static constexpr int offStat = offD + kSmallTile;     // dk/dv: per compute warp -lse2[64], -delta[64]
  static constexpr int offBar = offStat + 4 * 128 * 4;
  static constexpr int kSlack = 512;
  static constexpr int kTotal = offBar + 256 + kSlack;  // 232192 <= 232448
};

// dQ: one CTA per 128-query tile and query head, streaming 64-key tiles.
// TMEM: S[2] at 0 / 64, dP[2] at 128 / 192, dQ at 256.  Tensor-core order: S(j+1), dP(j+1), dQ(j).
__global__ void __launch_bounds__(THREADS, 1)
attn256_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, Params p) {
  using L = BwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_smem<L::kSlack>(smem_raw);
  if (smem == nullptr) { if (threadIdx.x == 0) atomicCAS(p.status, 0, kErrTimeoutOther); return; }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* qdo_full = bars;       // 1
  uint64_t* acc_done = bars + 1;   // 1
  uint64_t* k_full = bars + 2;     // 2
  uint64_t* k_empty = bars + 4;    // 2
  uint64_t* v_full = bars + 6;     // 1
  uint64_t* v_empty = bars + 7;    // 1
  uint64_t* s_full = bars + 8;     // 2
  uint64_t* dp_full = bars + 10;   // 2
  uint64_t* ds_full = bars + 12;   // 2 (4 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, BR);
  if (!ti.valid) return;
  const int hq = blockIdx.y;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int kv_end = p.causal ? min(ti.doc_len, ti.q0 + BR) : ti.doc_len;
  const int J = (kv_end + BC - 1) / BC;
  constexpr int S_COL = 0, DP_COL = 128, DQ_COL = 256;

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1); mbar_init(acc_done, 1); mbar_init(v_full, 1); mbar_init(v_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&dp_full[i], 1);
      mbar_init(&ds_full[i], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc<512>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int qrow = ti.doc_start + ti.q0;
      mbar_expect_tx(qdo_full, 2 * kBigTile);
      load_big(smem + L::offA, &tmQ, qdo_full, hq * HD, qrow);
      load_big(smem + L::offB, &tmdO, qdo_full, hq * HD, qrow);
      for (int j = 0; j < J; ++j) {
        const int s = j & 1;
        const int krow = ti.doc_start + j * BC;
        if (!mbar_wait(&k_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&k_full[s], kSmallTile);
        load_small(smem + L::offC + s * kSmallTile, &tmK, &k_full[s], hkv * HD, krow);
        if (!mbar_wait(v_empty, (j & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(v_full, kSmallTile);
        load_small(smem + L::offD, &tmV, v_full, hkv * HD, krow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BR, BC, false, false);
      constexpr uint32_t idesc_g = make_idesc_bf16(BR, HD, false, true);
      const SmemDesc dQ = make_desc(smem_u32(smem + L::offA), 16, 1024), dO = make_desc(smem_u32(smem + L::offB), 16, 1024);
      const SmemDesc dKk = make_desc(smem_u32(smem + L::offC), 16, 1024);            // K tile, K-major view (scores)
      const SmemDesc dKm = make_desc(smem_u32(smem + L::offC), kSmallBlock, 1024);   // K tile, MN-major view (dQ += dS K)
      const SmemDesc dVk = make_desc(smem_u32(smem + L::offD), 16, 1024);
      bool ok = mbar_wait(qdo_full, 0, abort_flag, p.status, kErrTimeoutFull);
      auto issue_step = [&](int j) -> bool {   // S(j) and dP(j) into the buffers of parity j & 1
        const int b = j & 1;
        if (!mbar_wait(&k_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) return false;
        tc_fence_after();
        issue_scores(tmem_base + S_COL + b * BC, dQ, desc_off(dKk, b * kSmallTile), idesc_s);
        umma_commit(&s_full[b]);
        if (!mbar_wait(v_full, j & 1, abort_flag, p.status, kErrTimeoutFull)) return false;
        tc_fence_after();
        issue_scores(tmem_base + DP_COL + b * BC, dO, dVk, idesc_s);
        umma_commit(&dp_full[b]);
        umma_commit(v_empty);              // V_j was last read by dP(j)
        return true;
      };
      if (ok && J > 0) ok = issue_step(0);
      for (int j = 0; j < J && ok; ++j) {
        const int b = j & 1;
        // the buffers of parity (j + 1) & 1 held S(j - 1) (in registers of the compute warps since ds_full(j - 1)) and
        // dS(j - 1) (read by dQ(j - 1), issued earlier by this thread)
        if (j + 1 < J && !issue_step(j + 1)) { ok = false; break; }
        if (!mbar_wait(&ds_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        issue_accumulate(tmem_base + DQ_COL, tmem_base + DP_COL + b * BC, desc_off(dKm, b * kSmallTile), idesc_g, (uint32_t)j);
        umma_commit(&k_empty[b]);          // K_j was last read by dQ(j)
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int q = warp & 3;
    const int r = q * 32 + lane;
    const int qi = ti.q0 + r;
    const bool q_ok = qi < ti.doc_len;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const size_t sidx = (size_t)hq * p.T + ti.doc_start + (q_ok ? qi : 0);
    const float neg_lse2 = q_ok ? -p.LSE[sidx] * kLog2e : -INFINITY;   // rows beyond the document: P = 0
    const float neg_delta = q_ok ? -p.delta[sidx] : 0.f;
    bool ok = true;
    for (int j = 0; j < J && ok; ++j) {
      const int b = j & 1;
      const uint32_t s_addr = tmem_base + S_COL + b * BC + lane_addr, dp_addr = tmem_base + DP_COL + b * BC + lane_addr;
      if (!mbar_wait(&s_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      uint32_t s[BC];
      tmem_ld_32x32(s_addr, *reinterpret_cast<uint32_t(*)[32]>(&s[0]));
      tmem_ld_32x32(s_addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&s[32]));
      tmem_ld_wait();
      const int kv0 = j * BC;
      const int limit = (p.causal ? min(ti.doc_len - 1, qi) : ti.doc_len - 1) - kv0;   // last visible column
      float pr[BC];
#pragma unroll
      for (int i = 0; i < BC; ++i) {
        const float x = fmaf(__uint_as_float(s[i]), p.scale_log2, neg_lse2);
        pr[i] = i > limit ? 0.f : ex2_approx(x);
      }
      if (!mbar_wait(&dp_full[b], (j >> 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < BC / 32; ++c) {
        uint32_t dr[32];
        tmem_ld_32x32(dp_addr + c * 32, dr);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
          const float d0 = pr[c * 32 + 2 * u] * (__uint_as_float(dr[2 * u]) + neg_delta);
          const float d1 = pr[c * 32 + 2 * u + 1] * (__uint_as_float(dr[2 * u + 1]) + neg_delta);
          pk[u] = pack_bf16x2(d0, d1);
        }
        tmem_st_32x16(dp_addr + c * 16, pk);   // dS(j), packed, over the first 32 columns of the dP buffer
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[b]);
    }
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      if (J > 0) {
        __nv_bfloat16* dst = p.dQ + ((size_t)(ti.doc_start + qi) * p.Hq + hq) * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + DQ_COL + lane_addr + c * 32, o);
          tmem_ld_wait();
          if (q_ok) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 pk;
              pk.x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]) * p.scale, __uint_as_float(o[u * 8 + 1]) * p.scale);
              pk.y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]) * p.scale, __uint_as_float(o[u * 8 + 3]) * p.scale);
              pk.z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]) * p.scale, __uint_as_float(o[u * 8 + 5]) * p.scale);
              pk.w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]) * p.scale, __uint_as_float(o[u * 8 + 7]) * p.scale);
              *reinterpret_cast<uint4*>(dst + c * 32 + u * 8) = pk;
            }
          }
        }
      }
    }
  }
  teardown(abort_flag, warp, tmem_base);
}

// dK (DV = false) or dV (DV = true): one CTA per 128-key tile and kv head; rows = keys; loops over the 64-query tiles that
// see the key tile and over the query heads of the GQA group.
// TMEM: S^T[2] at 0 / 64, dP^T[2] at 128 / 192 (dK pass), accumulator at 256.
//   dV pass: S^T(it+1), dV(it) += P^T(it) dO_it         dK pass: S^T(it+1), dP^T(it+1), dK(it) += dS^T(it) Q_it
template <bool DV>
__global__ void __launch_bounds__(THREADS, 1)
attn256_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO, Params p) {
  using L = BwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = align_smem<L::kSlack>(smem_raw);
  if (smem == nullptr) { if (threadIdx.x == 0) atomicCAS(p.status, 0, kErrTimeoutOther); return; }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::offBar);
  uint64_t* kv_full = bars;        // 1
  uint64_t* acc_done = bars + 1;   // 1
  uint64_t* q_full = bars + 2;     // 2
  uint64_t* q_empty = bars + 4;    // 2
  uint64_t* do_full = bars + 6;    // 1
  uint64_t* do_empty = bars + 7;   // 1
  uint64_t* s_full = bars + 8;     // 2
  uint64_t* dp_full = bars + 10;   // 2
  uint64_t* a_full = bars + 12;    // 2 (4 warps): the A operand of the accumulation (P^T or dS^T) of parity it & 1 is in TMEM
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stat = reinterpret_cast<float*>(smem + L::offStat);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const TileInfo ti = find_tile(p.cu, p.n_docs, blockIdx.x, BR);
  if (!ti.valid) return;
  const int hkv = blockIdx.y;
  const int group = p.Hq / p.Hkv;
  const int k0 = ti.q0;   // first key row of the tile (local to the document)
  const int n_qtiles = (ti.doc_len + BC - 1) / BC;
  const int i_first = p.causal ? k0 / BC : 0;
  const int n_iter = (n_qtiles - i_first) * group;
  constexpr int S_COL = 0, DP_COL = 128, ACC_COL = 256;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(acc_done, 1); mbar_init(do_full, 1); mbar_init(do_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); mbar_init(&s_full[i], 1); mbar_init(&dp_full[i], 1);
      mbar_init(&a_full[i], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc<512>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      const int krow = ti.doc_start + k0;
      mbar_expect_tx(kv_full, DV ? kBigTile : 2 * kBigTile);
      load_big(smem + L::offA, &tmK, kv_full, hkv * HD, krow);
      if (!DV) load_big(smem + L::offB, &tmV, kv_full, hkv * HD, krow);
      for (int it = 0; it < n_iter; ++it) {
        const int s = it & 1;
        const int i = i_first + it / group, hq = hkv * group + it % group;
        const int qrow = ti.doc_start + i * BC;
        if (!mbar_wait(&q_empty[s], ((it >> 1) & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(&q_full[s], kSmallTile);
        load_small(smem + L::offC + s * kSmallTile, &tmQ, &q_full[s], hq * HD, qrow);
        if (!mbar_wait(do_empty, (it & 1) ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) break;
        mbar_expect_tx(do_full, kSmallTile);
        load_small(smem + L::offD, &tmdO, do_full, hq * HD, qrow);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(BR, BC, false, false);   // [128 keys] x [64 queries], contraction over channels
      constexpr uint32_t idesc_g = make_idesc_bf16(BR, HD, false, true);     // [128 keys] x [256], contraction over 64 queries
      const SmemDesc dK = make_desc(smem_u32(smem + L::offA), 16, 1024), dV = make_desc(smem_u32(smem + L::offB), 16, 1024);
      const SmemDesc dQk = make_desc(smem_u32(smem + L::offC), 16, 1024), dQm = make_desc(smem_u32(smem + L::offC), kSmallBlock, 1024);
      const SmemDesc dOk = make_desc(smem_u32(smem + L::offD), 16, 1024), dOm = make_desc(smem_u32(smem + L::offD), kSmallBlock, 1024);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.status, kErrTimeoutFull);
      auto issue_step = [&](int it) -> bool {   // S^T(it) (and dP^T(it)) into the buffers of parity it & 1
        const int b = it & 1;
        if (!mbar_wait(&q_full[b], (it >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) return false;
        tc_fence_after();
        issue_scores(tmem_base + S_COL + b * BC, dK, desc_off(dQk, b * kSmallTile), idesc_s);
        umma_commit(&s_full[b]);
        if (!DV) {
          if (!mbar_wait(do_full, it & 1, abort_flag, p.status, kErrTimeoutFull)) return false;
          tc_fence_after();
          issue_scores(tmem_base + DP_COL + b * BC, dV, dOk, idesc_s);
          umma_commit(&dp_full[b]);
          umma_commit(do_empty);           // dO_it was last read by dP^T(it)
        } else {
          umma_commit(&q_empty[b]);        // the dV pass needs Q_it only for the scores
        }
        return true;
      };
      if (ok && n_iter > 0) ok = issue_step(0);
      for (int it = 0; it < n_iter && ok; ++it) {
        const int b = it & 1;
        if (it + 1 < n_iter && !issue_step(it + 1)) { ok = false; break; }
        if (!mbar_wait(&a_full[b], (it >> 1) & 1, abort_flag, p.status, kErrTimeoutOther)) { ok = false; break; }
        tc_fence_after();
        if (DV) {
          if (!mbar_wait(do_full, it & 1, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          issue_accumulate(tmem_base + ACC_COL, tmem_base + S_COL + b * BC, dOm, idesc_g, (uint32_t)it);
          umma_commit(do_empty);           // dO_it was last read by dV(it)
        } else {
          issue_accumulate(tmem_base + ACC_COL, tmem_base + DP_COL + b * BC, desc_off(dQm, b * kSmallTile), idesc_g, (uint32_t)it);
          umma_commit(&q_empty[b]);        // Q_it was last read by dK(it)
        }
      }
      if (ok) umma_commit(acc_done);
    }
  } else {
    const int cw = warp - 2;
    const int q = warp & 3;
    const int r = q * 32 + lane;           // key row of the tile owned by this thread
    const int kvi = k0 + r;                // key index local to the document
    const bool key_ok = kvi < ti.doc_len;
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    float* wstat = stat + cw * 128;        // this warp's copy of the step's per-query statistics
    bool ok = true;
    for (int it = 0; it < n_iter && ok; ++it) {
      const int b = it & 1;
      const int i = i_first + it / group, hq = hkv * group + it % group;
      const int q0 = i * BC;               // first query (column) of the step, local to the document
      __syncwarp();                        // every lane is done with the previous step's statistics
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int qq = q0 + h * 32 + lane;
        const bool qok = qq < ti.doc_len;
        const size_t idx = (size_t)hq * p.T + ti.doc_start + (qok ? qq : 0);
        wstat[h * 32 + lane] = qok ? -p.LSE[idx] * kLog2e : -INFINITY;   // exp2(-inf) = 0 for queries beyond the document
        if (!DV) wstat[64 + h * 32 + lane] = qok ? -p.delta[idx] : 0.f;
      }
      __syncwarp();
      const uint32_t s_addr = tmem_base + S_COL + b * BC + lane_addr, dp_addr = tmem_base + DP_COL + b * BC + lane_addr;
      if (!mbar_wait(&s_full[b], (it >> 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      // column c (query q0 + c) is visible to this key iff the key exists and (causal) kvi <= q0 + c
      const int cmin = !key_ok ? (1 << 30) : (p.causal ? kvi - q0 : -(1 << 30));
      float pr[BC];
#pragma unroll
      for (int c = 0; c < BC / 32; ++c) {
        uint32_t sr[32];
        tmem_ld_32x32(s_addr + c * 32, sr);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 32; ++u) {
          const float x = fmaf(__uint_as_float(sr[u]), p.scale_log2, wstat[c * 32 + u]);
          pr[c * 32 + u] = (c * 32 + u < cmin) ? 0.f : ex2_approx(x);
        }
        if (DV) {
          uint32_t pk[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) pk[u] = pack_bf16x2(pr[c * 32 + 2 * u], pr[c * 32 + 2 * u + 1]);
          tmem_st_32x16(s_addr + c * 16, pk);   // P^T(it), packed, over the first 32 columns of the score buffer
        }
      }
      if (!DV) {
        if (!mbar_wait(&dp_full[b], (it >> 1) & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < BC / 32; ++c) {
          uint32_t dr[32];
          tmem_ld_32x32(dp_addr + c * 32, dr);
          tmem_ld_wait();
          uint32_t pk[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) {
            const float d0 = pr[c * 32 + 2 * u] * (__uint_as_float(dr[2 * u]) + wstat[64 + c * 32 + 2 * u]);
            const float d1 = pr[c * 32 + 2 * u + 1] * (__uint_as_float(dr[2 * u + 1]) + wstat[64 + c * 32 + 2 * u + 1]);
            pk[u] = pack_bf16x2(d0, d1);
          }
          tmem_st_32x16(dp_addr + c * 16, pk);  // dS^T(it), packed, over the first 32 columns of the dP^T buffer
        }
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[b]);
    }
    if (ok && mbar_wait(acc_done, 0, abort_flag, p.status, kErrTimeoutTmemFull)) {
      tc_fence_after();
      if (n_iter > 0) {
        __nv_bfloat16* base = DV ? p.dV : p.dK;
        const float f = DV ? 1.f : p.scale;
        __nv_bfloat16* dst = base + ((size_t)(ti.doc_start + kvi) * p.Hkv + hkv) * HD;
#pragma unroll 1
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(tmem_base + ACC_COL + lane_addr + c * 32, o);
          tmem_ld_wait();
          if (key_ok) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint4 pk;
              pk.x = pack_bf16x2(__uint_as_float(o[u * 8 + 0]) * f, __uint_as_float(o[u * 8 + 1]) * f);
              pk.y = pack_bf16x2(__uint_as_float(o[u * 8 + 2]) * f, __uint_as_float(o[u * 8 + 3]) * f);
              pk.z = pack_bf16x2(__uint_as_float(o[u * 8 + 4]) * f, __uint_as_float(o[u * 8 + 5]) * f);
              pk.w = pack_bf16x2(__uint_as_float(o[u * 8 + 6]) * f, __uint_as_float(o[u * 8 + 7]) * f);
              *reinterpret_cast<uint4*>(dst + c * 32 + u * 8) = pk;
            }
          }
        }
      }
    }
  }
  teardown(abort_flag, warp, tmem_base);
}

// delta[h, t] = sum_d dO[t,h,d] * O[t,h,d]
__global__ void attn256_delta_kernel(const __nv_bfloat16* __restrict__ dO, const __nv_bfloat16* __restrict__ O, float* __restrict__ delta,
                                     int T, int H) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T * H) return;
  const int t = warp / H, h = warp - t * H;
  const uint4 a = reinterpret_cast<const uint4*>(dO + ((size_t)t * H + h) * HD)[lane];
  const uint4 b = reinterpret_cast<const uint4*>(O + ((size_t)t * H + h) * HD)[lane];
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
    acc += fa.x * fb.x + fa.y * fb.y;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) delta[(size_t)h * T + t] = acc;
}

int make_map(CUtensorMap* m, const void* base, int T, int cols, long ld, int box_rows) {
  return vlmt_make_tmap_2d_bf16(m, base, (uint64_t)cols, (uint64_t)T, (uint64_t)ld * 2, 64, (uint32_t)box_rows);
}
template <typename K>
int set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}
}  // namespace

extern "C" int vlmt_attn256_fwd(const void* q, const void* k, const void* v, void* o, float* lse, const int* cu, int n_docs, int T, int Hq,
                                int Hkv, long ldq, long ldk, long ldv, float scale, int causal, int* status, cudaStream_t st) {
  if (T <= 0 || n_docs <= 0) return 0;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = make_map(&tq, q, T, Hq * HD, ldq, BR))) return 1000 + r;
  if ((r = make_map(&tk, k, T, Hkv * HD, ldk, BC))) return 2000 + r;
  if ((r = make_map(&tv, v, T, Hkv * HD, ldv, BC))) return 3000 + r;
  Params p{};
  p.O = reinterpret_cast<__nv_bfloat16*>(o); p.LSE = lse; p.cu = cu; p.n_docs = n_docs; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * kLog2e; p.causal = causal; p.status = status;
  if ((r = set_smem(attn256_fwd_kernel, FwdSmem::kTotal))) return r;
  dim3 grid(T / BR + n_docs + 1, Hq);
  attn256_fwd_kernel<<<grid, THREADS, FwdSmem::kTotal, st>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

extern "C" int vlmt_attn256_bwd(const void* dout, const void* q, const void* k, const void* v, const void* o, const float* lse, float* delta,
                                void* dq, void* dk, void* dv, const int* cu, int n_docs, int T, int Hq, int Hkv, float scale, int causal,
                                int* status, cudaStream_t st) {
  if (T <= 0 || n_docs <= 0) return 0;
  attn256_delta_kernel<<<(T * Hq * 32 + 255) / 256, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(dout),
                                                                  reinterpret_cast<const __nv_bfloat16*>(o), delta, T, Hq);
  CUtensorMap q_big, q_small, k_big, k_small, v_big, v_small, do_big, do_small;
  int r;
  const long ldq = (long)Hq * HD, ldk = (long)Hkv * HD;
  if ((r = make_map(&q_big, q, T, Hq * HD, ldq, BR)) || (r = make_map(&q_small, q, T, Hq * HD, ldq, BC))) return 1000 + r;
  if ((r = make_map(&k_big, k, T, Hkv * HD, ldk, BR)) || (r = make_map(&k_small, k, T, Hkv * HD, ldk, BC))) return 2000 + r;
  if ((r = make_map(&v_big, v, T, Hkv * HD, ldk, BR)) || (r = make_map(&v_small, v, T, Hkv * HD, ldk, BC))) return 3000 + r;
  if ((r = make_map(&do_big, dout, T, Hq * HD, ldq, BR)) || (r = make_map(&do_small, dout, T, Hq * HD, ldq, BC))) return 4000 + r;
  Params p{};
  p.dQ = reinterpret_cast<__nv_bfloat16*>(dq); p.dK = reinterpret_cast<__nv_bfloat16*>(dk); p.dV = reinterpret_cast<__nv_bfloat16*>(dv);
  p.LSE = const_cast<float*>(lse); p.delta = delta; p.cu = cu; p.n_docs = n_docs; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.scale = scale; p.scale_log2 = scale * kLog2e; p.causal = causal; p.status = status;
  if ((r = set_smem(attn256_bwd_dq_kernel, BwdSmem::kTotal))) return r;
  if ((r = set_smem(attn256_bwd_dkv_kernel<true>, BwdSmem::kTotal))) return r;
  if ((r = set_smem(attn256_bwd_dkv_kernel<false>, BwdSmem::kTotal))) return r;
  dim3 grid_kv(T / BR + n_docs + 1, Hkv), grid_q(T / BR + n_docs + 1, Hq);
  attn256_bwd_dkv_kernel<true><<<grid_kv, THREADS, BwdSmem::kTotal, st>>>(q_small, k_big, v_big, do_small, p);
  attn256_bwd_dkv_kernel<false><<<grid_kv, THREADS, BwdSmem::kTotal, st>>>(q_small, k_big, v_big, do_small, p);
  attn256_bwd_dq_kernel<<<grid_q, THREADS, BwdSmem::kTotal, st>>>(q_big, k_small, v_small, do_big, p);
  return (int)cudaGetLastError();
}
