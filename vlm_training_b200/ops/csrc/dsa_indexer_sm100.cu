// DSA lightning indexer: scores and per-query top-k selection as two kernels (sm_100a).
//
// score[t, s] = sum_h w[t, h] * relu(iq[t, h, :] . ik[s, :])   for the causal keys s <= t of t's document
// (reference: the indexer of the DSA variant, models/qwen3_5 of the reference tree; 4 heads of 64 channels here).
//
//   dsa_index_scores_kernel : one CTA per (128 queries, 128 keys) tile pair of a query block.  The four heads' products
//                             [128 x 64] . [64 x 128] run as tcgen05.mma into four 128-column TMEM accumulators; the
//                             row-owning threads fold them into one score with relu and the per-query head weights and
//                             write fp32 scores.  Tiles above the diagonal are not launched; entries above the diagonal
//                             inside a tile are written but never read (the selection kernel knows every row's length).
//   dsa_topk_kernel         : one CTA per query: its n = position + 1 scores sit in shared memory as order-preserving
//                             32-bit keys; three histogram passes (11 + 11 + 10 bits) find the k-th largest value, then an
//                             ordered compaction writes the indices above it and, in index order, as many equal ones as are
//                             still needed.  Rows with n <= k keep every key.  Deterministic; unused slots are -1.
#include "dsa_attention.h"
#include "gemm_sm100.h"
#include "sm100.cuh"

#include <cuda_bf16.h>

namespace {
using namespace sm100;

constexpr int HI = 4, DI = 64;

struct ScoreParams {
  const float* w;       // [T, HI] head weights of every query (global token index)
  float* scores;        // [B, ld] of the block
  int q_tok0;           // global token of the block's first query
  int k_tok0;           // global token of the document's first key
  int B, n_keys, ld;
  int q_pos0;           // position of the block's first query inside the document
  int* status;
};

__global__ void __launch_bounds__(128, 1)
dsa_index_scores_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, ScoreParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int kQ = 4 * 16384, kK = 16384;         // [128 x 256] and [128 x 64] bf16 tiles
  uint64_t* bar_tma = reinterpret_cast<uint64_t*>(smem + kQ + kK);
  uint64_t* bar_mma = bar_tma + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_tma + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int tq = blockIdx.x, tk = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // causal: the tile pair has work only if its first key is not after its last query
  if (tk * 128 > p.q_pos0 + tq * 128 + 127) return;
  constexpr int TMEM_COLS = 512;
  if (tid == 0) {
    mbar_init(bar_tma, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) tmem_alloc<TMEM_COLS>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  if (tid == 0) {
    mbar_expect_tx(bar_tma, kQ + kK);
#pragma unroll
    for (int h = 0; h < HI; ++h) tma_load_2d(smem + h * 16384, &tmQ, bar_tma, h * DI, p.q_tok0 + tq * 128);
    tma_load_2d(smem + kQ, &tmK, bar_tma, 0, p.k_tok0 + tk * 128);
  }
  bool ok = mbar_wait(bar_tma, 0, abort_flag, p.status, kErrTimeoutFull);
  ok = __syncthreads_and(ok);
  if (ok) {
    if (tid == 0) {
      tc_fence_after();
      constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, false);
      const SmemDesc b0 = make_desc(smem_u32(smem + kQ), 16, 1024);
#pragma unroll
      for (int h = 0; h < HI; ++h) {
        const SmemDesc a0 = make_desc(smem_u32(smem + h * 16384), 16, 1024);
#pragma unroll
        for (int kk = 0; kk < DI / 16; ++kk) {
          if (kk == 0) umma_ss<0>(tmem_base + h * 128, a0, b0, idesc);
          else umma_ss<1>(tmem_base + h * 128, desc_off(a0, kk * 32), desc_off(b0, kk * 32), idesc);
        }
      }
      umma_commit(bar_mma);
    }
    ok = mbar_wait(bar_mma, 0, abort_flag, p.status, kErrTimeoutTmemFull);
    ok = __syncthreads_and(ok);
    if (ok) {
      tc_fence_after();
      const int row = tq * 128 + tid;                    // query of the block owned by this thread
      const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
      float wh[HI];
#pragma unroll
      for (int h = 0; h < HI; ++h) wh[h] = row < p.B ? p.w[(size_t)(p.q_tok0 + row) * HI + h] : 0.f;
      float* dst = p.scores + (size_t)row * p.ld + tk * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
#pragma unroll
        for (int h = 0; h < HI; ++h) {
          uint32_t x[32];
          tmem_ld_32x32(tmem_base + lane_addr + h * 128 + c * 32, x);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) acc[i] = fmaf(wh[h], fmaxf(__uint_as_float(x[i]), 0.f), acc[i]);
        }
        if (row < p.B) {
          const int col0 = tk * 128 + c * 32;
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            if (col0 + i + 3 < p.n_keys) {
              *reinterpret_cast<float4*>(dst + c * 32 + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
            } else {
              for (int u = 0; u < 4; ++u) if (col0 + i + u < p.n_keys) dst[c * 32 + i + u] = acc[i + u];
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
  if (warp == 0) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// ------------------------------------------------------------------------------------------------ top-k
// order-preserving map float -> uint32 (larger float <-> larger key); NaN sorts above everything, as torch.topk does
__device__ __forceinline__ uint32_t fkey(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

constexpr int TOPK_THREADS = 256;

// For the digit `shift / bits` of the keys that match `prefix` under `mask`: the bin that holds the `want`-th largest of
// them, and how many matching keys lie in higher bins.  Every thread returns the same pair.
__device__ __forceinline__ void select_digit(const uint32_t* keys, int n, uint32_t prefix, uint32_t mask, int shift, int bits, int want,
                                             uint32_t* hist, int* bin_out, int* above_out, int* sh_res) {
  const int nb = 1 << bits;
  for (int i = threadIdx.x; i < nb; i += TOPK_THREADS) hist[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += TOPK_THREADS) {
    const uint32_t kx = keys[i];
    if ((kx & mask) == prefix) atomicAdd(&hist[(kx >> shift) & (nb - 1)], 1u);
  }
  __syncthreads();
  // suffix counts: thread t owns nb / 256 consecutive bins; walk from the top
  if (threadIdx.x < 32) {
    // one warp scans the bins from the highest down in chunks of 32
    int above = 0;
    int found_bin = -1, found_above = 0;
    for (int base = nb - 32; base >= 0 && found_bin < 0; base -= 32) {
      const int b = base + 31 - threadIdx.x;          // lane 0 takes the highest bin of the chunk
      const int c = (int)hist[b];
      int incl = c;                                   // inclusive prefix over lanes (higher bins first)
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if ((int)threadIdx.x >= o) incl += v;
      }
      const bool hit = above + incl >= want && above + incl - c < want;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (m) {
        const int src = __ffs(m) - 1;
        found_bin = __shfl_sync(0xffffffffu, b, src);
        found_above = __shfl_sync(0xffffffffu, above + incl - c, src);
      }
      above += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (threadIdx.x == 0) { sh_res[0] = found_bin; sh_res[1] = found_above; }
  }
  __syncthreads();
  *bin_out = sh_res[0];
  *above_out = sh_res[1];
  __syncthreads();
}

struct TopkParams {
  const float* scores;   // [B, ld]
  int* sel;              // [B, kk]
  int B, ld, kk, q_pos0;
};

__global__ void __launch_bounds__(TOPK_THREADS) dsa_topk_kernel(TopkParams p) {
  extern __shared__ uint32_t keys[];            // n keys, then the histogram (2048 bins) and scratch
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = p.q_pos0 + b + 1;               // causal keys of this query
  int* out = p.sel + (size_t)b * p.kk;
  if (n <= p.kk) {                              // every causal key is kept
    for (int j = tid; j < p.kk; j += TOPK_THREADS) out[j] = j < n ? j : -1;
    return;
  }
  uint32_t* hist = keys + ((n + 3) & ~3);
  int* sh_res = reinterpret_cast<int*>(hist + 2048);
  int* warp_cnt = sh_res + 4;                   // [2][8]
  const float* row = p.scores + (size_t)b * p.ld;
  for (int i = tid; i < n; i += TOPK_THREADS) keys[i] = fkey(row[i]);
  __syncthreads();
  int bin, above, want = p.kk;
  uint32_t prefix = 0, mask = 0;
  select_digit(keys, n, prefix, mask, 21, 11, want, hist, &bin, &above, sh_res);
  prefix |= (uint32_t)bin << 21; mask |= 0x7ffu << 21; want -= above;
  select_digit(keys, n, prefix, mask, 10, 11, want, hist, &bin, &above, sh_res);
  prefix |= (uint32_t)bin << 10; mask |= 0x7ffu << 10; want -= above;
  select_digit(keys, n, prefix, mask, 0, 10, want, hist, &bin, &above, sh_res);
  const uint32_t thr = prefix | (uint32_t)bin;  // key of the k-th largest score
  const int need_eq = want - above;             // how many keys equal to it are kept (the first ones in index order)
  // ordered compaction, 256 keys per round
  int base_gt = 0, base_eq = 0;                 // kept so far (same in every thread)
  for (int i0 = 0; i0 < n; i0 += TOPK_THREADS) {
    const int i = i0 + tid;
    const uint32_t kx = i < n ? keys[i] : 0u;
    const bool gt = i < n && kx > thr, eq = i < n && kx == thr;
    const unsigned mg = __ballot_sync(0xffffffffu, gt), me = __ballot_sync(0xffffffffu, eq);
    if (lane == 0) { warp_cnt[warp] = __popc(mg); warp_cnt[8 + warp] = __popc(me); }
    __syncthreads();
    int og = 0, oe = 0, tg = 0, te = 0;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const int cg = warp_cnt[w], ce = warp_cnt[8 + w];
      if (w < warp) { og += cg; oe += ce; }
      tg += cg; te += ce;
    }
    const int rank_g = base_gt + og + __popc(mg & ((1u << lane) - 1));
    const int rank_e = base_eq + oe + __popc(me & ((1u << lane) - 1));
    // slots: the keys above the threshold fill [0, kk - need_eq), the equal ones the tail
    if (gt) out[rank_g] = i;
    if (eq && rank_e < need_eq) out[p.kk - need_eq + rank_e] = i;
    base_gt += tg; base_eq += te;
    __syncthreads();
  }
}
}  // namespace

// scores of one query block: queries [q_tok0, q_tok0 + B) (global tokens) at document positions q_pos0.., keys
// [k_tok0, k_tok0 + n_keys); iq [T, 4 * 64] bf16, ik [T, 64] bf16, w [T, 4] fp32; scores fp32 [B, ld] (ld >= n_keys, multiple of 4)
extern "C" int vlmt_dsa_index_scores(const void* iq, const void* ik, const float* w, int T, int q_tok0, int q_pos0, int k_tok0, int B,
                                     int n_keys, float* scores, int ld, int* status, cudaStream_t st) {
  if (B <= 0 || n_keys <= 0) return 0;
  if (ld & 3) return -2;
  CUtensorMap tq, tk;
  int r;
  if ((r = vlmt_make_tmap_2d_bf16(&tq, iq, HI * DI, (uint64_t)T, HI * DI * 2, 64, 128))) return 1000 + r;
  if ((r = vlmt_make_tmap_2d_bf16(&tk, ik, DI, (uint64_t)T, DI * 2, 64, 128))) return 2000 + r;
  ScoreParams p;
  p.w = w; p.scores = scores; p.q_tok0 = q_tok0; p.k_tok0 = k_tok0; p.B = B; p.n_keys = n_keys; p.ld = ld; p.q_pos0 = q_pos0;
  p.status = status;
  const int smem = 4 * 16384 + 16384 + 64 + 1024;
  if (cudaFuncSetAttribute(dsa_index_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
  dim3 grid((B + 127) / 128, (n_keys + 127) / 128);
  dsa_index_scores_kernel<<<grid, 128, smem, st>>>(tq, tk, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

// sel [B, kk] int32: for query b (document position q_pos0 + b) the kk highest-scoring causal keys in index order
// (-1 in unused slots when the query has fewer than kk causal keys)
extern "C" int vlmt_dsa_topk(const float* scores, int B, int ld, int q_pos0, int kk, int* sel, cudaStream_t st) {
  if (B <= 0 || kk <= 0) return 0;
  TopkParams p;
  p.scores = scores; p.sel = sel; p.B = B; p.ld = ld; p.kk = kk; p.q_pos0 = q_pos0;
  const int n_max = q_pos0 + B;
  const int smem = (((n_max + 3) & ~3) + 2048 + 4 + 16) * 4;
  if (smem > 227 * 1024) return -3;
  if (cudaFuncSetAttribute(dsa_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -4;
  dsa_topk_kernel<<<B, TOPK_THREADS, smem, st>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -5;
}
