// Everything of the gated delta rule that happens INSIDE a 64-token chunk, as tcgen05 kernels (sm_100a).
//
// The chunk form of the rule (reference: models/qwen3_5/model.py:180-186 calls fla's chunk_gated_delta_rule, whose
// kernels are chunk_scaled_dot_kkt + solve_tril, recompute_w_u, chunk_fwd_o and their backward counterparts) splits into
//   prepare : per chunk, from q, k, v, g, beta:  the decay matrix, A = strict_lower(beta k k^T decay), T = (I + A)^-1,
//             w = T (beta e^gc k), u = T (beta v), P = lower(q k^T decay), and the scan operands k e^(g_last - gc), q e^gc
//   scan    : the only sequential part (gdn_scan_sm100.cu): v_new = u - w S, S' = S e^g_last + kdec^T v_new
//   output  : o = (q e^gc) S^T + P v_new
// and the same three stages backwards.  This file holds prepare and output, forward and backward: four kernels, one CTA
// per (chunk, head), 128 threads.
//
// All matrix products run on the tensor cores as M = 128 tcgen05.mma with the chunk's 64 rows in TMEM lanes 0-63 (the A
// operand's rows 64-127 are whatever follows the tile in shared memory and land in lanes that nobody reads); operands
// are bf16 tiles in the 128-byte-swizzle layout that TMA writes, accumulators fp32 in TMEM.  Between two products the
// row-owning threads (warps 0 and 1: TMEM lane = chunk row) read the accumulator, apply the element-wise part (decay
// factors, masks, row scalings) and write the next operand tile back to shared memory.  The 64 x 64 triangular inverse
// is a forward substitution in fp32 registers, one thread per column.
//
// Every wait is bounded; a wait that runs out sets the status word and the CTA leaves through the common teardown.
#include "gdn_chunk_sm100.h"
#include "gemm_sm100.h"
#include "sm100.cuh"

#include <cuda_bf16.h>

namespace {
using namespace sm100;

constexpr int C = 64, D = 128;
constexpr int kBlk = C * 128;          // one swizzled block of a 64-row tile: 64 rows x 64 bf16 columns
constexpr int kT = 2 * kBlk;           // [64 x 128] tile
constexpr int kSq = kBlk;              // [64 x 64] tile
constexpr int kSBlk = D * 128;         // one block of a 128-row tile
constexpr int kS = 2 * kSBlk;          // [128 x 128] tile
constexpr int THREADS = 128;
constexpr int ASTRIDE = 68;            // floats per row of the fp32 copy of A (16-byte aligned rows, fewer bank conflicts)

// byte offset of the 16-byte group `c16` (8 bf16 columns) of row r inside one swizzled 64-column block
__device__ __forceinline__ uint32_t swz(int r, int c16) { return (uint32_t)(r * 128 + ((c16 ^ (r & 7)) << 4)); }
// 8 consecutive bf16 columns [8 col8, 8 col8 + 8) of row r of a tile whose 64-column blocks are `blk` bytes apart
__device__ __forceinline__ uint4* row8(uint8_t* tile, int blk, int r, int col8) {
  return reinterpret_cast<uint4*>(tile + (col8 >> 3) * blk + swz(r, col8 & 7));
}
__device__ __forceinline__ float lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  f[0] = lo(v.x); f[1] = hi(v.x); f[2] = lo(v.y); f[3] = hi(v.y); f[4] = lo(v.z); f[5] = hi(v.z); f[6] = lo(v.w); f[7] = hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}
__device__ __forceinline__ void store_bf16(uint8_t* tile, int blk, int r, int c, float v) {
  *reinterpret_cast<__nv_bfloat16*>(tile + (c >> 6) * blk + swz(r, (c & 63) >> 3) + (c & 7) * 2) = __float2bfloat16(v);
}

// D[tmem] (+)= A x B with M = 128, N = n, K = 16 * ksteps.
//   K-major operand : tile of rows x 64-column blocks, `blk` bytes between blocks.
//   MN-major operand: the same tile read with its rows as the contraction index; `blk` = distance between 64-element groups
//                     along M / N.
template <bool A_MN, bool B_MN>
__device__ __forceinline__ void issue(uint32_t d, const uint8_t* a, uint32_t a_blk, const uint8_t* b, uint32_t b_blk, int n, int ksteps,
                                      bool accumulate) {
  const SmemDesc da = A_MN ? make_desc(smem_u32(a), a_blk, 1024) : make_desc(smem_u32(a), 16, 1024);
  const SmemDesc db = B_MN ? make_desc(smem_u32(b), b_blk, 1024) : make_desc(smem_u32(b), 16, 1024);
  const uint32_t idesc = make_idesc_bf16(128, n, A_MN, B_MN);
  for (int kk = 0; kk < ksteps; ++kk) {
    const uint32_t oa = A_MN ? kk * 2048 : (kk >> 2) * a_blk + (kk & 3) * 32;
    const uint32_t ob = B_MN ? kk * 2048 : (kk >> 2) * b_blk + (kk & 3) * 32;
    umma_ss<2>(d, desc_off(da, oa), desc_off(db, ob), idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

struct Ctl {
  uint64_t* bar_tma;
  uint64_t* bar_mma;
  uint32_t* tmem_slot;
  volatile int* abort_flag;
  uint32_t mma_phase;
};

template <int TMEM_COLS>
__device__ __forceinline__ uint32_t cta_setup(Ctl& c, uint8_t* ctl_mem) {
  c.bar_tma = reinterpret_cast<uint64_t*>(ctl_mem);
  c.bar_mma = c.bar_tma + 1;
  c.tmem_slot = reinterpret_cast<uint32_t*>(c.bar_tma + 2);
  c.abort_flag = reinterpret_cast<volatile int*>(c.tmem_slot + 1);
  c.mma_phase = 0;
  if (threadIdx.x == 0) {
    mbar_init(c.bar_tma, 1);
    mbar_init(c.bar_mma, 1);
    *c.abort_flag = 0;
    fence_mbar_init();
  }
  if ((threadIdx.x >> 5) == 0) tmem_alloc<TMEM_COLS>(c.tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  return *c.tmem_slot;
}

template <int TMEM_COLS>
__device__ __forceinline__ void cta_teardown(Ctl& c, uint32_t tmem_base) {
  tc_fence_before();
  __syncthreads();
  if (*c.abort_flag) {  // let copies in flight land before the shared memory goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if ((threadIdx.x >> 5) == 0) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// thread 0 has issued MMAs: commit them and have every thread wait for their completion (CTA-uniform result)
__device__ __forceinline__ bool mma_done(Ctl& c, int* status) {
  if (threadIdx.x == 0) umma_commit(c.bar_mma);
  const bool ok = mbar_wait(c.bar_mma, c.mma_phase, c.abort_flag, status, kErrTimeoutTmemFull);
  c.mma_phase ^= 1;
  tc_fence_after();
  return __syncthreads_and(ok);
}
// writes to shared memory by ordinary stores become visible to the tensor core / TMA; TMEM reads are finished
__device__ __forceinline__ void publish() {
  tmem_ld_wait();
  fence_async_proxy();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

__device__ __forceinline__ void ld64(uint32_t taddr, uint32_t (&x)[64]) {
  tmem_ld_32x32(taddr, *reinterpret_cast<uint32_t(*)[32]>(&x[0]));
  tmem_ld_32x32(taddr + 32, *reinterpret_cast<uint32_t(*)[32]>(&x[32]));
  tmem_ld_wait();
}

// ============================================================================================ prepare, forward
struct PrepParams {
  const float* g;        // [T, H]
  const float* beta;     // [T, H]
  const int2* chunks;    // [N]: first token of the chunk, rows (1..64)
  __nv_bfloat16 *w, *u, *kdec, *qg;   // [H, N, 64, 128]
  __nv_bfloat16 *P, *Tm;              // [H, N, 64, 64]
  float* gc;                          // [H, N, 64]
  float* decay;                       // [H, N]
  float scale, eps;
  int H, N;
  int* status;
};

struct PrepSmem {
  static constexpr int offK = 0, offQ = offK + kT, offTm = offQ + kT, offKbg = offTm + kSq, offV = offKbg + kT;
  static constexpr int offA = offV + kT;                       // fp32 A, [64][ASTRIDE]
  static constexpr int offF = offA + C * ASTRIDE * 4;          // sg, sb, sgc [64] each; part [2][2][64]
  static constexpr int offCtl = offF + (3 * 64 + 4 * 64) * 4;
  static constexpr int kTotal = offCtl + 64 + 1024;
};

__global__ void __launch_bounds__(THREADS, 2)
gdn_prepare_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, PrepParams p) {
  using L = PrepSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sg = reinterpret_cast<float*>(smem + L::offF);
  float* sb = sg + 64;
  float* sgc = sb + 64;
  float* part = sgc + 64;
  float* As = reinterpret_cast<float*>(smem + L::offA);
  Ctl ctl;
  constexpr int TMEM_COLS = 256;
  const uint32_t tmem_base = cta_setup<TMEM_COLS>(ctl, smem + L::offCtl);

  const int n = blockIdx.x, h = blockIdx.y;
  const int2 ch = p.chunks[n];
  const int tok0 = ch.x, len = ch.y;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int r = t & 63, cb = t >> 6;
  const bool valid = r < len;
  const size_t tile = (size_t)h * p.N + n;

  if (t == 0) {
    mbar_expect_tx(ctl.bar_tma, 3 * kT);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(smem + L::offK + b * kBlk, &tmK, ctl.bar_tma, h * D + 64 * b, tok0);
      tma_load_2d(smem + L::offQ + b * kBlk, &tmQ, ctl.bar_tma, h * D + 64 * b, tok0);
      tma_load_2d(smem + L::offV + b * kBlk, &tmV, ctl.bar_tma, h * D + 64 * b, tok0);
    }
  }
  if (cb == 0) {
    sg[r] = valid ? p.g[(size_t)(tok0 + r) * p.H + h] : 0.f;
    sb[r] = valid ? p.beta[(size_t)(tok0 + r) * p.H + h] : 0.f;
  }
  bool ok = mbar_wait(ctl.bar_tma, 0, ctl.abort_flag, p.status, kErrTimeoutFull);
  ok = __syncthreads_and(ok);
  if (ok) {
    // ---- phase 1: row statistics and the operand tiles
    uint4 kr[8], qr[8];
    float ssk = 0.f, ssq = 0.f;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      kr[c] = *row8(smem + L::offK, kBlk, r, cb * 8 + c);
      qr[c] = *row8(smem + L::offQ, kBlk, r, cb * 8 + c);
      float f[8];
      unpack8(kr[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ssk = fmaf(f[i], f[i], ssk);
      unpack8(qr[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ssq = fmaf(f[i], f[i], ssq);
    }
    part[cb * 64 + r] = ssk;
    part[128 + cb * 64 + r] = ssq;
    float gcr = 0.f, last = 0.f;
    for (int j = 0; j < 64; ++j) {
      const float gj = sg[j];
      last += gj;
      if (j <= r) gcr += gj;
    }
    __syncthreads();
    const float rk = valid ? rsqrtf(part[r] + part[64 + r] + p.eps) : 0.f;
    const float rq = valid ? rsqrtf(part[128 + r] + part[192 + r] + p.eps) * p.scale : 0.f;
    const float E = __expf(gcr), F = __expf(last - gcr), b = sb[r];
    if (cb == 0) {
      sgc[r] = gcr;
      p.gc[tile * 64 + r] = gcr;
    }
    if (t == 0) p.decay[tile] = __expf(last);
    __nv_bfloat16* kdec_row = p.kdec + (tile * 64 + r) * D + cb * 64;
    __nv_bfloat16* qg_row = p.qg + (tile * 64 + r) * D + cb * 64;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      float f[8], o1[8], o2[8];
      unpack8(kr[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) { f[i] *= rk; o1[i] = f[i] * (b * E); o2[i] = f[i] * F; }
      *row8(smem + L::offK, kBlk, r, cb * 8 + c) = pack8(f);
      *row8(smem + L::offKbg, kBlk, r, cb * 8 + c) = pack8(o1);
      reinterpret_cast<uint4*>(kdec_row)[c] = pack8(o2);
      unpack8(qr[c], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) { f[i] *= rq; o1[i] = f[i] * E; }
      *row8(smem + L::offQ, kBlk, r, cb * 8 + c) = pack8(f);
      reinterpret_cast<uint4*>(qg_row)[c] = pack8(o1);
      const uint4 vr = *row8(smem + L::offV, kBlk, r, cb * 8 + c);
      unpack8(vr, f);
      const float bv = valid ? b : 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = valid ? f[i] * bv : 0.f;
      *row8(smem + L::offV, kBlk, r, cb * 8 + c) = pack8(f);
    }
    publish();
    // ---- phase 2: k k^T and q k^T
    if (t == 0) {
      issue<false, false>(tmem_base + 0, smem + L::offK, kBlk, smem + L::offK, kBlk, 64, 8, false);
      issue<false, false>(tmem_base + 64, smem + L::offQ, kBlk, smem + L::offK, kBlk, 64, 8, false);
    }
    ok = mma_done(ctl, p.status);
    if (ok) {
      // ---- phase 3: A (fp32, for the substitution) and P (bf16, to global memory)
      if (t < 64) {
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        uint32_t x[64];
        ld64(tmem_base + lane_addr, x);
        float* arow = As + r * ASTRIDE;
#pragma unroll
        for (int j = 0; j < 64; j += 4) {
          float4 a4;
          a4.x = (j + 0 < r) ? b * __uint_as_float(x[j + 0]) * __expf(gcr - sgc[j + 0]) : 0.f;
          a4.y = (j + 1 < r) ? b * __uint_as_float(x[j + 1]) * __expf(gcr - sgc[j + 1]) : 0.f;
          a4.z = (j + 2 < r) ? b * __uint_as_float(x[j + 2]) * __expf(gcr - sgc[j + 2]) : 0.f;
          a4.w = (j + 3 < r) ? b * __uint_as_float(x[j + 3]) * __expf(gcr - sgc[j + 3]) : 0.f;
          *reinterpret_cast<float4*>(arow + j) = a4;
        }
        ld64(tmem_base + lane_addr + 64, x);
        __nv_bfloat16* prow = p.P + (tile * 64 + r) * 64;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int j = c * 8 + i;
            f[i] = (j <= r) ? __uint_as_float(x[j]) * __expf(gcr - sgc[j]) : 0.f;
          }
          reinterpret_cast<uint4*>(prow)[c] = pack8(f);
        }
      }
      tc_fence_before();
      __syncthreads();
      // ---- phase 4: T = (I + A)^-1, thread j solves column j by forward substitution
      if (t < 64) {
        float col[64];
#pragma unroll
        for (int i = 0; i < 64; ++i) col[i] = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          float acc = (i == t) ? 1.f : 0.f;
          const float4* arow = reinterpret_cast<const float4*>(As + i * ASTRIDE);
#pragma unroll
          for (int m4 = 0; m4 < (i + 3) / 4; ++m4) {   // A[i][m] = 0 for m >= i, col[m] = 0 until it is computed
            const float4 a = arow[m4];
            acc = fmaf(-a.x, col[4 * m4 + 0], acc);
            acc = fmaf(-a.y, col[4 * m4 + 1], acc);
            acc = fmaf(-a.z, col[4 * m4 + 2], acc);
            acc = fmaf(-a.w, col[4 * m4 + 3], acc);
          }
          col[i] = acc;
        }
        __nv_bfloat16* tg = p.Tm + tile * 64 * 64 + t;
#pragma unroll
        for (int i = 0; i < 64; ++i) {
          store_bf16(smem + L::offTm, kBlk, i, t, col[i]);
          tg[i * 64] = __float2bfloat16(col[i]);
        }
      }
      publish();
      // ---- phase 5: w = T (beta e^gc k), u = T (beta v)
      if (t == 0) {
        issue<false, true>(tmem_base + 0, smem + L::offTm, kBlk, smem + L::offKbg, kBlk, 128, 4, false);
        issue<false, true>(tmem_base + 128, smem + L::offTm, kBlk, smem + L::offV, kBlk, 128, 4, false);
      }
      ok = mma_done(ctl, p.status);
      if (ok && t < 64) {
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
#pragma unroll 1
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* dst = (which == 0 ? p.w : p.u) + (tile * 64 + r) * D;
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t x[64];
            ld64(tmem_base + lane_addr + which * 128 + c2 * 64, x);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(x[c * 8 + i]);
              reinterpret_cast<uint4*>(dst + c2 * 64)[c] = pack8(f);
            }
          }
        }
      }
    }
  }
  (void)lane;
  cta_teardown<TMEM_COLS>(ctl, tmem_base);
}

// ============================================================================================ output, forward
struct OutParams {
  const int2* chunks;
  __nv_bfloat16* o;       // [T, H, 128]
  int H, N;
  int* status;
};
struct OutSmem {
  static constexpr int offQg = 0, offP = offQg + kT, offS = offP + kSq, offVn = offS + kS;
  static constexpr int offCtl = offVn + kT;
  static constexpr int kTotal = offCtl + 64 + 1024;
};

// o = qg S^T + P v_new for one chunk; rows beyond the chunk's length are not written
__global__ void __launch_bounds__(THREADS, 2)
gdn_output_fwd_kernel(const __grid_constant__ CUtensorMap tmQg, const __grid_constant__ CUtensorMap tmP,
                      const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmVn, OutParams p) {
  using L = OutSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctl ctl;
  constexpr int TMEM_COLS = 128;
  const uint32_t tmem_base = cta_setup<TMEM_COLS>(ctl, smem + L::offCtl);
  const int n = blockIdx.x, h = blockIdx.y;
  const int2 ch = p.chunks[n];
  const int t = threadIdx.x, warp = t >> 5;
  const int tile = h * p.N + n;
  if (t == 0) {
    mbar_expect_tx(ctl.bar_tma, 2 * kT + kSq + kS);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(smem + L::offQg + b * kBlk, &tmQg, ctl.bar_tma, 64 * b, tile * 64);
      tma_load_2d(smem + L::offVn + b * kBlk, &tmVn, ctl.bar_tma, 64 * b, tile * 64);
      tma_load_2d(smem + L::offS + b * kSBlk, &tmS, ctl.bar_tma, 64 * b, tile * 128);
    }
    tma_load_2d(smem + L::offP, &tmP, ctl.bar_tma, 0, tile * 64);
  }
  bool ok = mbar_wait(ctl.bar_tma, 0, ctl.abort_flag, p.status, kErrTimeoutFull);
  ok = __syncthreads_and(ok);
  if (ok) {
    if (t == 0) {
      tc_fence_after();
      issue<false, false>(tmem_base, smem + L::offQg, kBlk, smem + L::offS, kSBlk, 128, 8, false);
      issue<false, true>(tmem_base, smem + L::offP, kBlk, smem + L::offVn, kBlk, 128, 4, true);
    }
    ok = mma_done(ctl, p.status);
    if (ok && t < 64) {
      const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
      __nv_bfloat16* dst = p.o + ((size_t)(ch.x + t) * p.H + h) * D;
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t x[64];
        ld64(tmem_base + lane_addr + c2 * 64, x);
        if (t < ch.y) {
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(x[c * 8 + i]);
            reinterpret_cast<uint4*>(dst + c2 * 64)[c] = pack8(f);
          }
        }
      }
    }
  }
  cta_teardown<TMEM_COLS>(ctl, tmem_base);
}

// ============================================================================================ output, backward
struct OutBwdParams {
  const int2* chunks;
  __nv_bfloat16 *dqg, *dvn;   // [H, N, 64, 128]
  __nv_bfloat16* dP;          // [H, N, 64, 64]
  __nv_bfloat16* dS;          // [H, N, 128, 128]
  int H, N;
  int* status;
};
struct OutBwdSmem {
  static constexpr int offDo = 0, offP = offDo + kT, offS = offP + kSq, offVn = offS + kS, offQg = offVn + kT;
  static constexpr int offCtl = offQg + kT;
  static constexpr int kTotal = offCtl + 64 + 1024;
};

// From do (token layout): dqg = do S, dP = lower(do v_new^T), dv_new = P^T do, dS = do^T qg
__global__ void __launch_bounds__(THREADS, 2)
gdn_output_bwd_kernel(const __grid_constant__ CUtensorMap tmDo, const __grid_constant__ CUtensorMap tmQg,
                      const __grid_constant__ CUtensorMap tmP, const __grid_constant__ CUtensorMap tmS,
                      const __grid_constant__ CUtensorMap tmVn, OutBwdParams p) {
  using L = OutBwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Ctl ctl;
  constexpr int TMEM_COLS = 256;
  const uint32_t tmem_base = cta_setup<TMEM_COLS>(ctl, smem + L::offCtl);
  const int n = blockIdx.x, h = blockIdx.y;
  const int2 ch = p.chunks[n];
  const int t = threadIdx.x, warp = t >> 5;
  const int r = t & 63, cb = t >> 6;
  const int tile = h * p.N + n;
  if (t == 0) {
    mbar_expect_tx(ctl.bar_tma, 3 * kT + kSq + kS);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(smem + L::offDo + b * kBlk, &tmDo, ctl.bar_tma, h * D + 64 * b, ch.x);
      tma_load_2d(smem + L::offQg + b * kBlk, &tmQg, ctl.bar_tma, 64 * b, tile * 64);
      tma_load_2d(smem + L::offVn + b * kBlk, &tmVn, ctl.bar_tma, 64 * b, tile * 64);
      tma_load_2d(smem + L::offS + b * kSBlk, &tmS, ctl.bar_tma, 64 * b, tile * 128);
    }
    tma_load_2d(smem + L::offP, &tmP, ctl.bar_tma, 0, tile * 64);
  }
  bool ok = mbar_wait(ctl.bar_tma, 0, ctl.abort_flag, p.status, kErrTimeoutFull);
  ok = __syncthreads_and(ok);
  if (ok) {
    if (r >= ch.y) {  // rows of the box beyond the chunk belong to the next document
      const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int c = 0; c < 8; ++c) *row8(smem + L::offDo, kBlk, r, cb * 8 + c) = z;
    }
    publish();
    if (t == 0) {
      issue<false, true>(tmem_base + 0, smem + L::offDo, kBlk, smem + L::offS, kSBlk, 128, 8, false);      // do S
      issue<false, false>(tmem_base + 128, smem + L::offDo, kBlk, smem + L::offVn, kBlk, 64, 8, false);    // do v_new^T
    }
    ok = mma_done(ctl, p.status);
    if (ok) {
      if (t < 64) {
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        __nv_bfloat16* dst = p.dqg + ((size_t)tile * 64 + t) * D;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t x[64];
          ld64(tmem_base + lane_addr + c2 * 64, x);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(x[c * 8 + i]);
            reinterpret_cast<uint4*>(dst + c2 * 64)[c] = pack8(f);
          }
        }
        uint32_t x[64];
        ld64(tmem_base + lane_addr + 128, x);
        __nv_bfloat16* prow = p.dP + ((size_t)tile * 64 + t) * 64;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = (c * 8 + i <= t) ? __uint_as_float(x[c * 8 + i]) : 0.f;
          reinterpret_cast<uint4*>(prow)[c] = pack8(f);
        }
      }
      tmem_ld_wait();
      tc_fence_before();
      __syncthreads();
      if (t == 0) {
        tc_fence_after();
        issue<true, true>(tmem_base + 0, smem + L::offP, kBlk, smem + L::offDo, kBlk, 128, 4, false);       // P^T do
        issue<true, true>(tmem_base + 128, smem + L::offDo, kBlk, smem + L::offQg, kBlk, 128, 4, false);    // do^T qg
      }
      ok = mma_done(ctl, p.status);
      if (ok) {
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        if (t < 64) {
          __nv_bfloat16* dst = p.dvn + ((size_t)tile * 64 + t) * D;
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t x[64];
            ld64(tmem_base + lane_addr + c2 * 64, x);
#pragma unroll
            for (int c = 0; c < 8; ++c) {
              float f[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(x[c * 8 + i]);
              reinterpret_cast<uint4*>(dst + c2 * 64)[c] = pack8(f);
            }
          }
        }
        __nv_bfloat16* dst = p.dS + ((size_t)tile * 128 + t) * D;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t x[64];
          ld64(tmem_base + lane_addr + 128 + c2 * 64, x);
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            float f[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(x[c * 8 + i]);
            reinterpret_cast<uint4*>(dst + c2 * 64)[c] = pack8(f);
          }
        }
      }
    }
  }
  cta_teardown<TMEM_COLS>(ctl, tmem_base);
}

// ============================================================================================ prepare, backward
struct PrepBwdParams {
  const float* beta;     // [T, H]
  const float* gc;       // [H, N, 64]
  const int2* chunks;
  __nv_bfloat16 *dq, *dk, *dv;   // [T, H, 128]
  float *dg, *dbeta;             // [T, H]
  float scale, eps;
  int H, N;
  int* status;
};

struct PrepBwdSmem {
  // region 1: the scan's tensors for the first products, then the tiles made along the way
  static constexpr int offS = 0, offG = offS + kS, offVn = offG + kS;
  static constexpr int offDw = 0, offDtm = offDw + kT, offY = offDtm + kSq, offMs = offY + kSq, offNt = offMs + kSq;
  static constexpr int offSc = offNt + kSq + kBlk;   // fp32 [64][65]: R + Rp, summed by columns (after the slack a 128-row A read may touch)
  // region 2
  static constexpr int offDu = offVn + kT, offK = offDu + kT, offQ = offK + kT, offV = offQ + kT, offVb = offV + kT;
  static constexpr int offKbg = offVb + kT, offDqg = offKbg + kT, offTm = offDqg + kT, offDp = offTm + kSq, offPp = offDp + kSq;
  static constexpr int offF = offPp + kSq;     // floats: sb, sgc, (2 unused), dgc [64] each; part [4][64]; scal [4]
  static constexpr int offCtl = offF + (5 * 64 + 4 * 64 + 4) * 4;
  static constexpr int kTotal = offCtl + 64 + 1024;
};
static_assert(PrepBwdSmem::offSc + 64 * 65 * 4 <= PrepBwdSmem::offDu, "tiles made along the way stay inside region 1");
static_assert(PrepBwdSmem::kTotal <= 232448, "shared memory of the prepare-backward kernel");

__global__ void __launch_bounds__(THREADS, 1)
gdn_prepare_bwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmS,
                       const __grid_constant__ CUtensorMap tmG, const __grid_constant__ CUtensorMap tmVn,
                       const __grid_constant__ CUtensorMap tmDu, const __grid_constant__ CUtensorMap tmDqg,
                       const __grid_constant__ CUtensorMap tmDp, const __grid_constant__ CUtensorMap tmPp,
                       const __grid_constant__ CUtensorMap tmTm, PrepBwdParams p) {
  using L = PrepBwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* sb = reinterpret_cast<float*>(smem + L::offF);
  float* sgc = sb + 64;
  float* sdgc = sgc + 3 * 64;
  float* sc = reinterpret_cast<float*>(smem + L::offSc);
  float* part = sdgc + 64;
  float* scal = part + 256;   // [0] <S, G>, [1] sum of s_i
  Ctl ctl;
  constexpr int TMEM_COLS = 512;
  constexpr int cDW = 0, cDKDEC = 128, cKK = 256, cSQ = 320, cDQF = 256, cDKF = 384;   // columns, see the stages below
  const uint32_t tmem_base = cta_setup<TMEM_COLS>(ctl, smem + L::offCtl);

  const int n = blockIdx.x, h = blockIdx.y;
  const int2 ch = p.chunks[n];
  const int tok0 = ch.x, len = ch.y;
  const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
  const int r = t & 63, cb = t >> 6;
  const bool valid = r < len;
  const int tile = h * p.N + n;
  const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;

  if (t == 0) {
    mbar_expect_tx(ctl.bar_tma, 2 * kS + 6 * kT + 3 * kSq);
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      tma_load_2d(smem + L::offS + b * kSBlk, &tmS, ctl.bar_tma, 64 * b, tile * 128);
      tma_load_2d(smem + L::offG + b * kSBlk, &tmG, ctl.bar_tma, 64 * b, tile * 128);
      tma_load_2d(smem + L::offVn + b * kBlk, &tmVn, ctl.bar_tma, 64 * b, tile * 64);
      tma_load_2d(smem + L::offDu + b * kBlk, &tmDu, ctl.bar_tma, 64 * b, tile * 64);
      tma_load_2d(smem + L::offDqg + b * kBlk, &tmDqg, ctl.bar_tma, 64 * b, tile * 64);
      tma_load_2d(smem + L::offK + b * kBlk, &tmK, ctl.bar_tma, h * D + 64 * b, tok0);
      tma_load_2d(smem + L::offQ + b * kBlk, &tmQ, ctl.bar_tma, h * D + 64 * b, tok0);
      tma_load_2d(smem + L::offV + b * kBlk, &tmV, ctl.bar_tma, h * D + 64 * b, tok0);
    }
    tma_load_2d(smem + L::offDp, &tmDp, ctl.bar_tma, 0, tile * 64);
    tma_load_2d(smem + L::offPp, &tmPp, ctl.bar_tma, 0, tile * 64);
    tma_load_2d(smem + L::offTm, &tmTm, ctl.bar_tma, 0, tile * 64);
  }
  if (cb == 0) {
    sb[r] = valid ? p.beta[(size_t)(tok0 + r) * p.H + h] : 0.f;
    sgc[r] = p.gc[(size_t)tile * 64 + r];
  }
  if (t == 0) { scal[0] = 0.f; scal[1] = 0.f; }
  bool ok = mbar_wait(ctl.bar_tma, 0, ctl.abort_flag, p.status, kErrTimeoutFull);
  ok = __syncthreads_and(ok);
  float rk = 0.f, rq = 0.f, E = 0.f, F = 0.f, b = 0.f, gcr = 0.f, last = 0.f;
  float dbeta = 0.f, dgc = 0.f;
  if (ok) {
    // ---- phase 1: the operand tiles of the forward pass again (kf, qf in place; beta e^gc k; beta v)
    {
      uint4 kr[8], qr[8];
      float ssk = 0.f, ssq = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        kr[c] = *row8(smem + L::offK, kBlk, r, cb * 8 + c);
        qr[c] = *row8(smem + L::offQ, kBlk, r, cb * 8 + c);
        float f[8];
        unpack8(kr[c], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ssk = fmaf(f[i], f[i], ssk);
        unpack8(qr[c], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) ssq = fmaf(f[i], f[i], ssq);
      }
      part[cb * 64 + r] = ssk;
      part[128 + cb * 64 + r] = ssq;
      __syncthreads();
      gcr = sgc[r];
      last = sgc[63];
      rk = valid ? rsqrtf(part[r] + part[64 + r] + p.eps) : 0.f;
      rq = valid ? rsqrtf(part[128 + r] + part[192 + r] + p.eps) * p.scale : 0.f;
      E = __expf(gcr); F = __expf(last - gcr); b = sb[r];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float f[8], o1[8];
        unpack8(kr[c], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) { f[i] *= rk; o1[i] = f[i] * (b * E); }
        *row8(smem + L::offK, kBlk, r, cb * 8 + c) = pack8(f);
        *row8(smem + L::offKbg, kBlk, r, cb * 8 + c) = pack8(o1);
        unpack8(qr[c], f);
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] *= rq;
        *row8(smem + L::offQ, kBlk, r, cb * 8 + c) = pack8(f);
        const uint4 vr = *row8(smem + L::offV, kBlk, r, cb * 8 + c);
        unpack8(vr, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) { f[i] = valid ? f[i] : 0.f; o1[i] = f[i] * b; }
        *row8(smem + L::offV, kBlk, r, cb * 8 + c) = pack8(f);
        *row8(smem + L::offVb, kBlk, r, cb * 8 + c) = pack8(o1);
      }
    }
    publish();
    // ---- stage A: dw = -du S, dkdec = v_new G, k k^T; meanwhile <S, G> for the gradient of the chunk's decay
    if (t == 0) {
      issue<false, true>(tmem_base + cDW, smem + L::offDu, kBlk, smem + L::offS, kSBlk, 128, 8, false);
      issue<false, true>(tmem_base + cDKDEC, smem + L::offVn, kBlk, smem + L::offG, kSBlk, 128, 8, false);
      issue<false, false>(tmem_base + cKK, smem + L::offK, kBlk, smem + L::offK, kBlk, 64, 8, false);
    }
    {
      float acc = 0.f;
      const uint4* s4 = reinterpret_cast<const uint4*>(smem + L::offS);
      const uint4* g4 = reinterpret_cast<const uint4*>(smem + L::offG);
      for (int i = t; i < kS / 16; i += THREADS) {   // same layout on both sides: the element-wise product needs no indices
        float a[8], c8[8];
        unpack8(s4[i], a);
        unpack8(g4[i], c8);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc = fmaf(a[u], c8[u], acc);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (lane == 0) atomicAdd(&scal[0], acc);
    }
    ok = mma_done(ctl, p.status);
  }
  if (ok) {
    if (t < 64) {  // dw -> bf16 tile (over the state tile, which is no longer read)
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t x[64];
        ld64(tmem_base + lane_addr + cDW + c2 * 64, x);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float f[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) f[i] = -__uint_as_float(x[c * 8 + i]);
          *row8(smem + L::offDw, kBlk, r, c2 * 8 + c) = pack8(f);
        }
      }
    }
    publish();
    // ---- stage B: dT = dw (beta e^gc k)^T + du (beta v)^T ; X2 = T^T du
    if (t == 0) {
      issue<false, false>(tmem_base + cSQ, smem + L::offDw, kBlk, smem + L::offKbg, kBlk, 64, 8, false);
      issue<false, false>(tmem_base + cSQ, smem + L::offDu, kBlk, smem + L::offVb, kBlk, 64, 8, true);
      issue<true, true>(tmem_base + cDW, smem + L::offTm, kBlk, smem + L::offDu, kBlk, 128, 4, false);
    }
    ok = mma_done(ctl, p.status);
  }
  if (ok) {
    if (t < 64) {
      uint32_t x[64];
      ld64(tmem_base + lane_addr + cSQ, x);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(x[c * 8 + i]);
        *row8(smem + L::offDtm, kBlk, r, c) = pack8(f);
      }
      // dv = beta X2 ; dbeta += X2 . v
      __nv_bfloat16* dst = p.dv + ((size_t)(tok0 + r) * p.H + h) * D;
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        ld64(tmem_base + lane_addr + cDW + c2 * 64, x);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float f[8], v[8];
          unpack8(*row8(smem + L::offV, kBlk, r, c2 * 8 + c), v);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float x2 = __uint_as_float(x[c * 8 + i]);
            dbeta = fmaf(x2, v[i], dbeta);
            f[i] = x2 * b;
          }
          if (valid) reinterpret_cast<uint4*>(dst + c2 * 64)[c] = pack8(f);
        }
      }
    }
    publish();
    // ---- stage C: Y = dT T^T
    if (t == 0) issue<false, false>(tmem_base + cSQ, smem + L::offDtm, kBlk, smem + L::offTm, kBlk, 64, 4, false);
    ok = mma_done(ctl, p.status);
  }
  if (ok) {
    if (t < 64) {
      uint32_t x[64];
      ld64(tmem_base + lane_addr + cSQ, x);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float f[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = __uint_as_float(x[c * 8 + i]);
        *row8(smem + L::offY, kBlk, r, c) = pack8(f);
      }
    }
    publish();
    // ---- stage D: dA = -T^T Y ; X1 = T^T dw
    if (t == 0) {
      issue<true, true>(tmem_base + cSQ, smem + L::offTm, kBlk, smem + L::offY, kBlk, 64, 4, false);
      issue<true, true>(tmem_base + cDW, smem + L::offTm, kBlk, smem + L::offDw, kBlk, 128, 4, false);
    }
    ok = mma_done(ctl, p.status);
  }
  if (ok) {
    if (t < 64) {
      uint32_t da[64], kk[64];
      ld64(tmem_base + lane_addr + cSQ, da);
      ld64(tmem_base + lane_addr + cKK, kk);
      float ci = 0.f;
      float* srow = sc + r * 65;
      store_bf16(smem + L::offMs, kBlk, r, r, 0.f);
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        float rij = 0.f;
        if (j < r) {
          const float dec = __expf(gcr - sgc[j]);
          const float dA = -__uint_as_float(da[j]);
          const float kd = __uint_as_float(kk[j]) * dec;
          ci = fmaf(dA, kd, ci);
          rij = b * dA * kd;
          const float m = dA * b * dec;
          store_bf16(smem + L::offMs, kBlk, r, j, m);
          store_bf16(smem + L::offMs, kBlk, j, r, m);
        }
        srow[j] = rij;
      }
      dbeta += ci;
      dgc += b * ci;
      // N = dP * decay (lower, diagonal included); Rp = dP * P
      float rowp = 0.f;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float dp[8], pp[8], f[8];
        unpack8(*row8(smem + L::offDp, kBlk, r, c), dp);
        unpack8(*row8(smem + L::offPp, kBlk, r, c), pp);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = c * 8 + i;
          if (j <= r) {
            const float rp = dp[i] * pp[i];
            rowp += rp;
            srow[j] += rp;
            f[i] = dp[i] * __expf(gcr - sgc[j]);
          } else {
            f[i] = 0.f;
          }
        }
        *row8(smem + L::offNt, kBlk, r, c) = pack8(f);
      }
      dgc += rowp;
    }
    publish();
    // ---- stage E: dkf = (M + M^T) kf + N^T qf ; dqf = N kf
    if (t == 0) {
      issue<false, true>(tmem_base + cDKF, smem + L::offMs, kBlk, smem + L::offK, kBlk, 128, 4, false);
      issue<true, true>(tmem_base + cDKF, smem + L::offNt, kBlk, smem + L::offQ, kBlk, 128, 4, true);
      issue<false, true>(tmem_base + cDQF, smem + L::offNt, kBlk, smem + L::offK, kBlk, 128, 4, false);
    }
    ok = mma_done(ctl, p.status);
  }
  if (ok) {
    float s_r = 0.f;
    if (t < 64) {
      // pass 1: the row dot products
      float d1 = 0.f, d2 = 0.f, b1 = 0.f, e1 = 0.f, sd = 0.f;
      const float bE = b * E;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t xa[32], xb[32], xc[32], xd[32];
        tmem_ld_32x32(tmem_base + lane_addr + cDKF + c4 * 32, xa);
        tmem_ld_32x32(tmem_base + lane_addr + cDW + c4 * 32, xb);      // X1
        tmem_ld_32x32(tmem_base + lane_addr + cDKDEC + c4 * 32, xc);
        tmem_ld_32x32(tmem_base + lane_addr + cDQF + c4 * 32, xd);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float kf[8], qf[8], dq8[8];
          unpack8(*row8(smem + L::offK, kBlk, r, c4 * 4 + c), kf);
          unpack8(*row8(smem + L::offQ, kBlk, r, c4 * 4 + c), qf);
          unpack8(*row8(smem + L::offDqg, kBlk, r, c4 * 4 + c), dq8);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float x1 = __uint_as_float(xb[c * 8 + i]), dkd = __uint_as_float(xc[c * 8 + i]);
            const float dkf = __uint_as_float(xa[c * 8 + i]) + bE * x1 + F * dkd;
            const float dqf = __uint_as_float(xd[c * 8 + i]) + E * dq8[i];
            d1 = fmaf(dkf, kf[i], d1);
            b1 = fmaf(x1, kf[i], b1);
            sd = fmaf(dkd, kf[i], sd);
            d2 = fmaf(dqf, qf[i], d2);
            e1 = fmaf(dq8[i], qf[i], e1);
          }
        }
      }
      s_r = F * sd;
      dbeta += E * b1;
      float colsum = 0.f;
      for (int i = 0; i < 64; ++i) colsum += sc[i * 65 + r];
      dgc += bE * b1 + E * e1 - s_r - colsum;
      // pass 2: gradients of the raw q and k through the l2 normalisation
      const float rstd_q = rq / p.scale;
      __nv_bfloat16* dkrow = p.dk + ((size_t)(tok0 + r) * p.H + h) * D;
      __nv_bfloat16* dqrow = p.dq + ((size_t)(tok0 + r) * p.H + h) * D;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t xa[32], xb[32], xc[32], xd[32];
        tmem_ld_32x32(tmem_base + lane_addr + cDKF + c4 * 32, xa);
        tmem_ld_32x32(tmem_base + lane_addr + cDW + c4 * 32, xb);
        tmem_ld_32x32(tmem_base + lane_addr + cDKDEC + c4 * 32, xc);
        tmem_ld_32x32(tmem_base + lane_addr + cDQF + c4 * 32, xd);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          float kf[8], qf[8], dq8[8], ok8[8], oq8[8];
          unpack8(*row8(smem + L::offK, kBlk, r, c4 * 4 + c), kf);
          unpack8(*row8(smem + L::offQ, kBlk, r, c4 * 4 + c), qf);
          unpack8(*row8(smem + L::offDqg, kBlk, r, c4 * 4 + c), dq8);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float x1 = __uint_as_float(xb[c * 8 + i]), dkd = __uint_as_float(xc[c * 8 + i]);
            const float dkf = __uint_as_float(xa[c * 8 + i]) + bE * x1 + F * dkd;
            const float dqf = __uint_as_float(xd[c * 8 + i]) + E * dq8[i];
            ok8[i] = rk * (dkf - kf[i] * d1);
            oq8[i] = rstd_q * (p.scale * dqf - qf[i] * d2 / p.scale);
          }
          if (valid) {
            reinterpret_cast<uint4*>(dkrow + c4 * 32)[c] = pack8(ok8);
            reinterpret_cast<uint4*>(dqrow + c4 * 32)[c] = pack8(oq8);
          }
        }
      }
      sdgc[r] = dgc;
    }
    if (t < 64) {
      float v = s_r;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (lane == 0) atomicAdd(&scal[1], v);
    }
    __syncthreads();
    if (t < 64 && valid) {
      // dg = reverse cumulative sum of dgc; the chunk's last cumulative decay also feeds exp(last) and every exp(last - gc)
      float acc = scal[0] * __expf(last) + scal[1];
      for (int i = r; i < 64; ++i) acc += sdgc[i];
      p.dg[(size_t)(tok0 + r) * p.H + h] = acc;
      p.dbeta[(size_t)(tok0 + r) * p.H + h] = dbeta;
    }
  }
  cta_teardown<TMEM_COLS>(ctl, tmem_base);
}

template <typename K>
int set_smem(K kern, int bytes) {
  return (int)cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

// tensor map over a head-major tile stack: [tiles * rows, cols] bf16, boxes of {64 columns, box_rows}
int stack_map(CUtensorMap* m, const void* base, long tiles, int rows, int cols, int box_rows) {
  return vlmt_make_tmap_2d_bf16(m, base, (uint64_t)cols, (uint64_t)tiles * rows, (uint64_t)cols * 2, 64, (uint32_t)box_rows);
}
// tensor map over a token-layout activation [T, H * 128] with row stride `ld` elements, boxes of {64 columns, 64 tokens}
int token_map(CUtensorMap* m, const void* base, int T, int H, long ld) {
  return vlmt_make_tmap_2d_bf16(m, base, (uint64_t)H * D, (uint64_t)T, (uint64_t)ld * 2, 64, 64);
}
}  // namespace

extern "C" int vlmt_gdn_prepare_fwd(const void* q, const void* k, const void* v, long ldq, long ldk, long ldv, const float* g,
                                    const float* beta, const int* chunks, int T, int H, int N, float scale, float eps, void* w, void* u,
                                    void* kdec, void* qg, void* P, void* Tm, float* gc, float* decay, int* status, cudaStream_t st) {
  if (N <= 0) return 0;
  CUtensorMap tq, tk, tv;
  int r;
  if ((r = token_map(&tq, q, T, H, ldq))) return 1000 + r;
  if ((r = token_map(&tk, k, T, H, ldk))) return 2000 + r;
  if ((r = token_map(&tv, v, T, H, ldv))) return 3000 + r;
  PrepParams p;
  p.g = g; p.beta = beta; p.chunks = reinterpret_cast<const int2*>(chunks);
  p.w = (__nv_bfloat16*)w; p.u = (__nv_bfloat16*)u; p.kdec = (__nv_bfloat16*)kdec; p.qg = (__nv_bfloat16*)qg;
  p.P = (__nv_bfloat16*)P; p.Tm = (__nv_bfloat16*)Tm; p.gc = gc; p.decay = decay;
  p.scale = scale; p.eps = eps; p.H = H; p.N = N; p.status = status;
  if ((r = set_smem(gdn_prepare_fwd_kernel, PrepSmem::kTotal))) return r;
  gdn_prepare_fwd_kernel<<<dim3(N, H), THREADS, PrepSmem::kTotal, st>>>(tq, tk, tv, p);
  return (int)cudaGetLastError();
}

extern "C" int vlmt_gdn_output_fwd(const void* qg, const void* P, const void* states, const void* vnew, const int* chunks, int H, int N,
                                   void* o, int* status, cudaStream_t st) {
  if (N <= 0) return 0;
  CUtensorMap tqg, tp, ts, tvn;
  int r;
  const long tiles = (long)H * N;
  if ((r = stack_map(&tqg, qg, tiles, 64, 128, 64))) return 1000 + r;
  if ((r = stack_map(&tp, P, tiles, 64, 64, 64))) return 2000 + r;
  if ((r = stack_map(&ts, states, tiles, 128, 128, 128))) return 3000 + r;
  if ((r = stack_map(&tvn, vnew, tiles, 64, 128, 64))) return 4000 + r;
  OutParams p;
  p.chunks = reinterpret_cast<const int2*>(chunks); p.o = (__nv_bfloat16*)o; p.H = H; p.N = N; p.status = status;
  if ((r = set_smem(gdn_output_fwd_kernel, OutSmem::kTotal))) return r;
  gdn_output_fwd_kernel<<<dim3(N, H), THREADS, OutSmem::kTotal, st>>>(tqg, tp, ts, tvn, p);
  return (int)cudaGetLastError();
}

extern "C" int vlmt_gdn_output_bwd(const void* dout, long ld_do, const void* qg, const void* P, const void* states, const void* vnew,
                                   const int* chunks, int T, int H, int N, void* dqg, void* dP, void* dvn, void* dS, int* status,
                                   cudaStream_t st) {
  if (N <= 0) return 0;
  CUtensorMap tdo, tqg, tp, ts, tvn;
  int r;
  const long tiles = (long)H * N;
  if ((r = token_map(&tdo, dout, T, H, ld_do))) return 500 + r;
  if ((r = stack_map(&tqg, qg, tiles, 64, 128, 64))) return 1000 + r;
  if ((r = stack_map(&tp, P, tiles, 64, 64, 64))) return 2000 + r;
  if ((r = stack_map(&ts, states, tiles, 128, 128, 128))) return 3000 + r;
  if ((r = stack_map(&tvn, vnew, tiles, 64, 128, 64))) return 4000 + r;
  OutBwdParams p;
  p.chunks = reinterpret_cast<const int2*>(chunks);
  p.dqg = (__nv_bfloat16*)dqg; p.dvn = (__nv_bfloat16*)dvn; p.dP = (__nv_bfloat16*)dP; p.dS = (__nv_bfloat16*)dS;
  p.H = H; p.N = N; p.status = status;
  if ((r = set_smem(gdn_output_bwd_kernel, OutBwdSmem::kTotal))) return r;
  gdn_output_bwd_kernel<<<dim3(N, H), THREADS, OutBwdSmem::kTotal, st>>>(tdo, tqg, tp, ts, tvn, p);
  return (int)cudaGetLastError();
}

extern "C" int vlmt_gdn_prepare_bwd(const void* q, const void* k, const void* v, long ldq, long ldk, long ldv, const float* beta,
                                    const float* gc, const int* chunks, int T, int H, int N, float scale, float eps, const void* states,
                                    const void* adj, const void* vnew, const void* du, const void* dqg, const void* dP, const void* P,
                                    const void* Tm, void* dq, void* dk, void* dv, float* dg, float* dbeta, int* status, cudaStream_t st) {
  if (N <= 0) return 0;
  CUtensorMap tq, tk, tv, ts, tg, tvn, tdu, tdqg, tdp, tpp, ttm;
  int r;
  const long tiles = (long)H * N;
  if ((r = token_map(&tq, q, T, H, ldq))) return 1000 + r;
  if ((r = token_map(&tk, k, T, H, ldk))) return 2000 + r;
  if ((r = token_map(&tv, v, T, H, ldv))) return 3000 + r;
  if ((r = stack_map(&ts, states, tiles, 128, 128, 128))) return 4000 + r;
  if ((r = stack_map(&tg, adj, tiles, 128, 128, 128))) return 5000 + r;
  if ((r = stack_map(&tvn, vnew, tiles, 64, 128, 64))) return 6000 + r;
  if ((r = stack_map(&tdu, du, tiles, 64, 128, 64))) return 7000 + r;
  if ((r = stack_map(&tdqg, dqg, tiles, 64, 128, 64))) return 8000 + r;
  if ((r = stack_map(&tdp, dP, tiles, 64, 64, 64))) return 9000 + r;
  if ((r = stack_map(&tpp, P, tiles, 64, 64, 64))) return 10000 + r;
  if ((r = stack_map(&ttm, Tm, tiles, 64, 64, 64))) return 11000 + r;
  PrepBwdParams p;
  p.beta = beta; p.gc = gc; p.chunks = reinterpret_cast<const int2*>(chunks);
  p.dq = (__nv_bfloat16*)dq; p.dk = (__nv_bfloat16*)dk; p.dv = (__nv_bfloat16*)dv; p.dg = dg; p.dbeta = dbeta;
  p.scale = scale; p.eps = eps; p.H = H; p.N = N; p.status = status;
  if ((r = set_smem(gdn_prepare_bwd_kernel, PrepBwdSmem::kTotal))) return r;
  gdn_prepare_bwd_kernel<<<dim3(N, H), THREADS, PrepBwdSmem::kTotal, st>>>(tq, tk, tv, ts, tg, tvn, tdu, tdqg, tdp, tpp, ttm, p);
  return (int)cudaGetLastError();
}
