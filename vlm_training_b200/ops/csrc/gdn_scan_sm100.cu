// Chunk-to-chunk recurrence of the gated delta rule as one tcgen05 kernel (sm_100a).
//
// One CTA per (document, head) walks the document's 64-token chunks in order (or in reverse, for the backward pass)
// and carries the state Z [Dv = 128, Dk = 128] in tensor memory:
//
//     states[c] = Z                                       (bf16, the state entering step c)
//     Y[c]      = E[c] + s1 * (X1[c] Z^T)                 [64, Dv]
//     Z         = ext[c'] + decay[c'] * ( ... )           prepared for the next step c' as soon as Z is known
//     Z         = Z_prepared + s2 * Y[c]^T X2[c]
//
// forward  (s1 = -1, s2 = +1, no ext): X1 = w, X2 = k * exp(g_last - g), E = u   ->  Y = v_new, states = S^T
// backward (s1 = +1, s2 = -1):         X1 = k * exp(..), X2 = w, E = dv_new, ext = dS  ->  total dv_new, adjoint states
//
// Both products have M = 128 (the Dv rows of Z^T live on the 128 TMEM lanes):
//     Yacc [Dv, 64]  = Zbf16 [Dv, Dk] . X1^T      A from TMEM (packed bf16), B = X1 tile K-major,  N = 64,  K = 128
//     ACC  [Dv, Dk] += (s2 Y)^T [Dv, 64] . X2     A from TMEM (packed bf16), B = X2 tile MN-major, N = 128, K = 64
// so the state never leaves the SM: the fp32 accumulator ACC stays in TMEM for the whole document, its bf16 copy (the A
// operand of the first product) is rewritten once per chunk by the four compute warps, which also scale it by the
// next chunk's decay, add the external gradient (backward) and store the entering state for the batched products that
// follow the scan.  TMEM: ACC 128 columns, A1 64, Yacc 64 (its first 32 columns are reused for the packed s2 * Y).
//
// Warps: 0 = TMA producer (X1, X2, E tiles of the next chunk, two stages), 1 = MMA issue (one thread), 2-5 = compute
// (warp w owns TMEM lanes 32 (w % 4) ...).  Every wait is bounded; a wait that runs out sets the status word and the
// CTA leaves through the common teardown (TMEM freed).
#include "gdn_scan_sm100.h"
#include "gemm_sm100.h"
#include "sm100.cuh"

#include <cuda_bf16.h>

namespace {
using namespace sm100;

constexpr int C = 64, DK = 128, DV = 128;
constexpr int THREADS = 192;
constexpr int kTile = C * 128 * 2;          // one [64, 128] bf16 tile = two 64x64 swizzled boxes
constexpr int kStage = 3 * kTile;           // X1, X2, E
constexpr int kStages = 2;
constexpr int offBar = kStages * kStage;
constexpr int kSmem = offBar + 256 + 1024;
constexpr int TMEM_COLS = 256;
constexpr int ACC_COL = 0, A1_COL = 128, Y_COL = 192;

struct Params {
  const float* decay;           // [N, H]
  const __nv_bfloat16* ext;     // [N, H, DV, DK] or null
  __nv_bfloat16* Y;             // [N, H, 64, DV]
  __nv_bfloat16* states;        // [N, H, DV, DK]
  const int2* ranges;           // per document: first chunk, chunk count
  int H;
  int cs, hs;                   // tile index of (chunk c, head h) = c * cs + h * hs: [N, H] or [H, N] tile order
  int* status;
};

template <bool REVERSE>
__global__ void __launch_bounds__(THREADS, 2)
gdn_scan_kernel(const __grid_constant__ CUtensorMap tmX1, const __grid_constant__ CUtensorMap tmX2,
                const __grid_constant__ CUtensorMap tmE, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + offBar);
  uint64_t* x_full = bars;         // 2
  uint64_t* x_empty = bars + 2;    // 2
  uint64_t* a1_ready = bars + 4;   // 4 compute warps: A1 and ACC hold the state for this step
  uint64_t* y_full = bars + 5;     // first product done
  uint64_t* a2_ready = bars + 6;   // 4 compute warps: packed s2 * Y written
  uint64_t* z_full = bars + 7;     // second product done: ACC holds the new state
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int2 range = p.ranges[blockIdx.x];
  const int h = blockIdx.y;
  const int n_steps = range.y;
  if (n_steps <= 0) return;  // uniform for the CTA
  // chunk visited at step n
  auto chunk_of = [&](int n) { return REVERSE ? range.x + n_steps - 1 - n : range.x + n; };
  auto tile_of = [&](int chunk) { return chunk * p.cs + h * p.hs; };

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) { mbar_init(&x_full[i], 1); mbar_init(&x_empty[i], 1); }
    mbar_init(a1_ready, 4); mbar_init(y_full, 1); mbar_init(a2_ready, 4); mbar_init(z_full, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmX1); tma_prefetch_desc(&tmX2); tma_prefetch_desc(&tmE);
  }
  if (warp == 1) tmem_alloc<TMEM_COLS>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int n = 0; n < n_steps; ++n) {
        const int s = n & 1;
        const uint32_t ph = ((n >> 1) & 1) ^ 1;
        if (!mbar_wait(&x_empty[s], ph, abort_flag, p.status, kErrTimeoutEmpty)) break;
        const int row = tile_of(chunk_of(n)) * C;
        uint8_t* st = smem + s * kStage;
        mbar_expect_tx(&x_full[s], kStage);
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          tma_load_2d(st + b * 8192, &tmX1, &x_full[s], 64 * b, row);
          tma_load_2d(st + kTile + b * 8192, &tmX2, &x_full[s], 64 * b, row);
          tma_load_2d(st + 2 * kTile + b * 8192, &tmE, &x_full[s], 64 * b, row);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc1 = make_idesc_bf16(128, C, false, false);
      constexpr uint32_t idesc2 = make_idesc_bf16(128, DK, false, true);
      const uint32_t acc = tmem_base + ACC_COL, a1 = tmem_base + A1_COL, yacc = tmem_base + Y_COL;
      for (int n = 0; n < n_steps; ++n) {
        const int s = n & 1;
        if (!mbar_wait(&x_full[s], (n >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) break;
        if (!mbar_wait(a1_ready, n & 1, abort_flag, p.status, kErrTimeoutOther)) break;
        tc_fence_after();
        const SmemDesc b1 = make_desc(smem_u32(smem + s * kStage), 16, 1024);             // X1: K-major, 64 rows
        const SmemDesc b2 = make_desc(smem_u32(smem + s * kStage + kTile), 8192, 1024);   // X2: MN-major, 64 k-lines
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk) {
          const SmemDesc b = desc_off(b1, (kk >> 2) * 8192 + (kk & 3) * 32);
          if (kk == 0) umma_ts<0>(yacc, a1, b, idesc1); else umma_ts<1>(yacc, a1 + kk * 8, b, idesc1);
        }
        umma_commit(y_full);
        if (n + 1 == n_steps) break;   // the state after the last step is not used: every MMA issued has a waiter
        if (!mbar_wait(a2_ready, n & 1, abort_flag, p.status, kErrTimeoutOther)) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < C / 16; ++kk) umma_ts<1>(acc, yacc + kk * 8, desc_off(b2, kk * 2048), idesc2);
        umma_commit(z_full);
        umma_commit(&x_empty[s]);
      }
    }
  } else {
    const int q = warp & 3;
    const int dv = q * 32 + lane;                      // row of Z^T owned by this thread
    const uint32_t lane_addr = (uint32_t)(q * 32) << 16;
    const uint32_t acc = tmem_base + ACC_COL + lane_addr, a1 = tmem_base + A1_COL + lane_addr, yacc = tmem_base + Y_COL + lane_addr;
    constexpr float s1 = REVERSE ? 1.f : -1.f, s2 = REVERSE ? -1.f : 1.f;
    auto state_row = [&](int chunk) { return ((size_t)tile_of(chunk) * DV + dv) * DK; };

    // ---- prologue: Z = 0 entering the first step; ACC = ext[first]
    {
      const int c0 = chunk_of(0);
      __nv_bfloat16* srow = p.states + state_row(c0);
      const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int i = 0; i < DK / 8; ++i) reinterpret_cast<uint4*>(srow)[i] = z4;
      uint32_t z[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) z[i] = 0u;
      tmem_st_32x32(a1, z);
      tmem_st_32x32(a1 + 32, z);
#pragma unroll
      for (int cb = 0; cb < DK / 32; ++cb) {
        uint32_t v[32];
        if (REVERSE && p.ext != nullptr) {
          const uint4* er = reinterpret_cast<const uint4*>(p.ext + state_row(c0) + cb * 32);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint4 e4 = er[u];
            const uint32_t w4[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[u * 8 + 2 * j] = w4[j] << 16;             // bf16 -> fp32 bit pattern
              v[u * 8 + 2 * j + 1] = w4[j] & 0xffff0000u;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        tmem_st_32x32(acc + cb * 32, v);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(a1_ready);
    }

    bool ok = true;
    for (int n = 0; n < n_steps && ok; ++n) {
      const int s = n & 1;
      const int c = chunk_of(n);
      const bool has_next = n + 1 < n_steps;
      const int cn = has_next ? chunk_of(n + 1) : c;
      // ---- Y = E + s1 * acc1
      if (!mbar_wait(&x_full[s], (n >> 1) & 1, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
      if (!mbar_wait(y_full, n & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t r[64];
        tmem_ld_32x32(yacc, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_ld_32x32(yacc + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_ld_wait();
        const uint8_t* et = smem + s * kStage + 2 * kTile + (dv >> 6) * 8192;
        const int ci = (dv & 63) >> 3, ce = (dv & 7) * 2;
        __nv_bfloat16* yrow = p.Y + ((size_t)tile_of(c) * C) * DV + dv;
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < C; i += 2) {
          const float e0 = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(et + i * 128 + ((ci ^ (i & 7)) << 4) + ce));
          const float e1 = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(et + (i + 1) * 128 + ((ci ^ ((i + 1) & 7)) << 4) + ce));
          const float y0 = fmaf(s1, __uint_as_float(r[i]), e0), y1 = fmaf(s1, __uint_as_float(r[i + 1]), e1);
          const __nv_bfloat16 b0 = __float2bfloat16(y0), b1 = __float2bfloat16(y1);
          yrow[(size_t)i * DV] = b0;
          yrow[(size_t)(i + 1) * DV] = b1;
          // the second product uses the rounded values that were stored, with the sign of s2
          pk[i >> 1] = pack_bf16x2(s2 * __bfloat162float(b0), s2 * __bfloat162float(b1));
        }
        tmem_st_32x32(yacc, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(a2_ready);
      }
      if (!has_next) break;
      // ---- new state: store it, repack it, prepare ACC for the next step
      const float dn = p.decay[tile_of(cn)];
      uint4 ex[16];
      if (REVERSE && p.ext != nullptr) {   // independent of the recurrence: in flight while the second product runs
        const uint4* er = reinterpret_cast<const uint4*>(p.ext + state_row(cn));
#pragma unroll
        for (int u = 0; u < 16; ++u) ex[u] = er[u];
      }
      if (!mbar_wait(z_full, n & 1, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      __nv_bfloat16* srow = p.states + state_row(cn);
#pragma unroll
      for (int cb = 0; cb < DK / 32; ++cb) {
        uint32_t v[32];
        tmem_ld_32x32(acc + cb * 32, v);
        tmem_ld_wait();
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = pack_bf16x2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
#pragma unroll
        for (int u = 0; u < 4; ++u)
          reinterpret_cast<uint4*>(srow + cb * 32)[u] = make_uint4(pk[u * 4], pk[u * 4 + 1], pk[u * 4 + 2], pk[u * 4 + 3]);
        tmem_st_32x16(a1 + cb * 16, pk);
        // ACC for the next step: ext + decay * Z (the fp32 value, not the rounded copy)
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * dn);
        if (REVERSE && p.ext != nullptr) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const uint4 e4 = ex[cb * 4 + u];
            const uint32_t w4[4] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[u * 8 + 2 * j] = __float_as_uint(__uint_as_float(v[u * 8 + 2 * j]) + __uint_as_float(w4[j] << 16));
              v[u * 8 + 2 * j + 1] = __float_as_uint(__uint_as_float(v[u * 8 + 2 * j + 1]) + __uint_as_float(w4[j] & 0xffff0000u));
            }
          }
        }
        tmem_st_32x32(acc + cb * 32, v);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(a1_ready);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {  // let copies in flight land before the shared memory goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

template <bool REVERSE>
int launch(const CUtensorMap& t1, const CUtensorMap& t2, const CUtensorMap& te, const Params& p, int n_docs, cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gdn_scan_kernel<REVERSE>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem) != cudaSuccess) return -10;
    attr_set = true;
  }
  dim3 grid(n_docs, p.H);
  gdn_scan_kernel<REVERSE><<<grid, THREADS, kSmem, stream>>>(t1, t2, te, p);
  return cudaGetLastError() == cudaSuccess ? 0 : -11;
}
}  // namespace

extern "C" int vlmt_gdn_scan(const void* x1, const void* x2, const void* e, const float* decay, const void* ext, void* y,
                             void* states, const int* ranges, int n_docs, int n_chunks, int H, int head_major, int reverse, int* status,
                             cudaStream_t stream) {
  if (n_docs <= 0 || n_chunks <= 0) return 0;
  const uint64_t rows = (uint64_t)n_chunks * H * C;
  CUtensorMap t1, t2, te;
  int r;
  if ((r = vlmt_make_tmap_2d_bf16(&t1, x1, DK, rows, DK * 2, 64, 64))) return 1000 + r;
  if ((r = vlmt_make_tmap_2d_bf16(&t2, x2, DK, rows, DK * 2, 64, 64))) return 2000 + r;
  if ((r = vlmt_make_tmap_2d_bf16(&te, e, DV, rows, DV * 2, 64, 64))) return 3000 + r;
  Params p;
  p.decay = decay;
  p.ext = reinterpret_cast<const __nv_bfloat16*>(ext);
  p.Y = reinterpret_cast<__nv_bfloat16*>(y);
  p.states = reinterpret_cast<__nv_bfloat16*>(states);
  p.ranges = reinterpret_cast<const int2*>(ranges);
  p.H = H;
  p.cs = head_major ? 1 : H;
  p.hs = head_major ? n_chunks : 1;
  p.status = status;
  return reverse ? launch<true>(t1, t2, te, p, n_docs, stream) : launch<false>(t1, t2, te, p, n_docs, stream);
}
