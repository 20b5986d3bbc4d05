// FP8 training path for sm_100a: tensor-wise dynamic quantisation of bf16 matrices and a persistent FP8 GEMM.
//
//   amax_kernel   max |x| of a bf16 matrix (one atomic per block)
//   cast_kernel   q = saturate(x * format_max / amax) as e4m3 or e5m2, written as it is and / or transposed in one pass
//                 (128 x 64 tiles through shared memory); the transposed copy exists because the FP8 GEMM below takes
//                 K-major operands only, so the weight gradient dY^T . X and the input gradient dY . W read transposes
//   gemm_fp8_kernel   D[M,N] (+)= s * A(M,K) * B(N,K)^T, one byte per element, fp32 accumulation in TMEM
//                 (tcgen05.mma kind::f8f6f4, 128 x 256 x 32 per instruction: twice the bf16 rate), bf16 output
//       warp 0      TMA producer: 128-byte-swizzled tiles of 128 K-bytes into a 4-stage ring
//       warp 1      allocates TMEM (two 256-column accumulators), one lane issues the MMAs
//       warps 2..5  epilogue: tcgen05.ld, scale, bf16, swizzled staging, TMA store or TMA reduce-add
//   The scale s = rec_a[1] * rec_b[1] is read from device memory, so quantisation and GEMM queue without a host sync.
#include "sm100.cuh"

#include <cuda_fp8.h>
#include <stdlib.h>

#include "fp8_sm100.h"
#include "gemm_sm100.h"

namespace {
using namespace sm100;

// ------------------------------------------------------------------------------------------------ quantisation
__global__ void __launch_bounds__(256) amax_kernel(const __nv_bfloat16* __restrict__ x, long ld, long rows, int vec_per_row,
                                                   float* __restrict__ rec) {
  const long nvec = rows * vec_per_row;
  __nv_bfloat162 m2 = __floats2bfloat162_rn(0.f, 0.f);
  for (long v = (long)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += (long)gridDim.x * blockDim.x) {
    const long r = v / vec_per_row;
    const int c = (int)(v - r * vec_per_row);
    const uint4 q = *reinterpret_cast<const uint4*>(x + r * ld + c * 8);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) m2 = __hmax2(m2, __habs2(h[i]));
  }
  float m = fmaxf(__bfloat162float(m2.x), __bfloat162float(m2.y));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float wm[8];
  if ((threadIdx.x & 31) == 0) wm[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w) m = fmaxf(m, wm[w]);
    atomicMax(reinterpret_cast<int*>(rec), __float_as_int(m));   // non-negative floats order like their bit patterns
  }
}

constexpr int CT_ROWS = 128, CT_COLS = 64, CT_PITCH = 80;   // tile of the cast kernel; smem row pitch keeps 16-byte alignment

template <int FMT>
__device__ __forceinline__ uint32_t cvt4(float a, float b, float c, float d) {
  constexpr __nv_fp8_interpretation_t kind = FMT == FP8_E4M3 ? __NV_E4M3 : __NV_E5M2;
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, kind);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, kind);
  return lo | (hi << 16);
}

template <int FMT>
__global__ void __launch_bounds__(256) cast_kernel(const __nv_bfloat16* __restrict__ x, long ld, long rows, long cols,
                                                   float* __restrict__ rec, uint8_t* __restrict__ out_rm, long ld_rm,
                                                   uint8_t* __restrict__ out_t, long ld_t) {
  __shared__ __align__(16) uint8_t tile[CT_ROWS * CT_PITCH];
  constexpr float kMax = FMT == FP8_E4M3 ? 448.f : 57344.f;
  const float amax = fmaxf(rec[0], 1e-12f);
  const float s = __fdiv_rn(kMax, amax);   // correctly rounded whatever the compiler's fast-math setting: the host emulation must agree
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) rec[1] = __fdiv_rn(amax, kMax);
  const long row0 = (long)blockIdx.y * CT_ROWS, col0 = (long)blockIdx.x * CT_COLS;
#pragma unroll
  for (int h = 0; h < 4; ++h) {
    const int r = (threadIdx.x >> 3) + 32 * h, c = (threadIdx.x & 7) * 8;
    const long row = row0 + r, col = col0 + c;
    uint2 q = make_uint2(0u, 0u);
    if (row < rows && col < cols) {   // cols is a multiple of 8: a vector is inside or outside as a whole
      const uint4 v = *reinterpret_cast<const uint4*>(x + row * ld + col);
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&v);
      const float2 f0 = __bfloat1622float2(b2[0]), f1 = __bfloat1622float2(b2[1]), f2 = __bfloat1622float2(b2[2]),
                   f3 = __bfloat1622float2(b2[3]);
      q.x = cvt4<FMT>(f0.x * s, f0.y * s, f1.x * s, f1.y * s);
      q.y = cvt4<FMT>(f2.x * s, f2.y * s, f3.x * s, f3.y * s);
      if (out_rm != nullptr) *reinterpret_cast<uint2*>(out_rm + row * ld_rm + col) = q;
    }
    *reinterpret_cast<uint2*>(tile + r * CT_PITCH + c) = q;
  }
  if (out_t == nullptr) return;
  __syncthreads();
  // thread (column, quarter): 32 consecutive rows of one column = 32 contiguous bytes of the transpose
  const int c = threadIdx.x & 63, part = threadIdx.x >> 6;
  const long col = col0 + c, row = row0 + part * 32;
  if (col < cols && row < rows) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      uint32_t v = 0;
#pragma unroll
      for (int j = 0; j < 4; ++j) v |= (uint32_t)tile[(part * 32 + i * 4 + j) * CT_PITCH + c] << (8 * j);
      w[i] = v;
    }
    uint8_t* dst = out_t + col * ld_t + row;
    // ld_t is a multiple of 16 that covers `rows`, so whole 16-byte groups stay inside the row of the transpose
    *reinterpret_cast<uint4*>(dst) = make_uint4(w[0], w[1], w[2], w[3]);
    if (row + 16 < ld_t) *reinterpret_cast<uint4*>(dst + 16) = make_uint4(w[4], w[5], w[6], w[7]);
  }
}

// ------------------------------------------------------------------------------------------------ GEMM
constexpr int BM = 128, BN = 256, BK = 128, STAGES = 4, UMMA_K = 32;   // BK, UMMA_K in bytes = elements
constexpr int NUM_THREADS = 192, GROUP_M = 16;
constexpr int kABytes = BM * BK, kBBytes = BN * BK, kStageBytes = kABytes + kBBytes;
constexpr int kOutOffset = STAGES * kStageBytes;   // epilogue staging: 4 warps x 2 buffers x [32 rows][128 B]
constexpr int kOutBytes = 4 * 2 * 4096;
constexpr int kBarOffset = kOutOffset + kOutBytes;
constexpr int kSmemTotal = kBarOffset + 256 + 1024;   // + barriers + slack for 1024-byte alignment

struct Fp8Params {
  int M, N, K;
  int accumulate;
  int k_splits, kb_per_split;   // with accumulate: the K range in parts, every part a work item that adds its tile into D
  const float* rec_a;           // rec[1]: the factor that undoes the operand's scaling
  const float* rec_b;
  uint32_t idesc;
  int* status;
};

// instruction descriptor of kind::f8f6f4: fp32 accumulator, the two operand formats (0 = e4m3, 1 = e5m2), both K-major
constexpr uint32_t make_idesc_f8(int m, int n, int a_fmt, int b_fmt) {
  return (1u << 4) | ((uint32_t)a_fmt << 7) | ((uint32_t)b_fmt << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

template <int ACC>
__device__ __forceinline__ void umma_f8_ss(uint32_t tmem_d, SmemDesc a, SmemDesc b, uint32_t idesc, uint32_t flag = 0) {
  if constexpr (ACC == 2) {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %5, p;\n\t}"
                 ::"r"(tmem_d), "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi), "r"(idesc), "r"(flag) : "memory");
  } else {
    asm volatile("{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\tsetp.ne.b32 p, %6, 0;\n\tmov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %5, p;\n\t}"
                 ::"r"(tmem_d), "r"(a.lo), "r"(a.hi), "r"(b.lo), "r"(b.hi), "r"(idesc), "n"(ACC) : "memory");
  }
}

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_fp8_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_d, Fp8Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.N + BN - 1) / BN, tiles_m = (p.M + BM - 1) / BM;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_items = num_tiles * p.k_splits;
  constexpr int TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 4); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_d);
  }
  if (warp == 1) tmem_alloc<TMEM_COLS>(tmem_slot);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        const int ks = item / num_tiles, tile = item - ks * num_tiles;
        const int kb_lo = p.k_splits > 1 ? ks * p.kb_per_split : 0;
        const int kb_hi = p.k_splits > 1 ? min(num_kb, kb_lo + p.kb_per_split) : num_kb;
        int tm, tn;
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) { ok = false; break; }
          uint8_t* sa = smem + stage * kStageBytes;
          uint8_t* sb = sa + kABytes;
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          const int k0 = kb * BK;                                            // a multiple of 128 bytes
          tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);                // boxes {128 k-bytes, 128 rows}
          tma_load_2d(sb, &tmap_b, &full_bar[stage], k0, n0);
          tma_load_2d(sb + 16384, &tmap_b, &full_bar[stage], k0, n0 + 128);  // outside the matrix: zero fill
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = p.idesc;
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        const int ks = item / num_tiles;
        const int kb_lo = p.k_splits > 1 ? ks * p.kb_per_split : 0;
        const int kb_hi = p.k_splits > 1 ? min(num_kb, kb_lo + p.kb_per_split) : num_kb;
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrTimeoutFull)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * kStageBytes);
          const SmemDesc a0 = make_desc(sa, 16, 1024), b0 = make_desc(sa + kABytes, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const SmemDesc ad = desc_off(a0, k * 32), bd = desc_off(b0, k * 32);
            if (k == 0) umma_f8_ss<2>(d_tmem, ad, bd, idesc, (uint32_t)(kb - kb_lo));   // the first k-block of a tile overwrites
            else umma_f8_ss<1>(d_tmem, ad, bd, idesc);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const float scale = p.rec_a[1] * p.rec_b[1];
    int it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++it) {
      const int tile = item % num_tiles;
      int tm, tn;
      tile_coords(tile, tiles_m, tiles_n, tm, tn);
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, kErrTimeoutTmemFull)) { ok = false; break; }
      tc_fence_after();
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      uint8_t* stage = smem + kOutOffset + q * 8192;
#pragma unroll 1
      for (int c = 0; c < BN / 64; ++c) {
        const int col0 = n0 + c * 64;
        if (col0 >= p.N) break;
        uint8_t* buf = stage + (c & 1) * 4096;
        if (lane == 0) tma_store_wait_read<1>();  // the store issued two slabs ago has finished reading this buffer
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 64 + h * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            uint4 pk;
            uint32_t* w = reinterpret_cast<uint32_t*>(&pk);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              w[j] = pack_bf16x2(__uint_as_float(r[t * 8 + 2 * j]) * scale, __uint_as_float(r[t * 8 + 2 * j + 1]) * scale);
            const int ci = h * 4 + t;
            *reinterpret_cast<uint4*>(buf + lane * 128 + ((ci ^ (lane & 7)) << 4)) = pk;
          }
        }
        fence_async_proxy();
        __syncwarp();
        if (lane == 0) {
          if (p.accumulate) tma_reduce_add_2d(&tmap_d, buf, col0, tm * BM + q * 32);
          else tma_store_2d(&tmap_d, buf, col0, tm * BM + q * 32);
          tma_store_commit();
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  // ---------------------------------------------------------------- teardown
  if (warp >= 2 && lane == 0) tma_store_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give copies that are still in flight time to land before the smem goes away
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

bool split_k_enabled() {
  static const bool on = [] { const char* e = getenv("VLMT_GEMM_SPLITK"); return !(e && e[0] == '0'); }();
  return on;
}
}  // namespace

extern "C" int vlmt_fp8_amax(const void* x, long ld, long rows, long cols, float* rec, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(x) & 15)) return -2;
  cudaError_t e = cudaMemsetAsync(rec, 0, 2 * sizeof(float), stream);
  if (e != cudaSuccess) return (int)e;
  const long nvec = rows * (cols / 8);
  const int grid = (int)((nvec + 255) / 256 < 1184 ? (nvec + 255) / 256 : 1184);   // 8 blocks per SM
  amax_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ld, rows, (int)(cols / 8), rec);
  return (int)cudaGetLastError();
}

extern "C" int vlmt_fp8_cast(const void* x, long ld, long rows, long cols, float* rec, int format, void* out_rm, long ld_rm, void* out_t,
                             long ld_t, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  if ((cols & 7) || (ld & 7) || (reinterpret_cast<uintptr_t>(x) & 15)) return -2;
  if (out_rm != nullptr && ((ld_rm & 7) || ld_rm < cols || (reinterpret_cast<uintptr_t>(out_rm) & 7))) return -3;
  if (out_t != nullptr && ((ld_t & 15) || ld_t < rows || (reinterpret_cast<uintptr_t>(out_t) & 15))) return -4;
  const dim3 grid((unsigned)((cols + CT_COLS - 1) / CT_COLS), (unsigned)((rows + CT_ROWS - 1) / CT_ROWS));
  if (grid.y > 65535u) return -5;
  auto* xp = reinterpret_cast<const __nv_bfloat16*>(x);
  auto* rm = reinterpret_cast<uint8_t*>(out_rm);
  auto* tp = reinterpret_cast<uint8_t*>(out_t);
  if (format == FP8_E4M3) cast_kernel<FP8_E4M3><<<grid, 256, 0, stream>>>(xp, ld, rows, cols, rec, rm, ld_rm, tp, ld_t);
  else if (format == FP8_E5M2) cast_kernel<FP8_E5M2><<<grid, 256, 0, stream>>>(xp, ld, rows, cols, rec, rm, ld_rm, tp, ld_t);
  else return -6;
  return (int)cudaGetLastError();
}

extern "C" int vlmt_gemm_fp8(const void* A, const void* B, void* D, int M, int N, int K, long lda, long ldb, long ldd, int a_format,
                             int b_format, const float* rec_a, const float* rec_b, int accumulate, int* status, int num_sms,
                             cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 15) || (ldb & 15) || (ldd & 7)) return -2;   // TMA needs 16-byte row strides
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (reinterpret_cast<uintptr_t>(D) & 15)) return -3;
  if ((a_format != FP8_E4M3 && a_format != FP8_E5M2) || (b_format != FP8_E4M3 && b_format != FP8_E5M2)) return -6;
  CUtensorMap ta, tb, td;
  int r = vlmt_make_tmap_2d_u8(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda, 128, 128);
  if (r) return 1000 + r;
  r = vlmt_make_tmap_2d_u8(&tb, B, (uint64_t)K, (uint64_t)N, (uint64_t)ldb, 128, 128);
  if (r) return 2000 + r;
  r = vlmt_make_tmap_2d_bf16(&td, D, (uint64_t)N, (uint64_t)M, (uint64_t)ldd * 2, 64, 32);
  if (r) return 3000 + r;
  Fp8Params p;
  p.M = M; p.N = N; p.K = K;
  p.accumulate = accumulate;
  p.rec_a = rec_a; p.rec_b = rec_b;
  p.idesc = make_idesc_f8(BM, BN, a_format, b_format);
  p.status = status;
  p.k_splits = 1; p.kb_per_split = 0;
  const long tiles = (long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if (accumulate && split_k_enabled()) {
    // few output tiles and a long K: cut K so that the work items fill whole waves of SMs (at least 2048 of K per part)
    const int num_kb = (K + BK - 1) / BK;
    auto wave_eff = [&](long items) { return (double)items / (double)(((items + num_sms - 1) / num_sms) * num_sms); };
    int best = 1;
    double best_eff = wave_eff(tiles);
    for (int sp : {2, 3, 4, 6, 8}) {
      if (num_kb / sp < 16) break;
      const double e = wave_eff(tiles * sp);
      if (e > best_eff + 0.04) { best = sp; best_eff = e; }
    }
    if (best > 1) {
      p.kb_per_split = (num_kb + best - 1) / best;
      p.k_splits = (num_kb + p.kb_per_split - 1) / p.kb_per_split;
    }
  }
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_fp8_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const long items = tiles * p.k_splits;
  const int grid = (int)(items < num_sms ? items : num_sms);
  gemm_fp8_kernel<<<grid, NUM_THREADS, kSmemTotal, stream>>>(ta, tb, td, p);
  return (int)cudaGetLastError();
}
