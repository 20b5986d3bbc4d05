// Persistent bf16 GEMM for sm_100a:  D[M,N] (+)= A(M,K) * B(N,K)^T  with fp32 accumulation.
//
//   warp 0      TMA producer: per-CTA tiled loads (128-byte swizzle) into a 4-stage smem ring
//   warp 1      allocates TMEM, one lane issues tcgen05.mma (128 x BN x 16) into one of two
//               accumulator buffers, commits to the ring's "empty" barriers and to "tmem_full"
//   warps 2..5  epilogue: tcgen05.ld the finished accumulator (one row per thread), apply
//               bias / GELU / accumulate, convert to bf16, store
//
// Operand layouts (bf16):
//   A K-major : A stored [M, K] row-major      (activations in a forward linear, dY in dgrad)
//   A MN-major: A stored [K, M] row-major      (dY in wgrad: contraction over tokens)
//   B K-major : B stored [N, K] row-major      (weights W[out,in] in a forward linear)
//   B MN-major: B stored [K, N] row-major      (W in dgrad, X in wgrad)
// so one kernel covers forward (K,K), dgrad (K,MN) and wgrad (MN,MN) without transposes.
//
// The tile loop is static round-robin over a grouped raster (16 M-tiles per group) so the
// 148 concurrently resident tiles share A and B panels in L2.
//
// All-gather fused into the A operand (template flag AG; tensor-parallel column linear on sequence-sharded rows):
// every rank holds `rows` of the M dimension.  Two extra warps per CTA copy this rank's rows into the gathered
// buffer of EVERY rank (plain 16-byte stores into peer memory over NVLink) while the MMA pipeline already works on
// the tiles of the own rows, which it reads from the local source; the last CTA to finish its share stores the
// collective's number into every peer's flag array.  The TMA producer waits (bounded) for a peer's flag before it
// loads the first tile of that peer's rows from the LOCAL gathered buffer, so remote rows cross NVLink once and the
// transfer hides behind the own rows' tiles.
#include "sm100.cuh"

#include <stdlib.h>
#include "gemm_sm100.h"

#include <cuda_runtime.h>
#include <mutex>
#include <stdio.h>

namespace {
using namespace sm100;

constexpr int BM = 128, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int NUM_THREADS = 192;
constexpr int AG_PUSH_THREADS = 64;   // warps 6 and 7 of the all-gather variant
constexpr int GROUP_M = 16;
constexpr int MAX_RANKS = 8;

// wall-clock bound of a wait for a peer's flag inside the GEMM (set with vlmt_gemm_set_flag_wait_ms)
__device__ unsigned long long g_gemm_flag_wait_ns = 20000000000ull;

template <int BN>
struct SmemLayout {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kOutOffset = STAGES * kStageBytes;          // epilogue staging: 4 warps x 2 buffers x [32 rows][128 B]
  static constexpr int kOutBytes = 4 * 2 * 4096;
  static constexpr int kBarOffset = kOutOffset + kOutBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;  // + barriers + slack for 1024-B alignment
};

struct RsMaps { CUtensorMap m[MAX_RANKS]; };  // one tensor map per owner over its [rs_rows, N] destination block

struct Params {
  int M, N, K;
  int ldd;             // row stride of D in elements
  __nv_bfloat16* D;
  const __nv_bfloat16* bias;  // [N] or null
  float* Dacc32;       // optional fp32 destination (wgrad into fp32 main grads) or null
  int epilogue;        // GemmEpilogue
  int accumulate;      // D += result
  // split-K (needs accumulate + tma_store): the K range is cut into k_splits parts of kb_per_split k-blocks; every part is
  // a work item of its own whose tile is ADDED to D by the memory system, so a GEMM with few output tiles but a long K
  // (weight gradients) fills all SMs
  int k_splits, kb_per_split;
  int tma_store;       // bf16 output goes through smem staging + TMA stores (coalesced, clipped at the edges)
  // GEMM -> reduce-scatter: output rows are owned by ranks in blocks of rs_rows; the tile for owner o is stored straight
  // into rs_dst[o] (a buffer in rank o's memory, reached over NVLink), so the transfer overlaps the remaining tiles
  int rs_world, rs_rows;
  __nv_bfloat16* rs_dst[MAX_RANKS];
  // all-gather -> GEMM (AG variant): M = ag_world * ag_rows; this rank's rows come from ag_src (tensor map tmap_a2), the
  // others from the local gathered buffer (tmap_a) once flags[r] >= ag_epoch
  int ag_world, ag_rank, ag_rows, ag_epoch;
  const uint4* ag_src;          // this rank's rows, contiguous [ag_rows, K]
  uint4* ag_dst[MAX_RANKS];     // the gathered buffer [M, K] of every rank (own included)
  int* ag_flag_dst[MAX_RANKS];  // flag array of every rank
  const int* ag_flags;          // this rank's flag array
  unsigned* ag_counter;         // local: CTAs that have finished their share of the push (reset by the last one)
  // parameter all-gather -> GEMM (AG variant, wg_world > 0): B is a weight [N, K] that lives at element wg_lo of a flat
  // parameter bucket sharded over wg_world ranks (wg_shard elements each).  Warps 6 and 7 copy every owner's part of the
  // weight from that owner's shard (peer loads) into the local whole bucket, owner by owner starting with this rank; the
  // TMA producer waits for the owners of a tile's weight rows before it loads them from LOCAL memory.
  int wg_world, wg_rank, wg_epoch;
  long wg_shard, wg_lo;
  const __nv_bfloat16* wg_src[MAX_RANKS];   // shard base of every rank
  __nv_bfloat16* wg_dst;                    // local bucket base
  int* wg_flags;                            // local: wg_flags[o] = wg_epoch once owner o's part is here
  unsigned* wg_counters;                    // local, one per owner
  // Grouped GEMM (one launch for all experts of a MoE layer).  Rows of every group are padded to whole 128-row tiles
  // and laid out back to back; grp_prefix[g] (device memory, G + 1 ints) is the first tile of group g.
  //   grp_mode 1 (forward / dgrad): groups partition the M dimension; group g multiplies its rows with its own B
  //                                 (B rows g * grp_b_rows ...).  The number of M tiles is read from grp_prefix[G].
  //   grp_mode 2 (wgrad):           groups partition the K dimension (the padded rows); group g produces its own
  //                                 [M, N] output at D rows g * M ...; an empty group writes zeros.
  const int* grp_prefix;
  int grp_count, grp_mode, grp_b_rows;
  int* status;
};

// group that owns M tile `tm`: largest g with prefix[g] <= tm
__device__ __forceinline__ int group_of_tile(const int* __restrict__ prefix, int G, int tm) {
  int lo = 0, hi = G - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (prefix[mid] <= tm) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float gelu_tanh_f(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float u = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.f + erff(x * 0.7071067811865476f)); }

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int per_group = GROUP_M * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsz = min(GROUP_M, tiles_m - first_m);
  const int r = tile - g * per_group;
  tm = first_m + r % gsz;
  tn = r / gsz;
}

__device__ __forceinline__ int ld_acquire_sys_s32(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_16B(const void* p) {   // peer memory: never through a stale L1 line
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ void st_release_sys_s32(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

template <int BN, bool A_MN, bool B_MN, bool AG>
__global__ void __launch_bounds__(AG ? NUM_THREADS + AG_PUSH_THREADS : NUM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const __grid_constant__ CUtensorMap tmap_d, const __grid_constant__ CUtensorMap tmap_a2,
            const __grid_constant__ RsMaps rs_maps, Params p) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tmem_full = empty_bar + STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles_m = p.grp_mode == 1 ? p.grp_prefix[p.grp_count] : (p.M + BM - 1) / BM;
  const int tiles_per_group = tiles_m * tiles_n;                       // grp_mode 2: one [M, N] output per group
  const int num_tiles = p.grp_mode == 2 ? tiles_per_group * p.grp_count : tiles_per_group;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_items = num_tiles * p.k_splits;
  const int m_limit = p.grp_mode == 1 ? tiles_m * BM : p.M;           // rows that exist
  constexpr int TMEM_COLS = 2 * BN;  // 256 or 512: a power of two >= 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], 4); }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    if (AG) tma_prefetch_desc(&tmap_a2);
  }
  // AG: M tiles are visited starting with this rank's own block, so the peers' rows are needed as late as possible
  const int ag_rot = (AG && p.ag_world > 0) ? p.ag_rank * (p.ag_rows / BM) : 0;
  // weight gather: N tiles are visited starting with the first tile of this rank's own part of the weight
  int wg_rot = 0;
  if (AG && p.wg_world > 0) {
    const long own = (long)p.wg_rank * p.wg_shard - p.wg_lo;       // first element of the weight inside this rank's shard
    const long row = own <= 0 ? 0 : (own + p.K - 1) / p.K;
    wg_rot = (int)min((long)(tiles_n - 1), row / BN);
  }
  // the MMA thread and the epilogue depend on a producer that may be waiting for a peer: their own bound covers that wait
  const unsigned long long wait_ns = AG ? kWaitLimitNs + g_gemm_flag_wait_ns : kWaitLimitNs;
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
      uint32_t ag_ready = 0;  // AG: peers whose flag has been seen
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x) {
        int tile = item, tm, tn, kb_lo = 0, kb_hi = num_kb, b_row = 0;
        if (p.k_splits > 1) {
          const int ks = item / num_tiles;
          tile = item - ks * num_tiles;
          kb_lo = ks * p.kb_per_split;
          kb_hi = min(num_kb, kb_lo + p.kb_per_split);
        }
        if (p.grp_mode == 2) {
          const int g = tile / tiles_per_group;
          tile_coords(tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
          kb_lo = p.grp_prefix[g] * (BM / BK);
          kb_hi = p.grp_prefix[g + 1] * (BM / BK);
        } else {
          tile_coords(tile, tiles_m, tiles_n, tm, tn);
          if (p.grp_mode == 1) b_row = group_of_tile(p.grp_prefix, p.grp_count, tm) * p.grp_b_rows;
        }
        if (AG) { tm += ag_rot; if (tm >= tiles_m) tm -= tiles_m; tn += wg_rot; if (tn >= tiles_n) tn -= tiles_n; }
        const int m0 = tm * BM, n0 = tn * BN;
        bool own_rows = false;
        if (AG && p.wg_world > 0) {
          // owners of the weight rows [n0, n0 + BN): wait (bounded) until their parts are in the local bucket
          const long f_lo = p.wg_lo + (long)n0 * p.K, f_hi = p.wg_lo + (long)min(n0 + BN, p.N) * p.K;
          const int o_lo = (int)(f_lo / p.wg_shard), o_hi = (int)((f_hi - 1) / p.wg_shard);
          for (int o = o_lo; o <= o_hi && ok; ++o) {
            if ((ag_ready >> o) & 1u) continue;
            const unsigned long long t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (ld_acquire_sys_s32(p.wg_flags + o) < p.wg_epoch) {
              if ((++spins & 0xff) == 0) {
                if (*abort_flag) { ok = false; break; }
                if (globaltimer_ns() - t0 > g_gemm_flag_wait_ns) {
                  *abort_flag = 1;
                  atomicCAS(p.status, 0, 100 + o);
                  ok = false;
                  break;
                }
              }
            }
            if (ok) ag_ready |= 1u << o;
          }
          if (!ok) break;
          asm volatile("fence.proxy.async;" ::: "memory");  // written by ordinary stores of other CTAs, read through TMA
        }
        if (AG && p.ag_world > 0) {
          const int owner = m0 / p.ag_rows;
          own_rows = owner == p.ag_rank;
          if (!own_rows && !((ag_ready >> owner) & 1u)) {
            // first tile of this peer's rows: wait until its push has landed in the local gathered buffer
            const unsigned long long t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (ld_acquire_sys_s32(p.ag_flags + owner) < p.ag_epoch) {
              if ((++spins & 0xff) == 0) {
                if (*abort_flag) { ok = false; break; }
                if (globaltimer_ns() - t0 > g_gemm_flag_wait_ns) {
                  *abort_flag = 1;
                  atomicCAS(p.status, 0, 100 + owner);
                  ok = false;
                  break;
                }
              }
            }
            if (!ok) break;
            asm volatile("fence.proxy.async;" ::: "memory");  // the peer's stores are read through the async proxy (TMA)
            ag_ready |= 1u << owner;
          }
        }
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1, abort_flag, p.status, kErrTimeoutEmpty)) { ok = false; break; }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          const int k0 = kb * BK;
          if (!A_MN) {
            if (AG && own_rows) tma_load_2d(sa, &tmap_a2, &full_bar[stage], k0, m0 - p.ag_rank * p.ag_rows);
            else tma_load_2d(sa, &tmap_a, &full_bar[stage], k0, m0);          // box {64 k, 128 m}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)                                    // boxes {64 m, 64 k}
              tma_load_2d(sa + j * 8192, &tmap_a, &full_bar[stage], m0 + 64 * j, k0);
          }
          if (!B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 128; ++j)                                   // boxes {64 k, 128 n}
              tma_load_2d(sb + j * 16384, &tmap_b, &full_bar[stage], k0, b_row + n0 + 128 * j);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)                                    // boxes {64 n, 64 k}
              tma_load_2d(sb + j * 8192, &tmap_b, &full_bar[stage], n0 + 64 * j, b_row + k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN, B_MN);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1, abort_flag, p.status, kErrTimeoutTmemEmpty, wait_ns)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int tile = item, kb_lo = 0, kb_hi = num_kb;
        if (p.k_splits > 1) {
          const int ks = item / num_tiles;
          tile = item - ks * num_tiles;
          kb_lo = ks * p.kb_per_split;
          kb_hi = min(num_kb, kb_lo + p.kb_per_split);
        }
        if (p.grp_mode == 2) {
          const int g = tile / tiles_per_group;
          kb_lo = p.grp_prefix[g] * (BM / BK);
          kb_hi = p.grp_prefix[g + 1] * (BM / BK);
        }
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, abort_flag, p.status, kErrTimeoutFull, wait_ns)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t sb = sa + L::kABytes;
          const SmemDesc a0 = A_MN ? make_desc(sa, 8192, 1024) : make_desc(sa, 16, 1024);
          const SmemDesc b0 = B_MN ? make_desc(sb, 8192, 1024) : make_desc(sb, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const SmemDesc ad = desc_off(a0, A_MN ? k * 2048 : k * 32), bd = desc_off(b0, B_MN ? k * 2048 : k * 32);
            if (k == 0) umma_ss<2>(d_tmem, ad, bd, idesc, (uint32_t)(kb - kb_lo));   // the first k-block of a tile overwrites
            else umma_ss<1>(d_tmem, ad, bd, idesc);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
  } else if (AG && warp >= 6 && p.wg_world > 0) {
    // ------------------------------------------------------------ weight gather (warps 6, 7): peer shards -> local bucket
    const int t = threadIdx.x - NUM_THREADS;
    const long stride = (long)gridDim.x * AG_PUSH_THREADS;
    const long w_hi = p.wg_lo + (long)p.N * p.K;
    for (int step = 0; step < p.wg_world; ++step) {
      const int o = (p.wg_rank + step) % p.wg_world;
      const long lo = max(p.wg_lo, (long)o * p.wg_shard), hi = min(w_hi, (long)(o + 1) * p.wg_shard);
      if (hi > lo) {
        const uint4* src = reinterpret_cast<const uint4*>(p.wg_src[o] + (lo - (long)o * p.wg_shard));
        uint4* dst = reinterpret_cast<uint4*>(p.wg_dst + lo);
        const long nvec = (hi - lo) >> 3;
        long i = (long)blockIdx.x * AG_PUSH_THREADS + t;
        for (; i + 7 * stride < nvec; i += 8 * stride) {   // eight 16-byte loads in flight per thread: the link's latency is long
          uint4 v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = ld_volatile_16B(src + i + u * stride);
#pragma unroll
          for (int u = 0; u < 8; ++u) dst[i + u * stride] = v[u];
        }
        for (; i < nvec; i += stride) dst[i] = ld_volatile_16B(src + i);
      }
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(AG_PUSH_THREADS) : "memory");
      if (t == 0) {
        const unsigned done = atomicAdd(p.wg_counters + o, 1u);
        if (done == gridDim.x - 1) {                           // every CTA's share of this owner's part has been stored
          p.wg_counters[o] = 0;                                // ready for the next launch (stream-ordered)
          __threadfence();
          st_release_sys_s32(p.wg_flags + o, p.wg_epoch);
        }
      }
    }
  } else if (AG && warp >= 6) {
    // ------------------------------------------------------------ all-gather push (warps 6, 7)
    // this rank's rows -> the gathered buffer of every rank; 16-byte vectors, four loads in flight per thread
    const long nvec = (long)p.ag_rows * p.K / 8;
    const long off = (long)p.ag_rank * nvec;
    const int t = threadIdx.x - NUM_THREADS;
    const long stride = (long)gridDim.x * AG_PUSH_THREADS;
    long i = (long)blockIdx.x * AG_PUSH_THREADS + t;
    for (; i + 3 * stride < nvec; i += 4 * stride) {
      const uint4 a = p.ag_src[i], b = p.ag_src[i + stride], c = p.ag_src[i + 2 * stride], d = p.ag_src[i + 3 * stride];
      for (int r = 0; r < p.ag_world; ++r) {
        uint4* dst = p.ag_dst[r] + off;
        dst[i] = a; dst[i + stride] = b; dst[i + 2 * stride] = c; dst[i + 3 * stride] = d;
      }
    }
    for (; i < nvec; i += stride) {
      const uint4 a = p.ag_src[i];
      for (int r = 0; r < p.ag_world; ++r) p.ag_dst[r][off + i] = a;
    }
    __threadfence_system();                                    // this thread's stores are visible system-wide
    asm volatile("bar.sync 1, %0;" ::"n"(AG_PUSH_THREADS) : "memory");
    if (t == 0) {
      const unsigned done = atomicAdd(p.ag_counter, 1u);
      if (done == gridDim.x - 1) {                             // every CTA's share has been stored
        *p.ag_counter = 0;                                     // ready for the next launch (stream-ordered)
        __threadfence_system();
        for (int r = 0; r < p.ag_world; ++r)
          if (r != p.ag_rank) st_release_sys_s32(p.ag_flag_dst[r] + p.ag_rank, p.ag_epoch);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    bool ok = true;
    for (int item = blockIdx.x; item < num_items && ok; item += gridDim.x, ++it) {
      const int tile = p.k_splits > 1 ? item % num_tiles : item;
      int tm, tn, d_row0 = 0;
      bool empty_group = false;   // grp_mode 2: no rows for this group, the accumulator was never written -> zeros
      if (p.grp_mode == 2) {
        const int g = tile / tiles_per_group;
        tile_coords(tile - g * tiles_per_group, tiles_m, tiles_n, tm, tn);
        d_row0 = g * p.M;
        empty_group = p.grp_prefix[g + 1] == p.grp_prefix[g];
      } else {
        tile_coords(tile, tiles_m, tiles_n, tm, tn);
      }
      if (AG) { tm += ag_rot; if (tm >= tiles_m) tm -= tiles_m; tn += wg_rot; if (tn >= tiles_n) tn -= tiles_n; }
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_phase, abort_flag, p.status, kErrTimeoutTmemFull, wait_ns)) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + q * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(q * 32) << 16);
      const bool row_ok = row < m_limit;
      if (p.tma_store) {
        // 64-column slabs: TMEM -> registers -> (bias / GELU) -> bf16 -> swizzled smem -> one TMA store per slab and warp
        uint8_t* stage = smem + L::kOutOffset + q * 8192;
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
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = empty_group ? 0.f : __uint_as_float(r[i]);
            if (p.bias != nullptr) {
#pragma unroll
              for (int i = 0; i < 32; ++i) if (col0 + h * 32 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + h * 32 + i]);
            }
            if (p.epilogue == GEMM_EPI_GELU_TANH) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_f(v[i]);
            } else if (p.epilogue == GEMM_EPI_GELU_ERF) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] = gelu_erf_f(v[i]);
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              uint4 pk;
              __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
              for (int j = 0; j < 4; ++j) p2[j] = __floats2bfloat162_rn(v[t * 8 + 2 * j], v[t * 8 + 2 * j + 1]);
              const int ci = h * 4 + t;
              *reinterpret_cast<uint4*>(buf + lane * 128 + ((ci ^ (lane & 7)) << 4)) = pk;
            }
          }
          fence_async_proxy();
          __syncwarp();
          if (lane == 0) {
            if (p.rs_world > 0) {  // the tile's rows belong to one owner (rs_rows is a multiple of the tile height)
              const int owner = (tm * BM) / p.rs_rows;
              tma_store_2d(&rs_maps.m[owner], buf, col0, tm * BM - owner * p.rs_rows + q * 32);
            } else if (p.accumulate) {
              tma_reduce_add_2d(&tmap_d, buf, col0, d_row0 + tm * BM + q * 32);
            } else {
              tma_store_2d(&tmap_d, buf, col0, d_row0 + tm * BM + q * 32);
            }
            tma_store_commit();
          }
        }
      } else {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        const int col0 = n0 + c * 32;
        if (row_ok && col0 < p.N) {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (p.bias != nullptr) {
#pragma unroll
            for (int i = 0; i < 32; ++i) if (col0 + i < p.N) v[i] += __bfloat162float(p.bias[col0 + i]);
          }
          if (p.epilogue == GEMM_EPI_GELU_TANH) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_tanh_f(v[i]);
          } else if (p.epilogue == GEMM_EPI_GELU_ERF) {
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = gelu_erf_f(v[i]);
          }
          if (p.Dacc32 != nullptr) {
            float* dst = p.Dacc32 + (size_t)row * p.ldd + col0;
            if (col0 + 32 <= p.N && (p.ldd & 3) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 4) {
                float4 o = p.accumulate ? *reinterpret_cast<float4*>(dst + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                o.x += v[i]; o.y += v[i + 1]; o.z += v[i + 2]; o.w += v[i + 3];
                *reinterpret_cast<float4*>(dst + i) = o;
              }
            } else {
              for (int i = 0; i < 32 && col0 + i < p.N; ++i) dst[i] = (p.accumulate ? dst[i] : 0.f) + v[i];
            }
          } else {
            __nv_bfloat16* dst;
            if (p.rs_world > 0) {
              const int owner = row / p.rs_rows;
              dst = p.rs_dst[owner] + (size_t)(row - owner * p.rs_rows) * p.ldd + col0;
            } else {
              dst = p.D + (size_t)row * p.ldd + col0;
            }
            if (col0 + 32 <= p.N && (p.ldd & 7) == 0) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                if (p.accumulate) {
                  uint4 old = *reinterpret_cast<const uint4*>(dst + i);
                  const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int j = 0; j < 4; ++j) { float2 f = __bfloat1622float2(o2[j]); v[i + 2 * j] += f.x; v[i + 2 * j + 1] += f.y; }
                }
                uint4 pk;
                __nv_bfloat162* p2 = reinterpret_cast<__nv_bfloat162*>(&pk);
#pragma unroll
                for (int j = 0; j < 4; ++j) p2[j] = __floats2bfloat162_rn(v[i + 2 * j], v[i + 2 * j + 1]);
                *reinterpret_cast<uint4*>(dst + i) = pk;
              }
            } else {
              for (int i = 0; i < 32 && col0 + i < p.N; ++i) {
                float o = p.accumulate ? __bfloat162float(dst[i]) : 0.f;
                dst[i] = __float2bfloat16(o + v[i]);
              }
            }
          }
        }
      }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

  // ---------------------------------------------------------------- teardown
  if (warp >= 2 && warp < 6 && lane == 0 && p.tma_store) tma_store_wait<0>();
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

// -------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

}  // namespace

// Tensor maps are pure functions of (base, shape, stride, box); training re-issues the same few hundred GEMM shapes on the
// same buffers every step, so the encoded maps are kept per thread and looked up instead of re-encoded.
#include <unordered_map>
namespace {
struct TmapKey {
  uint64_t base, inner, outer, stride;
  uint32_t box_inner, box_outer;
  int dtype;
  bool operator==(const TmapKey& o) const {
    return base == o.base && inner == o.inner && outer == o.outer && stride == o.stride && box_inner == o.box_inner &&
           box_outer == o.box_outer && dtype == o.dtype;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    uint64_t h = k.base * 0x9E3779B97F4A7C15ull;
    h ^= (k.inner + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.outer + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (k.stride + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= (((uint64_t)k.box_inner << 32 | k.box_outer) + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    h ^= ((uint64_t)k.dtype + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2));
    return (size_t)h;
  }
};
}  // namespace

namespace {
int make_tmap_2d(void* out_map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner,
                 uint32_t box_outer, CUtensorMapDataType dtype) {
  static thread_local std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const TmapKey key{reinterpret_cast<uint64_t>(base), inner, outer, row_stride_bytes, box_inner, box_outer, (int)dtype};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *reinterpret_cast<CUtensorMap*>(out_map) = it->second;
    return 0;
  }
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  // The encode call is a driver-API entry point and needs a current context on the calling thread.
  // Threads that only ever used the runtime API lazily (autograd workers) may not have bound the
  // primary context yet; cudaSetDevice on the current device binds it.
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -4;
    ctx_bound = true;
  }
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out_map), dtype, 2, const_cast<void*>(base), dims,
                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) {
    if (cache.size() > 16384) cache.clear();  // shapes that change every step (variable packing) must not grow it forever
    cache.emplace(key, *reinterpret_cast<CUtensorMap*>(out_map));
  }
  return (int)r;
}
}  // namespace

extern "C" int vlmt_make_tmap_2d_bf16(void* out_map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                                      uint32_t box_inner, uint32_t box_outer) {
  return make_tmap_2d(out_map, base, inner, outer, row_stride_bytes, box_inner, box_outer, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
}

// one byte per element (fp8 operands): inner extent, stride and box_inner are bytes
extern "C" int vlmt_make_tmap_2d_u8(void* out_map, const void* base, uint64_t inner, uint64_t outer, uint64_t row_stride_bytes,
                                    uint32_t box_inner, uint32_t box_outer) {
  return make_tmap_2d(out_map, base, inner, outer, row_stride_bytes, box_inner, box_outer, CU_TENSOR_MAP_DATA_TYPE_UINT8);
}

// 3-D tensor map [d2][d1][d0] (d0 innermost, contiguous) with byte strides for d1 and d2, 128-byte swizzle, zero fill
// outside the tensor.  Not cached: the callers (attention) build a handful per launch.
extern "C" int vlmt_make_tmap_3d_bf16(void* out_map, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1_bytes,
                                      uint64_t stride2_bytes, uint32_t box0, uint32_t box1, uint32_t box2) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) return -4;
    ctx_bound = true;
  }
  if ((stride1_bytes & 15) || (stride2_bytes & 15) || (reinterpret_cast<uintptr_t>(base) & 15)) return -5;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out_map), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

namespace {
// Everything one launch needs besides the plain GEMM arguments; passed explicitly down to the launcher.
struct GemmExtras {
  // GEMM -> reduce-scatter: output rows owned by rank o (blocks of rs_rows) are stored into rs_dst[o]
  int rs_world = 0, rs_rows = 0;
  void* const* rs_dst = nullptr;
  // grouped GEMM
  const int* grp_prefix = nullptr;
  int grp_count = 0, grp_mode = 0, grp_b_rows = 0;
  // all-gather -> GEMM
  int ag_world = 0, ag_rank = 0, ag_rows = 0, ag_epoch = 0;
  const void* ag_src = nullptr;
  void* const* ag_dst = nullptr;
  void* const* ag_flag_dst = nullptr;
  const int* ag_flags = nullptr;
  unsigned* ag_counter = nullptr;
  // parameter all-gather -> GEMM
  int wg_world = 0, wg_rank = 0, wg_epoch = 0;
  long wg_shard = 0, wg_lo = 0;
  const void* const* wg_src = nullptr;
  void* wg_dst = nullptr;
  int* wg_flags = nullptr;
  unsigned* wg_counters = nullptr;
};

bool split_k_enabled() {
  static const bool on = [] { const char* e = getenv("VLMT_GEMM_SPLITK"); return !(e && e[0] == '0'); }();
  return on;
}

template <int BN, bool A_MN, bool B_MN, bool AG>
int launch_variant(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& td, const CUtensorMap& ta2, const RsMaps& rsm,
                   const Params& p, int num_sms, cudaStream_t stream) {
  using L = SmemLayout<BN>;
  auto kern = gemm_kernel<BN, A_MN, B_MN, AG>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN) * (p.grp_mode == 2 ? p.grp_count : 1) * p.k_splits;
  const int grid = tiles < num_sms ? tiles : num_sms;   // grp_mode 1: p.M is the row capacity, an upper bound
  kern<<<grid, AG ? NUM_THREADS + AG_PUSH_THREADS : NUM_THREADS, L::kTotal, stream>>>(ta, tb, td, ta2, rsm, p);
  return (int)cudaGetLastError();
}

int gemm_launch(const void* A, const void* B, void* D, float* Dacc32, const void* bias, int M, int N, int K, int lda, int ldb, int ldd,
                int a_mn_major, int b_mn_major, int epilogue, int accumulate, const GemmExtras& x, int* status, int num_sms,
                cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda & 7) || (ldb & 7)) return -2;  // TMA needs 16-byte row strides
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -3;
  CUtensorMap ta, tb;
  int r;
  if (!a_mn_major) r = vlmt_make_tmap_2d_bf16(&ta, A, (uint64_t)K, (uint64_t)M, (uint64_t)lda * 2, 64, 128);
  else r = vlmt_make_tmap_2d_bf16(&ta, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda * 2, 64, 64);
  if (r) return 1000 + r;
  const bool bn256 = N > 128;
  const uint64_t b_groups = x.grp_mode == 1 ? (uint64_t)x.grp_count : 1;   // grouped forward / dgrad: one B per group, stacked along the rows
  if (!b_mn_major) r = vlmt_make_tmap_2d_bf16(&tb, B, (uint64_t)K, (uint64_t)N * b_groups, (uint64_t)ldb * 2, 64, 128);
  else r = vlmt_make_tmap_2d_bf16(&tb, B, (uint64_t)N, (uint64_t)K * b_groups, (uint64_t)ldb * 2, 64, 64);
  if (r) return 2000 + r;
  Params p;
  CUtensorMap td = ta, ta2 = ta;  // placeholders where the direct-store epilogue / a single A source is used
  static const RsMaps kNoRsMaps = {};
  RsMaps rsm_local;
  const RsMaps* rsm = &kNoRsMaps;
  p.tma_store = 0;
  p.rs_world = 0; p.rs_rows = 0;
  if (x.rs_world > 0) {
    p.rs_world = x.rs_world; p.rs_rows = x.rs_rows;
    for (int i = 0; i < x.rs_world; ++i) p.rs_dst[i] = reinterpret_cast<__nv_bfloat16*>(x.rs_dst[i]);
    // whole 64-column slabs go out as TMA stores into the owners' memory (large NVLink writes); the per-thread 16-byte
    // stores of the direct epilogue are kept as the fallback
    if (Dacc32 == nullptr && !accumulate && !bias && epilogue == GEMM_EPI_NONE && (ldd & 7) == 0) {
      bool maps_ok = true;
      for (int i = 0; i < x.rs_world && maps_ok; ++i) {
        if (reinterpret_cast<uintptr_t>(x.rs_dst[i]) & 15) maps_ok = false;
        else if (vlmt_make_tmap_2d_bf16(&rsm_local.m[i], x.rs_dst[i], (uint64_t)N, (uint64_t)x.rs_rows, (uint64_t)ldd * 2, 64, 32))
          maps_ok = false;
      }
      if (maps_ok) {
        for (int i = x.rs_world; i < MAX_RANKS; ++i) rsm_local.m[i] = rsm_local.m[0];
        rsm = &rsm_local;
        p.tma_store = 1;
      }
    }
  }
  // with `accumulate` the slabs go out as TMA reduce-adds (bf16 addition in the memory system), so a weight gradient can
  // be added straight into the optimizer's gradient buffer without reading it back into the SM
  if (x.rs_world == 0 && Dacc32 == nullptr && (ldd & 7) == 0 && (reinterpret_cast<uintptr_t>(D) & 15) == 0) {
    const uint64_t d_rows = x.grp_mode == 2 ? (uint64_t)M * x.grp_count : (uint64_t)M;
    r = vlmt_make_tmap_2d_bf16(&td, D, (uint64_t)N, d_rows, (uint64_t)ldd * 2, 64, 32);
    if (r == 0) p.tma_store = 1;
  }
  p.M = M; p.N = N; p.K = K; p.ldd = ldd;
  p.grp_prefix = x.grp_prefix; p.grp_count = x.grp_count; p.grp_mode = x.grp_mode; p.grp_b_rows = x.grp_b_rows;
  if (p.grp_mode == 2 && !p.tma_store) return -30;  // grouped wgrad writes through the TMA-store epilogue only
  p.D = reinterpret_cast<__nv_bfloat16*>(D);
  p.bias = reinterpret_cast<const __nv_bfloat16*>(bias);
  p.Dacc32 = Dacc32;
  p.epilogue = epilogue; p.accumulate = accumulate; p.status = status;
  p.k_splits = 1; p.kb_per_split = 0;
  if (accumulate && p.tma_store && x.grp_mode == 0 && x.rs_world == 0 && x.ag_world == 0 && bias == nullptr && epilogue == GEMM_EPI_NONE &&
      Dacc32 == nullptr && split_k_enabled()) {
    // few output tiles and a long K: cut K so that the work items fill whole waves of SMs (at least 1024 of K per part)
    const long tiles = (long)((M + BM - 1) / BM) * ((N + (bn256 ? 256 : 128) - 1) / (bn256 ? 256 : 128));
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
  p.ag_world = 0; p.ag_rank = 0; p.ag_rows = 0; p.ag_epoch = 0;
  p.ag_src = nullptr; p.ag_flags = nullptr; p.ag_counter = nullptr;
  p.wg_world = 0; p.wg_rank = 0; p.wg_epoch = 0; p.wg_shard = 0; p.wg_lo = 0; p.wg_dst = nullptr; p.wg_flags = nullptr; p.wg_counters = nullptr;
  if (x.wg_world > 0) {
    // the weight's rows are gathered inside the kernel: K-major B only, every owner's part a whole number of 16-byte vectors
    if (a_mn_major || b_mn_major || !bn256 || x.wg_world > MAX_RANKS || (x.wg_shard & 7) || (x.wg_lo & 7) || (((long)N * K) & 7) || ldb != K ||
        x.ag_world > 0 || x.rs_world > 0 || x.grp_mode != 0)
      return -41;
    p.wg_world = x.wg_world; p.wg_rank = x.wg_rank; p.wg_epoch = x.wg_epoch; p.wg_shard = x.wg_shard; p.wg_lo = x.wg_lo;
    for (int i = 0; i < x.wg_world; ++i) p.wg_src[i] = reinterpret_cast<const __nv_bfloat16*>(x.wg_src[i]);
    p.wg_dst = reinterpret_cast<__nv_bfloat16*>(x.wg_dst);
    p.wg_flags = x.wg_flags; p.wg_counters = x.wg_counters;
    return launch_variant<256, false, false, true>(ta, tb, td, ta2, *rsm, p, num_sms, stream);
  }
  if (x.ag_world > 0) {
    if (a_mn_major || !bn256 || x.ag_world > MAX_RANKS || x.ag_rows % BM != 0 || x.ag_rows * x.ag_world != M || (K & 7) ||
        (reinterpret_cast<uintptr_t>(x.ag_src) & 15))
      return -40;
    r = vlmt_make_tmap_2d_bf16(&ta2, x.ag_src, (uint64_t)K, (uint64_t)x.ag_rows, (uint64_t)K * 2, 64, 128);
    if (r) return 4000 + r;
    p.ag_world = x.ag_world; p.ag_rank = x.ag_rank; p.ag_rows = x.ag_rows; p.ag_epoch = x.ag_epoch;
    p.ag_src = reinterpret_cast<const uint4*>(x.ag_src);
    for (int i = 0; i < x.ag_world; ++i) {
      p.ag_dst[i] = reinterpret_cast<uint4*>(x.ag_dst[i]);
      p.ag_flag_dst[i] = reinterpret_cast<int*>(x.ag_flag_dst[i]);
    }
    p.ag_flags = x.ag_flags; p.ag_counter = x.ag_counter;
    if (!b_mn_major) return launch_variant<256, false, false, true>(ta, tb, td, ta2, *rsm, p, num_sms, stream);
    return launch_variant<256, false, true, true>(ta, tb, td, ta2, *rsm, p, num_sms, stream);
  }
#define DISPATCH(BN_)                                                                                                     \
  do {                                                                                                                    \
    if (!a_mn_major && !b_mn_major) return launch_variant<BN_, false, false, false>(ta, tb, td, ta2, *rsm, p, num_sms, stream); \
    if (!a_mn_major && b_mn_major) return launch_variant<BN_, false, true, false>(ta, tb, td, ta2, *rsm, p, num_sms, stream);   \
    if (a_mn_major && b_mn_major) return launch_variant<BN_, true, true, false>(ta, tb, td, ta2, *rsm, p, num_sms, stream);     \
    return launch_variant<BN_, true, false, false>(ta, tb, td, ta2, *rsm, p, num_sms, stream);                                  \
  } while (0)
  if (bn256) DISPATCH(256);
  DISPATCH(128);
#undef DISPATCH
}
}  // namespace

extern "C" int vlmt_gemm_bf16(const void* A, const void* B, void* D, float* Dacc32, const void* bias, int M, int N, int K,
                              int lda, int ldb, int ldd, int a_mn_major, int b_mn_major, int epilogue, int accumulate,
                              int* status, int num_sms, cudaStream_t stream) {
  return gemm_launch(A, B, D, Dacc32, bias, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, epilogue, accumulate, GemmExtras{}, status,
                     num_sms, stream);
}

// D rows [o * rows_per_rank, (o + 1) * rows_per_rank) are written to dst[o] (row stride ldd) instead of a local D:
// the producer half of a tensor-parallel GEMM -> reduce-scatter (the consumer sums the `world` partial blocks it received).
// B is K-major (a row-parallel forward linear) or MN-major (the input gradient of a column-parallel linear).
extern "C" int vlmt_gemm_bf16_rs_push(const void* A, const void* B, void* const* dst, int world, int rows_per_rank, int M, int N, int K,
                                      int lda, int ldb, int ldd, int b_mn_major, int* status, int num_sms, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rows_per_rank % BM != 0 || rows_per_rank * world != M) return -20;
  GemmExtras x;
  x.rs_world = world; x.rs_rows = rows_per_rank; x.rs_dst = dst;
  return gemm_launch(A, B, dst[0], nullptr, nullptr, M, N, K, lda, ldb, ldd, 0, b_mn_major, GEMM_EPI_NONE, 0, x, status, num_sms, stream);
}

// One launch for all groups (experts).  `prefix` (device, G + 1 ints): first 128-row tile of every group in the padded
// row layout.
//   mode 1: D[rows, N] = A[rows, K] x B_g  with A K-major [row_capacity, K]; B K-major [G * N, K] (forward) or
//           MN-major [G * K, N] (dgrad); M = row capacity (tiles beyond prefix[G] are not touched).
//   mode 2: D_g[M, N] = sum over the rows of group g of A[row, M]^T B[row, N]  (A, B MN-major, K = row capacity);
//           D is [G * M, N]; needs M % 128 == 0 and a 16-byte aligned D.
extern "C" int vlmt_gemm_bf16_grouped(const void* A, const void* B, void* D, const int* prefix, int groups, int mode, int M, int N, int K,
                                      int lda, int ldb, int ldd, int a_mn_major, int b_mn_major, int* status, int num_sms,
                                      cudaStream_t stream) {
  if (groups < 1 || (mode != 1 && mode != 2) || prefix == nullptr) return -31;
  if (mode == 1 && a_mn_major) return -32;
  if (mode == 2 && (!a_mn_major || !b_mn_major || (M % BM) != 0)) return -33;
  GemmExtras x;
  x.grp_prefix = prefix; x.grp_count = groups; x.grp_mode = mode;
  x.grp_b_rows = mode == 1 ? (b_mn_major ? K : N) : 0;
  return gemm_launch(A, B, D, nullptr, nullptr, M, N, K, lda, ldb, ldd, a_mn_major, b_mn_major, GEMM_EPI_NONE, 0, x, status, num_sms,
                     stream);
}

// All-gather fused into the GEMM: D[M, N] = gathered(A) x op(B) with M = world * rows.  This rank's rows `src` [rows, K]
// (contiguous) are copied by the kernel into gathered[r] + rank * rows * K for every rank r (gathered[rank] is the local
// buffer `A_full` [M, K], whose peer blocks the kernel reads once flags[r] >= epoch) and the collective's number `epoch`
// is stored into flag_dst[r][rank] of every peer when the copy is complete.  `counter`: one zero-initialised unsigned in
// local memory, shared by all launches of a stream.
extern "C" int vlmt_gemm_bf16_ag(const void* src, void* A_full, const void* B, void* D, void* const* gathered, void* const* flag_dst,
                                 const int* flags, unsigned* counter, int epoch, int world, int rank, int rows, int N, int K, int ldb,
                                 int ldd, int b_mn_major, int* status, int num_sms, cudaStream_t stream) {
  if (world < 1 || world > MAX_RANKS || rank < 0 || rank >= world || gathered[rank] != A_full) return -41;
  GemmExtras x;
  x.ag_world = world; x.ag_rank = rank; x.ag_rows = rows; x.ag_epoch = epoch;
  x.ag_src = src; x.ag_dst = gathered; x.ag_flag_dst = flag_dst; x.ag_flags = flags; x.ag_counter = counter;
  return gemm_launch(A_full, B, D, nullptr, nullptr, world * rows, N, K, K, ldb, ldd, 0, b_mn_major, GEMM_EPI_NONE, 0, x, status, num_sms,
                     stream);
}

extern "C" int vlmt_gemm_set_flag_wait_ms(long ms) {
  const unsigned long long ns = (unsigned long long)(ms < 1 ? 1 : ms) * 1000000ull;
  return (int)cudaMemcpyToSymbol(g_gemm_flag_wait_ns, &ns, sizeof(ns));
}

// Y[M, N] = X[M, K] . W^T where W [N, K] sits at element `w_lo` of a flat parameter bucket that is sharded over `world`
// ranks (`shard` elements each): the kernel copies every owner's part of W from `shard_ptrs[o]` (peer memory) into the
// local bucket `bucket` while its first tiles run on this rank's own part.  `flags` / `counters`: local int32 / uint32
// arrays of `world` entries (zero before the first use); `epoch` grows with every call that uses them.
extern "C" int vlmt_gemm_bf16_wgather(const void* X, void* D, const void* bias, int M, int N, int K, int ldx, int ldd, void* bucket, long w_lo,
                                      const void* const* shard_ptrs, long shard, int world, int rank, int* flags, unsigned* counters,
                                      int epoch, int* status, int num_sms, cudaStream_t stream) {
  GemmExtras x;
  x.wg_world = world; x.wg_rank = rank; x.wg_epoch = epoch; x.wg_shard = shard; x.wg_lo = w_lo;
  x.wg_src = shard_ptrs; x.wg_dst = bucket; x.wg_flags = flags; x.wg_counters = counters;
  const void* W = reinterpret_cast<const __nv_bfloat16*>(bucket) + w_lo;
  return gemm_launch(X, W, D, nullptr, bias, M, N, K, ldx, K, ldd, 0, 0, GEMM_EPI_NONE, 0, x, status, num_sms, stream);
}
