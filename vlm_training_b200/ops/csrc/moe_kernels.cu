// Mixture-of-experts routing and token permutation without a host round trip.
//
//   route      one warp per token: softmax over E experts, top-k (ties to the lower expert id), optional
//              renormalisation; writes weights [T,k] fp32 and expert ids [T,k] int32       (fwd + bwd)
//   plan       stable counting sort of the T*k slots by expert into a padded row layout in which every expert owns
//              whole 128-row tiles: tile prefix per expert (what the grouped GEMM reads), destination row of every
//              slot, and the slot held by every row (-1 for padding).  Deterministic: a slot's row depends only on
//              the routing, not on thread timing.
//   dispatch   rows[dest[slot]] = x[token(slot)] (padding rows zero)                       (also: backward of combine)
//   combine    out[t] = sum_j w[t,j] * rows[dest[t*k+j]] in slot order, fp32 accumulation  (also: backward of dispatch)
//
// With expert parallelism the same plan is built over the slots of ALL ranks of the group (every rank knows every
// rank's per-expert counts), dispatch stores a slot's row straight into the memory of the rank that owns the expert, and
// the owner stores the expert output back into the source rank's per-slot buffer (kernels at the end of this file).
#include "moe_kernels.h"

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {
typedef __nv_bfloat16 bf16;
constexpr int TILE = 128;
constexpr int MAX_E_PER_LANE = 16;  // E <= 512
constexpr int PLAN_THREADS = 256;
constexpr int PLAN_CHUNK = 2048;    // slots per block of the plan kernels

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---------------------------------------------------------------------------------------------------- route
// logits [T, E] (bf16 or fp32), E <= 512.  lane l holds experts l, l + 32, ...
template <typename LT>
__global__ void moe_route_fwd_kernel(const LT* __restrict__ logits, int T, int E, int k, int renorm, float* __restrict__ weights,
                                     int* __restrict__ experts, int* __restrict__ counts) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const LT* row = logits + (size_t)warp * E;
  float v[MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? (float)row[e] : -INFINITY;
    mx = fmaxf(mx, v[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    v[i] = (lane + 32 * i) < E ? __expf(v[i] - mx) : 0.f;   // unnormalised probabilities (>= 0)
    sum += v[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  float sel_sum = 0.f;
  float my_w = 0.f;
  int my_e = 0;
  for (int j = 0; j < k; ++j) {
    // arg max over the remaining experts, ties to the lower id
    float best = -1.f;
    int best_e = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best) { best = v[i]; best_e = e; }   // increasing e within a lane: first maximum wins
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
    }
    if ((best_e & 31) == lane) {                        // taken (static indices keep v in registers)
#pragma unroll
      for (int i = 0; i < MAX_E_PER_LANE; ++i) if (i == (best_e >> 5)) v[i] = -1.f;
    }
    if (lane == j) { my_w = best * inv; my_e = best_e; }
    sel_sum += best * inv;
  }
  if (lane < k) {
    weights[(size_t)warp * k + lane] = renorm ? my_w / sel_sum : my_w;
    experts[(size_t)warp * k + lane] = my_e;
    if (counts != nullptr) atomicAdd(counts + my_e, 1);
  }
}

// dlogits = p * (dp - sum p dp) with dp_e = dL/dp_e nonzero only on the selected experts:
//   renorm: w_j = p_j / S, S = sum of the selected p  ->  dp_j = (dw_j - sum_i dw_i w_i) / S;  else dp_j = dw_j
template <typename LT>
__global__ void moe_route_bwd_kernel(const LT* __restrict__ logits, const int* __restrict__ experts, const float* __restrict__ weights,
                                     const float* __restrict__ dweights, int T, int E, int k, int renorm, LT* __restrict__ dlogits) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (warp >= T) return;
  const LT* row = logits + (size_t)warp * E;
  float p[MAX_E_PER_LANE], dp[MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    p[i] = e < E ? (float)row[e] : -INFINITY;
    dp[i] = 0.f;
    mx = fmaxf(mx, p[i]);
  }
  mx = warp_max(mx);
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    p[i] = (lane + 32 * i) < E ? __expf(p[i] - mx) : 0.f;
    sum += p[i];
  }
  sum = warp_sum(sum);
  const float inv = 1.f / sum;
  // selected experts: lane j < k holds (e_j, w_j, dw_j)
  const int e_j = lane < k ? experts[(size_t)warp * k + lane] : -1;
  const float w_j = lane < k ? weights[(size_t)warp * k + lane] : 0.f;
  const float dw_j = lane < k ? dweights[(size_t)warp * k + lane] : 0.f;
  const float dot = warp_sum(dw_j * w_j);
  float S = 1.f;
  if (renorm) {
    float pj = 0.f;
    // p of my selected expert: held by lane (e_j & 31) at index e_j >> 5 -> recompute from the logit instead of a shuffle chain
    if (lane < k) pj = __expf((float)row[e_j] - mx) * inv;
    S = warp_sum(pj);
  }
  const float dpj = renorm ? (dw_j - dot) / S : dw_j;
  float pdp = warp_sum(lane < k ? (renorm ? (w_j * S) : w_j) * dpj : 0.f);   // sum_e p_e dp_e (p_j = w_j S under renorm)
  // scatter dp_j to the lane that owns expert e_j
  for (int j = 0; j < k; ++j) {
    const int e = __shfl_sync(0xffffffffu, e_j, j);
    const float d = __shfl_sync(0xffffffffu, dpj, j);
    if ((e & 31) == lane) {
#pragma unroll
      for (int i = 0; i < MAX_E_PER_LANE; ++i) if (i == (e >> 5)) dp[i] = d;
    }
  }
  LT* out = dlogits + (size_t)warp * E;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (e < E) out[e] = (LT)(p[i] * inv * (dp[i] - pdp));
  }
}

// ---------------------------------------------------------------------------------------------------- plan
// Pass 1: per-block histogram of the experts of its chunk of slots -> hist[block][E]
__global__ void moe_plan_hist_kernel(const int* __restrict__ experts, long n_slots, int E, int* __restrict__ hist) {
  extern __shared__ int sh[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) sh[e] = 0;
  __syncthreads();
  const long lo = (long)blockIdx.x * PLAN_CHUNK, hi = min(n_slots, lo + PLAN_CHUNK);
  for (long s = lo + threadIdx.x; s < hi; s += blockDim.x) atomicAdd(&sh[experts[s]], 1);
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[(size_t)blockIdx.x * E + e] = sh[e];
}

// Pass 2 (one block): hist[b][e] becomes the exclusive prefix over blocks; counts[e] the total; prefix[e] the first tile of
// expert e; prefix[E] the number of tiles in use.
__global__ void moe_plan_scan_kernel(int* __restrict__ hist, int n_blocks, int E, int* __restrict__ counts, int* __restrict__ prefix) {
  extern __shared__ int tiles[];
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int run = 0;
    for (int b = 0; b < n_blocks; ++b) {
      const int h = hist[(size_t)b * E + e];
      hist[(size_t)b * E + e] = run;
      run += h;
    }
    counts[e] = run;
    tiles[e] = (run + TILE - 1) / TILE;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) { prefix[e] = run; run += tiles[e]; }
    prefix[E] = run;
  }
}

// Pass 3: destination row of every slot = first row of its expert + slots of the same expert in earlier blocks + its
// stable rank inside the block (warps take turns in slot order; inside a warp the rank comes from match_any).
// row_base (optional): first row per expert given by the caller (expert parallelism: a row of the OWNER's buffer) instead of
// prefix[e] * 128.  Rows at or beyond cap_rows are not placed (dest = -1).  slot_of_row may be null.
__global__ void moe_plan_place_kernel(const int* __restrict__ experts, long n_slots, int E, const int* __restrict__ hist,
                                      const int* __restrict__ prefix, const int* __restrict__ row_base, long cap_rows,
                                      int* __restrict__ dest, int* __restrict__ slot_of_row) {
  extern __shared__ int cursor[];
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    cursor[e] = (row_base ? row_base[e] : prefix[e] * TILE) + hist[(size_t)blockIdx.x * E + e];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const long lo = (long)blockIdx.x * PLAN_CHUNK, hi = min(n_slots, lo + PLAN_CHUNK);
  for (long base = lo; base < hi; base += blockDim.x) {
    for (int w = 0; w < n_warps; ++w) {
      if (w == warp) {
        const long s = base + threadIdx.x;
        const bool live = s < hi;
        const int e = live ? experts[s] : -1 - lane;          // dead lanes match nobody
        const unsigned same = __match_any_sync(0xffffffffu, e);
        const int rank = __popc(same & ((1u << lane) - 1u));
        if (live) {
          const int row = cursor[e] + rank;
          const bool fits = row < cap_rows;
          dest[s] = fits ? row : -1;
          if (fits && slot_of_row != nullptr) slot_of_row[row] = (int)s;
        }
        __syncwarp();
        if (live && rank == 0) cursor[e] += __popc(same);      // one lane per expert advances the cursor
      }
      __syncthreads();
    }
  }
}

// ---------------------------------------------------------------------------------------------------- dispatch / combine
// rows[r, :] = scale(slot) * src[slot / k, :] for the slot held by row r, zero for padding; only rows of tiles in use.
// scale: optional per-slot factor (the routing weight in the backward of combine).  One warp per row, 16-byte vectors.
__global__ void moe_rows_from_tokens_kernel(const bf16* __restrict__ src, const int* __restrict__ slot_of_row, const int* __restrict__ prefix,
                                            int E, int k, int H, const float* __restrict__ scale, bf16* __restrict__ rows, long cap_rows) {
  const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long used = (long)prefix[E] * TILE;
  if (row >= used || row >= cap_rows) return;
  const int slot = slot_of_row[row];
  uint4* out = reinterpret_cast<uint4*>(rows + row * H);
  const int nvec = H >> 3;
  if (slot < 0) {
    for (int c = lane; c < nvec; c += 32) out[c] = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  const uint4* in = reinterpret_cast<const uint4*>(src + (size_t)(slot / k) * H);
  if (scale == nullptr) {
    for (int c = lane; c < nvec; c += 32) out[c] = in[c];
  } else {
    const float sc = scale[slot];
    for (int c = lane; c < nvec; c += 32) {
      uint4 v = in[c];
      __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f = __bfloat1622float2(p[i]);
        p[i] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
      }
      out[c] = v;
    }
  }
}

// out[t, :] = sum_j (w ? w[t*k+j] : 1) * rows[dest[t*k+j], :]   (fp32 accumulation, slot order); optionally also
// dw[t*k+j] = <g[t, :], rows[dest[t*k+j], :]>  (the routing-weight gradient, when g is given).  One warp per token.
__global__ void moe_tokens_from_rows_kernel(const bf16* __restrict__ rows, const int* __restrict__ dest, const float* __restrict__ w,
                                            int T, int k, int H, bf16* __restrict__ out, const bf16* __restrict__ g,
                                            float* __restrict__ dw) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (t >= T) return;
  const int nvec = H >> 3;
  for (int c0 = 0; c0 < nvec; c0 += 32) {
    const int c = c0 + lane;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (c < nvec && out != nullptr) {
      for (int j = 0; j < k; ++j) {
        const float wj = w ? w[(size_t)t * k + j] : 1.f;
        const uint4 v = reinterpret_cast<const uint4*>(rows + (size_t)dest[(size_t)t * k + j] * H)[c];
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(p[i]);
          acc[2 * i] += wj * f.x;
          acc[2 * i + 1] += wj * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
      reinterpret_cast<uint4*>(out + (size_t)t * H)[c] = o;
    }
  }
  if (g != nullptr && dw != nullptr) {
    for (int j = 0; j < k; ++j) {
      const bf16* r = rows + (size_t)dest[(size_t)t * k + j] * H;
      float dot = 0.f;
      for (int c = lane; c < nvec; c += 32) {
        const uint4 a = reinterpret_cast<const uint4*>(g + (size_t)t * H)[c], b = reinterpret_cast<const uint4*>(r)[c];
        const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 fa = __bfloat1622float2(pa[i]), fb = __bfloat1622float2(pb[i]);
          dot += fa.x * fb.x + fa.y * fb.y;
        }
      }
      dot = warp_sum(dot);
      if (lane == 0) dw[(size_t)t * k + j] = dot;
    }
  }
}

// ---------------------------------------------------------------------------------------------------- expert parallelism
constexpr int EP_MAX_RANKS = 16;
struct EpPtrs { void* p[EP_MAX_RANKS]; };

// counts[E] of this rank -> row `me` of every rank's count matrix [ep, E]
__global__ void ep_push_counts_kernel(const int* __restrict__ counts, int E, EpPtrs mats, int ep, int me) {
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < E * ep; i += gridDim.x * blockDim.x) {
    const int r = i / E, e = i - r * E;
    reinterpret_cast<int*>(mats.p[r])[(size_t)me * E + e] = counts[e];
  }
}

// One block.  counts_all [ep, E]: row s = slots per expert of source rank s.  Expert e lives on rank e / El; in the owner's
// buffer the rows of an expert are ordered by source rank, every expert padded to whole 128-row tiles.
//   row_base[e]      first row (in the owner's buffer) of THIS rank's slots of expert e
//   prefix_local     [El + 1] tile prefix of this rank's own experts (what the grouped GEMM reads)
//   tot_local        [El] rows per local expert (all sources)
// An owner whose rows exceed cap_rows sets status 200 (the sender side then drops the slots that do not fit).
__global__ void ep_plan_kernel(const int* __restrict__ counts_all, int ep, int E, int me, int cap_rows, int* __restrict__ row_base,
                               int* __restrict__ prefix_local, int* __restrict__ tot_local, int* __restrict__ status) {
  extern __shared__ int sh[];       // tot[E] | before[E] | tile_first[E]
  int* tot = sh;
  int* before = sh + E;
  int* tile_first = sh + 2 * E;
  const int El = E / ep;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < ep; ++s) {
      const int c = counts_all[(size_t)s * E + e];
      if (s < me) b += c;
      t += c;
    }
    tot[e] = t;
    before[e] = b;
  }
  __syncthreads();
  if ((int)threadIdx.x < ep) {
    const int o = threadIdx.x;
    int run = 0;
    for (int i = 0; i < El; ++i) {
      const int e = o * El + i;
      tile_first[e] = run;
      if (o == me) { prefix_local[i] = run; tot_local[i] = tot[e]; }
      run += (tot[e] + TILE - 1) / TILE;
    }
    if (o == me) prefix_local[El] = run;
    if ((long)run * TILE > cap_rows) atomicCAS(status, 0, 200);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) row_base[e] = tile_first[e] * TILE + before[e];
}

// One warp per slot: rows_of_owner[dest[slot], :] = scale[slot] * src[slot / k, :] and src_of_row[dest[slot]] = me * n_slots + slot
// (peer stores into the memory of the rank that owns the slot's expert).
__global__ void ep_dispatch_kernel(const bf16* __restrict__ src, const int* __restrict__ experts, const int* __restrict__ dest,
                                   const float* __restrict__ scale, long n_slots, int k, int H, int El, int me, EpPtrs rows, EpPtrs srcs) {
  const long slot = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (slot >= n_slots) return;
  const int row = dest[slot];
  if (row < 0) return;
  const int o = experts[slot] / El;
  const uint4* in = reinterpret_cast<const uint4*>(src + (size_t)(slot / k) * H);
  uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(rows.p[o]) + (size_t)row * H);
  const int nvec = H >> 3;
  if (scale == nullptr) {
    for (int c = lane; c < nvec; c += 32) out[c] = in[c];
  } else {
    const float sc = scale[slot];
    for (int c = lane; c < nvec; c += 32) {
      uint4 v = in[c];
      __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(p[i]);
        p[i] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
      }
      out[c] = v;
    }
  }
  if (lane == 0) reinterpret_cast<int*>(srcs.p[o])[row] = me * (int)n_slots + (int)slot;
}

// Owner side, after all sources have signalled: padding rows of every local expert's last tile -> zero, src_of_row -> -1.
// One block per local expert.
__global__ void ep_zero_padding_kernel(bf16* __restrict__ rows, int* __restrict__ src_of_row, const int* __restrict__ prefix_local,
                                       const int* __restrict__ tot_local, int H, long cap_rows) {
  const int e = blockIdx.x;
  const long first = (long)prefix_local[e] * TILE + tot_local[e];
  long last = (long)prefix_local[e + 1] * TILE;
  if (last > cap_rows) last = cap_rows;
  const int nvec = H >> 3;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  for (long r = first + warp; r < last; r += n_warps) {
    uint4* out = reinterpret_cast<uint4*>(rows + r * H);
    for (int c = lane; c < nvec; c += 32) out[c] = make_uint4(0u, 0u, 0u, 0u);
    if (lane == 0) src_of_row[r] = -1;
  }
}

// Owner side: every row that holds a slot goes back to its source: back_of_source[slot, :] = y[row, :].  One warp per row.
__global__ void ep_return_kernel(const bf16* __restrict__ y, const int* __restrict__ src_of_row, const int* __restrict__ prefix_local,
                                 int El, long n_slots, int H, long cap_rows, EpPtrs backs) {
  const long row = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  long used = (long)prefix_local[El] * TILE;
  if (used > cap_rows) used = cap_rows;
  if (row >= used) return;
  const int s = src_of_row[row];
  if (s < 0) return;
  const int rank = s / (int)n_slots;
  const long slot = s - (long)rank * n_slots;
  const uint4* in = reinterpret_cast<const uint4*>(y + row * H);
  uint4* out = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(backs.p[rank]) + slot * H);
  const int nvec = H >> 3;
  for (int c = lane; c < nvec; c += 32) out[c] = in[c];
}
}  // namespace

extern "C" {
int vlmt_moe_route_fwd(const void* logits, int logits_fp32, int T, int E, int k, int renorm, float* weights, int* experts, int* counts,
                       cudaStream_t st) {
  if (E > 32 * MAX_E_PER_LANE || k > 32 || k > E) return -1;
  if (T <= 0) return 0;
  const int blocks = (T + 7) / 8;
  if (logits_fp32) moe_route_fwd_kernel<float><<<blocks, 256, 0, st>>>((const float*)logits, T, E, k, renorm, weights, experts, counts);
  else moe_route_fwd_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)logits, T, E, k, renorm, weights, experts, counts);
  return (int)cudaGetLastError();
}
int vlmt_moe_route_bwd(const void* logits, int logits_fp32, const int* experts, const float* weights, const float* dweights, int T, int E,
                       int k, int renorm, void* dlogits, cudaStream_t st) {
  if (E > 32 * MAX_E_PER_LANE || k > 32 || k > E) return -1;
  if (T <= 0) return 0;
  const int blocks = (T + 7) / 8;
  if (logits_fp32)
    moe_route_bwd_kernel<float><<<blocks, 256, 0, st>>>((const float*)logits, experts, weights, dweights, T, E, k, renorm, (float*)dlogits);
  else
    moe_route_bwd_kernel<bf16><<<blocks, 256, 0, st>>>((const bf16*)logits, experts, weights, dweights, T, E, k, renorm, (bf16*)dlogits);
  return (int)cudaGetLastError();
}
int vlmt_moe_plan_blocks(long n_slots) { return (int)((n_slots + PLAN_CHUNK - 1) / PLAN_CHUNK); }
// stage 1: hist (scratch of plan_blocks(n_slots) * E ints, left as per-block exclusive prefixes), counts [E], prefix [E + 1]
int vlmt_moe_plan_count(const int* experts, long n_slots, int E, int* hist, int* counts, int* prefix, cudaStream_t st) {
  if (E > 4096) return -1;
  const int nb = vlmt_moe_plan_blocks(n_slots);
  if (nb > 0) moe_plan_hist_kernel<<<nb, PLAN_THREADS, E * sizeof(int), st>>>(experts, n_slots, E, hist);
  moe_plan_scan_kernel<<<1, 256, E * sizeof(int), st>>>(hist, nb, E, counts, prefix);
  return (int)cudaGetLastError();
}
// stage 2: dest [n_slots]; slot_of_row [cap_rows] (optional; set to -1 first); row_base (optional) replaces prefix * 128
int vlmt_moe_plan_place(const int* experts, long n_slots, int E, const int* hist, const int* prefix, const int* row_base, int* dest,
                        int* slot_of_row, long cap_rows, cudaStream_t st) {
  if (E > 4096) return -1;
  if (slot_of_row != nullptr) {
    cudaError_t e = cudaMemsetAsync(slot_of_row, 0xff, (size_t)cap_rows * sizeof(int), st);
    if (e != cudaSuccess) return (int)e;
  }
  const int nb = vlmt_moe_plan_blocks(n_slots);
  if (nb > 0)
    moe_plan_place_kernel<<<nb, PLAN_THREADS, E * sizeof(int), st>>>(experts, n_slots, E, hist, prefix, row_base, cap_rows, dest, slot_of_row);
  return (int)cudaGetLastError();
}
int vlmt_moe_plan(const int* experts, long n_slots, int E, int* hist, int* counts, int* prefix, int* dest, int* slot_of_row, long cap_rows,
                  cudaStream_t st) {
  int r = vlmt_moe_plan_count(experts, n_slots, E, hist, counts, prefix, st);
  if (r) return r;
  return vlmt_moe_plan_place(experts, n_slots, E, hist, prefix, nullptr, dest, slot_of_row, cap_rows, st);
}
int vlmt_moe_rows_from_tokens(const void* src, const int* slot_of_row, const int* prefix, int E, int k, int H, const float* scale, void* rows,
                              long cap_rows, cudaStream_t st) {
  if (H & 7) return -1;
  if (cap_rows <= 0) return 0;
  const long blocks = (cap_rows + 7) / 8;
  moe_rows_from_tokens_kernel<<<(unsigned)blocks, 256, 0, st>>>((const bf16*)src, slot_of_row, prefix, E, k, H, scale, (bf16*)rows, cap_rows);
  return (int)cudaGetLastError();
}
int vlmt_moe_tokens_from_rows(const void* rows, const int* dest, const float* w, int T, int k, int H, void* out, const void* g, float* dw,
                              cudaStream_t st) {
  if (H & 7) return -1;
  if (T <= 0) return 0;
  moe_tokens_from_rows_kernel<<<(T + 7) / 8, 256, 0, st>>>((const bf16*)rows, dest, w, T, k, H, (bf16*)out, (const bf16*)g, dw);
  return (int)cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ expert parallelism
static void fill(EpPtrs& d, void* const* p, int n) { for (int i = 0; i < n; ++i) d.p[i] = p[i]; }
int vlmt_ep_push_counts(const int* counts, int E, void* const* mats, int ep, int me, cudaStream_t st) {
  if (ep > EP_MAX_RANKS) return -1;
  EpPtrs m; fill(m, mats, ep);
  ep_push_counts_kernel<<<(E * ep + 255) / 256, 256, 0, st>>>(counts, E, m, ep, me);
  return (int)cudaGetLastError();
}
int vlmt_ep_plan(const int* counts_all, int ep, int E, int me, int cap_rows, int* row_base, int* prefix_local, int* tot_local, int* status,
                 cudaStream_t st) {
  if (ep > EP_MAX_RANKS || E % ep != 0 || E > 4096) return -1;
  ep_plan_kernel<<<1, 256, 3 * E * sizeof(int), st>>>(counts_all, ep, E, me, cap_rows, row_base, prefix_local, tot_local, status);
  return (int)cudaGetLastError();
}
int vlmt_ep_dispatch(const void* src, const int* experts, const int* dest, const float* scale, long n_slots, int k, int H, int El, int me,
                     void* const* rows, void* const* srcs, int ep, cudaStream_t st) {
  if (ep > EP_MAX_RANKS || (H & 7)) return -1;
  if (n_slots <= 0) return 0;
  EpPtrs r, s; fill(r, rows, ep); fill(s, srcs, ep);
  ep_dispatch_kernel<<<(unsigned)((n_slots + 7) / 8), 256, 0, st>>>((const bf16*)src, experts, dest, scale, n_slots, k, H, El, me, r, s);
  return (int)cudaGetLastError();
}
int vlmt_ep_zero_padding(void* rows, int* src_of_row, const int* prefix_local, const int* tot_local, int El, int H, long cap_rows,
                         cudaStream_t st) {
  ep_zero_padding_kernel<<<El, 256, 0, st>>>((bf16*)rows, src_of_row, prefix_local, tot_local, H, cap_rows);
  return (int)cudaGetLastError();
}
int vlmt_ep_return(const void* y, const int* src_of_row, const int* prefix_local, int El, long n_slots, int H, long cap_rows,
                   void* const* backs, int ep, cudaStream_t st) {
  if (ep > EP_MAX_RANKS || (H & 7)) return -1;
  EpPtrs b; fill(b, backs, ep);
  ep_return_kernel<<<(unsigned)((cap_rows + 7) / 8), 256, 0, st>>>((const bf16*)y, src_of_row, prefix_local, El, n_slots, H, cap_rows, b);
  return (int)cudaGetLastError();
}
}
