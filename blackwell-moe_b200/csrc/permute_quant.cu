// Token permutation (stable counting sort by expert), segment amax / scales,
// gather + E4M3 quantisation, segment requantisation of h, weighted combine.
//
// Takes over the roles of the torch sort/bincount/cumsum/gather of
// src/blackwell_moe/kernels/fp8_moe_v3.py:39-48, of the Triton segment kernels
// (src/blackwell_moe/kernels/segment_ops.py:15-120) and of the scatter-add combine
// (src/blackwell_moe/kernels/scatter.py:25-72).
#include <mutex>

#include "common.cuh"

namespace bwmoe {
namespace {

constexpr int kPlanThreads = 1024;
constexpr int kSlotsPerBlock = 4096;   // slots ranked by one block (4 rounds of 1024)
constexpr int kMaxE = 256;

// ---- pass 1: per-block histogram of expert ids + per-segment max of the row amax ----
__global__ void __launch_bounds__(kPlanThreads)
plan_hist_kernel(const int32_t* __restrict__ indices, const float* __restrict__ row_amax, int M, int E,
                 int K, int32_t* __restrict__ block_hist, float* __restrict__ seg_amax,
                 int32_t* __restrict__ status) {
  __shared__ int hist[kMaxE];
  __shared__ unsigned int amax[kMaxE];
  for (int e = threadIdx.x; e < E; e += blockDim.x) hist[e] = 0, amax[e] = 0u;
  __syncthreads();
  const int s0 = blockIdx.x * kSlotsPerBlock;
  for (int i = threadIdx.x; i < kSlotsPerBlock; i += blockDim.x) {
    const int s = s0 + i;
    if (s >= M) break;
    const int e = indices[s];
    if (e < 0 || e >= E) {
      atomicOr(status, BWMOE_STATUS_BAD_EXPERT);
      continue;
    }
    atomicAdd(&hist[e], 1);
    if (row_amax != nullptr) atomicMax(&amax[e], __float_as_uint(row_amax[s / K]));
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    block_hist[(size_t)blockIdx.x * E + e] = hist[e];
    if (seg_amax != nullptr && amax[e] != 0u) atomicMax(reinterpret_cast<unsigned int*>(seg_amax) + e, amax[e]);
  }
}

// ---- pass 2: offsets[E+1] and, per block, the first row of each expert's slots ----
__global__ void __launch_bounds__(kMaxE)
plan_scan_kernel(int32_t* __restrict__ block_hist, int B, int E, int32_t* __restrict__ offsets) {
  __shared__ int total[kMaxE];
  __shared__ int start[kMaxE + 1];
  const int e = threadIdx.x;
  if (e < E) {
    int run = 0;
    for (int b = 0; b < B; ++b) {
      const int c = block_hist[(size_t)b * E + e];
      block_hist[(size_t)b * E + e] = run;   // exclusive prefix over blocks
      run += c;
    }
    total[e] = run;
  }
  __syncthreads();
  if (e == 0) {
    int run = 0;
    for (int i = 0; i < E; ++i) {
      start[i] = run;
      run += total[i];
    }
    start[E] = run;
  }
  __syncthreads();
  if (e < E) offsets[e] = start[e];
  if (e == 0) offsets[E] = start[E];
  if (e < E) {
    const int base = start[e];
    for (int b = 0; b < B; ++b) block_hist[(size_t)b * E + e] += base;
  }
}

// ---- pass 3: stable rank of every slot inside its block -> permuted row ----
__global__ void __launch_bounds__(kPlanThreads)
plan_rank_kernel(const int32_t* __restrict__ indices, int M, int E, const int32_t* __restrict__ block_base,
                 const int32_t* __restrict__ offsets, int32_t* __restrict__ pos, int32_t* __restrict__ row_slot,
                 int32_t* __restrict__ row_expert) {
  extern __shared__ int cnt[];            // [32 warps][E] counts of this pass, then exclusive prefixes
  __shared__ int round_base[kMaxE];       // slots of earlier rounds in this block, per expert
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int n_rows = offsets[E];          // rows that exist (slots with a valid expert id)
  for (int e = threadIdx.x; e < E; e += blockDim.x) round_base[e] = block_base[(size_t)blockIdx.x * E + e];
  const int s0 = blockIdx.x * kSlotsPerBlock;
  for (int r = 0; r < kSlotsPerBlock / kPlanThreads; ++r) {
    if (s0 + r * kPlanThreads >= M) break;   // uniform for the block
    for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) cnt[i] = 0;
    __syncthreads();
    const int s = s0 + r * kPlanThreads + threadIdx.x;
    int e = -1;
    if (s < M) {
      e = indices[s];
      if (e < 0 || e >= E) e = -1;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) cnt[warp * E + e] = __popc(peers);
    __syncthreads();
    for (int ee = threadIdx.x; ee < E; ee += blockDim.x) {
      int run = 0;
      for (int w = 0; w < 32; ++w) {
        const int c = cnt[w * E + ee];
        cnt[w * E + ee] = run;
        run += c;
      }
      // total of this pass is added to round_base after everyone has read it
      cnt[32 * E + ee] = run;
    }
    __syncthreads();
    if (e >= 0) {
      const int p = round_base[e] + cnt[warp * E + e] + rank_in_warp;
      pos[s] = p;
      row_slot[p] = s;
      row_expert[p] = e;
    } else if (s < M) {
      pos[s] = -1;
    }
    // slots with an expert id out of range own no row: the rows past the last segment are marked
    // so that the row-wise kernels behind the plan skip them
    if (s < M && s >= n_rows) row_slot[s] = -1, row_expert[s] = -1;
    __syncthreads();
    for (int ee = threadIdx.x; ee < E; ee += blockDim.x) round_base[ee] += cnt[32 * E + ee];
    __syncthreads();
  }
}

// ---- all three passes in one block, for at most 1024 slots (decode-sized batches) ----
// Also emits the per-segment quantisation scale when asked to (scales_out != nullptr).
__global__ void __launch_bounds__(kPlanThreads)
plan_small_kernel(const int32_t* __restrict__ indices, const float* __restrict__ row_amax, int M, int E, int K,
                  int32_t* __restrict__ offsets, int32_t* __restrict__ pos, int32_t* __restrict__ row_slot,
                  int32_t* __restrict__ row_expert, float* __restrict__ seg_amax, float* __restrict__ scales_out,
                  int32_t* __restrict__ status) {
  chain_wait();
  extern __shared__ int cnt[];            // [32 warps][E] per-warp counts -> exclusive prefixes
  __shared__ int start[kMaxE + 1];
  __shared__ unsigned int amax[kMaxE];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * E; i += blockDim.x) cnt[i] = 0;
  for (int e = threadIdx.x; e < E; e += blockDim.x) amax[e] = 0u;
  __syncthreads();
  const int s = threadIdx.x;
  int e = -1;
  if (s < M) {
    e = indices[s];
    if (e < 0 || e >= E) {
      atomicOr(status, BWMOE_STATUS_BAD_EXPERT);
      e = -1;
    } else if (row_amax != nullptr) {
      atomicMax(&amax[e], __float_as_uint(row_amax[s / K]));
    }
  }
  const unsigned peers = __match_any_sync(0xffffffffu, e);
  const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
  if (e >= 0 && rank_in_warp == 0) cnt[warp * E + e] = __popc(peers);
  __syncthreads();
  for (int ee = threadIdx.x; ee < E; ee += blockDim.x) {
    int run = 0;
    for (int w = 0; w < 32; ++w) {
      const int c = cnt[w * E + ee];
      cnt[w * E + ee] = run;
      run += c;
    }
    start[ee + 1] = run;                 // count of expert ee, turned into an offset below
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    start[0] = 0;
    for (int i = 0; i < E; ++i) start[i + 1] += start[i];
  }
  __syncthreads();
  for (int ee = threadIdx.x; ee <= E; ee += blockDim.x) offsets[ee] = start[ee];
  for (int ee = threadIdx.x; ee < E; ee += blockDim.x) {
    const float a = __uint_as_float(amax[ee]);
    if (seg_amax != nullptr) seg_amax[ee] = a;
    if (scales_out != nullptr) scales_out[ee] = start[ee + 1] > start[ee] ? scale_from_amax(a) : 1.0f;
  }
  if (e >= 0) {
    const int p = start[e] + cnt[warp * E + e] + rank_in_warp;
    pos[s] = p;
    row_slot[p] = s;
    row_expert[p] = e;
  } else if (s < M) {
    pos[s] = -1;
  }
  // rows past the last segment (slots with an out-of-range expert id own none): marked as absent
  if (s < M && s >= start[E]) row_slot[s] = -1, row_expert[s] = -1;
}

__global__ void segment_scales_kernel(const float* __restrict__ seg_amax, const int32_t* __restrict__ offsets,
                                      int E, float* __restrict__ scales) {
  chain_wait();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const bool empty = offsets != nullptr && offsets[e + 1] <= offsets[e];
  scales[e] = empty ? 1.0f : scale_from_amax(seg_amax[e]);
}

// ---- row-wise bf16 -> e4m3 with a per-row-selected scale; one thread per 8 elements, one block per row chunk ----
// SRC_BY_SLOT: source row = row_slot[m] / K (gather from token order); else source row = m.
// FROM_AMAX: `scales` holds the segment amax; the scale is derived here and published to scales_out.
__device__ __forceinline__ unsigned long long splat2(float v) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "r"(__float_as_uint(v)));
  return r;
}
// Eight bf16 (one 16-byte vector) -> eight E4M3 codes: fp32 product with the scale (packed two at a
// time), then one saturating round-to-nearest-even conversion.  The conversion's saturation is the
// clamp to +-448 of the recipe, so no separate min/max is spent.
__device__ __forceinline__ uint32_t e4m3x4_scaled(uint32_t w0, uint32_t w1, unsigned long long s2) {
  unsigned long long a, b;
  asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "r"(w0 << 16), "r"(w0 & 0xffff0000u));
  asm("mov.b64 %0, {%1, %2};" : "=l"(b) : "r"(w1 << 16), "r"(w1 & 0xffff0000u));
  asm("mul.rn.f32x2 %0, %0, %1;" : "+l"(a) : "l"(s2));
  asm("mul.rn.f32x2 %0, %0, %1;" : "+l"(b) : "l"(s2));
  uint32_t a0, a1, b0, b1;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(a0), "=r"(a1) : "l"(a));
  asm("mov.b64 {%0, %1}, %2;" : "=r"(b0), "=r"(b1) : "l"(b));
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(__uint_as_float(a1)), "f"(__uint_as_float(a0)));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(__uint_as_float(b1)), "f"(__uint_as_float(b0)));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

// Rows -> E4M3 with the scale of the row's expert.  Flat: one thread per 16 consecutive elements of
// the [M, W] output (two 16-byte loads, one 16-byte store), the row found by one 32-bit division.
// Measured against row-structured variants (a block or a thread group per row chunk, with and without
// software pipelining) this plain form was the only one to reach the copy rate of the part for short
// rows (W = 1408: 6.3 TB/s against 3.5).
template <bool SRC_BY_SLOT, bool FROM_AMAX>
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ row_slot,
                  const int32_t* __restrict__ row_expert, const float* __restrict__ scales,
                  float* __restrict__ scales_out, unsigned M, unsigned W, int K, uint8_t* __restrict__ dst) {
  chain_wait();
  const unsigned per_row = W / 16;
  const unsigned p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= M * per_row) return;
  const unsigned m = p / per_row, c = p - m * per_row;
  // A row that no slot owns (expert id out of range: row_expert = -1) is not skipped by a branch, which would
  // put a dependent round trip in front of the data loads of this bandwidth-bound kernel: it is quantised with
  // scale 0 (its place in dst exists), and only its index uses are guarded.
  const int expert = row_expert[m];
  const size_t srow = SRC_BY_SLOT ? (size_t)(max(row_slot[m], 0) / K) : (size_t)m;
  const uint4* in = reinterpret_cast<const uint4*>(src + srow * W) + 2 * c;
  const uint4 r0 = in[0], r1 = in[1];
  float scale = expert >= 0 ? scales[expert] : 0.f;
  if (FROM_AMAX && expert >= 0) {
    scale = scale_from_amax(scale);
    // published once per segment, by its first row (a store per row piled a hundred thousand stores onto a few
    // dozen addresses)
    if (c == 0 && (m == 0 || row_expert[m - 1] != expert)) scales_out[expert] = scale;
  }
  const unsigned long long s2 = splat2(scale);
  reinterpret_cast<uint4*>(dst + (size_t)m * W)[c] =
      make_uint4(e4m3x4_scaled(r0.x, r0.y, s2), e4m3x4_scaled(r0.z, r0.w, s2), e4m3x4_scaled(r1.x, r1.y, s2),
                 e4m3x4_scaled(r1.z, r1.w, s2));
}

// Rows of expert-contiguous segments -> E4M3 with the segment's scale, the number of rows known only on
// the device (offsets[E]): a fixed grid strides over rows x 16-element pieces, the expert of a row is
// found by bisection of the offsets.  For callers that must not wait for row counts on the host (expert
// parallelism: the rows a rank receives are counted on the device).
__global__ void __launch_bounds__(256)
quant_segments_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ offsets, int E,
                      const float* __restrict__ scales, unsigned W, uint8_t* __restrict__ dst) {
  const unsigned per_row = W / 16;
  const unsigned long long total = (unsigned long long)offsets[E] * per_row;
  for (unsigned long long p = (unsigned long long)blockIdx.x * blockDim.x + threadIdx.x; p < total;
       p += (unsigned long long)gridDim.x * blockDim.x) {
    const unsigned m = (unsigned)(p / per_row), c = (unsigned)(p - (unsigned long long)m * per_row);
    int lo = 0, hi = E;                          // largest e with offsets[e] <= m
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if ((unsigned)offsets[mid] <= m) lo = mid; else hi = mid;
    }
    const uint4* in = reinterpret_cast<const uint4*>(src + (size_t)m * W) + 2 * c;
    const uint4 r0 = in[0], r1 = in[1];
    const unsigned long long s2 = splat2(scales[lo]);
    reinterpret_cast<uint4*>(dst + (size_t)m * W)[c] =
        make_uint4(e4m3x4_scaled(r0.x, r0.y, s2), e4m3x4_scaled(r0.z, r0.w, s2), e4m3x4_scaled(r1.x, r1.y, s2),
                   e4m3x4_scaled(r1.z, r1.w, s2));
  }
}

// Token-major form of the gather + quantisation: a token's row is read once and written to each of
// its K destination rows with that row's expert scale (K x fewer reads than walking the permuted rows).
// One thread per 16 consecutive elements of x[T, W].
__global__ void __launch_bounds__(256)
scatter_quant_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ pos,
                     const int32_t* __restrict__ indices, const float* __restrict__ scales, unsigned T,
                     unsigned W, int K, uint8_t* __restrict__ dst, const float* __restrict__ weights,
                     float* __restrict__ row_w) {
  chain_wait();
  const unsigned per_row = W / 16;
  const unsigned p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= T * per_row) return;
  const unsigned t = p / per_row, c = p - t * per_row;
  const uint4* in = reinterpret_cast<const uint4*>(x + (size_t)t * W) + 2 * c;
  const uint4 r0 = in[0], r1 = in[1];
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    const int row = pos[(size_t)t * K + k];
    if (row < 0) continue;                       // slot with an out-of-range expert: no row
    if (row_w != nullptr && c == 0) row_w[row] = weights[(size_t)t * K + k];   // routing weight in row order
    const unsigned long long s2 = splat2(scales[indices[(size_t)t * K + k]]);
    reinterpret_cast<uint4*>(dst + (size_t)row * W)[c] =
        make_uint4(e4m3x4_scaled(r0.x, r0.y, s2), e4m3x4_scaled(r0.z, r0.w, s2), e4m3x4_scaled(r1.x, r1.y, s2),
                   e4m3x4_scaled(r1.z, r1.w, s2));
  }
}

// Index maps of one expert-parallel step, from the gathered [G, E] row counts (one block):
//   delta[e]       where this rank's rows of expert e land inside e's segment on its owner, minus where
//                  they start in this rank's own permuted order (offsets[e])
//   offsets_l      the local experts' segments (exclusive scan of their total rows)
//   home_counts / home_first [G, el]   rows of local expert j that came from rank s, and the row of
//                  rank s's own permuted order they return to
__global__ void __launch_bounds__(256)
ep_maps_kernel(const int32_t* __restrict__ counts, const int32_t* __restrict__ offsets, int G, int E, int rank,
               int32_t* __restrict__ delta, int32_t* __restrict__ offsets_l, int32_t* __restrict__ home_counts,
               int32_t* __restrict__ home_first) {
  __shared__ int total[256], below[256], seg_start[256];
  const int el = E / G;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int t = 0, b = 0;
    for (int s = 0; s < G; ++s) {
      const int c = counts[s * E + e];
      t += c;
      if (s < rank) b += c;
    }
    total[e] = t, below[e] = b;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {      // exclusive scan inside the owner's expert range
    const int first = (e / el) * el;
    int acc = 0;
    for (int j = first; j < e; ++j) acc += total[j];
    seg_start[e] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) delta[e] = seg_start[e] + below[e] - offsets[e];
  for (int j = threadIdx.x; j <= el; j += blockDim.x)
    offsets_l[j] = j < el ? seg_start[rank * el + j] : seg_start[rank * el + el - 1] + total[rank * el + el - 1];
  for (int i = threadIdx.x; i < G * el; i += blockDim.x) {
    const int s = i / el, e = rank * el + i % el;
    int first = 0;
    for (int j = 0; j < e; ++j) first += counts[s * E + j];
    home_counts[i] = counts[s * E + e];
    home_first[i] = first;
  }
}

// Expert-parallel dispatch fused into the quantisation: the row of slot (t, k), bound for expert e, is
// written straight into the memory of the rank that owns e (peer stores over NVLink; the owner's own rows
// are ordinary local stores).  dst[r] is rank r's receive buffer; the row lands at
// pos[t, k] + delta[e], which is its place in the owner's per-expert segments ordered by (source rank,
// source row).  No multicast, no bulk copies: plain 16-byte stores.
__global__ void __launch_bounds__(256)
scatter_quant_peers_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ pos,
                           const int32_t* __restrict__ indices, const float* __restrict__ scales,
                           const int32_t* __restrict__ delta, unsigned T, unsigned W, int K, int experts_per_rank,
                           const PeerPtrs dst, int rows_cap, int32_t* __restrict__ status) {
  const unsigned per_row = W / 16;
  const unsigned p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= T * per_row) return;
  const unsigned t = p / per_row, c = p - t * per_row;
  const uint4* in = reinterpret_cast<const uint4*>(x + (size_t)t * W) + 2 * c;
  const uint4 r0 = in[0], r1 = in[1];
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    const int row = pos[(size_t)t * K + k];
    if (row < 0) continue;
    const int e = indices[(size_t)t * K + k];
    const int dst_row = row + delta[e];
    if (dst_row < 0 || dst_row >= rows_cap) {      // the owner's buffer is smaller than what the ranks send it
      if (c == 0 && status != nullptr) atomicOr(status, BWMOE_STATUS_EP_OVERFLOW);
      continue;
    }
    const unsigned long long s2 = splat2(scales[e]);
    uint8_t* base = static_cast<uint8_t*>(dst.p[e / experts_per_rank]);
    reinterpret_cast<uint4*>(base + (size_t)dst_row * W)[c] =
        make_uint4(e4m3x4_scaled(r0.x, r0.y, s2), e4m3x4_scaled(r0.z, r0.w, s2), e4m3x4_scaled(r1.x, r1.y, s2),
                   e4m3x4_scaled(r1.z, r1.w, s2));
  }
}

// Expert-parallel way back fused into the combine: the result row of slot (t, k) is read from the
// memory of the rank that computed it (peer loads), same arithmetic and order as combine_kernel.
__global__ void __launch_bounds__(256)
combine_peers_kernel(const PeerPtrs src, const int32_t* __restrict__ pos, const int32_t* __restrict__ indices,
                     const float* __restrict__ weights, const int32_t* __restrict__ delta, int experts_per_rank,
                     int T, int D, int K, __nv_bfloat16* __restrict__ out) {
  const int vec_per_row = D / 8;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (size_t)T * vec_per_row) return;
  const int t = (int)(gid / vec_per_row), v = (int)(gid % vec_per_row);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    const int p = pos[(size_t)t * K + k];
    if (p < 0) continue;
    const int e = indices[(size_t)t * K + k];
    const float w = bf16_round(weights[(size_t)t * K + k]);
    const __nv_bfloat16* y = static_cast<const __nv_bfloat16*>(src.p[e / experts_per_rank]);
    const uint4 raw = reinterpret_cast<const uint4*>(y + (size_t)(p + delta[e]) * D)[v];
    const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(q[i]);
      acc[2 * i] += bf16_round(f.x * w);
      acc[2 * i + 1] += bf16_round(f.y * w);
    }
  }
  uint4 o;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) op[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  reinterpret_cast<uint4*>(out + (size_t)t * D)[v] = o;
}

// ---- out[t,:] = bf16( sum_k float( bf16( y[pos[t*K+k],:] * bf16(w[t,k]) ) ) ) ----
// Optional tail (the block glue of FP8MoELayer.forward, src/blackwell_moe/runtime/deepseek_patch.py:51-53):
//   out = bf16( bf16(routed * scale) + residual ) with routed = the bf16 sum above.
// PREWEIGHTED: the rows already carry bf16(y * bf16(w)) (the down projection's epilogue multiplied them), so
// only the sum over k remains; the result is bit-identical either way.
// n_tail: the last n_tail slots of every token are always-on (shared) experts run as extra groups of the same
// pipeline; their rows are the `shared` term of the glue above: out = bf16( bf16(routed * scale) + bf16(sum of
// the tail rows) ).
template <bool PREWEIGHTED>
__global__ void __launch_bounds__(256)
combine_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ pos,
               const float* __restrict__ weights, int T, int D, int K, __nv_bfloat16* __restrict__ out,
               float scale, const __nv_bfloat16* __restrict__ residual, int n_tail) {
  chain_wait();
  const int vec_per_row = D / 8;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (size_t)T * vec_per_row) return;
  const int t = (int)(gid / vec_per_row), v = (int)(gid % vec_per_row);
  const int k_routed = K - n_tail;
  float acc[8], tail[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f, tail[i] = 0.f;
  // three rows at a time: their vectors are all requested before the first is used (one load in flight
  // per thread left the gather at 5.2 TB/s; eight cost too many registers)
  constexpr int kRows = 3;
  for (int k0 = 0; k0 < K; k0 += kRows) {
    int p[kRows];
    float w[kRows];
    uint4 raw[kRows];
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      const bool in_k = k0 + j < K;
      p[j] = in_k ? pos[(size_t)t * K + k0 + j] : -1;
      w[j] = (in_k && !PREWEIGHTED) ? weights[(size_t)t * K + k0 + j] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kRows; ++j)
      raw[j] = p[j] >= 0 ? reinterpret_cast<const uint4*>(y + (size_t)p[j] * D)[v] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int j = 0; j < kRows; ++j) {
      if (p[j] < 0) continue;
      const float wk = bf16_round(w[j]);
      const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&raw[j]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(q[i]);
        const float a = PREWEIGHTED ? f.x : bf16_round(f.x * wk), b = PREWEIGHTED ? f.y : bf16_round(f.y * wk);
        if (k0 + j < k_routed) acc[2 * i] += a, acc[2 * i + 1] += b;
        else                   tail[2 * i] += a, tail[2 * i + 1] += b;
      }
    }
  }
  if (scale != 1.0f) {     // bf16 tensor times a Python scalar: torch multiplies in fp32 by the unrounded scalar
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = bf16_round(bf16_round(acc[i]) * scale);
  }
  if (residual != nullptr) {
    const uint4 raw = reinterpret_cast<const uint4*>(residual + (size_t)t * D)[v];
    const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(q[i]);
      acc[2 * i] = bf16_round(acc[2 * i]) + f.x;
      acc[2 * i + 1] = bf16_round(acc[2 * i + 1]) + f.y;
    }
  }
  if (n_tail > 0) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = bf16_round(acc[i]) + bf16_round(tail[i]);
  }
  uint4 o;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) op[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  reinterpret_cast<uint4*>(out + (size_t)t * D)[v] = o;
}

// Routing of a block with S always-on experts appended as groups E .. E+S-1: every token keeps its K routed
// slots and gets S more with weight 1.
__global__ void append_shared_slots_kernel(const int32_t* __restrict__ idx_r, const float* __restrict__ w_r, int T,
                                           int K, int E, int S, int32_t* __restrict__ idx, float* __restrict__ w) {
  chain_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int KS = K + S;
  if (i >= T * KS) return;
  const int t = i / KS, k = i - t * KS;
  idx[i] = k < K ? idx_r[t * K + k] : E + (k - K);
  w[i] = k < K ? w_r[t * K + k] : 1.0f;
}

// amax[first .. first+count) <- their common maximum: groups that are pieces of one tensor share its scale
__global__ void merge_amax_kernel(float* __restrict__ amax, int first, int count) {
  chain_wait();
  float m = 0.f;
  for (int i = 0; i < count; ++i) m = fmaxf(m, amax[first + i]);
  for (int i = 0; i < count; ++i) amax[first + i] = m;
}

}  // namespace

int launch_append_shared_slots(const int32_t* idx_r, const float* w_r, int T, int K, int E, int S, int32_t* idx,
                               float* w, cudaStream_t st) {
  const int n = T * (K + S);
  BWMOE_CUDA_OK(launch_chained(append_shared_slots_kernel, dim3(ceil_div(n, 256)), dim3(256), 0, st, idx_r, w_r, T, K, E, S, idx, w));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_merge_amax(float* amax, int first, int count, cudaStream_t st) {
  BWMOE_CUDA_OK(launch_chained(merge_amax_kernel, dim3(1), dim3(1), 0, st, amax, first, count));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

inline unsigned quant_grid(int M, int W) { return (unsigned)(((size_t)M * (W / 16) + 255) / 256); }

size_t plan_scratch_bytes(int T, int E, int K) {
  const long long M = (long long)T * K;
  const long long B = (M + kSlotsPerBlock - 1) / kSlotsPerBlock;
  return (size_t)(B * E * sizeof(int32_t) + 256);
}

int launch_plan(const int32_t* indices, const float* row_amax, int T, int E, int K, int32_t* offsets,
                int32_t* pos, int32_t* row_slot, int32_t* row_expert, float* seg_amax, int32_t* status,
                void* scratch, cudaStream_t st, float* scales_out) {
  BWMOE_REQUIRE(T > 0 && E > 0 && K > 0, BWMOE_ERR_BAD_SHAPE, "plan: T=%d E=%d K=%d", T, E, K);
  BWMOE_REQUIRE(E <= kMaxE, BWMOE_ERR_UNSUPPORTED, "plan: E=%d > %d", E, kMaxE);
  BWMOE_REQUIRE((long long)T * K < (1ll << 31), BWMOE_ERR_UNSUPPORTED, "plan: T*K too large");
  BWMOE_REQUIRE(indices && offsets && pos && row_slot && row_expert && status && scratch, BWMOE_ERR_NULL,
                "plan: null pointer");
  const int M = T * K;
  if (M <= kPlanThreads) {
    BWMOE_CUDA_OK(launch_chained(plan_small_kernel, dim3(1), dim3(kPlanThreads), (size_t)32 * E * sizeof(int), st,
        indices, row_amax, M, E, K, offsets, pos, row_slot, row_expert, seg_amax, scales_out, status));
    BWMOE_CUDA_OK(cudaGetLastError());
    return BWMOE_OK;
  }
  const int B = ceil_div(M, kSlotsPerBlock);
  int32_t* block_hist = static_cast<int32_t*>(scratch);
  if (seg_amax != nullptr) BWMOE_CUDA_OK(cudaMemsetAsync(seg_amax, 0, sizeof(float) * E, st));
  plan_hist_kernel<<<B, kPlanThreads, 0, counted(st)>>>(indices, row_amax, M, E, K, block_hist,
                                               row_amax ? seg_amax : nullptr, status);
  plan_scan_kernel<<<1, kMaxE, 0, counted(st)>>>(block_hist, B, E, offsets);
  const size_t smem = (size_t)33 * E * sizeof(int);
  plan_rank_kernel<<<B, kPlanThreads, smem, counted(st)>>>(indices, M, E, block_hist, offsets, pos, row_slot, row_expert);
  BWMOE_CUDA_OK(cudaGetLastError());
  if (scales_out != nullptr) return launch_segment_scales(seg_amax, offsets, E, scales_out, st);
  return BWMOE_OK;
}

// ---- allocation-free variant of the permutation plan ------------------------------
// Scratch for callers that cannot hand the library a scratch buffer: a fixed array
// that lives in every GPU's memory from the moment the library is loaded there.
constexpr int kStaticPlanBlocks = 64;                       // 64 * 4096 = 262144 slots at most
static __device__ __align__(256) int32_t g_static_plan_scratch[kStaticPlanBlocks * kMaxE];   // 64 KiB

int launch_plan_static(const int32_t* indices, const float* row_amax, int T, int E, int K, int32_t* offsets,
                       int32_t* pos, int32_t* row_slot, int32_t* row_expert, float* seg_amax, int32_t* status,
                       cudaStream_t st) {
  BWMOE_REQUIRE(T > 0 && E > 0 && K > 0, BWMOE_ERR_BAD_SHAPE, "plan_static: T=%d E=%d K=%d", T, E, K);
  BWMOE_REQUIRE(E <= kMaxE, BWMOE_ERR_UNSUPPORTED, "plan_static: E=%d > %d", E, kMaxE);
  const long long max_slots = (long long)kStaticPlanBlocks * kSlotsPerBlock;
  BWMOE_REQUIRE((long long)T * K <= max_slots, BWMOE_ERR_UNSUPPORTED,
                "plan_static: T*K=%lld exceeds the %lld slots the built-in scratch covers; "
                "use bwmoe_permute_plan with a caller-provided scratch buffer",
                (long long)T * K, max_slots);
  // In host code `g_static_plan_scratch` is only a handle for the symbol, not a device
  // address: ask the runtime where the array lives on the CURRENT device, once per device.
  static std::mutex mu;
  static void* dev_ptr[64] = {nullptr};
  int dev = 0;
  BWMOE_CUDA_OK(cudaGetDevice(&dev));
  BWMOE_REQUIRE(dev >= 0 && dev < 64, BWMOE_ERR_UNSUPPORTED, "plan_static: device ordinal %d out of range", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev_ptr[dev] == nullptr) {
      void* p = nullptr;
      BWMOE_CUDA_OK(cudaGetSymbolAddress(&p, g_static_plan_scratch));
      BWMOE_REQUIRE(p != nullptr, BWMOE_ERR_CUDA, "plan_static: cudaGetSymbolAddress returned null");
      dev_ptr[dev] = p;
    }
    scratch = dev_ptr[dev];
  }
  // Nothing in the array has to start at zero: the histogram pass overwrites every entry
  // the later passes read (blocks 0..B-1 x experts 0..E-1) before they read it.
  return launch_plan(indices, row_amax, T, E, K, offsets, pos, row_slot, row_expert, seg_amax, status, scratch, st,
                     nullptr);
}

int launch_segment_scales(const float* seg_amax, const int32_t* offsets, int E, float* scales,
                          cudaStream_t st) {
  BWMOE_REQUIRE(E > 0, BWMOE_ERR_BAD_SHAPE, "segment_scales: E=%d", E);
  BWMOE_REQUIRE(seg_amax && scales, BWMOE_ERR_NULL, "segment_scales: null pointer");
  BWMOE_CUDA_OK(launch_chained(segment_scales_kernel, dim3(ceil_div(E, 128)), dim3(128), 0, st, seg_amax, offsets, E, scales));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_gather_quant(const void* x, const int32_t* row_slot, const int32_t* row_expert,
                        const float* scales, int M, int D, int K, void* xq, cudaStream_t st) {
  BWMOE_REQUIRE(M > 0 && D > 0 && K > 0 && D % 16 == 0, BWMOE_ERR_BAD_SHAPE, "gather_quant: M=%d D=%d K=%d", M, D, K);
  BWMOE_REQUIRE(x && row_slot && row_expert && scales && xq, BWMOE_ERR_NULL, "gather_quant: null pointer");
  BWMOE_REQUIRE(aligned16(x) && aligned16(xq), BWMOE_ERR_BAD_ALIGN, "gather_quant: pointers must be 16-byte aligned");
  BWMOE_CUDA_OK(launch_chained(quant_rows_kernel<true, false>, dim3(quant_grid(M, D)), dim3(256), 0, st,
      static_cast<const __nv_bfloat16*>(x), row_slot, row_expert, scales, nullptr, M, D, K, static_cast<uint8_t*>(xq)));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_scatter_quant(const void* x, const int32_t* pos, const int32_t* indices, const float* scales, int T,
                         int D, int K, void* xq, cudaStream_t st, const float* weights, float* row_w) {
  BWMOE_REQUIRE(T > 0 && D > 0 && K > 0 && D % 16 == 0, BWMOE_ERR_BAD_SHAPE, "scatter_quant: T=%d D=%d K=%d", T, D, K);
  BWMOE_REQUIRE(x && pos && indices && scales && xq, BWMOE_ERR_NULL, "scatter_quant: null pointer");
  BWMOE_REQUIRE(aligned16(x) && aligned16(xq), BWMOE_ERR_BAD_ALIGN, "scatter_quant: pointers must be 16-byte aligned");
  BWMOE_REQUIRE(row_w == nullptr || weights != nullptr, BWMOE_ERR_NULL, "scatter_quant: row weights without weights");
  BWMOE_CUDA_OK(launch_chained(scatter_quant_kernel, dim3(quant_grid(T, D)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x), pos, indices, scales,
                                                         T, D, K, static_cast<uint8_t*>(xq), weights, row_w));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_requant(const void* h, const int32_t* row_expert, const float* scales_h, int M, int H,
                   void* hq, cudaStream_t st, float* scales_from_amax_out) {
  BWMOE_REQUIRE(M > 0 && H > 0 && H % 16 == 0, BWMOE_ERR_BAD_SHAPE, "requant: M=%d H=%d", M, H);
  BWMOE_REQUIRE(h && row_expert && scales_h && hq, BWMOE_ERR_NULL, "requant: null pointer");
  BWMOE_REQUIRE(aligned16(h) && aligned16(hq), BWMOE_ERR_BAD_ALIGN, "requant: pointers must be 16-byte aligned");
  if (scales_from_amax_out != nullptr)   // scales_h holds the segment amax; scales are derived and published
    BWMOE_CUDA_OK(launch_chained(quant_rows_kernel<false, true>, dim3(quant_grid(M, H)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(h), nullptr,
                                                                     row_expert, scales_h, scales_from_amax_out, M, H, 1,
                                                                     static_cast<uint8_t*>(hq)));
  else
    BWMOE_CUDA_OK(launch_chained(quant_rows_kernel<false, false>, dim3(quant_grid(M, H)), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(h), nullptr,
                                                                      row_expert, scales_h, nullptr, M, H, 1,
                                                                      static_cast<uint8_t*>(hq)));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_requant_segments(const void* h, const int32_t* offsets, const float* scales_h, int E, int H, void* hq,
                            cudaStream_t st) {
  BWMOE_REQUIRE(E > 0 && E <= kMaxE && H > 0 && H % 16 == 0, BWMOE_ERR_BAD_SHAPE, "requant_segments: E=%d H=%d", E, H);
  BWMOE_REQUIRE(h && offsets && scales_h && hq, BWMOE_ERR_NULL, "requant_segments: null pointer");
  BWMOE_REQUIRE(aligned16(h) && aligned16(hq), BWMOE_ERR_BAD_ALIGN, "requant_segments: pointers must be 16-byte aligned");
  quant_segments_kernel<<<sm_count() * 16, 256, 0, counted(st)>>>(static_cast<const __nv_bfloat16*>(h), offsets, E, scales_h,
                                                                  (unsigned)H, static_cast<uint8_t*>(hq));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

// ---- dense (always-on) expert: one segment holding every row ----
__global__ void __launch_bounds__(1024)
dense_prepare_kernel(const float* __restrict__ row_amax, int T, int32_t* __restrict__ offsets,
                     float* __restrict__ seg_amax) {
  __shared__ float red[32];
  float m = 0.f;
  for (int t = threadIdx.x; t < T; t += blockDim.x) m = fmaxf(m, row_amax[t]);
  for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) m = fmaxf(m, red[w]);
    seg_amax[0] = m;
    offsets[0] = 0;
    offsets[1] = T;
  }
}

int launch_dense_prepare(const float* row_amax, int T, int32_t* offsets, float* seg_amax, cudaStream_t st) {
  dense_prepare_kernel<<<1, 1024, 0, counted(st)>>>(row_amax, T, offsets, seg_amax);
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

// rows in place (no gather), scale derived from the segment amax and published
int launch_quant_rows_from_amax(const void* x, const int32_t* row_expert, const float* seg_amax, int M, int W,
                                void* xq, float* scales_out, cudaStream_t st) {
  BWMOE_CUDA_OK(launch_chained(quant_rows_kernel<false, true>, dim3(quant_grid(M, W)), dim3(256), 0, st,
      static_cast<const __nv_bfloat16*>(x), nullptr, row_expert, seg_amax, scales_out, M, W, 1,
      static_cast<uint8_t*>(xq)));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_combine(const void* y, const int32_t* pos, const float* weights, int T, int D, int K,
                   void* out, cudaStream_t st, float scale, const void* residual, bool preweighted, int n_tail) {
  BWMOE_REQUIRE(n_tail >= 0 && n_tail < K, BWMOE_ERR_BAD_SHAPE, "combine: %d always-on slots of %d", n_tail, K);
  BWMOE_REQUIRE(T > 0 && D > 0 && K > 0 && D % 8 == 0, BWMOE_ERR_BAD_SHAPE, "combine: T=%d D=%d K=%d", T, D, K);
  BWMOE_REQUIRE(y && pos && weights && out, BWMOE_ERR_NULL, "combine: null pointer");
  BWMOE_REQUIRE(aligned16(y) && aligned16(out), BWMOE_ERR_BAD_ALIGN, "combine: pointers must be 16-byte aligned");
  const size_t n = (size_t)T * (D / 8);
  if (preweighted)
    BWMOE_CUDA_OK(launch_chained(combine_kernel<true>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st,
        static_cast<const __nv_bfloat16*>(y), pos, weights, T, D, K, static_cast<__nv_bfloat16*>(out), scale,
        static_cast<const __nv_bfloat16*>(residual), n_tail));
  else
    BWMOE_CUDA_OK(launch_chained(combine_kernel<false>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st,
        static_cast<const __nv_bfloat16*>(y), pos, weights, T, D, K, static_cast<__nv_bfloat16*>(out), scale,
        static_cast<const __nv_bfloat16*>(residual), n_tail));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_scatter_quant_peers(const void* x, const int32_t* pos, const int32_t* indices, const float* scales,
                               const int32_t* delta, int T, int D, int K, int experts_per_rank, void* const* dst,
                               int n_ranks, int rows_cap, int32_t* status, cudaStream_t st) {
  BWMOE_REQUIRE(T > 0 && D > 0 && K > 0 && D % 16 == 0, BWMOE_ERR_BAD_SHAPE, "scatter_quant_peers: T=%d D=%d K=%d", T, D, K);
  BWMOE_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers && experts_per_rank >= 1, BWMOE_ERR_UNSUPPORTED,
                "scatter_quant_peers: %d ranks (at most %d)", n_ranks, kMaxPeers);
  BWMOE_REQUIRE(x && pos && indices && scales && delta && dst, BWMOE_ERR_NULL, "scatter_quant_peers: null pointer");
  BWMOE_REQUIRE(rows_cap > 0, BWMOE_ERR_BAD_SHAPE, "scatter_quant_peers: rows_cap=%d", rows_cap);
  PeerPtrs pp{};
  for (int r = 0; r < n_ranks; ++r) {
    BWMOE_REQUIRE(dst[r] != nullptr && aligned16(dst[r]), BWMOE_ERR_BAD_ALIGN, "scatter_quant_peers: buffer of rank %d", r);
    pp.p[r] = dst[r];
  }
  BWMOE_REQUIRE(aligned16(x), BWMOE_ERR_BAD_ALIGN, "scatter_quant_peers: x must be 16-byte aligned");
  scatter_quant_peers_kernel<<<quant_grid(T, D), 256, 0, counted(st)>>>(static_cast<const __nv_bfloat16*>(x), pos, indices,
                                                               scales, delta, T, D, K, experts_per_rank, pp, rows_cap,
                                                               status);
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_combine_peers(void* const* src, int n_ranks, const int32_t* pos, const int32_t* indices,
                         const float* weights, const int32_t* delta, int experts_per_rank, int T, int D, int K,
                         void* out, cudaStream_t st) {
  BWMOE_REQUIRE(T > 0 && D > 0 && K > 0 && D % 8 == 0, BWMOE_ERR_BAD_SHAPE, "combine_peers: T=%d D=%d K=%d", T, D, K);
  BWMOE_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers && experts_per_rank >= 1, BWMOE_ERR_UNSUPPORTED,
                "combine_peers: %d ranks (at most %d)", n_ranks, kMaxPeers);
  BWMOE_REQUIRE(src && pos && indices && weights && delta && out, BWMOE_ERR_NULL, "combine_peers: null pointer");
  PeerPtrs pp{};
  for (int r = 0; r < n_ranks; ++r) {
    BWMOE_REQUIRE(src[r] != nullptr && aligned16(src[r]), BWMOE_ERR_BAD_ALIGN, "combine_peers: buffer of rank %d", r);
    pp.p[r] = src[r];
  }
  BWMOE_REQUIRE(aligned16(out), BWMOE_ERR_BAD_ALIGN, "combine_peers: out must be 16-byte aligned");
  const size_t n = (size_t)T * (D / 8);
  combine_peers_kernel<<<(unsigned)((n + 255) / 256), 256, 0, counted(st)>>>(pp, pos, indices, weights, delta, experts_per_rank,
                                                                    T, D, K, static_cast<__nv_bfloat16*>(out));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_ep_maps(const int32_t* counts, const int32_t* offsets, int n_ranks, int E, int rank, int32_t* delta,
                   int32_t* offsets_local, int32_t* home_counts, int32_t* home_first, cudaStream_t st) {
  BWMOE_REQUIRE(n_ranks >= 1 && E >= 1 && E <= 256 && E % n_ranks == 0 && rank >= 0 && rank < n_ranks,
                BWMOE_ERR_BAD_SHAPE, "ep_maps: ranks=%d E=%d rank=%d", n_ranks, E, rank);
  BWMOE_REQUIRE(counts && offsets && delta && offsets_local && home_counts && home_first, BWMOE_ERR_NULL,
                "ep_maps: null pointer");
  ep_maps_kernel<<<1, 256, 0, counted(st)>>>(counts, offsets, n_ranks, E, rank, delta, offsets_local, home_counts, home_first);
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

}  // namespace bwmoe
