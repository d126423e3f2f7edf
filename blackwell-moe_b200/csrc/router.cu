// Fused gate -> softmax -> top-k -> renormalise router.
//
// Takes over the role of the reference's _top_k_gate_kernel
// (src/blackwell_moe/kernels/routing.py:14-58) and of the torch routing inlined in
// src/blackwell_moe/kernels/fp8_moe_v3.py:34-37.
//
// Selection target: the exact dot products x[t,:].w_gate[:,e] rounded once to fp32,
// ordered by (value descending, expert id ascending).  bf16 x bf16 products are exact in
// fp32, so the only error of an fp32 evaluation is in the additions.  The kernel sums
// blocks of 16 products with plain FMAs and adds the blocks with compensated (Kahan)
// summation, which bounds the error of a logit by about 20 * 2^-24 * sum|x_d * w_de|.
// Tokens for which two neighbouring logits among ranks 1..K+1 are closer than twice that
// bound are re-evaluated in fp64 by the whole block, so the chosen experts and their
// order equal the exactly-rounded ones for every token.  The kernel for small batches
// (router_token_kernel) accumulates in fp64 from the start and needs neither bound nor second pass.
#include <cooperative_groups.h>

#include "common.cuh"

namespace bwmoe {
namespace {
namespace cg = cooperative_groups;

constexpr int kThreads = 256;
constexpr int kChunk = 256;   // D elements staged per step
constexpr int kInner = 16;    // products per plain-FMA block
constexpr int kMaxEJ = 8;     // E <= 32 * kMaxEJ

// Kahan step: (sum, comp) += y.  Kept out of reach of re-association by the intrinsics.
__device__ __forceinline__ void kahan_add(float& sum, float& comp, float y) {
  const float yc = __fsub_rn(y, comp);
  const float t = __fadd_rn(sum, yc);
  comp = __fsub_rn(__fsub_rn(t, sum), yc);
  sum = t;
}

// Top-K (+1) selection of one token by one warp.  Writes weights/indices; returns true when
// two neighbouring selected logits (or the K-th and the best rejected one) are within thr.
// Lane l holds the logits of experts l, l+32, ... (EJ of them); every round takes the best remaining
// (value desc, id asc) with two warp-wide reductions: the largest key, then the lowest id that has it.
template <int EJ>
__device__ __forceinline__ bool select_token_regs(const float* lg_row, int E, int K, float thr_rel, float thr_abs,
                                                  float* w_out, int32_t* i_out, int lane, float* cut_out) {
  unsigned key[EJ];
  float lmax = 0.f;
#pragma unroll
  for (int j = 0; j < EJ; ++j) {
    const int ee = lane + 32 * j;
    const float v = ee < E ? lg_row[ee] : -INFINITY;
    key[j] = ee < E ? order_key(v) : 0u;                 // 0 is below the key of every float
    if (ee < E && fabsf(v) < INFINITY) lmax = fmaxf(lmax, fabsf(v));
  }
  for (int off = 16; off; off >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, off));
  const float thr = thr_abs + lmax * thr_rel;
  bool ambiguous = false;
  float prev = 0.f;
  float chosen_v = 0.f;                                   // lane i keeps the i-th selected (value, id)
  int chosen_i = 0;
  const int rounds = K < E ? K + 1 : K;
  for (int it = 0; it < rounds; ++it) {
    unsigned bk = 0u;
    int bj = 0;
#pragma unroll
    for (int j = 0; j < EJ; ++j)                          // ids ascend with j: the first maximum is the lowest id
      if (key[j] > bk) bk = key[j], bj = j;
    const unsigned top = __reduce_max_sync(0xffffffffu, bk);
    const unsigned mine = (bk == top && top != 0u) ? (unsigned)(lane + 32 * bj) : 0x7fffffffu;
    const int bi = (int)__reduce_min_sync(0xffffffffu, mine);
    const float bv = order_value(top);
    if ((bi & 31) == lane) {
#pragma unroll
      for (int j = 0; j < EJ; ++j)
        if (j == (bi >> 5)) key[j] = 0u;                  // taken
    }
    if (it > 0 && prev - bv <= thr) ambiguous = true;
    prev = bv;
    if (it < K && lane == it) chosen_v = bv, chosen_i = bi;
  }
  // Experts whose approximate logit lies below this cannot reach the top K whatever the rounding did
  // (prev is the best rejected logit, or the K-th one when K == E).
  if (cut_out != nullptr && lane == 0) *cut_out = prev - thr;
  // weights: softmax over the selected logits == softmax over all experts, renormalised
  const float top = __shfl_sync(0xffffffffu, chosen_v, 0);
  const float p = lane < K ? expf(chosen_v - top) : 0.f;
  float z = p;
  for (int off = 16; off; off >>= 1) z += __shfl_xor_sync(0xffffffffu, z, off);
  if (lane < K) {
    w_out[lane] = p / z;
    i_out[lane] = chosen_i;
  }
  return ambiguous;
}
__device__ __forceinline__ bool select_token(const float* lg_row, int E, int K, float thr_rel, float thr_abs,
                                             float* w_out, int32_t* i_out, int lane, float* cut_out = nullptr) {
  if (E <= 32) return select_token_regs<1>(lg_row, E, K, thr_rel, thr_abs, w_out, i_out, lane, cut_out);
  if (E <= 64) return select_token_regs<2>(lg_row, E, K, thr_rel, thr_abs, w_out, i_out, lane, cut_out);
  if (E <= 128) return select_token_regs<4>(lg_row, E, K, thr_rel, thr_abs, w_out, i_out, lane, cut_out);
  return select_token_regs<kMaxEJ>(lg_row, E, K, thr_rel, thr_abs, w_out, i_out, lane, cut_out);
}

// Exact logits of one token in fp64 by the whole block, then rounded once to fp32.
// Threads are laid out as (expert octet ev, d-group dg): each loads 8 gate weights (16 bytes)
// per d.  Needs E % 8 == 0 and w_gate 16-byte aligned; otherwise one expert per thread.
// The partial sums are combined in a fixed order (shuffle tree, then warp by warp).
__device__ void exact_logits_block(const __nv_bfloat16* __restrict__ xrow, const __nv_bfloat16* __restrict__ wg,
                                   int D, int E, float* lg_row, double* dsum /* smem [E] */) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nthreads = blockDim.x;
  const bool vec = (E % 8 == 0) && (E / 8 <= 32) && ((reinterpret_cast<uintptr_t>(wg) & 15u) == 0);
  for (int i = tid; i < E; i += nthreads) dsum[i] = 0.0;
  __syncthreads();
  if (vec) {
    int V = 1;
    while (V < E / 8) V <<= 1;                 // lanes per d, padded to a power of two
    const int ev = tid % V, dg = tid / V, NG = nthreads / V;
    double a[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = 0.0;
    if (ev < E / 8) {
#pragma unroll 4
      for (int d = dg; d < D; d += NG) {
        const double xv = (double)__bfloat162float(xrow[d]);
        const uint4 raw = *reinterpret_cast<const uint4*>(wg + (size_t)d * E + 8 * ev);
        const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(pw[j]);
          a[2 * j] = fma(xv, (double)f.x, a[2 * j]);
          a[2 * j + 1] = fma(xv, (double)f.y, a[2 * j + 1]);
        }
      }
    }
    for (int off = V; off < 32; off <<= 1) {
#pragma unroll
      for (int j = 0; j < 8; ++j) a[j] += __shfl_xor_sync(0xffffffffu, a[j], off);
    }
    for (int w = 0; w < nthreads / 32; ++w) {
      if (warp == w && lane < V && ev < E / 8) {
#pragma unroll
        for (int j = 0; j < 8; ++j) dsum[8 * ev + j] += a[j];
      }
      __syncthreads();
    }
  } else {
    int GE = 8;
    while (GE < E) GE <<= 1;
    if (GE > nthreads) GE = nthreads;
    const int ee = tid % GE, dg = tid / GE, NG = nthreads / GE;
    for (int e0 = 0; e0 < E; e0 += GE) {        // GE < E only when E > blockDim
      double a = 0.0;
      if (e0 + ee < E) {
#pragma unroll 8
        for (int d = dg; d < D; d += NG)
          a = fma((double)__bfloat162float(xrow[d]), (double)__bfloat162float(wg[(size_t)d * E + e0 + ee]), a);
      }
      for (int g = 0; g < NG; ++g) {
        if (dg == g && e0 + ee < E) dsum[e0 + ee] += a;
        __syncthreads();
      }
    }
  }
  for (int i = tid; i < E; i += nthreads) lg_row[i] = (float)dsum[i];
  __syncthreads();
}

// ---------------------------------------------------------------------------------------
// One thread-block cluster per token, for small batches (decode): threads = (expert octet, d-group), the
// d-groups spread over the 1-8 CTAs of the cluster so that a few tokens still pull the gate matrix through
// many SMs at once.  The products (exact in fp32) are accumulated in fp64 - a few thousand DFMAs per SM
// disappear behind the loads here - so the sums ARE the exact logits, rounded once to fp32: no error
// bound, no tie detection, no second pass.  Every CTA reduces its own share in a fixed shuffle tree to
// partial logits in its shared memory; after a cluster barrier CTA 0 adds the partials of its peers in
// rank order (distributed shared memory) and selects.
// ---------------------------------------------------------------------------------------
constexpr int kTokenSmemBytes = 32 * 256 * (int)sizeof(double);     // per-warp partial logits
__global__ void __launch_bounds__(1024)
router_token_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, int T, int D,
                    int E, int K, float* __restrict__ weights, int32_t* __restrict__ indices,
                    float* __restrict__ row_amax) {
  extern __shared__ __align__(16) double token_part[];          // [nwarps][256]
  __shared__ double lgd[256];                                   // this CTA's partial logits
  __shared__ float lg[256];
  __shared__ float s_max[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  cg::cluster_group cluster = cg::this_cluster();
  const int C = (int)cluster.num_blocks(), rank = (int)cluster.block_rank();
  const int tok = blockIdx.x / C;
  const __nv_bfloat16* xrow = x + (size_t)tok * D;
  int V = 1;
  while (V < E / 8) V <<= 1;
  const int NG = blockDim.x / V;                          // d-groups of this CTA
  const int ev = tid % V, dg = rank * NG + tid / V;       // d-group among those of the whole cluster
  const bool ev_ok = ev < E / 8;

  double acc[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.0;
  float xmax = 0.f;
  // A step of a thread: 8 consecutive d (one 16-byte load of x) against its expert octet in those 8 gate rows,
  // so a warp reads whole runs of consecutive rows and all eight row loads are issued before the first is
  // used.  Rows past D multiply by zero and change nothing.
  const bool vec_x = (reinterpret_cast<uintptr_t>(xrow) & 15u) == 0 && D % 8 == 0;
  for (int d = dg * 8; d < D; d += NG * C * 8) {
    float xv[8];
    uint4 raw[8];
    if (vec_x) {
      const uint4 xr = *reinterpret_cast<const uint4*>(xrow + d);
      const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&xr);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(px[q]);
        xv[2 * q] = f.x, xv[2 * q + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) xv[q] = d + q < D ? __bfloat162float(xrow[d + q]) : 0.f;
    }
#pragma unroll
    for (int q = 0; q < 8; ++q)
      raw[q] = (d + q < D && ev_ok) ? *reinterpret_cast<const uint4*>(wg + (size_t)(d + q) * E + 8 * ev)
                                    : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (ev == 0) xmax = fmaxf(xmax, fabsf(xv[q]));
      const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&raw[q]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(pw[j]);
        // a bf16 x bf16 product has 16 significant bits: exact in fp32, and unchanged by the conversion
        acc[2 * j] += (double)__fmul_rn(xv[q], f.x);
        acc[2 * j + 1] += (double)__fmul_rn(xv[q], f.y);
      }
    }
  }
  // d-groups inside the warp, then the warps, then the CTAs: one fixed tree, so the result is reproducible
  for (int off = V; off < 32; off <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
  }
  if (lane < V && ev_ok) {
#pragma unroll
    for (int j = 0; j < 8; ++j) token_part[warp * 256 + 8 * ev + j] = acc[j];
  }
  for (int off = 16; off; off >>= 1) xmax = fmaxf(xmax, __shfl_xor_sync(0xffffffffu, xmax, off));
  if (lane == 0) s_max[warp] = xmax;
  __syncthreads();
  // warp w sums experts w, w + nwarps, ...; lane l brings warp l's part
  for (int e = warp; e < E; e += nwarps) {
    double v = lane < nwarps ? token_part[lane * 256 + e] : 0.0;
    for (int off = 16; off; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    if (lane == 0) lgd[e] = v;
  }
  if (C > 1) {
    cluster.sync();
    if (rank == 0) {
      for (int e = tid; e < E; e += blockDim.x) {
        double v = lgd[e];
        for (int r = 1; r < C; ++r) v += cluster.map_shared_rank(lgd, r)[e];
        lg[e] = (float)v;                                 // the one rounding to fp32
      }
      if (tid < nwarps) {
        float m = s_max[tid];
        for (int r = 1; r < C; ++r) m = fmaxf(m, cluster.map_shared_rank(s_max, r)[tid]);
        s_max[tid] = m;
      }
    }
    cluster.sync();                     // the peers' shared memory has been read: they may leave
    if (rank != 0) return;
  } else {
    __syncthreads();
    for (int e = tid; e < E; e += blockDim.x) lg[e] = (float)lgd[e];
    __syncthreads();
  }
  if (warp == 0) {
    float m_tok = lane < nwarps ? s_max[lane] : 0.f;
    for (int off = 16; off; off >>= 1) m_tok = fmaxf(m_tok, __shfl_xor_sync(0xffffffffu, m_tok, off));
    select_token(lg, E, K, 0.f, -1.f, weights + (size_t)tok * K, indices + (size_t)tok * K, lane);
    if (lane == 0 && row_amax != nullptr) row_amax[tok] = m_tok;
  }
}

// ---------------------------------------------------------------------------------------
// One warp per token, for narrow gates (E <= 16) and large batches: w_gate (<= 128 KiB at
// D=4096) is served by L1, every lane streams its share of the row, no block-level barrier
// sits on the main path.  Lanes are laid out as (expert octet, d-group) like the block kernel.
// ---------------------------------------------------------------------------------------
constexpr int kWarpTokWarps = 8;
__global__ void __launch_bounds__(kWarpTokWarps * 32)
router_warp_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, int T, int D,
                   int E, int K, float* __restrict__ weights, int32_t* __restrict__ indices,
                   float* __restrict__ row_amax) {
  __shared__ float lg[kWarpTokWarps][16];
  __shared__ float s_wnorm;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tok = blockIdx.x * kWarpTokWarps + warp;
  const bool tok_ok = tok < T;
  const __nv_bfloat16* xrow = x + (size_t)(tok_ok ? tok : 0) * D;
  const int V = E > 8 ? 2 : 1;
  const int ev = lane % V, dg = lane / V, NG = 32 / V;
  const bool want_wsq = warp == 0;          // column norms of w_gate: once per block

  float acc[8], comp[8], inner[8], wsq[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f, comp[j] = 0.f, inner[j] = 0.f, wsq[j] = 0.f;
  float xsq = 0.f, xmax = 0.f;
  int inner_n = 0;
  // each step: 8 consecutive d (one 16-byte load of x) against 8 rows of this lane's expert octet
#pragma unroll 2
  for (int d0 = dg * 8; d0 < D; d0 += NG * 8) {
    // x streams past L1 (read once); w_gate is re-read by every warp and should stay in L1
    const uint4 xraw = __ldcg(reinterpret_cast<const uint4*>(xrow + d0));
    uint4 wraw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) wraw[i] = __ldg(reinterpret_cast<const uint4*>(wg + (size_t)(d0 + i) * E + 8 * ev));
    const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&xraw);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float2 xp2 = __bfloat1622float2(px[i >> 1]);
      const float xv = (i & 1) ? xp2.y : xp2.x;
      xsq = fmaf(xv, xv, xsq);
      xmax = fmaxf(xmax, fabsf(xv));
      const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&wraw[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(pw[j]);
        if (want_wsq) {
          wsq[2 * j] = fmaf(f.x, f.x, wsq[2 * j]);
          wsq[2 * j + 1] = fmaf(f.y, f.y, wsq[2 * j + 1]);
        }
        inner[2 * j] = fmaf(xv, f.x, inner[2 * j]);
        inner[2 * j + 1] = fmaf(xv, f.y, inner[2 * j + 1]);
      }
    }
    inner_n += 8;
    if (inner_n == kInner) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        kahan_add(acc[j], comp[j], inner[j]);
        inner[j] = 0.f;
      }
      inner_n = 0;
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    kahan_add(acc[j], comp[j], inner[j]);
    acc[j] = __fsub_rn(acc[j], comp[j]);
  }
  for (int off = V; off < 32; off <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], off);
  }
  if (V == 2) {                       // both octets count the same x: halve the duplicated statistics
    xsq *= 0.5f;
  }
  for (int off = 16; off; off >>= 1) {
    xsq += __shfl_xor_sync(0xffffffffu, xsq, off);
    xmax = fmaxf(xmax, __shfl_xor_sync(0xffffffffu, xmax, off));
  }
  if (want_wsq) {
    float m = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      for (int off = V; off < 32; off <<= 1) wsq[j] += __shfl_xor_sync(0xffffffffu, wsq[j], off);
      m = fmaxf(m, wsq[j]);
    }
    m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));    // the other octet when V == 2
    if (lane == 0) s_wnorm = sqrtf(m) * 1.001f;
  }
  if (lane < V) {
#pragma unroll
    for (int j = 0; j < 8; ++j) lg[warp][8 * ev + j] = acc[j];
  }
  __syncthreads();
  if (!tok_ok) return;
  // blocks of kInner FMAs + compensated outer sum (2) + shuffle tree (<= 5)
  const float gamma = (float)(kInner + 8) * 5.9604645e-8f * 1.05f;
  const float thr_abs = 2.f * gamma * s_wnorm * sqrtf(xsq) * 1.001f;
  const bool amb = select_token(lg[warp], E, K, 1.0e-6f, thr_abs, weights + (size_t)tok * K,
                                indices + (size_t)tok * K, lane);
  if (lane == 0 && row_amax != nullptr) row_amax[tok] = xmax;
  if (!amb) return;
  // near-tie: exact fp64 logits by this warp alone, same lane layout
  double a[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = 0.0;
#pragma unroll 4
  for (int d = dg; d < D; d += NG) {
    const double xv = (double)__bfloat162float(xrow[d]);
    const uint4 raw = *reinterpret_cast<const uint4*>(wg + (size_t)d * E + 8 * ev);
    const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(pw[j]);
      a[2 * j] = fma(xv, (double)f.x, a[2 * j]);
      a[2 * j + 1] = fma(xv, (double)f.y, a[2 * j + 1]);
    }
  }
  for (int off = V; off < 32; off <<= 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += __shfl_xor_sync(0xffffffffu, a[j], off);
  }
  if (lane < V) {
#pragma unroll
    for (int j = 0; j < 8; ++j) lg[warp][8 * ev + j] = (float)a[j];
  }
  __syncwarp();
  select_token(lg[warp], E, K, 0.f, -1.f, weights + (size_t)tok * K, indices + (size_t)tok * K, lane);
}

template <int TOK>
__global__ void __launch_bounds__(kThreads)
router_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, int T, int D,
              int E, int K, int Epad, float* __restrict__ weights, int32_t* __restrict__ indices,
              float* __restrict__ row_amax) {
  // xs: staged activations [kChunk][TOK] fp32; later reused for the cross-slice reduction
  // and (as doubles) for the fp64 partial sums
  __shared__ __align__(16) float xs[kThreads * TOK];
  __shared__ float lg[TOK][256];
  __shared__ float s_abs[TOK], s_max[TOK];
  __shared__ float s_red[kThreads / 32][TOK], s_red2[kThreads / 32][TOK];
  __shared__ float s_wsq[256];         // squared column norms of w_gate
  __shared__ int s_flag[TOK];
  __shared__ int s_nflag;
  static_assert(kChunk == kThreads, "xs is sized for both uses");
  static_assert(kThreads * TOK * sizeof(float) >= kThreads * sizeof(double), "fp64 partials fit in xs");

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok0 = blockIdx.x * TOK;
  const int DS = kThreads / Epad;       // d-slices; thread (e, ds) sums d = ds, ds+DS, ...
  const int e = tid % Epad, ds = tid / Epad;
  const bool e_ok = e < E;
  const bool vec_ok = (D % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
  if (tid == 0) s_nflag = 0;
  s_wsq[tid] = 0.f;

  float acc[TOK], comp[TOK], inner[TOK];
#pragma unroll
  for (int t = 0; t < TOK; ++t) acc[t] = 0.f, comp[t] = 0.f, inner[t] = 0.f;
  float wsq = 0.f, my_abs = 0.f, my_max = 0.f;    // statistics gathered while staging / streaming
  int inner_n = 0;

  for (int c0 = 0; c0 < D; c0 += kChunk) {
    // stage x[tok0..tok0+TOK, c0..c0+kChunk) transposed to [d][token]; a thread always serves
    // token tid % TOK, so its running |x| statistics belong to one token
    if (vec_ok) {
      // 16-byte loads: lanes run over tokens, each taking 8 consecutive d
      for (int idx = tid; idx < (kChunk / 8) * TOK; idx += kThreads) {
        const int t = idx % TOK, dd0 = (idx / TOK) * 8;
        uint4 raw = make_uint4(0u, 0u, 0u, 0u);
        if (tok0 + t < T && c0 + dd0 < D)
          raw = *reinterpret_cast<const uint4*>(x + (size_t)(tok0 + t) * D + c0 + dd0);
        const __nv_bfloat162* pr = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(pr[j]);
          xs[(dd0 + 2 * j) * TOK + t] = f.x;
          xs[(dd0 + 2 * j + 1) * TOK + t] = f.y;
          my_abs = fmaf(f.x, f.x, fmaf(f.y, f.y, my_abs));
          my_max = fmaxf(my_max, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
      }
    } else {
      for (int idx = tid; idx < kChunk * TOK; idx += kThreads) {
        const int t = idx % TOK, dd = idx / TOK;
        float v = 0.f;
        if (tok0 + t < T && c0 + dd < D) v = __bfloat162float(x[(size_t)(tok0 + t) * D + c0 + dd]);
        xs[dd * TOK + t] = v;
        my_abs = fmaf(v, v, my_abs);
        my_max = fmaxf(my_max, fabsf(v));
      }
    }
    __syncthreads();
    const int dlim = min(kChunk, D - c0);
#pragma unroll 4
    for (int dd = ds; dd < dlim; dd += DS) {
      float w = 0.f;
      if (e_ok) w = __bfloat162float(wg[(size_t)(c0 + dd) * E + e]);
      wsq = fmaf(w, w, wsq);
      const float* xr = xs + dd * TOK;
      if constexpr (TOK % 4 == 0) {
#pragma unroll
        for (int t4 = 0; t4 < TOK / 4; ++t4) {
          const float4 xv = reinterpret_cast<const float4*>(xr)[t4];
          inner[4 * t4 + 0] = fmaf(xv.x, w, inner[4 * t4 + 0]);
          inner[4 * t4 + 1] = fmaf(xv.y, w, inner[4 * t4 + 1]);
          inner[4 * t4 + 2] = fmaf(xv.z, w, inner[4 * t4 + 2]);
          inner[4 * t4 + 3] = fmaf(xv.w, w, inner[4 * t4 + 3]);
        }
      } else {
#pragma unroll
        for (int t = 0; t < TOK; ++t) inner[t] = fmaf(xr[t], w, inner[t]);
      }
      if (++inner_n == kInner) {
#pragma unroll
        for (int t = 0; t < TOK; ++t) {
          kahan_add(acc[t], comp[t], inner[t]);
          inner[t] = 0.f;
        }
        inner_n = 0;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int t = 0; t < TOK; ++t) {
    kahan_add(acc[t], comp[t], inner[t]);
    acc[t] = __fsub_rn(acc[t], comp[t]);
  }

  // ---- cross-slice reduction (fixed order, compensated), logits into lg[t][e] ----
#pragma unroll
  for (int t = 0; t < TOK; ++t) xs[(ds * TOK + t) * Epad + e] = acc[t];
  {
    // squared norms and maxima of x per token (lanes l, l+TOK, ... of a warp serve the same token)
    float a = my_abs, m = my_max;
    for (int off = TOK; off < 32; off <<= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, off);
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    }
    if (lane < TOK) {
      s_red[warp][lane] = a;
      s_red2[warp][lane] = m;
    }
    if (e_ok) atomicAdd(&s_wsq[e], wsq);           // only feeds the tie threshold: order does not matter
  }
  __syncthreads();
  for (int idx = tid; idx < TOK * Epad; idx += kThreads) {
    const int t = idx / Epad, ee = idx % Epad;
    float s = 0.f, c = 0.f;
    for (int q = 0; q < DS; ++q) kahan_add(s, c, xs[(q * TOK + t) * Epad + ee]);
    lg[t][ee] = __fsub_rn(s, c);
  }
  if (tid < TOK) {
    float a = 0.f, m = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) a += s_red[w][tid], m = fmaxf(m, s_red2[w][tid]);
    s_abs[tid] = a;
    s_max[tid] = m;
  }
  __syncthreads();
  float w_sq = 0.f;
  for (int i = 0; i < E; ++i) w_sq = fmaxf(w_sq, s_wsq[i]);
  const float w_norm = sqrtf(w_sq) * 1.001f;

  // error of one logit <= (kInner + 4) * 2^-24 * sum|x_d w_de|  (plain-FMA blocks; the compensated
  // additions contribute ~2 ulp of the result, covered by the relative term); a pair of logits
  // can therefore be mis-ordered only when closer than twice that
  const float gamma = (float)(kInner + 4) * 5.9604645e-8f * 1.05f;
  const float thr_rel = 1.0e-6f;   // ~8 ulp of the larger logit: final roundings + fp32 ties after rounding

  // ---- selection pass 1: one warp per token ----
  for (int t = warp; t < TOK; t += kThreads / 32) {
    if (tok0 + t >= T) continue;
    const size_t tok = tok0 + t;
    // Cauchy-Schwarz: sum_d |x_d w_de| <= |x|_2 * |w_e|_2 (s_abs holds the squared norm of x)
    const float thr_abs = 2.f * gamma * w_norm * sqrtf(s_abs[t]);
    const bool amb = select_token(lg[t], E, K, thr_rel, thr_abs, weights + tok * K, indices + tok * K, lane);
    if (lane == 0) {
      if (row_amax != nullptr) row_amax[tok] = s_max[t];
      if (amb) s_flag[atomicAdd(&s_nflag, 1)] = t;
    }
  }
  __syncthreads();
  const int nflag = s_nflag;
  if (nflag == 0) return;

  // ---- near-ties: exact fp64 logits, whole block per flagged token ----
  double* dsum = reinterpret_cast<double*>(xs);          // [E] doubles; xs is free by now
  for (int f = 0; f < nflag; ++f) {
    const int t = s_flag[f];
    exact_logits_block(x + (size_t)(tok0 + t) * D, wg, D, E, lg[t], dsum);
  }
  // ---- selection pass 2 on the exact logits ----
  for (int f = warp; f < nflag; f += kThreads / 32) {
    const int t = s_flag[f];
    const size_t tok = tok0 + t;
    select_token(lg[t], E, K, 0.f, -1.f, weights + tok * K, indices + tok * K, lane);
  }
}

// Exact (fp64) routing of the tokens in a device-side list; used behind the tensor-core router
// for tokens whose candidate list overflowed.  Blocks stride over the list.
__global__ void __launch_bounds__(256)
router_fallback_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, int D, int E,
                       int K, float* __restrict__ weights, int32_t* __restrict__ indices,
                       const int32_t* __restrict__ list, const int32_t* __restrict__ count) {
  chain_wait();
  __shared__ float lg[256];
  __shared__ double dsum[256];
  const int n = *count;
  for (int f = blockIdx.x; f < n; f += gridDim.x) {
    const int tok = list[f];
    exact_logits_block(x + (size_t)tok * D, wg, D, E, lg, dsum);
    if (threadIdx.x < 32)
      select_token(lg, E, K, 0.f, -1.f, weights + (size_t)tok * K, indices + (size_t)tok * K, threadIdx.x);
    __syncthreads();
  }
}

}  // namespace

int launch_router_fallback(const void* x, const void* wg, int T, int D, int E, int K, float* weights,
                           int32_t* indices, const int32_t* list, const int32_t* count, cudaStream_t st) {
  (void)T;
  BWMOE_CUDA_OK(launch_chained(router_fallback_kernel, dim3(64), dim3(256), 0, st, static_cast<const __nv_bfloat16*>(x),
                                             static_cast<const __nv_bfloat16*>(wg), D, E, K, weights, indices, list,
                                             count));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

size_t router_scratch_bytes(int T, int D, int E, int K, int T_as) {
  return router_tc_applicable(T_as > 0 ? T_as : T, D, E, K) ? router_tc_scratch_bytes(T, D, E) : 0;
}

int launch_router(const void* x, const void* wg, int T, int D, int E, int K, float* weights,
                  int32_t* indices, float* row_amax, cudaStream_t st, void* scratch, size_t scratch_bytes,
                  int32_t* status, int T_as) {
  const int Tc = T_as > 0 ? T_as : T;       // the batch size that picks the kernel (launch sizes follow T)
  BWMOE_REQUIRE(T > 0 && D > 0 && E > 0 && K > 0, BWMOE_ERR_BAD_SHAPE, "router: T=%d D=%d E=%d K=%d", T, D, E, K);
  BWMOE_REQUIRE(E <= 256, BWMOE_ERR_UNSUPPORTED, "router: E=%d > 256", E);
  BWMOE_REQUIRE(K <= E && K <= 32, BWMOE_ERR_UNSUPPORTED, "router: K=%d must be <= min(E,32)", K);
  BWMOE_REQUIRE(x && wg && weights && indices, BWMOE_ERR_NULL, "router: null pointer");
  if (router_tc_applicable(Tc, D, E, K) && scratch != nullptr && scratch_bytes >= router_tc_scratch_bytes(T, D, E) &&
      aligned16(x) && aligned16(wg))
    return launch_router_tc(x, wg, T, D, E, K, weights, indices, row_amax, status, scratch, st);
  int Epad = 8;
  while (Epad < E) Epad <<= 1;
  auto xp = static_cast<const __nv_bfloat16*>(x);
  auto wp = static_cast<const __nv_bfloat16*>(wg);
  const bool vec_gate = (E % 8 == 0) && ((reinterpret_cast<uintptr_t>(wg) & 15u) == 0);
  const bool vec_x = (D % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);
  if (vec_gate && vec_x && E <= 16 && Tc >= 1024) {
    router_warp_kernel<<<ceil_div(T, kWarpTokWarps), kWarpTokWarps * 32, 0, counted(st)>>>(xp, wp, T, D, E, K, weights,
                                                                                 indices, row_amax);
  } else if (vec_gate && Tc < 1024 && (long long)Tc * E * D <= (1ll << 26)) {    // fp64 sums: small batches only
    // Few tokens: a cluster of up to 8 CTAs per token (as many as keep the grid within the SMs), and enough
    // threads that every (expert octet, 8 consecutive d) pair has a thread of its own where that fits.
    static unsigned char smem_set[64] = {0};
    BWMOE_CUDA_OK(ensure_dynamic_smem(router_token_kernel, kTokenSmemBytes, smem_set));
    int C = 1;
    while (C < 8 && T * C * 2 <= sm_count()) C *= 2;
    int V = 1;
    while (V < E / 8) V <<= 1;
    int threads = 256;
    while (threads < 1024 && (long long)threads * C < (long long)V * ceil_div(D, 8)) threads *= 2;
    if (T > 64 && E < 128) threads = 256;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(T * C));
    cfg.blockDim = dim3((unsigned)threads);
    cfg.dynamicSmemBytes = kTokenSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)C;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    note_launch();
    BWMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, router_token_kernel, xp, wp, T, D, E, K, weights, indices, row_amax));
  } else if (Tc >= 2048) {       // both token tilings run the same arithmetic per token
    constexpr int TOK = 16;
    router_kernel<TOK><<<ceil_div(T, TOK), kThreads, 0, counted(st)>>>(xp, wp, T, D, E, K, Epad, weights, indices, row_amax);
  } else {
    constexpr int TOK = 4;
    router_kernel<TOK><<<ceil_div(T, TOK), kThreads, 0, counted(st)>>>(xp, wp, T, D, E, K, Epad, weights, indices, row_amax);
  }
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

}  // namespace bwmoe
