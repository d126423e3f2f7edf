// Fused gate -> softmax -> top-k -> renormalise router.
//
// Takes over the role of the reference's _top_k_gate_kernel
// (src/blackwell_moe/kernels/routing.py:14-58) and of the torch routing inlined in
// src/blackwell_moe/kernels/fp8_moe_v3.py:34-37.
//
// Selection target: the exact dot products x[t,:].w_gate[:,e] rounded once to fp32,
// ordered by (value descending, expert id ascending).  The kernel accumulates in
// fp32 with a two-level blocked sum whose worst-case error is known, and re-evaluates
// in fp64 only the tokens for which two neighbouring logits among ranks 1..K+1 are
// closer than that error bound, so the chosen experts and their order equal the
// exactly-rounded ones for every token.
#include "common.cuh"

namespace bwmoe {
namespace {

constexpr int kThreads = 256;
constexpr int kChunk = 256;   // D elements staged per step
constexpr int kInner = 32;    // terms per first-level partial sum
constexpr int kMaxEJ = 8;     // E <= 32 * kMaxEJ

struct Cand {
  float v;
  int i;
};
// true when a ranks ahead of b: larger value, or equal value and lower id
__device__ __forceinline__ bool ahead(const Cand& a, const Cand& b) {
  return a.v > b.v || (a.v == b.v && a.i < b.i);
}

template <int TOK>
__global__ void __launch_bounds__(kThreads)
router_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wg, int T, int D,
              int E, int K, int Epad, float* __restrict__ weights, int32_t* __restrict__ indices,
              float* __restrict__ row_amax) {
  // xs: staged activations [kChunk][TOK] fp32; reused afterwards for the cross-slice reduction
  __shared__ __align__(16) float xs[kChunk * TOK > kThreads * TOK ? kChunk * TOK : kThreads * TOK];
  __shared__ float lg[TOK][256];
  __shared__ float s_abs[TOK], s_max[TOK];
  __shared__ float s_red[kThreads / 32][TOK], s_red2[kThreads / 32][TOK];
  __shared__ float s_wmax[kThreads / 32];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok0 = blockIdx.x * TOK;
  const int DS = kThreads / Epad;       // d-slices; thread (e, ds) sums d = ds, ds+DS, ...
  const int e = tid % Epad, ds = tid / Epad;
  const bool e_ok = e < E;
  const bool vec_ok = (D % 8 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15u) == 0);

  float acc[TOK], inner[TOK];
#pragma unroll
  for (int t = 0; t < TOK; ++t) acc[t] = 0.f, inner[t] = 0.f;
  float wmax = 0.f, my_abs = 0.f, my_max = 0.f;   // staging-side statistics of x
  int inner_n = 0;

  for (int c0 = 0; c0 < D; c0 += kChunk) {
    // stage x[tok0..tok0+TOK, c0..c0+kChunk) transposed to [d][token]; a thread always serves
    // token tid % TOK, so its running |x| statistics belong to one token
    if (vec_ok) {
      // 16-byte loads: lanes run over tokens, each taking 8 consecutive d; two lanes share a 32-byte sector
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
          my_abs += fabsf(f.x) + fabsf(f.y);
          my_max = fmaxf(my_max, fmaxf(fabsf(f.x), fabsf(f.y)));
        }
      }
    } else {
      for (int idx = tid; idx < kChunk * TOK; idx += kThreads) {
        const int t = idx % TOK, dd = idx / TOK;
        float v = 0.f;
        if (tok0 + t < T && c0 + dd < D) v = __bfloat162float(x[(size_t)(tok0 + t) * D + c0 + dd]);
        xs[dd * TOK + t] = v;
        my_abs += fabsf(v);
        my_max = fmaxf(my_max, fabsf(v));
      }
    }
    __syncthreads();
    const int dlim = min(kChunk, D - c0);
    for (int dd = ds; dd < dlim; dd += DS) {
      float w = 0.f;
      if (e_ok) w = __bfloat162float(wg[(size_t)(c0 + dd) * E + e]);
      wmax = fmaxf(wmax, fabsf(w));
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
        for (int t = 0; t < TOK; ++t) acc[t] += inner[t], inner[t] = 0.f;
        inner_n = 0;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int t = 0; t < TOK; ++t) acc[t] += inner[t];

  // ---- cross-slice reduction (fixed order), logits into lg[t][e] ----
#pragma unroll
  for (int t = 0; t < TOK; ++t) xs[(ds * TOK + t) * Epad + e] = acc[t];
  // statistics: |x| sums and maxima per token; max |w_gate|
  {
    // thread's staged elements all belong to token tid % TOK; lanes l and l+TOK (if TOK<32) share it
    float a = my_abs, m = my_max;
    for (int off = TOK; off < 32; off <<= 1) {
      a += __shfl_xor_sync(0xffffffffu, a, off);
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    }
    if (TOK >= 32 ? true : lane < TOK) {
      // TOK <= 32 is guaranteed by the launcher
      s_red[warp][lane % TOK] = a;
      s_red2[warp][lane % TOK] = m;
    }
    float wm = wmax;
    for (int off = 16; off; off >>= 1) wm = fmaxf(wm, __shfl_xor_sync(0xffffffffu, wm, off));
    if (lane == 0) s_wmax[warp] = wm;
  }
  __syncthreads();
  for (int idx = tid; idx < TOK * Epad; idx += kThreads) {
    const int t = idx / Epad, ee = idx % Epad;
    float s = 0.f;
    for (int q = 0; q < DS; ++q) s += xs[(q * TOK + t) * Epad + ee];
    lg[t][ee] = s;
  }
  if (tid < TOK) {
    float a = 0.f, m = 0.f;
    for (int w = 0; w < kThreads / 32; ++w) a += s_red[w][tid], m = fmaxf(m, s_red2[w][tid]);
    s_abs[tid] = a;
    s_max[tid] = m;
  }
  __syncthreads();
  float wm_all = 0.f;
  for (int w = 0; w < kThreads / 32; ++w) wm_all = fmaxf(wm_all, s_wmax[w]);

  // worst-case bound of the blocked fp32 sum: (inner terms + outer blocks + slices) * 2^-24
  const int per_thread = (D + DS - 1) / DS;
  const float gamma = (float)(kInner + 8 + (per_thread + kInner - 1) / kInner + DS) * 5.9604645e-8f * 1.02f;

  // ---- selection: one warp per token ----
  for (int t = warp; t < TOK; t += kThreads / 32) {
    if (tok0 + t >= T) continue;
    const size_t tok = tok0 + t;
    bool exact = false;
    Cand chosen = {0.f, 0};     // lane i keeps the i-th selected (value, id)
    float vals_next = 0.f;
    for (int pass = 0; pass < 2; ++pass) {
      float v[kMaxEJ];
      float lmax = 0.f;
#pragma unroll
      for (int j = 0; j < kMaxEJ; ++j) {
        const int ee = lane + 32 * j;
        v[j] = ee < E ? lg[t][ee] : -INFINITY;
        if (ee < E) lmax = fmaxf(lmax, fabsf(v[j]));
      }
      for (int off = 16; off; off >>= 1) lmax = fmaxf(lmax, __shfl_xor_sync(0xffffffffu, lmax, off));
      const float thr = 2.f * gamma * wm_all * s_abs[t] + lmax * 4.8e-7f;
      unsigned taken = 0;
      bool ambiguous = false;
      float prev = 0.f;
      const int rounds = K < E ? K + 1 : K;
      for (int it = 0; it < rounds; ++it) {
        Cand best = {-INFINITY, 0x7fffffff};
#pragma unroll
        for (int j = 0; j < kMaxEJ; ++j) {
          Cand c = {v[j], lane + 32 * j};
          if (!((taken >> j) & 1u) && lane + 32 * j < E && ahead(c, best)) best = c;
        }
        for (int off = 16; off; off >>= 1) {
          Cand o = {__shfl_xor_sync(0xffffffffu, best.v, off), __shfl_xor_sync(0xffffffffu, best.i, off)};
          if (ahead(o, best)) best = o;
        }
        if ((best.i & 31) == lane) taken |= 1u << (best.i >> 5);
        if (it > 0 && prev - best.v <= thr) ambiguous = true;
        prev = best.v;
        if (it < K) {
          if (lane == it) chosen = best;
        } else {
          vals_next = best.v;
        }
      }
      (void)vals_next;
      if (!ambiguous || exact) break;
      // near-tie: exact fp64 logits for this token, lanes over experts
      double accd[kMaxEJ];
#pragma unroll
      for (int j = 0; j < kMaxEJ; ++j) accd[j] = 0.0;
      for (int d = 0; d < D; ++d) {
        const double xv = (double)__bfloat162float(x[tok * D + d]);
#pragma unroll
        for (int j = 0; j < kMaxEJ; ++j) {
          const int ee = lane + 32 * j;
          if (ee < E) accd[j] = fma(xv, (double)__bfloat162float(wg[(size_t)d * E + ee]), accd[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxEJ; ++j) {
        const int ee = lane + 32 * j;
        if (ee < E) lg[t][ee] = (float)accd[j];
      }
      __syncwarp();
      exact = true;
    }
    // weights: softmax over the selected logits == softmax over all, renormalised
    const float top = __shfl_sync(0xffffffffu, chosen.v, 0);
    float p = lane < K ? expf(chosen.v - top) : 0.f;
    float z = p;
    for (int off = 16; off; off >>= 1) z += __shfl_xor_sync(0xffffffffu, z, off);
    if (lane < K) {
      weights[tok * K + lane] = p / z;
      indices[tok * K + lane] = chosen.i;
    }
    if (row_amax != nullptr && lane == 0) row_amax[tok] = s_max[t];
  }
}

}  // namespace

int launch_router(const void* x, const void* wg, int T, int D, int E, int K, float* weights,
                  int32_t* indices, float* row_amax, cudaStream_t st) {
  BWMOE_REQUIRE(T > 0 && D > 0 && E > 0 && K > 0, BWMOE_ERR_BAD_SHAPE, "router: T=%d D=%d E=%d K=%d", T, D, E, K);
  BWMOE_REQUIRE(E <= 256, BWMOE_ERR_UNSUPPORTED, "router: E=%d > 256", E);
  BWMOE_REQUIRE(K <= E && K <= 32, BWMOE_ERR_UNSUPPORTED, "router: K=%d must be <= min(E,32)", K);
  BWMOE_REQUIRE(x && wg && weights && indices, BWMOE_ERR_NULL, "router: null pointer");
  int Epad = 8;
  while (Epad < E) Epad <<= 1;
  auto xp = static_cast<const __nv_bfloat16*>(x);
  auto wp = static_cast<const __nv_bfloat16*>(wg);
  if (T >= 2048) {
    constexpr int TOK = 16;
    router_kernel<TOK><<<ceil_div(T, TOK), kThreads, 0, st>>>(xp, wp, T, D, E, K, Epad, weights, indices, row_amax);
  } else {
    constexpr int TOK = 4;
    router_kernel<TOK><<<ceil_div(T, TOK), kThreads, 0, st>>>(xp, wp, T, D, E, K, Epad, weights, indices, row_amax);
  }
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

}  // namespace bwmoe
