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
                 int32_t* __restrict__ pos, int32_t* __restrict__ row_slot, int32_t* __restrict__ row_expert) {
  extern __shared__ int cnt[];            // [32 warps][E] counts of this round, then exclusive prefixes
  __shared__ int round_base[kMaxE];       // slots of earlier rounds in this block, per expert
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
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
      // total of this round is added to round_base after everyone has read it
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
}

__global__ void segment_scales_kernel(const float* __restrict__ seg_amax, const int32_t* __restrict__ offsets,
                                      int E, float* __restrict__ scales) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= E) return;
  const bool empty = offsets != nullptr && offsets[e + 1] <= offsets[e];
  scales[e] = empty ? 1.0f : scale_from_amax(seg_amax[e]);
}

// ---- row-wise bf16 -> e4m3 with a per-row-selected scale; one thread per 8 elements, one block per row chunk ----
// SRC_BY_SLOT: source row = row_slot[m] / K (gather from token order); else source row = m.
// FROM_AMAX: `scales` holds the segment amax; the scale is derived here and published to scales_out.
constexpr int kQuantVecs = 4;   // 16-byte vectors in flight per thread
template <bool SRC_BY_SLOT, bool FROM_AMAX>
__global__ void __launch_bounds__(256)
quant_rows_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ row_slot,
                  const int32_t* __restrict__ row_expert, const float* __restrict__ scales,
                  float* __restrict__ scales_out, int M, int W, int K, uint8_t* __restrict__ dst) {
  // a block serves one chunk of one row: blockIdx.x = row * chunks_per_row + chunk (one uniform
  // division); a thread converts up to kQuantVecs vectors, all loaded before the first is used
  const int vec_per_row = W / 8;
  const unsigned per_block = blockDim.x * kQuantVecs;
  const unsigned chunks_per_row = (vec_per_row + per_block - 1) / per_block;
  const int m = (int)(blockIdx.x / chunks_per_row);
  const int v0 = (int)(blockIdx.x % chunks_per_row) * per_block + threadIdx.x;
  // Two dependent round trips, not three: the row's data is requested as soon as its source row is
  // known, and the scale (expert id -> scale) is fetched while the data is in flight.
  const int expert = row_expert[m];
  const size_t srow = SRC_BY_SLOT ? (size_t)(row_slot[m] / K) : (size_t)m;
  const uint4* in = reinterpret_cast<const uint4*>(src + srow * W);
  uint2* out = reinterpret_cast<uint2*>(dst + (size_t)m * W);
  uint4 raw[kQuantVecs];
#pragma unroll
  for (int i = 0; i < kQuantVecs; ++i) {
    const int v = v0 + i * blockDim.x;
    raw[i] = v < vec_per_row ? in[v] : make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("" ::: "memory");                 // keep the scale load behind the data loads
  float scale = scales[expert];
  if (FROM_AMAX) {
    scale = scale_from_amax(scale);
    if (v0 == 0) scales_out[expert] = scale;     // every row of the segment writes the same value
  }
#pragma unroll
  for (int i = 0; i < kQuantVecs; ++i) {
    const int v = v0 + i * blockDim.x;
    if (v >= vec_per_row) break;
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
    uint32_t lo, hi;
    {
      const float2 a = __bfloat1622float2(p[0]), b = __bfloat1622float2(p[1]);
      lo = (uint32_t)to_e4m3x2(a.x * scale, a.y * scale) | ((uint32_t)to_e4m3x2(b.x * scale, b.y * scale) << 16);
    }
    {
      const float2 a = __bfloat1622float2(p[2]), b = __bfloat1622float2(p[3]);
      hi = (uint32_t)to_e4m3x2(a.x * scale, a.y * scale) | ((uint32_t)to_e4m3x2(b.x * scale, b.y * scale) << 16);
    }
    out[v] = make_uint2(lo, hi);
  }
}

// ---- out[t,:] = bf16( sum_k float( bf16( y[pos[t*K+k],:] * bf16(w[t,k]) ) ) ) ----
// Optional tail (the block glue of FP8MoELayer.forward, src/blackwell_moe/runtime/deepseek_patch.py:51-53):
//   out = bf16( bf16(routed * scale) + residual ) with routed = the bf16 sum above.
__global__ void __launch_bounds__(256)
combine_kernel(const __nv_bfloat16* __restrict__ y, const int32_t* __restrict__ pos,
               const float* __restrict__ weights, int T, int D, int K, __nv_bfloat16* __restrict__ out,
               float scale, const __nv_bfloat16* __restrict__ residual) {
  const int vec_per_row = D / 8;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (size_t)T * vec_per_row) return;
  const int t = (int)(gid / vec_per_row), v = (int)(gid % vec_per_row);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  for (int k = 0; k < K; ++k) {
    const int p = pos[(size_t)t * K + k];
    if (p < 0) continue;
    const float w = bf16_round(weights[(size_t)t * K + k]);
    const uint4 raw = reinterpret_cast<const uint4*>(y + (size_t)p * D)[v];
    const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(q[i]);
      acc[2 * i] += bf16_round(f.x * w);
      acc[2 * i + 1] += bf16_round(f.y * w);
    }
  }
  if (scale != 1.0f) {
    const float sb = bf16_round(scale);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = bf16_round(bf16_round(acc[i]) * sb);
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
  uint4 o;
  __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) op[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
  reinterpret_cast<uint4*>(out + (size_t)t * D)[v] = o;
}

}  // namespace

inline int quant_block_threads(int vec_per_row) {
  int t = 32;
  while (t < 256 && t * kQuantVecs < vec_per_row) t <<= 1;
  return t;
}
inline unsigned quant_grid(int M, int vec_per_row, int threads) {
  const int per_block = threads * kQuantVecs;
  return (unsigned)((size_t)M * ((vec_per_row + per_block - 1) / per_block));
}

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
    plan_small_kernel<<<1, kPlanThreads, (size_t)32 * E * sizeof(int), st>>>(
        indices, row_amax, M, E, K, offsets, pos, row_slot, row_expert, seg_amax, scales_out, status);
    BWMOE_CUDA_OK(cudaGetLastError());
    return BWMOE_OK;
  }
  const int B = ceil_div(M, kSlotsPerBlock);
  int32_t* block_hist = static_cast<int32_t*>(scratch);
  if (seg_amax != nullptr) BWMOE_CUDA_OK(cudaMemsetAsync(seg_amax, 0, sizeof(float) * E, st));
  plan_hist_kernel<<<B, kPlanThreads, 0, st>>>(indices, row_amax, M, E, K, block_hist,
                                               row_amax ? seg_amax : nullptr, status);
  plan_scan_kernel<<<1, kMaxE, 0, st>>>(block_hist, B, E, offsets);
  const size_t smem = (size_t)33 * E * sizeof(int);
  plan_rank_kernel<<<B, kPlanThreads, smem, st>>>(indices, M, E, block_hist, pos, row_slot, row_expert);
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
  segment_scales_kernel<<<ceil_div(E, 128), 128, 0, st>>>(seg_amax, offsets, E, scales);
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_gather_quant(const void* x, const int32_t* row_slot, const int32_t* row_expert,
                        const float* scales, int M, int D, int K, void* xq, cudaStream_t st) {
  BWMOE_REQUIRE(M > 0 && D > 0 && K > 0 && D % 16 == 0, BWMOE_ERR_BAD_SHAPE, "gather_quant: M=%d D=%d K=%d", M, D, K);
  BWMOE_REQUIRE(x && row_slot && row_expert && scales && xq, BWMOE_ERR_NULL, "gather_quant: null pointer");
  BWMOE_REQUIRE(aligned16(x) && aligned16(xq), BWMOE_ERR_BAD_ALIGN, "gather_quant: pointers must be 16-byte aligned");
  const int threads = quant_block_threads(D / 8);
  quant_rows_kernel<true, false><<<quant_grid(M, D / 8, threads), threads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), row_slot, row_expert, scales, nullptr, M, D, K, static_cast<uint8_t*>(xq));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_requant(const void* h, const int32_t* row_expert, const float* scales_h, int M, int H,
                   void* hq, cudaStream_t st, float* scales_from_amax_out) {
  BWMOE_REQUIRE(M > 0 && H > 0 && H % 16 == 0, BWMOE_ERR_BAD_SHAPE, "requant: M=%d H=%d", M, H);
  BWMOE_REQUIRE(h && row_expert && scales_h && hq, BWMOE_ERR_NULL, "requant: null pointer");
  BWMOE_REQUIRE(aligned16(h) && aligned16(hq), BWMOE_ERR_BAD_ALIGN, "requant: pointers must be 16-byte aligned");
  const int threads = quant_block_threads(H / 8);
  const unsigned grid = quant_grid(M, H / 8, threads);
  if (scales_from_amax_out != nullptr)   // scales_h holds the segment amax; scales are derived and published
    quant_rows_kernel<false, true><<<grid, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(h), nullptr, row_expert,
                                                         scales_h, scales_from_amax_out, M, H, 1,
                                                         static_cast<uint8_t*>(hq));
  else
    quant_rows_kernel<false, false><<<grid, threads, 0, st>>>(static_cast<const __nv_bfloat16*>(h), nullptr, row_expert,
                                                          scales_h, nullptr, M, H, 1, static_cast<uint8_t*>(hq));
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
  dense_prepare_kernel<<<1, 1024, 0, st>>>(row_amax, T, offsets, seg_amax);
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

// rows in place (no gather), scale derived from the segment amax and published
int launch_quant_rows_from_amax(const void* x, const int32_t* row_expert, const float* seg_amax, int M, int W,
                                void* xq, float* scales_out, cudaStream_t st) {
  const int threads = quant_block_threads(W / 8);
  quant_rows_kernel<false, true><<<quant_grid(M, W / 8, threads), threads, 0, st>>>(
      static_cast<const __nv_bfloat16*>(x), nullptr, row_expert, seg_amax, scales_out, M, W, 1,
      static_cast<uint8_t*>(xq));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_combine(const void* y, const int32_t* pos, const float* weights, int T, int D, int K,
                   void* out, cudaStream_t st, float scale, const void* residual) {
  BWMOE_REQUIRE(T > 0 && D > 0 && K > 0 && D % 8 == 0, BWMOE_ERR_BAD_SHAPE, "combine: T=%d D=%d K=%d", T, D, K);
  BWMOE_REQUIRE(y && pos && weights && out, BWMOE_ERR_NULL, "combine: null pointer");
  BWMOE_REQUIRE(aligned16(y) && aligned16(out), BWMOE_ERR_BAD_ALIGN, "combine: pointers must be 16-byte aligned");
  const size_t n = (size_t)T * (D / 8);
  combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(y), pos,
                                                              weights, T, D, K,
                                                              static_cast<__nv_bfloat16*>(out), scale,
                                                              static_cast<const __nv_bfloat16*>(residual));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

}  // namespace bwmoe
