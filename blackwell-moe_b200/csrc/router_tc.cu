// Router for wide gates and large batches: logits on the tensor cores, selection exact.
//
// Same contract as the other router kernels (selection on the exactly-rounded fp32 logits,
// ties to the lower expert id; role of src/blackwell_moe/kernels/routing.py:14-79).  Three steps:
//   1. transpose_gate_kernel : w_gate[D,E] -> w_gate^T[E,D] (so that one expert's column is
//                              contiguous) and the squared column norms
//   2. tc_logits_kernel      : logits = x . w_gate with tcgen05.mma kind::f16 (bf16 inputs, fp32
//                              accumulators in tensor memory), written to a [T, E] fp32 scratch
//   3. refine_kernel         : one warp per token.  Warp-wide selection of the 12 best tensor-core
//                              logits, sorted.  Those logits are only trusted to
//                              t = 2^-14 * |x|_2 * |w_e|_2 (four times the worst case of a
//                              truncating fp32 accumulation of 4096 products).  Every expert within
//                              2t of the K-th best is a candidate; candidates more than 2t apart are
//                              certainly in the right order already.  Runs of candidates that are
//                              closer than 2t to a neighbour are recomputed with the blocked
//                              compensated fp32 sum of the SIMT routers (error bound known), and in
//                              fp64 if still within that bound of each other; the final top-K is
//                              read off the mixed list.  A token whose 12 best all fall within the
//                              cut is recomputed over all experts by the exact fallback kernel.
// An expert outside the candidate set has an exact logit below that of K candidates, so the
// result equals the exact selection.
#include "sm100_gemm.cuh"

namespace bwmoe {
namespace {
using namespace sm100;

constexpr int L_CAND = 12;                 // candidates kept per token (K <= 8)
constexpr int R_BK = 64;                   // bf16 K elements per stage (128 bytes)
constexpr int R_A_BYTES = BM * R_BK * 2;   // 16 KiB
constexpr int R_BCHUNK_BYTES = R_BK * 128; // 64 K rows x 64 experts x 2 B = 8 KiB
constexpr int R_STAGE_BYTES = R_A_BYTES + 4 * R_BCHUNK_BYTES;   // 48 KiB (up to 256 experts)
constexpr int R_MAX_STAGES = 2 * STAGES;   // ring depth when a stage holds one expert chunk only
constexpr int R_SMEM_BYTES = STAGES * R_STAGE_BYTES + 1024 + 256;
constexpr float kTcTrust = 6.103515625e-05f;   // 2^-14

// ---- 1. transpose + column norms ------------------------------------------------------
__global__ void __launch_bounds__(256)
transpose_gate_kernel(const __nv_bfloat16* __restrict__ wg, int D, int E, __nv_bfloat16* __restrict__ wgt,
                      float* __restrict__ wnorm2) {
  chain_wait();
  __shared__ __nv_bfloat16 tile[32][33];
  const int d0 = blockIdx.x * 32, e0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;     // 32 x 8
  for (int r = ty; r < 32; r += 8) {
    const int d = d0 + r, e = e0 + tx;
    tile[r][tx] = (d < D && e < E) ? wg[(size_t)d * E + e] : __float2bfloat16(0.f);
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {
    const int e = e0 + r, d = d0 + tx;
    const __nv_bfloat16 v = tile[tx][r];
    if (e < E && d < D) wgt[(size_t)e * D + d] = v;
    float sq = __bfloat162float(v);
    sq *= sq;
    for (int off = 16; off; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
    if (tx == 0 && e < E) atomicAdd(wnorm2 + e, sq);          // feeds thresholds only: order irrelevant
  }
}

// ---- 2. tensor-core logits + per-token candidate list ------------------------------------
struct TcParams {
  float* logits;        // [T, n_mma] fp32
  int32_t* status;
  int T, D, E, n_chunks, n_mma;   // n_chunks = ceil(E/64) weight boxes; n_mma = MMA N (multiple of 16)
  int split_n;                    // 1: a work item is (row tile, one 64-expert chunk) - few row tiles, many SMs
};

__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// bf16 MN-major operand: 64 N-elements (128 bytes) contiguous per K row; next 64 N-elements
// R_BCHUNK_BYTES further (leading offset); 8-K-row groups 1024 bytes apart (stride offset)
__device__ __forceinline__ uint64_t desc_nmajor_bf16(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)(R_BCHUNK_BYTES >> 4) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
tc_logits_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const TcParams p) {
  chain_wait();
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  // With one expert chunk per item a stage is half the size and the ring twice as deep.
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles_base + STAGES * R_STAGE_BYTES;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * R_MAX_STAGES;
  const uint32_t bar_tfull = bars + 16 * R_MAX_STAGES, bar_tempty = bar_tfull + 16;
  const uint32_t n_stages = p.split_n ? R_MAX_STAGES : STAGES;
  const uint32_t stage_bytes = p.split_n ? R_A_BYTES + R_BCHUNK_BYTES : R_STAGE_BYTES;
  const int chunks_per_item = p.split_n ? 1 : p.n_chunks;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s_abort;

  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < R_MAX_STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 4);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int total_tiles = ((p.T + BM - 1) / BM) * (p.split_n ? p.n_chunks : 1);      // work items
  const int k_blocks = (p.D + R_BK - 1) / R_BK;
  const uint32_t stage_tx = R_A_BYTES + chunks_per_item * R_BCHUNK_BYTES;
  // item -> (row tile, first expert chunk, experts of the item rounded up to the MMA's N granularity)
  auto item_of = [&](int item, int& tile, int& c0, int& n_cols) {
    tile = p.split_n ? item / p.n_chunks : item;
    c0 = p.split_n ? item % p.n_chunks : 0;
    n_cols = p.split_n ? min(64, p.n_mma - 64 * c0) : p.n_mma;
  };
  // D=f32, A=B=bf16, A K-major, B MN-major, M=128; N is set per item
  const uint32_t idesc0 = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(BM >> 4) << 24);

  if (warp == 0) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_tiles; item += gridDim.x) {
        int tile, c0, n_cols;
        item_of(item, tile, c0, n_cols);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status))) break;
          const uint32_t sa = tiles_base + stage * stage_bytes;
          const uint32_t full = bar_full + 8 * stage;
          mbar_expect_tx(full, stage_tx);
          tma_load_2d(sa, &map_x, full, kb * R_BK, tile * BM);
          for (int c = 0; c < chunks_per_item; ++c)
            tma_load_2d(sa + R_A_BYTES + c * R_BCHUNK_BYTES, &map_w, full, (c0 + c) * 64, kb * R_BK);
          if (++stage == n_stages) stage = 0, phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, local = 0;
      bool ok = true;
      for (int item = blockIdx.x; ok && item < total_tiles; item += gridDim.x, ++local) {
        int tile, c0, n_cols;
        item_of(item, tile, c0, n_cols);
        const uint32_t idesc = idesc0 | ((uint32_t)(n_cols >> 3) << 17);
        const uint32_t buf = local & 1u, use = local >> 1;
        if (!(ok = mbar_wait(bar_tempty + 8 * buf, (use & 1u) ^ 1u, abort_flag, p.status))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status))) break;
          tc_fence_after();
          const uint32_t sa = tiles_base + stage * stage_bytes;
          const uint64_t da = desc_kmajor(sa), db = desc_nmajor_bf16(sa + R_A_BYTES);
#pragma unroll
          for (int k = 0; k < R_BK / 16; ++k)   // A: +32 bytes per 16 K; B: +16 K rows = 2048 bytes
            mma_bf16(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 128), idesc, (kb | k) != 0 ? 1u : 0u);
          mma_commit(bar_empty + 8 * stage);
          if (++stage == n_stages) stage = 0, phase ^= 1u;
        }
        if (ok) mma_commit(bar_tfull + 8 * buf);
      }
    }
    __syncwarp();
  } else {
    const int quarter = warp & 3;
    const int r_in_tile = quarter * 32 + lane;
    uint32_t local = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < total_tiles; item += gridDim.x, ++local) {
      int tile, c0, n_cols;
      item_of(item, tile, c0, n_cols);
      const uint32_t buf = local & 1u, use = local >> 1;
      ok = mbar_wait(bar_tfull + 8 * buf, use & 1u, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * 256;
      const int row = tile * BM + r_in_tile;
      float* dst = p.logits + (size_t)row * p.n_mma + c0 * 64;
      for (int c = 0; c < n_cols; c += 32) {
        uint32_t r[32];
        tmem_ld32(t_row + c, r);
        tmem_ld_wait();
        if (row < p.T) {
#pragma unroll
          for (int v = 0; v < 8; ++v)
            if (c + 4 * v < n_cols)
              reinterpret_cast<uint4*>(dst + c)[v] = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);
    }
  }
  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// ---- 3. exact refinement of the candidates: one warp per token ------------------------------
constexpr int kInnerR = 16;   // products per plain-FMA block of the recomputation
__device__ __forceinline__ void kahan_add_r(float& sum, float& comp, float y) {
  const float yc = __fsub_rn(y, comp);
  const float t = __fadd_rn(sum, yc);
  comp = __fsub_rn(__fsub_rn(t, sum), yc);
  sum = t;
}

template <int EJ>   // 32 * EJ >= E: logits each lane holds
__global__ void __launch_bounds__(256)
refine_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ wgt,
              const float* __restrict__ wnorm2, const float* __restrict__ logits, int ld_logits, int T, int D,
              int E, int K, float* __restrict__ weights, int32_t* __restrict__ indices,
              float* __restrict__ row_amax, int32_t* __restrict__ fallback_count,
              int32_t* __restrict__ fallback_list) {
  chain_wait();
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= T) return;
  const __nv_bfloat16* xrow = x + (size_t)tok * D;

  // ---- |x|_2, max|x|, largest column norm ----
  float xsq = 0.f, xmax = 0.f;
  for (int d0 = lane * 8; d0 < D; d0 += 256) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xrow + d0);
    const __nv_bfloat162* px = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(px[j]);
      xsq = fmaf(f.x, f.x, fmaf(f.y, f.y, xsq));
      xmax = fmaxf(xmax, fmaxf(fabsf(f.x), fabsf(f.y)));
    }
  }
  for (int off = 16; off; off >>= 1) {
    xsq += __shfl_xor_sync(0xffffffffu, xsq, off);
    xmax = fmaxf(xmax, __shfl_xor_sync(0xffffffffu, xmax, off));
  }
  if (lane == 0 && row_amax != nullptr) row_amax[tok] = xmax;
  float wn2 = 0.f;
  for (int e = lane; e < E; e += 32) wn2 = fmaxf(wn2, wnorm2[e]);
  for (int off = 16; off; off >>= 1) wn2 = fmaxf(wn2, __shfl_xor_sync(0xffffffffu, wn2, off));
  const float xw = sqrtf(xsq) * sqrtf(wn2) * 1.002f;      // >= sum_d |x_d w_de| for every expert
  const float t2 = 2.f * kTcTrust * xw;                   // two logits further apart are ordered for sure

  // ---- the best tensor-core logits, sorted by (value desc, id asc): lane j keeps entry j.  The list
  //      stops at 12 entries, or earlier once an entry past the K-th falls below kth - 2t: nothing
  //      after it can be a candidate. ----
  // (two warp-wide reductions per entry: the largest order-preserving key, then the lowest id that has it)
  unsigned key[EJ];
#pragma unroll
  for (int j = 0; j < EJ; ++j) {
    const int e = lane + 32 * j;
    key[j] = e < E ? order_key(logits[(size_t)tok * ld_logits + e]) : 0u;      // 0: below every float's key
  }
  float cv = -INFINITY;
  int ci = 0x7fffffff;
  const int n_max = E < L_CAND ? E : L_CAND;
  int n_list = 0;
  float kth_tc = 0.f;
  for (int it = 0; it < n_max; ++it) {
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
    if (lane == it) cv = bv, ci = bi;
    n_list = it + 1;
    if (it == K - 1) kth_tc = bv;
    if (it >= K && bv < kth_tc - t2) break;      // warp-uniform: bv is the same in every lane
  }

  // ---- candidates: the list prefix within 2t of the K-th entry ----
  const float kth = __shfl_sync(0xffffffffu, cv, K - 1);
  const unsigned in_mask = __ballot_sync(0xffffffffu, lane < n_list && cv >= kth - t2);
  const int n_cand = __popc(in_mask);
  if (n_cand >= L_CAND && E > L_CAND) {
    // the list may be missing experts that are just as close: all-expert exact kernel
    if (lane == 0) fallback_list[atomicAdd(fallback_count, 1)] = tok;
    return;
  }
  // ---- runs of candidates closer than 2t to a neighbour need exact logits ----
  const float prev = __shfl_up_sync(0xffffffffu, cv, 1);
  const bool close_up = lane > 0 && lane < n_cand && prev - cv <= t2;
  const unsigned up_mask = __ballot_sync(0xffffffffu, close_up);
  const unsigned redo = (up_mask | (up_mask >> 1)) & ((1u << n_cand) - 1u);   // both members of every close pair
  float mine = cv;
  if (redo != 0u) {
    // one candidate at a time (usually two or three): x is re-read from L1, few registers are live
    for (unsigned rm = redo; rm != 0u; rm &= rm - 1u) {        // warp-uniform
      const int c = __ffs(rm) - 1;
      const __nv_bfloat16* wrow = wgt + (size_t)__shfl_sync(0xffffffffu, ci, c) * D;
      float acc = 0.f, comp = 0.f;
      for (int d0 = lane * 8; d0 < D; d0 += 512) {             // two 8-product steps = one plain-FMA block
        const bool two = d0 + 256 < D;
        const uint4 x0 = *reinterpret_cast<const uint4*>(xrow + d0);
        const uint4 w0 = __ldg(reinterpret_cast<const uint4*>(wrow + d0));
        const uint4 x1 = two ? *reinterpret_cast<const uint4*>(xrow + d0 + 256) : make_uint4(0u, 0u, 0u, 0u);
        const uint4 w1 = two ? __ldg(reinterpret_cast<const uint4*>(wrow + d0 + 256)) : make_uint4(0u, 0u, 0u, 0u);
        const __nv_bfloat162* px0 = reinterpret_cast<const __nv_bfloat162*>(&x0);
        const __nv_bfloat162* pw0 = reinterpret_cast<const __nv_bfloat162*>(&w0);
        const __nv_bfloat162* px1 = reinterpret_cast<const __nv_bfloat162*>(&x1);
        const __nv_bfloat162* pw1 = reinterpret_cast<const __nv_bfloat162*>(&w1);
        float inner = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fx = __bfloat1622float2(px0[j]), fw = __bfloat1622float2(pw0[j]);
          inner = fmaf(fx.x, fw.x, inner);
          inner = fmaf(fx.y, fw.y, inner);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 fx = __bfloat1622float2(px1[j]), fw = __bfloat1622float2(pw1[j]);
          inner = fmaf(fx.x, fw.x, inner);
          inner = fmaf(fx.y, fw.y, inner);
        }
        kahan_add_r(acc, comp, inner);
      }
      float sum = __fsub_rn(acc, comp);
      for (int off = 16; off; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
      if (lane == c) mine = sum;
    }
    // recomputed logits carry a known bound; pairs of them still inside it go to fp64
    const float gamma = (float)(kInnerR + 8) * 5.9604645e-8f * 1.05f;
    const float thr = 2.f * gamma * xw + fabsf(kth) * 1.0e-6f + 1e-30f;
    unsigned exact = 0u;
    for (int c = 0; c < L_CAND; ++c) {
      const float vc = __shfl_sync(0xffffffffu, mine, c);
      const bool hit = ((redo >> c) & 1u) && ((redo >> lane) & 1u) && lane < L_CAND && c != lane &&
                       fabsf(vc - mine) <= thr;
      exact |= __ballot_sync(0xffffffffu, hit);
    }
#pragma unroll 1
    for (int c = 0; c < n_cand; ++c) {
      if (!((exact >> c) & 1u)) continue;
      const int e = __shfl_sync(0xffffffffu, ci, c);
      double a = 0.0;
      for (int d = lane; d < D; d += 32)
        a = fma((double)__bfloat162float(xrow[d]), (double)__bfloat162float(wgt[(size_t)e * D + d]), a);
      for (int off = 16; off; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
      if (lane == c) mine = (float)a;
    }
  }
  // ---- final top-K among the candidates: rank = number of candidates ahead of mine ----
  int rank = 0;
  for (int c = 0; c < L_CAND; ++c) {
    const float vc = __shfl_sync(0xffffffffu, mine, c);
    const int ic = __shfl_sync(0xffffffffu, ci, c);
    if (c < n_cand && (vc > mine || (vc == mine && ic < ci))) ++rank;
  }
  const bool chosen = lane < n_cand && rank < K;
  float top = chosen && rank == 0 ? mine : -INFINITY;
  for (int off = 16; off; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
  const float pexp = chosen ? expf(mine - top) : 0.f;
  float z = pexp;
  for (int off = 16; off; off >>= 1) z += __shfl_xor_sync(0xffffffffu, z, off);
  if (chosen) {
    weights[(size_t)tok * K + rank] = pexp / z;
    indices[(size_t)tok * K + rank] = ci;
  }
}

int make_map_bf16(CUtensorMap* map, const void* base, int rows, int cols, int box_cols, int box_rows) {
  auto fn = encode_fn();
  BWMOE_REQUIRE(fn != nullptr, BWMOE_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BWMOE_REQUIRE(r == CUDA_SUCCESS, BWMOE_ERR_CUDA, "cuTensorMapEncodeTiled(bf16 %dx%d) failed: %d", rows, cols, (int)r);
  return BWMOE_OK;
}

struct TcScratch {
  size_t wgt, wnorm2, logits, fb_count, fb_list, total;
};
TcScratch tc_layout(int T, int D, int E) {
  TcScratch s;
  size_t o = 0;
  auto take = [&](size_t bytes) {
    const size_t at = o;
    o = (o + bytes + 255) / 256 * 256;
    return at;
  };
  s.wnorm2 = take(sizeof(float) * E);
  s.fb_count = take(sizeof(int32_t) * 4);
  s.wgt = take((size_t)E * D * 2);
  s.logits = take(sizeof(float) * (size_t)T * (size_t)((E + 15) / 16 * 16));
  s.fb_list = take(sizeof(int32_t) * (size_t)T);
  s.total = o;
  return s;
}

}  // namespace

// D <= 4096: the trust bound kTcTrust on the tensor-core logits is argued for sums of at most 4096
// products; wider hidden sizes take the SIMT routers, whose error bound scales with D by construction.
bool router_tc_applicable(int T, int D, int E, int K) {
  return (T >= 1024 || (T >= 96 && E >= 64)) && E >= 8 && E <= 256 && E % 8 == 0 && K <= 8 && K < E && D % 64 == 0 && D <= 4096;
}

size_t router_tc_scratch_bytes(int T, int D, int E) { return tc_layout(T, D, E).total; }

// Exact router for the tokens the candidate list could not settle (device list, count read on the device).
int launch_router_fallback(const void* x, const void* wg, int T, int D, int E, int K, float* weights,
                           int32_t* indices, const int32_t* list, const int32_t* count, cudaStream_t st);

int launch_router_tc(const void* x, const void* wg, int T, int D, int E, int K, float* weights, int32_t* indices,
                     float* row_amax, int32_t* status, void* scratch, cudaStream_t st) {
  BWMOE_REQUIRE(scratch != nullptr && aligned16(scratch), BWMOE_ERR_WORKSPACE, "router: scratch buffer required");
  BWMOE_REQUIRE(aligned16(x) && aligned16(wg), BWMOE_ERR_BAD_ALIGN, "router: pointers must be 16-byte aligned");
  const TcScratch L = tc_layout(T, D, E);
  uint8_t* base = static_cast<uint8_t*>(scratch);
  auto* wgt = reinterpret_cast<__nv_bfloat16*>(base + L.wgt);
  auto* wnorm2 = reinterpret_cast<float*>(base + L.wnorm2);
  auto* logits = reinterpret_cast<float*>(base + L.logits);
  auto* fb_count = reinterpret_cast<int32_t*>(base + L.fb_count);
  auto* fb_list = reinterpret_cast<int32_t*>(base + L.fb_list);
  BWMOE_CUDA_OK(cudaMemsetAsync(base, 0, L.wgt, st));        // column norms, fallback counter, private status word
  if (status == nullptr) status = fb_count + 1;
  BWMOE_CUDA_OK(launch_chained(transpose_gate_kernel, dim3(ceil_div(D, 32), ceil_div(E, 32)), dim3(256), 0, st,
                               static_cast<const __nv_bfloat16*>(wg), D, E, wgt, wnorm2));
  BWMOE_CUDA_OK(cudaGetLastError());

  CUtensorMap mx, mw;
  if (int rc = make_map_bf16(&mx, x, T, D, R_BK, BM)) return rc;
  if (int rc = make_map_bf16(&mw, wg, D, E, 64, R_BK)) return rc;
  static unsigned char smem_set[64] = {0};
  BWMOE_CUDA_OK(ensure_dynamic_smem(tc_logits_kernel, R_SMEM_BYTES, smem_set));
  TcParams p{logits, status, T, D, E, ceil_div(E, 64), ceil_div(E, 16) * 16, 0};
  // few row tiles: one 64-expert chunk per CTA, so that a small batch is spread over several SMs
  p.split_n = (p.n_chunks > 1 && ceil_div(T, BM) * p.n_chunks * 2 <= sm_count()) ? 1 : 0;
  const int grid = std::min(sm_count(), ceil_div(T, BM) * (p.split_n ? p.n_chunks : 1));
  BWMOE_CUDA_OK(launch_chained(tc_logits_kernel, dim3(grid), dim3(NUM_THREADS), R_SMEM_BYTES, st, mx, mw, p));
  BWMOE_CUDA_OK(cudaGetLastError());
  auto xb = static_cast<const __nv_bfloat16*>(x);
  const unsigned rgrid = (unsigned)ceil_div(T, 8);
  if (E <= 32)
    BWMOE_CUDA_OK(launch_chained(refine_kernel<1>, dim3(rgrid), dim3(256), 0, st, xb, wgt, wnorm2, logits, p.n_mma, T, D, E, K, weights, indices, row_amax,
                                            fb_count, fb_list));
  else if (E <= 64)
    BWMOE_CUDA_OK(launch_chained(refine_kernel<2>, dim3(rgrid), dim3(256), 0, st, xb, wgt, wnorm2, logits, p.n_mma, T, D, E, K, weights, indices, row_amax,
                                            fb_count, fb_list));
  else if (E <= 128)
    BWMOE_CUDA_OK(launch_chained(refine_kernel<4>, dim3(rgrid), dim3(256), 0, st, xb, wgt, wnorm2, logits, p.n_mma, T, D, E, K, weights, indices, row_amax,
                                            fb_count, fb_list));
  else
    BWMOE_CUDA_OK(launch_chained(refine_kernel<8>, dim3(rgrid), dim3(256), 0, st, xb, wgt, wnorm2, logits, p.n_mma, T, D, E, K, weights, indices, row_amax,
                                            fb_count, fb_list));
  BWMOE_CUDA_OK(cudaGetLastError());
  return launch_router_fallback(x, wg, T, D, E, K, weights, indices, fb_list, fb_count, st);
}

}  // namespace bwmoe
