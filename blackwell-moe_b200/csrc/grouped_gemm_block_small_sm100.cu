// Block-scale grouped FP8 GEMMs for small batches (decode): operands swapped.
//
// With a handful of rows per expert, 128-row tiles are almost empty and the per-K-block fold of the
// large-batch kernel (grouped_gemm_block_sm100.cu) works on 128 x 256 accumulators of which a few rows are
// real.  Here the weight tile takes the M side of the MMA and the tokens the N side:
//
//   D^T[128 output features (tensor-memory lanes), 32 tokens (columns)] += W^T[features, k] * X^T[k, tokens]
//
// A = a weight tile exactly as the large-batch kernel stages it ([128 k][128 features], feature-contiguous,
// read MN-major), B = 32 activation rows (K-major).  A tile has two weight tiles that share the activation
// rows - the gate and the up tile of 128 h columns, or two neighbouring 128-feature tiles of the down
// projection (256 contiguous bytes of every weight row) - so one K block is 2 x (128 x 32) accumulators, tensor
// memory holds a ring of eight K blocks and the fold is 64 FMAs per thread per K block with the same
// arithmetic as the large-batch kernel: acc += partial * (a_inv[row,kb] * w_inv[kb,nb]).
// Same roles as there (reference: src/blackwell_moe/runtime/qwen_patch.py:108-129 computes these products
// in bf16 after dequantising).
//
// CTA = 192 threads: warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 fold + epilogue (one per tensor-
// memory lane quarter; a thread owns one output feature and the tile's 32 token columns).  A tile is
// (expert, 32 of its rows, 128 output features); tiles run expert-major, then feature block, then row block.
// Every wait is bounded as in the other GEMM kernels; the fold warps meet on an mbarrier, not on bar.sync,
// so that a warp that gave up cannot strand the others.
#include "sm100_gemm.cuh"

namespace bwmoe {
namespace {
using namespace sm100;

constexpr int S_NT = 32;                          // token columns per tile
constexpr int S_THREADS = 192;
constexpr int S_FOLD_WARP0 = 2;
constexpr int S_X_BYTES = S_NT * BK;              // 4 KiB: 32 rows x 128 K bytes
constexpr int S_BUF_COLS = 64;                    // gate 32 | up 32, or the two feature tiles of a down tile
constexpr int S_NBUF = TMEM_COLS / S_BUF_COLS;    // 8 K blocks in flight in tensor memory
constexpr int S_KB_MAX = 32;                      // K blocks per tile (one weight scale per lane)
constexpr float kSmallAmaxFloor = 1e-4f;
constexpr int S_W_BYTES = 2 * B_HALF_BYTES;                   // two weight tiles per stage
constexpr int S_STAGE_BYTES = S_W_BYTES + S_X_BYTES;          // 36 KiB
constexpr int S_STAGES = 5;
constexpr int S_SMEM_BYTES = S_STAGES * S_STAGE_BYTES + 1024 /*alignment slack*/ + 512 /*barriers*/;
// D=f32, A=B=e4m3, A MN-major (the weight tile), B K-major (the activation rows), N=32, M=128
constexpr uint32_t IDESC_SMALL = (1u << 4) | (1u << 15) | ((uint32_t)(S_NT >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

struct SmallParams {
  const int32_t* offsets;   // [E+1]
  const float* a_inv;       // [M, k_blocks] activation inverse scales
  const float* w0_inv;      // [E, k_blocks, nb] gate (or down) block scales
  const float* w1_inv;      // [E, k_blocks, nb] up block scales (GATE_UP only)
  void* out;                // GATE_UP: hq e4m3 [M, N_out];  DOWN: y bf16 [M, N_out]
  float* out_inv;           // GATE_UP: [M, nb] inverse scales of hq
  int32_t* status;
  int E, N_out, n_ft, k_blocks, nb;
};

struct SmallCursor {
  const int* cum;
  const int* offsets;
  int E, n_ft, e;
  __device__ bool locate(int tile, int& expert, int& row0, int& row_end, int& ft) {
    while (e < E && tile >= cum[e + 1]) ++e;
    if (e >= E) return false;
    const int seg0 = offsets[e], seg1 = offsets[e + 1];
    const int t_tiles = (seg1 - seg0 + S_NT - 1) / S_NT;
    const int within = tile - cum[e];
    ft = within / t_tiles;
    row0 = seg0 + (within % t_tiles) * S_NT;
    row_end = seg1;
    expert = e;
    return true;
  }
};

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ uint8_t e4m3_of(float v) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.f), "f"(v));
  return (uint8_t)(r & 0xffu);
}

template <bool GATE_UP>
__global__ void __launch_bounds__(S_THREADS, 1)
block_gemm_small_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w0,
                        const __grid_constant__ CUtensorMap map_w1, const SmallParams p) {
  chain_wait();
  constexpr int NSTAGE = S_STAGES;
  constexpr int STAGE_SZ = S_STAGE_BYTES;
  constexpr int W_BYTES = S_W_BYTES;
  constexpr int FT_COLS = GATE_UP ? BN_HALF : 2 * BN_HALF;      // output columns a tile covers in its weight tensor(s)
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_cum[257];
  __shared__ int s_off[257];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_xinv[2][S_KB_MAX][S_NT];     // [tile parity][K block][token column]
  __shared__ float s_cmax[2][4][S_NT];            // [tile parity][lane quarter][token column]

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles_base + NSTAGE * STAGE_SZ;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * NSTAGE;
  const uint32_t bar_tfull = bars + 16 * NSTAGE, bar_tempty = bar_tfull + 8 * S_NBUF;
  const uint32_t bar_fold = bar_tempty + 8 * S_NBUF;            // where the four fold warps meet
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s_abort;

  for (int e = threadIdx.x; e < 256; e += S_THREADS) {
    int t = 0;
    if (e < p.E) {
      const int o0 = p.offsets[e], o1 = p.offsets[e + 1];
      t = ((o1 - o0 + S_NT - 1) / S_NT) * p.n_ft;
      s_off[e] = o0;
      if (e == p.E - 1) s_off[p.E] = o1;
    }
    s_cum[e + 1] = t;
  }
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < S_NBUF; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, 4);
    }
    mbar_init(bar_fold, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    int v[8], run = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      run += s_cum[1 + lane * 8 + j];
      v[j] = run;
    }
    int incl = run;
    for (int off = 1; off < 32; off <<= 1) {
      const int o = __shfl_up_sync(0xffffffffu, incl, off);
      if (lane >= off) incl += o;
    }
    const int base = incl - run;
#pragma unroll
    for (int j = 0; j < 8; ++j) s_cum[1 + lane * 8 + j] = base + v[j];
    if (lane == 0) s_cum[0] = 0;
  }
  if (warp == 1) tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int total_tiles = s_cum[p.E];
  const int k_blocks = p.k_blocks;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      SmallCursor cur{s_cum, s_off, p.E, p.n_ft, 0};
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        int e, row0, row_end, ft;
        if (!cur.locate(tile, e, row0, row_end, ft)) break;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status))) break;
          const uint32_t sw = tiles_base + stage * STAGE_SZ;
          const uint32_t full = bar_full + 8 * stage;
          mbar_expect_tx(full, STAGE_SZ);
          tma_load_3d(sw, &map_w0, full, ft * FT_COLS, kb * BK, e);
          if (GATE_UP) tma_load_3d(sw + B_HALF_BYTES, &map_w1, full, ft * FT_COLS, kb * BK, e);
          else         tma_load_3d(sw + B_HALF_BYTES, &map_w0, full, ft * FT_COLS + BN_HALF, kb * BK, e);
          tma_load_2d(sw + W_BYTES, &map_x, full, kb * BK, row0);
          if (++stage == NSTAGE) stage = 0, phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer: one fresh 32-column accumulator (gate/up: two) per K block =====================
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t buf = it % S_NBUF, use = it / S_NBUF;
          if (!(ok = mbar_wait(bar_tempty + 8 * buf, (use & 1u) ^ 1u, abort_flag, p.status))) break;
          if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status))) break;
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * S_BUF_COLS;
          const uint32_t sw = tiles_base + stage * STAGE_SZ;
          const uint64_t db = desc_kmajor(sw + W_BYTES);
          const uint64_t da0 = desc_nmajor(sw);
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)       // weights: +32 K rows = 4096 bytes; activations: +32 bytes along K
            mma_f8(d_tmem, da0 + (uint64_t)(k * 256), db + (uint64_t)(k * 2), IDESC_SMALL, k > 0 ? 1u : 0u);
          const uint64_t da1 = desc_nmajor(sw + B_HALF_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 32; ++k)
            mma_f8(d_tmem + S_NT, da1 + (uint64_t)(k * 256), db + (uint64_t)(k * 2), IDESC_SMALL, k > 0 ? 1u : 0u);
          mma_commit(bar_empty + 8 * stage);
          mma_commit(bar_tfull + 8 * buf);
          if (++stage == NSTAGE) stage = 0, phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else {
    // ===================== fold K blocks into registers, then finish the tile =====================
    const int quarter = warp & 3;
    const int f_in_tile = quarter * 32 + lane;              // output feature of this thread inside the tile
    const int fold_tid = (warp - S_FOLD_WARP0) * 32 + lane;
    SmallCursor cur{s_cum, s_off, p.E, p.n_ft, 0};
    uint32_t it = 0, local = 0, fold_phase = 0;
    bool ok = true;
    // the four fold warps meet here (bounded like every other wait)
    auto fold_sync = [&]() -> bool {
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_fold);
      bool good = mbar_wait(bar_fold, fold_phase, abort_flag, p.status);
      fold_phase ^= 1u;
      return __all_sync(0xffffffffu, good);
    };
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local) {
      int e, row0, row_end, ft;
      if (!cur.locate(tile, e, row0, row_end, ft)) break;
      const int n_valid = min(S_NT, row_end - row0);
      const uint32_t par = local & 1u;
      // activation scales of the tile's rows: [K block][column]; rows past the segment take the first row's
      for (int i = fold_tid; i < S_NT * k_blocks; i += 128) {
        const int c = i / k_blocks, kb = i - c * k_blocks;
        s_xinv[par][kb][c] = p.a_inv[(size_t)(row0 + (c < n_valid ? c : 0)) * k_blocks + kb];
      }
      // weight scales of the tile: lane kb holds K block kb's
      float w0_reg, w1_reg;
      {
        const size_t at = ((size_t)e * k_blocks + min(lane, k_blocks - 1)) * p.nb;
        if (GATE_UP) {
          w0_reg = p.w0_inv[at + min(ft, p.nb - 1)];
          w1_reg = p.w1_inv[at + min(ft, p.nb - 1)];
        } else {
          w0_reg = p.w0_inv[at + min(2 * ft, p.nb - 1)];
          w1_reg = p.w0_inv[at + min(2 * ft + 1, p.nb - 1)];
        }
      }
      if (!(ok = fold_sync())) break;
      float acc0[S_NT], acc1[S_NT];
#pragma unroll
      for (int c = 0; c < S_NT; ++c) acc0[c] = 0.f, acc1[c] = 0.f;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const uint32_t buf = it % S_NBUF, use = it / S_NBUF;
        const float w0 = __shfl_sync(0xffffffffu, w0_reg, kb);
        const float w1 = __shfl_sync(0xffffffffu, w1_reg, kb);
        ok = mbar_wait(bar_tfull + 8 * buf, use & 1u, abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * S_BUF_COLS;
        uint32_t r0[32], r1[32];
        tmem_ld32(t_row, r0);
        tmem_ld32(t_row + S_NT, r1);
        tmem_ld_wait();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * buf);      // the loads have landed: the buffer may be reused
        const float* xs = s_xinv[par][kb];
#pragma unroll
        for (int c = 0; c < S_NT; ++c) {
          const float a = xs[c];
          acc0[c] = fmaf(__uint_as_float(r0[c]), a * w0, acc0[c]);
          acc1[c] = fmaf(__uint_as_float(r1[c]), a * w1, acc1[c]);
        }
      }
      if (!ok) break;
      const int n0 = ft * FT_COLS;
      const bool f_ok = n0 + f_in_tile < p.N_out;
      if constexpr (GATE_UP) {
        // h = silu(gate) * up with the recipe's bf16 rounding points; one quantisation group = this tile's
        // 128 features of a token, so the group maximum is a maximum over the 128 lanes of the four warps
#pragma unroll
        for (int c = 0; c < S_NT; ++c) {
          const float g = bf16r(acc0[c]), u = bf16r(acc1[c]);
          const float a = bf16r(silu_f(g));
          const float h = f_ok ? bf16r(a * u) : 0.f;
          acc0[c] = h;
          const unsigned m = __reduce_max_sync(0xffffffffu, __float_as_uint(fabsf(h)));   // |h| >= 0: bit order = value order
          if (lane == 0) s_cmax[par][quarter][c] = __uint_as_float(m);
        }
        if (!(ok = fold_sync())) break;
        uint8_t* out = static_cast<uint8_t*>(p.out);
#pragma unroll
        for (int c = 0; c < S_NT; ++c) {
          float amax = fmaxf(fmaxf(s_cmax[par][0][c], s_cmax[par][1][c]), fmaxf(s_cmax[par][2][c], s_cmax[par][3][c]));
          amax = fmaxf(amax, kSmallAmaxFloor);
          const float s = __fmul_rn(__frcp_rn(amax), kFp8Max);   // torch evaluates 448 / amax this way
          if (c < n_valid) {
            if (f_ok) out[(size_t)(row0 + c) * p.N_out + n0 + f_in_tile] = e4m3_of(acc0[c] * s);
            if (f_in_tile == c) p.out_inv[(size_t)(row0 + c) * p.nb + ft] = __fdiv_rn(amax, kFp8Max);
          }
        }
      } else {
        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
        const bool f1_ok = n0 + BN_HALF + f_in_tile < p.N_out;
#pragma unroll
        for (int c = 0; c < S_NT; ++c) {
          if (c < n_valid) {
            __nv_bfloat16* row = out + (size_t)(row0 + c) * p.N_out + n0 + f_in_tile;
            if (f_ok) row[0] = __float2bfloat16_rn(acc0[c]);
            if (f1_ok) row[BN_HALF] = __float2bfloat16_rn(acc1[c]);
          }
        }
      }
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

// activations [rows, kdim] e4m3 row-major: box 128 (K) x 32 (rows), 128-byte swizzle
int make_map_x32(CUtensorMap* map, const void* base, int rows, int kdim) {
  if (tensor_map_lookup(2, base, rows, kdim, 0, map)) return BWMOE_OK;
  auto fn = encode_fn();
  BWMOE_REQUIRE(fn != nullptr, BWMOE_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)kdim, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)kdim};
  cuuint32_t box[2] = {BK, S_NT};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BWMOE_REQUIRE(r == CUDA_SUCCESS, BWMOE_ERR_CUDA, "cuTensorMapEncodeTiled(X: rows=%d k=%d) failed: %d", rows, kdim, (int)r);
  tensor_map_store(2, base, rows, kdim, 0, *map);
  return BWMOE_OK;
}

template <bool GATE_UP>
int launch_small(const CUtensorMap& mx, const CUtensorMap& mw0, const CUtensorMap& mw1, const SmallParams& p, int M,
                 cudaStream_t st) {
  static unsigned char smem_set[64] = {0};
  BWMOE_CUDA_OK(ensure_dynamic_smem(block_gemm_small_kernel<GATE_UP>, S_SMEM_BYTES, smem_set));
  const long long max_tiles = (long long)(ceil_div(M, S_NT) + p.E) * p.n_ft;
  const int grid = (int)std::min<long long>(gemm_sm_budget(), max_tiles);
  BWMOE_CUDA_OK(launch_chained(block_gemm_small_kernel<GATE_UP>, dim3(grid), dim3(S_THREADS), S_SMEM_BYTES, st, mx, mw0,
                               mw1, p));
  return BWMOE_OK;
}

}  // namespace

// A handful of rows per expert, and a K loop whose weight scales fit one per lane
bool block_small_applicable(int M, int Kdim, int E) {
  return M <= 4096 && M <= 8 * E && ceil_div(Kdim, BK) <= S_KB_MAX;
}

int launch_gateup_block_small(const void* xq, const float* x_inv, const int32_t* offsets, const void* wg, const void* wu,
                              const float* inv_g, const float* inv_u, int M, int D, int H, int E, void* hq,
                              float* h_inv, int32_t* status, cudaStream_t st) {
  CUtensorMap mx, mg, mu;
  if (int rc = make_map_x32(&mx, xq, M, D)) return rc;
  if (int rc = make_map_b(&mg, wg, E, D, H)) return rc;
  if (int rc = make_map_b(&mu, wu, E, D, H)) return rc;
  SmallParams p{offsets, x_inv, inv_g, inv_u, hq, h_inv, status, E, H, ceil_div(H, BN_HALF), ceil_div(D, BK),
                ceil_div(H, 128)};
  return launch_small<true>(mx, mg, mu, p, M, st);
}

int launch_down_block_small(const void* hq, const float* h_inv, const int32_t* offsets, const void* wd,
                            const float* inv_d, int M, int D, int H, int E, void* y, int32_t* status, cudaStream_t st) {
  CUtensorMap mx, mw;
  if (int rc = make_map_x32(&mx, hq, M, H)) return rc;
  if (int rc = make_map_b(&mw, wd, E, H, D)) return rc;
  SmallParams p{offsets, h_inv, inv_d, nullptr, y, nullptr, status, E, D, ceil_div(D, 2 * BN_HALF), ceil_div(H, BK),
                ceil_div(D, 128)};
  return launch_small<false>(mx, mw, mw, p, M, st);
}

}  // namespace bwmoe
