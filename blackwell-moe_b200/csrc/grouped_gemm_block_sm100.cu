// Grouped FP8 GEMMs for the 128x128 block-scale recipe (weights: one inverse scale per
// 128x128 block; activations: one per token per 128 consecutive K elements).
//
// The reference has no FP8 kernel for this recipe: its Qwen path dequantises block-FP8 weights
// to bf16 (src/blackwell_moe/runtime/qwen_patch.py:30-40) and runs F.linear per expert
// (qwen_patch.py:108-129).  This kernel keeps the operands in FP8 on the tensor cores and
// applies the scales where the recipe puts them: every 128-wide K block is multiplied on its
// own (tcgen05.mma into a fresh tensor-memory buffer), and the epilogue warps fold the block's
// partial sums into fp32 register accumulators with  acc += partial * (a_inv[row,kb] * w_inv[kb,nb]).
// Two tensor-memory buffers alternate, so the tensor pipe multiplies block kb+1 while block kb
// is being folded in.
//
//   GATE_UP : hq = e4m3(h * s), h = silu(gate) * up with the bf16 rounding points of the
//             per-tensor recipe; s per token per 128 columns of h, computed in the epilogue
//             (a tile's 128 h columns are exactly one group) - no bf16 intermediate is written
//   DOWN    : y = bf16(acc)
//
// CTA = 384 threads in three warpgroups: warp 0 TMA producer, warp 1 MMA issuer (warps 2-3 idle),
// warps 4..11 fold + epilogue (two warps per tensor-memory lane quarter; each thread owns one row
// and 2 x 64 accumulator columns).  The first warpgroup hands most of its registers to the other
// two (setmaxnreg), so that a fold thread can hold its 128 fp32 accumulators and 64 words of
// tensor-memory loads in flight without spilling.
// The scales never stall the fold: a row's activation scales for the NEXT tile are copied into
// shared memory with cp.async while the current tile is folded (three buffers, so that the copy
// never lands in a buffer the partner warp of the same rows may still read), and the per-K-block
// weight scales of a tile sit in registers, one K block per lane, broadcast by a shuffle.
// Every barrier wait is bounded exactly as in the per-tensor kernel.
// Batches with a handful of rows per expert go to the operand-swapped kernel of
// grouped_gemm_block_small_sm100.cu instead (the launchers at the end of this file decide).
#include "sm100_gemm.cuh"

namespace bwmoe {
namespace {
using namespace sm100;

constexpr int NUM_THREADS_BLK = 384;      // 3 warpgroups: {TMA, MMA, 2 idle}, 2 x 4 fold warps
constexpr int FOLD_WARP0 = 4;             // first fold warp
constexpr int REGS_SMALL = 40;            // per thread after setmaxnreg: first warpgroup
constexpr int REGS_FOLD = 232;            //                              fold warpgroups  (128*40 + 256*232 = 384*168)
constexpr int SCALE_KB_MAX = 16;          // K blocks whose activation scales the shared-memory staging holds
constexpr float kGroupAmaxFloor = 1e-4f;

__device__ __forceinline__ void cp_async4(uint32_t dst_smem, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// two fp32 -> bf16 (round to nearest even) -> back to fp32, with one packed conversion
__device__ __forceinline__ void bf16_round2(float& a, float& b) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
  a = __uint_as_float(r << 16);
  b = __uint_as_float(r & 0xffff0000u);
}
// four fp32 -> four E4M3 codes; the conversion saturates at +-448, which is the clamp of the recipe
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(b), "f"(a));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(d), "f"(c));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}

struct BlockGemmParams {
  const int32_t* offsets;   // [E+1]
  const float* a_inv;       // [M, k_blocks] activation inverse scales
  const float* w0_inv;      // [E, k_blocks, nb] gate (or down) block scales
  const float* w1_inv;      // [E, k_blocks, nb] up block scales (GATE_UP only)
  void* out;                // GATE_UP: hq e4m3 [M, N_out];  DOWN: y bf16 [M, N_out]
  float* out_inv;           // GATE_UP: [M, nb] inverse scales of hq
  int32_t* status;
  int E, Kdim, N_out, n_tiles, k_blocks, nb;
  // expert-parallel way back fused into the DOWN epilogue (see HomeRoute); off when n_home == 0
  int n_home = 0;
  const int32_t* home_counts = nullptr;
  const int32_t* home_first = nullptr;
  void* home[kMaxPeers] = {};
};

struct Cursor {
  const int* cum;
  const int* offsets;     // shared-memory copy of the segment offsets
  int E, n_tiles, e;
  __device__ bool locate(int tile, int& expert, int& row0, int& row_end, int& n_idx) {
    while (e < E && tile >= cum[e + 1]) ++e;
    if (e >= E) return false;
    const int seg0 = offsets[e], seg1 = offsets[e + 1];
    const int m_tiles = (seg1 - seg0 + BM - 1) / BM;
    const int within = tile - cum[e];
    n_idx = within / m_tiles;
    row0 = seg0 + (within % m_tiles) * BM;
    row_end = seg1;
    expert = e;
    return true;
  }
};

// acc(2 x fp32) += part(2 x fp32) * scale(2 x fp32): the packed fp32 FMA of sm_100 halves the
// instruction count of the fold, which is what bounds this kernel.
__device__ __forceinline__ void fma2(unsigned long long& acc, uint32_t p0, uint32_t p1, unsigned long long s2) {
  unsigned long long part;
  asm("mov.b64 %0, {%1, %2};" : "=l"(part) : "r"(p0), "r"(p1));
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(part), "l"(s2));
}
__device__ __forceinline__ unsigned long long splat2(float v) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %1};" : "=l"(r) : "r"(__float_as_uint(v)));
  return r;
}
__device__ __forceinline__ float2 unpack2(unsigned long long v) {
  uint32_t lo, hi;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
  return make_float2(__uint_as_float(lo), __uint_as_float(hi));
}

template <bool GATE_UP>
__global__ void __launch_bounds__(NUM_THREADS_BLK, 1)
block_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                  const __grid_constant__ CUtensorMap map_b1, const BlockGemmParams p) {
  chain_wait();
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_cum[257];
  __shared__ int s_off[257];              // segment offsets: every role looks tiles up without touching global memory
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;
  __shared__ float s_amax[2][2][BM];     // [tile parity][column half][row]
  __shared__ int s_seq[2][BM];           // tiles whose amax each (half, row) thread has published
  __shared__ float s_ainv[3][SCALE_KB_MAX][BM];   // [tile % 3][K block][row] activation scales of a tile's rows

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles_base + STAGES * STAGE_BYTES;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * STAGES;
  // accumulator barriers: [K-block parity][column half]; gate/up tiles use the first of each pair for the whole buffer
  const uint32_t bar_tfull = bars + 16 * STAGES, bar_tempty = bar_tfull + 32;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s_abort;

  for (int e = threadIdx.x; e < 256; e += NUM_THREADS_BLK) {
    int t = 0;
    if (e < p.E) {
      const int o0 = p.offsets[e], o1 = p.offsets[e + 1];
      t = ((o1 - o0 + BM - 1) / BM) * p.n_tiles;
      s_off[e] = o0;
      if (e == p.E - 1) s_off[p.E] = o1;
    }
    s_cum[e + 1] = t;
  }
  for (int i = threadIdx.x; i < 2 * BM; i += NUM_THREADS_BLK) (&s_seq[0][0])[i] = 0;
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      // one arrival per fold warp that reads the (half-)buffer: all eight for a gate/up buffer, the four
      // warps that own the column half for a down half-buffer
      mbar_init(bar_tempty + 8 * b, GATE_UP ? 8 : 4);
    }
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

  // Register hand-over between the warpgroups: every warp of a warpgroup executes its instruction, and
  // each does so at the top of its own branch (after a common point the compiler would have to assume
  // the smaller budget for everything that follows).
  if (warp == 0) {
    // ===================== TMA producer =====================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_SMALL));
    if (lane == 0) {
      Cursor cur{s_cum, s_off, p.E, p.n_tiles, 0};
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        int e, row0, row_end, n_idx;
        if (!cur.locate(tile, e, row0, row_end, n_idx)) break;
        const int n0 = GATE_UP ? n_idx * BN_HALF : n_idx * BN;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status))) break;
          const uint32_t sa = tiles_base + stage * STAGE_BYTES;
          const uint32_t full = bar_full + 8 * stage;
          mbar_expect_tx(full, STAGE_BYTES);
          tma_load_2d(sa, &map_a, full, kb * BK, row0);
          tma_load_3d(sa + A_BYTES, &map_b0, full, n0, kb * BK, e);
          if (GATE_UP) tma_load_3d(sa + A_BYTES + B_HALF_BYTES, &map_b1, full, n0, kb * BK, e);
          else         tma_load_3d(sa + A_BYTES + B_HALF_BYTES, &map_b0, full, n0 + BN_HALF, kb * BK, e);
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===================== MMA issuer: one fresh accumulator per K block =====================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_SMALL));
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x) {
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const uint32_t buf = it & 1u, use = it >> 1;
          if constexpr (GATE_UP) {
            // one 256-column accumulator per K block (every fold thread needs gate and up of its columns)
            if (!(ok = mbar_wait_spin(bar_tempty + 16 * buf, (use & 1u) ^ 1u, abort_flag, p.status))) break;
            if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status))) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + buf * BN;
            const uint32_t sa = tiles_base + stage * STAGE_BYTES;
            const uint64_t da = desc_kmajor(sa), db = desc_nmajor(sa + A_BYTES);
#pragma unroll
            for (int k = 0; k < BK / 32; ++k)
              mma_f8(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 256), IDESC, k > 0 ? 1u : 0u);
            mma_commit(bar_tfull + 16 * buf);
          } else {
            // Down tiles: the K block is issued as two 128-column halves, each into its own half-buffer with its
            // own "full" signal.  A fold warp reads one half only, so a half-buffer is recycled as soon as its
            // four readers are done and the fold of the first half runs while the tensor pipe works on the
            // second (measured 8 % faster than whole buffers here; for gate/up tiles, where every warp needs
            // both halves, the extra barrier round per K block cost more than it gave).
            for (uint32_t h = 0; ok && h < 2; ++h) {
              const uint32_t hb = buf * 2 + h;
              if (!(ok = mbar_wait_spin(bar_tempty + 8 * hb, (use & 1u) ^ 1u, abort_flag, p.status))) break;
              if (h == 0 && !(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status))) break;
              tc_fence_after();
              const uint32_t d_tmem = tmem_base + buf * BN + h * BN_HALF;
              const uint32_t sa = tiles_base + stage * STAGE_BYTES;
              const uint64_t da = desc_kmajor(sa), db = desc_nmajor(sa + A_BYTES + h * B_HALF_BYTES);
#pragma unroll
              for (int k = 0; k < BK / 32; ++k)
                mma_f8(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 256), IDESC_HALF, k > 0 ? 1u : 0u);
              mma_commit(bar_tfull + 8 * hb);
            }
          }
          if (!ok) break;
          mma_commit(bar_empty + 8 * stage);
          if (++stage == STAGES) stage = 0, phase ^= 1u;
        }
      }
    }
    __syncwarp();
  } else if (warp < FOLD_WARP0) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS_SMALL));     // idle warps of the first warpgroup
  } else {
    // ===================== fold K blocks into registers, then finish the tile =====================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS_FOLD));
    const int quarter = warp & 3;
    const int half = (warp - FOLD_WARP0) >> 2;        // which 2 x 64 columns this warp owns
    const int r_in_tile = quarter * 32 + lane;
    // accumulator column offsets of this thread's two 64-column chunks
    const int colA = GATE_UP ? half * 64 : half * 128;
    const int colB = GATE_UP ? BN_HALF + half * 64 : half * 128 + 64;
    Cursor cur{s_cum, s_off, p.E, p.n_tiles, 0};
    Cursor ahead{s_cum, s_off, p.E, p.n_tiles, 0};
    uint32_t it = 0, local = 0;
    bool ok = true;
    // Scales staged ahead of the fold when the K loop has 3..16 blocks (with fewer, a fast warp could run two
    // tiles ahead of its partner and overwrite a buffer still in use; with more, the staging does not fit).
    const bool staged = k_blocks >= 3 && k_blocks <= SCALE_KB_MAX;
    const uint32_t ainv_s = smem_u32(&s_ainv[0][0][0]);
    // a tile's scales of row `r_in_tile` -> s_ainv[buf][kb][r_in_tile]; rows past the segment take the first row's
    auto stage_row_scales = [&](uint32_t buf, int row0, int row_end) {
      const int row = row0 + r_in_tile;
      const float* src = p.a_inv + (size_t)(row < row_end ? row : row0) * k_blocks;
      const uint32_t dst = ainv_s + (uint32_t)((buf * SCALE_KB_MAX) * BM + r_in_tile) * 4u;
      for (int kb = 0; kb < k_blocks; ++kb) cp_async4(dst + (uint32_t)(kb * BM) * 4u, src + kb);
    };
    // weight scales of a tile: lane kb holds K block kb's (k_blocks <= 32)
    auto load_w_scales = [&](int e, int n_idx, float& wa, float& wb) {
      const int n0 = GATE_UP ? n_idx * BN_HALF : n_idx * BN;
      const int nbA = GATE_UP ? n_idx : min(n0 / 128 + half, p.nb - 1);
      const size_t at = ((size_t)e * k_blocks + min(lane, k_blocks - 1)) * p.nb + nbA;
      wa = p.w0_inv[at];
      wb = GATE_UP ? p.w1_inv[at] : wa;
    };
    float wA_nx_reg = 0.f, wB_nx_reg = 0.f;
    if (staged && (int)blockIdx.x < total_tiles) {
      int e, row0, row_end, n_idx;
      if (ahead.locate(blockIdx.x, e, row0, row_end, n_idx)) {
        stage_row_scales(0u, row0, row_end);
        load_w_scales(e, n_idx, wA_nx_reg, wB_nx_reg);
      }
      cp_async_commit();
    }
    for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++local) {
      int e, row0, row_end, n_idx;
      if (!cur.locate(tile, e, row0, row_end, n_idx)) break;
      const int row = row0 + r_in_tile;
      const bool row_ok = row < row_end;
      const int n0 = GATE_UP ? n_idx * BN_HALF : n_idx * BN;
      const float wA_reg = wA_nx_reg, wB_reg = wB_nx_reg;
      const float* sa_row = &s_ainv[local % 3u][0][r_in_tile];
      if (staged) {
        // the next tile's scales travel while this tile is folded
        int e2, r2, re2, n2;
        if (tile + (int)gridDim.x < total_tiles && ahead.locate(tile + gridDim.x, e2, r2, re2, n2)) {
          stage_row_scales((local + 1u) % 3u, r2, re2);
          load_w_scales(e2, n2, wA_nx_reg, wB_nx_reg);
        }
        cp_async_commit();
        cp_async_wait_but_one();           // everything but the group just committed has landed: this tile's scales
      }
      unsigned long long accA2[32], accB2[32];      // 2 x 64 fp32 accumulators, packed in pairs
#pragma unroll
      for (int j = 0; j < 32; ++j) accA2[j] = 0ull, accB2[j] = 0ull;
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        const uint32_t buf = it & 1u, use = it >> 1;
        float sA, sB;
        if (staged) {
          const float a = sa_row[kb * BM];
          sA = a * __shfl_sync(0xffffffffu, wA_reg, kb);
          sB = a * __shfl_sync(0xffffffffu, wB_reg, kb);
        } else {
          // weight-scale block column of each chunk
          const int nbA = GATE_UP ? n_idx : min(n0 / 128 + half, p.nb - 1);
          const size_t at = ((size_t)e * k_blocks + kb) * p.nb + nbA;
          const float a = p.a_inv[(size_t)(row_ok ? row : row0) * k_blocks + kb];
          sA = a * p.w0_inv[at];
          sB = GATE_UP ? a * p.w1_inv[at] : sA;
        }
        // barrier pair of this warp's columns: the whole buffer (gate/up), or the half that holds them (down)
        const uint32_t hbA = buf * 2 + (GATE_UP ? 0u : (uint32_t)half);
        ok = mbar_wait_spin(bar_tfull + 8 * hbA, use & 1u, abort_flag, p.status);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
        if constexpr (GATE_UP) {
          // Four 32-column chunks, software-pipelined: the load of chunk i+1 is in flight while chunk i is folded
          // (tcgen05.wait::ld waits for every load issued so far, so each wait is followed by the next load and
          // only then by the FMAs of the chunk that just landed).  The buffer is handed back to the tensor pipe
          // as soon as its last chunk is in registers - before the last chunk's FMAs, which need it no more.
          {
            uint32_t ra[32], rb[32];
            const unsigned long long sA2 = splat2(sA), sB2 = splat2(sB);
            tmem_ld32(t_row + colA, ra);
            tmem_ld_wait();
            tmem_ld32(t_row + colA + 32, rb);
#pragma unroll
            for (int j = 0; j < 16; ++j) fma2(accA2[j], ra[2 * j], ra[2 * j + 1], sA2);
            tmem_ld_wait();
            tmem_ld32(t_row + colB, ra);
#pragma unroll
            for (int j = 0; j < 16; ++j) fma2(accA2[16 + j], rb[2 * j], rb[2 * j + 1], sA2);
            tmem_ld_wait();
            tmem_ld32(t_row + colB + 32, rb);
#pragma unroll
            for (int j = 0; j < 16; ++j) fma2(accB2[j], ra[2 * j], ra[2 * j + 1], sB2);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty + 8 * hbA);
#pragma unroll
            for (int j = 0; j < 16; ++j) fma2(accB2[16 + j], rb[2 * j], rb[2 * j + 1], sB2);
          }
        } else {
          // Down tiles (a K loop of 4-11 blocks, then 64 KiB of output per tile: the stores set the pace) measured
          // 4 % faster with the plain order: two rounds of two loads, the buffer released after the FMAs.
          {
            uint32_t r0[32], r1[32];
            tmem_ld32(t_row + colA, r0);
            tmem_ld32(t_row + colA + 32, r1);
            tmem_ld_wait();
            const unsigned long long s2 = splat2(sA);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              fma2(accA2[j], r0[2 * j], r0[2 * j + 1], s2);
              fma2(accA2[16 + j], r1[2 * j], r1[2 * j + 1], s2);
            }
          }
          {
            uint32_t r0[32], r1[32];
            tmem_ld32(t_row + colB, r0);
            tmem_ld32(t_row + colB + 32, r1);
            tmem_ld_wait();
            const unsigned long long s2 = splat2(sB);
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              fma2(accB2[j], r0[2 * j], r0[2 * j + 1], s2);
              fma2(accB2[16 + j], r1[2 * j], r1[2 * j + 1], s2);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_tempty + 8 * hbA);
        }
      }
      if (!ok) break;
      float accA[64], accB[64];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float2 a = unpack2(accA2[j]), b = unpack2(accB2[j]);
        accA[2 * j] = a.x, accA[2 * j + 1] = a.y;
        accB[2 * j] = b.x, accB[2 * j + 1] = b.y;
      }
      if constexpr (GATE_UP) {
        // h for this thread's 64 columns; the row's group amax needs the other half too
        float amax = 0.f;
#pragma unroll
        for (int j = 0; j < 64; j += 2) {
          float g0 = accA[j], g1 = accA[j + 1], u0 = accB[j], u1 = accB[j + 1];
          bf16_round2(g0, g1);                       // the reference's rounding points: gate, up,
          bf16_round2(u0, u1);
          float a0 = silu_f(g0), a1 = silu_f(g1);
          bf16_round2(a0, a1);                       // silu(gate),
          a0 *= u0, a1 *= u1;
          bf16_round2(a0, a1);                       // and the product
          accA[j] = a0, accA[j + 1] = a1;
          amax = fmaxf(amax, fmaxf(fabsf(a0), fabsf(a1)));
        }
        // publish this half's maximum, then wait (bounded) for the thread that owns the other half of
        // the row.  The parity buffer cannot be overwritten early: its owner reaches tile local+2 only
        // after it has seen this thread's sequence number for tile local+1.
        s_amax[local & 1u][half][r_in_tile] = amax;
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&s_seq[half][r_in_tile]) = (int)local + 1;
        {
          const volatile int* other = &s_seq[half ^ 1][r_in_tile];
          bool seen = *other > (int)local;
          if (!seen) {
            const unsigned long long t0 = global_ns();
            for (uint32_t spin = 1; !(seen = *other > (int)local); ++spin) {
              if ((spin & 255u) == 0u) {
                if (*abort_flag) break;
                if (global_ns() - t0 > WAIT_LIMIT_NS) {
                  *abort_flag = 1;
                  atomicOr(p.status, BWMOE_STATUS_WAIT_TIMEOUT);
                  break;
                }
              }
            }
          }
          ok = __all_sync(0xffffffffu, seen);
          if (!ok) break;
        }
        __threadfence_block();
        amax = fmaxf(amax, *reinterpret_cast<volatile float*>(&s_amax[local & 1u][half ^ 1][r_in_tile]));
        amax = fmaxf(amax, kGroupAmaxFloor);
        const float s = __fmul_rn(__frcp_rn(amax), kFp8Max);   // torch evaluates 448 / amax this way
        if (row_ok) {
          uint8_t* dst = static_cast<uint8_t*>(p.out) + (size_t)row * p.N_out + n0 + half * 64;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (n0 + half * 64 + v * 16 < p.N_out) {
              uint32_t w[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int j = v * 16 + q * 4;
                w[q] = e4m3x4(accA[j] * s, accA[j + 1] * s, accA[j + 2] * s, accA[j + 3] * s);
              }
              reinterpret_cast<uint4*>(dst)[v] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
          if (half == 0) p.out_inv[(size_t)row * p.nb + n_idx] = __fdiv_rn(amax, kFp8Max);
        }
      } else {
        // where this lane's row goes: the local result buffer, or the row's place on its home rank
        __nv_bfloat16* out_row = static_cast<__nv_bfloat16*>(p.out) + (size_t)row * p.N_out;
        if (p.n_home > 0 && row_ok) {
          int j = row - s_off[e], s = 0;
          for (; s < p.n_home - 1; ++s) {
            const int c = p.home_counts[s * p.E + e];
            if (j < c) break;
            j -= c;
          }
          out_row = static_cast<__nv_bfloat16*>(p.home[s]) + (size_t)(p.home_first[s * p.E + e] + j) * p.N_out;
        }
        // transposed stores: the eight lanes of a group exchange 16-byte pieces so that one instruction
        // writes 128 contiguous bytes of each of four rows (16-byte writes cross NVLink at ~140 GB/s only)
        const unsigned ok_rows = __ballot_sync(0xffffffffu, row_ok);
        const int piece = lane & 7;
        unsigned long long row_ptr[8];
        group8_row_pointers(out_row, lane, row_ptr);
#pragma unroll
        for (int part = 0; part < 2; ++part) {          // accA then accB: 64 columns each
          const float* src = part == 0 ? accA : accB;
          uint4 v[8];
#pragma unroll
          for (int pc = 0; pc < 8; ++pc) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              __nv_bfloat162 b2 = __floats2bfloat162_rn(src[pc * 8 + 2 * q], src[pc * 8 + 2 * q + 1]);
              w[q] = *reinterpret_cast<uint32_t*>(&b2);
            }
            v[pc] = make_uint4(w[0], w[1], w[2], w[3]);
          }
          group8_transpose(v, lane);
          const int col = n0 + half * 128 + part * 64 + piece * 8;
          if (col < p.N_out) group8_store(v, row_ptr, ok_rows, lane, col);
        }
      }
    }
    asm volatile("cp.async.wait_all;" ::: "memory");     // no copy into the scale staging may outlive the CTA
  }

  if (*abort_flag) {
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <bool GATE_UP>
int launch_block_gemm(const CUtensorMap& ma, const CUtensorMap& mb0, const CUtensorMap& mb1,
                      const BlockGemmParams& p, int M, cudaStream_t st) {
  static unsigned char smem_set[64] = {0};
  BWMOE_CUDA_OK(ensure_dynamic_smem(block_gemm_kernel<GATE_UP>, SMEM_BYTES, smem_set));
  const long long max_tiles = (long long)(ceil_div(M, BM) + p.E) * p.n_tiles;
  const int grid = (int)std::min<long long>(gemm_sm_budget(), max_tiles);
  BWMOE_CUDA_OK(launch_chained(block_gemm_kernel<GATE_UP>, dim3(grid), dim3(NUM_THREADS_BLK), SMEM_BYTES, st, ma, mb0, mb1,
                               p));
  return BWMOE_OK;
}

// ---- per-token, per-128-element activation quantisation (gather from token order) ----
// q = e4m3(clamp(x * s)), s = 448 / max(amax, 1e-4) (torch's reciprocal-then-multiply),
// inv = max(amax, 1e-4) / 448.  A thread owns 8 elements of kGroupVecs different groups (all loaded
// before the first is used); the 16 threads of a group reduce the maximum with shuffles.
constexpr int kGroupVecs = 4;
// SCATTER: `m` is a token; its codes and scales go to each of its K permuted rows pos[m*K + k] (token-major:
// the row is read and quantised once and written K times - the codes of a row do not depend on the expert).
template <bool SCATTER>
__global__ void __launch_bounds__(256)
quant_group_rows_kernel(const __nv_bfloat16* __restrict__ src, const int32_t* __restrict__ row_slot, int M, int W,
                        int K, uint8_t* __restrict__ dst, float* __restrict__ inv_out,
                        const int32_t* __restrict__ pos) {
  chain_wait();
  const int groups = (W + 127) / 128;
  const unsigned per_block = blockDim.x * kGroupVecs;
  const unsigned chunks_per_row = (groups * 16 + per_block - 1) / per_block;
  const int m = (int)(blockIdx.x / chunks_per_row);
  const int v0 = (int)(blockIdx.x % chunks_per_row) * per_block + threadIdx.x;     // 8-element vector index
  const size_t srow = (!SCATTER && row_slot != nullptr) ? (size_t)(row_slot[m] / K) : (size_t)m;
  const uint4* in = reinterpret_cast<const uint4*>(src + srow * W);
  uint4 raw[kGroupVecs];
#pragma unroll
  for (int i = 0; i < kGroupVecs; ++i) {
    const int v = v0 + i * blockDim.x;
    raw[i] = v * 8 < W ? in[v] : make_uint4(0u, 0u, 0u, 0u);
  }
#pragma unroll
  for (int i = 0; i < kGroupVecs; ++i) {
    const int v = v0 + i * blockDim.x;
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
    float f[8];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = __bfloat1622float2(p[j]);
      f[2 * j] = t.x, f[2 * j + 1] = t.y;
      amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
    }
    for (int off = 8; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off, 16));
    amax = fmaxf(amax, kGroupAmaxFloor);
    const float s = __fmul_rn(__frcp_rn(amax), kFp8Max);
    if (v * 8 < W) {
      const uint32_t lo = (uint32_t)to_e4m3x2(f[0] * s, f[1] * s) | ((uint32_t)to_e4m3x2(f[2] * s, f[3] * s) << 16);
      const uint32_t hi = (uint32_t)to_e4m3x2(f[4] * s, f[5] * s) | ((uint32_t)to_e4m3x2(f[6] * s, f[7] * s) << 16);
      const float inv = __fdiv_rn(amax, kFp8Max);
      if constexpr (SCATTER) {
        for (int k = 0; k < K; ++k) {
          const int row = pos[(size_t)m * K + k];
          if (row < 0) continue;                       // slot with an out-of-range expert: no row
          reinterpret_cast<uint2*>(dst + (size_t)row * W)[v] = make_uint2(lo, hi);
          if ((v & 15) == 0) inv_out[(size_t)row * groups + (v >> 4)] = inv;
        }
      } else {
        reinterpret_cast<uint2*>(dst + (size_t)m * W)[v] = make_uint2(lo, hi);
        if ((v & 15) == 0) inv_out[(size_t)m * groups + (v >> 4)] = inv;
      }
    }
  }
}

// Token-major form for expert parallelism: the codes and group scales of token t go to the place of
// each of its K rows in the owner rank's buffers (row pos[t,k] + delta[expert]); read once, stored K
// times, remote rows as plain peer stores.
__global__ void __launch_bounds__(256)
scatter_quantised_rows_peers_kernel(const uint8_t* __restrict__ xq_tok, const float* __restrict__ inv_tok,
                                    const int32_t* __restrict__ pos, const int32_t* __restrict__ indices,
                                    const int32_t* __restrict__ delta, unsigned T, unsigned D, int K, int groups,
                                    int experts_per_rank, const PeerPtrs xq_dst, const PeerPtrs inv_dst, int rows_cap,
                                    int32_t* __restrict__ status) {
  const unsigned vec_per_row = D / 16;
  const unsigned p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= T * vec_per_row) return;
  const unsigned t = p / vec_per_row, v = p - t * vec_per_row;
  const uint4 codes = reinterpret_cast<const uint4*>(xq_tok + (size_t)t * D)[v];
  const float inv = v < (unsigned)groups ? inv_tok[(size_t)t * groups + v] : 0.f;
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    const int row = pos[(size_t)t * K + k];
    if (row < 0) continue;
    const int e = indices[(size_t)t * K + k];
    const int r = e / experts_per_rank;
    const int dr = row + delta[e];
    if (dr < 0 || dr >= rows_cap) {                // the owner's buffer is smaller than what the ranks send it
      if (v == 0 && status != nullptr) atomicOr(status, BWMOE_STATUS_EP_OVERFLOW);
      continue;
    }
    const size_t dst_row = (size_t)dr;
    reinterpret_cast<uint4*>(static_cast<uint8_t*>(xq_dst.p[r]) + dst_row * D)[v] = codes;
    if (v < (unsigned)groups) static_cast<float*>(inv_dst.p[r])[dst_row * groups + v] = inv;
  }
}

int check_block(const char* who, int M, int D, int H, int E) {
  BWMOE_REQUIRE(M > 0 && D > 0 && H > 0 && E > 0, BWMOE_ERR_BAD_SHAPE, "%s: M=%d D=%d H=%d E=%d", who, M, D, H, E);
  BWMOE_REQUIRE(D % 16 == 0 && H % 16 == 0, BWMOE_ERR_BAD_SHAPE, "%s: D=%d and H=%d must be multiples of 16", who, D, H);
  BWMOE_REQUIRE(E <= 256, BWMOE_ERR_UNSUPPORTED, "%s: E=%d > 256", who, E);
  return BWMOE_OK;
}

}  // namespace

int launch_gather_quant_group(const void* x, const int32_t* row_slot, int M, int D, int K, void* xq, float* x_inv,
                              cudaStream_t st) {
  BWMOE_REQUIRE(M > 0 && D > 0 && K > 0 && D % 16 == 0, BWMOE_ERR_BAD_SHAPE, "gather_quant_group: M=%d D=%d K=%d", M, D, K);
  BWMOE_REQUIRE(x && xq && x_inv, BWMOE_ERR_NULL, "gather_quant_group: null pointer");
  BWMOE_REQUIRE(aligned16(x) && aligned16(xq), BWMOE_ERR_BAD_ALIGN, "gather_quant_group: pointers must be 16-byte aligned");
  const int vecs_per_row = ceil_div(D, 128) * 16;
  int threads = 32;
  while (threads < 256 && threads * kGroupVecs < vecs_per_row) threads <<= 1;
  const unsigned grid = (unsigned)((size_t)M * ceil_div(vecs_per_row, threads * kGroupVecs));
  BWMOE_CUDA_OK(launch_chained(quant_group_rows_kernel<false>, dim3(grid), dim3(threads), 0, st,
                               static_cast<const __nv_bfloat16*>(x), row_slot, M, D, K, static_cast<uint8_t*>(xq), x_inv,
                               nullptr));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

// Token-major quantise + scatter: every token row is read and quantised once and its codes and group scales
// are written to each of its K permuted rows.
int launch_quant_scatter_group(const void* x, const int32_t* pos, int T, int D, int K, void* xq, float* x_inv,
                               cudaStream_t st) {
  BWMOE_REQUIRE(T > 0 && D > 0 && K > 0 && D % 16 == 0, BWMOE_ERR_BAD_SHAPE, "quant_scatter_group: T=%d D=%d K=%d", T, D, K);
  BWMOE_REQUIRE(x && pos && xq && x_inv, BWMOE_ERR_NULL, "quant_scatter_group: null pointer");
  BWMOE_REQUIRE(aligned16(x) && aligned16(xq), BWMOE_ERR_BAD_ALIGN, "quant_scatter_group: pointers must be 16-byte aligned");
  const int vecs_per_row = ceil_div(D, 128) * 16;
  int threads = 32;
  while (threads < 256 && threads * kGroupVecs < vecs_per_row) threads <<= 1;
  const unsigned grid = (unsigned)((size_t)T * ceil_div(vecs_per_row, threads * kGroupVecs));
  BWMOE_CUDA_OK(launch_chained(quant_group_rows_kernel<true>, dim3(grid), dim3(threads), 0, st,
                               static_cast<const __nv_bfloat16*>(x), nullptr, T, D, K, static_cast<uint8_t*>(xq), x_inv, pos));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_gateup_block(const void* xq, const float* x_inv, const int32_t* offsets, const void* wg, const void* wu,
                        const float* inv_g, const float* inv_u, int M, int D, int H, int E, void* hq, float* h_inv,
                        int32_t* status, cudaStream_t st) {
  BWMOE_REQUIRE(xq && x_inv && offsets && wg && wu && inv_g && inv_u && hq && h_inv && status, BWMOE_ERR_NULL,
                "gateup_block: null pointer");
  if (int rc = check_block("gateup_block", M, D, H, E)) return rc;
  BWMOE_REQUIRE(aligned16(xq) && aligned16(hq) && aligned16(wg) && aligned16(wu), BWMOE_ERR_BAD_ALIGN,
                "gateup_block: pointers must be 16-byte aligned");
  if (block_small_applicable(M, D, E))
    return launch_gateup_block_small(xq, x_inv, offsets, wg, wu, inv_g, inv_u, M, D, H, E, hq, h_inv, status, st);
  CUtensorMap ma, mg, mu;
  if (int rc = make_map_a(&ma, xq, M, D)) return rc;
  if (int rc = make_map_b(&mg, wg, E, D, H)) return rc;
  if (int rc = make_map_b(&mu, wu, E, D, H)) return rc;
  BlockGemmParams p{offsets, x_inv, inv_g, inv_u, hq, h_inv, status, E, D, H, ceil_div(H, BN_HALF),
                    ceil_div(D, BK), ceil_div(H, 128)};
  return launch_block_gemm<true>(ma, mg, mu, p, M, st);
}

int launch_down_block(const void* hq, const float* h_inv, const int32_t* offsets, const void* wd,
                      const float* inv_d, int M, int D, int H, int E, void* y, int32_t* status, cudaStream_t st,
                      const HomeRoute* route) {
  BWMOE_REQUIRE(hq && h_inv && offsets && wd && inv_d && y && status, BWMOE_ERR_NULL, "down_block: null pointer");
  if (int rc = check_block("down_block", M, D, H, E)) return rc;
  BWMOE_REQUIRE(aligned16(hq) && aligned16(y) && aligned16(wd), BWMOE_ERR_BAD_ALIGN,
                "down_block: pointers must be 16-byte aligned");
  if (route == nullptr && block_small_applicable(M, H, E))
    return launch_down_block_small(hq, h_inv, offsets, wd, inv_d, M, D, H, E, y, status, st);
  CUtensorMap ma, mb;
  if (int rc = make_map_a(&ma, hq, M, H)) return rc;
  if (int rc = make_map_b(&mb, wd, E, H, D)) return rc;
  BlockGemmParams p{offsets, h_inv, inv_d, nullptr, y, nullptr, status, E, H, D, ceil_div(D, BN),
                    ceil_div(H, BK), ceil_div(D, 128)};
  if (route != nullptr) {
    BWMOE_REQUIRE(route->n_ranks >= 1 && route->n_ranks <= kMaxPeers && route->counts && route->first && route->home,
                  BWMOE_ERR_UNSUPPORTED, "down_block: home route with %d ranks", route->n_ranks);
    p.n_home = route->n_ranks;
    p.home_counts = route->counts;
    p.home_first = route->first;
    for (int r = 0; r < route->n_ranks; ++r) {
      BWMOE_REQUIRE(route->home[r] != nullptr && aligned16(route->home[r]), BWMOE_ERR_BAD_ALIGN,
                    "down_block: result buffer of rank %d", r);
      p.home[r] = route->home[r];
    }
  }
  return launch_block_gemm<false>(ma, mb, mb, p, M, st);
}

int launch_scatter_rows_group_peers(const void* xq_tok, const float* inv_tok, const int32_t* pos,
                                    const int32_t* indices, const int32_t* delta, int T, int D, int K,
                                    int experts_per_rank, void* const* xq_of_rank, void* const* inv_of_rank,
                                    int n_ranks, int rows_cap, int32_t* status, cudaStream_t st) {
  BWMOE_REQUIRE(T > 0 && D > 0 && K > 0 && D % 16 == 0, BWMOE_ERR_BAD_SHAPE, "scatter_rows_group_peers: T=%d D=%d K=%d", T, D, K);
  BWMOE_REQUIRE(n_ranks >= 1 && n_ranks <= kMaxPeers && experts_per_rank >= 1, BWMOE_ERR_UNSUPPORTED,
                "scatter_rows_group_peers: %d ranks (at most %d)", n_ranks, kMaxPeers);
  BWMOE_REQUIRE(xq_tok && inv_tok && pos && indices && delta && xq_of_rank && inv_of_rank, BWMOE_ERR_NULL,
                "scatter_rows_group_peers: null pointer");
  const int groups = ceil_div(D, 128);
  BWMOE_REQUIRE(groups <= D / 16, BWMOE_ERR_BAD_SHAPE, "scatter_rows_group_peers: D=%d too narrow", D);
  PeerPtrs px{}, pi{};
  for (int r = 0; r < n_ranks; ++r) {
    BWMOE_REQUIRE(xq_of_rank[r] && inv_of_rank[r] && aligned16(xq_of_rank[r]), BWMOE_ERR_BAD_ALIGN,
                  "scatter_rows_group_peers: buffers of rank %d", r);
    px.p[r] = xq_of_rank[r];
    pi.p[r] = inv_of_rank[r];
  }
  const size_t n = (size_t)T * (D / 16);
  scatter_quantised_rows_peers_kernel<<<(unsigned)((n + 255) / 256), 256, 0, counted(st)>>>(
      static_cast<const uint8_t*>(xq_tok), inv_tok, pos, indices, delta, T, D, K, groups, experts_per_rank, px, pi,
      rows_cap, status);
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

}  // namespace bwmoe
