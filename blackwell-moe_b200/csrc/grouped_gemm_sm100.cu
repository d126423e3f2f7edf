// Grouped FP8 (E4M3) GEMMs of the MoE block on the 5th-generation tensor cores.
//
// One persistent, warp-specialised kernel template serves both projections:
//   GATE_UP : [rows of expert e] x (Wg[e] | Wu[e])  ->  h = silu(gate) * up   (bf16) + segment amax
//   DOWN    : [rows of expert e] x Wd[e]            ->  y                     (bf16)
// Takes over the roles of the reference's Triton kernels _fused_gate_up_kernel
// (src/blackwell_moe/kernels/grouped_fp8_gateup.py:42-101) and _grouped_fp8_gemm_kernel
// (src/blackwell_moe/kernels/grouped_fp8.py:36-89), and of F.silu(gate)*up
// (src/blackwell_moe/kernels/fp8_moe_v3.py:60).
//
// Structure per CTA (320 threads, one CTA per SM):
//   warp 0      : TMA producer - activations (K-major) and weights (N-major, as the
//                 caller's [E,K,N] layout dictates) into a 4-stage 128B-swizzled ring
//   warp 1      : tcgen05.mma issuer, kind::f8f6f4, M=128 N=256 K=32, fp32 accumulators
//                 in tensor memory, two 256-column buffers so that the epilogue of tile i
//                 overlaps the main loop of tile i+1
//   warps 2..9  : epilogue, two warps per tensor-memory lane quarter with half of the tile's
//                 columns each - tcgen05.ld, dequantise, SwiGLU / bf16 rounding (DOWN: times the
//                 row's routing weight), stores transposed across lane groups so that every
//                 store instruction writes whole 128-byte lines (or, for the combine by
//                 reduction, 16-byte vector bf16 reductions into the token's output row)
// A tile is 128 permuted rows of ONE expert x 256 accumulator columns (GATE_UP: 128 gate +
// 128 up columns -> 128 h columns; DOWN: 256 output columns).  Tiles are ordered expert-major,
// then column block, then row block, so that concurrently running CTAs share weight tiles
// and an expert's activations stay in L2 while its weights stream through once.
//
// Large batches run the DOWN projection on CTA pairs (two-CTA clusters, cta_group::2, 256-row tiles; see the
// kernel's PAIR parameter); everything else runs one CTA per tile.
//
// Every barrier wait is bounded: when a wait runs out the kernel sets
// BWMOE_STATUS_WAIT_TIMEOUT in the status word, tells the other warps to stop, waits for
// copies in flight, frees its tensor memory and returns.
#include "sm100_gemm.cuh"

namespace bwmoe {
namespace {
using namespace sm100;


struct GemmParams {
  const int32_t* offsets;   // [E+1]
  const float* scale_a;     // [E] activation scale per segment
  const float* scale_b0;    // [E] weight scale (gate, or down)
  const float* scale_b1;    // [E] weight scale (up); unused for DOWN
  void* out;                // GATE_UP: h bf16 [M, N_out];  DOWN: y bf16 [M, N_out]
  float* seg_amax;          // GATE_UP: [E] amax of h per segment
  int32_t* status;
  int E, Kdim, N_out, n_tiles;
  // split-K mode (RAW kernels): every tile covers `k_per_split` K blocks and dumps its fp32
  // accumulators into slab `split` of `partial` ([split_k][M][ldp] floats) for a later fixed-order sum
  int split_k, k_per_split, M, ldp;
  float* partial;
  // Expert-parallel way back fused into the DOWN epilogue (n_home > 0): the rows of segment e are the
  // rows ranks 0..n_home-1 sent, in that order; home_counts[s*E+e] of them came from rank s and return
  // to rows home_first[s*E+e] ... of rank s's result buffer home[s] (peer stores; the own rank's are local).
  int n_home = 0;
  const int32_t* home_counts = nullptr;
  const int32_t* home_first = nullptr;
  void* home[8] = {};
  // Weighted combine in the DOWN epilogue (row_w != nullptr): every finished row is multiplied by the routing
  // weight of its slot, bf16(bf16(y) * bf16(w)) - the product the combine would form.  With tok_out set as
  // well, the weighted row is added straight into out[token] with vector bf16 reductions (token =
  // row_slot[row] / top_k; out zeroed beforehand) and no result row is written at all.
  const float* row_w = nullptr;
  const int32_t* row_slot = nullptr;
  void* tok_out = nullptr;
  int top_k = 1;
};


// tile index -> (expert, first row, end of segment, column block); every role walks the
// same monotone sequence, so a forward-moving expert cursor suffices.
struct TileCursor {
  const int* cum;       // smem [E+1]: tiles before expert e
  const int32_t* offsets;
  int E, n_tiles, e;
  int bm = BM;          // rows per tile: 128, or 256 when a CTA pair shares the tile
  __device__ bool locate(int tile, int& expert, int& row0, int& row_end, int& n_idx, int& split) {
    while (e < E && tile >= cum[e + 1]) ++e;
    if (e >= E) return false;
    const int seg0 = offsets[e], seg1 = offsets[e + 1];
    const int m_tiles = (seg1 - seg0 + bm - 1) / bm;
    const int within = tile - cum[e];
    const int rest = within / m_tiles;
    n_idx = rest % n_tiles;
    split = rest / n_tiles;
    row0 = seg0 + (within % m_tiles) * bm;
    row_end = seg1;
    expert = e;
    return true;
  }
};

// Eight epilogue warps: two per tensor-memory lane quarter, each taking half of the tile's columns.
// With four, the short K loops (K = 1408: 11 blocks) finished before the previous tile's 64 KiB of
// output had left the SM, and the MMA warp waited for its accumulator buffer.
constexpr int EPI_WARPS = 8;
constexpr int GEMM_THREADS = 64 + 32 * EPI_WARPS;

// PAIR: the CTAs of a two-CTA cluster share 256-row tiles (cta_group::2).  CTA `rank` of the pair loads rows
// rank*128.. of the tile and one 128-column half of the weight tile (GATE_UP: rank 0 the gate box, rank 1 the
// up box), so every weight byte enters one of the two shared memories only; the even CTA issues M=256 MMAs
// that read both shared memories and write each CTA's 128 rows into that CTA's tensor memory.  Stages are
// 32 KiB per CTA, so the ring is six deep.  Barriers: loads of both CTAs report to the even CTA's full
// barrier; the issuer commits to the stage's empty barrier and to the accumulator's full barrier of each CTA
// in turn; the odd CTA's epilogue warps hand accumulator buffers back on the even CTA's barrier.
// Measured inside whole forwards on one B200 (same process order, both builds twice): the down projection
// gains 2 % (Mixtral shape, 16384 tokens: 1531 -> 1498 us; DeepSeek shape: 373 -> 365 us), the gate/up
// projection loses 2-5 % (2863 -> 2910 us; 1476 -> 1548 us at 8192 tokens), so the launcher pairs the down
// projection only.  Both forms run with the SM clock already lowered by the power limit (1.55 GHz of 1.97
// at 71-77 % tensor-pipe activity), which is why halving the weight traffic into shared memory buys so little.
template <bool GATE_UP, bool RAW, bool PAIR>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b0,
                    const __grid_constant__ CUtensorMap map_b1, const GemmParams p) {
  chain_wait();
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_cum[257];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_abort;

  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles_base = (raw + 1023u) & ~1023u;
  static_assert(!(PAIR && RAW), "split-K tiles are not paired");
  constexpr int NSTAGE = PAIR ? PAIR_STAGES : STAGES;
  constexpr int STAGE_SZ = PAIR ? PAIR_STAGE_BYTES : STAGE_BYTES;
  constexpr int TILE_ROWS = PAIR ? 2 * BM : BM;
  const uint32_t bars = tiles_base + NSTAGE * STAGE_SZ;
  const uint32_t bar_full = bars, bar_empty = bars + 8 * NSTAGE;
  const uint32_t bar_tfull = bars + 16 * NSTAGE, bar_tempty = bar_tfull + 16;
  const uint32_t rank = PAIR ? cluster_ctarank() : 0u;            // place in the pair
  const int first_tile = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
  const int tile_step = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &s_abort;

  // ---- set-up ----
  // tiles before each expert: every thread fetches the segments it owns, warp 0 scans
  for (int e = threadIdx.x; e < 256; e += GEMM_THREADS) {
    int t = 0;
    if (e < p.E) {
      const int rows = p.offsets[e + 1] - p.offsets[e];
      t = ((rows + TILE_ROWS - 1) / TILE_ROWS) * p.n_tiles * p.split_k;
    }
    s_cum[e + 1] = t;
  }
  if (threadIdx.x == 0) {
    s_abort = 0;
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_tfull + 8 * b, 1);
      mbar_init(bar_tempty + 8 * b, PAIR ? 2 * EPI_WARPS : EPI_WARPS);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  if (warp == 0) {
    // inclusive scan of s_cum[1..256]: 8 values per lane, then a shuffle scan of the lane totals
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
  if (warp == 1) {
    if constexpr (PAIR) tmem_alloc_pair(smem_u32(&s_tmem_base), TMEM_COLS);
    else                tmem_alloc(smem_u32(&s_tmem_base), TMEM_COLS);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();       // the peer's barriers and tensor memory exist from here on
  tc_fence_after();
  const uint32_t tmem_base = s_tmem_base;
  const int total_tiles = s_cum[p.E];
  const int k_blocks = (p.Kdim + BK - 1) / BK;

  if (warp == 0) {
    // ===================== TMA producer =====================
    if (lane == 0) {
      TileCursor cur{s_cum, p.offsets, p.E, p.n_tiles, 0, TILE_ROWS};
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step) {
        int e, row0, row_end, n_idx, split;
        if (!cur.locate(tile, e, row0, row_end, n_idx, split)) break;
        const int n0 = GATE_UP ? n_idx * BN_HALF : n_idx * BN;
        const int kb0 = split * p.k_per_split, kb1 = min(k_blocks, kb0 + p.k_per_split);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!(ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status))) break;
          const uint32_t sa = tiles_base + stage * STAGE_SZ;
          const uint32_t full = bar_full + 8 * stage;
          if constexpr (PAIR) {
            // both CTAs' bytes are counted by the even CTA's barrier, which alone announces them
            const uint32_t full_even = map_to_cta(full, 0);
            if (rank == 0) mbar_expect_tx(full, 2 * PAIR_STAGE_BYTES);
            tma_load_2d_pair(sa, &map_a, full_even, kb * BK, row0 + (int)rank * BM);
            if (GATE_UP) tma_load_3d_pair(sa + A_BYTES, rank ? &map_b1 : &map_b0, full_even, n0, kb * BK, e);
            else         tma_load_3d_pair(sa + A_BYTES, &map_b0, full_even, n0 + (int)rank * BN_HALF, kb * BK, e);
          } else {
            mbar_expect_tx(full, STAGE_BYTES);
            tma_load_2d(sa, &map_a, full, kb * BK, row0);
            tma_load_3d(sa + A_BYTES, &map_b0, full, n0, kb * BK, e);
            if (GATE_UP) tma_load_3d(sa + A_BYTES + B_HALF_BYTES, &map_b1, full, n0, kb * BK, e);
            else         tma_load_3d(sa + A_BYTES + B_HALF_BYTES, &map_b0, full, n0 + BN_HALF, kb * BK, e);
          }
          if (++stage == NSTAGE) stage = 0, phase ^= 1u;
        }
      }
      if constexpr (PAIR) {
        // the issuer's last commits arrive on this CTA's empty barriers from the other CTA: let them land
        // before this CTA can leave
        for (int i = 0; ok && i < NSTAGE; ++i) {
          ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1u, abort_flag, p.status);
          if (++stage == NSTAGE) stage = 0, phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ===================== MMA issuer =====================
    if (lane == 0 && rank == 0) {
      uint32_t stage = 0, phase = 0, local = 0;
      bool ok = true;
      TileCursor cur{s_cum, p.offsets, p.E, p.n_tiles, 0, TILE_ROWS};
      for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step, ++local) {
        int e, row0, row_end, n_idx, split;
        if (!cur.locate(tile, e, row0, row_end, n_idx, split)) break;
        const int kb0 = split * p.k_per_split, kb1 = min(k_blocks, kb0 + p.k_per_split);
        const uint32_t buf = local & 1u, use = local >> 1;
        // wait until the epilogue has drained this accumulator buffer (first use passes at once)
        if (!(ok = mbar_wait(bar_tempty + 8 * buf, (use & 1u) ^ 1u, abort_flag, p.status))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!(ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status))) break;
          tc_fence_after();
          const uint32_t sa = tiles_base + stage * STAGE_SZ;
          const uint64_t da = desc_kmajor(sa), db = desc_nmajor(sa + A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 32; ++k) {
            // A: +32 bytes along K inside the swizzle atom; B: +32 K rows = 4096 bytes
            const uint32_t acc = (kb > kb0 || k > 0) ? 1u : 0u;
            if constexpr (PAIR) mma_f8_pair(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 256), IDESC_PAIR, acc);
            else                mma_f8(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 256), IDESC, acc);
          }
          // frees the stage (in both CTAs of a pair) when these MMAs retire
          if constexpr (PAIR) {
            mma_commit_pair(bar_empty + 8 * stage);
            mma_commit_pair(map_to_cta(bar_empty + 8 * stage, 1));
          } else {
            mma_commit(bar_empty + 8 * stage);
          }
          if (++stage == NSTAGE) stage = 0, phase ^= 1u;
        }
        if (ok) {                                      // accumulator complete
          if constexpr (PAIR) {
            mma_commit_pair(bar_tfull + 8 * buf);
            mma_commit_pair(map_to_cta(bar_tfull + 8 * buf, 1));
          } else {
            mma_commit(bar_tfull + 8 * buf);
          }
        }
      }
    }
  } else {
    // ===================== epilogue (warps 2..9) =====================
    const int quarter = warp & 3;                      // TMEM lane group this warp may read
    const int half = (warp - 2) >> 2;                  // which half of the tile's columns
    const int r_in_tile = quarter * 32 + lane;
    TileCursor cur{s_cum, p.offsets, p.E, p.n_tiles, 0, TILE_ROWS};
    uint32_t local = 0;
    bool ok = true;
    __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
    for (int tile = first_tile; ok && tile < total_tiles; tile += tile_step, ++local) {
      int e, row0, row_end, n_idx, split;
      if (!cur.locate(tile, e, row0, row_end, n_idx, split)) break;
      row0 += (int)rank * BM;                          // this CTA's half of a pair's tile
      const uint32_t buf = local & 1u, use = local >> 1;
      ok = mbar_wait(bar_tfull + 8 * buf, use & 1u, abort_flag, p.status);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      const int row = row0 + r_in_tile;
      const bool row_ok = row < row_end;
      if constexpr (RAW) {
        // split-K: raw fp32 accumulators into this split's slab; GATE_UP puts the up half at column H + n
        const int n0 = GATE_UP ? n_idx * BN_HALF : n_idx * BN;
        float* dst_row = p.partial + ((size_t)split * p.M + row) * p.ldp;
#pragma unroll 1
        for (int c = half * (BN / 64); c < (half + 1) * (BN / 64); ++c) {
          uint32_t a[32];
          tmem_ld32(t_row + c * 32, a);
          tmem_ld_wait();
          int col = n0 + c * 32;
          if (GATE_UP && c >= BN_HALF / 32) col = p.N_out + n0 + (c - BN_HALF / 32) * 32;
          const int lim = (GATE_UP && c >= BN_HALF / 32) ? 2 * p.N_out : p.N_out;
          if (row_ok) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              if (col + v * 4 < lim)
                reinterpret_cast<uint4*>(dst_row + col)[v] = make_uint4(a[4 * v], a[4 * v + 1], a[4 * v + 2], a[4 * v + 3]);
            }
          }
        }
      } else if constexpr (GATE_UP) {
        const float sa = p.scale_a[e];
        const float inv_g = 1.0f / (sa * p.scale_b0[e]);
        const float inv_u = 1.0f / (sa * p.scale_b1[e]);
        const int n0 = n_idx * BN_HALF;
        float amax = 0.f;
        const unsigned ok_rows = __ballot_sync(0xffffffffu, row_ok);
        unsigned long long row_ptr[8];
        group8_row_pointers(out + (size_t)row * p.N_out, lane, row_ptr);
        uint4 v[8];                                    // this warp's 64 columns of h as eight 16-byte pieces
#pragma unroll
        for (int cc = 0; cc < BN_HALF / 64; ++cc) {
          const int c = half * (BN_HALF / 64) + cc;
          uint32_t g[32], u[32];
          tmem_ld32(t_row + c * 32, g);
          tmem_ld32(t_row + BN_HALF + c * 32, u);
          tmem_ld_wait();
#pragma unroll
          for (int pc = 0; pc < 4; ++pc) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              float hv[2];
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                // the reference's bf16 rounding points: gate, up, silu(gate), product
                const float gate = bf16_round(__uint_as_float(g[pc * 8 + 2 * j + q]) * inv_g);
                const float up = bf16_round(__uint_as_float(u[pc * 8 + 2 * j + q]) * inv_u);
                const float act = bf16_round(silu_f(gate));
                hv[q] = bf16_round(act * up);
                amax = fmaxf(amax, fabsf(hv[q]));
              }
              __nv_bfloat162 b2 = __floats2bfloat162_rn(hv[0], hv[1]);
              w[j] = *reinterpret_cast<uint32_t*>(&b2);
            }
            v[cc * 4 + pc] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
        static_assert(BN_HALF / 64 == 2, "two 32-column chunks per epilogue warp make the eight pieces");
        group8_transpose(v, lane);
        {
          const int col = n0 + half * 64 + (lane & 7) * 8;
          if (col < p.N_out) group8_store(v, row_ptr, ok_rows, lane, col);
        }
        // rows past the segment and columns past H hold other data / zero fill: exclude them
        // (zero-filled columns give h = 0, which cannot raise the maximum)
        if (!row_ok) amax = 0.f;
        for (int off = 16; off; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        if (lane == 0 && amax > 0.f) atomic_max_nonneg(p.seg_amax + e, amax);
      } else {
        const float sa = p.scale_a[e];
        const float inv = 1.0f / (sa * p.scale_b0[e]);
        const int n0 = n_idx * BN;
        // where this lane's row goes: the local result buffer, the row's place on its home rank, or (combine
        // by reduction) the output row of the row's token
        __nv_bfloat16* out_row = out + (size_t)row * p.N_out;
        const bool weighted = p.row_w != nullptr;
        const bool reduce = p.tok_out != nullptr;
        const float w_row = (weighted && row_ok) ? bf16_round(p.row_w[row]) : 1.0f;
        if (reduce && row_ok)
          out_row = static_cast<__nv_bfloat16*>(p.tok_out) + (size_t)(p.row_slot[row] / p.top_k) * p.N_out;
        if (p.n_home > 0 && row_ok) {
          int j = row - p.offsets[e], s = 0;
          for (; s < p.n_home - 1; ++s) {
            const int c = p.home_counts[s * p.E + e];
            if (j < c) break;
            j -= c;
          }
          out_row = static_cast<__nv_bfloat16*>(p.home[s]) + (size_t)(p.home_first[s * p.E + e] + j) * p.N_out;
        }
        // Stores are issued transposed: the eight lanes of a group exchange their 16-byte pieces so that one
        // instruction writes 128 contiguous bytes of each of four rows (a lane per row would emit 16-byte
        // writes; over NVLink those reach only ~140 GB/s).  Lane l of a group ends up with piece (l & 7)
        // of the group's eight rows, and needs those rows' destinations.
        const unsigned ok_rows = __ballot_sync(0xffffffffu, row_ok);
        const int piece = lane & 7;
        unsigned long long row_ptr[8];
        group8_row_pointers(out_row, lane, row_ptr);
#pragma unroll 1
        for (int c2 = half * (BN / 128); c2 < (half + 1) * (BN / 128); ++c2) {
          uint32_t a[2][32];                           // two 32-column loads per wait
          tmem_ld32(t_row + c2 * 64, a[0]);
          tmem_ld32(t_row + c2 * 64 + 32, a[1]);
          tmem_ld_wait();
          uint4 v[8];                                  // this lane's row: 64 columns as eight 16-byte pieces
#pragma unroll
          for (int pc = 0; pc < 8; ++pc) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int i = (pc & 3) * 8 + 2 * j;
              __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(a[pc >> 2][i]) * inv,
                                                        __uint_as_float(a[pc >> 2][i + 1]) * inv);
              if (weighted) {                          // bf16(y) * bf16(w), rounded to bf16: the combine's product
                const float2 f = __bfloat1622float2(b2);
                b2 = __floats2bfloat162_rn(f.x * w_row, f.y * w_row);
              }
              w[j] = *reinterpret_cast<uint32_t*>(&b2);
            }
            v[pc] = make_uint4(w[0], w[1], w[2], w[3]);
          }
          group8_transpose(v, lane);
          const int col = n0 + c2 * 64 + piece * 8;
          if (col < p.N_out) {
            if (reduce) group8_reduce(v, row_ptr, ok_rows, lane, col);
            else        group8_store(v, row_ptr, ok_rows, lane, col);
          }
        }
      }
      // hand the accumulator buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (PAIR && rank != 0) mbar_arrive_cluster(map_to_cta(bar_tempty + 8 * buf, 0));
        else                   mbar_arrive(bar_tempty + 8 * buf);
      }
    }
  }

  // ---- teardown ----
  if (*abort_flag) {
    // give copies that are still in flight time to land before the shared memory is released
    for (int i = 0; i < 200; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();       // neither CTA leaves while the other may still signal it
  tc_fence_after();
  if (warp == 1) {
    if constexpr (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS);
    else                tmem_dealloc(tmem_base, TMEM_COLS);
  }
}


// ---- split-K post-passes (small batches only) ---------------------------------------
constexpr int kSplitMaxRows = 64;   // rows (T*K) up to which the K loop is split
constexpr int kSplitMax = 8;        // slabs at most
__device__ __forceinline__ int expert_of_row(const int32_t* __restrict__ offsets, int E, int row) {
  int lo = 0, hi = E;                       // largest e with offsets[e] <= row
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (offsets[mid] <= row) lo = mid; else hi = mid;
  }
  return lo;
}

// h = silu(gate) * up from the summed split-K slabs, with the same bf16 rounding points as the
// fused epilogue, plus the per-segment amax.  One thread per (row, 4 columns).
__global__ void __launch_bounds__(256)
swiglu_from_partials_kernel(const float* __restrict__ partial, int S, int M, int H, const int32_t* __restrict__ offsets,
                            int E, const float* __restrict__ sx, const float* __restrict__ sg,
                            const float* __restrict__ su, __nv_bfloat16* __restrict__ h, float* __restrict__ seg_amax) {
  chain_wait();
  const int vec_per_row = H / 4;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  bool live = gid < (size_t)M * vec_per_row;
  const int m = live ? (int)(gid / vec_per_row) : 0, v = live ? (int)(gid % vec_per_row) : 0;
  live = live && m < offsets[E];              // rows past the last segment belong to no expert
  const int e = expert_of_row(offsets, E, m);
  float amax = 0.f;
  if (live) {
    float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
    float4 a[kSplitMax], b[kSplitMax];       // every slab is requested before the first is used
#pragma unroll
    for (int s = 0; s < kSplitMax; ++s) {
      const float* row = partial + ((size_t)s * M + m) * (2 * H);
      a[s] = s < S ? reinterpret_cast<const float4*>(row)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
      b[s] = s < S ? reinterpret_cast<const float4*>(row + H)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int s = 0; s < kSplitMax; ++s) {    // fixed order: deterministic (absent slabs add +0)
      g[0] += a[s].x, g[1] += a[s].y, g[2] += a[s].z, g[3] += a[s].w;
      u[0] += b[s].x, u[1] += b[s].y, u[2] += b[s].z, u[3] += b[s].w;
    }
    const float inv_g = 1.0f / (sx[e] * sg[e]), inv_u = 1.0f / (sx[e] * su[e]);
    float hv[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float gate = bf16_round(g[q] * inv_g);
      const float up = bf16_round(u[q] * inv_u);
      hv[q] = bf16_round(bf16_round(silu_f(gate)) * up);
      amax = fmaxf(amax, fabsf(hv[q]));
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(hv[0], hv[1]), hi = __floats2bfloat162_rn(hv[2], hv[3]);
    reinterpret_cast<uint2*>(h + (size_t)m * H)[v] =
        make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
  }
  // one atomic per warp when the whole warp works on one expert (the common case), else per thread
  const int key = live ? e : -1;
  const int key0 = __shfl_sync(0xffffffffu, key, 0);
  if (__all_sync(0xffffffffu, key == key0)) {
    float mx = amax;
    for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if ((threadIdx.x & 31) == 0 && key0 >= 0 && mx > 0.f) atomic_max_nonneg(seg_amax + key0, mx);
  } else if (live && amax > 0.f) {
    atomic_max_nonneg(seg_amax + e, amax);
  }
}

// The same SwiGLU from the slabs, followed in the same kernel by the requantisation of h with its segment
// scale: no 16-bit h is written at all.  The scale needs the maximum over the whole segment, so the kernel
// has two phases separated by a grid-wide counter: every thread keeps its h values (at most kFusedItems x 4)
// in registers, publishes their maxima, the blocks meet (bounded wait; all blocks are resident, the grid is at
// most one block per SM), and then every thread quantises what it holds.  Same arithmetic as
// swiglu_from_partials_kernel + quant_rows_kernel.
constexpr int kFusedItems = 8;
__global__ void __launch_bounds__(256)
swiglu_requant_from_partials_kernel(const float* __restrict__ partial, int S, int M, int H,
                                    const int32_t* __restrict__ offsets, int E, const float* __restrict__ sx,
                                    const float* __restrict__ sg, const float* __restrict__ su,
                                    uint8_t* __restrict__ hq, float* __restrict__ seg_amax,
                                    float* __restrict__ scale_h, unsigned int* __restrict__ arrivals,
                                    int32_t* __restrict__ status) {
  chain_wait();
  __shared__ int s_ok;
  const int vec_per_row = H / 4;
  const int n_rows = min(M, offsets[E]);
  const long long total = (long long)n_rows * vec_per_row;
  float hv[kFusedItems][4];
  int ex[kFusedItems];
#pragma unroll
  for (int i = 0; i < kFusedItems; ++i) {
    const long long item = ((long long)i * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;   // spread over all blocks
    ex[i] = -1;
    hv[i][0] = hv[i][1] = hv[i][2] = hv[i][3] = 0.f;
    float amax = 0.f;
    if (item < total) {
    const int m = (int)(item / vec_per_row), v = (int)(item % vec_per_row);
    const int e = expert_of_row(offsets, E, m);
    ex[i] = e;
    float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
    float4 a[kSplitMax], b[kSplitMax];
#pragma unroll
    for (int s = 0; s < kSplitMax; ++s) {
      const float* row = partial + ((size_t)s * M + m) * (2 * H);
      a[s] = s < S ? reinterpret_cast<const float4*>(row)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
      b[s] = s < S ? reinterpret_cast<const float4*>(row + H)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int s = 0; s < kSplitMax; ++s) {    // fixed order: deterministic (absent slabs add +0)
      g[0] += a[s].x, g[1] += a[s].y, g[2] += a[s].z, g[3] += a[s].w;
      u[0] += b[s].x, u[1] += b[s].y, u[2] += b[s].z, u[3] += b[s].w;
    }
    const float inv_g = 1.0f / (sx[e] * sg[e]), inv_u = 1.0f / (sx[e] * su[e]);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float gate = bf16_round(g[q] * inv_g);
      const float up = bf16_round(u[q] * inv_u);
      hv[i][q] = bf16_round(bf16_round(silu_f(gate)) * up);
      amax = fmaxf(amax, fabsf(hv[i][q]));
    }
    }
    // one atomic per warp when the whole warp works on one expert (the common case), else per thread: tens of
    // thousands of atomics on one address would serialise for longer than the rest of the kernel takes
    const int key = ex[i];
    const int key0 = __shfl_sync(0xffffffffu, key, 0);
    if (__all_sync(0xffffffffu, key == key0)) {
      float mx = amax;
      for (int off = 16; off; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
      if ((threadIdx.x & 31) == 0 && key0 >= 0 && mx > 0.f) atomic_max_nonneg(seg_amax + key0, mx);
    } else if (key >= 0 && amax > 0.f) {
      atomic_max_nonneg(seg_amax + key, amax);
    }
  }
  // ---- all blocks meet: every maximum is published before any scale is read ----
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicAdd(arrivals, 1u);
    bool ok = true;
    const unsigned long long t0 = global_ns();
    // polled with plain acquire loads and a pause: pollers that hammer the counter with atomics delay the
    // arrivals they are waiting for
    auto arrived = [&]() {
      unsigned v;
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(arrivals) : "memory");
      return v;
    };
    for (uint32_t spin = 1; arrived() < gridDim.x; ++spin) {
      __nanosleep(64);
      if ((spin & 63u) == 0u && global_ns() - t0 > WAIT_LIMIT_NS) {
        atomicOr(status, BWMOE_STATUS_WAIT_TIMEOUT);
        ok = false;
        break;
      }
    }
    __threadfence();
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  if (!s_ok) return;
#pragma unroll
  for (int i = 0; i < kFusedItems; ++i) {
    if (ex[i] < 0) continue;
    const long long item = ((long long)i * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
    const int m = (int)(item / vec_per_row), v = (int)(item % vec_per_row);
    const float scale = scale_from_amax(__ldcg(seg_amax + ex[i]));
    if (v == 0) scale_h[ex[i]] = scale;            // every row of the segment writes the same value
    reinterpret_cast<uint32_t*>(hq + (size_t)m * H)[v] =
        (uint32_t)to_e4m3x2(hv[i][0] * scale, hv[i][1] * scale) |
        ((uint32_t)to_e4m3x2(hv[i][2] * scale, hv[i][3] * scale) << 16);
  }
}

// y = bf16(sum of slabs * 1/(s_h * s_d)); one thread per (row, 4 columns)
__global__ void __launch_bounds__(256)
down_from_partials_kernel(const float* __restrict__ partial, int S, int M, int D, const int32_t* __restrict__ offsets,
                          int E, const float* __restrict__ sh, const float* __restrict__ sd,
                          __nv_bfloat16* __restrict__ y) {
  chain_wait();
  const int vec_per_row = D / 4;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (size_t)M * vec_per_row) return;
  const int m = (int)(gid / vec_per_row), v = (int)(gid % vec_per_row);
  if (m >= offsets[E]) return;                // rows past the last segment belong to no expert
  const int e = expert_of_row(offsets, E, m);
  float a[4] = {0.f, 0.f, 0.f, 0.f};
  float4 t[kSplitMax];
#pragma unroll
  for (int s = 0; s < kSplitMax; ++s)
    t[s] = s < S ? reinterpret_cast<const float4*>(partial + ((size_t)s * M + m) * D)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int s = 0; s < kSplitMax; ++s) a[0] += t[s].x, a[1] += t[s].y, a[2] += t[s].z, a[3] += t[s].w;
  const float inv = 1.0f / (sh[e] * sd[e]);
  __nv_bfloat162 lo = __floats2bfloat162_rn(a[0] * inv, a[1] * inv), hi = __floats2bfloat162_rn(a[2] * inv, a[3] * inv);
  reinterpret_cast<uint2*>(y + (size_t)m * D)[v] =
      make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
}

// The same sum, followed at once by the weighted combine of the token's K rows: one thread per
// (token, 4 columns).  Arithmetic and order equal down_from_partials_kernel + the combine kernel
// (bf16 y, bf16 weight, bf16 product, fp32 sum over k in order, optional scale and residual);
// y is still written so that the staged view of the workspace stays complete.
__global__ void __launch_bounds__(256)
down_combine_from_partials_kernel(const float* __restrict__ partial, int S, int M, int D,
                                  const int32_t* __restrict__ offsets, int E, const float* __restrict__ sh,
                                  const float* __restrict__ sd, __nv_bfloat16* __restrict__ y,
                                  const int32_t* __restrict__ pos, const float* __restrict__ weights, int T, int K,
                                  __nv_bfloat16* __restrict__ out, float scale,
                                  const __nv_bfloat16* __restrict__ residual, int n_tail) {
  chain_wait();
  const int vec_per_row = D / 4;
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= (size_t)T * vec_per_row) return;
  const int t = (int)(gid / vec_per_row), v = (int)(gid % vec_per_row);
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, tail[4] = {0.f, 0.f, 0.f, 0.f};
  for (int k = 0; k < K; ++k) {
    const int m = pos[(size_t)t * K + k];
    if (m < 0) continue;
    const int e = expert_of_row(offsets, E, m);
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    float4 q[kSplitMax];
#pragma unroll
    for (int s = 0; s < kSplitMax; ++s)
      q[s] = s < S ? reinterpret_cast<const float4*>(partial + ((size_t)s * M + m) * D)[v] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s = 0; s < kSplitMax; ++s) a[0] += q[s].x, a[1] += q[s].y, a[2] += q[s].z, a[3] += q[s].w;
    const float inv = 1.0f / (sh[e] * sd[e]);
    const __nv_bfloat162 lo = __floats2bfloat162_rn(a[0] * inv, a[1] * inv), hi = __floats2bfloat162_rn(a[2] * inv, a[3] * inv);
    reinterpret_cast<uint2*>(y + (size_t)m * D)[v] =
        make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
    const float w = bf16_round(weights[(size_t)t * K + k]);
    const float2 f0 = __bfloat1622float2(lo), f1 = __bfloat1622float2(hi);
    float* dst = k < K - n_tail ? acc : tail;          // always-on slots are summed apart (see combine_kernel)
    dst[0] += bf16_round(f0.x * w);
    dst[1] += bf16_round(f0.y * w);
    dst[2] += bf16_round(f1.x * w);
    dst[3] += bf16_round(f1.y * w);
  }
  if (scale != 1.0f) {     // bf16 tensor times a Python scalar: fp32 product with the unrounded scalar
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = bf16_round(bf16_round(acc[i]) * scale);
  }
  if (residual != nullptr) {
    const uint2 raw = reinterpret_cast<const uint2*>(residual + (size_t)t * D)[v];
    const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float2 f = __bfloat1622float2(q[i]);
      acc[2 * i] = bf16_round(acc[2 * i]) + f.x;
      acc[2 * i + 1] = bf16_round(acc[2 * i + 1]) + f.y;
    }
  }
  if (n_tail > 0) {
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[i] = bf16_round(acc[i]) + bf16_round(tail[i]);
  }
  const __nv_bfloat162 o0 = __floats2bfloat162_rn(acc[0], acc[1]), o1 = __floats2bfloat162_rn(acc[2], acc[3]);
  reinterpret_cast<uint2*>(out + (size_t)t * D)[v] =
      make_uint2(*reinterpret_cast<const uint32_t*>(&o0), *reinterpret_cast<const uint32_t*>(&o1));
}

// Split-K is for small batches, where a few experts x column blocks cannot occupy every SM:
// the K loop of each tile is cut so that about four waves of tiles exist.
struct SplitPlan {
  int split_k, k_per_split;
};
SplitPlan choose_split(int M, int E, int k_blocks, int n_tiles) {
  SplitPlan sp{1, k_blocks};
  if (M > kSplitMaxRows) return sp;
  const long long tiles = (long long)std::min(M, E) * n_tiles;      // one row tile per active expert, at most
  int S = (int)std::min<long long>(kSplitMax, (4ll * sm_count() + tiles - 1) / tiles);
  S = std::max(1, std::min(S, k_blocks / 2));
  sp.k_per_split = ceil_div(k_blocks, S);
  sp.split_k = ceil_div(k_blocks, sp.k_per_split);
  return sp;
}

// Pairs pay when an expert's segment fills several 256-row tiles: below that the rows a pair computes past the
// end of a segment outweigh what the halved weight traffic into shared memory saves.
constexpr int kPairMinRowsPerExpert = 1024;
bool pair_tiles_pay(bool gate_up, int M, int E) {
  return !gate_up && M / E >= kPairMinRowsPerExpert && gemm_sm_budget() >= 2;
}

template <bool GATE_UP, bool RAW>
int launch_gemm(const CUtensorMap& ma, const CUtensorMap& mb0, const CUtensorMap& mb1, const GemmParams& p,
                int M, cudaStream_t st) {
  if constexpr (!RAW && !GATE_UP) {
    if (pair_tiles_pay(GATE_UP, M, p.E)) {
      static unsigned char smem_set[64] = {0};
      BWMOE_CUDA_OK(ensure_dynamic_smem(grouped_gemm_kernel<GATE_UP, false, true>, PAIR_SMEM_BYTES, smem_set));
      const long long max_tiles = (long long)(ceil_div(M, 2 * BM) + p.E) * p.n_tiles;
      const int pairs = (int)std::min<long long>(gemm_sm_budget() / 2, max_tiles);
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * pairs);
      cfg.blockDim = dim3(GEMM_THREADS);
      cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
      cfg.stream = st;
      cudaLaunchAttribute attr[2];
      attr[0].id = cudaLaunchAttributeClusterDimension;
      attr[0].val.clusterDim.x = 2;
      attr[0].val.clusterDim.y = 1;
      attr[0].val.clusterDim.z = 1;
      attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;     // the kernel starts with chain_wait()
      attr[1].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 2;
      // pairs that can be resident at once (per device, asked once): the persistent loop needs no more
      static int resident_pairs[64] = {0};
      int dev = 0;
      BWMOE_CUDA_OK(cudaGetDevice(&dev));
      if (dev >= 0 && dev < 64) {
        if (resident_pairs[dev] == 0) {
          int n = 0;
          cfg.gridDim = dim3(2 * (sm_count() / 2));
          BWMOE_CUDA_OK(cudaOccupancyMaxActiveClusters(&n, grouped_gemm_kernel<GATE_UP, false, true>, &cfg));
          BWMOE_REQUIRE(n >= 1, BWMOE_ERR_CUDA, "no CTA pair of the grouped GEMM fits on this device");
          resident_pairs[dev] = n;
        }
        cfg.gridDim = dim3(2 * std::min(pairs, resident_pairs[dev]));
      }
      note_launch();
      BWMOE_CUDA_OK(cudaLaunchKernelEx(&cfg, grouped_gemm_kernel<GATE_UP, false, true>, ma, mb0, mb1, p));
      return BWMOE_OK;
    }
  }
  static unsigned char smem_set[64] = {0};
  BWMOE_CUDA_OK(ensure_dynamic_smem(grouped_gemm_kernel<GATE_UP, RAW, false>, SMEM_BYTES, smem_set));
  const long long max_tiles = (long long)(ceil_div(M, BM) + p.E) * p.n_tiles * p.split_k;
  const int grid = (int)std::min<long long>(gemm_sm_budget(), max_tiles);
  BWMOE_CUDA_OK(launch_chained(grouped_gemm_kernel<GATE_UP, RAW, false>, dim3(grid), dim3(GEMM_THREADS), SMEM_BYTES, st, ma, mb0, mb1, p));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int check_common(const char* who, const void* a, const void* b, int M, int D, int H, int E) {
  BWMOE_REQUIRE(M > 0 && D > 0 && H > 0 && E > 0, BWMOE_ERR_BAD_SHAPE, "%s: M=%d D=%d H=%d E=%d", who, M, D, H, E);
  BWMOE_REQUIRE(D % 16 == 0 && H % 16 == 0, BWMOE_ERR_BAD_SHAPE, "%s: D=%d and H=%d must be multiples of 16", who, D, H);
  BWMOE_REQUIRE(E <= 256, BWMOE_ERR_UNSUPPORTED, "%s: E=%d > 256", who, E);
  BWMOE_REQUIRE(aligned16(a) && aligned16(b), BWMOE_ERR_BAD_ALIGN, "%s: pointers must be 16-byte aligned", who);
  return BWMOE_OK;
}

}  // namespace

size_t gemm_scratch_bytes(int M, int D, int H, int /*E*/) {
  if (M > kSplitMaxRows) return 256;
  return (size_t)kSplitMax * M * std::max(2 * H, D) * sizeof(float) + 256;
}

int launch_gateup(const void* xq, const int32_t* offsets, const float* sx, const void* wg, const void* wu,
                  const float* sg, const float* su, int M, int D, int H, int E, void* h, float* amax_h,
                  int32_t* status, void* scratch, cudaStream_t st, const FusedRequant* fr, bool* requant_done) {
  if (requant_done) *requant_done = false;
  BWMOE_REQUIRE(xq && offsets && sx && wg && wu && sg && su && h && amax_h && status, BWMOE_ERR_NULL,
                "gateup: null pointer");
  if (int rc = check_common("gateup", xq, h, M, D, H, E)) return rc;
  BWMOE_REQUIRE(aligned16(wg) && aligned16(wu), BWMOE_ERR_BAD_ALIGN, "gateup: weights must be 16-byte aligned");
  CUtensorMap ma, mg, mu;
  if (int rc = make_map_a(&ma, xq, M, D)) return rc;
  if (int rc = make_map_b(&mg, wg, E, D, H)) return rc;
  if (int rc = make_map_b(&mu, wu, E, D, H)) return rc;
  const int k_blocks = ceil_div(D, BK), n_tiles = ceil_div(H, BN_HALF);
  const SplitPlan sp = choose_split(M, E, k_blocks, n_tiles);
  GemmParams p{offsets, sx, sg, su, h, amax_h, status, E, D, H, n_tiles, sp.split_k, sp.k_per_split, M, 2 * H, nullptr};
  if (sp.split_k == 1) return launch_gemm<true, false>(ma, mg, mu, p, M, st);
  BWMOE_REQUIRE(scratch != nullptr && aligned16(scratch), BWMOE_ERR_WORKSPACE, "gateup: scratch buffer required");
  p.partial = static_cast<float*>(scratch);
  if (int rc = launch_gemm<true, true>(ma, mg, mu, p, M, st)) return rc;
  const size_t n = (size_t)M * (H / 4);
  // small batches inside the whole forward: SwiGLU and the requantisation of h in one kernel (no 16-bit h)
  // as many blocks as there are SMs (all resident at once: they meet inside the kernel), at most kFusedItems items
  // per thread
  const size_t fused_blocks = std::min<size_t>((size_t)sm_count(), (n + 255) / 256);
  if (fr != nullptr && requant_done != nullptr && n <= fused_blocks * 256 * kFusedItems) {
    BWMOE_CUDA_OK(launch_chained(swiglu_requant_from_partials_kernel, dim3((unsigned)fused_blocks), dim3(256), 0, st,
        p.partial, sp.split_k, M, H, offsets, E, sx, sg, su, static_cast<uint8_t*>(fr->hq), amax_h, fr->scale_h,
        fr->arrivals, status));
    BWMOE_CUDA_OK(cudaGetLastError());
    *requant_done = true;
    return BWMOE_OK;
  }
  BWMOE_CUDA_OK(launch_chained(swiglu_from_partials_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st,
      p.partial, sp.split_k, M, H, offsets, E, sx, sg, su, static_cast<__nv_bfloat16*>(h), amax_h));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

int launch_down(const void* hq, const int32_t* offsets, const float* sh, const void* wd, const float* sd,
                int M, int D, int H, int E, void* y, int32_t* status, void* scratch, cudaStream_t st,
                const CombineArgs* combine, int* combine_state, const HomeRoute* route) {
  if (combine_state) *combine_state = kCombinePlain;
  BWMOE_REQUIRE(hq && offsets && sh && wd && sd && y && status, BWMOE_ERR_NULL, "down: null pointer");
  if (int rc = check_common("down", hq, y, M, D, H, E)) return rc;
  BWMOE_REQUIRE(aligned16(wd), BWMOE_ERR_BAD_ALIGN, "down: weights must be 16-byte aligned");
  CUtensorMap ma, mb;
  if (int rc = make_map_a(&ma, hq, M, H)) return rc;
  if (int rc = make_map_b(&mb, wd, E, H, D)) return rc;
  const int k_blocks = ceil_div(H, BK), n_tiles = ceil_div(D, BN);
  SplitPlan sp = choose_split(M, E, k_blocks, n_tiles);
  if (route != nullptr) sp = SplitPlan{1, k_blocks};      // rows leave from the epilogue: no slab pass
  GemmParams p{offsets, sh, sd, nullptr, y, nullptr, status, E, H, D, n_tiles, sp.split_k, sp.k_per_split, M, D, nullptr};
  if (route != nullptr) {
    BWMOE_REQUIRE(route->n_ranks >= 1 && route->n_ranks <= 8 && route->counts && route->first && route->home,
                  BWMOE_ERR_UNSUPPORTED, "down: home route with %d ranks", route->n_ranks);
    p.n_home = route->n_ranks;
    p.home_counts = route->counts;
    p.home_first = route->first;
    for (int r = 0; r < route->n_ranks; ++r) {
      BWMOE_REQUIRE(route->home[r] != nullptr && aligned16(route->home[r]), BWMOE_ERR_BAD_ALIGN,
                    "down: result buffer of rank %d", r);
      p.home[r] = route->home[r];
    }
  }
  if (sp.split_k == 1) {
    // the combine starts in the epilogue when the caller handed over the rows' routing weights
    if (combine != nullptr && combine_state != nullptr && route == nullptr && combine->row_w != nullptr) {
      p.row_w = combine->row_w;
      *combine_state = kCombinePreweighted;
      if (combine->reduce && combine->row_slot != nullptr && combine->scale == 1.0f && combine->residual == nullptr &&
          combine->n_tail == 0) {
        p.row_slot = combine->row_slot;
        p.tok_out = combine->out;
        p.top_k = combine->K;
        *combine_state = kCombineDone;
      }
    }
    return launch_gemm<false, false>(ma, mb, mb, p, M, st);
  }
  BWMOE_REQUIRE(scratch != nullptr && aligned16(scratch), BWMOE_ERR_WORKSPACE, "down: scratch buffer required");
  p.partial = static_cast<float*>(scratch);
  if (int rc = launch_gemm<false, true>(ma, mb, mb, p, M, st)) return rc;
  if (combine != nullptr && combine_state != nullptr && combine->T * combine->K == M) {
    const size_t nt = (size_t)combine->T * (D / 4);
    BWMOE_CUDA_OK(launch_chained(down_combine_from_partials_kernel, dim3((unsigned)((nt + 255) / 256)), dim3(256), 0, st,
        p.partial, sp.split_k, M, D, offsets, E, sh, sd, static_cast<__nv_bfloat16*>(y), combine->pos,
        combine->weights, combine->T, combine->K, static_cast<__nv_bfloat16*>(combine->out), combine->scale,
        static_cast<const __nv_bfloat16*>(combine->residual), combine->n_tail));
    BWMOE_CUDA_OK(cudaGetLastError());
    *combine_state = kCombineDone;
    return BWMOE_OK;
  }
  const size_t n = (size_t)M * (D / 4);
  BWMOE_CUDA_OK(launch_chained(down_from_partials_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, p.partial, sp.split_k, M, D, offsets, E, sh,
                                                                        sd, static_cast<__nv_bfloat16*>(y)));
  BWMOE_CUDA_OK(cudaGetLastError());
  return BWMOE_OK;
}

}  // namespace bwmoe
