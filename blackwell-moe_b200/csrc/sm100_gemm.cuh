// Building blocks shared by the tcgen05 GEMM kernels: tile constants, PTX wrappers
// (mbarrier, TMA, tensor-memory allocation, tcgen05.mma / ld / commit), shared-memory matrix
// descriptors, and the host-side tensor-map encoders.  sm_100a only.
#pragma once

#include <cuda.h>
#include <cudaTypedefs.h>

#include <algorithm>
#include <mutex>

#include "common.cuh"

namespace bwmoe {
namespace sm100 {


constexpr int BM = 128;            // rows per tile
constexpr int BK = 128;            // K elements (= bytes) per pipeline stage
constexpr int BN_HALF = 128;       // accumulator columns per weight box
constexpr int BN = 2 * BN_HALF;    // accumulator columns per tile
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;               // 16 KiB
constexpr int B_HALF_BYTES = BK * BN_HALF;     // 16 KiB
constexpr int STAGE_BYTES = A_BYTES + 2 * B_HALF_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s

// tcgen05 instruction descriptor: D=f32, A=B=e4m3, A K-major, B MN-major, N=256, M=128
constexpr uint32_t IDESC = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (1u << 16) |
                           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// the same with N = 128 (one weight box)
constexpr uint32_t IDESC_HALF = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (1u << 16) |
                                ((uint32_t)(BN_HALF >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait.  Returns false (after flagging) when the limit is hit or another warp gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* status) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 63u) == 0u) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicOr(status, BWMOE_STATUS_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}
// Same contract as mbar_wait, but polls with the non-suspending test_wait: for waits that sit on
// the critical path of every K block, where the wake-up latency of a suspended try_wait shows.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                               int32_t* status) {
  if (mbar_test_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (uint32_t it = 1;; ++it) {
    if (mbar_test_wait(bar, parity)) return true;
    __nanosleep(20);                      // keep the poll loop from crowding the warps that still have work
    if ((it & 1023u) == 0u) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > WAIT_LIMIT_NS) {
        *abort_flag = 1;
        atomicOr(status, BWMOE_STATUS_WAIT_TIMEOUT);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y,
                                            int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void mma_f8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// ---- CTA pairs (cta_group::2): two CTAs of a cluster run one 256-row tile.  Each loads its own 128 rows of A
// and its own half of the tile's B columns; the even CTA issues the MMAs for both, every CTA keeps the
// accumulators of its own rows in its own tensor memory.  None of the loads is a multicast.
constexpr int PAIR_STAGES = 6;
constexpr int PAIR_STAGE_BYTES = A_BYTES + B_HALF_BYTES;     // 32 KiB per CTA and stage
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;
// instruction descriptor of the pair: M = 256 (128 rows per CTA), N = 256
constexpr uint32_t IDESC_PAIR = (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (1u << 16) |
                                ((uint32_t)(BN >> 3) << 17) | ((uint32_t)((2 * BM) >> 4) << 24);
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// every thread of both CTAs
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the shared::cluster address of this CTA's shared-memory address `addr` in the CTA of rank `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar) : "memory");
}
// loads into THIS CTA's shared memory that report their bytes to a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x,
                                                 int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t cluster_bar, int x,
                                                 int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// one warp of EACH CTA of the pair executes these; both receive the same address
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void mma_f8_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// arrives on ONE barrier (of this CTA or, through its shared::cluster address, of the peer) when the pair's
// MMAs issued so far have retired; the issuer calls it once per CTA that has to hear of it
__device__ __forceinline__ void mma_commit_pair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptors (16-byte units; version 1; 128-byte swizzle = layout type 2).
// K-major operand: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// MN-major operand: 128 N-elements contiguous per K row; the next 128 N-elements lie
// B_HALF_BYTES further (leading offset); 8-K-row groups are 1024 bytes apart (stride offset).
__device__ __forceinline__ uint64_t desc_nmajor(uint32_t saddr) {
  return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)(B_HALF_BYTES >> 4) << 16) |
         ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ float silu_f(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

// Eight 16-byte pieces per lane, transposed across the eight lanes of a group (butterfly over lane bits
// 4, 2, 1): afterwards v[k] of lane l is what lane (l & ~7) + k held in v[l & 7].  Epilogues use it so
// that one store instruction writes 128 contiguous bytes of a row (eight lanes x 16 bytes) instead of 16
// bytes of 32 different rows.
__device__ __forceinline__ void group8_transpose(uint4 (&v)[8], int lane) {
#pragma unroll
  for (int sft = 4; sft >= 1; sft >>= 1) {
    const bool upper = (lane & sft) != 0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k & sft) continue;
      const uint4 send = upper ? v[k] : v[k | sft];
      uint4 recv;
      recv.x = __shfl_xor_sync(0xffffffffu, send.x, sft);
      recv.y = __shfl_xor_sync(0xffffffffu, send.y, sft);
      recv.z = __shfl_xor_sync(0xffffffffu, send.z, sft);
      recv.w = __shfl_xor_sync(0xffffffffu, send.w, sft);
      if (upper) v[k] = recv; else v[k | sft] = recv;
    }
  }
}
// v[k] -> 16 bytes at element column `col` of the row whose pointer lane (l & ~7) + k holds; rows whose
// bit in ok_rows is clear are skipped.
__device__ __forceinline__ void group8_store(const uint4 (&v)[8], const unsigned long long (&row_ptr)[8],
                                             unsigned ok_rows, int lane, int col) {
  const int g0 = lane & ~7;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if ((ok_rows >> (g0 + k)) & 1u)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(static_cast<uintptr_t>(row_ptr[k])) + col) = v[k];
  }
}
// The same addressing, but v[k] (eight bf16) is ADDED to the destination with one 16-byte vector reduction
// (red.global.add.noftz.v4.bf16x2: rounds to bf16 after every addition, order of arrival).
__device__ __forceinline__ void group8_reduce(const uint4 (&v)[8], const unsigned long long (&row_ptr)[8],
                                              unsigned ok_rows, int lane, int col) {
  const int g0 = lane & ~7;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if ((ok_rows >> (g0 + k)) & 1u) {
      const unsigned long long addr = row_ptr[k] + (unsigned long long)col * 2ull;
      asm volatile("red.global.add.noftz.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(addr), "r"(v[k].x), "r"(v[k].y),
                   "r"(v[k].z), "r"(v[k].w)
                   : "memory");
    }
  }
}
__device__ __forceinline__ void group8_row_pointers(const void* my_row, int lane, unsigned long long (&row_ptr)[8]) {
  const int g0 = lane & ~7;
#pragma unroll
  for (int k = 0; k < 8; ++k)
    row_ptr[k] = __shfl_sync(0xffffffffu, (unsigned long long)reinterpret_cast<uintptr_t>(my_row), g0 + k);
}

// ---------------------------------------------------------------- host side
inline PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  });
  return fn;
}

// Encoded tensor maps are a pure function of (base pointer, shape): a small cache keyed by them takes the
// driver calls off the host path of repeated forwards (five encodes per forward otherwise).  The entries
// hold no data pointers of their own and never go stale by a change of the CONTENTS behind a pointer (an
// expert cache swapping a slot's weights); bwmoe_invalidate() empties the cache for callers that want that
// after freeing memory.  Implemented in api.cu.
bool tensor_map_lookup(int kind, const void* base, int d0, int d1, int d2, CUtensorMap* out);
void tensor_map_store(int kind, const void* base, int d0, int d1, int d2, const CUtensorMap& map);

// activations [rows, kdim] e4m3 row-major: box 128 (K) x 128 (rows), 128-byte swizzle
inline int make_map_a(CUtensorMap* map, const void* base, int rows, int kdim) {
  if (tensor_map_lookup(0, base, rows, kdim, 0, map)) return BWMOE_OK;
  auto fn = encode_fn();
  BWMOE_REQUIRE(fn != nullptr, BWMOE_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t dims[2] = {(cuuint64_t)kdim, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)kdim};
  cuuint32_t box[2] = {BK, BM};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BWMOE_REQUIRE(r == CUDA_SUCCESS, BWMOE_ERR_CUDA, "cuTensorMapEncodeTiled(A: rows=%d k=%d) failed: %d", rows,
                kdim, (int)r);
  tensor_map_store(0, base, rows, kdim, 0, *map);
  return BWMOE_OK;
}
// weights [E, kdim, n] e4m3, n contiguous: box 128 (N) x 128 (K) x 1, 128-byte swizzle
inline int make_map_b(CUtensorMap* map, const void* base, int E, int kdim, int n) {
  if (tensor_map_lookup(1, base, E, kdim, n, map)) return BWMOE_OK;
  auto fn = encode_fn();
  BWMOE_REQUIRE(fn != nullptr, BWMOE_ERR_CUDA, "cuTensorMapEncodeTiled not available from the driver");
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)kdim, (cuuint64_t)E};
  cuuint64_t strides[2] = {(cuuint64_t)n, (cuuint64_t)n * (cuuint64_t)kdim};
  cuuint32_t box[3] = {BN_HALF, BK, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  BWMOE_REQUIRE(r == CUDA_SUCCESS, BWMOE_ERR_CUDA, "cuTensorMapEncodeTiled(B: E=%d k=%d n=%d) failed: %d", E,
                kdim, n, (int)r);
  tensor_map_store(1, base, E, kdim, n, *map);
  return BWMOE_OK;
}

}  // namespace sm100
}  // namespace bwmoe
