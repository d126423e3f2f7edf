// Shared helpers for the libbwmoe kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/bwmoe.h"

namespace bwmoe {

// ---- host-side error plumbing --------------------------------------------
int set_error(int code, const char* fmt, ...);
#define BWMOE_CUDA_OK(expr)                                                              \
  do {                                                                                   \
    cudaError_t e__ = (expr);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return ::bwmoe::set_error(BWMOE_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)
#define BWMOE_REQUIRE(cond, code, ...) \
  do {                                 \
    if (!(cond)) return ::bwmoe::set_error(code, __VA_ARGS__); \
  } while (0)

// Kernels this library has launched in the process so far (bwmoe_launch_count).  Every launch passes its
// stream through counted(), so the figure is a count of launches, not an estimate.
void note_launch();
inline cudaStream_t counted(cudaStream_t st) {
  note_launch();
  return st;
}

// Programmatic dependent launch: a kernel launched through launch_chained() may be scheduled while the kernel
// before it in the stream is still draining (its launch latency and block start-up overlap that tail).
// Such a kernel executes chain_wait() before it touches global memory: the instruction returns when every
// kernel it depends on has completed and its writes are visible.  A kernel that calls chain_wait() may
// also be launched the ordinary way (the instruction then returns at once), but a kernel launched through
// launch_chained() MUST call it.
__device__ __forceinline__ void chain_wait() {
#if defined(__CUDA_ARCH__)
  asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  note_launch();
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
int sm_count();
int gemm_sm_budget();   // sm_count() minus the SMs reserved through bwmoe_set_sm_reserve

// The dynamic shared-memory limit of a kernel is a per-device attribute: raise it once on every
// device the kernel is launched on.  `done` is one flag array per kernel (a function-local static
// of the caller); setting the attribute twice from two racing threads is harmless.
template <class Kernel>
inline cudaError_t ensure_dynamic_smem(Kernel kernel, int bytes, unsigned char (&done)[64]) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (done[dev]) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) done[dev] = 1;
  return e;
}

// ---- arithmetic shared by several kernels ---------------------------------
constexpr float kFp8Max = 448.0f;
// The reference clamps amax in the tensor's own dtype (bf16), so the floor is
// bf16(1e-4) = 0x38D2, not the fp32 literal.
constexpr float kAmaxFloor = 0.00010013580322265625f;

// The reference writes `448.0 / amax` with a Python scalar on the left, which torch
// evaluates as reciprocal(amax) * 448 (two roundings); reproduce exactly that.
__device__ __forceinline__ float scale_from_amax(float amax) {
  return __fmul_rn(__frcp_rn(fmaxf(amax, kAmaxFloor)), kFp8Max);
}

// e4m3(clamp(v, +-448)), round-to-nearest-even, as torch's cast after the clamp.
__device__ __forceinline__ uint8_t to_e4m3(float v) {
  v = fminf(fmaxf(v, -kFp8Max), kFp8Max);
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint16_t to_e4m3x2(float lo, float hi) {
  lo = fminf(fmaxf(lo, -kFp8Max), kFp8Max);
  hi = fminf(fmaxf(hi, -kFp8Max), kFp8Max);
  return static_cast<uint16_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}

__device__ __forceinline__ float bf16_round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// non-negative floats order like their bit patterns: atomicMax on the uint view.
__device__ __forceinline__ void atomic_max_nonneg(float* addr, float v) {
  atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}

// ---- launchers implemented in the individual .cu files ---------------------
// scratch (optional): enables the tensor-core router where it applies; needs router_scratch_bytes()
// T_as > 0: choose the routing kernel a batch of T_as tokens would get (the kernels agree on the selected
// experts always, but their fp32 weights differ in the last bits: a rank that routes a slice of a larger batch
// passes the size of the whole batch to obtain the weights the whole batch would have got).
size_t router_scratch_bytes(int T, int D, int E, int K, int T_as = 0);
int launch_router(const void* x, const void* wg, int T, int D, int E, int K, float* weights,
                  int32_t* indices, float* row_amax, cudaStream_t st, void* scratch = nullptr,
                  size_t scratch_bytes = 0, int32_t* status = nullptr, int T_as = 0);
bool router_tc_applicable(int T, int D, int E, int K);
size_t router_tc_scratch_bytes(int T, int D, int E);
int launch_router_tc(const void* x, const void* wg, int T, int D, int E, int K, float* weights, int32_t* indices,
                     float* row_amax, int32_t* status, void* scratch, cudaStream_t st);
int launch_router_fallback(const void* x, const void* wg, int T, int D, int E, int K, float* weights,
                           int32_t* indices, const int32_t* list, const int32_t* count, cudaStream_t st);
size_t plan_scratch_bytes(int T, int E, int K);
int launch_plan(const int32_t* indices, const float* row_amax, int T, int E, int K, int32_t* offsets,
                int32_t* pos, int32_t* row_slot, int32_t* row_expert, float* seg_amax, int32_t* status,
                void* scratch, cudaStream_t st, float* scales_out = nullptr);
int launch_plan_static(const int32_t* indices, const float* row_amax, int T, int E, int K, int32_t* offsets,
                       int32_t* pos, int32_t* row_slot, int32_t* row_expert, float* seg_amax, int32_t* status,
                       cudaStream_t st);
int launch_segment_scales(const float* seg_amax, const int32_t* offsets, int E, float* scales,
                          cudaStream_t st);
int launch_scatter_quant(const void* x, const int32_t* pos, const int32_t* indices, const float* scales, int T,
                         int D, int K, void* xq, cudaStream_t st, const float* weights = nullptr,
                         float* row_w = nullptr);
int launch_ep_maps(const int32_t* counts, const int32_t* offsets, int n_ranks, int E, int rank, int32_t* delta,
                   int32_t* offsets_local, int32_t* home_counts, int32_t* home_first, cudaStream_t st);
int launch_scatter_quant_peers(const void* x, const int32_t* pos, const int32_t* indices, const float* scales,
                               const int32_t* delta, int T, int D, int K, int experts_per_rank, void* const* dst,
                               int n_ranks, int rows_cap, int32_t* status, cudaStream_t st);
int launch_combine_peers(void* const* src, int n_ranks, const int32_t* pos, const int32_t* indices,
                         const float* weights, const int32_t* delta, int experts_per_rank, int T, int D, int K,
                         void* out, cudaStream_t st);
int launch_gather_quant(const void* x, const int32_t* row_slot, const int32_t* row_expert,
                        const float* scales, int M, int D, int K, void* xq, cudaStream_t st);
int launch_requant(const void* h, const int32_t* row_expert, const float* scales_h, int M, int H,
                   void* hq, cudaStream_t st, float* scales_from_amax_out = nullptr);
int launch_requant_segments(const void* h, const int32_t* offsets, const float* scales_h, int E, int H, void* hq,
                            cudaStream_t st);
int launch_combine(const void* y, const int32_t* pos, const float* weights, int T, int D, int K,
                   void* out, cudaStream_t st, float scale = 1.0f, const void* residual = nullptr,
                   bool preweighted = false, int n_tail = 0);
int launch_append_shared_slots(const int32_t* idx_r, const float* w_r, int T, int K, int E, int S, int32_t* idx,
                               float* w, cudaStream_t st);
int launch_merge_amax(float* amax, int first, int count, cudaStream_t st);
int launch_dense_prepare(const float* row_amax, int T, int32_t* offsets, float* seg_amax, cudaStream_t st);
int launch_quant_rows_from_amax(const void* x, const int32_t* row_expert, const float* seg_amax, int M, int W,
                                void* xq, float* scales_out, cudaStream_t st);
size_t gemm_scratch_bytes(int M, int D, int H, int E);
// Handed to launch_gateup by the whole-forward entry points: where the requantised h, its scales and the
// zero-initialised arrival counter of the fused small-batch kernel live.  *requant_done tells the caller
// whether hq and scale_h were produced (then no 16-bit h exists and no requantisation pass is needed).
struct FusedRequant {
  void* hq;
  float* scale_h;
  unsigned int* arrivals;
};
int launch_gateup(const void* xq, const int32_t* offsets, const float* sx, const void* wg, const void* wu,
                  const float* sg, const float* su, int M, int D, int H, int E, void* h, float* amax_h,
                  int32_t* status, void* scratch, cudaStream_t st, const FusedRequant* fr = nullptr,
                  bool* requant_done = nullptr);
// What the weighted combine needs; handed to launch_down so that a split-K down projection can sum its
// slabs and combine in one kernel (*fused reports whether it did; otherwise the caller combines).
struct CombineArgs {
  const int32_t* pos;
  const float* weights;
  int T, K;
  void* out;
  float scale;
  const void* residual;
  // for a combine that starts in the down projection's epilogue: the routing weight and the slot of every
  // permuted row; reduce = add the weighted rows straight into `out` (zeroed by the caller) from the epilogue
  const float* row_w = nullptr;
  const int32_t* row_slot = nullptr;
  bool reduce = false;
  int n_tail = 0;      // always-on slots at the end of every token's K: added after the scale (see combine_kernel)
};
// What launch_down left for the caller to do about the combine.
enum CombineState {
  kCombinePlain = 0,        // y holds unweighted rows: run the weighted combine
  kCombinePreweighted = 1,  // y holds rows already multiplied by their routing weight: run the sum-only combine
  kCombineDone = 2          // out is complete
};
// One device pointer per rank of an expert-parallel group, passed to kernels by value.
constexpr int kMaxPeers = 8;
struct PeerPtrs {
  void* p[kMaxPeers];
};

// Expert-parallel return route for the down projection's epilogue: counts[s*E+e] rows of segment e came
// from rank s and go back to rows first[s*E+e]... of home[s] (device pointers valid on this GPU).
struct HomeRoute {
  int n_ranks;
  const int32_t* counts;
  const int32_t* first;
  void* const* home;
};
int launch_down(const void* hq, const int32_t* offsets, const float* sh, const void* wd, const float* sd,
                int M, int D, int H, int E, void* y, int32_t* status, void* scratch, cudaStream_t st,
                const CombineArgs* combine = nullptr, int* combine_state = nullptr, const HomeRoute* route = nullptr);

// 128x128 block-scale recipe
int launch_gather_quant_group(const void* x, const int32_t* row_slot, int M, int D, int K, void* xq, float* x_inv,
                              cudaStream_t st);
int launch_quant_scatter_group(const void* x, const int32_t* pos, int T, int D, int K, void* xq, float* x_inv,
                               cudaStream_t st);
// Small batches of the block-scale recipe (a handful of rows per expert): operand-swapped tiles, see
// grouped_gemm_block_small_sm100.cu.  launch_gateup_block / launch_down_block pick them by themselves.
bool block_small_applicable(int M, int Kdim, int E);
int launch_gateup_block_small(const void* xq, const float* x_inv, const int32_t* offsets, const void* wg, const void* wu,
                              const float* inv_g, const float* inv_u, int M, int D, int H, int E, void* hq,
                              float* h_inv, int32_t* status, cudaStream_t st);
int launch_down_block_small(const void* hq, const float* h_inv, const int32_t* offsets, const void* wd,
                            const float* inv_d, int M, int D, int H, int E, void* y, int32_t* status, cudaStream_t st);
int launch_gateup_block(const void* xq, const float* x_inv, const int32_t* offsets, const void* wg, const void* wu,
                        const float* inv_g, const float* inv_u, int M, int D, int H, int E, void* hq, float* h_inv,
                        int32_t* status, cudaStream_t st);
int launch_down_block(const void* hq, const float* h_inv, const int32_t* offsets, const void* wd,
                      const float* inv_d, int M, int D, int H, int E, void* y, int32_t* status, cudaStream_t st,
                      const HomeRoute* route = nullptr);
// token-order codes + group scales -> the rows' places in their owners' buffers (block recipe dispatch)
int launch_scatter_rows_group_peers(const void* xq_tok, const float* inv_tok, const int32_t* pos,
                                    const int32_t* indices, const int32_t* delta, int T, int D, int K,
                                    int experts_per_rank, void* const* xq_of_rank, void* const* inv_of_rank,
                                    int n_ranks, int rows_cap, int32_t* status, cudaStream_t st);

// Monotone map of a float onto unsigned integers (a < b  <=>  key(a) < key(b); -0 is folded onto +0 first).
__device__ __forceinline__ unsigned order_key(float v) {
  const unsigned u = __float_as_uint(v + 0.0f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float order_value(unsigned k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

}  // namespace bwmoe
