// extern "C" surface of libbwmoe.so: argument checks, workspace layout, and the
// composition of the stage kernels into the whole-block forward.
#include <algorithm>
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include <mutex>

#include "sm100_gemm.cuh"

namespace bwmoe {
namespace sm100 {
namespace {
struct MapEntry {
  int kind = -1, dev = -1, d0 = 0, d1 = 0, d2 = 0;
  const void* base = nullptr;
  CUtensorMap map;
};
constexpr int kMapCache = 64;
MapEntry g_maps[kMapCache];
int g_map_next = 0;
std::mutex g_map_mu;
int current_device() {
  int dev = -1;
  return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}
}  // namespace

bool tensor_map_lookup(int kind, const void* base, int d0, int d1, int d2, CUtensorMap* out) {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_map_mu);
  for (const MapEntry& m : g_maps)
    if (m.kind == kind && m.base == base && m.dev == dev && m.d0 == d0 && m.d1 == d1 && m.d2 == d2) {
      *out = m.map;
      return true;
    }
  return false;
}
void tensor_map_store(int kind, const void* base, int d0, int d1, int d2, const CUtensorMap& map) {
  const int dev = current_device();
  std::lock_guard<std::mutex> lock(g_map_mu);
  MapEntry& m = g_maps[g_map_next];
  g_map_next = (g_map_next + 1) % kMapCache;
  m.kind = kind, m.dev = dev, m.base = base, m.d0 = d0, m.d1 = d1, m.d2 = d2, m.map = map;
}
void tensor_map_clear() {
  std::lock_guard<std::mutex> lock(g_map_mu);
  for (MapEntry& m : g_maps) m.kind = -1;
}
}  // namespace sm100

namespace {
thread_local char g_error[512] = "";
}

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

namespace {
// SMs the persistent GEMM grids leave free (for collectives running beside them).  Per calling thread:
// the launches of one forward are issued by one thread, so two threads never see each other's setting.
thread_local int g_sm_reserve = 0;
}
namespace {
std::atomic<long long> g_launches{0};
}
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int gemm_sm_budget() { return std::max(1, sm_count() - g_sm_reserve); }

int sm_count() {
  // per-device cache; the library may be used from one process per GPU or several devices
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

namespace {

constexpr size_t kAlign = 1024;
inline size_t align_up(size_t v) { return (v + kAlign - 1) / kAlign * kAlign; }

// Workspace layout.  The first block (status .. amax_h) is cleared by one memset per call.
struct Layout {
  size_t status, amax_x, amax_h, arrivals, zero_end;
  size_t offsets, scale_x, scale_h, topk_idx, topk_w, row_amax, pos, row_slot, row_expert, row_w;
  size_t plan_scratch, gemm_scratch, router_scratch, router_scratch_bytes, xq, h, hq, y, total;
};

// n_shared: the last n_shared experts / slots are always-on groups; the router works on the others only
bool make_layout(int T, int D, int H, int E, int K, Layout* L, int n_shared = 0) {
  if (T <= 0 || D <= 0 || H <= 0 || E <= 0 || K <= 0 || E > 256 || K > E || K > 32) return false;
  if ((long long)T * K >= (1ll << 31)) return false;
  const size_t M = (size_t)T * K;
  size_t o = 0;
  auto take = [&](size_t bytes) {
    const size_t at = o;
    o = align_up(o + bytes);
    return at;
  };
  L->status = take(16);
  L->amax_x = take(sizeof(float) * E);
  L->amax_h = take(sizeof(float) * E);
  L->arrivals = take(16);
  L->zero_end = o;
  L->offsets = take(sizeof(int32_t) * (E + 1));
  L->scale_x = take(sizeof(float) * E);
  L->scale_h = take(sizeof(float) * E);
  L->topk_idx = take(sizeof(int32_t) * M);
  L->topk_w = take(sizeof(float) * M);
  L->row_amax = take(sizeof(float) * T);
  L->pos = take(sizeof(int32_t) * M);
  L->row_slot = take(sizeof(int32_t) * M);
  L->row_expert = take(sizeof(int32_t) * M);
  L->row_w = take(sizeof(float) * M);
  L->plan_scratch = take(plan_scratch_bytes(T, E, K));
  L->gemm_scratch = take(gemm_scratch_bytes((int)M, D, H, E));
  L->xq = take(M * D);
  L->h = take(M * H * 2);
  L->hq = take(M * H);
  L->y = take(M * D * 2);
  // last, so that no other offset depends on how many of the experts the router sees
  L->router_scratch_bytes = router_scratch_bytes(T, D, E - n_shared, K - n_shared);
  L->router_scratch = take(L->router_scratch_bytes);
  L->total = o;
  return true;
}

// Workspace of the block-scale recipe: no bf16 h, no segment statistics; per-row group scales instead.
struct BlockLayout {
  size_t status, zero_end, offsets, topk_idx, topk_w, row_amax, pos, row_slot, row_expert, plan_scratch;
  size_t router_scratch, router_scratch_bytes, xq, x_inv, hq, h_inv, y, total;
};

bool make_block_layout(int T, int D, int H, int E, int K, BlockLayout* L) {
  if (T <= 0 || D <= 0 || H <= 0 || E <= 0 || K <= 0 || E > 256 || K > E || K > 32) return false;
  if ((long long)T * K >= (1ll << 31)) return false;
  const size_t M = (size_t)T * K;
  size_t o = 0;
  auto take = [&](size_t bytes) {
    const size_t at = o;
    o = align_up(o + bytes);
    return at;
  };
  L->status = take(16);
  L->zero_end = o;
  L->offsets = take(sizeof(int32_t) * (E + 1));
  L->topk_idx = take(sizeof(int32_t) * M);
  L->topk_w = take(sizeof(float) * M);
  L->row_amax = take(sizeof(float) * T);
  L->pos = take(sizeof(int32_t) * M);
  L->row_slot = take(sizeof(int32_t) * M);
  L->row_expert = take(sizeof(int32_t) * M);
  L->plan_scratch = take(plan_scratch_bytes(T, E, K));
  L->router_scratch_bytes = router_scratch_bytes(T, D, E, K);
  L->router_scratch = take(L->router_scratch_bytes);
  L->xq = take(M * D);
  L->x_inv = take(sizeof(float) * M * ((D + 127) / 128));
  L->hq = take(M * H);
  L->h_inv = take(sizeof(float) * M * ((H + 127) / 128));
  L->y = take(M * D * 2);
  L->total = o;
  return true;
}

template <class T>
T* at(void* ws, size_t off) {
  return reinterpret_cast<T*>(static_cast<uint8_t*>(ws) + off);
}

int check_forward_args(const char* who, const void* x, const void* wg, const void* wu, const void* wd,
                       const float* sg, const float* su, const float* sd, int T, int D, int H, int E, int K,
                       void* out, void* ws, size_t ws_bytes, Layout* L, size_t extra, int n_shared = 0) {
  BWMOE_REQUIRE(T > 0 && D > 0 && H > 0 && E > 0 && K > 0, BWMOE_ERR_BAD_SHAPE, "%s: T=%d D=%d H=%d E=%d K=%d",
                who, T, D, H, E, K);
  BWMOE_REQUIRE(D % 16 == 0 && H % 16 == 0, BWMOE_ERR_BAD_SHAPE, "%s: D=%d and H=%d must be multiples of 16", who, D, H);
  BWMOE_REQUIRE(E <= 256, BWMOE_ERR_UNSUPPORTED, "%s: E=%d > 256 experts", who, E);
  BWMOE_REQUIRE(K <= E && K <= 32, BWMOE_ERR_UNSUPPORTED, "%s: top_k=%d must be <= min(E,32)", who, K);
  BWMOE_REQUIRE(x && wg && wu && wd && sg && su && sd && out, BWMOE_ERR_NULL, "%s: null pointer", who);
  BWMOE_REQUIRE(make_layout(T, D, H, E, K, L, n_shared), BWMOE_ERR_BAD_SHAPE, "%s: shape not representable", who);
  BWMOE_REQUIRE(ws != nullptr && ws_bytes >= L->total + extra, BWMOE_ERR_WORKSPACE,
                "%s: workspace of %zu bytes given, %zu needed", who, ws_bytes, L->total + extra);
  BWMOE_REQUIRE(aligned16(x) && aligned16(out) && aligned16(wg) && aligned16(wu) && aligned16(wd) &&
                    (reinterpret_cast<uintptr_t>(ws) % 256 == 0),
                BWMOE_ERR_BAD_ALIGN, "%s: tensors must be 16-byte and the workspace 256-byte aligned", who);
  return BWMOE_OK;
}

// permute plan -> quantise -> gate/up -> requant -> down -> combine, given routing in the workspace
int run_pipeline(const void* x, const float* weights, const int32_t* indices, const float* row_amax,
                 const void* wg, const void* wu, const void* wd, const float* sg, const float* su,
                 const float* sd, int T, int D, int H, int E, int K, void* out, void* ws, const Layout& L,
                 cudaStream_t st, float out_scale = 1.0f, const void* residual = nullptr, unsigned flags = 0,
                 int n_shared = 0) {
  const int M = T * K;
  int32_t* status = at<int32_t>(ws, L.status);
  int32_t* offsets = at<int32_t>(ws, L.offsets);
  int32_t* pos = at<int32_t>(ws, L.pos);
  int32_t* row_slot = at<int32_t>(ws, L.row_slot);
  int32_t* row_expert = at<int32_t>(ws, L.row_expert);
  float* amax_x = at<float>(ws, L.amax_x);
  float* amax_h = at<float>(ws, L.amax_h);
  float* scale_x = at<float>(ws, L.scale_x);
  float* scale_h = at<float>(ws, L.scale_h);
  int rc;
  if ((rc = launch_plan(indices, row_amax, T, E, K, offsets, pos, row_slot, row_expert, amax_x, status,
                        at<void>(ws, L.plan_scratch), st, scale_x)))
    return rc;
  float* row_w = at<float>(ws, L.row_w);
  if ((rc = launch_scatter_quant(x, pos, indices, scale_x, T, D, K, at<void>(ws, L.xq), st, weights, row_w))) return rc;
  const FusedRequant fr{at<void>(ws, L.hq), scale_h, at<unsigned int>(ws, L.arrivals)};
  bool requant_done = false;
  // The always-on groups E-n_shared .. E-1 are column pieces of ONE shared MLP whose h is quantised with one
  // scale (FP8SharedExpert, shared_expert_fp8.py:64): their maxima are merged before the requantisation,
  // which therefore cannot be fused into the small-batch SwiGLU kernel.
  const bool merge = n_shared > 1;
  if ((rc = launch_gateup(at<void>(ws, L.xq), offsets, scale_x, wg, wu, sg, su, M, D, H, E, at<void>(ws, L.h),
                          amax_h, status, at<void>(ws, L.gemm_scratch), st, merge ? nullptr : &fr,
                          merge ? nullptr : &requant_done)))
    return rc;
  if (merge && (rc = launch_merge_amax(amax_h, E - n_shared, n_shared, st))) return rc;
  // scale_h is derived from amax_h inside the requantisation kernel
  if (!requant_done &&
      (rc = launch_requant(at<void>(ws, L.h), row_expert, amax_h, M, H, at<void>(ws, L.hq), st, scale_h)))
    return rc;
  CombineArgs ca{pos, weights, T, K, out, out_scale, residual};
  ca.row_w = row_w;
  ca.row_slot = row_slot;
  ca.n_tail = n_shared;
  ca.reduce = (flags & BWMOE_FLAG_REDUCE_COMBINE) != 0 && out_scale == 1.0f && residual == nullptr && M > 64;
  if (ca.reduce) BWMOE_CUDA_OK(cudaMemsetAsync(out, 0, (size_t)T * D * 2, st));   // the epilogue adds into it
  int state = kCombinePlain;
  if ((rc = launch_down(at<void>(ws, L.hq), offsets, scale_h, wd, sd, M, D, H, E, at<void>(ws, L.y), status,
                        at<void>(ws, L.gemm_scratch), st, &ca, &state)))
    return rc;
  if (state == kCombineDone) return BWMOE_OK;
  return launch_combine(at<void>(ws, L.y), pos, weights, T, D, K, out, st, out_scale, residual,
                        state == kCombinePreweighted, n_shared);
}

// max|x| per row, for callers that bring their own routing
__global__ void row_amax_kernel(const __nv_bfloat16* __restrict__ x, int T, int D, float* __restrict__ row_amax) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= T) return;
  const int lane = threadIdx.x & 31;
  float m = 0.f;
  for (int d = lane; d < D; d += 32) m = fmaxf(m, fabsf(__bfloat162float(x[(size_t)t * D + d])));
  for (int off = 16; off; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
  if (lane == 0) row_amax[t] = m;
}

// Expert ids of the whole model -> slots of a resident expert pool.  An id outside [0, n_ids) or an
// expert without a slot (remap < 0) becomes -1, which the plan reports as BWMOE_STATUS_BAD_EXPERT.
__global__ void remap_ids_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ remap, int n_ids,
                                 int n, int32_t* __restrict__ slots) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int id = ids[i];
  slots[i] = (id >= 0 && id < n_ids) ? remap[id] : -1;
}

// The block-scale pipeline behind the routing: plan -> per-token group quantisation -> rows into expert
// order -> gate/up (+ SwiGLU + requant) -> down -> combine.
int run_block_pipeline(const void* x, const float* weights, const int32_t* indices, const void* wg, const void* wu,
                       const void* wd, const float* inv_g, const float* inv_u, const float* inv_d, int T, int D,
                       int H, int E, int K, void* out, void* ws, const BlockLayout& L, cudaStream_t st) {
  const int M = T * K;
  int32_t* status = at<int32_t>(ws, L.status);
  int32_t* offsets = at<int32_t>(ws, L.offsets);
  int rc;
  if ((rc = launch_plan(indices, nullptr, T, E, K, offsets, at<int32_t>(ws, L.pos), at<int32_t>(ws, L.row_slot),
                        at<int32_t>(ws, L.row_expert), nullptr, status, at<void>(ws, L.plan_scratch), st)))
    return rc;
  // token-major: a row is read and quantised once, its codes and group scales written to its K rows
  if ((rc = launch_quant_scatter_group(x, at<int32_t>(ws, L.pos), T, D, K, at<void>(ws, L.xq), at<float>(ws, L.x_inv), st)))
    return rc;
  if ((rc = launch_gateup_block(at<void>(ws, L.xq), at<float>(ws, L.x_inv), offsets, wg, wu, inv_g, inv_u, M, D, H, E,
                                at<void>(ws, L.hq), at<float>(ws, L.h_inv), status, st)))
    return rc;
  if ((rc = launch_down_block(at<void>(ws, L.hq), at<float>(ws, L.h_inv), offsets, wd, inv_d, M, D, H, E,
                              at<void>(ws, L.y), status, st)))
    return rc;
  return launch_combine(at<void>(ws, L.y), at<int32_t>(ws, L.pos), weights, T, D, K, out, st);
}

int check_block_args(const char* who, const void* x, const void* wg, const void* wu, const void* wd,
                     const float* inv_g, const float* inv_u, const float* inv_d, int T, int D, int H, int E, int K,
                     void* out, void* ws, size_t ws_bytes, BlockLayout* L) {
  BWMOE_REQUIRE(T > 0 && D > 0 && H > 0 && E > 0 && K > 0, BWMOE_ERR_BAD_SHAPE, "%s: T=%d D=%d H=%d E=%d K=%d", who,
                T, D, H, E, K);
  BWMOE_REQUIRE(D % 16 == 0 && H % 16 == 0, BWMOE_ERR_BAD_SHAPE, "%s: D=%d and H=%d must be multiples of 16", who, D, H);
  BWMOE_REQUIRE(E <= 256, BWMOE_ERR_UNSUPPORTED, "%s: E=%d > 256 experts", who, E);
  BWMOE_REQUIRE(K <= E && K <= 32, BWMOE_ERR_UNSUPPORTED, "%s: top_k=%d must be <= min(E,32)", who, K);
  BWMOE_REQUIRE(x && wg && wu && wd && inv_g && inv_u && inv_d && out, BWMOE_ERR_NULL, "%s: null pointer", who);
  BWMOE_REQUIRE(make_block_layout(T, D, H, E, K, L), BWMOE_ERR_BAD_SHAPE, "%s: shape not representable", who);
  BWMOE_REQUIRE(ws != nullptr && ws_bytes >= L->total, BWMOE_ERR_WORKSPACE,
                "%s: workspace of %zu bytes given, %zu needed", who, ws_bytes, L->total);
  BWMOE_REQUIRE(aligned16(x) && aligned16(out) && aligned16(wg) && aligned16(wu) && aligned16(wd) &&
                    (reinterpret_cast<uintptr_t>(ws) % 256 == 0),
                BWMOE_ERR_BAD_ALIGN, "%s: tensors must be 16-byte and the workspace 256-byte aligned", who);
  return BWMOE_OK;
}

}  // namespace
}  // namespace bwmoe

using namespace bwmoe;

extern "C" {

int bwmoe_version(void) { return BWMOE_VERSION; }

int bwmoe_set_sm_reserve(int n) {
  BWMOE_REQUIRE(n >= 0 && n < 128, BWMOE_ERR_BAD_SHAPE, "set_sm_reserve: %d out of range", n);
  g_sm_reserve = n;
  return BWMOE_OK;
}

int bwmoe_invalidate(void) {
  sm100::tensor_map_clear();
  return BWMOE_OK;
}

long long bwmoe_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int bwmoe_last_error(char* buf, size_t len) {
  const size_t n = strlen(g_error);
  if (buf != nullptr && len > 0) {
    const size_t c = std::min(n, len - 1);
    memcpy(buf, g_error, c);
    buf[c] = '\0';
  }
  return (int)n;
}

size_t bwmoe_workspace_bytes(int T, int D, int H, int E, int K) {
  Layout L;
  if (D % 16 != 0 || H % 16 != 0 || !make_layout(T, D, H, E, K, &L)) return 0;
  return L.total;
}

size_t bwmoe_workspace_bytes_shared(int T, int D, int H, int E, int K, int S) {
  Layout L;
  if (S < 1 || D % 16 != 0 || H % 16 != 0 || !make_layout(T, D, H, E + S, K + S, &L, S)) return 0;
  return L.total;
}

size_t bwmoe_workspace_bytes_host(int T, int D, int H, int E, int K) {
  const size_t base = bwmoe_workspace_bytes(T, D, H, E, K);
  return base == 0 ? 0 : base + 2 * align_up((size_t)T * D * 2);
}

int bwmoe_workspace_view(void* ws, int T, int D, int H, int E, int K, int which, void** ptr, size_t* bytes) {
  Layout L;
  BWMOE_REQUIRE(ws && ptr && bytes, BWMOE_ERR_NULL, "workspace_view: null pointer");
  BWMOE_REQUIRE(make_layout(T, D, H, E, K, &L), BWMOE_ERR_BAD_SHAPE, "workspace_view: bad shape");
  const size_t M = (size_t)T * K;
  size_t off = 0, n = 0;
  switch (which) {
    case BWMOE_WS_STATUS: off = L.status, n = 16; break;
    case BWMOE_WS_OFFSETS: off = L.offsets, n = 4 * (size_t)(E + 1); break;
    case BWMOE_WS_TOPK_IDX: off = L.topk_idx, n = 4 * M; break;
    case BWMOE_WS_TOPK_W: off = L.topk_w, n = 4 * M; break;
    case BWMOE_WS_POS: off = L.pos, n = 4 * M; break;
    case BWMOE_WS_ROW_SLOT: off = L.row_slot, n = 4 * M; break;
    case BWMOE_WS_SCALE_X: off = L.scale_x, n = 4 * (size_t)E; break;
    case BWMOE_WS_SCALE_H: off = L.scale_h, n = 4 * (size_t)E; break;
    case BWMOE_WS_XQ: off = L.xq, n = M * D; break;
    case BWMOE_WS_HQ: off = L.hq, n = M * H; break;
    case BWMOE_WS_H: off = L.h, n = 2 * M * H; break;
    case BWMOE_WS_Y: off = L.y, n = 2 * M * D; break;
    case BWMOE_WS_ROW_EXPERT: off = L.row_expert, n = 4 * M; break;
    default: return set_error(BWMOE_ERR_UNSUPPORTED, "workspace_view: unknown selector %d", which);
  }
  *ptr = static_cast<uint8_t*>(ws) + off;
  *bytes = n;
  return BWMOE_OK;
}

int bwmoe_read_status(void* ws, void* stream, int32_t* status) {
  BWMOE_REQUIRE(ws && status, BWMOE_ERR_NULL, "read_status: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BWMOE_CUDA_OK(cudaMemcpyAsync(status, ws, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  BWMOE_CUDA_OK(cudaStreamSynchronize(st));
  return BWMOE_OK;
}

size_t bwmoe_router_scratch_bytes(int T, int D, int E, int K) {
  if (T <= 0 || D <= 0 || E <= 0 || K <= 0) return 0;
  return router_scratch_bytes(T, D, E, K);
}

int bwmoe_router(const void* x, const void* wg, int T, int D, int E, int K, float* weights, int32_t* indices,
                 float* row_amax, void* scratch, size_t scratch_bytes, void* stream) {
  return launch_router(x, wg, T, D, E, K, weights, indices, row_amax, static_cast<cudaStream_t>(stream), scratch,
                       scratch_bytes, nullptr);
}

size_t bwmoe_router_scratch_bytes_as(int T, int D, int E, int K, int T_as) {
  if (T <= 0 || D <= 0 || E <= 0 || K <= 0) return 0;
  return router_scratch_bytes(T, D, E, K, T_as);
}

int bwmoe_router_as(const void* x, const void* wg, int T, int D, int E, int K, int T_as, float* weights,
                    int32_t* indices, float* row_amax, void* scratch, size_t scratch_bytes, void* stream) {
  return launch_router(x, wg, T, D, E, K, weights, indices, row_amax, static_cast<cudaStream_t>(stream), scratch,
                       scratch_bytes, nullptr, T_as);
}

int bwmoe_moe_forward(const void* x, const void* w_gate, const void* wg, const void* wu, const void* wd,
                      const float* sg, const float* su, const float* sd, int T, int D, int H, int E, int K,
                      void* out, void* ws, size_t ws_bytes, void* stream) {
  Layout L;
  if (int rc = check_forward_args("moe_forward", x, wg, wu, wd, sg, su, sd, T, D, H, E, K, out, ws, ws_bytes, &L, 0))
    return rc;
  BWMOE_REQUIRE(w_gate != nullptr, BWMOE_ERR_NULL, "moe_forward: w_gate is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  float* weights = at<float>(ws, L.topk_w);
  int32_t* indices = at<int32_t>(ws, L.topk_idx);
  float* row_amax = at<float>(ws, L.row_amax);
  if (int rc = launch_router(x, w_gate, T, D, E, K, weights, indices, row_amax, st, at<void>(ws, L.router_scratch),
                             L.router_scratch_bytes, at<int32_t>(ws, L.status)))
    return rc;
  return run_pipeline(x, weights, indices, row_amax, wg, wu, wd, sg, su, sd, T, D, H, E, K, out, ws, L, st);
}

int bwmoe_moe_forward_flags(const void* x, const void* w_gate, const void* wg, const void* wu, const void* wd,
                            const float* sg, const float* su, const float* sd, int T, int D, int H, int E, int K,
                            void* out, void* ws, size_t ws_bytes, void* stream, unsigned flags) {
  Layout L;
  if (int rc = check_forward_args("moe_forward_flags", x, wg, wu, wd, sg, su, sd, T, D, H, E, K, out, ws, ws_bytes, &L, 0))
    return rc;
  BWMOE_REQUIRE(w_gate != nullptr, BWMOE_ERR_NULL, "moe_forward_flags: w_gate is null");
  BWMOE_REQUIRE((flags & ~BWMOE_FLAG_REDUCE_COMBINE) == 0, BWMOE_ERR_UNSUPPORTED, "moe_forward_flags: unknown flag bits %#x", flags);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  float* weights = at<float>(ws, L.topk_w);
  int32_t* indices = at<int32_t>(ws, L.topk_idx);
  float* row_amax = at<float>(ws, L.row_amax);
  if (int rc = launch_router(x, w_gate, T, D, E, K, weights, indices, row_amax, st, at<void>(ws, L.router_scratch),
                             L.router_scratch_bytes, at<int32_t>(ws, L.status)))
    return rc;
  return run_pipeline(x, weights, indices, row_amax, wg, wu, wd, sg, su, sd, T, D, H, E, K, out, ws, L, st, 1.0f, nullptr,
                      flags);
}

int bwmoe_moe_forward_shared(const void* x, const void* w_gate, const void* wg, const void* wu, const void* wd,
                             const float* sg, const float* su, const float* sd, int T, int D, int H, int E, int K,
                             int S, float routed_scale, void* out, void* ws, size_t ws_bytes, void* stream) {
  Layout L;
  BWMOE_REQUIRE(S >= 1 && E >= 1 && K >= 1, BWMOE_ERR_BAD_SHAPE, "moe_forward_shared: E=%d K=%d S=%d", E, K, S);
  BWMOE_REQUIRE(K <= E, BWMOE_ERR_UNSUPPORTED, "moe_forward_shared: top_k=%d > %d routed experts", K, E);
  if (int rc = check_forward_args("moe_forward_shared", x, wg, wu, wd, sg, su, sd, T, D, H, E + S, K + S, out, ws,
                                  ws_bytes, &L, 0, S))
    return rc;
  BWMOE_REQUIRE(w_gate != nullptr, BWMOE_ERR_NULL, "moe_forward_shared: w_gate is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  // routing of the E routed experts into scratch that later stages overwrite (pos, row_w), then the S always-on
  // slots are appended: indices / weights [T, K+S]
  int32_t* idx_r = at<int32_t>(ws, L.pos);
  float* w_r = at<float>(ws, L.row_w);
  float* weights = at<float>(ws, L.topk_w);
  int32_t* indices = at<int32_t>(ws, L.topk_idx);
  float* row_amax = at<float>(ws, L.row_amax);
  if (int rc = launch_router(x, w_gate, T, D, E, K, w_r, idx_r, row_amax, st, at<void>(ws, L.router_scratch),
                             L.router_scratch_bytes, at<int32_t>(ws, L.status)))
    return rc;
  if (int rc = launch_append_shared_slots(idx_r, w_r, T, K, E, S, indices, weights, st)) return rc;
  return run_pipeline(x, weights, indices, row_amax, wg, wu, wd, sg, su, sd, T, D, H, E + S, K + S, out, ws, L, st,
                      routed_scale, nullptr, 0, S);
}

int bwmoe_moe_forward_ex(const void* x, const void* w_gate, const void* wg, const void* wu, const void* wd,
                         const float* sg, const float* su, const float* sd, int T, int D, int H, int E, int K,
                         float routed_scale, const void* residual, void* out, void* ws, size_t ws_bytes,
                         void* stream) {
  Layout L;
  if (int rc = check_forward_args("moe_forward_ex", x, wg, wu, wd, sg, su, sd, T, D, H, E, K, out, ws, ws_bytes, &L, 0))
    return rc;
  BWMOE_REQUIRE(w_gate != nullptr, BWMOE_ERR_NULL, "moe_forward_ex: w_gate is null");
  BWMOE_REQUIRE(residual == nullptr || aligned16(residual), BWMOE_ERR_BAD_ALIGN, "moe_forward_ex: residual alignment");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  float* weights = at<float>(ws, L.topk_w);
  int32_t* indices = at<int32_t>(ws, L.topk_idx);
  float* row_amax = at<float>(ws, L.row_amax);
  if (int rc = launch_router(x, w_gate, T, D, E, K, weights, indices, row_amax, st, at<void>(ws, L.router_scratch),
                             L.router_scratch_bytes, at<int32_t>(ws, L.status)))
    return rc;
  return run_pipeline(x, weights, indices, row_amax, wg, wu, wd, sg, su, sd, T, D, H, E, K, out, ws, L, st,
                      routed_scale, residual);
}

int bwmoe_dense_mlp(const void* x, const void* wg, const void* wu, const void* wd, const float* sg, const float* su,
                    const float* sd, int T, int D, int H, void* out, void* ws, size_t ws_bytes, void* stream) {
  Layout L;
  if (int rc = check_forward_args("dense_mlp", x, wg, wu, wd, sg, su, sd, T, D, H, 1, 1, out, ws, ws_bytes, &L, 0))
    return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // one segment with every row: row_expert = 0 everywhere, whole-tensor scales for x and h
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  BWMOE_CUDA_OK(cudaMemsetAsync(at<void>(ws, L.row_expert), 0, sizeof(int32_t) * (size_t)T, st));
  float* row_amax = at<float>(ws, L.row_amax);
  int32_t* offsets = at<int32_t>(ws, L.offsets);
  int32_t* status = at<int32_t>(ws, L.status);
  row_amax_kernel<<<ceil_div(T, 8), 256, 0, counted(st)>>>(static_cast<const __nv_bfloat16*>(x), T, D, row_amax);
  BWMOE_CUDA_OK(cudaGetLastError());
  int rc;
  if ((rc = launch_dense_prepare(row_amax, T, offsets, at<float>(ws, L.amax_x), st))) return rc;
  if ((rc = launch_quant_rows_from_amax(x, at<int32_t>(ws, L.row_expert), at<float>(ws, L.amax_x), T, D,
                                        at<void>(ws, L.xq), at<float>(ws, L.scale_x), st)))
    return rc;
  const FusedRequant fr{at<void>(ws, L.hq), at<float>(ws, L.scale_h), at<unsigned int>(ws, L.arrivals)};
  bool requant_done = false;
  if ((rc = launch_gateup(at<void>(ws, L.xq), offsets, at<float>(ws, L.scale_x), wg, wu, sg, su, T, D, H, 1,
                          at<void>(ws, L.h), at<float>(ws, L.amax_h), status, at<void>(ws, L.gemm_scratch), st, &fr,
                          &requant_done)))
    return rc;
  if (!requant_done &&
      (rc = launch_requant(at<void>(ws, L.h), at<int32_t>(ws, L.row_expert), at<float>(ws, L.amax_h), T, H,
                           at<void>(ws, L.hq), st, at<float>(ws, L.scale_h))))
    return rc;
  return launch_down(at<void>(ws, L.hq), offsets, at<float>(ws, L.scale_h), wd, sd, T, D, H, 1, out, status,
                     at<void>(ws, L.gemm_scratch), st);
}

int bwmoe_moe_forward_routed(const void* x, const float* weights, const int32_t* indices, const void* wg,
                             const void* wu, const void* wd, const float* sg, const float* su, const float* sd,
                             int T, int D, int H, int E, int K, void* out, void* ws, size_t ws_bytes,
                             void* stream) {
  Layout L;
  if (int rc = check_forward_args("moe_forward_routed", x, wg, wu, wd, sg, su, sd, T, D, H, E, K, out, ws,
                                  ws_bytes, &L, 0))
    return rc;
  BWMOE_REQUIRE(weights && indices, BWMOE_ERR_NULL, "moe_forward_routed: routing is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  float* row_amax = at<float>(ws, L.row_amax);
  row_amax_kernel<<<ceil_div(T, 8), 256, 0, counted(st)>>>(static_cast<const __nv_bfloat16*>(x), T, D, row_amax);
  BWMOE_CUDA_OK(cudaGetLastError());
  // keep a copy of the routing in the workspace so that the views stay meaningful
  BWMOE_CUDA_OK(cudaMemcpyAsync(at<void>(ws, L.topk_idx), indices, sizeof(int32_t) * (size_t)T * K,
                                cudaMemcpyDeviceToDevice, st));
  BWMOE_CUDA_OK(cudaMemcpyAsync(at<void>(ws, L.topk_w), weights, sizeof(float) * (size_t)T * K,
                                cudaMemcpyDeviceToDevice, st));
  return run_pipeline(x, weights, indices, row_amax, wg, wu, wd, sg, su, sd, T, D, H, E, K, out, ws, L, st);
}

int bwmoe_moe_forward_routed_remap(const void* x, const float* weights, const int32_t* expert_ids,
                                   const int32_t* remap, int n_experts_total, const void* wg, const void* wu,
                                   const void* wd, const float* sg, const float* su, const float* sd, int T, int D,
                                   int H, int n_slots, int K, void* out, void* ws, size_t ws_bytes, void* stream) {
  Layout L;
  if (int rc = check_forward_args("moe_forward_routed_remap", x, wg, wu, wd, sg, su, sd, T, D, H, n_slots, K, out, ws,
                                  ws_bytes, &L, 0))
    return rc;
  BWMOE_REQUIRE(weights && expert_ids && remap, BWMOE_ERR_NULL, "moe_forward_routed_remap: routing or remap is null");
  BWMOE_REQUIRE(n_experts_total > 0, BWMOE_ERR_BAD_SHAPE, "moe_forward_routed_remap: %d experts", n_experts_total);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int M = T * K;
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  float* row_amax = at<float>(ws, L.row_amax);
  row_amax_kernel<<<ceil_div(T, 8), 256, 0, counted(st)>>>(static_cast<const __nv_bfloat16*>(x), T, D, row_amax);
  BWMOE_CUDA_OK(cudaGetLastError());
  int32_t* slots = at<int32_t>(ws, L.topk_idx);                 // the workspace's routing view holds slot ids
  remap_ids_kernel<<<ceil_div(M, 256), 256, 0, counted(st)>>>(expert_ids, remap, n_experts_total, M, slots);
  BWMOE_CUDA_OK(cudaGetLastError());
  BWMOE_CUDA_OK(cudaMemcpyAsync(at<void>(ws, L.topk_w), weights, sizeof(float) * (size_t)M,
                                cudaMemcpyDeviceToDevice, st));
  return run_pipeline(x, weights, slots, row_amax, wg, wu, wd, sg, su, sd, T, D, H, n_slots, K, out, ws, L, st);
}

int bwmoe_moe_forward_host(const void* h_x, const void* w_gate, const void* wg, const void* wu, const void* wd,
                           const float* sg, const float* su, const float* sd, int T, int D, int H, int E, int K,
                           void* h_out, void* ws, size_t ws_bytes, void* stream) {
  Layout L;
  const size_t act = align_up((size_t)T * D * 2);
  // the device copies of x and out live behind the regular workspace
  BWMOE_REQUIRE(h_x && h_out, BWMOE_ERR_NULL, "moe_forward_host: null host pointer");
  BWMOE_REQUIRE(make_layout(T, D, H, E, K, &L), BWMOE_ERR_BAD_SHAPE, "moe_forward_host: bad shape");
  BWMOE_REQUIRE(ws != nullptr && ws_bytes >= L.total + 2 * act, BWMOE_ERR_WORKSPACE,
                "moe_forward_host: workspace of %zu bytes given, %zu needed", ws_bytes, L.total + 2 * act);
  void* d_x = static_cast<uint8_t*>(ws) + L.total;
  void* d_out = static_cast<uint8_t*>(ws) + L.total + act;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BWMOE_CUDA_OK(cudaMemcpyAsync(d_x, h_x, (size_t)T * D * 2, cudaMemcpyHostToDevice, st));
  if (int rc = bwmoe_moe_forward(d_x, w_gate, wg, wu, wd, sg, su, sd, T, D, H, E, K, d_out, ws, L.total, stream))
    return rc;
  BWMOE_CUDA_OK(cudaMemcpyAsync(h_out, d_out, (size_t)T * D * 2, cudaMemcpyDeviceToHost, st));
  BWMOE_CUDA_OK(cudaStreamSynchronize(st));
  return BWMOE_OK;
}

size_t bwmoe_workspace_bytes_block(int T, int D, int H, int E, int K) {
  BlockLayout L;
  if (D % 16 != 0 || H % 16 != 0 || !make_block_layout(T, D, H, E, K, &L)) return 0;
  return L.total;
}

int bwmoe_workspace_view_block(void* ws, int T, int D, int H, int E, int K, int which, void** ptr, size_t* bytes) {
  BlockLayout L;
  BWMOE_REQUIRE(ws && ptr && bytes, BWMOE_ERR_NULL, "workspace_view_block: null pointer");
  BWMOE_REQUIRE(make_block_layout(T, D, H, E, K, &L), BWMOE_ERR_BAD_SHAPE, "workspace_view_block: bad shape");
  const size_t M = (size_t)T * K;
  size_t off = 0, n = 0;
  switch (which) {
    case BWMOE_WS_STATUS: off = L.status, n = 16; break;
    case BWMOE_WS_OFFSETS: off = L.offsets, n = 4 * (size_t)(E + 1); break;
    case BWMOE_WS_TOPK_IDX: off = L.topk_idx, n = 4 * M; break;
    case BWMOE_WS_TOPK_W: off = L.topk_w, n = 4 * M; break;
    case BWMOE_WS_POS: off = L.pos, n = 4 * M; break;
    case BWMOE_WS_ROW_SLOT: off = L.row_slot, n = 4 * M; break;
    case BWMOE_WS_ROW_EXPERT: off = L.row_expert, n = 4 * M; break;
    case BWMOE_WS_XQ: off = L.xq, n = M * D; break;
    case BWMOE_WS_HQ: off = L.hq, n = M * H; break;
    case BWMOE_WS_Y: off = L.y, n = 2 * M * D; break;
    case BWMOE_WS_X_INV: off = L.x_inv, n = 4 * M * ((D + 127) / 128); break;
    case BWMOE_WS_H_INV: off = L.h_inv, n = 4 * M * ((H + 127) / 128); break;
    default: return set_error(BWMOE_ERR_UNSUPPORTED, "workspace_view_block: selector %d not part of this recipe", which);
  }
  *ptr = static_cast<uint8_t*>(ws) + off;
  *bytes = n;
  return BWMOE_OK;
}

int bwmoe_moe_forward_block(const void* x, const void* w_gate, const void* wg, const void* wu, const void* wd,
                            const float* inv_g, const float* inv_u, const float* inv_d, int T, int D, int H, int E,
                            int K, void* out, void* ws, size_t ws_bytes, void* stream) {
  BlockLayout L;
  if (int rc = check_block_args("moe_forward_block", x, wg, wu, wd, inv_g, inv_u, inv_d, T, D, H, E, K, out, ws,
                                ws_bytes, &L))
    return rc;
  BWMOE_REQUIRE(w_gate != nullptr, BWMOE_ERR_NULL, "moe_forward_block: w_gate is null");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  float* weights = at<float>(ws, L.topk_w);
  int32_t* indices = at<int32_t>(ws, L.topk_idx);
  if (int rc = launch_router(x, w_gate, T, D, E, K, weights, indices, nullptr, st, at<void>(ws, L.router_scratch),
                             L.router_scratch_bytes, at<int32_t>(ws, L.status)))
    return rc;
  return run_block_pipeline(x, weights, indices, wg, wu, wd, inv_g, inv_u, inv_d, T, D, H, E, K, out, ws, L, st);
}

int bwmoe_moe_forward_block_routed(const void* x, const float* weights, const int32_t* expert_ids,
                                   const int32_t* remap, int n_experts_total, const void* wg, const void* wu,
                                   const void* wd, const float* inv_g, const float* inv_u, const float* inv_d, int T,
                                   int D, int H, int n_slots, int K, void* out, void* ws, size_t ws_bytes,
                                   void* stream) {
  BlockLayout L;
  if (int rc = check_block_args("moe_forward_block_routed", x, wg, wu, wd, inv_g, inv_u, inv_d, T, D, H, n_slots, K,
                                out, ws, ws_bytes, &L))
    return rc;
  BWMOE_REQUIRE(weights && expert_ids, BWMOE_ERR_NULL, "moe_forward_block_routed: routing is null");
  BWMOE_REQUIRE(remap == nullptr || n_experts_total > 0, BWMOE_ERR_BAD_SHAPE,
                "moe_forward_block_routed: remap given with %d experts", n_experts_total);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int M = T * K;
  BWMOE_CUDA_OK(cudaMemsetAsync(ws, 0, L.zero_end, st));
  int32_t* slots = at<int32_t>(ws, L.topk_idx);
  if (remap != nullptr) {
    remap_ids_kernel<<<ceil_div(M, 256), 256, 0, counted(st)>>>(expert_ids, remap, n_experts_total, M, slots);
    BWMOE_CUDA_OK(cudaGetLastError());
  } else {
    BWMOE_CUDA_OK(cudaMemcpyAsync(slots, expert_ids, sizeof(int32_t) * (size_t)M, cudaMemcpyDeviceToDevice, st));
  }
  BWMOE_CUDA_OK(cudaMemcpyAsync(at<void>(ws, L.topk_w), weights, sizeof(float) * (size_t)M,
                                cudaMemcpyDeviceToDevice, st));
  return run_block_pipeline(x, weights, slots, wg, wu, wd, inv_g, inv_u, inv_d, T, D, H, n_slots, K, out, ws, L, st);
}

int bwmoe_gather_quant_group(const void* x, const int32_t* row_slot, int M, int D, int K, void* xq, float* x_inv,
                             void* stream) {
  return launch_gather_quant_group(x, row_slot, M, D, K, xq, x_inv, static_cast<cudaStream_t>(stream));
}

int bwmoe_gateup_swiglu_block(const void* xq, const float* x_inv, const int32_t* offsets, const void* wg,
                              const void* wu, const float* inv_g, const float* inv_u, int M, int D, int H, int E,
                              void* hq, float* h_inv, int32_t* status, void* stream) {
  return launch_gateup_block(xq, x_inv, offsets, wg, wu, inv_g, inv_u, M, D, H, E, hq, h_inv, status,
                             static_cast<cudaStream_t>(stream));
}

int bwmoe_down_block(const void* hq, const float* h_inv, const int32_t* offsets, const void* wd, const float* inv_d,
                     int M, int D, int H, int E, void* y, int32_t* status, void* stream) {
  return launch_down_block(hq, h_inv, offsets, wd, inv_d, M, D, H, E, y, status, static_cast<cudaStream_t>(stream));
}

size_t bwmoe_plan_scratch_bytes(int T, int E, int K) {
  if (T <= 0 || E <= 0 || K <= 0) return 0;
  return plan_scratch_bytes(T, E, K);
}

int bwmoe_permute_plan(const int32_t* indices, const float* row_amax, int T, int E, int K, int32_t* offsets,
                       int32_t* pos, int32_t* row_slot, int32_t* row_expert, float* seg_amax, int32_t* status,
                       void* scratch, void* stream) {
  return launch_plan(indices, row_amax, T, E, K, offsets, pos, row_slot, row_expert, seg_amax, status, scratch,
                     static_cast<cudaStream_t>(stream));
}

int bwmoe_permute_plan_static(const int32_t* indices, const float* row_amax, int T, int E, int K,
                              int32_t* offsets, int32_t* pos, int32_t* row_slot, int32_t* row_expert,
                              float* seg_amax, int32_t* status, void* stream) {
  BWMOE_REQUIRE(indices && offsets && pos && row_slot && row_expert && status, BWMOE_ERR_NULL,
                "plan_static: null pointer");
  return launch_plan_static(indices, row_amax, T, E, K, offsets, pos, row_slot, row_expert, seg_amax, status,
                            static_cast<cudaStream_t>(stream));
}

int bwmoe_segment_scales(const float* seg_amax, const int32_t* offsets, int E, float* scales, void* stream) {
  return launch_segment_scales(seg_amax, offsets, E, scales, static_cast<cudaStream_t>(stream));
}

int bwmoe_gather_quant(const void* x, const int32_t* row_slot, const int32_t* row_expert, const float* scales,
                       int M, int D, int K, void* xq, void* stream) {
  return launch_gather_quant(x, row_slot, row_expert, scales, M, D, K, xq, static_cast<cudaStream_t>(stream));
}

size_t bwmoe_gemm_scratch_bytes(int M, int D, int H, int E) {
  if (M <= 0 || D <= 0 || H <= 0 || E <= 0) return 0;
  return gemm_scratch_bytes(M, D, H, E);
}

int bwmoe_gateup_swiglu(const void* xq, const int32_t* offsets, const float* sx, const void* wg, const void* wu,
                        const float* sg, const float* su, int M, int D, int H, int E, void* h, float* amax_h,
                        int32_t* status, void* scratch, void* stream) {
  return launch_gateup(xq, offsets, sx, wg, wu, sg, su, M, D, H, E, h, amax_h, status, scratch,
                       static_cast<cudaStream_t>(stream));
}

int bwmoe_requant(const void* h, const int32_t* row_expert, const float* scales_h, int M, int H, void* hq,
                  void* stream) {
  return launch_requant(h, row_expert, scales_h, M, H, hq, static_cast<cudaStream_t>(stream));
}

int bwmoe_requant_segments(const void* h, const int32_t* offsets, const float* scales_h, int E, int H, void* hq,
                           void* stream) {
  return launch_requant_segments(h, offsets, scales_h, E, H, hq, static_cast<cudaStream_t>(stream));
}

int bwmoe_down(const void* hq, const int32_t* offsets, const float* sh, const void* wd, const float* sd, int M,
               int D, int H, int E, void* y, int32_t* status, void* scratch, void* stream) {
  return launch_down(hq, offsets, sh, wd, sd, M, D, H, E, y, status, scratch, static_cast<cudaStream_t>(stream));
}

int bwmoe_down_peers(const void* hq, const int32_t* offsets, const float* sh, const void* wd, const float* sd, int M,
                     int D, int H, int E, const int32_t* home_counts, const int32_t* home_first,
                     void* const* y_of_rank, int n_ranks, int32_t* status, void* stream) {
  BWMOE_REQUIRE(y_of_rank != nullptr && n_ranks >= 1 && n_ranks <= 8, BWMOE_ERR_UNSUPPORTED, "down_peers: %d ranks", n_ranks);
  const HomeRoute route{n_ranks, home_counts, home_first, y_of_rank};
  return launch_down(hq, offsets, sh, wd, sd, M, D, H, E, y_of_rank[0], status, nullptr, static_cast<cudaStream_t>(stream),
                     nullptr, nullptr, &route);
}

int bwmoe_down_block_peers(const void* hq, const float* h_inv, const int32_t* offsets, const void* wd,
                           const float* inv_d, int M, int D, int H, int E, const int32_t* home_counts,
                           const int32_t* home_first, void* const* y_of_rank, int n_ranks, int32_t* status,
                           void* stream) {
  BWMOE_REQUIRE(y_of_rank != nullptr && n_ranks >= 1 && n_ranks <= 8, BWMOE_ERR_UNSUPPORTED, "down_block_peers: %d ranks", n_ranks);
  const HomeRoute route{n_ranks, home_counts, home_first, y_of_rank};
  return launch_down_block(hq, h_inv, offsets, wd, inv_d, M, D, H, E, y_of_rank[0], status,
                           static_cast<cudaStream_t>(stream), &route);
}

int bwmoe_scatter_rows_group_peers(const void* xq_tok, const float* inv_tok, const int32_t* pos, const int32_t* indices,
                                   const int32_t* delta, int T, int D, int K, int experts_per_rank,
                                   void* const* xq_of_rank, void* const* inv_of_rank, int n_ranks, int rows_cap,
                                   int32_t* status, void* stream) {
  return launch_scatter_rows_group_peers(xq_tok, inv_tok, pos, indices, delta, T, D, K, experts_per_rank, xq_of_rank,
                                         inv_of_rank, n_ranks, rows_cap, status, static_cast<cudaStream_t>(stream));
}

int bwmoe_ep_maps(const int32_t* counts, const int32_t* offsets, int n_ranks, int E, int rank, int32_t* delta,
                  int32_t* offsets_local, int32_t* home_counts, int32_t* home_first, void* stream) {
  return launch_ep_maps(counts, offsets, n_ranks, E, rank, delta, offsets_local, home_counts, home_first,
                        static_cast<cudaStream_t>(stream));
}

int bwmoe_scatter_quant_peers(const void* x, const int32_t* pos, const int32_t* indices, const float* scales,
                              const int32_t* delta, int T, int D, int K, int experts_per_rank,
                              void* const* dst_of_rank, int n_ranks, int rows_cap, int32_t* status, void* stream) {
  return launch_scatter_quant_peers(x, pos, indices, scales, delta, T, D, K, experts_per_rank, dst_of_rank, n_ranks,
                                    rows_cap, status, static_cast<cudaStream_t>(stream));
}

int bwmoe_combine_peers(void* const* y_of_rank, int n_ranks, const int32_t* pos, const int32_t* indices,
                        const float* weights, const int32_t* delta, int experts_per_rank, int T, int D, int K,
                        void* out, void* stream) {
  return launch_combine_peers(y_of_rank, n_ranks, pos, indices, weights, delta, experts_per_rank, T, D, K, out,
                              static_cast<cudaStream_t>(stream));
}

int bwmoe_combine(const void* y, const int32_t* pos, const float* weights, int T, int D, int K, void* out,
                  void* stream) {
  return launch_combine(y, pos, weights, T, D, K, out, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
