/*
 * bwmoe.h -- C ABI of libbwmoe.so: the FP8 Mixture-of-Experts block forward
 * for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - every pointer named d_* is a DEVICE pointer owned by the caller; h_* is a
 *     HOST pointer.  The library allocates no device memory, frees nothing and
 *     dereferences no pointer after a call returns (it remembers base addresses only as
 *     keys of its host-side cache of encoded TMA descriptors, see bwmoe_invalidate).
 *   - all work is enqueued on `stream` (a cudaStream_t passed as void*); no call
 *     synchronises the device except bwmoe_moe_forward_host and bwmoe_read_status.
 *   - every function returns 0 on success or a negative BWMOE_ERR_* code;
 *     bwmoe_last_error() gives the thread-local message of the last failure.
 *   - shapes: T tokens, D hidden, H expert intermediate, E experts, K = top_k,
 *     M = T*K permuted rows.  Tensors are dense row-major:
 *       x[T,D] bf16, w_gate[D,E] bf16, experts_w_gate/up[E,D,H] e4m3,
 *       experts_w_down[E,H,D] e4m3, scales_*[E] fp32 (forward multipliers
 *       448/amax: dequantisation divides by them), out[T,D] bf16.
 *   - device-side anomalies (a bounded wait that ran out, an expert id out of
 *     range) never trap: they set a status word in the workspace which
 *     bwmoe_read_status returns.
 *
 * "replaces" comments cite the reference implementation (paths relative to the
 * reference project's root) whose role each entry point takes over.
 */
#ifndef BWMOE_H_
#define BWMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BWMOE_VERSION 100

enum {
  BWMOE_OK = 0,
  BWMOE_ERR_BAD_SHAPE = -1,   /* a dimension is zero/negative or violates a divisibility rule */
  BWMOE_ERR_BAD_ALIGN = -2,   /* a pointer is not 16-byte aligned */
  BWMOE_ERR_WORKSPACE = -3,   /* workspace null or smaller than bwmoe_workspace_bytes() */
  BWMOE_ERR_UNSUPPORTED = -4, /* valid request the kernels do not cover (e.g. E > 256) */
  BWMOE_ERR_CUDA = -5,        /* a CUDA runtime/driver call failed (message has the detail) */
  BWMOE_ERR_NULL = -6,        /* a required pointer is null */
  BWMOE_ERR_DEVICE_STATUS = -7 /* a kernel reported an anomaly through the status word */
};

/* Bits of the device status word (bwmoe_read_status). */
enum {
  BWMOE_STATUS_WAIT_TIMEOUT = 1, /* a bounded barrier wait inside a GEMM kernel gave up */
  BWMOE_STATUS_BAD_EXPERT = 2,   /* an expert id outside [0,E) was met while planning */
  BWMOE_STATUS_EP_OVERFLOW = 4   /* expert parallel: a rank was sent more rows than its receive buffer holds;
                                    the surplus rows were dropped, not written past the buffer */
};

/* Selectors for bwmoe_workspace_view: intermediates kept in the workspace after
 * a forward, exposed so that tests can check each stage bit for bit. */
enum {
  BWMOE_WS_STATUS = 0,     /* int32[4]                                   */
  BWMOE_WS_OFFSETS = 1,    /* int32[E+1]  segment offsets                */
  BWMOE_WS_TOPK_IDX = 2,   /* int32[T*K]  routing indices                */
  BWMOE_WS_TOPK_W = 3,     /* float[T*K]  routing weights                */
  BWMOE_WS_POS = 4,        /* int32[M]    slot (t*K+k) -> permuted row   */
  BWMOE_WS_ROW_SLOT = 5,   /* int32[M]    permuted row -> slot           */
  BWMOE_WS_SCALE_X = 6,    /* float[E]    per-segment scale of x         */
  BWMOE_WS_SCALE_H = 7,    /* float[E]    per-segment scale of h         */
  BWMOE_WS_XQ = 8,         /* e4m3[M*D]   quantised permuted activations */
  BWMOE_WS_HQ = 9,         /* e4m3[M*H]   quantised SwiGLU output        */
  BWMOE_WS_H = 10,         /* bf16[M*H]   SwiGLU output before requant   */
  BWMOE_WS_Y = 11,         /* bf16[M*D]   down-projection rows (per-tensor recipe, M > 64: already times the routing weight) */
  BWMOE_WS_ROW_EXPERT = 12, /* int32[M]   permuted row -> expert         */
  BWMOE_WS_X_INV = 13,     /* float[M*ceil(D/128)] block recipe: inverse scales of xq */
  BWMOE_WS_H_INV = 14      /* float[M*ceil(H/128)] block recipe: inverse scales of hq */
};

int bwmoe_version(void);

/* For the calling thread: the persistent GEMM kernels it launches from now on use (SM count - n) SMs,
 * leaving n free for kernels that must run beside them (the dispatch of the next token chunk, or NCCL
 * collectives, of the expert-parallel path).  Default 0.  Other threads keep their own setting.
 * No counterpart in the reference (it is single-GPU). */
int bwmoe_set_sm_reserve(int n);

/* Empties the library's cache of encoded TMA descriptors (keyed by base pointer and shape; at most 64, on the
 * host).  Never needed for correctness - a descriptor does not depend on the contents behind its pointer, so
 * an expert cache may swap a slot's weights freely - only to drop entries of memory that has been freed.
 * The one piece of state the library keeps between calls.  No counterpart in the reference. */
int bwmoe_invalidate(void);

/* Number of kernels the library has launched in this process so far (all threads, all devices).
 * For benchmarks that report how many of the library's kernels ran inside a timed region.
 * No counterpart in the reference. */
long long bwmoe_launch_count(void);

/* Copies the calling thread's last error message (NUL-terminated, truncated to
 * `len`) and returns its length. */
int bwmoe_last_error(char* buf, size_t len);

/* Bytes of device workspace one forward of this shape needs (0 on a bad shape). */
size_t bwmoe_workspace_bytes(int T, int D, int H, int E, int K);

/* Workspace size for bwmoe_moe_forward_host (0 on a bad shape). */
size_t bwmoe_workspace_bytes_host(int T, int D, int H, int E, int K);

/* Device pointer and byte size of one intermediate inside a workspace. */
int bwmoe_workspace_view(void* d_workspace, int T, int D, int H, int E, int K, int which,
                         void** d_ptr, size_t* bytes);

/* Blocks until `stream` is idle and returns the device status word (0 = clean)
 * in *status. */
int bwmoe_read_status(void* d_workspace, void* stream, int32_t* status);

/*
 * Fused gate -> softmax -> top-k -> renormalise.
 * replaces: top_k_router / _top_k_gate_kernel, src/blackwell_moe/kernels/routing.py:14-79
 *           (and the torch routing inlined at src/blackwell_moe/kernels/fp8_moe_v3.py:34-37).
 * Selection is on the exactly-rounded fp32 logits; equal logits go to the lower
 * expert id.  d_weights[T,K] fp32 sum to 1, d_indices[T,K] int32 are ordered by
 * decreasing probability.  d_row_amax[T] (optional, may be null) receives
 * max|x[t,:]|.  Any E in [1,256], any K in [1,min(E,32)].  d_scratch is optional: with
 * bwmoe_router_scratch_bytes() bytes of it (non-zero for wide gates and large batches) the
 * logits are computed on the tensor cores and only the few experts near the cut are
 * re-evaluated exactly; the selection is the same either way.
 */
size_t bwmoe_router_scratch_bytes(int T, int D, int E, int K);
int bwmoe_router(const void* d_x, const void* d_w_gate, int T, int D, int E, int K,
                 float* d_weights, int32_t* d_indices, float* d_row_amax,
                 void* d_scratch, size_t scratch_bytes, void* stream);
/*
 * The same for T tokens that are a slice of a batch of T_as tokens routed elsewhere (expert parallelism: every
 * rank routes its own tokens).  The routing kernels - chosen by batch size - select the same experts always,
 * but their fp32 weights can differ in the last bits; with T_as the slice is routed by the kernel the whole
 * batch would get, so that its weights equal, bit for bit, those of the whole batch routed in one call.
 * No counterpart in the reference (single GPU).
 */
size_t bwmoe_router_scratch_bytes_as(int T, int D, int E, int K, int T_as);
int bwmoe_router_as(const void* d_x, const void* d_w_gate, int T, int D, int E, int K, int T_as,
                    float* d_weights, int32_t* d_indices, float* d_row_amax,
                    void* d_scratch, size_t scratch_bytes, void* stream);

/*
 * Whole block: router -> permute + segment-amax + E4M3 quant -> grouped gate+up
 * GEMM + SwiGLU -> segment requant -> grouped down GEMM -> weighted combine.
 * replaces: fp8_moe_forward, src/blackwell_moe/kernels/fp8_moe.py:111-164, and
 *           fp8_moe_forward_v3, src/blackwell_moe/kernels/fp8_moe_v3.py:19-74.
 * Requires D % 16 == 0, H % 16 == 0, E <= 256, K <= min(E,32).
 */
int bwmoe_moe_forward(const void* d_x, const void* d_w_gate,
                      const void* d_experts_w_gate, const void* d_experts_w_up,
                      const void* d_experts_w_down,
                      const float* d_scales_gate, const float* d_scales_up, const float* d_scales_down,
                      int T, int D, int H, int E, int K,
                      void* d_out, void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * bwmoe_moe_forward with options (flags = 0 is bwmoe_moe_forward).
 *   BWMOE_FLAG_REDUCE_COMBINE: the down projection's epilogue multiplies every finished row by its routing
 *   weight and ADDS it straight into out[token] with vector bf16 reductions - no result rows are written
 *   and no combine kernel runs.  This is how the reference combines (bf16 atomic adds in arrival order,
 *   src/blackwell_moe/kernels/scatter.py:25-72): the sum is rounded to bf16 after every addition and its
 *   order is not fixed, so two calls may differ in the last bit; within the 1e-2 bound, but not the
 *   bit-reproducible default (which multiplies in the epilogue too and sums the K rows of a token in a
 *   fixed order in a separate pass).  Batches of at most 64 rows ignore the flag.
 */
#define BWMOE_FLAG_REDUCE_COMBINE 1u
int bwmoe_moe_forward_flags(const void* d_x, const void* d_w_gate,
                            const void* d_experts_w_gate, const void* d_experts_w_up,
                            const void* d_experts_w_down,
                            const float* d_scales_gate, const float* d_scales_up, const float* d_scales_down,
                            int T, int D, int H, int E, int K,
                            void* d_out, void* d_workspace, size_t workspace_bytes, void* stream,
                            unsigned flags);

/*
 * bwmoe_moe_forward with the glue of the DeepSeek drop-in fused into the combine:
 *   out = bf16( bf16(routed * routed_scale) + residual )   (d_residual[T,D] bf16 may be null)
 * replaces: the tail of FP8MoELayer.forward, src/blackwell_moe/runtime/deepseek_patch.py:51-53.
 */
int bwmoe_moe_forward_ex(const void* d_x, const void* d_w_gate,
                         const void* d_experts_w_gate, const void* d_experts_w_up,
                         const void* d_experts_w_down,
                         const float* d_scales_gate, const float* d_scales_up, const float* d_scales_down,
                         int T, int D, int H, int E, int K, float routed_scale, const void* d_residual,
                         void* d_out, void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * The DeepSeek block in ONE pipeline: E routed experts (top-K) plus S always-on shared experts run as groups
 * E .. E+S-1 of the same permute / grouped-GEMM / combine kernels, every token being routed to them with
 * weight 1:   out = bf16( bf16(routed * routed_scale) + shared ).
 * The weight tensors hold E+S experts: d_experts_w_gate/up[E+S, D, H], d_experts_w_down[E+S, H, D],
 * d_scales_*[E+S].  A shared MLP of intermediate S*H (HF DeepseekV2MLP with n_shared_experts * H) is passed as
 * S column pieces of its gate/up matrices and S row pieces of its down matrix, each with the MLP's per-tensor
 * scale; the pieces then share one activation scale for x (all rows) and one for h (their maxima are merged),
 * as FP8SharedExpert quantises them.  d_w_gate is the router's [D, E].
 * Workspace: bwmoe_workspace_bytes_shared(T, D, H, E, K, S) (the layout of E+S experts and K+S slots per
 * token, with the router's scratch sized for the E routed experts); bwmoe_workspace_view with (E+S, K+S)
 * addresses its intermediates.
 * replaces: FP8MoELayer.forward, src/blackwell_moe/runtime/deepseek_patch.py:39-53, including the
 *           shared-expert call FP8SharedExpert.forward, src/blackwell_moe/runtime/shared_expert_fp8.py:57-68.
 */
size_t bwmoe_workspace_bytes_shared(int T, int D, int H, int E, int K, int S);
int bwmoe_moe_forward_shared(const void* d_x, const void* d_w_gate,
                             const void* d_experts_w_gate, const void* d_experts_w_up,
                             const void* d_experts_w_down,
                             const float* d_scales_gate, const float* d_scales_up, const float* d_scales_down,
                             int T, int D, int H, int E, int K, int S, float routed_scale,
                             void* d_out, void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * Dense (always-on) FP8 SwiGLU MLP over all T rows with whole-tensor scales for x and h:
 * the shared experts of a DeepSeek block.  Weights [D,H] / [H,D] e4m3, scales [1] fp32.
 * Workspace: bwmoe_workspace_bytes(T, D, H, 1, 1).
 * replaces: FP8SharedExpert.forward, src/blackwell_moe/runtime/shared_expert_fp8.py:57-68.
 */
int bwmoe_dense_mlp(const void* d_x, const void* d_w_gate, const void* d_w_up, const void* d_w_down,
                    const float* d_scale_gate, const float* d_scale_up, const float* d_scale_down,
                    int T, int D, int H, void* d_out, void* d_workspace, size_t workspace_bytes,
                    void* stream);

/*
 * Same block with the routing decided by the caller: d_weights[T,K] fp32 and
 * d_indices[T,K] int32 index the E expert slots of the weight tensors.
 * replaces: fp8_moe_forward_fastcache, src/blackwell_moe/kernels/fp8_moe_fastcache.py:16-55,
 *           and the pipeline half of streaming_moe_forward,
 *           src/blackwell_moe/runtime/streaming_moe.py:78-106.
 */
int bwmoe_moe_forward_routed(const void* d_x, const float* d_weights, const int32_t* d_indices,
                             const void* d_experts_w_gate, const void* d_experts_w_up,
                             const void* d_experts_w_down,
                             const float* d_scales_gate, const float* d_scales_up,
                             const float* d_scales_down,
                             int T, int D, int H, int E, int K,
                             void* d_out, void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * The routed form for an expert-residency cache: d_expert_ids[T,K] int32 are expert ids of the whole
 * model and d_remap[n_experts_total] int32 maps each id to its slot in the resident pool (the
 * [n_slots, ...] weight tensors), -1 for an expert that is not resident.  The lookup runs on the
 * device; a slot of -1 (or an id outside [0, n_experts_total)) is skipped and raises
 * BWMOE_STATUS_BAD_EXPERT.  Workspace: bwmoe_workspace_bytes(T, D, H, n_slots, K).
 * replaces: the `remap[expert_indices]` gather of fp8_moe_forward_fastcache,
 *           src/blackwell_moe/kernels/fp8_moe_fastcache.py:16-34, and the per-expert Python loop that
 *           builds slot ids in streaming_moe_forward, src/blackwell_moe/runtime/streaming_moe.py:61-76.
 */
int bwmoe_moe_forward_routed_remap(const void* d_x, const float* d_weights, const int32_t* d_expert_ids,
                                   const int32_t* d_remap, int n_experts_total,
                                   const void* d_slots_w_gate, const void* d_slots_w_up,
                                   const void* d_slots_w_down,
                                   const float* d_scales_gate, const float* d_scales_up,
                                   const float* d_scales_down,
                                   int T, int D, int H, int n_slots, int K,
                                   void* d_out, void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * bwmoe_moe_forward for callers that hold activations in host memory: copies
 * h_x[T,D] to the device (into the workspace), runs the block, copies the result
 * to h_out[T,D] and waits for it.  Weights stay device-resident.  The workspace
 * must hold bwmoe_workspace_bytes_host() bytes (the regular workspace plus device
 * copies of x and out).
 * replaces: the same call as bwmoe_moe_forward, as made by FP8MoELayer.forward,
 *           src/blackwell_moe/runtime/deepseek_patch.py:39-53, on host activations.
 */
int bwmoe_moe_forward_host(const void* h_x, const void* d_w_gate,
                           const void* d_experts_w_gate, const void* d_experts_w_up,
                           const void* d_experts_w_down,
                           const float* d_scales_gate, const float* d_scales_up,
                           const float* d_scales_down,
                           int T, int D, int H, int E, int K,
                           void* h_out, void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * The block with 128x128 block-scaled FP8 weights (HF `weight_scale_inv` convention:
 * w = code * inv, d_inv_*[E, ceil(in/128), ceil(out/128)] fp32, weights still [E,in,out]) and
 * per-token, per-128-element FP8 activations, multiplied in FP8 with the scales applied per
 * K block.  SwiGLU and the requantisation of h run in the gate/up epilogue: no 16-bit
 * intermediate is written.
 * replaces: the dequantise-to-bf16 + F.linear expert loop of StreamingQwenMoE.forward,
 *           src/blackwell_moe/runtime/qwen_patch.py:100-136 (weight semantics of
 *           _dequant_block_fp8, qwen_patch.py:30-40).
 */
size_t bwmoe_workspace_bytes_block(int T, int D, int H, int E, int K);
int bwmoe_workspace_view_block(void* d_workspace, int T, int D, int H, int E, int K, int which,
                               void** d_ptr, size_t* bytes);
int bwmoe_moe_forward_block(const void* d_x, const void* d_w_gate,
                            const void* d_experts_w_gate, const void* d_experts_w_up,
                            const void* d_experts_w_down,
                            const float* d_inv_gate, const float* d_inv_up, const float* d_inv_down,
                            int T, int D, int H, int E, int K,
                            void* d_out, void* d_workspace, size_t workspace_bytes, void* stream);

/*
 * bwmoe_moe_forward_block with the routing decided by the caller.  d_remap may be null (the ids then
 * index the n_slots weight slots directly); otherwise as in bwmoe_moe_forward_routed_remap.
 * Workspace: bwmoe_workspace_bytes_block(T, D, H, n_slots, K).
 * replaces: the per-expert loop of StreamingQwenMoE.forward over resident experts,
 *           src/blackwell_moe/runtime/qwen_patch.py:100-136.
 */
int bwmoe_moe_forward_block_routed(const void* d_x, const float* d_weights, const int32_t* d_expert_ids,
                                   const int32_t* d_remap, int n_experts_total,
                                   const void* d_slots_w_gate, const void* d_slots_w_up,
                                   const void* d_slots_w_down,
                                   const float* d_inv_gate, const float* d_inv_up, const float* d_inv_down,
                                   int T, int D, int H, int n_slots, int K,
                                   void* d_out, void* d_workspace, size_t workspace_bytes, void* stream);

/* Stages of the block-scale recipe (d_row_slot may be null: rows are then taken in order). */
int bwmoe_gather_quant_group(const void* d_x, const int32_t* d_row_slot, int M, int D, int K,
                             void* d_xq, float* d_x_inv, void* stream);
int bwmoe_gateup_swiglu_block(const void* d_xq, const float* d_x_inv, const int32_t* d_offsets,
                              const void* d_experts_w_gate, const void* d_experts_w_up,
                              const float* d_inv_gate, const float* d_inv_up,
                              int M, int D, int H, int E, void* d_hq, float* d_h_inv,
                              int32_t* d_status, void* stream);
int bwmoe_down_block(const void* d_hq, const float* d_h_inv, const int32_t* d_offsets,
                     const void* d_experts_w_down, const float* d_inv_down,
                     int M, int D, int H, int E, void* d_y, int32_t* d_status, void* stream);

/* ---- stage entry points (used by the expert-parallel host code and by tests) ---- */

/*
 * Plan the permutation: stable counting sort of the T*K slots by expert id.
 * replaces: the sort/bincount/cumsum of src/blackwell_moe/kernels/fp8_moe_v3.py:39-48
 *           (permute_tokens, src/blackwell_moe/kernels/permute.py:12-39).
 * Outputs: d_offsets[E+1], d_pos[M] (slot -> row), d_row_slot[M] (row -> slot),
 * d_row_expert[M], d_seg_amax[E] (max of d_row_amax over each segment; pass
 * d_row_amax = null to skip it).  d_scratch needs bwmoe_plan_scratch_bytes().
 */
size_t bwmoe_plan_scratch_bytes(int T, int E, int K);
int bwmoe_permute_plan(const int32_t* d_indices, const float* d_row_amax, int T, int E, int K,
                       int32_t* d_offsets, int32_t* d_pos, int32_t* d_row_slot,
                       int32_t* d_row_expert, float* d_seg_amax, int32_t* d_status,
                       void* d_scratch, void* stream);

/*
 * bwmoe_permute_plan without a scratch argument, for callers that have no way to
 * obtain device memory of their own at the point of the call: code running inside a
 * framework's allocator callback or out-of-memory handler, a plugin that was handed
 * only its input and output buffers, a real-time loop that has frozen its memory
 * pool.  (No counterpart in the reference, which allocates freely through torch.)
 * The scratch is a 64 KiB array built into the library image; every GPU that loads
 * the library holds it until the process exits.  Limits and rules:
 *   - T*K <= 262144 slots and E <= 256; larger requests fail with
 *     BWMOE_ERR_UNSUPPORTED and a message pointing to bwmoe_permute_plan.
 *   - inputs and outputs are still the caller's buffers, exactly as in
 *     bwmoe_permute_plan; results are identical to it.
 *   - the call allocates and frees nothing, on the host or the device.
 *   - the first call on each device looks up the array's device address (with that
 *     device current); make that first call outside any stream capture.
 *   - all calls on one GPU share the one array and it keeps whatever the last call
 *     left in it (nothing in it needs clearing between calls); two calls whose kernels
 *     can overlap on the GPU - different streams without an ordering between them -
 *     race on it.  Keep calls on one stream, or order them with events.
 */
int bwmoe_permute_plan_static(const int32_t* d_indices, const float* d_row_amax, int T, int E, int K,
                              int32_t* d_offsets, int32_t* d_pos, int32_t* d_row_slot,
                              int32_t* d_row_expert, float* d_seg_amax, int32_t* d_status,
                              void* stream);

/*
 * scale[e] = 448 / max(amax[e], bf16(1e-4)); 1.0 for an empty segment.
 * replaces: segment_fp8_scales, src/blackwell_moe/kernels/segment_ops.py:15-65
 *           (single-tensor form quant_fp8_e4m3, src/blackwell_moe/kernels/fp8_quant.py:24-32).
 */
int bwmoe_segment_scales(const float* d_seg_amax, const int32_t* d_offsets, int E, float* d_scales,
                         void* stream);

/*
 * Gather rows of x into expert-contiguous order and quantise them to E4M3 with
 * the per-segment scale: xq[m,:] = e4m3(clamp(x[row_slot[m]/K,:] * scale[row_expert[m]], +-448)).
 * replaces: x[inverse_idx] + segment_quant_fp8, src/blackwell_moe/kernels/fp8_moe_v3.py:44,51
 *           and src/blackwell_moe/kernels/segment_ops.py:68-120.
 */
int bwmoe_gather_quant(const void* d_x, const int32_t* d_row_slot, const int32_t* d_row_expert,
                       const float* d_scales, int M, int D, int K, void* d_xq, void* stream);

/*
 * Grouped gate+up FP8 GEMM with SwiGLU: h[m,:] = silu(gate) * up in bf16 with the
 * reference's bf16 rounding points, plus d_seg_amax_h[e] = max|h| per segment
 * (d_seg_amax_h must be zero on entry).  d_scratch needs bwmoe_gemm_scratch_bytes(M, D, H, E)
 * bytes (small batches split the K loop and sum fp32 partials from it in a fixed order).
 * replaces: fused_gate_up_gemm, src/blackwell_moe/kernels/grouped_fp8_gateup.py:42-138,
 *           and F.silu(gate)*up, src/blackwell_moe/kernels/fp8_moe_v3.py:60.
 */
size_t bwmoe_gemm_scratch_bytes(int M, int D, int H, int E);
int bwmoe_gateup_swiglu(const void* d_xq, const int32_t* d_offsets, const float* d_scales_x,
                        const void* d_experts_w_gate, const void* d_experts_w_up,
                        const float* d_scales_gate, const float* d_scales_up,
                        int M, int D, int H, int E,
                        void* d_h, float* d_seg_amax_h, int32_t* d_status, void* d_scratch,
                        void* stream);

/*
 * Per-segment requantisation of h to E4M3.
 * replaces: segment_fp8_scales + segment_quant_fp8 on h,
 *           src/blackwell_moe/kernels/fp8_moe_v3.py:61-62.
 */
int bwmoe_requant(const void* d_h, const int32_t* d_row_expert, const float* d_scales_h, int M, int H,
                  void* d_hq, void* stream);

/*
 * bwmoe_requant for callers that do not know the number of rows on the host: the rows are those of the
 * segments d_offsets[0 .. E] (row count d_offsets[E], read on the device), each quantised with its
 * segment's scale.  Used by the expert-parallel path, where the rows a rank receives are counted on the
 * device and the host never waits for the count.
 * replaces: segment_quant_fp8 on h, src/blackwell_moe/kernels/segment_ops.py:68-120 (whose launch grid
 *           needs the largest segment on the host, segment_ops.py:107).
 */
int bwmoe_requant_segments(const void* d_h, const int32_t* d_offsets, const float* d_scales_h, int E, int H,
                           void* d_hq, void* stream);

/*
 * Grouped down FP8 GEMM: y[m,:] = bf16(acc / (scale_h[e] * scale_down[e])).
 * replaces: grouped_fp8_gemm, src/blackwell_moe/kernels/grouped_fp8.py:36-128.
 */
int bwmoe_down(const void* d_hq, const int32_t* d_offsets, const float* d_scales_h,
               const void* d_experts_w_down, const float* d_scales_down,
               int M, int D, int H, int E,
               void* d_y, int32_t* d_status, void* d_scratch, void* stream);

/*
 * Weighted combine back to token order, deterministic:
 * out[t,:] = bf16( sum_k float( bf16( y[pos[t*K+k],:] * bf16(w[t,k]) ) ) ), k ascending.
 * replaces: flat_w multiply + scatter_add, src/blackwell_moe/kernels/fp8_moe_v3.py:70-73
 *           and src/blackwell_moe/kernels/scatter.py:25-72.
 */
int bwmoe_combine(const void* d_y, const int32_t* d_pos, const float* d_weights, int T, int D, int K,
                  void* d_out, void* stream);

/*
 * Expert-parallel transport over peer memory (one process per GPU, the buffers of every rank mapped
 * into each process; the host pointer arrays hold one device pointer per rank).  No counterpart in
 * the reference, which is single-GPU (the design notes under its docs/ directory name expert parallelism as
 * future work).
 *
 * bwmoe_scatter_quant_peers: quantise the token rows (as bwmoe_gather_quant does) and store the row of
 *   slot (t,k), routed to expert e, into row d_pos[t*K+k] + d_delta[e] of the receive buffer of rank
 *   e / experts_per_rank.  d_delta[e] = (first row of e's segment on its owner, plus the rows the lower
 *   ranks send to e) - (first row of e among the caller's permuted rows).
 * bwmoe_combine_peers: bwmoe_combine, reading the result row of slot (t,k) from the same place in the
 *   result buffer of the rank that owns its expert.
 * The caller orders the steps across ranks (a barrier before the stores, one after them, one before
 * the loads).  At most 8 ranks.  rows_cap is the row capacity of every rank's receive buffer: a row that
 * would land beyond it is dropped and BWMOE_STATUS_EP_OVERFLOW is raised in d_status (may be null).
 */
/*
 * Index maps of one expert-parallel step from the all-gathered row counts d_counts[n_ranks, E]
 * (d_counts[s*E+e] = rows rank s has for expert e) and the caller's own d_offsets[E+1]:
 * d_delta[E] (see bwmoe_scatter_quant_peers), d_offsets_local[E/n_ranks + 1] (segments of the experts
 * this rank owns), d_home_counts / d_home_first [n_ranks, E/n_ranks] (see bwmoe_down_peers).
 */
int bwmoe_ep_maps(const int32_t* d_counts, const int32_t* d_offsets, int n_ranks, int E, int rank,
                  int32_t* d_delta, int32_t* d_offsets_local, int32_t* d_home_counts, int32_t* d_home_first,
                  void* stream);
/*
 * bwmoe_down with the expert-parallel way back fused into its epilogue: segment e holds the rows that
 * ranks 0..n_ranks-1 sent (in that order, d_home_counts[s*E+e] from rank s); each finished row is stored
 * straight to row d_home_first[s*E+e] + i of rank s's result buffer h_y_of_rank[s], where a plain
 * bwmoe_combine over the home rank's own permutation picks it up.  One barrier between this call and
 * the combine.  No split-K in this form.
 */
int bwmoe_down_peers(const void* d_hq, const int32_t* d_offsets, const float* d_scales_h, const void* d_w_down,
                     const float* d_scales_down, int M, int D, int H, int E, const int32_t* d_home_counts,
                     const int32_t* d_home_first, void* const* h_y_of_rank, int n_ranks, int32_t* d_status,
                     void* stream);
/* The same for the block-scale recipe: the epilogue of bwmoe_down_block stores the rows at home. */
int bwmoe_down_block_peers(const void* d_hq, const float* d_h_inv, const int32_t* d_offsets, const void* d_w_down,
                           const float* d_inv_down, int M, int D, int H, int E, const int32_t* d_home_counts,
                           const int32_t* d_home_first, void* const* h_y_of_rank, int n_ranks, int32_t* d_status,
                           void* stream);
/*
 * Block-scale dispatch over peer memory: the codes d_xq_tok[T,D] and group scales d_inv_tok[T,ceil(D/128)]
 * of the tokens (token order, from bwmoe_gather_quant_group with no slot map) are stored to the place of
 * each of their K rows (d_pos[t*K+k] + d_delta[expert]) in the owner rank's code and scale buffers.
 */
int bwmoe_scatter_rows_group_peers(const void* d_xq_tok, const float* d_inv_tok, const int32_t* d_pos,
                                   const int32_t* d_indices, const int32_t* d_delta, int T, int D, int K,
                                   int experts_per_rank, void* const* h_xq_of_rank, void* const* h_inv_of_rank,
                                   int n_ranks, int rows_cap, int32_t* d_status, void* stream);
int bwmoe_scatter_quant_peers(const void* d_x, const int32_t* d_pos, const int32_t* d_indices,
                              const float* d_scales, const int32_t* d_delta, int T, int D, int K,
                              int experts_per_rank, void* const* h_dst_of_rank, int n_ranks, int rows_cap,
                              int32_t* d_status, void* stream);
int bwmoe_combine_peers(void* const* h_y_of_rank, int n_ranks, const int32_t* d_pos, const int32_t* d_indices,
                        const float* d_weights, const int32_t* d_delta, int experts_per_rank, int T, int D,
                        int K, void* d_out, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BWMOE_H_ */
