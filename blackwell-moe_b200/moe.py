"""Host-side mirror of the reference's MoE-block API on top of libbwmoe.so.

Signatures, argument meaning and error behaviour follow
``fp8_moe_forward`` (src/blackwell_moe/kernels/fp8_moe.py:111-121) and
``top_k_router`` (src/blackwell_moe/kernels/routing.py:61-66): pure functions
that return fresh tensors and never modify their inputs.  PyTorch is used for
device memory and streams only.
"""

from __future__ import annotations

import ctypes as C

import torch

from . import _lib

_FP8 = torch.float8_e4m3fn
_workspaces: dict = {}


def _require_cuda(*tensors):
    dev = None
    for t in tensors:
        if not t.is_cuda:
            raise ValueError("libbwmoe works on CUDA tensors only (there is no CPU path)")
        if dev is None:
            dev = t.device
        elif t.device != dev:
            raise ValueError(f"tensors on different devices: {t.device} vs {dev}")
    return dev


def _contig(t: torch.Tensor, name: str) -> torch.Tensor:
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")
    return t


def _stream(dev) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _workspace(dev, nbytes: int) -> torch.Tensor:
    """One grow-only workspace per (device, stream): calls on one stream are
    ordered, so they can share it; different streams get their own."""
    key = (dev.index, _stream(dev))
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        _workspaces[key] = ws
    return ws


def release_workspaces() -> None:
    _workspaces.clear()


def top_k_router(hidden: torch.Tensor, gate_w: torch.Tensor, k: int, *, as_batch: int = None):
    """Return ``(weights[T,k] fp32, indices[T,k] int32)``: softmax over all
    experts, top-k, renormalised; equal logits go to the lower expert id.

    ``as_batch``: route these tokens with the kernel a batch of that many tokens would get.  The kernels
    (picked by batch size) always select the same experts, but their fp32 weights may differ in the last
    bits; a caller that routes a slice of a larger batch passes the size of the whole batch and obtains
    exactly the weights the whole batch would get in one call."""
    assert hidden.dim() == 2 and gate_w.dim() == 2 and hidden.shape[1] == gate_w.shape[0], \
        (hidden.shape, gate_w.shape)
    assert hidden.dtype == torch.bfloat16 and gate_w.dtype == torch.bfloat16, (hidden.dtype, gate_w.dtype)
    dev = _require_cuda(hidden, gate_w)
    T, D = hidden.shape
    E = gate_w.shape[1]
    hidden, gate_w = _contig(hidden, "hidden"), _contig(gate_w, "gate_w")
    lib = _lib.lib()
    with torch.cuda.device(dev):
        w_out = torch.empty((T, k), device=dev, dtype=torch.float32)
        i_out = torch.empty((T, k), device=dev, dtype=torch.int32)
        t_as = int(as_batch) if as_batch else 0
        need = lib.bwmoe_router_scratch_bytes_as(T, D, E, k, t_as)
        scratch = torch.empty(need, dtype=torch.uint8, device=dev) if need else None
        _lib.check(lib.bwmoe_router_as(hidden.data_ptr(), gate_w.data_ptr(), T, D, E, k, t_as, w_out.data_ptr(),
                                       i_out.data_ptr(), None, scratch.data_ptr() if need else None, need,
                                       _stream(dev)))
    return w_out, i_out


def _check_experts(x, experts_w_gate, experts_w_up, experts_w_down, scales_gate, scales_up, scales_down):
    assert x.dim() == 2, x.shape
    T, D = x.shape
    assert experts_w_gate.dim() == 3 and experts_w_gate.shape[1] == D, (experts_w_gate.shape, D)
    E, _, H = experts_w_gate.shape
    assert tuple(experts_w_up.shape) == (E, D, H), experts_w_up.shape
    assert tuple(experts_w_down.shape) == (E, H, D), experts_w_down.shape
    block = scales_gate.dim() == 3
    if block:   # 128x128 block scales, HF `weight_scale_inv` convention, [E, ceil(in/128), ceil(out/128)]
        nd, nh = (D + 127) // 128, (H + 127) // 128
        assert tuple(scales_gate.shape) == (E, nd, nh) and tuple(scales_up.shape) == (E, nd, nh), scales_gate.shape
        assert tuple(scales_down.shape) == (E, nh, nd), scales_down.shape
    for s in (scales_gate, scales_up, scales_down):
        assert (block or s.numel() == E) and s.dtype == torch.float32, (s.shape, s.dtype)
    for w in (experts_w_gate, experts_w_up, experts_w_down):
        assert w.dtype == _FP8, w.dtype
    assert x.dtype == torch.bfloat16, x.dtype
    return T, D, H, E


def fp8_moe_forward(x, w_gate, experts_w_gate, experts_w_up, experts_w_down,
                    scales_gate, scales_up, scales_down, top_k: int = 8, *,
                    routed_scale: float = 1.0, residual=None, combine: str = "deterministic") -> torch.Tensor:
    """FP8 MoE-block forward: ``x[T,D] bf16 -> out[T,D] bf16``.

    ``scales_*`` of shape ``[E]`` select the reference's per-tensor recipe (forward
    multipliers ``448/amax``); of shape ``[E, ceil(in/128), ceil(out/128)]`` the
    128x128 block-scale recipe (inverse scales, as in HF ``weight_scale_inv``).

    ``x`` on the GPU: everything stays on the device and the result is a new
    CUDA tensor.  ``x`` in (pinned) host memory: the library copies it in,
    runs the block and copies the result back into a new pinned host tensor
    (weights must still be CUDA tensors).

    Keyword-only extras (per-tensor recipe, device activations): ``routed_scale`` and
    ``residual[T,D] bf16`` fuse the tail of the reference's DeepSeek layer into the combine,
    ``out = bf16(bf16(routed * routed_scale) + residual)``
    (src/blackwell_moe/runtime/deepseek_patch.py:51-53).  ``combine="atomic"`` lets the down projection's
    epilogue add the weighted rows straight into the output (bf16 reductions in arrival order, as the
    reference's scatter_add does, src/blackwell_moe/kernels/scatter.py:25-72): faster, within the same
    1e-2 bound, but not bit-reproducible; the default sums a token's K rows in a fixed order."""
    if combine not in ("deterministic", "atomic"):
        raise ValueError(f"combine={combine!r}: expected 'deterministic' or 'atomic'")
    T, D, H, E = _check_experts(x, experts_w_gate, experts_w_up, experts_w_down,
                                scales_gate, scales_up, scales_down)
    assert w_gate.shape == (D, E) and w_gate.dtype == torch.bfloat16, (w_gate.shape, w_gate.dtype)
    weights = [_contig(t, "weight tensor") for t in (w_gate, experts_w_gate, experts_w_up, experts_w_down,
                                                     scales_gate, scales_up, scales_down)]
    dev = _require_cuda(*weights)
    lib = _lib.lib()
    x = _contig(x, "x")
    with torch.cuda.device(dev):
        ptrs = [t.data_ptr() for t in weights]
        if routed_scale != 1.0 or residual is not None:
            if scales_gate.dim() == 3 or not x.is_cuda:
                raise ValueError("routed_scale / residual are available for the per-tensor recipe on device activations")
        if scales_gate.dim() == 3:
            host_x = not x.is_cuda
            if host_x:      # host activations: copy in, run, copy out and wait (pinned memory makes the copies async)
                x = x.to(dev, non_blocking=True)
            _require_cuda(x, w_gate)
            need = lib.bwmoe_workspace_bytes_block(T, D, H, E, top_k)
            if need == 0:
                raise ValueError(f"unsupported shape T={T} D={D} H={H} E={E} top_k={top_k}")
            ws = _workspace(dev, need)
            out = torch.empty_like(x)
            _lib.check(lib.bwmoe_moe_forward_block(x.data_ptr(), *ptrs, T, D, H, E, top_k, out.data_ptr(),
                                                   ws.data_ptr(), ws.numel(), _stream(dev)))
            if host_x:
                host = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
                host.copy_(out, non_blocking=True)
                torch.cuda.current_stream(dev).synchronize()
                return host
            return out
        if x.is_cuda:
            _require_cuda(x, w_gate)
            need = lib.bwmoe_workspace_bytes(T, D, H, E, top_k)
            if need == 0:
                raise ValueError(f"unsupported shape T={T} D={D} H={H} E={E} top_k={top_k} "
                                 "(D and H must be multiples of 16, E <= 256, top_k <= min(E, 32))")
            ws = _workspace(dev, need)
            out = torch.empty_like(x)
            if routed_scale != 1.0 or residual is not None:
                if residual is not None:
                    assert residual.shape == x.shape and residual.dtype == torch.bfloat16, (residual.shape, residual.dtype)
                    residual = _contig(residual, "residual")
                    _require_cuda(x, residual)
                _lib.check(lib.bwmoe_moe_forward_ex(x.data_ptr(), *ptrs, T, D, H, E, top_k, float(routed_scale),
                                                    residual.data_ptr() if residual is not None else None,
                                                    out.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev)))
                return out
            if combine == "atomic":
                _lib.check(lib.bwmoe_moe_forward_flags(x.data_ptr(), *ptrs, T, D, H, E, top_k, out.data_ptr(),
                                                       ws.data_ptr(), ws.numel(), _stream(dev), 1))
                return out
            _lib.check(lib.bwmoe_moe_forward(x.data_ptr(), *ptrs, T, D, H, E, top_k, out.data_ptr(),
                                             ws.data_ptr(), ws.numel(), _stream(dev)))
            return out
        need = lib.bwmoe_workspace_bytes_host(T, D, H, E, top_k)
        if need == 0:
            raise ValueError(f"unsupported shape T={T} D={D} H={H} E={E} top_k={top_k}")
        ws = _workspace(dev, need)
        out = torch.empty(x.shape, dtype=x.dtype, pin_memory=True)
        _lib.check(lib.bwmoe_moe_forward_host(x.data_ptr(), *ptrs, T, D, H, E, top_k, out.data_ptr(),
                                              ws.data_ptr(), ws.numel(), _stream(dev)))
        return out


def fp8_moe_forward_shared(x, w_gate, experts_w_gate, experts_w_up, experts_w_down, scales_gate, scales_up, scales_down,
                           top_k: int, n_shared: int, routed_scale: float = 1.0) -> torch.Tensor:
    """The DeepSeek block in one pipeline: ``E`` routed experts (top-k of the router ``w_gate[D,E]``) plus
    ``n_shared`` always-on experts that are the last ``n_shared`` entries of the stacked weight tensors
    (``[E + n_shared, ...]``); ``out = bf16(bf16(routed * routed_scale) + shared)``.  Takes over
    ``FP8MoELayer.forward`` (src/blackwell_moe/runtime/deepseek_patch.py:39-53) including its shared-expert call
    (src/blackwell_moe/runtime/shared_expert_fp8.py:57-68); :func:`stack_shared_experts` prepares the tensors."""
    T, D, H, EA = _check_experts(x, experts_w_gate, experts_w_up, experts_w_down, scales_gate, scales_up, scales_down)
    E = EA - n_shared
    assert n_shared >= 1 and E >= top_k >= 1, (EA, n_shared, top_k)
    assert scales_gate.dim() == 1, "the shared-expert pipeline exists for the per-tensor recipe"
    assert w_gate.shape == (D, E) and w_gate.dtype == torch.bfloat16, (w_gate.shape, w_gate.dtype)
    tensors = [_contig(t, "tensor") for t in (x, w_gate, experts_w_gate, experts_w_up, experts_w_down,
                                              scales_gate, scales_up, scales_down)]
    dev = _require_cuda(*tensors)
    lib = _lib.lib()
    with torch.cuda.device(dev):
        need = lib.bwmoe_workspace_bytes_shared(T, D, H, E, top_k, n_shared)
        if need == 0:
            raise ValueError(f"unsupported shape T={T} D={D} H={H} E={E}+{n_shared} top_k={top_k}+{n_shared}")
        ws = _workspace(dev, need)
        out = torch.empty_like(x)
        _lib.check(lib.bwmoe_moe_forward_shared(*[t.data_ptr() for t in tensors], T, D, H, E, top_k, n_shared,
                                                float(routed_scale), out.data_ptr(), ws.data_ptr(), ws.numel(),
                                                _stream(dev)))
    return out


def stack_shared_experts(experts_w_gate, experts_w_up, experts_w_down, scales_gate, scales_up, scales_down,
                         shared_w_gate, shared_w_up, shared_w_down, shared_s_gate, shared_s_up, shared_s_down):
    """Append a shared MLP (``[D, S*H]`` gate/up, ``[S*H, D]`` down, per-tensor scales) to stacked routed experts
    as ``S`` more experts of intermediate ``H``: column pieces of gate/up, row pieces of down, each with the
    MLP's scale.  Returns the six ``[E+S, ...]`` tensors and ``S`` (load time, plain torch)."""
    E, D, H = experts_w_gate.shape
    Hs = shared_w_gate.shape[1]
    assert tuple(shared_w_gate.shape) == (D, Hs) and tuple(shared_w_down.shape) == (Hs, D) and Hs % H == 0, \
        (shared_w_gate.shape, shared_w_down.shape, H)
    S = Hs // H
    u8 = torch.uint8

    def cat(a, b):                      # float8 tensors are concatenated through their byte view
        return torch.cat([a.contiguous().view(u8), b.contiguous().view(u8)]).view(_FP8).contiguous()
    gate = cat(experts_w_gate, shared_w_gate.view(u8).view(D, S, H).permute(1, 0, 2))
    up = cat(experts_w_up, shared_w_up.view(u8).view(D, S, H).permute(1, 0, 2))
    down = cat(experts_w_down, shared_w_down.view(u8).view(S, H, D))
    f32 = torch.float32
    scales = [torch.cat([r.to(f32).reshape(-1), s.to(f32).reshape(1).expand(S)]).contiguous()
              for r, s in ((scales_gate, shared_s_gate), (scales_up, shared_s_up), (scales_down, shared_s_down))]
    return gate, up, down, scales[0], scales[1], scales[2], S


def fp8_moe_forward_routed(x, router_weights, expert_indices, experts_w_gate, experts_w_up, experts_w_down,
                           scales_gate, scales_up, scales_down, remap=None) -> torch.Tensor:
    """Same block with caller-supplied routing (``router_weights[T,K] fp32``,
    ``expert_indices[T,K] int32``) - the entry point an expert-residency cache uses
    (src/blackwell_moe/kernels/fp8_moe_fastcache.py:16-55).

    Without ``remap`` the indices address the E weight slots directly.  With
    ``remap[E_total] int32`` they are expert ids of the whole model and
    ``remap[id]`` is the slot that holds the expert (``-1``: not resident); the
    lookup runs on the device.  3-D ``scales_*`` select the block-scale recipe."""
    T, D, H, E = _check_experts(x, experts_w_gate, experts_w_up, experts_w_down,
                                scales_gate, scales_up, scales_down)
    assert router_weights.shape == expert_indices.shape and router_weights.shape[0] == T
    K = router_weights.shape[1]
    block = scales_gate.dim() == 3
    tensors = [_contig(t, "tensor") for t in (x, router_weights.to(torch.float32), expert_indices.to(torch.int32),
                                              experts_w_gate, experts_w_up, experts_w_down,
                                              scales_gate, scales_up, scales_down)]
    dev = _require_cuda(*tensors)
    n_total = 0
    if remap is not None:
        remap = _contig(remap.to(torch.int32), "remap")
        _require_cuda(x, remap)
        n_total = remap.numel()
    lib = _lib.lib()
    with torch.cuda.device(dev):
        need = (lib.bwmoe_workspace_bytes_block if block else lib.bwmoe_workspace_bytes)(T, D, H, E, K)
        if need == 0:
            raise ValueError(f"unsupported shape T={T} D={D} H={H} E={E} top_k={K}")
        ws = _workspace(dev, need)
        out = torch.empty_like(x)
        p = [t.data_ptr() for t in tensors]
        tail = (T, D, H, E, K, out.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev))
        if block:
            _lib.check(lib.bwmoe_moe_forward_block_routed(p[0], p[1], p[2], remap.data_ptr() if remap is not None else None,
                                                          n_total, *p[3:], *tail))
        elif remap is not None:
            _lib.check(lib.bwmoe_moe_forward_routed_remap(p[0], p[1], p[2], remap.data_ptr(), n_total, *p[3:], *tail))
        else:
            _lib.check(lib.bwmoe_moe_forward_routed(*p, *tail))
    return out


def fp8_moe_forward_fastcache(x, router_weights, expert_indices, remap, cache_g, cache_u, cache_d,
                              cache_sg, cache_su, cache_sd, n_slots: int, top_k: int = 8) -> torch.Tensor:
    """Signature of the reference's ``fp8_moe_forward_fastcache``
    (src/blackwell_moe/kernels/fp8_moe_fastcache.py:16-29): original expert ids plus the
    cache's ``remap`` tensor, experts taken from the ``[n_slots, ...]`` pool tensors."""
    assert cache_g.shape[0] == n_slots and expert_indices.shape[1] == top_k, (cache_g.shape, n_slots, top_k)
    return fp8_moe_forward_routed(x, router_weights, expert_indices, cache_g, cache_u, cache_d,
                                  cache_sg, cache_su, cache_sd, remap=remap)


def streaming_moe_forward(x, w_gate, cache, layer_idx: int, top_k: int, prefetch_next_layer=None) -> torch.Tensor:
    """MoE-block forward over an expert-residency cache, with the call protocol of the reference's
    ``streaming_moe_forward`` (src/blackwell_moe/runtime/streaming_moe.py:32-107).  ``cache`` is any
    object with the interface of ``ThreeTierExpertCache``
    (src/blackwell_moe/runtime/disk_expert_pool.py:89-268): ``gpu`` (dict of ``[gpu_slots, ...]``
    pool tensors ``gate_q/up_q/down_q/scale_g/scale_u/scale_d``), ``gpu_slots``, ``n_experts``,
    ``fetch(layer_idx, expert_ids) -> slot tensor`` and ``prefetch_layer``; the cache itself stays
    host-side code and is not part of this package.

    The router, the id -> slot lookup and the whole pipeline run in the library; what remains on the
    host is what the cache's interface demands: the list of distinct expert ids of the batch."""
    if prefetch_next_layer is not None:
        cache.prefetch_layer(prefetch_next_layer)
    weights, indices = top_k_router(x, w_gate, top_k)
    unique_eids = torch.unique(indices.flatten())
    slots = cache.fetch(layer_idx, unique_eids.tolist())
    n_total = max(int(w_gate.shape[1]), int(getattr(cache, "n_experts", 0)))
    remap = torch.full((n_total,), -1, dtype=torch.int32, device=x.device)
    remap[unique_eids.long()] = slots.to(device=x.device, dtype=torch.int32)
    gpu = cache.gpu
    return fp8_moe_forward_routed(x, weights, indices, gpu["gate_q"], gpu["up_q"], gpu["down_q"],
                                  gpu["scale_g"], gpu["scale_u"], gpu["scale_d"], remap=remap)


_VIEWS = {
    "status": (0, torch.int32), "offsets": (1, torch.int32), "indices": (2, torch.int32),
    "weights": (3, torch.float32), "pos": (4, torch.int32), "row_slot": (5, torch.int32),
    "scale_x": (6, torch.float32), "scale_h": (7, torch.float32), "xq": (8, torch.uint8),
    "hq": (9, torch.uint8), "h": (10, torch.bfloat16), "y": (11, torch.bfloat16),
    "row_expert": (12, torch.int32),
}


_BLOCK_ONLY = {"x_inv": (13, torch.float32), "h_inv": (14, torch.float32)}
_TENSOR_ONLY = ("scale_x", "scale_h", "h")


def moe_stage_views(dev, T: int, D: int, H: int, E: int, K: int, block: bool = False) -> dict:
    """Copies of the intermediates the last forward of this shape on the current
    stream left in its workspace (routing, permutation, FP8 codes, scales) and
    the device status word.  For stage-level checks; synchronises."""
    dev = torch.device(dev)
    lib = _lib.lib()
    ws = _workspaces[(dev.index, _stream(dev))]
    out = {}
    torch.cuda.synchronize(dev)
    views = dict(_VIEWS)
    fn = lib.bwmoe_workspace_view
    if block:
        for k in _TENSOR_ONLY:
            views.pop(k)
        views.update(_BLOCK_ONLY)
        fn = lib.bwmoe_workspace_view_block
    for name, (sel, dtype) in views.items():
        ptr, nbytes = C.c_void_p(), C.c_size_t()
        _lib.check(fn(ws.data_ptr(), T, D, H, E, K, sel, C.byref(ptr), C.byref(nbytes)))
        off = ptr.value - ws.data_ptr()
        out[name] = ws[off:off + nbytes.value].clone().view(dtype)
    M = T * K
    out["indices"] = out["indices"].view(T, K)
    out["weights"] = out["weights"].view(T, K)
    out["xq"] = out["xq"].view(M, D).view(_FP8)
    out["hq"] = out["hq"].view(M, H).view(_FP8)
    out["y"] = out["y"].view(M, D)
    if block:
        out["x_inv"] = out["x_inv"].view(M, -1)
        out["h_inv"] = out["h_inv"].view(M, -1)
    else:
        out["h"] = out["h"].view(M, H)
    return out


class HostPipeline:
    """MoE-block forward for callers whose activations live in (pinned) host memory, with the
    host->device copy of batch i+1 and the device->host copy of batch i-1 overlapping the
    compute of batch i (three CUDA streams, ``depth`` slots of device buffers).  Numerically it
    is :func:`fp8_moe_forward` on every batch; only the scheduling differs.

        pipe = HostPipeline(w_gate, wg, wu, wd, sg, su, sd, top_k=2, max_tokens=16384)
        t0 = pipe.submit(x0)          # returns at once
        t1 = pipe.submit(x1)
        y0 = pipe.result(t0)          # pinned host tensor, valid until its slot is reused
    """

    def __init__(self, w_gate, experts_w_gate, experts_w_up, experts_w_down, scales_gate, scales_up, scales_down,
                 top_k: int, max_tokens: int, depth: int = 2):
        self.weights = [_contig(t, "weight tensor") for t in (w_gate, experts_w_gate, experts_w_up, experts_w_down,
                                                             scales_gate, scales_up, scales_down)]
        self.dev = _require_cuda(*self.weights)
        self.block = scales_gate.dim() == 3
        self.K, self.Tmax, self.depth = top_k, max_tokens, depth
        self.E, self.D, self.H = experts_w_gate.shape
        lib = _lib.lib()
        size_fn = lib.bwmoe_workspace_bytes_block if self.block else lib.bwmoe_workspace_bytes
        need = size_fn(max_tokens, self.D, self.H, self.E, top_k)
        if need == 0:
            raise ValueError("unsupported shape")
        with torch.cuda.device(self.dev):
            self.s_in, self.s_cmp, self.s_out = (torch.cuda.Stream(self.dev) for _ in range(3))
            self.slots = []
            for _ in range(depth):
                self.slots.append(dict(
                    x=torch.empty(max_tokens, self.D, dtype=torch.bfloat16, device=self.dev),
                    y=torch.empty(max_tokens, self.D, dtype=torch.bfloat16, device=self.dev),
                    ws=torch.empty(need, dtype=torch.uint8, device=self.dev),
                    host=torch.empty(max_tokens, self.D, dtype=torch.bfloat16, pin_memory=True),
                    in_done=torch.cuda.Event(), cmp_done=torch.cuda.Event(), out_done=torch.cuda.Event(), T=0))
        self.ticket = 0

    def submit(self, x_host: torch.Tensor) -> int:
        assert not x_host.is_cuda and x_host.dtype == torch.bfloat16 and x_host.shape[1] == self.D
        T = x_host.shape[0]
        assert 0 < T <= self.Tmax
        lib = _lib.lib()
        slot = self.slots[self.ticket % self.depth]
        first_use = self.ticket < self.depth
        with torch.cuda.device(self.dev):
            if not first_use:
                self.s_in.wait_event(slot["cmp_done"])        # the previous batch in this slot has been consumed
            with torch.cuda.stream(self.s_in):
                slot["x"][:T].copy_(x_host, non_blocking=True)
                slot["in_done"].record(self.s_in)
            self.s_cmp.wait_event(slot["in_done"])
            if not first_use:
                self.s_cmp.wait_event(slot["out_done"])       # its previous result has left the device
            fn = lib.bwmoe_moe_forward_block if self.block else lib.bwmoe_moe_forward
            _lib.check(fn(slot["x"].data_ptr(), *[t.data_ptr() for t in self.weights], T, self.D, self.H, self.E,
                          self.K, slot["y"].data_ptr(), slot["ws"].data_ptr(), slot["ws"].numel(),
                          self.s_cmp.cuda_stream))
            slot["cmp_done"].record(self.s_cmp)
            self.s_out.wait_event(slot["cmp_done"])
            with torch.cuda.stream(self.s_out):
                slot["host"][:T].copy_(slot["y"][:T], non_blocking=True)
                slot["out_done"].record(self.s_out)
        slot["T"] = T
        self.ticket += 1
        return self.ticket - 1

    def result(self, ticket: int) -> torch.Tensor:
        assert self.ticket - self.depth <= ticket < self.ticket, "result no longer (or not yet) available"
        slot = self.slots[ticket % self.depth]
        slot["out_done"].synchronize()
        return slot["host"][:slot["T"]]

    def drain(self) -> None:
        for slot in self.slots:
            slot["out_done"].synchronize()
