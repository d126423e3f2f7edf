"""CPU restatement of the reference's per-tensor FP8 MoE-block forward.

TEST INFRASTRUCTURE ONLY (see the package docstring).  All tensors are CPU
torch tensors.  Each function names the reference lines it follows (paths are
relative to the reference project's root).
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

FP8_MAX = 448.0  # src/blackwell_moe/kernels/fp8_quant.py:21


# --------------------------------------------------------------------------
# quantisation (src/blackwell_moe/kernels/fp8_quant.py:24-36; the same
# arithmetic is what the segment kernels compute per expert segment,
# src/blackwell_moe/kernels/segment_ops.py:15-44,68-93)
# --------------------------------------------------------------------------
def quant_fp8_e4m3(x: torch.Tensor):
    """``scale = 448 / max(amax, 1e-4)``; ``q = e4m3(clamp(x * scale, +-448))``.

    Returns ``(q, scale)`` with ``scale`` a 0-d fp32 tensor (a forward
    multiplier: dequantisation divides by it).
    """
    amax = x.abs().amax().clamp(min=1e-4).to(torch.float32)
    scale = (FP8_MAX / amax).to(torch.float32)
    q = (x.to(torch.float32) * scale).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, scale


def dequant_fp8_e4m3(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return (q.to(torch.float32) / scale).to(torch.bfloat16)


# --------------------------------------------------------------------------
# routing
# --------------------------------------------------------------------------
def router_literal(hidden: torch.Tensor, gate_w: torch.Tensor, k: int):
    """Literal restatement of ``top_k_router_ref``
    (src/blackwell_moe/kernels/routing.py:82-90): fp32 matmul, softmax,
    ``torch.topk``, renormalise.  Tie order and near-tie order follow the
    library's fp32 summation order, so this is *not* a unique target."""
    logits = hidden.to(torch.float32) @ gate_w.to(torch.float32)
    probs = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, k=k, dim=-1)
    w = w / w.sum(dim=-1, keepdim=True)
    return w, idx.to(torch.int32)


def canonical_logits(hidden: torch.Tensor, gate_w: torch.Tensor) -> torch.Tensor:
    """The exact dot products rounded once to fp32.

    bf16 x bf16 products are exact in fp32; the only freedom the reference's
    fp32 matmul (routing.py:86) has is the summation order.  Summing in fp64
    and rounding once removes that freedom and gives every implementation
    the same target."""
    return (hidden.to(torch.float64) @ gate_w.to(torch.float64)).to(torch.float32)


def router_canonical(hidden: torch.Tensor, gate_w: torch.Tensor, k: int):
    """Canonical router: same maths as ``top_k_router_ref`` (routing.py:82-90)
    evaluated on :func:`canonical_logits`, with the selection done by a stable
    descending sort so that equal logits go to the lower expert id.

    Returns ``(weights[T,k] fp32, indices[T,k] int32)`` ordered by decreasing
    probability."""
    logits = canonical_logits(hidden, gate_w)
    order = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, :k]
    probs = torch.softmax(logits, dim=-1)
    w = torch.gather(probs, 1, order)
    w = w / w.sum(dim=-1, keepdim=True)
    return w, order.to(torch.int32)


# --------------------------------------------------------------------------
# permutation (src/blackwell_moe/kernels/fp8_moe_v3.py:39-48, same as
# src/blackwell_moe/kernels/permute.py:12-39)
# --------------------------------------------------------------------------
def permutation(indices: torch.Tensor, num_experts: int):
    """Stable sort of the flattened ``[T,K]`` slots by expert id.

    Returns ``(sort_perm[M] int64, inverse_idx[M] int64, offsets[E+1] int32)``:
    permuted row ``m`` holds slot ``sort_perm[m]`` whose token is
    ``inverse_idx[m]``; expert ``e`` owns rows ``offsets[e]:offsets[e+1]``."""
    T, K = indices.shape
    flat = indices.reshape(-1).to(torch.int32)
    sorted_ids, sort_perm = torch.sort(flat, stable=True)
    src = torch.arange(T * K, dtype=torch.long) // K
    inverse_idx = src[sort_perm]
    counts = torch.bincount(sorted_ids.to(torch.long), minlength=num_experts)
    offsets = torch.zeros(num_experts + 1, dtype=torch.int32)
    offsets[1:] = counts.cumsum(0).to(torch.int32)
    return sort_perm, inverse_idx, offsets


# --------------------------------------------------------------------------
# bf16 reference forward (src/blackwell_moe/kernels/reference.py:9-39)
# --------------------------------------------------------------------------
def moe_forward_bf16(x, w_gate, experts_w_gate, experts_w_up, experts_w_down, top_k=8,
                     routing=None):
    """bf16 eager MoE forward.  ``routing=(weights, indices)`` overrides the
    literal fp32-matmul/topk routing (used to feed the canonical routing)."""
    if routing is None:
        logits = x.to(torch.float32) @ w_gate.to(torch.float32)
        probs = F.softmax(logits, dim=-1)
        w, idx = torch.topk(probs, k=top_k, dim=-1)
        w = (w / w.sum(dim=-1, keepdim=True)).to(x.dtype)
    else:
        w, idx = routing
        w = w.to(x.dtype)
        idx = idx.to(torch.long)
    out = torch.zeros_like(x)
    E = experts_w_gate.shape[0]
    for e in range(E):
        mask = (idx == e).any(dim=-1)
        if not mask.any():
            continue
        tok = mask.nonzero(as_tuple=True)[0]
        x_e = x[tok]
        gate = x_e @ experts_w_gate[e]
        up = x_e @ experts_w_up[e]
        h = F.silu(gate) * up
        y = h @ experts_w_down[e]
        w_slot = (idx[tok] == e).to(x.dtype)
        w_e = (w[tok] * w_slot).sum(dim=-1, keepdim=True)
        out.index_add_(0, tok, y * w_e)
    return out


# --------------------------------------------------------------------------
# FP8 recipe forward = data flow of fp8_moe_forward_v3
# (src/blackwell_moe/kernels/fp8_moe_v3.py:51-73) with the segment kernels
# replaced by their single-tensor definition (fp8_quant.py:24-32) and the
# grouped GEMMs by an fp32 matmul of the FP8 codes followed by the same
# ``acc / (sx * sw)`` -> bf16 epilogue (grouped_fp8.py:83-88,
# grouped_fp8_gateup.py:91-101).
# --------------------------------------------------------------------------
def moe_forward_fp8_recipe(x, w_gate, wq_gate, wq_up, wq_down, s_gate, s_up, s_down,
                           top_k=8, routing=None, intermediates=None, experts=None):
    """Per-expert-segment FP8 recipe.  ``intermediates`` (a dict) receives the
    permutation, FP8 codes and scales for stage-level parity checks.

    ``experts`` (an iterable of expert ids) restricts the per-expert work to those
    segments, for shapes whose full forward is too slow on CPU: routing and
    permutation are still computed for every row, the rows of the other segments
    stay zero, and the weight tensors may then be dicts ``{expert id: tensor}``
    holding the chosen experts only (the ``[E]`` scale tensors stay whole)."""
    T, D = x.shape
    if isinstance(wq_gate, dict):
        E, H = int(s_gate.shape[0]), next(iter(wq_gate.values())).shape[1]
    else:
        E, _, H = wq_gate.shape
    if routing is None:
        routing = router_canonical(x, w_gate, top_k)
    weights, indices = routing
    sort_perm, inverse_idx, offsets = permutation(indices, E)
    M = sort_perm.numel()
    x_perm = x[inverse_idx]

    xq_all = torch.zeros(M, D, dtype=torch.float8_e4m3fn)
    hq_all = torch.zeros(M, H, dtype=torch.float8_e4m3fn)
    h_all = torch.zeros(M, H, dtype=torch.bfloat16)
    y_perm = torch.zeros(M, D, dtype=torch.bfloat16)
    sx_all = torch.ones(E, dtype=torch.float32)   # empty segment -> 1.0 (segment_ops.py:27-29)
    sh_all = torch.ones(E, dtype=torch.float32)
    for e in (range(E) if experts is None else experts):
        s, t = int(offsets[e]), int(offsets[e + 1])
        if t <= s:
            continue
        xq, sx = quant_fp8_e4m3(x_perm[s:t])
        xf = xq.to(torch.float32)
        gate = ((xf @ wq_gate[e].to(torch.float32)) / (sx * s_gate[e])).to(torch.bfloat16)
        up = ((xf @ wq_up[e].to(torch.float32)) / (sx * s_up[e])).to(torch.bfloat16)
        h = F.silu(gate) * up                                   # bf16, fp8_moe_v3.py:60
        hq, sh = quant_fp8_e4m3(h)
        y = ((hq.to(torch.float32) @ wq_down[e].to(torch.float32)) / (sh * s_down[e])).to(torch.bfloat16)
        xq_all[s:t], hq_all[s:t], h_all[s:t], y_perm[s:t] = xq, hq, h, y
        sx_all[e], sh_all[e] = sx, sh

    flat_w = weights.reshape(-1)[sort_perm].to(torch.bfloat16).unsqueeze(-1)  # v3:70
    weighted = (y_perm * flat_w).to(torch.bfloat16)
    out = torch.zeros(T, D, dtype=torch.bfloat16)
    out.index_add_(0, inverse_idx, weighted)                                   # scatter_add, v3:72-73
    if intermediates is not None:
        intermediates.update(weights=weights, indices=indices, sort_perm=sort_perm,
                             inverse_idx=inverse_idx, offsets=offsets, xq=xq_all, sx=sx_all,
                             h=h_all, hq=hq_all, sh=sh_all, y_perm=y_perm, weighted=weighted)
    return out


# --------------------------------------------------------------------------
# shared experts (src/blackwell_moe/runtime/shared_expert_fp8.py:57-68):
# dense FP8 SwiGLU over all T rows, whole-tensor scales for x and h.
# Weights are passed in the [in, out] orientation used by the routed experts.
# --------------------------------------------------------------------------
def shared_expert_fp8(x, wq_gate, wq_up, wq_down, s_gate, s_up, s_down):
    xq, sx = quant_fp8_e4m3(x)
    xf = xq.to(torch.float32)
    gate = ((xf @ wq_gate.to(torch.float32)) / (sx * s_gate)).to(torch.bfloat16)
    up = ((xf @ wq_up.to(torch.float32)) / (sx * s_up)).to(torch.bfloat16)
    h = F.silu(gate) * up
    hq, sh = quant_fp8_e4m3(h)
    return ((hq.to(torch.float32) @ wq_down.to(torch.float32)) / (sh * s_down)).to(torch.bfloat16)


def rel_l1(a: torch.Tensor, b: torch.Tensor) -> float:
    """mean|a-b| / mean|b| in fp64 (the metric of scripts/verify_v3.py:31-34)."""
    a64, b64 = a.to(torch.float64), b.to(torch.float64)
    return float((a64 - b64).abs().mean() / b64.abs().mean().clamp(min=1e-30))
