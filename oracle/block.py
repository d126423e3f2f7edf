"""CPU restatement of the 128x128 block-scale FP8 recipe.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED for the FP8 arithmetic: the reference never multiplies
block-scaled FP8 operands.  Its Qwen path dequantises the weights to bf16
(src/blackwell_moe/runtime/qwen_patch.py:30-40) and runs ``F.linear`` per
expert (qwen_patch.py:108-129).  What *is* pinned by fixtures: the
weight-scale semantics (``dequant_block_128`` must reproduce the reference's
``_dequant_block_fp8`` bit for bit) and the block's output
(``streaming_qwen_forward`` restates the reference's StreamingQwenMoE.forward
and is checked against an output of that very method; the FP8 recipe must stay
within the reference's stated ~7 % of it).  The rest of this file is our own
definition of the recipe: weights carry one multiplicative inverse scale per
128x128 block, activations one per token per 128 consecutive K elements, and
the bf16 rounding points are those of the per-tensor recipe
(src/blackwell_moe/kernels/fp8_moe_v3.py:54-73).

Weight orientation: ``[in, out]`` per expert as everywhere else in the hot
path (src/blackwell_moe/kernels/fp8_moe.py:114-116); block scales are
``[ceil(in/128), ceil(out/128)]``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .recipe import FP8_MAX, permutation, router_canonical

BLOCK = 128


def _expand(scale: torch.Tensor, rows: int, cols: int) -> torch.Tensor:
    s = scale.repeat_interleave(BLOCK, dim=0)[:rows]
    return s.repeat_interleave(BLOCK, dim=1)[:, :cols]


def quant_block_128(w: torch.Tensor):
    """Inverse of ``_dequant_block_fp8``: per 128x128 block
    ``scale_inv = max(amax, 1e-4) / 448``; ``q = e4m3(clamp(w / scale_inv))``.
    Returns ``(q[in,out] e4m3, scale_inv[ceil(in/128), ceil(out/128)] fp32)``."""
    R, C = w.shape
    rb, cb = (R + BLOCK - 1) // BLOCK, (C + BLOCK - 1) // BLOCK
    wf = torch.zeros(rb * BLOCK, cb * BLOCK, dtype=torch.float32)
    wf[:R, :C] = w.to(torch.float32)
    amax = wf.view(rb, BLOCK, cb, BLOCK).abs().amax(dim=(1, 3)).clamp(min=1e-4)
    scale_inv = (amax / FP8_MAX).to(torch.float32)
    q = (w.to(torch.float32) / _expand(scale_inv, R, C)).clamp(-FP8_MAX, FP8_MAX)
    return q.to(torch.float8_e4m3fn), scale_inv


def dequant_block_128(q: torch.Tensor, scale_inv: torch.Tensor) -> torch.Tensor:
    """``_dequant_block_fp8`` (src/blackwell_moe/runtime/qwen_patch.py:30-40):
    both the codes and the scales are cast to bf16 and multiplied in bf16."""
    R, C = q.shape
    w = q.to(torch.bfloat16)
    s = _expand(scale_inv.to(torch.bfloat16), R, C)
    return (w * s).contiguous()


def quant_act_group_128(x: torch.Tensor):
    """Per token, per 128 consecutive K elements:
    ``s = 448 / max(amax, 1e-4)``, ``q = e4m3(clamp(x * s))``,
    ``inv = max(amax, 1e-4) / 448``.  Returns ``(q[M,K], inv[M, ceil(K/128)])``."""
    M, K = x.shape
    g = (K + BLOCK - 1) // BLOCK
    xf = torch.zeros(M, g * BLOCK, dtype=torch.float32)
    xf[:, :K] = x.to(torch.float32)
    amax = xf.view(M, g, BLOCK).abs().amax(dim=2).clamp(min=1e-4)
    s = (FP8_MAX / amax).to(torch.float32)
    inv = (amax / FP8_MAX).to(torch.float32)
    q = (xf.view(M, g, BLOCK) * s.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).view(M, g * BLOCK)[:, :K]
    return q.to(torch.float8_e4m3fn), inv


def block_gemm(aq, a_inv, wq, w_inv):
    """``out[m,n] = sum_kb (sum_{k in kb} aq[m,k]*wq[k,n]) * a_inv[m,kb] * w_inv[kb,n//128]``
    with fp32 partial sums, K groups added in ascending order."""
    M, K = aq.shape
    N = wq.shape[1]
    out = torch.zeros(M, N, dtype=torch.float32)
    af, wf = aq.to(torch.float32), wq.to(torch.float32)
    for kb in range((K + BLOCK - 1) // BLOCK):
        k0, k1 = kb * BLOCK, min(K, (kb + 1) * BLOCK)
        part = af[:, k0:k1] @ wf[k0:k1]
        wn = w_inv[kb].repeat_interleave(BLOCK)[:N]
        out += part * (a_inv[:, kb:kb + 1] * wn.unsqueeze(0))
    return out


def moe_forward_block_recipe(x, w_gate, wq_gate, wq_up, wq_down, inv_gate, inv_up, inv_down,
                             top_k=8, routing=None, intermediates=None, experts=None, num_experts=None):
    """Block-scale MoE forward; scales ``inv_*`` are ``[E, ceil(in/128), ceil(out/128)]``.

    ``experts`` restricts the per-expert work (activation quantisation included) to the given
    segments, for shapes whose full forward is too slow on CPU; routing and permutation still
    cover every row and the other segments' rows stay zero.  The weight and scale arguments may
    then be dicts ``{expert id: tensor}`` with ``num_experts`` giving E."""
    T, D = x.shape
    if isinstance(wq_gate, dict):
        E, H = int(num_experts), next(iter(wq_gate.values())).shape[1]
    else:
        E, _, H = wq_gate.shape
    if routing is None:
        routing = router_canonical(x, w_gate, top_k)
    weights, indices = routing
    sort_perm, inverse_idx, offsets = permutation(indices, E)
    M = sort_perm.numel()
    g = (D + BLOCK - 1) // BLOCK
    if experts is None:
        xq, x_inv = quant_act_group_128(x[inverse_idx])
    else:       # quantisation is per row, so doing it segment by segment gives the same codes
        xq = torch.zeros(M, D, dtype=torch.float8_e4m3fn)
        x_inv = torch.zeros(M, g, dtype=torch.float32)
        for e in experts:
            s, t = int(offsets[e]), int(offsets[e + 1])
            if t > s:
                xq[s:t], x_inv[s:t] = quant_act_group_128(x[inverse_idx[s:t]])
    y_perm = torch.zeros(M, D, dtype=torch.bfloat16)
    hq_all = torch.zeros(M, H, dtype=torch.float8_e4m3fn)
    for e in (range(E) if experts is None else experts):
        s, t = int(offsets[e]), int(offsets[e + 1])
        if t <= s:
            continue
        gate = block_gemm(xq[s:t], x_inv[s:t], wq_gate[e], inv_gate[e]).to(torch.bfloat16)
        up = block_gemm(xq[s:t], x_inv[s:t], wq_up[e], inv_up[e]).to(torch.bfloat16)
        h = F.silu(gate) * up
        hq, h_inv = quant_act_group_128(h)
        y_perm[s:t] = block_gemm(hq, h_inv, wq_down[e], inv_down[e]).to(torch.bfloat16)
        hq_all[s:t] = hq
    flat_w = weights.reshape(-1)[sort_perm].to(torch.bfloat16).unsqueeze(-1)
    weighted = (y_perm * flat_w).to(torch.bfloat16)
    out = torch.zeros(T, D, dtype=torch.bfloat16)
    out.index_add_(0, inverse_idx, weighted)
    if intermediates is not None:
        intermediates.update(weights=weights, indices=indices, sort_perm=sort_perm,
                             inverse_idx=inverse_idx, offsets=offsets, xq=xq, x_inv=x_inv,
                             hq=hq_all, y_perm=y_perm)
    return out


def streaming_qwen_forward(x, weights, indices, hf_gate, hf_up, hf_down):
    """The routed part of StreamingQwenMoE.forward (src/blackwell_moe/runtime/qwen_patch.py:98-134):
    experts in ascending id, weights dequantised to bf16, ``F.linear`` in bf16, the weighted rows added
    into a bf16 output one expert after the other.  ``hf_*[e]`` = ``(codes[out, in], scale_inv[out/128, in/128])``."""
    out = torch.zeros_like(x)
    for eid in torch.unique(indices).tolist():
        pos = (indices == eid).nonzero(as_tuple=False)
        token_idx, k_idx = pos[:, 0], pos[:, 1]
        cur = x[token_idx]
        deq = lambda pair: dequant_block_128(pair[0], pair[1])      # noqa: E731  ([out, in] orientation here)
        gate = F.linear(cur, deq(hf_gate[eid]))
        up = F.linear(cur, deq(hf_up[eid]))
        y = F.linear(F.silu(gate) * up, deq(hf_down[eid]))
        w = weights[token_idx, k_idx].unsqueeze(-1).to(y.dtype)
        out.index_add_(0, token_idx, (y * w).to(out.dtype))
    return out
