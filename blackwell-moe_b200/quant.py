"""Load-time weight preparation (not on the hot path).

Same arithmetic and names as the reference's
``src/blackwell_moe/kernels/fp8_quant.py:21-36``; runs as ordinary torch ops
on whatever device the weights are on, once, when a checkpoint is loaded.
The per-call activation quantisation is done by the CUDA kernels instead.
"""

from __future__ import annotations

import torch

FP8_MAX_E4M3: float = 448.0


def quant_fp8_e4m3(x: torch.Tensor):
    """Per-tensor symmetric E4M3 quantisation: ``(q, scale)`` with ``q / scale ~= x``."""
    amax = x.abs().amax().clamp(min=1e-4).to(torch.float32)
    scale = (FP8_MAX_E4M3 / amax).to(torch.float32)
    q = (x.to(torch.float32) * scale).clamp(-FP8_MAX_E4M3, FP8_MAX_E4M3).to(torch.float8_e4m3fn)
    return q, scale


def dequant_fp8_e4m3(x_fp8: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    return (x_fp8.to(torch.float32) / scale).to(torch.bfloat16)


def quantize_expert_weights(w: torch.Tensor):
    """Quantise a stack ``[E, in, out]`` expert by expert, as the reference's bench
    and loaders do (src/blackwell_moe/bench/cli.py:62-70).  Returns
    ``(q[E,in,out] e4m3, scales[E] fp32)``."""
    qs, ss = zip(*(quant_fp8_e4m3(w[e]) for e in range(w.shape[0])))
    return torch.stack(list(qs)).contiguous(), torch.stack(list(ss)).to(torch.float32).contiguous()


def quant_fp8_block_128(w: torch.Tensor):
    """128x128 block quantisation of one ``[in, out]`` matrix in the convention of HF block-FP8
    checkpoints, i.e. the inverse of the reference's ``_dequant_block_fp8``
    (src/blackwell_moe/runtime/qwen_patch.py:30-40): ``w ~= code * scale_inv``.
    Returns ``(code[in,out] e4m3, scale_inv[ceil(in/128), ceil(out/128)] fp32)``."""
    R, C = w.shape
    rb, cb = (R + 127) // 128, (C + 127) // 128
    wf = torch.zeros(rb * 128, cb * 128, dtype=torch.float32, device=w.device)
    wf[:R, :C] = w.to(torch.float32)
    amax = wf.view(rb, 128, cb, 128).abs().amax(dim=(1, 3)).clamp(min=1e-4)
    # tensor / tensor: an IEEE division on every device (tensor / python-scalar is a reciprocal multiply on CUDA)
    scale_inv = (amax / torch.full_like(amax, FP8_MAX_E4M3)).to(torch.float32)
    full = scale_inv.repeat_interleave(128, dim=0)[:R].repeat_interleave(128, dim=1)[:, :C]
    q = (w.to(torch.float32) / full).clamp(-FP8_MAX_E4M3, FP8_MAX_E4M3).to(torch.float8_e4m3fn)
    return q, scale_inv


def quantize_expert_weights_block(w: torch.Tensor):
    """:func:`quant_fp8_block_128` over a stack ``[E, in, out]`` -> ``(codes, scale_inv[E, in/128, out/128])``."""
    qs, ss = zip(*(quant_fp8_block_128(w[e]) for e in range(w.shape[0])))
    return torch.stack(list(qs)).contiguous(), torch.stack(list(ss)).contiguous()
