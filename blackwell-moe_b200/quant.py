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
