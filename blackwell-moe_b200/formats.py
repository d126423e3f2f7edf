"""Weight-format adapters either side of the MoE-block forward (load time, not hot path).

* the reference's per-expert files ``expert_L{layer:03d}_E{expert:03d}.safetensors`` with keys
  ``gate_q, up_q, down_q, scale_g, scale_u, scale_d`` (``[in, out]`` E4M3 weights, forward
  scales; src/blackwell_moe/runtime/disk_expert_pool.py:38-66) <-> the stacked ``[E, in, out]``
  tensors the block takes;
* Hugging Face block-FP8 experts (``weight`` ``[out, in]`` E4M3 + ``weight_scale_inv``
  ``[ceil(out/128), ceil(in/128)]``, the layout ``_dequant_block_fp8`` reads,
  src/blackwell_moe/runtime/qwen_patch.py:30-40) -> ``[E, in, out]`` codes and
  ``[E, ceil(in/128), ceil(out/128)]`` inverse scales.
"""

from __future__ import annotations

from pathlib import Path

import torch

_KEYS = ("gate_q", "up_q", "down_q", "scale_g", "scale_u", "scale_d")


def expert_file(root, layer_idx: int, expert_idx: int) -> Path:
    return Path(root) / f"expert_L{layer_idx:03d}_E{expert_idx:03d}.safetensors"


def save_layer_experts(root, layer_idx: int, q_gate, q_up, q_down, s_gate, s_up, s_down) -> list:
    """Write one file per expert in the reference's on-disk format."""
    from safetensors.torch import save_file
    Path(root).mkdir(parents=True, exist_ok=True)
    paths = []
    for e in range(q_gate.shape[0]):
        f = expert_file(root, layer_idx, e)
        save_file({"gate_q": q_gate[e].cpu().contiguous(), "up_q": q_up[e].cpu().contiguous(),
                   "down_q": q_down[e].cpu().contiguous(),
                   "scale_g": s_gate[e].cpu().to(torch.float32).reshape(()),
                   "scale_u": s_up[e].cpu().to(torch.float32).reshape(()),
                   "scale_d": s_down[e].cpu().to(torch.float32).reshape(())}, str(f))
        paths.append(f)
    return paths


def load_layer_experts(root, layer_idx: int, num_experts: int, device="cpu"):
    """Read the reference's per-expert files of one layer into stacked tensors
    ``(q_gate[E,D,H], q_up[E,D,H], q_down[E,H,D], s_gate[E], s_up[E], s_down[E])``."""
    from safetensors import safe_open
    cols = {k: [] for k in _KEYS}
    for e in range(num_experts):
        with safe_open(str(expert_file(root, layer_idx, e)), framework="pt", device="cpu") as f:
            for k in _KEYS:
                cols[k].append(f.get_tensor(k))
    q = [torch.stack(cols[k]).contiguous().to(device) for k in _KEYS[:3]]
    s = [torch.stack([t.reshape(()) for t in cols[k]]).to(torch.float32).contiguous().to(device) for k in _KEYS[3:]]
    return (*q, *s)


def from_hf_block_fp8(weights, scale_invs):
    """Stack HF block-FP8 projections of E experts for the block-scale recipe.

    ``weights[e]``: ``[out, in]`` E4M3; ``scale_invs[e]``: ``[ceil(out/128), ceil(in/128)]``.
    Returns ``(codes[E, in, out] e4m3, inv[E, ceil(in/128), ceil(out/128)] fp32)``: a pure
    transposition, the numbers are untouched."""
    codes = torch.stack([w.view(torch.uint8).t().contiguous() for w in weights]).view(torch.float8_e4m3fn)
    inv = torch.stack([s.to(torch.float32).t().contiguous() for s in scale_invs])
    return codes.contiguous(), inv.contiguous()
