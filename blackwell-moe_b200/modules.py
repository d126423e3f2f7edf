"""nn.Module drop-ins that sit either side of the MoE-block forward.

Drop-in replacements must keep the attribute names, buffer names and the lookup of the patched
modules by class-name string, so the following parts FOLLOW THE REFERENCE LINE FOR LINE:
``FP8SharedExpert.__init__`` and ``patch_shared_experts``
(src/blackwell_moe/runtime/shared_expert_fp8.py:36-55,71-81), ``FP8MoELayer.__init__`` and
``patch_deepseek_moe_with_store`` (src/blackwell_moe/runtime/deepseek_patch.py:15-37,56-73).
Everything that computes is new and runs on libbwmoe: the ``forward`` methods, ``fp8_dense_mlp``,
and ``FP8MixtralSparseMoeBlock`` (which keeps only the ``(out, zeros(1))`` return contract of
src/blackwell_moe/runtime/mixtral_patch.py:39-48).
"""

from __future__ import annotations

import torch
import torch.nn as nn

from . import _lib
from .moe import (_contig, _require_cuda, _stream, _workspace, fp8_moe_forward, fp8_moe_forward_shared,
                  stack_shared_experts)
from .quant import quant_fp8_e4m3

_FP8 = torch.float8_e4m3fn


def fp8_dense_mlp(x, w_gate, w_up, w_down, s_gate, s_up, s_down) -> torch.Tensor:
    """Dense FP8 SwiGLU MLP over all rows with whole-tensor scales for ``x`` and ``h``:
    ``x[T,D] bf16``, weights ``[D,H]`` / ``[H,D]`` e4m3, scales fp32 scalars."""
    assert x.dim() == 2 and x.dtype == torch.bfloat16, (x.shape, x.dtype)
    T, D = x.shape
    H = w_gate.shape[1]
    assert tuple(w_gate.shape) == (D, H) and tuple(w_up.shape) == (D, H) and tuple(w_down.shape) == (H, D)
    ts = [_contig(t, "tensor") for t in (x, w_gate, w_up, w_down)]
    ss = [s.reshape(1).to(torch.float32).contiguous() for s in (s_gate, s_up, s_down)]
    dev = _require_cuda(*ts, *ss)
    lib = _lib.lib()
    with torch.cuda.device(dev):
        need = lib.bwmoe_workspace_bytes(T, D, H, 1, 1)
        if need == 0:
            raise ValueError(f"unsupported shape T={T} D={D} H={H}")
        ws = _workspace(dev, need)
        out = torch.empty_like(x)
        _lib.check(lib.bwmoe_dense_mlp(*[t.data_ptr() for t in ts], *[s.data_ptr() for s in ss], T, D, H,
                                       out.data_ptr(), ws.data_ptr(), ws.numel(), _stream(dev)))
    return out


class FP8SharedExpert(nn.Module):
    """Drop-in FP8 replacement for a ``gate_proj/up_proj/down_proj`` MLP (DeepseekV2MLP used as
    ``shared_experts``): weights quantised per tensor at construction, activations per call."""

    def __init__(self, mlp: nn.Module):
        super().__init__()
        gp = mlp.gate_proj.weight.detach().t().contiguous()      # [D, H_inter]
        up = mlp.up_proj.weight.detach().t().contiguous()
        dp = mlp.down_proj.weight.detach().t().contiguous()      # [H_inter, D]
        g_q, sg = quant_fp8_e4m3(gp.to(torch.bfloat16))
        u_q, su = quant_fp8_e4m3(up.to(torch.bfloat16))
        d_q, sd = quant_fp8_e4m3(dp.to(torch.bfloat16))
        self.register_buffer("w_gate", g_q.contiguous())
        self.register_buffer("w_up", u_q.contiguous())
        self.register_buffer("w_down", d_q.contiguous())
        self.register_buffer("s_gate", sg)
        self.register_buffer("s_up", su)
        self.register_buffer("s_down", sd)
        self.hidden_size = gp.shape[0]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        flat = x.reshape(-1, self.hidden_size).to(torch.bfloat16).contiguous()
        y = fp8_dense_mlp(flat, self.w_gate, self.w_up, self.w_down, self.s_gate, self.s_up, self.s_down)
        return y.reshape(shape)


def patch_shared_experts(model: nn.Module) -> int:
    """Replace DeepseekV2MLP used as ``.shared_experts`` with the FP8 version."""
    patched = 0
    for module in model.modules():
        if hasattr(module, "shared_experts") and module.__class__.__name__ == "DeepseekV2MoE":
            if module.shared_experts.__class__.__name__ == "DeepseekV2MLP":
                dev = next(module.shared_experts.parameters()).device
                module.shared_experts = FP8SharedExpert(module.shared_experts).to(dev)
                patched += 1
    return patched


class FP8MoELayer(nn.Module):
    """Replaces ``DeepseekV2MoE``: routed experts through the FP8 block, plus the shared
    experts and ``routed_scaling_factor``; the scale and the shared-expert add are fused into
    the block's combine kernel."""

    def __init__(self, deepseek_moe: nn.Module, fp8_weights: dict):
        super().__init__()
        cfg = deepseek_moe.config
        self.n_experts = cfg.n_routed_experts
        self.top_k = cfg.num_experts_per_tok
        self.hidden_dim = cfg.hidden_size
        self.routed_scale = cfg.routed_scaling_factor
        gate_w = deepseek_moe.gate.weight.detach().clone()            # [E, D]
        self.register_buffer("w_router", gate_w.t().contiguous().to(torch.bfloat16))   # [D, E]
        self.register_buffer("experts_w_gate_fp8", fp8_weights["gate"])
        self.register_buffer("experts_w_up_fp8", fp8_weights["up"])
        self.register_buffer("experts_w_down_fp8", fp8_weights["down"])
        self.register_buffer("scales_gate", fp8_weights["s_g"])
        self.register_buffer("scales_up", fp8_weights["s_u"])
        self.register_buffer("scales_down", fp8_weights["s_d"])
        self.shared_experts = deepseek_moe.shared_experts
        self.gate = deepseek_moe.gate

    #: run the shared experts as always-on groups of the routed pipeline (one set of launches for the whole
    #: block) when they are an :class:`FP8SharedExpert` whose intermediate size is a multiple of the routed
    #: experts'; set to False to keep the two separate calls of the reference's forward
    fold_shared = True
    _folded = None

    def _fold(self):
        """Stack the shared MLP behind the routed experts once (the routed buffers are replaced by the
        stacked ones, so nothing is held twice)."""
        sh = self.shared_experts
        E, D, H = self.experts_w_gate_fp8.shape
        ok = (self.fold_shared and isinstance(sh, FP8SharedExpert) and sh.w_gate.shape[0] == D
              and sh.w_gate.shape[1] % H == 0 and sh.w_gate.device == self.experts_w_gate_fp8.device)
        if ok:
            S = sh.w_gate.shape[1] // H
            ok = E + S <= 256 and self.top_k + S <= 32
        if not ok:
            self._folded = False
            return
        g, u, d, sg, su, sd, S = stack_shared_experts(
            self.experts_w_gate_fp8, self.experts_w_up_fp8, self.experts_w_down_fp8, self.scales_gate, self.scales_up,
            self.scales_down, sh.w_gate, sh.w_up, sh.w_down, sh.s_gate, sh.s_up, sh.s_down)
        self.experts_w_gate_fp8, self.experts_w_up_fp8, self.experts_w_down_fp8 = g, u, d
        self.scales_gate, self.scales_up, self.scales_down = sg, su, sd
        self._folded = S

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, self.hidden_dim).to(torch.bfloat16).contiguous()
        if self._folded is None:
            self._fold()
        if self._folded:
            out = fp8_moe_forward_shared(x, self.w_router, self.experts_w_gate_fp8, self.experts_w_up_fp8,
                                         self.experts_w_down_fp8, self.scales_gate, self.scales_up, self.scales_down,
                                         top_k=self.top_k, n_shared=self._folded, routed_scale=float(self.routed_scale))
            return out.reshape(shape)
        shared_out = self.shared_experts(hidden_states).reshape(-1, self.hidden_dim).to(torch.bfloat16).contiguous()
        out = fp8_moe_forward(x, self.w_router, self.experts_w_gate_fp8, self.experts_w_up_fp8,
                              self.experts_w_down_fp8, self.scales_gate, self.scales_up, self.scales_down,
                              top_k=self.top_k, routed_scale=float(self.routed_scale), residual=shared_out)
        return out.reshape(shape)


def patch_deepseek_moe_with_store(model: nn.Module, fp8_store: dict) -> int:
    """Install :class:`FP8MoELayer` over every ``DeepseekV2MoE`` whose layer index is in the store."""
    patched = 0
    for name, module in list(model.named_modules()):
        if module.__class__.__name__ != "DeepseekV2MoE":
            continue
        layer_idx = int(name.split(".")[2])       # "model.layers.<i>.mlp"
        if layer_idx not in fp8_store:
            continue
        parent_name = ".".join(name.split(".")[:-1])
        child_name = name.split(".")[-1]
        parent = model.get_submodule(parent_name) if parent_name else model
        setattr(parent, child_name, FP8MoELayer(module, fp8_store[layer_idx]))
        patched += 1
    return patched


class FP8MixtralSparseMoeBlock(nn.Module):
    """Replaces ``MixtralSparseMoeBlock`` with device-resident FP8 experts.  Returns
    ``(out, zeros(1))`` like the reference's Mixtral drop-in (HF expects ``(hidden, router_logits)``)."""

    def __init__(self, w_router, experts_w_gate, experts_w_up, experts_w_down, scales_gate, scales_up, scales_down,
                 top_k: int):
        super().__init__()
        for name, t in (("w_router", w_router), ("experts_w_gate_fp8", experts_w_gate),
                        ("experts_w_up_fp8", experts_w_up), ("experts_w_down_fp8", experts_w_down),
                        ("scales_gate", scales_gate), ("scales_up", scales_up), ("scales_down", scales_down)):
            self.register_buffer(name, t)
        self.top_k = top_k

    @classmethod
    def from_hf_block(cls, block: nn.Module) -> "FP8MixtralSparseMoeBlock":
        """Quantise the experts of a HF ``MixtralSparseMoeBlock`` (``experts[i].w1/w3/w2`` as gate/up/down,
        ``[out,in]`` weights transposed to the ``[in,out]`` layout of the FP8 block)."""
        qs = {"g": [], "u": [], "d": []}
        ss = {"g": [], "u": [], "d": []}
        for ex in block.experts:
            for key, lin in (("g", ex.w1), ("u", ex.w3), ("d", ex.w2)):
                q, s = quant_fp8_e4m3(lin.weight.detach().t().contiguous().to(torch.bfloat16))
                qs[key].append(q), ss[key].append(s)
        stack = lambda xs: torch.stack(xs).contiguous()                               # noqa: E731
        return cls(block.gate.weight.detach().t().contiguous().to(torch.bfloat16), stack(qs["g"]), stack(qs["u"]),
                   stack(qs["d"]), stack(ss["g"]).float(), stack(ss["u"]).float(), stack(ss["d"]).float(),
                   top_k=block.top_k)

    def forward(self, hidden_states: torch.Tensor):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1]).to(torch.bfloat16).contiguous()
        out = fp8_moe_forward(x, self.w_router, self.experts_w_gate_fp8, self.experts_w_up_fp8,
                              self.experts_w_down_fp8, self.scales_gate, self.scales_up, self.scales_down,
                              top_k=self.top_k)
        return out.reshape(shape), torch.zeros(1, device=hidden_states.device, dtype=hidden_states.dtype)
