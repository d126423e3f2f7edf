"""Parity of the CUDA path at the real dimensions of every benchmark configuration.

Each case runs the whole block through the public API on the GPU at the configuration's own
(T, D, H, E, top_k) and checks it stage by stage against the CPU oracle.  Where the full oracle is
too slow the *experts* are subsampled, never the rows: segment scales depend on every row of a
segment, so the oracle computes the chosen experts' segments completely.  Bars: routing indices,
offsets, permutation, activation scales and activation codes bit-exact (on every row for the
integer stages, on the checked segments for the codes); h within 5e-3, result rows and block output
within 1e-2 relative L1 of the oracle; the combine stage checked on all rows against the reference's
combine applied to the GPU's own result rows.
"""

import types

import pytest
import torch
import torch.nn as nn

import oracle
from helpers import BF16, combine_on_cpu, expert_subset, make_activations, make_gpu_weights

pytestmark = pytest.mark.gpu

_weights_cache = {}


def _weights(E, D, H, seed, block):
    """One set of weights per shape for the whole module (the Mixtral set alone is 1.4 GB)."""
    key = (E, D, H, seed, block)
    if key not in _weights_cache:
        _weights_cache.clear()
        torch.cuda.empty_cache()
        _weights_cache[key] = make_gpu_weights(E, D, H, seed, block=block)
    return _weights_cache[key]


def _pick_experts(offsets, n):
    """Up to n non-empty experts: the fullest, the emptiest, and evenly spaced ones in between."""
    counts = (offsets[1:] - offsets[:-1]).long()
    live = torch.nonzero(counts > 0).flatten()
    order = live[torch.argsort(counts[live], descending=True)]
    if order.numel() <= n:
        return [int(e) for e in order]
    pick = torch.linspace(0, order.numel() - 1, n).round().long()
    return sorted({int(order[i]) for i in pick})


def _check_integer_stages(v, inter, T, K):
    assert int(v["status"][0]) == 0, f"device status {int(v['status'][0])}"
    assert torch.equal(v["indices"], inter["indices"]), "routing indices differ"
    torch.testing.assert_close(v["weights"], inter["weights"], rtol=1e-3, atol=1e-4)
    assert torch.equal(v["offsets"], inter["offsets"]), "segment offsets differ"
    assert torch.equal(v["row_slot"].long(), inter["sort_perm"]), "permutation differs"
    M = T * K
    assert torch.equal(v["pos"].long()[inter["sort_perm"]], torch.arange(M)), "pos is not the inverse"


# (name, T, D, H, E, K, experts checked by the oracle (None = all))
PER_TENSOR = [
    ("mixtral", 1, 4096, 14336, 8, 2, None),          # split-K path, 32 / 112 K blocks
    ("mixtral", 16, 4096, 14336, 8, 2, None),
    ("mixtral", 64, 4096, 14336, 8, 2, None),
    ("mixtral", 1024, 4096, 14336, 8, 2, 3),
    ("deepseek", 1, 2048, 1408, 64, 6, None),
    ("deepseek", 64, 2048, 1408, 64, 6, None),
    ("deepseek", 4096, 2048, 1408, 64, 6, 6),
]


@pytest.mark.parametrize("name,T,D,H,E,K,n_check", PER_TENSOR)
def test_per_tensor_recipe_at_benchmark_dimensions(name, T, D, H, E, K, n_check):
    import blackwell_moe_b200 as bw
    W = _weights(E, D, H, seed=5, block=False)
    x, w_gate = make_activations(T, D, E, seed=100 + T)
    out = bw.fp8_moe_forward(x.cuda(), w_gate.cuda(), W["q_gate"], W["q_up"], W["q_down"],
                             W["s_gate"], W["s_up"], W["s_down"], top_k=K).cpu()
    v = {k: t.cpu() for k, t in bw.moe_stage_views("cuda:0", T, D, H, E, K).items()}
    experts = range(E) if n_check is None else _pick_experts(v["offsets"], n_check)
    sub = expert_subset(W, experts)
    inter = {}
    ref = oracle.moe_forward_fp8_recipe(x, w_gate, sub["q_gate"], sub["q_up"], sub["q_down"], sub["s_gate"],
                                        sub["s_up"], sub["s_down"], top_k=K, intermediates=inter, experts=experts)
    _check_integer_stages(v, inter, T, K)
    off = inter["offsets"]
    # Above 64 rows the down projection's epilogue multiplies each row by its routing weight (the product the
    # reference forms before its scatter_add, fp8_moe_v3.py:70-71); smaller batches keep plain rows.
    preweighted = T * K > 64
    want_rows = inter["weighted"] if preweighted else inter["y_perm"]
    for e in experts:
        s, t = int(off[e]), int(off[e + 1])
        if t <= s:
            continue
        assert float(v["scale_x"][e]) == float(inter["sx"][e]), f"x scale of expert {e}"
        assert torch.equal(v["xq"][s:t].view(torch.uint8), inter["xq"][s:t].view(torch.uint8)), f"x codes, expert {e}"
        if preweighted:
            assert oracle.rel_l1(v["h"][s:t], inter["h"][s:t]) < 5e-3, f"h, expert {e}"
        else:       # at most 64 rows: h is requantised inside the SwiGLU kernel, no 16-bit h is written
            mism = (v["hq"][s:t].view(torch.uint8) != inter["hq"][s:t].view(torch.uint8)).float().mean().item()
            assert mism < 0.02, f"{mism:.4f} of the h codes of expert {e} differ"
        torch.testing.assert_close(v["scale_h"][e], inter["sh"][e], rtol=1.6e-2, atol=0)
        assert oracle.rel_l1(v["y"][s:t], want_rows[s:t]) < 1e-2, f"y, expert {e}"
    # the combine on every row: the reference's combine applied to the GPU's own result rows
    n_rows = int(off[-1])
    comb = combine_on_cpu(v["y"][:n_rows], inter["weights"], inter["sort_perm"], inter["inverse_idx"], T,
                          preweighted=preweighted)
    assert oracle.rel_l1(out, comb) < 3e-3
    if n_check is None:
        assert oracle.rel_l1(out, ref) < 1e-2


# (name, T, D, H, E, K, zipf, experts checked)
BLOCK = [
    ("qwen3-30b", 1, 2048, 768, 128, 8, True, None),
    ("qwen3-30b", 256, 2048, 768, 128, 8, True, 6),
    ("qwen3-30b", 8192, 2048, 768, 128, 8, True, 6),
    ("qwen3.6", 128, 2048, 512, 256, 8, False, 8),
    ("qwen3.6", 32768, 2048, 512, 256, 8, False, 5),
]


@pytest.mark.parametrize("name,T,D,H,E,K,zipf,n_check", BLOCK)
def test_block_recipe_at_benchmark_dimensions(name, T, D, H, E, K, zipf, n_check):
    """The arithmetic of this recipe is pinned by our own restatement only (the reference has no FP8
    block-scale GEMM); the weight-scale semantics are the reference's."""
    import blackwell_moe_b200 as bw
    W = _weights(E, D, H, seed=6, block=True)
    x, w_gate = make_activations(T, D, E, seed=200 + T, zipf=zipf)
    out = bw.fp8_moe_forward(x.cuda(), w_gate.cuda(), W["q_gate"], W["q_up"], W["q_down"],
                             W["s_gate"], W["s_up"], W["s_down"], top_k=K).cpu()
    v = {k: t.cpu() for k, t in bw.moe_stage_views("cuda:0", T, D, H, E, K, block=True).items()}
    live = _pick_experts(v["offsets"], E)
    experts = live if n_check is None else _pick_experts(v["offsets"], n_check)
    sub = {k: {int(e): W[k][int(e)].cpu() for e in experts} for k in W}
    inter = {}
    oracle.moe_forward_block_recipe(x, w_gate, sub["q_gate"], sub["q_up"], sub["q_down"], sub["s_gate"], sub["s_up"],
                                    sub["s_down"], top_k=K, intermediates=inter, experts=experts, num_experts=E)
    _check_integer_stages(v, inter, T, K)
    off = inter["offsets"]
    for e in experts:
        s, t = int(off[e]), int(off[e + 1])
        assert torch.equal(v["x_inv"][s:t], inter["x_inv"][s:t]), f"activation group scales, expert {e}"
        assert torch.equal(v["xq"][s:t].view(torch.uint8), inter["xq"][s:t].view(torch.uint8)), f"x codes, expert {e}"
        mism = (v["hq"][s:t].view(torch.uint8) != inter["hq"][s:t].view(torch.uint8)).float().mean().item()
        assert mism < 0.02, f"{mism:.4f} of the h codes of expert {e} differ"
        assert oracle.rel_l1(v["y"][s:t], inter["y_perm"][s:t]) < 1e-2, f"y, expert {e}"
    comb = combine_on_cpu(v["y"], inter["weights"], inter["sort_perm"], inter["inverse_idx"], T)
    assert oracle.rel_l1(out, comb) < 3e-3


class _MLP(nn.Module):
    def __init__(self, D, Hs, gen):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = (nn.Linear(D, Hs, bias=False), nn.Linear(D, Hs, bias=False),
                                                        nn.Linear(Hs, D, bias=False))
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=gen) * 0.02)


def test_deepseek_layer_with_shared_experts_at_benchmark_dimensions():
    """DeepSeek-V2-Lite block as the drop-in module runs it: 64 routed experts (top-6, H=1408) plus the
    shared MLP of intermediate 2 x 1408 in FP8, out = routed * routed_scaling_factor + shared, T=4096."""
    import blackwell_moe_b200 as bw
    T, D, H, E, K, Hs, scale = 4096, 2048, 1408, 64, 6, 2816, 1.0
    W = _weights(E, D, H, seed=5, block=False)
    x, w_gate = make_activations(T, D, E, seed=300)
    mlp = _MLP(D, Hs, torch.Generator().manual_seed(301))
    shared = bw.FP8SharedExpert(mlp).cuda()

    class DeepseekV2MoE(nn.Module):
        def __init__(self):
            super().__init__()
            self.config = types.SimpleNamespace(n_routed_experts=E, num_experts_per_tok=K, hidden_size=D,
                                                routed_scaling_factor=scale)
            self.gate = nn.Linear(D, E, bias=False)
            with torch.no_grad():
                self.gate.weight.copy_(w_gate.t().float())
            self.shared_experts = shared

    store = dict(gate=W["q_gate"], up=W["q_up"], down=W["q_down"], s_g=W["s_gate"], s_u=W["s_up"], s_d=W["s_down"])
    layer = bw.FP8MoELayer(DeepseekV2MoE().cuda(), store).cuda()
    out = layer(x.view(4, T // 4, D).cuda()).cpu().view(T, D)
    wq = [oracle.quant_fp8_e4m3(getattr(mlp, n).weight.detach().t().contiguous().to(BF16))
          for n in ("gate_proj", "up_proj", "down_proj")]
    sh_ref = oracle.shared_expert_fp8(x, wq[0][0], wq[1][0], wq[2][0], wq[0][1], wq[1][1], wq[2][1])
    assert oracle.rel_l1(shared(x.cuda()).cpu(), sh_ref) < 1e-2
    sub = expert_subset(W, range(E))
    routed = oracle.moe_forward_fp8_recipe(x, w_gate, sub["q_gate"], sub["q_up"], sub["q_down"], sub["s_gate"],
                                           sub["s_up"], sub["s_down"], top_k=K)
    ref = (routed * scale) + sh_ref                       # deepseek_patch.py:51-53
    assert oracle.rel_l1(out, ref) < 1e-2
