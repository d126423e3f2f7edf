"""Module drop-ins (shared experts, DeepSeek MoE layer, Mixtral block) on the GPU against the
oracle and against the reference's own FP8SharedExpert output stored as a fixture."""

import types

import pytest
import torch
import torch.nn as nn

import oracle
from conftest import from_bits
from helpers import BF16, FP8, make_inputs

pytestmark = pytest.mark.gpu


def test_dense_mlp_matches_reference_shared_expert_fixture(golden):
    import blackwell_moe_b200 as bw
    g = golden("block_shared")
    x = from_bits(g["sx"], BF16)
    w = [from_bits(g[k], FP8) for k in ("s_wg", "s_wu", "s_wd")]
    s = [torch.from_numpy(g[k]) for k in ("s_sg", "s_su", "s_sd")]
    y = bw.fp8_dense_mlp(x.cuda(), *[t.cuda() for t in w], *[t.cuda() for t in s]).cpu()
    assert oracle.rel_l1(y, oracle.shared_expert_fp8(x, *w, *s)) < 1e-2
    assert oracle.rel_l1(y, from_bits(g["sy"], BF16)) < 1e-2          # reference FP8SharedExpert.forward on CPU


class _MLP(nn.Module):
    def __init__(self, D, Hs, gen):
        super().__init__()
        self.gate_proj, self.up_proj, self.down_proj = (nn.Linear(D, Hs, bias=False), nn.Linear(D, Hs, bias=False),
                                                        nn.Linear(Hs, D, bias=False))
        with torch.no_grad():
            for p in self.parameters():
                p.copy_(torch.randn(p.shape, generator=gen) * 0.03)


def test_shared_expert_module_and_deepseek_layer():
    import blackwell_moe_b200 as bw
    T, D, E, K, H, Hs = 96, 256, 8, 2, 128, 384
    inp = make_inputs(T, D, E, K, H, seed=31, keep_bf16=False)
    gen = torch.Generator().manual_seed(32)
    mlp = _MLP(D, Hs, gen)
    shared = bw.FP8SharedExpert(mlp).cuda()
    # oracle for the shared expert, weights quantised the same way
    wq = [oracle.quant_fp8_e4m3(getattr(mlp, n).weight.detach().t().contiguous().to(BF16))
          for n in ("gate_proj", "up_proj", "down_proj")]
    x3 = inp["x"].view(4, 24, D)
    sh_ref = oracle.shared_expert_fp8(inp["x"], wq[0][0], wq[1][0], wq[2][0], wq[0][1], wq[1][1], wq[2][1])
    sh_out = shared(x3.cuda()).cpu().view(T, D)
    assert oracle.rel_l1(sh_out, sh_ref) < 1e-2

    class DeepseekV2MoE(nn.Module):          # the class name is what the patch function looks for
        def __init__(self):
            super().__init__()
            self.config = types.SimpleNamespace(n_routed_experts=E, num_experts_per_tok=K, hidden_size=D,
                                                routed_scaling_factor=2.5)
            self.gate = nn.Linear(D, E, bias=False)
            with torch.no_grad():
                self.gate.weight.copy_(inp["w_gate"].t().float())
            self.shared_experts = shared

    store = dict(gate=inp["q_gate"].cuda(), up=inp["q_up"].cuda(), down=inp["q_down"].cuda(),
                 s_g=inp["s_gate"].cuda(), s_u=inp["s_up"].cuda(), s_d=inp["s_down"].cuda())
    layer = bw.FP8MoELayer(DeepseekV2MoE().cuda(), store).cuda()
    out = layer(x3.cuda()).cpu().view(T, D)
    routed = oracle.moe_forward_fp8_recipe(inp["x"], inp["w_gate"], inp["q_gate"], inp["q_up"], inp["q_down"],
                                           inp["s_gate"], inp["s_up"], inp["s_down"], top_k=K)
    # reference glue: routed * routed_scale (bf16) + shared_out (bf16), deepseek_patch.py:51-53
    ref = (routed * 2.5) + sh_ref
    assert oracle.rel_l1(out, ref) < 1e-2

    assert layer._folded == 3        # Hs = 3 x H: the shared MLP runs as three always-on groups of the routed pipeline
    # the reference's two separate calls (shared MLP, then routed experts with the add fused into the combine)
    layer2 = bw.FP8MoELayer(DeepseekV2MoE().cuda(), store).cuda()
    layer2.fold_shared = False
    out2 = layer2(x3.cuda()).cpu().view(T, D)
    assert layer2._folded is False
    assert oracle.rel_l1(out2, ref) < 1e-2
    assert oracle.rel_l1(out, out2) < 5e-3

    # the patch helper finds the module by class name
    model = nn.Module()
    model.model = nn.Module()
    model.model.layers = nn.ModuleList([nn.Module(), nn.Module()])
    model.model.layers[1].mlp = DeepseekV2MoE().cuda()
    assert bw.patch_deepseek_moe_with_store(model, {1: store}) == 1
    assert isinstance(model.model.layers[1].mlp, bw.FP8MoELayer)


def test_mixtral_block_contract():
    import blackwell_moe_b200 as bw
    T, D, E, K, H = 64, 256, 8, 2, 256
    inp = make_inputs(T, D, E, K, H, seed=41, keep_bf16=False)
    c = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in inp.items()}
    blk = bw.FP8MixtralSparseMoeBlock(c["w_gate"], c["q_gate"], c["q_up"], c["q_down"], c["s_gate"], c["s_up"],
                                      c["s_down"], top_k=K)
    out, aux = blk(c["x"].view(2, 32, D))
    assert out.shape == (2, 32, D) and aux.shape == (1,) and float(aux) == 0.0
    ref = oracle.moe_forward_fp8_recipe(inp["x"], inp["w_gate"], inp["q_gate"], inp["q_up"], inp["q_down"],
                                        inp["s_gate"], inp["s_up"], inp["s_down"], top_k=K)
    assert oracle.rel_l1(out.cpu().view(T, D), ref) < 1e-2
