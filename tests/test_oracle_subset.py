"""The oracle's expert-subsampling mode (used by the full-size GPU parity tests) against its full mode."""

import torch

import oracle
from helpers import BF16, make_inputs


def test_per_tensor_subset_equals_full_on_the_chosen_segments():
    inp = make_inputs(90, 128, 6, 2, 96, seed=2, keep_bf16=False)
    args = (inp["x"], inp["w_gate"])
    full, sub = {}, {}
    oracle.moe_forward_fp8_recipe(*args, inp["q_gate"], inp["q_up"], inp["q_down"], inp["s_gate"], inp["s_up"],
                                  inp["s_down"], top_k=2, intermediates=full)
    chosen = [1, 4]
    as_dict = lambda t: {e: t[e] for e in chosen}                                   # noqa: E731
    oracle.moe_forward_fp8_recipe(*args, as_dict(inp["q_gate"]), as_dict(inp["q_up"]), as_dict(inp["q_down"]),
                                  inp["s_gate"], inp["s_up"], inp["s_down"], top_k=2, intermediates=sub, experts=chosen)
    assert torch.equal(full["sort_perm"], sub["sort_perm"]) and torch.equal(full["offsets"], sub["offsets"])
    for e in chosen:
        s, t = int(full["offsets"][e]), int(full["offsets"][e + 1])
        assert t > s
        for k in ("xq", "hq"):
            assert torch.equal(full[k][s:t].view(torch.uint8), sub[k][s:t].view(torch.uint8))
        assert torch.equal(full["y_perm"][s:t], sub["y_perm"][s:t]) and torch.equal(full["h"][s:t], sub["h"][s:t])
        assert float(full["sx"][e]) == float(sub["sx"][e]) and float(full["sh"][e]) == float(sub["sh"][e])


def test_block_subset_equals_full_on_the_chosen_segments():
    g = torch.Generator().manual_seed(5)
    T, D, E, K, H = 70, 256, 6, 2, 128
    x = torch.randn(T, D, generator=g).to(BF16)
    w_gate = (torch.randn(D, E, generator=g) * 0.02).to(BF16)
    q, s = {}, {}
    for name, shape in (("gate", (D, H)), ("up", (D, H)), ("down", (H, D))):
        pairs = [oracle.quant_block_128((torch.randn(shape, generator=g) * 0.02).to(BF16)) for _ in range(E)]
        q[name], s[name] = torch.stack([p[0] for p in pairs]), torch.stack([p[1] for p in pairs])
    full, sub = {}, {}
    oracle.moe_forward_block_recipe(x, w_gate, q["gate"], q["up"], q["down"], s["gate"], s["up"], s["down"], top_k=K,
                                    intermediates=full)
    chosen = [0, 3]
    d = lambda t: {e: t[e] for e in chosen}                                         # noqa: E731
    oracle.moe_forward_block_recipe(x, w_gate, d(q["gate"]), d(q["up"]), d(q["down"]), d(s["gate"]), d(s["up"]),
                                    d(s["down"]), top_k=K, intermediates=sub, experts=chosen, num_experts=E)
    assert torch.equal(full["sort_perm"], sub["sort_perm"])
    for e in chosen:
        a, b = int(full["offsets"][e]), int(full["offsets"][e + 1])
        assert b > a
        assert torch.equal(full["xq"][a:b].view(torch.uint8), sub["xq"][a:b].view(torch.uint8))
        assert torch.equal(full["x_inv"][a:b], sub["x_inv"][a:b])
        assert torch.equal(full["hq"][a:b].view(torch.uint8), sub["hq"][a:b].view(torch.uint8))
        assert torch.equal(full["y_perm"][a:b], sub["y_perm"][a:b])
