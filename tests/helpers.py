"""Seeded synthetic inputs and comparison helpers shared by the tests."""

from __future__ import annotations

import torch

import oracle

BF16, FP8 = torch.bfloat16, torch.float8_e4m3fn


def make_inputs(T, D, E, K, H, seed=0, x_scale=1.0, w_scale=0.02, keep_bf16=True):
    """CPU tensors in the reference bench's order (src/blackwell_moe/bench/cli.py:39-70):
    x, w_gate, expert weights ~N(0, w_scale^2) quantised per expert matrix."""
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, D, generator=g) * x_scale).to(BF16)
    w_gate = (torch.randn(D, E, generator=g) * w_scale).to(BF16)
    out = dict(x=x, w_gate=w_gate, k=K)
    for name, (a, b) in (("gate", (D, H)), ("up", (D, H)), ("down", (H, D))):
        qs, ss, ws = [], [], []
        for _ in range(E):
            w = (torch.randn(a, b, generator=g) * w_scale).to(BF16)
            q, s = oracle.quant_fp8_e4m3(w)
            qs.append(q), ss.append(s)
            if keep_bf16:
                ws.append(w)
        out["q_" + name] = torch.stack(qs)
        out["s_" + name] = torch.stack(ss).to(torch.float32)
        if keep_bf16:
            out["bf_" + name] = torch.stack(ws)
    return out


def to_cuda(inp, dev="cuda:0"):
    return {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in inp.items()}


def run_cuda_forward(inp, dev="cuda:0"):
    import blackwell_moe_b200 as bw
    c = to_cuda(inp, dev)
    out = bw.fp8_moe_forward(c["x"], c["w_gate"], c["q_gate"], c["q_up"], c["q_down"],
                             c["s_gate"], c["s_up"], c["s_down"], top_k=inp["k"])
    T, D = inp["x"].shape
    E, _, H = inp["q_gate"].shape
    views = bw.moe_stage_views(dev, T, D, H, E, inp["k"])
    return out.cpu(), {k: v.cpu() for k, v in views.items()}


def run_oracle_forward(inp):
    inter = {}
    out = oracle.moe_forward_fp8_recipe(inp["x"], inp["w_gate"], inp["q_gate"], inp["q_up"], inp["q_down"],
                                        inp["s_gate"], inp["s_up"], inp["s_down"], top_k=inp["k"],
                                        intermediates=inter)
    return out, inter


def check_against_oracle(inp, out, views, ref_out, inter, tol=1e-2):
    """Bit-exact routing / permutation / x codes; tolerance on everything behind a GEMM."""
    E = inp["q_gate"].shape[0]
    assert int(views["status"][0]) == 0, f"device status {int(views['status'][0])}"
    assert torch.equal(views["indices"], inter["indices"]), "routing indices differ"
    torch.testing.assert_close(views["weights"], inter["weights"], rtol=1e-3, atol=1e-4)
    assert torch.equal(views["offsets"], inter["offsets"]), "segment offsets differ"
    assert torch.equal(views["row_slot"].long(), inter["sort_perm"]), "permutation differs"
    M = inter["sort_perm"].numel()
    assert torch.equal(views["pos"].long()[inter["sort_perm"]], torch.arange(M)), "pos is not the inverse"
    counts = inter["offsets"][1:] - inter["offsets"][:-1]
    live = counts > 0
    assert torch.equal(views["scale_x"][live], inter["sx"][live]), "x segment scales differ"
    assert torch.equal(views["xq"].view(torch.uint8), inter["xq"].view(torch.uint8)), "x FP8 codes differ"
    if M > 64:
        assert oracle.rel_l1(views["h"], inter["h"]) < 5e-3, "SwiGLU output off"
    else:   # small batches requantise h inside the SwiGLU kernel: no 16-bit h exists, the codes are what can be checked
        n = int(inter["offsets"][-1])
        mism = (views["hq"][:n].view(torch.uint8) != inter["hq"][:n].view(torch.uint8)).float().mean().item()
        assert mism < 0.02, f"{mism:.4f} of the h codes differ"
    torch.testing.assert_close(views["scale_h"][live], inter["sh"][live], rtol=1.6e-2, atol=0)
    err = oracle.rel_l1(out, ref_out)
    assert err < tol, f"rel-L1 vs FP8 recipe oracle {err:.4f} >= {tol}"
    return err


# ---- full-size shapes: weights are made and quantised on the GPU (seconds instead of minutes), and the
# oracle receives copies of the experts it checks only ----
def make_gpu_weights(E, D, H, seed, block=False, dev="cuda:0", w_scale=0.02):
    """Expert weights ~N(0, w_scale^2) bf16 generated expert by expert on the device and quantised there
    with the package's load-time quantisers (plain torch ops): per expert matrix, or 128x128 blocks.
    The codes and scales are *inputs* of both the CUDA path and the oracle."""
    import blackwell_moe_b200 as bw
    g = torch.Generator(device=dev)
    out = {"q_gate": [], "q_up": [], "q_down": [], "s_gate": [], "s_up": [], "s_down": []}
    for e in range(E):
        for i, (name, shape) in enumerate((("gate", (D, H)), ("up", (D, H)), ("down", (H, D)))):
            g.manual_seed(seed * 100003 + e * 7 + i)
            w = (torch.randn(shape, generator=g, device=dev) * w_scale).to(BF16)
            q, s = bw.quant_fp8_block_128(w) if block else bw.quant_fp8_e4m3(w)
            out["q_" + name].append(q), out["s_" + name].append(s)
    res = {k: torch.stack(v).contiguous() for k, v in out.items()}
    for k in ("s_gate", "s_up", "s_down"):
        res[k] = res[k].to(torch.float32)
    return res


def make_activations(T, D, E, seed, zipf=False):
    """CPU x ~N(0,1) and w_gate ~N(0,0.02^2) in bf16.  zipf: expert popularity ~ Zipf(1.1) produced inside the
    plain API by a constant input feature and a log-rank row of w_gate."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).to(BF16)
    w_gate = (torch.randn(D, E, generator=g) * 0.02).to(BF16)
    if zipf:
        ranks = torch.randperm(E, generator=g).float() + 1.0
        bias = -1.1 * torch.log(ranks)
        x[:, 0] = 1.0
        w_gate[0] = (bias - bias.mean()).to(BF16)
    return x, w_gate


def expert_subset(W, experts):
    """CPU copies of the chosen experts' codes as {expert id: tensor}; scales whole."""
    sub = {}
    for k in ("q_gate", "q_up", "q_down"):
        sub[k] = {int(e): W[k][int(e)].cpu() for e in experts}
    for k in ("s_gate", "s_up", "s_down"):
        sub[k] = W[k].cpu()
    return sub


def combine_on_cpu(y, weights, sort_perm, inverse_idx, T, preweighted=False):
    """The combine of fp8_moe_v3.py:70-73 applied to given result rows (bf16 products, bf16 index_add_);
    preweighted: the rows already are the bf16 products."""
    flat_w = weights.reshape(-1)[sort_perm].to(BF16).unsqueeze(-1)
    out = torch.zeros(T, y.shape[1], dtype=BF16)
    out.index_add_(0, inverse_idx, y if preweighted else (y * flat_w).to(BF16))
    return out
