"""128x128 block-scale recipe on the GPU against the CPU restatement (oracle.block).

The reference has no FP8 kernel for this recipe (it dequantises to bf16), so the
FP8 arithmetic itself is pinned only by our own oracle; what the reference does pin -
the meaning of the weight scales, and the bf16 output of its StreamingQwenMoE block on
a block-FP8 checkpoint - is covered by tests/test_oracle_golden.py and by the last test
here.  Bars:
routing, permutation, activation codes and activation scales bit-exact; output
within 1e-2 relative L1 of the block oracle and within ~7 % of the reference's bf16
forward on the dequantised weights (what its Qwen path computes)."""

import pytest
import torch

import oracle
from helpers import BF16, FP8

pytestmark = pytest.mark.gpu


def make_block_inputs(T, D, E, K, H, seed, zipf=False):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).to(BF16)
    w_gate = (torch.randn(D, E, generator=g) * 0.02).to(BF16)
    if zipf:   # expert popularity ~ Zipf(1.1) through a constant input feature, inside the plain API
        ranks = torch.randperm(E, generator=g).float() + 1.0
        bias = -1.1 * torch.log(ranks)
        x[:, 0] = 1.0
        w_gate[0] = (bias - bias.mean()).to(BF16)
    out = dict(x=x, w_gate=w_gate, k=K)
    for name, (a, b) in (("gate", (D, H)), ("up", (D, H)), ("down", (H, D))):
        qs, ss, ws = [], [], []
        for _ in range(E):
            w = (torch.randn(a, b, generator=g) * 0.02).to(BF16)
            q, s = oracle.quant_block_128(w)
            qs.append(q), ss.append(s), ws.append(oracle.dequant_block_128(q, s))
        out["q_" + name], out["inv_" + name], out["deq_" + name] = torch.stack(qs), torch.stack(ss), torch.stack(ws)
    return out


CASES = [(64, 256, 8, 2, 256, False), (300, 512, 16, 4, 384, False), (1, 256, 8, 2, 128, False),
         (130, 2048, 128, 8, 768, True), (96, 384, 6, 3, 144, False), (257, 256, 4, 2, 640, False)]


@pytest.mark.parametrize("T,D,E,K,H,zipf", CASES)
def test_block_forward_vs_oracle(T, D, E, K, H, zipf):
    import blackwell_moe_b200 as bw
    inp = make_block_inputs(T, D, E, K, H, seed=T + H, zipf=zipf)
    c = {k: (v.cuda() if isinstance(v, torch.Tensor) else v) for k, v in inp.items()}
    out = bw.fp8_moe_forward(c["x"], c["w_gate"], c["q_gate"], c["q_up"], c["q_down"],
                             c["inv_gate"], c["inv_up"], c["inv_down"], top_k=K).cpu()
    v = {k: t.cpu() for k, t in bw.moe_stage_views("cuda:0", T, D, H, E, K, block=True).items()}
    inter = {}
    ref = oracle.moe_forward_block_recipe(inp["x"], inp["w_gate"], inp["q_gate"], inp["q_up"], inp["q_down"],
                                          inp["inv_gate"], inp["inv_up"], inp["inv_down"], top_k=K,
                                          intermediates=inter)
    assert int(v["status"][0]) == 0
    assert torch.equal(v["indices"], inter["indices"])
    assert torch.equal(v["offsets"], inter["offsets"])
    assert torch.equal(v["row_slot"].long(), inter["sort_perm"])
    assert torch.equal(v["x_inv"], inter["x_inv"]), "activation group scales differ"
    assert torch.equal(v["xq"].view(torch.uint8), inter["xq"].view(torch.uint8)), "activation codes differ"
    mism = (v["hq"].view(torch.uint8) != inter["hq"].view(torch.uint8)).float().mean().item()
    assert mism < 0.02, f"{mism:.4f} of the h codes differ"
    assert oracle.rel_l1(v["y"], inter["y_perm"]) < 1e-2
    err = oracle.rel_l1(out, ref)
    assert err < 1e-2, err
    routing = (inter["weights"], inter["indices"])
    y_bf16 = oracle.moe_forward_bf16(inp["x"], inp["w_gate"], inp["deq_gate"], inp["deq_up"], inp["deq_down"],
                                     top_k=K, routing=routing)
    assert oracle.rel_l1(out, y_bf16) < 0.075


def test_block_weight_quantiser_matches_oracle():
    import blackwell_moe_b200 as bw
    g = torch.Generator().manual_seed(3)
    w = (torch.randn(2, 200, 300, generator=g) * 0.02).to(BF16)
    q, s = bw.quantize_expert_weights_block(w.cuda())
    for e in range(2):
        qo, so = oracle.quant_block_128(w[e])
        assert torch.equal(s[e].cpu(), so)
        assert torch.equal(q[e].cpu().view(torch.uint8), qo.view(torch.uint8))


def test_block_forward_against_an_output_of_the_reference_module(golden):
    """End to end on a block-FP8 checkpoint in the HF layout: weights through formats.from_hf_block_fp8, the
    CUDA block path, and the result against the fixture written by the reference's own
    StreamingQwenMoE.forward (src/blackwell_moe/runtime/qwen_patch.py:98-134), within the reference's stated
    ~7 % FP8-versus-bf16 relative L1; routing must equal the reference's."""
    import blackwell_moe_b200 as bw
    from blackwell_moe_b200 import formats
    from conftest import from_bits
    g = golden("streaming_qwen")
    E, K = g["gate_proj_q"].shape[0], int(g["k"])
    x, w_gate = from_bits(g["x"], BF16).cuda(), from_bits(g["wg"], BF16).cuda()
    packs = []
    for n in ("gate_proj", "up_proj", "down_proj"):
        q, inv = formats.from_hf_block_fp8([from_bits(g[n + "_q"][e], FP8) for e in range(E)],
                                           [torch.from_numpy(g[n + "_inv"][e]) for e in range(E)])
        packs += [q.cuda(), inv.cuda()]
    qg, ig, qu, iu, qd, idn = packs
    wt, idx = bw.top_k_router(x, w_gate, K)
    assert torch.equal(idx.cpu().long(), torch.from_numpy(g["indices"]).long())
    out = bw.fp8_moe_forward(x, w_gate, qg, qu, qd, ig, iu, idn, top_k=K)
    assert oracle.rel_l1(out.cpu(), from_bits(g["y"], BF16)) < 7e-2


def test_small_batch_tiles_equal_large_batch_tiles():
    """A handful of rows per expert takes the operand-swapped kernel (weights on the M side, 32 tokens on the
    N side); the same rows with fewer, fuller experts' worth of segments per expert count take the 128-row
    tiles.  Products, K order, scale products and rounding points are the same, so codes, group scales and
    result rows must agree bit for bit (ragged segments, an empty expert, H and D not multiples of the tile)."""
    from blackwell_moe_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(9)
    D, H, E_small, E_big = 384, 320, 16, 4
    seg = [0, 37, 37, 70, 96]                                  # rows of experts 0..3 (expert 1 empty)
    M = seg[-1]
    x = (torch.randn(M, D, generator=g)).to(BF16).to(dev)
    st = torch.cuda.current_stream().cuda_stream
    nd, nh = (D + 127) // 128, (H + 127) // 128
    xq, x_inv = torch.empty(M, D, dtype=torch.uint8, device=dev), torch.empty(M, nd, dtype=torch.float32, device=dev)
    _lib.check(lib.bwmoe_gather_quant_group(x.data_ptr(), None, M, D, 1, xq.data_ptr(), x_inv.data_ptr(), st))
    packs = {}
    for name, (a, b) in (("gate", (D, H)), ("up", (D, H)), ("down", (H, D))):
        qs, ss = zip(*[oracle.quant_block_128((torch.randn(a, b, generator=g) * 0.05).to(BF16)) for _ in range(E_small)])
        packs[name] = (torch.stack(qs).to(dev), torch.stack(ss).to(dev))
    results = []
    for E in (E_big, E_small):        # 24 rows per expert: 128-row tiles; 6 rows per expert: 32-token tiles
        offsets = torch.tensor(seg + [M] * (E - 4), dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        hq = torch.full((M, H), 0x7f, dtype=torch.uint8, device=dev)
        h_inv = torch.full((M, nh), -1.0, dtype=torch.float32, device=dev)
        y = torch.full((M, D), float("nan"), dtype=BF16, device=dev)
        (qg, ig), (qu, iu), (qd, idn) = packs["gate"], packs["up"], packs["down"]
        _lib.check(lib.bwmoe_gateup_swiglu_block(xq.data_ptr(), x_inv.data_ptr(), offsets.data_ptr(), qg.data_ptr(),
                                                 qu.data_ptr(), ig.data_ptr(), iu.data_ptr(), M, D, H, E,
                                                 hq.data_ptr(), h_inv.data_ptr(), status.data_ptr(), st))
        _lib.check(lib.bwmoe_down_block(hq.data_ptr(), h_inv.data_ptr(), offsets.data_ptr(), qd.data_ptr(),
                                        idn.data_ptr(), M, D, H, E, y.data_ptr(), status.data_ptr(), st))
        torch.cuda.synchronize()
        assert int(status[0]) == 0
        results.append((hq, h_inv, y))
    (hq_a, inv_a, y_a), (hq_b, inv_b, y_b) = results
    assert torch.equal(hq_a, hq_b)
    assert torch.equal(inv_a, inv_b)
    assert torch.equal(y_a.view(torch.int16), y_b.view(torch.int16))
    assert torch.isfinite(y_a.float()).all()
