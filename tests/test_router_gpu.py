"""Router kernel against the canonical oracle (bit-exact indices) and against the
reference's own outputs stored as fixtures (shapes and tolerances of the
reference's tests/test_router.py:7-33)."""

import numpy as np
import pytest
import torch

import oracle
from conftest import from_bits

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _route(x, w, k):
    import blackwell_moe_b200 as bw
    wt, idx = bw.top_k_router(x.cuda(), w.cuda(), k)
    return wt.cpu(), idx.cpu()


def test_router_matches_reference_fixtures(golden):
    g = golden("router")
    for i in range(int(g["n"])):
        x, w, k = from_bits(g[f"x{i}"], BF16), from_bits(g[f"w{i}"], BF16), int(g[f"k{i}"])
        wt, idx = _route(x, w, k)
        assert np.array_equal(idx.numpy(), g[f"indices{i}"]), "expert indices must match exactly"
        torch.testing.assert_close(wt, torch.from_numpy(g[f"weights{i}"]), rtol=1e-3, atol=1e-4)
        torch.testing.assert_close(wt.sum(-1), torch.ones(wt.shape[0]), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("T,D,E,K", [(1, 4096, 8, 2), (7, 2048, 64, 6), (300, 2048, 128, 8), (2500, 2048, 256, 8),
                                     (33, 1024, 12, 12), (64, 512, 1, 1), (5000, 4096, 8, 2), (129, 272, 200, 32),
                                     (4096, 2048, 64, 6), (3000, 1024, 128, 8), (1500, 512, 24, 4),
                                     (1100, 2048, 256, 8), (2048, 1024, 16, 2), (1024, 320, 40, 8),
                                     (50, 100, 16, 4), (3, 36, 8, 3)])
def test_router_bit_exact_vs_canonical(T, D, E, K):
    g = torch.Generator().manual_seed(T + E)
    x = torch.randn(T, D, generator=g).to(BF16)
    w = (torch.randn(D, E, generator=g) * 0.02).to(BF16)
    wt, idx = _route(x, w, K)
    wr, ir = oracle.router_canonical(x, w, K)
    assert torch.equal(idx, ir)
    torch.testing.assert_close(wt, wr, rtol=1e-3, atol=1e-4)


def test_router_ties_go_to_lower_id_and_near_ties_are_resolved_exactly():
    # exact ties: identical gate columns
    x = torch.randn(64, 256, generator=torch.Generator().manual_seed(1)).to(BF16)
    col = (torch.randn(256, 1, generator=torch.Generator().manual_seed(2)) * 0.02).to(BF16)
    w = col.repeat(1, 16).contiguous()
    _, idx = _route(x, w, 4)
    assert torch.equal(idx, torch.arange(4, dtype=torch.int32).repeat(64, 1))
    # near ties: columns that differ in one low-order element only
    w2 = w.clone()
    w2[7, 3] = (w2[7, 3].float() * 1.01).to(BF16)
    w2[100, 9] = (w2[100, 9].float() * 0.99).to(BF16)
    wt, idx = _route(x, w2, 5)
    wr, ir = oracle.router_canonical(x, w2, 5)
    assert torch.equal(idx, ir)
    # all-zero activations: every logit equal -> experts 0..K-1, uniform weights
    z = torch.zeros(3, 256, dtype=BF16)
    wt, idx = _route(z, w2, 4)
    assert torch.equal(idx, torch.arange(4, dtype=torch.int32).repeat(3, 1))
    torch.testing.assert_close(wt, torch.full((3, 4), 0.25))


def test_tensor_core_router_ties_and_candidate_overflow():
    """Large batch, wide gate: the tensor-core path.  Identical gate columns make every expert
    tie, which overflows the per-token candidate list and must fall back to the exact path;
    a few distinct columns exercise near ties inside the candidate list."""
    T, D, E, K = 1200, 512, 64, 6
    g = torch.Generator().manual_seed(8)
    x = torch.randn(T, D, generator=g).to(BF16)
    col = (torch.randn(D, 1, generator=g) * 0.02).to(BF16)
    w = col.repeat(1, E).contiguous()
    _, idx = _route(x, w, K)
    assert torch.equal(idx, torch.arange(K, dtype=torch.int32).repeat(T, 1))
    w2 = w.clone()
    for e in (3, 17, 40, 41, 63):
        w2[e % D, e] = (w2[e % D, e].float() * 1.02).to(BF16)
        w2[(7 * e) % D, e] = (w2[(7 * e) % D, e].float() * 0.97).to(BF16)
    wt, idx = _route(x, w2, K)
    wr, ir = oracle.router_canonical(x, w2, K)
    assert torch.equal(idx, ir)
    torch.testing.assert_close(wt, wr, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("D", [2048, 4096])
def test_router_one_million_tokens_zero_mismatches(D):
    """Stress of the bit-exactness claim, the tensor-core path above all: 131072 tokens for each of
    E = 8, 64, 128, 256 at this hidden size (1 M tokens over both sizes), every index compared with the
    canonical oracle.  A wrong index would be silent in the block's output, so the count must be zero."""
    import blackwell_moe_b200 as bw
    T, chunk = 131072, 16384
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(900 + D)
    x = torch.randn(T, D, generator=g, device=dev).to(BF16)
    x_cpu = x.cpu()
    for E, K in ((8, 2), (64, 6), (128, 8), (256, 8)):
        w = (torch.randn(D, E, generator=g, device=dev) * 0.02).to(BF16)
        _, idx = bw.top_k_router(x, w, K)
        idx, w_cpu = idx.cpu(), w.cpu()
        bad = 0
        for t0 in range(0, T, chunk):
            _, ref = oracle.router_canonical(x_cpu[t0:t0 + chunk], w_cpu, K)
            bad += int((idx[t0:t0 + chunk] != ref).any(dim=1).sum())
        assert bad == 0, f"{bad} of {T} tokens routed differently at D={D} E={E} K={K}"


def test_wide_hidden_sizes_take_the_simt_router():
    """D = 6144 (Mixtral-8x22B) is beyond what the tensor-core path's trust bound is argued for: the library
    must not ask for tensor-core scratch there, and the selection stays exact."""
    import blackwell_moe_b200 as bw
    T, D, E, K = 2048, 6144, 8, 2
    assert bw.lib().bwmoe_router_scratch_bytes(T, D, E, K) == 0
    assert bw.lib().bwmoe_router_scratch_bytes(T, 4096, 64, K) > 0
    g = torch.Generator().manual_seed(77)
    x = torch.randn(T, D, generator=g).to(BF16)
    w = (torch.randn(D, E, generator=g) * 0.02).to(BF16)
    _, idx = _route(x, w, K)
    _, ref = oracle.router_canonical(x, w, K)
    assert torch.equal(idx, ref)


def test_a_slice_routed_as_the_whole_batch_gets_the_whole_batch_weights():
    """The routing kernels are picked by batch size and agree on the experts, not on the last bits of the fp32
    weights.  A slice routed with as_batch = size of the whole batch must reproduce the whole batch's rows
    bit for bit (what expert parallelism relies on: every rank routes its own tokens)."""
    import blackwell_moe_b200 as bw
    g = torch.Generator().manual_seed(21)
    for (T, D, E, K, part) in ((4096, 4096, 8, 2, 512), (2048, 2048, 64, 6, 64), (1536, 1024, 16, 4, 96)):
        x = torch.randn(T, D, generator=g).to(torch.bfloat16).cuda()
        w = (torch.randn(D, E, generator=g) * 0.02).to(torch.bfloat16).cuda()
        w_all, i_all = bw.top_k_router(x, w, K)
        for s0 in (0, T - part):
            w_s, i_s = bw.top_k_router(x[s0:s0 + part].contiguous(), w, K, as_batch=T)
            assert torch.equal(i_s, i_all[s0:s0 + part])
            assert torch.equal(w_s, w_all[s0:s0 + part])
            w_own, i_own = bw.top_k_router(x[s0:s0 + part].contiguous(), w, K)      # its own kernel: same experts
            assert torch.equal(i_own, i_all[s0:s0 + part])
            torch.testing.assert_close(w_own, w_all[s0:s0 + part], rtol=1e-4, atol=1e-6)
