"""Expert-parallel exchange protocol on CPU: two `gloo` ranks.

The index arithmetic of blackwell_moe_b200.ep (split sizes, regrouping of the
received rows into per-expert segments, the way back) is device-agnostic; here
it moves CPU tensors while the per-expert arithmetic is done by the oracle, and
the assembled result must equal, bit for bit, the oracle's single-process
forward over the concatenated tokens."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp
import torch.nn.functional as F

ROOT = Path(__file__).resolve().parent.parent
WORLD = 2


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, port, fn_name, ret):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        globals()[fn_name](rank)
        ret[rank] = "ok"
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = traceback.format_exc() + repr(e)
    finally:
        dist.destroy_process_group()


def _run(fn_name):
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(port, fn_name, ret), nprocs=WORLD, join=True)
        for r in range(WORLD):
            assert ret.get(r) == "ok", f"rank {r}: {ret.get(r)}"


def _routing(T_per_rank, E, K, seed):
    g = torch.Generator().manual_seed(seed)
    scores = torch.rand(WORLD * T_per_rank, E, generator=g)
    scores[:, 3] -= 10.0                                   # an expert nobody picks
    return scores.topk(K, dim=-1).indices.to(torch.int32)


def _rows_travel_one_expert_per_rank(rank):
    _rows_travel_to_their_experts_and_back(rank, E=WORLD, K=1)


def _rows_travel_to_their_experts_and_back(rank, E=8, K=3):
    import oracle
    from blackwell_moe_b200.ep import ExchangePlan, combine_back, dispatch
    T = 37
    idx_all = _routing(T, E, K, seed=5) if E > 3 else torch.randint(0, E, (WORLD * T, K), generator=torch.Generator().manual_seed(6)).to(torch.int32)
    idx = idx_all[rank * T:(rank + 1) * T]
    sort_perm, _, offsets = oracle.permutation(idx, E)
    # payload: (global slot id, expert) per permuted row
    slot = rank * T * K + sort_perm
    rows = torch.stack([slot.float(), idx.reshape(-1)[sort_perm].float()], dim=1)
    counts = torch.empty(WORLD * E, dtype=torch.int32)
    dist.all_gather_into_tensor(counts, (offsets[1:] - offsets[:-1]).contiguous())
    counts = counts.view(WORLD, E)
    plan = ExchangePlan(counts, rank)
    got = dispatch(rows, plan)
    el = E // WORLD
    # what a single process would hold for my experts: global stable sort by expert
    gperm, _, goff = oracle.permutation(idx_all, E)
    lo, hi = int(goff[rank * el]), int(goff[(rank + 1) * el])
    assert torch.equal(got[:, 0].long(), gperm[lo:hi])
    assert torch.equal(plan.offsets, goff[rank * el:(rank + 1) * el + 1] - lo)
    assert torch.equal(got[:, 1].int() - rank * el, plan.row_expert)
    back = combine_back(got * 2.0, plan, T * K)
    assert torch.equal(back, rows * 2.0)


def _ep_forward_equals_single_process_oracle(rank):
    import oracle
    from blackwell_moe_b200.ep import ExchangePlan, combine_back, dispatch
    from helpers import make_inputs
    T, D, E, K, H = 24, 64, 4, 2, 48
    inp = make_inputs(WORLD * T, D, E, K, H, seed=9, keep_bf16=False)
    ref = oracle.moe_forward_fp8_recipe(inp["x"], inp["w_gate"], inp["q_gate"], inp["q_up"], inp["q_down"],
                                        inp["s_gate"], inp["s_up"], inp["s_down"], top_k=K)
    x = inp["x"][rank * T:(rank + 1) * T]
    weights, indices = oracle.router_canonical(x, inp["w_gate"], K)
    sort_perm, inverse_idx, offsets = oracle.permutation(indices, E)
    x_perm = x[inverse_idx]
    amax = torch.zeros(E)
    for e in range(E):
        seg = x_perm[int(offsets[e]):int(offsets[e + 1])]
        if seg.numel():
            amax[e] = seg.abs().amax().float()
    stats = torch.cat([amax, (offsets[1:] - offsets[:-1]).float()])
    gathered = torch.empty(WORLD * 2 * E)
    dist.all_gather_into_tensor(gathered, stats)
    gathered = gathered.view(WORLD, 2 * E)
    g_amax, counts = gathered[:, :E].amax(0), gathered[:, E:].to(torch.int32)
    scale = (1.0 / g_amax.clamp(min=float(torch.tensor(1e-4).bfloat16()))) * 448.0    # reciprocal * 448
    row_e = indices.reshape(-1)[sort_perm].long()
    xq = (x_perm.float() * scale[row_e].unsqueeze(1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    plan = ExchangePlan(counts, rank)
    xq_local = dispatch(xq.view(torch.uint8), plan).view(torch.float8_e4m3fn)
    el = E // WORLD
    y_local = torch.zeros(plan.rows_local, D, dtype=torch.bfloat16)
    for j in range(el):
        e = rank * el + j
        s, t = int(plan.offsets[j]), int(plan.offsets[j + 1])
        if t <= s:
            continue
        xf = xq_local[s:t].float()
        gate = ((xf @ inp["q_gate"][e].float()) / (scale[e] * inp["s_gate"][e])).bfloat16()
        up = ((xf @ inp["q_up"][e].float()) / (scale[e] * inp["s_up"][e])).bfloat16()
        hq, sh = oracle.quant_fp8_e4m3(F.silu(gate) * up)
        y_local[s:t] = ((hq.float() @ inp["q_down"][e].float()) / (sh * inp["s_down"][e])).bfloat16()
    y_home = combine_back(y_local.view(torch.uint8), plan, T * K).view(torch.bfloat16)   # gloo moves bytes
    flat_w = weights.reshape(-1)[sort_perm].bfloat16().unsqueeze(-1)
    out = torch.zeros(T, D, dtype=torch.bfloat16)
    out.index_add_(0, inverse_idx, (y_home * flat_w).bfloat16())
    assert torch.equal(out, ref[rank * T:(rank + 1) * T])


def _unequal_batches_agree_on_capacity_and_place_rows(rank):
    """Ranks bring different numbers of tokens: the receive-buffer capacity is agreed collectively (largest batch),
    a later batch above it is refused locally before any collective, and the peer-store placement (row
    pos + delta[expert] in the owner's buffer) reproduces the single-process row order."""
    import oracle
    from blackwell_moe_b200.ep import ExpertParallelMoE
    E, K, D, H = 8, 3, 16, 16
    el = E // WORLD
    Ts = [37, 11]
    T = Ts[rank]
    f8 = torch.float8_e4m3fn
    ep = ExpertParallelMoE(torch.zeros(D, E, dtype=torch.bfloat16), torch.zeros(el, D, H).to(f8), torch.zeros(el, D, H).to(f8),
                           torch.zeros(el, H, D).to(f8), torch.ones(el), torch.ones(el), torch.ones(el),
                           num_experts=E, top_k=K)
    cap = ep._agree_on_capacity(T)
    assert cap == WORLD * max(Ts) * K, cap
    assert ep._agree_on_capacity(5) == cap                     # smaller batches later: no collective, same answer
    with pytest.raises(ValueError):
        ep._agree_on_capacity(max(Ts) + 1)
    g = torch.Generator().manual_seed(17)
    idx_all = torch.rand(sum(Ts), E, generator=g).topk(K, dim=-1).indices.to(torch.int32)
    t0 = sum(Ts[:rank])
    idx = idx_all[t0:t0 + T]
    sort_perm, _, offsets = oracle.permutation(idx, E)
    counts = [torch.empty(E, dtype=torch.int32) for _ in range(WORLD)]
    dist.all_gather(counts, (offsets[1:] - offsets[:-1]).contiguous())
    counts = torch.stack(counts)
    delta, offsets_l, home_counts, home_first = ep._peer_maps(counts, offsets)
    pos = torch.empty(T * K, dtype=torch.long)
    pos[sort_perm] = torch.arange(T * K)
    flat = idx.reshape(-1).long()
    dst_rank, dst_row = flat // el, pos + delta[flat].long()
    assert int(dst_row.max()) < cap
    sent = [None] * WORLD
    dist.all_gather_object(sent, (dst_rank.tolist(), dst_row.tolist(), (t0 * K + torch.arange(T * K)).tolist()))
    buf = torch.full((cap,), -1, dtype=torch.long)
    for ranks_, rows_, slots_ in sent:
        for r_, row_, slot_ in zip(ranks_, rows_, slots_):
            if r_ == rank:
                assert buf[row_] == -1, "two rows stored to one place"
                buf[row_] = slot_
    gperm, _, goff = oracle.permutation(idx_all, E)
    lo, hi = int(goff[rank * el]), int(goff[(rank + 1) * el])
    assert torch.equal(buf[:hi - lo], gperm[lo:hi])            # (source rank, source row) order = single-process order
    assert torch.equal(offsets_l.long(), goff[rank * el:(rank + 1) * el + 1].long() - lo)
    # the way home: rows of local expert j that came from rank s return to rows home_first[s, j]... of rank s
    assert torch.equal(home_counts, counts[:, rank * el:(rank + 1) * el])


def test_unequal_batches_agree_on_capacity_and_place_rows():
    _run("_unequal_batches_agree_on_capacity_and_place_rows")


def test_rows_travel_to_their_experts_and_back():
    _run("_rows_travel_to_their_experts_and_back")


def test_rows_travel_with_one_expert_per_rank():
    _run("_rows_travel_one_expert_per_rank")


def test_ep_forward_equals_single_process_oracle():
    _run("_ep_forward_equals_single_process_oracle")
