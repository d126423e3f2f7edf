"""Index maps of the peer-memory expert-parallel step (torch form, used on CPU; the CUDA kernel
bwmoe_ep_maps is checked against the same formulas in tests/test_ep_emulated_gpu.py): every row must get
a distinct place inside its expert's segment on the owner, ordered by (source rank, source row), and the
way home must invert it."""

from types import SimpleNamespace

import pytest
import torch

from blackwell_moe_b200.ep import ExpertParallelMoE


@pytest.mark.parametrize("G,E", [(1, 4), (2, 8), (4, 8), (8, 8), (4, 64), (8, 256)])
def test_peer_maps_place_every_row_once(G, E):
    g = torch.Generator().manual_seed(G * 1000 + E)
    counts = torch.randint(0, 7, (G, E), generator=g, dtype=torch.int32)
    el = E // G
    dev = torch.device("cpu")
    total = counts.sum(0)
    seen = {r: set() for r in range(G)}            # (owner) -> occupied rows
    for rank in range(G):
        offsets = torch.zeros(E + 1, dtype=torch.int32)
        offsets[1:] = torch.cumsum(counts[rank], 0)
        me = SimpleNamespace(world=G, rank=rank, el=el, E=E, dev=dev)
        delta, offsets_l, home_counts, home_first = ExpertParallelMoE._peer_maps(me, counts, offsets)
        assert offsets_l.tolist() == [0] + torch.cumsum(total[rank * el:(rank + 1) * el], 0).tolist()
        for e in range(E):
            owner = e // el
            seg0 = int(total[owner * el:e].sum())
            for j in range(int(counts[rank, e])):
                dst = int(offsets[e]) + j + int(delta[e])
                # inside e's segment, after the rows of the lower ranks, in source order
                assert dst == seg0 + int(counts[:rank, e].sum()) + j
                assert dst not in seen[owner]
                seen[owner].add(dst)
        # the way home of the rows this rank holds
        for s in range(G):
            for jl in range(el):
                e = rank * el + jl
                assert int(home_counts[s, jl]) == int(counts[s, e])
                assert int(home_first[s, jl]) == int(counts[s, :e].sum())
    for owner in range(G):
        assert seen[owner] == set(range(int(total[owner * el:(owner + 1) * el].sum())))
