"""The peer-memory expert-parallel kernels on ONE GPU: the ranks of a 2- and a 4-rank group are played
one after the other on the same device, their "peer" buffers being ordinary allocations.  Covers
bwmoe_ep_maps, bwmoe_scatter_quant_peers, bwmoe_down_peers (rows stored at home from the GEMM epilogue)
and bwmoe_combine_peers (rows loaded from their owners) without a second device; the assembled output
must equal the single-GPU forward bit for bit."""

import ctypes as C

import pytest
import torch

from helpers import make_inputs

pytestmark = pytest.mark.gpu


def _ptrs(tensors):
    return (C.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _run(world, T, D, E, K, H, push):
    import blackwell_moe_b200 as bw
    from blackwell_moe_b200 import _lib
    lib = _lib.lib()
    dev = torch.device("cuda:0")
    st = torch.cuda.current_stream(dev).cuda_stream
    i32, f32, u8, bf16 = torch.int32, torch.float32, torch.uint8, torch.bfloat16
    inp = make_inputs(world * T, D, E, K, H, seed=T + E + world, keep_bf16=False)
    c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in inp.items()}
    el, M = E // world, T * K
    new = lambda *shape, dtype: torch.empty(shape, dtype=dtype, device=dev)      # noqa: E731
    status = torch.zeros(4, dtype=i32, device=dev)
    ranks = []
    for r in range(world):                      # route and plan every rank's tokens
        x = c["x"][r * T:(r + 1) * T].contiguous()
        w, idx = bw.top_k_router(x, c["w_gate"], K)
        row_amax = x.float().abs().amax(1).contiguous()
        s = dict(x=x, w=w.contiguous(), idx=idx.contiguous(), offsets=new(E + 1, dtype=i32), pos=new(M, dtype=i32),
                 row_slot=new(M, dtype=i32), row_expert=new(M, dtype=i32), amax=new(E, dtype=f32))
        scratch = new(lib.bwmoe_plan_scratch_bytes(T, E, K), dtype=u8)
        _lib.check(lib.bwmoe_permute_plan(s["idx"].data_ptr(), row_amax.data_ptr(), T, E, K, s["offsets"].data_ptr(),
                                          s["pos"].data_ptr(), s["row_slot"].data_ptr(), s["row_expert"].data_ptr(),
                                          s["amax"].data_ptr(), status.data_ptr(), scratch.data_ptr(), st))
        ranks.append(s)
    counts = torch.stack([(s["offsets"][1:] - s["offsets"][:-1]) for s in ranks]).contiguous()       # [G, E]
    amax = torch.stack([s["amax"] for s in ranks]).amax(0).contiguous()
    scale_x = new(E, dtype=f32)
    _lib.check(lib.bwmoe_segment_scales(amax.data_ptr(), None, E, scale_x.data_ptr(), st))
    cap = world * M
    xq_bufs = [new(cap, D, dtype=u8) for _ in range(world)]
    y_bufs = [torch.zeros(cap, D, dtype=bf16, device=dev) for _ in range(world)]
    for r, s in enumerate(ranks):               # maps, then every rank stores its rows at their owners
        s["delta"], s["offsets_l"] = new(E, dtype=i32), new(el + 1, dtype=i32)
        s["home_counts"], s["home_first"] = new(world, el, dtype=i32), new(world, el, dtype=i32)
        _lib.check(lib.bwmoe_ep_maps(counts.data_ptr(), s["offsets"].data_ptr(), world, E, r, s["delta"].data_ptr(),
                                     s["offsets_l"].data_ptr(), s["home_counts"].data_ptr(),
                                     s["home_first"].data_ptr(), st))
        total = counts.sum(0).view(world, el)                                    # the same maps in torch
        seg_start = (torch.cumsum(total, 1) - total).view(E)
        below = counts[:r].sum(0) if r else torch.zeros(E, dtype=torch.int64, device=dev)
        assert torch.equal(s["delta"].long(), seg_start + below - s["offsets"][:E])
        assert torch.equal(s["offsets_l"][1:].long(), torch.cumsum(total[r], 0))
        assert torch.equal(s["home_counts"], counts[:, r * el:(r + 1) * el])
        assert torch.equal(s["home_first"].long(), (torch.cumsum(counts, 1) - counts)[:, r * el:(r + 1) * el])
        _lib.check(lib.bwmoe_scatter_quant_peers(s["x"].data_ptr(), s["pos"].data_ptr(), s["idx"].data_ptr(),
                                                 scale_x.data_ptr(), s["delta"].data_ptr(), T, D, K, el,
                                                 _ptrs(xq_bufs), world, cap, status.data_ptr(), st))
    for r, s in enumerate(ranks):               # every rank's experts; result rows pushed home or kept
        sl = slice(r * el, (r + 1) * el)
        R = int(counts[:, sl].sum())
        if R == 0:
            continue
        sx = scale_x[sl].contiguous()
        amax_h = torch.zeros(el, dtype=f32, device=dev)
        h, hq = new(R, H, dtype=bf16), new(R, H, dtype=u8)
        gs = new(max(256, lib.bwmoe_gemm_scratch_bytes(R, D, H, el)), dtype=u8)
        wg, wu, wd = (c[k][sl].contiguous() for k in ("q_gate", "q_up", "q_down"))
        sg, su, sd = (c[k][sl].contiguous() for k in ("s_gate", "s_up", "s_down"))
        _lib.check(lib.bwmoe_gateup_swiglu(xq_bufs[r].data_ptr(), s["offsets_l"].data_ptr(), sx.data_ptr(),
                                           wg.data_ptr(), wu.data_ptr(), sg.data_ptr(), su.data_ptr(), R, D, H, el,
                                           h.data_ptr(), amax_h.data_ptr(), status.data_ptr(), gs.data_ptr(), st))
        scale_h = new(el, dtype=f32)
        _lib.check(lib.bwmoe_segment_scales(amax_h.data_ptr(), None, el, scale_h.data_ptr(), st))
        seg = (s["offsets_l"][1:] - s["offsets_l"][:-1]).long()
        row_expert_l = torch.repeat_interleave(torch.arange(el, device=dev, dtype=i32), seg, output_size=R)
        _lib.check(lib.bwmoe_requant(h.data_ptr(), row_expert_l.data_ptr(), scale_h.data_ptr(), R, H, hq.data_ptr(), st))
        if push:
            _lib.check(lib.bwmoe_down_peers(hq.data_ptr(), s["offsets_l"].data_ptr(), scale_h.data_ptr(), wd.data_ptr(),
                                            sd.data_ptr(), R, D, H, el, s["home_counts"].data_ptr(),
                                            s["home_first"].data_ptr(), _ptrs(y_bufs), world, status.data_ptr(), st))
        else:
            _lib.check(lib.bwmoe_down(hq.data_ptr(), s["offsets_l"].data_ptr(), scale_h.data_ptr(), wd.data_ptr(),
                                      sd.data_ptr(), R, D, H, el, y_bufs[r].data_ptr(), status.data_ptr(),
                                      gs.data_ptr(), st))
    outs = []
    for r, s in enumerate(ranks):
        out = new(T, D, dtype=bf16)
        if push:
            _lib.check(lib.bwmoe_combine(y_bufs[r].data_ptr(), s["pos"].data_ptr(), s["w"].data_ptr(), T, D, K,
                                         out.data_ptr(), st))
        else:
            _lib.check(lib.bwmoe_combine_peers(_ptrs(y_bufs), world, s["pos"].data_ptr(), s["idx"].data_ptr(),
                                               s["w"].data_ptr(), s["delta"].data_ptr(), el, T, D, K, out.data_ptr(), st))
        outs.append(out)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    ref = bw.fp8_moe_forward(c["x"], c["w_gate"], c["q_gate"], c["q_up"], c["q_down"], c["s_gate"], c["s_up"],
                             c["s_down"], top_k=K)
    assert torch.equal(torch.cat(outs), ref)


@pytest.mark.parametrize("push", [True, False], ids=["push", "pull"])
@pytest.mark.parametrize("world,T,D,E,K,H", [(2, 96, 256, 8, 2, 256), (4, 150, 512, 16, 4, 384), (2, 700, 256, 4, 2, 128),
                                             (8, 40, 256, 8, 2, 128),
                                             (2, 2600, 256, 4, 2, 128)])      # 2600 rows per expert: paired down tiles
def test_peer_kernels_with_ranks_played_on_one_gpu(world, T, D, E, K, H, push):
    _run(world, T, D, E, K, H, push)
