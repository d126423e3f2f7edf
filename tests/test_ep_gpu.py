"""Expert-parallel forward on 2 GPUs (both transports: NCCL all-to-all and peer memory) against the
single-GPU forward.

Needs two CUDA devices; skipped otherwise.  Every rank builds the same seeded
inputs, keeps its shard of the experts and its slice of the tokens; the
assembled output must equal the single-GPU result over all tokens bit for bit
(same per-expert scales, same row order inside each expert segment)."""

import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import blackwell_moe_b200 as bw
        from blackwell_moe_b200.ep import ExpertParallelMoE
        from helpers import make_inputs
        msgs = []
        # the last two shapes are split into micro-batches (asynchronous, overlapped exchanges)
        cases = [(s, "nccl") for s in ((96, 256, 8, 2, 256, 2048), (33, 512, 16, 4, 384, 2048),
                                       (700, 256, 4, 2, 128, 2048), (700, 256, 4, 2, 128, 100),
                                       (301, 256, 2, 2, 128, 50))]
        # rows stored straight into the owner's memory, results loaded from it (symmetric memory)
        cases += [(s, "peer") for s in ((96, 256, 8, 2, 256, 2048), (33, 512, 16, 4, 384, 2048),
                                        (700, 256, 4, 2, 128, 2048), (301, 256, 2, 2, 128, 2048))]
        # the same, with the result rows loaded by the combine instead of stored by the down projection
        cases += [(s, "peer-pull") for s in ((96, 256, 8, 2, 256, 2048), (700, 256, 4, 2, 128, 2048))]
        for (T, D, E, K, H, min_tok), transport in cases:
            inp = make_inputs(world * T, D, E, K, H, seed=T + E, keep_bf16=False)
            c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in inp.items()}
            el = E // world
            sl = slice(rank * el, (rank + 1) * el)
            ep = ExpertParallelMoE(c["w_gate"], c["q_gate"][sl], c["q_up"][sl], c["q_down"][sl], c["s_gate"][sl],
                                   c["s_up"][sl], c["s_down"][sl], num_experts=E, top_k=K)
            ep.micro_batch_min_tokens = min_tok
            ep.transport = transport.split("-")[0]
            ep.way_back = "pull" if transport.endswith("pull") else "push"       # ("auto" picks by H)
            out = ep.forward(c["x"][rank * T:(rank + 1) * T].contiguous())
            assert int(ep.last_status[0]) == 0
            full = torch.empty(world * T, D, dtype=out.dtype, device=dev)
            dist.all_gather_into_tensor(full, out)
            ref = bw.fp8_moe_forward(c["x"], c["w_gate"], c["q_gate"], c["q_up"], c["q_down"], c["s_gate"], c["s_up"],
                                     c["s_down"], top_k=K)
            if transport.startswith("peer"):
                assert ep._peer, "the peer transport was not set up"
                out2 = ep.forward(c["x"][rank * T:(rank + 1) * T].contiguous())     # buffers are reused
                if not torch.equal(out2, out):
                    msgs.append(f"shape {(T, D, E, K, H)} peer: second step differs")
            if not torch.equal(full, ref):
                msgs.append(f"shape {(T, D, E, K, H, min_tok)} {transport}: max diff {(full.float() - ref.float()).abs().max().item()}")
            host = ep.forward(inp["x"][rank * T:(rank + 1) * T].contiguous().pin_memory())
            if not torch.equal(host, out.cpu()):
                msgs.append(f"shape {(T, D, E, K, H)}: host-buffer path differs")
        # block-scale recipe (per-token group scales travel with the codes), both transports
        from test_block_gpu import make_block_inputs
        for (T, D, E, K, H), transport in [((64, 256, 8, 2, 256), "nccl"), ((64, 256, 8, 2, 256), "peer"),
                                           ((150, 512, 16, 4, 384), "peer"), ((150, 512, 16, 4, 384), "peer-pull")]:
            inp = make_block_inputs(world * T, D, E, K, H, seed=T + H)
            c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in inp.items()}
            el = E // world
            sl = slice(rank * el, (rank + 1) * el)
            ep = ExpertParallelMoE(c["w_gate"], c["q_gate"][sl], c["q_up"][sl], c["q_down"][sl], c["inv_gate"][sl],
                                   c["inv_up"][sl], c["inv_down"][sl], num_experts=E, top_k=K)
            ep.transport = transport.split("-")[0]
            ep.way_back = "pull" if transport.endswith("pull") else "push"
            out = ep.forward(c["x"][rank * T:(rank + 1) * T].contiguous())
            out = ep.forward(c["x"][rank * T:(rank + 1) * T].contiguous())        # second step: buffers reused
            assert int(ep.last_status[0]) == 0
            assert transport == "nccl" or ep._peer, "the peer transport was not set up"
            full = torch.empty(world * T, D, dtype=out.dtype, device=dev)
            dist.all_gather_into_tensor(full, out)
            ref = bw.fp8_moe_forward(c["x"], c["w_gate"], c["q_gate"], c["q_up"], c["q_down"], c["inv_gate"],
                                     c["inv_up"], c["inv_down"], top_k=K)
            if not torch.equal(full, ref):
                msgs.append(f"block shape {(T, D, E, K, H)} {transport}: max diff "
                            f"{(full.float() - ref.float()).abs().max().item()}")
            # the streaming interface: same batches through submit/result, one batch in flight behind
            if transport == "peer":
                pipe = ep.pipeline(max_tokens=T, depth=2)
                xs = [c["x"][rank * T:(rank + 1) * T].contiguous().cpu().pin_memory() for _ in range(3)]
                tickets, got = [], []
                for i, xb in enumerate(xs):
                    tickets.append(pipe.submit(xb))
                    if i >= 1:
                        got.append(pipe.result(tickets[i - 1]).clone())
                got.append(pipe.result(tickets[-1]).clone())
                for y in got:
                    if not torch.equal(y, out.cpu()):
                        msgs.append(f"block shape {(T, D, E, K, H)}: pipeline result differs from forward")
        # ranks bring different numbers of tokens (peer transport, both recipes): capacity agreed collectively
        for recipe in ("tensor", "block"):
            Ts = [96, 40][:world] if world == 2 else [64] * world
            D, E, K, H = 256, 8, 2, 256
            inp = make_block_inputs(sum(Ts), D, E, K, H, seed=77) if recipe == "block" else \
                make_inputs(sum(Ts), D, E, K, H, seed=77, keep_bf16=False)
            c = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in inp.items()}
            names = ("inv_gate", "inv_up", "inv_down") if recipe == "block" else ("s_gate", "s_up", "s_down")
            el = E // world
            sl = slice(rank * el, (rank + 1) * el)
            ep = ExpertParallelMoE(c["w_gate"], c["q_gate"][sl], c["q_up"][sl], c["q_down"][sl], c[names[0]][sl],
                                   c[names[1]][sl], c[names[2]][sl], num_experts=E, top_k=K)
            ep.transport = "peer"
            t0 = sum(Ts[:rank])
            out = ep.forward(c["x"][t0:t0 + Ts[rank]].contiguous())
            assert int(ep.last_status[0]) == 0 and ep._agreed_tokens == max(Ts)
            outs = [torch.empty(t, D, dtype=out.dtype, device=dev) for t in Ts]
            dist.all_gather(outs, out)
            ref = bw.fp8_moe_forward(c["x"], c["w_gate"], c["q_gate"], c["q_up"], c["q_down"], c[names[0]], c[names[1]],
                                     c[names[2]], top_k=K)
            if not torch.equal(torch.cat(outs), ref):
                msgs.append(f"unequal batches, {recipe} recipe: result differs from the single-GPU forward")
        ret[rank] = "ok" if not msgs else "; ".join(msgs)
    except Exception as e:  # noqa: BLE001
        import traceback
        ret[rank] = traceback.format_exc() + repr(e)
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_matches_single_gpu():
    world = 2
    port = _free_port()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        for r in range(world):
            assert ret.get(r) == "ok", f"rank {r}: {ret.get(r)}"
