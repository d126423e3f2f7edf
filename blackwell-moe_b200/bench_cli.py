"""``python -m blackwell_moe_b200.bench_cli`` - the reference's ``bwmoe-bench`` on this library.

Same flags, synthetic inputs, protocol and output columns as
src/blackwell_moe/bench/cli.py:24-144 (seed 0, x ~ 0.1 N(0,1), weights ~ 0.02 N(0,1) quantised
per expert, 5 warm-up + 20 timed forwards between synchronisations, tok/s = T / mean, peak MB),
plus ``--shape`` for the named shapes of scripts/bench_matrix.py:15-25.
"""

from __future__ import annotations

import argparse
import time

import torch

SHAPES = {
    "toy_E16": dict(T=256, D=1024, E=16, K=4, H=512),
    "olmoe_1B_7B": dict(T=1024, D=2048, E=64, K=8, H=1024),
    "qwen3_30B_A3B": dict(T=1024, D=2048, E=64, K=8, H=1536),
    "qwen3_moe_57B_14B": dict(T=1024, D=3584, E=64, K=8, H=2560),
    "mixtral_8x7B": dict(T=4096, D=4096, E=8, K=2, H=14336),
    "mixtral_8x22B_prefill": dict(T=512, D=6144, E=8, K=2, H=16384),
    "mixtral_8x22B_decode": dict(T=16, D=6144, E=8, K=2, H=16384),
    "deepseek_v2_lite": dict(T=1024, D=2048, E=64, K=6, H=1408),
    "deepseek_E128": dict(T=2048, D=4096, E=128, K=8, H=2048),
}


def _bench(fn, warmup: int = 5, iters: int = 20):
    torch.cuda.reset_peak_memory_stats()
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(iters):
        fn()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / iters
    return dt * 1000, torch.cuda.max_memory_allocated() / 1e6


def run(T: int, D: int, E: int, K: int, H: int, device: str = "cuda"):
    from . import fp8_moe_forward, quantize_expert_weights
    torch.manual_seed(0)
    x = torch.randn(T, D, device=device, dtype=torch.bfloat16) * 0.1
    w_gate = torch.randn(D, E, device=device, dtype=torch.bfloat16) * 0.02
    stacks = []
    for shape in ((E, D, H), (E, D, H), (E, H, D)):
        w = torch.randn(shape, device=device, dtype=torch.bfloat16) * 0.02
        stacks.append(quantize_expert_weights(w))
        del w
    (g, sg), (u, su), (d, sd) = stacks
    ms, peak = _bench(lambda: fp8_moe_forward(x, w_gate, g, u, d, sg, su, sd, top_k=K))
    print(f"T={T} D={D} E={E} K={K} H={H}")
    print(f"{'variant':<14} {'ms/iter':>10} {'tok/s':>12} {'peak MB':>10}")
    print("-" * 50)
    print(f"{'fp8 (sm_100a)':<14} {ms:>10.3f} {T / ms * 1000:>12.1f} {peak:>10.1f}")
    return ms, peak


def main() -> None:
    p = argparse.ArgumentParser()
    p.add_argument("--tokens", type=int, default=512)
    p.add_argument("--dim", type=int, default=2048)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--hidden", type=int, default=1536)
    p.add_argument("--shape", choices=sorted(SHAPES), help="a named shape of the reference's bench matrix")
    a = p.parse_args()
    if a.shape:
        run(**SHAPES[a.shape])
    else:
        run(a.tokens, a.dim, a.experts, a.topk, a.hidden)


if __name__ == "__main__":
    main()
