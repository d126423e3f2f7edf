"""``python -m blackwell_moe_b200.bench_cli`` - the reference's ``bwmoe-bench`` and bench matrix on this library.

Flags, synthetic inputs and output columns follow src/blackwell_moe/bench/cli.py:38-144 (seed 0,
x ~ 0.1 N(0,1), weights ~ 0.02 N(0,1) quantised per expert matrix, 5 warm-up + 20 timed forwards,
tok/s = T / mean time, peak MB) so that rows can be laid beside the reference's published tables.
``--matrix`` runs the nine shapes of scripts/bench_matrix.py:15-25 and writes
``bench_results/matrix.csv`` with that script's columns (shape, kernel, ms_per_iter,
tokens_per_sec, peak_mb); ``--json`` prints the rows as one JSON document instead of a table.

Variants timed per shape (the reference times its bf16 / v1..v4 / INT4 paths; this library has one
CUDA path, so the variants are ways of calling it):
  fp8_sm100        fp8_moe_forward, one call per iteration
  fp8_sm100_graph  the same call captured once in a CUDA graph and replayed
  fp8_sm100_block  the 128x128 block-scale recipe on the same shape (when D and H are multiples of 128)
"""

from __future__ import annotations

import argparse
import csv
import json
from dataclasses import asdict, dataclass
from pathlib import Path

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
CSV_COLUMNS = ("shape", "kernel", "ms_per_iter", "tokens_per_sec", "peak_mb")


@dataclass
class BenchResult:
    name: str
    mean_ms: float
    tok_per_s: float
    peak_mem_mb: float


def _time_ms(fn, warmup: int, iters: int) -> float:
    """Mean device time of one call, from CUDA events around `iters` back-to-back calls."""
    for _ in range(warmup):
        fn()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / iters


def run(T: int, D: int, E: int, K: int, H: int, device: str = "cuda", warmup: int = 5, iters: int = 20,
        quiet: bool = False) -> list:
    """Time every variant on one shape; returns a list of :class:`BenchResult`."""
    from . import fp8_moe_forward, quantize_expert_weights, quantize_expert_weights_block
    torch.manual_seed(0)
    x = torch.randn(T, D, device=device, dtype=torch.bfloat16) * 0.1
    w_gate = torch.randn(D, E, device=device, dtype=torch.bfloat16) * 0.02
    per_tensor, block = [], []
    want_block = D % 128 == 0 and H % 128 == 0
    for shape in ((E, D, H), (E, D, H), (E, H, D)):
        w = torch.randn(shape, device=device, dtype=torch.bfloat16) * 0.02
        per_tensor.append(quantize_expert_weights(w))
        if want_block:
            block.append(quantize_expert_weights_block(w))
        del w
    variants = {}
    (g, sg), (u, su), (d, sd) = per_tensor
    variants["fp8_sm100"] = lambda: fp8_moe_forward(x, w_gate, g, u, d, sg, su, sd, top_k=K)
    if want_block:
        (bg, ig), (bu, iu), (bd, idn) = block
        variants["fp8_sm100_block"] = lambda: fp8_moe_forward(x, w_gate, bg, bu, bd, ig, iu, idn, top_k=K)
    results = []
    for name, fn in variants.items():
        torch.cuda.reset_peak_memory_stats()
        ms = _time_ms(fn, warmup, iters)
        results.append(BenchResult(name, ms, T / (ms / 1e3), torch.cuda.max_memory_allocated() / 1e6))
        if name == "fp8_sm100":       # the library neither allocates nor synchronises: the call is capturable as is
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                fn()
            torch.cuda.current_stream().wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                fn()
            ms = _time_ms(graph.replay, warmup, iters)
            results.append(BenchResult("fp8_sm100_graph", ms, T / (ms / 1e3), torch.cuda.max_memory_allocated() / 1e6))
            del graph
    if not quiet:
        print(f"\nT={T} D={D} E={E} K={K} H={H}")
        print(f"{'impl':<16} {'ms/iter':>10} {'tok/s':>12} {'peak MB':>10}")
        print("-" * 52)
        for r in results:
            print(f"{r.name:<16} {r.mean_ms:>10.3f} {r.tok_per_s:>12.1f} {r.peak_mem_mb:>10.1f}")
    return results


def matrix_rows(names, runner=run, **kw) -> list:
    """One CSV row (a dict with CSV_COLUMNS keys) per (shape, variant)."""
    rows = []
    for name in names:
        cfg = SHAPES[name]
        for r in runner(cfg["T"], cfg["D"], cfg["E"], cfg["K"], cfg["H"], **kw):
            rows.append({"shape": name, "kernel": r.name, "ms_per_iter": round(r.mean_ms, 3),
                         "tokens_per_sec": round(r.tok_per_s, 1), "peak_mb": round(r.peak_mem_mb, 1)})
    return rows


def write_csv(rows, path) -> Path:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w", newline="") as f:
        w = csv.DictWriter(f, fieldnames=CSV_COLUMNS)
        w.writeheader()
        w.writerows(rows)
    return path


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--tokens", type=int, default=512)
    p.add_argument("--dim", type=int, default=2048)
    p.add_argument("--experts", type=int, default=64)
    p.add_argument("--topk", type=int, default=8)
    p.add_argument("--hidden", type=int, default=1536)
    p.add_argument("--shape", choices=sorted(SHAPES), help="a named shape of the reference's bench matrix")
    p.add_argument("--matrix", action="store_true", help="all named shapes (or --shapes) -> CSV")
    p.add_argument("--shapes", default="", help="comma-separated subset of the named shapes for --matrix")
    p.add_argument("--out", default="bench_results/matrix.csv", help="CSV path of --matrix")
    p.add_argument("--json", action="store_true", help="print the rows as JSON")
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--warmup", type=int, default=5)
    a = p.parse_args(argv)
    kw = dict(warmup=a.warmup, iters=a.iters, quiet=a.json)
    if a.matrix:
        names = [n for n in a.shapes.split(",") if n] or list(SHAPES)
        for n in names:
            if n not in SHAPES:
                p.error(f"unknown shape {n!r}")
        rows = matrix_rows(names, **kw)
        path = write_csv(rows, a.out)
        if a.json:
            print(json.dumps(rows))
        else:
            print(f"\nWrote {path} ({len(rows)} rows)")
        return 0
    cfg = SHAPES[a.shape] if a.shape else dict(T=a.tokens, D=a.dim, E=a.experts, K=a.topk, H=a.hidden)
    results = run(**cfg, **kw)
    if a.json:
        print(json.dumps([asdict(r) for r in results]))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
