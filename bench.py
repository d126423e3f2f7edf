"""MoE-block forward benchmark (tokens/s) on 1..8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--tokens T]
    python bench.py --impl reference ...        # the bf16 CPU path on the host cores

One "step" is one forward of the MoE block over one batch of T synthetic tokens
per GPU.  Default workload: the Mixtral-8x7B-shape block (hidden 4096,
intermediate 14336, 8 experts, top-2, per-tensor E4M3 weights) at T=16384
prefill tokens.  With N > 1 the experts are sharded over the ranks (expert
parallel) and every rank brings its own T tokens, so the job is weak-scaled.
Rank 0 prints ONE JSON line.  Beside the headline it carries:

  roofline      the gate+up grouped GEMM alone (CUDA events) against the FP8 tensor peak, or the HBM
                peak for decode-sized batches
  sweep         (one GPU) every (configuration, T) pair of the benchmark suite: time, roofline fraction
  extra         (N > 1) the E=256 block-scale shape, expert parallel, at T=32768 and T=128 per rank
  ep_load       (N > 1) rows received per rank in the last step, max over mean: the slowest rank sets the time
  ep_parity     (N > 1) one small expert-parallel step compared bit for bit with the single-GPU forward
  cpu_baseline  the bf16 CPU path on the host cores, same T
"""

from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    # name: (D, H, E, K, default T, shared-expert intermediate)
    "mixtral-8x7b": (4096, 14336, 8, 2, 16384, 0),
    "deepseek-v2-lite": (2048, 1408, 64, 6, 4096, 2816),  # + 2 always-on shared experts (one MLP of 2 x 1408)
    "toy": (1024, 2048, 16, 2, 256, 0),
    "qwen3-30b-a3b": (2048, 768, 128, 8, 8192, 0),        # 128x128 block-scale weights, Zipf(1.1) expert popularity
    "qwen3.6-35b-a3b": (2048, 512, 256, 8, 32768, 0),     # 128x128 block-scale weights
}
BLOCK_SCALE = {"qwen3-30b-a3b", "qwen3.6-35b-a3b"}
ZIPF = {"qwen3-30b-a3b"}
SWEEP = [("mixtral-8x7b", t) for t in (1, 16, 64, 1024, 16384)] + \
        [("deepseek-v2-lite", t) for t in (1, 64, 4096, 16384)] + [("toy", 256)] + \
        [("qwen3-30b-a3b", t) for t in (1, 256, 8192)] + [("qwen3.6-35b-a3b", t) for t in (128, 32768)]
FALLBACK_HBM_GBS, FALLBACK_BF16_TFLOPS = 6650.0, 1590.0          # used only when MEASURED_PEAKS.json is absent


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixtral-8x7b", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="tokens per GPU (default: the workload's prefill size)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true", help="one GPU: skip the sweep over the benchmark configurations")
    ap.add_argument("--no-extra", action="store_true", help="N > 1: skip the E=256 shape and the parity step")
    ap.add_argument("--graph", action="store_true",
                    help="one GPU: also time the forward captured once in a CUDA graph and replayed")
    ap.add_argument("--combine", default=None, choices=["deterministic", "atomic"],
                    help="one GPU: how the weighted combine runs (default: the library's default)")
    ap.add_argument("--ep-transport", default=None, choices=["auto", "nccl", "peer"],
                    help="expert-parallel exchange (N > 1): NCCL all-to-all or stores/loads over peer memory")
    return ap.parse_args()


def peaks():
    pk = ROOT / "MEASURED_PEAKS.json"
    if pk.exists():
        p = json.loads(pk.read_text())
        return {"hbm_gbs": p.get("hbm_gbs", FALLBACK_HBM_GBS), "bf16_tflops": p.get("bf16_tflops", FALLBACK_BF16_TFLOPS),
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained"), "of": "of measured"}
    return {"hbm_gbs": FALLBACK_HBM_GBS, "bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0,
            "of": "of fallback"}


# --------------------------------------------------------------------------- inputs
def synth_weights(D, H, E, dev, seed, experts=None, block=False):
    """Random-init weights of the workload's architecture: bf16 ~N(0, 0.02^2), quantised per
    expert matrix to E4M3 (scale 448/amax) exactly as the reference's bench does
    (src/blackwell_moe/bench/cli.py:39-70), or in 128x128 blocks.  Generated expert by expert on
    the device from per-expert seeds, so that any rank can regenerate any expert."""
    import blackwell_moe_b200 as bw
    experts = range(E) if experts is None else experts
    g = torch.Generator(device=dev)
    out = {"q_gate": [], "q_up": [], "q_down": [], "s_gate": [], "s_up": [], "s_down": []}
    for e in experts:
        for name, shape in (("gate", (D, H)), ("up", (D, H)), ("down", (H, D))):
            g.manual_seed(seed * 100003 + e * 7 + {"gate": 0, "up": 1, "down": 2}[name])
            w = (torch.randn(shape, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            q, s = bw.quant_fp8_block_128(w) if block else bw.quant_fp8_e4m3(w)
            out["q_" + name].append(q), out["s_" + name].append(s)
    res = {k: torch.stack(v).contiguous() for k, v in out.items()}
    for k in ("s_gate", "s_up", "s_down"):
        res[k] = res[k].to(torch.float32)
    return res


def synth_activations(T, D, E, dev, seed, zipf=False, gate_seed=None):
    """x ~ N(0,1) bf16, w_gate ~ N(0, 0.02^2) bf16.  zipf: expert popularity ~ Zipf(1.1) through a
    constant input feature and a log-rank row of w_gate, i.e. inside the plain API."""
    g = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn((T, D), generator=g, device=dev).to(torch.bfloat16)
    g.manual_seed(seed if gate_seed is None else gate_seed)
    w_gate = (torch.randn((D, E), generator=g, device=dev) * 0.02).to(torch.bfloat16)
    if zipf:
        ranks = torch.randperm(E, generator=g, device=dev).float() + 1.0
        bias = -1.1 * torch.log(ranks)
        x[:, 0] = 1.0
        w_gate[0] = (bias - bias.mean()).to(torch.bfloat16)
    return x, w_gate


class Block:
    """One workload resident on one GPU: weights, router, and the forward call a user would make."""

    def __init__(self, workload, dev, combine=None):
        import blackwell_moe_b200 as bw
        self.bw, self.name, self.dev = bw, workload, dev
        self.D, self.H, self.E, self.K, self.T_default, self.Hs = WORKLOADS[workload]
        self.block, self.zipf = workload in BLOCK_SCALE, workload in ZIPF
        self.W = synth_weights(self.D, self.H, self.E, dev, seed=7, block=self.block)
        self.n_shared = 0
        if self.Hs:     # the shared MLP (intermediate n_shared x H) appended as always-on groups of the same pipeline
            S = synth_weights(self.D, self.Hs, 1, dev, seed=11)
            W = self.W
            g, u, d, sg, su, sd, self.n_shared = bw.stack_shared_experts(
                W["q_gate"], W["q_up"], W["q_down"], W["s_gate"], W["s_up"], W["s_down"],
                S["q_gate"][0], S["q_up"][0], S["q_down"][0], S["s_gate"][0], S["s_up"][0], S["s_down"][0])
            self.W = {"q_gate": g, "q_up": u, "q_down": d, "s_gate": sg, "s_up": su, "s_down": sd}
        self.kw = {} if combine is None else {"combine": combine}

    def wargs(self, w_gate):
        W = self.W
        return (w_gate, W["q_gate"], W["q_up"], W["q_down"], W["s_gate"], W["s_up"], W["s_down"])

    def inputs(self, T, seed=1234):
        return synth_activations(T, self.D, self.E, self.dev, seed=seed, zipf=self.zipf, gate_seed=1234)

    def step_fn(self, x, w_gate):
        bw, K, wargs = self.bw, self.K, self.wargs(w_gate)
        if not self.n_shared:
            return lambda: bw.fp8_moe_forward(x, *wargs, top_k=K, **self.kw)
        S = self.n_shared          # the DeepSeek layer: routed and shared experts in one pipeline
        return lambda: bw.fp8_moe_forward_shared(x, *wargs, top_k=K, n_shared=S, routed_scale=1.0)

    def flops(self, T):
        return float(T) * (6.0 * self.K * self.D * self.H + 2.0 * self.D * self.E + 6.0 * self.D * self.Hs)

    def decode_bytes(self, T, used):
        scale_bytes = (3 * 4 * ((self.D + 127) // 128) * ((self.H + 127) // 128)) if self.block else 12
        return used * (3.0 * self.D * self.H + scale_bytes) + 3.0 * self.D * self.Hs + 2.0 * self.D * self.E + \
            4.0 * T * self.D


# --------------------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while a region runs."""

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# --------------------------------------------------------------------------- CPU arm
def cpu_bf16_tokens_per_s(workload, T, steps, warmup, seed=0, budget_s=150.0):
    """The bf16 MoE forward restated from the reference (src/blackwell_moe/kernels/reference.py:9-39) on
    the host cores, on the workload's full batch of T tokens (plus the shared-expert MLP in bf16 where the
    configuration has one).  When (warmup + steps) passes would exceed `budget_s`, fewer passes are timed;
    the batch is never cut.  Returns (tokens/s, seconds per pass, passes timed)."""
    import oracle
    import torch.nn.functional as F
    D, H, E, K, _, Hs = WORKLOADS[workload]
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    w_gate = (torch.randn(D, E, generator=g) * 0.02).to(torch.bfloat16)
    ws = []
    for a, b in ((D, H), (D, H), (H, D)):
        ws.append(torch.stack([(torch.randn(a, b, generator=g) * 0.02).to(torch.bfloat16) for _ in range(E)]))
    sh = [(torch.randn(a, b, generator=g) * 0.02).to(torch.bfloat16) for a, b in ((D, Hs), (D, Hs), (Hs, D))] if Hs else None

    def one():
        out = oracle.moe_forward_bf16(x, w_gate, *ws, top_k=K)
        if sh is not None:
            out = out + (F.silu(x @ sh[0]) * (x @ sh[1])) @ sh[2]
        return out

    t0 = time.perf_counter()
    one()                                                    # first pass: warm-up, and the estimate for the budget
    first = time.perf_counter() - t0
    extra_warm = max(0, warmup - 1) if first * (warmup + steps) < budget_s else 0
    for _ in range(extra_warm):
        one()
    n = max(1, min(steps, int((budget_s - first * (1 + extra_warm)) / max(first, 1e-6))))
    t0 = time.perf_counter()
    for _ in range(n):
        one()
    dt = (time.perf_counter() - t0) / n
    return T / dt, dt, n


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    D, H, E, K, T_default, Hs = WORKLOADS[args.workload]
    T = args.tokens or T_default
    tps, dt, n = cpu_bf16_tokens_per_s(args.workload, T, max(1, args.steps), max(1, args.warmup))
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "MoE-block tokens/s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload} D={D} H={H} E={E} top_k={K} T={T} per GPU"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"all {T} tokens per pass, {n} timed passes of the bf16 path restated from "
                                   "reference.py:9-39 (torch CPU, every host core)"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def time_region(fn, steps, stream, flush=None, each=False):
    """CUDA-event time of `steps` calls on the current stream, in seconds (a list of per-call times with
    `each`).  With `flush` (a buffer larger than L2) every call is timed on its own and the buffer is
    rewritten before it, so that nothing of the previous call is still L2-resident."""
    if flush is not None or each:
        # Everything is queued first and read back after one synchronisation: the flush in front of a call
        # gives the host the time to queue that call, so the events bracket device time even for forwards of
        # a few launches (with a host synchronisation per call the device would wait for the host's launches).
        marks = []
        for i in range(steps):
            if flush is not None:
                flush.fill_(i & 0x7f)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            marks.append((a, b))
        marks[-1][1].synchronize()
        times = [a.elapsed_time(b) / 1e3 for a, b in marks]
        return times if each else sum(times)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop) / 1e3


def measure_fp8_peak(dev, stream, seconds=2.0):
    """Dense FP8 (E4M3) GEMM rate of this GPU from the vendor library (torch._scaled_mm, 8192^3): best of 10
    single launches (burst) and the mean over ~`seconds` of back-to-back launches (sustained, power-capped)."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()          # column-major operand
        one = torch.ones((), device=dev)
        mm = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)    # noqa: E731
        for _ in range(3):
            mm()
        torch.cuda.synchronize(dev)
        burst = min(time_region(mm, 10, stream, each=True))
        flops = 2.0 * n ** 3
        reps = max(10, int(seconds / burst))
        with ClockSampler(dev.index) as clk:
            sustained = time_region(mm, reps, stream) / reps
        return {"fp8_tflops_burst": flops / burst / 1e12, "fp8_tflops_sustained": flops / sustained / 1e12,
                "how": f"torch._scaled_mm e4m3 8192^3, best of 10 / mean of {reps} back to back",
                "sm_mhz_sustained": clk.summary()["sm_mhz"]}
    except Exception as ex:                                                     # noqa: BLE001
        return {"error": repr(ex)[:200]}


def graph_of(step, dev, stream):
    side = torch.cuda.Stream(device=dev)
    side.wait_stream(stream)
    with torch.cuda.stream(side):
        for _ in range(2):
            step()
    stream.wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    for _ in range(2):
        g.replay()
    torch.cuda.synchronize(dev)
    return g


def median(xs):
    s = sorted(xs)
    return s[len(s) // 2]


def sweep_rows(dev, stream, pk, flush, have=None):
    """Every (configuration, T) pair of the benchmark suite on one GPU: median of 10 flushed forwards, the same
    forward replayed as a CUDA graph, and the fraction of the roofline that bounds the pair."""
    rows, blk = [], None
    fp8_peak = 2.0 * pk["bf16_tflops"]
    for workload, T in SWEEP:
        if blk is None or blk.name != workload:
            blk = None
            torch.cuda.empty_cache()
            blk = have if (have is not None and have.name == workload) else Block(workload, dev)
        x, w_gate = blk.inputs(T)
        step = blk.step_fn(x, w_gate)
        # at least 3 forwards; rows of at most 1024 tokens (forwards of 0.1-0.5 ms) also at least 50 ms of them,
        # or they would be timed while the clocks are still coming up from the idle the CPU arm leaves behind
        t0, n_warm = time.perf_counter(), 0
        while n_warm < 3 or (T <= 1024 and time.perf_counter() - t0 < 0.05):
            step()
            n_warm += 1
            if n_warm % 8 == 0:
                torch.cuda.synchronize(dev)
        torch.cuda.synchronize(dev)
        ms = median(time_region(step, 10, stream, flush, each=True)) * 1e3
        g = graph_of(step, dev, stream)
        gms = median(time_region(g.replay, 10, stream, flush, each=True)) * 1e3
        del g
        off = blk.bw.moe_stage_views(dev, T, blk.D, blk.H, blk.E + blk.n_shared, blk.K + blk.n_shared,
                                     block=blk.block)["offsets"]
        used = int(((off[1:blk.E + 1] - off[:blk.E]) > 0).sum())          # routed experts that were selected
        best = min(ms, gms)
        flops, nbytes = blk.flops(T), blk.decode_bytes(T, used)
        t_tensor, t_hbm = flops / (fp8_peak * 1e12), nbytes / (pk["hbm_gbs"] * 1e9)
        row = {"workload": workload, "T": T, "U": used, "ms": round(ms, 4), "graph_ms": round(gms, 4),
               "tflops": round(flops / (best * 1e-3) / 1e12, 1)}
        if t_tensor >= t_hbm:
            row.update(bound="tensor", frac=round(t_tensor / (best * 1e-3), 4),
                       basis=f"FLOP = T(6KDH + 2DE + 6D*H_shared) over the faster of ms / graph_ms; peak 2 x bf16_tflops "
                             f"(burst) = {fp8_peak:.0f} TFLOP/s {pk['of']}")
        else:
            row.update(bound="hbm", frac=round(t_hbm / (best * 1e-3), 4), gbs=round(nbytes / (best * 1e-3) / 1e9, 1),
                       basis=f"bytes = U*3DH + scales + shared + 2DE + 4TD over the faster of ms / graph_ms; peak hbm_gbs = "
                             f"{pk['hbm_gbs']:.0f} GB/s {pk['of']}")
        rows.append(row)
    return rows


def ep_parity_check(workload, tokens, dev, dist, rank, world, transport=None):
    """One small expert-parallel step against the single-GPU forward over the concatenated tokens (rank 0 holds
    every expert for it, regenerated from the per-expert seeds): the outputs must be bit-identical."""
    import blackwell_moe_b200 as bw
    from blackwell_moe_b200.ep import ExpertParallelMoE
    D, H, E, K, _, _ = WORKLOADS[workload]
    block = workload in BLOCK_SCALE
    x, w_gate = synth_activations(tokens, D, E, dev, seed=4321 + rank, zipf=workload in ZIPF, gate_seed=1234)
    mine = range(rank * (E // world), (rank + 1) * (E // world))
    W = synth_weights(D, H, E, dev, seed=7, experts=mine, block=block)
    ep = ExpertParallelMoE(w_gate, W["q_gate"], W["q_up"], W["q_down"], W["s_gate"], W["s_up"], W["s_down"],
                           num_experts=E, top_k=K, group=dist.group.WORLD)
    if transport:
        ep.transport = transport
    out = ep.forward(x)
    xs, outs = [torch.empty_like(x) for _ in range(world)], [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(xs, x)
    dist.all_gather(outs, out)
    res = None
    if rank == 0:
        del W
        Wall = synth_weights(D, H, E, dev, seed=7, block=block)
        ref = bw.fp8_moe_forward(torch.cat(xs), w_gate, Wall["q_gate"], Wall["q_up"], Wall["q_down"],
                                 Wall["s_gate"], Wall["s_up"], Wall["s_down"], top_k=K)
        got = torch.cat(outs)
        res = {"workload": workload, "tokens": tokens * world, "bit_exact": bool(torch.equal(ref, got)),
               "max_abs_diff": float((ref.float() - got.float()).abs().max())}
        del Wall
    del ep
    torch.cuda.empty_cache()
    return res


def run_ours(args):
    import blackwell_moe_b200 as bw
    from blackwell_moe_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run"
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    lib = bw.lib()
    pk = peaks()

    D, H, E, K, T_default, Hs = WORKLOADS[args.workload]
    T = args.tokens or T_default
    stream = torch.cuda.current_stream(dev)
    block, zipf = args.workload in BLOCK_SCALE, args.workload in ZIPF

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(*vals):
        if dist is None:
            return vals
        t = torch.tensor(list(vals), device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return tuple(float(v) for v in t)

    ep_parity = None
    if world > 1 and not args.no_extra:
        ep_parity = [ep_parity_check(args.workload, 512, dev, dist, rank, world, args.ep_transport)]
        if E_ok(world, "qwen3.6-35b-a3b") and args.workload != "qwen3.6-35b-a3b":
            ep_parity.append(ep_parity_check("qwen3.6-35b-a3b", 512, dev, dist, rank, world, args.ep_transport))

    blk = ep = None
    x, w_gate = synth_activations(T, D, E, dev, seed=1234 + rank, zipf=zipf, gate_seed=1234)   # router replicated
    if world == 1:
        blk = Block(args.workload, dev, combine=args.combine)
        W = blk.W
        step = blk.step_fn(x, w_gate)
    else:
        ep, W = make_ep(args.workload, w_gate, dev, dist, rank, world, args.ep_transport)
        step = lambda: ep.forward(x)                                     # noqa: E731

    # L2 hygiene: when one step touches less than ~4x the 126 MB L2 (decode sizes), flush between steps
    # (weights of the experts a step can reach, plus the permuted activation rows it writes and re-reads)
    touched = min(E, T * K) * 3.0 * D * H / world + 3.0 * T * K * D
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev) if touched < 4 * 126e6 else None
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    launches0 = lib.bwmoe_launch_count()
    with ClockSampler(local) as clocks:
        secs = time_region(step, args.steps, stream, flush)
        barrier()
    launches = lib.bwmoe_launch_count() - launches0
    (secs,) = max_over_ranks(secs)
    exchange = None if ep is None else ("peer memory" if getattr(ep, "_peer", None) else "NCCL all-to-all")
    # rows each rank's experts received in the last step: the slowest rank sets the step time
    ep_load = None
    if ep is not None and getattr(ep, "last_counts", None) is not None:
        per_rank = ep.last_counts.sum(0).view(world, -1).sum(1).float()
        ep_load = {"rows_per_rank_max_over_mean": round(float(per_rank.max() / per_rank.mean()), 4)}
    tokens_total = T * world * args.steps
    value = tokens_total / secs

    # ---- end to end through the public API with host buffers (pinned), copies inside the region ----
    # (a) synchronous call per step: copy in, compute, copy out, wait
    x_host = x.cpu().pin_memory()
    if world == 1:
        if not blk.n_shared:
            wargs = blk.wargs(w_gate)
            e2e_step = lambda: bw.fp8_moe_forward(x_host, *wargs, top_k=K)   # noqa: E731
        else:
            def e2e_step():
                xd = x_host.to(dev, non_blocking=True)
                y = blk.step_fn(xd, w_gate)()
                h = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
                h.copy_(y, non_blocking=True)
                stream.synchronize()
                return h
    else:
        e2e_step = lambda: ep.forward(x_host)                            # noqa: E731
    for _ in range(3):
        e2e_step()
    barrier()
    e2e_sync_secs = time_region(e2e_step, args.steps, stream)
    barrier()
    e2e_secs = e2e_sync_secs
    e2e_api = "fp8_moe_forward(x_host) per step" if world == 1 else "ExpertParallelMoE.forward(x_host) per step"
    # (b) the streaming API: the same per-step copies, overlapped with the neighbouring steps' compute
    pipe = None
    if world == 1 and not blk.n_shared:
        pipe = bw.HostPipeline(*blk.wargs(w_gate), top_k=K, max_tokens=T, depth=2)
        e2e_api = "HostPipeline.submit/result, depth 2 (H2D, compute, D2H of neighbouring steps overlap)"
    elif world > 1 and hasattr(ep, "pipeline"):
        pipe = ep.pipeline(max_tokens=T, depth=2)
        e2e_api = "ExpertParallelMoE.pipeline().submit/result, depth 2 (H2D, compute, D2H of neighbouring steps overlap)"
    if pipe is not None:
        for _ in range(3):
            pipe.result(pipe.submit(x_host))
        barrier()
        t0 = time.perf_counter()
        tickets = []
        for i in range(args.steps):
            tickets.append(pipe.submit(x_host))
            if i >= 1:
                pipe.result(tickets[i - 1])         # the step's result is read on the host
        pipe.result(tickets[-1])
        torch.cuda.synchronize(dev)
        e2e_secs = time.perf_counter() - t0
        barrier()
        del pipe
    e2e_secs, e2e_sync_secs = max_over_ranks(e2e_secs, e2e_sync_secs)
    e2e_value = tokens_total / e2e_secs

    # ---- N > 1: the E=256 block-scale shape beside the headline (same ranks, same run) ----
    extra = None
    if world > 1 and not args.no_extra and args.workload != "qwen3.6-35b-a3b" and E_ok(world, "qwen3.6-35b-a3b"):
        del ep, W, step, e2e_step
        torch.cuda.empty_cache()
        extra = []
        name = "qwen3.6-35b-a3b"
        D2, H2, E2, K2, _, _ = WORKLOADS[name]
        for T2 in (32768, 128):
            x2, wg2 = synth_activations(T2, D2, E2, dev, seed=1234 + rank, gate_seed=1234)
            ep2, W2 = make_ep(name, wg2, dev, dist, rank, world, args.ep_transport)
            # the decode batch touches less than L2 holds per rank: flush between its steps
            fl2 = None if T2 > 1024 else (flush if flush is not None else torch.empty(512 << 20, dtype=torch.uint8, device=dev))
            step2 = lambda: ep2.forward(x2)                              # noqa: E731
            for _ in range(3):
                step2()
            barrier()
            s2 = time_region(step2, args.steps, stream, fl2)
            barrier()
            xh2 = x2.cpu().pin_memory()
            api2 = "ExpertParallelMoE.forward(x_host) per step"
            if hasattr(ep2, "pipeline"):
                p2 = ep2.pipeline(max_tokens=T2, depth=2)
                for _ in range(3):
                    p2.result(p2.submit(xh2))
                barrier()
                t0 = time.perf_counter()
                tk = []
                for i in range(args.steps):
                    tk.append(p2.submit(xh2))
                    if i >= 1:
                        p2.result(tk[i - 1])
                p2.result(tk[-1])
                torch.cuda.synchronize(dev)
                e2 = time.perf_counter() - t0
                api2 = "ExpertParallelMoE.pipeline().submit/result, depth 2"
                del p2
            else:
                for _ in range(2):
                    ep2.forward(xh2)
                barrier()
                e2 = time_region(lambda: ep2.forward(xh2), args.steps, stream)
            barrier()
            s2, e2 = max_over_ranks(s2, e2)
            extra.append({"workload": name, "T": T2, "value": T2 * world * args.steps / s2, "unit": "tokens/s",
                          "ms_per_step": s2 / args.steps * 1e3,
                          "e2e": {"value": T2 * world * args.steps / e2, "ms_per_step": e2 / args.steps * 1e3, "api": api2},
                          "exchange": "peer memory" if getattr(ep2, "_peer", None) else "NCCL all-to-all"})
            del ep2, W2, step2
            torch.cuda.empty_cache()

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- dominant kernel alone: grouped gate+up GEMM, timed with events on its stream ----
    roofline = fp8 = None
    if world == 1:
        fp8 = measure_fp8_peak(dev, stream)
        step()
        E, K = E + blk.n_shared, K + blk.n_shared        # the pipeline's own dimensions (always-on groups included)
        M = T * K
        ws = bw.moe._workspaces[(dev.index, stream.cuda_stream)]
        view_fn = lib.bwmoe_workspace_view_block if block else lib.bwmoe_workspace_view

        def view(sel):
            p, n = C.c_void_p(), C.c_size_t()
            _lib.check(view_fn(ws.data_ptr(), T, D, H, E, K, sel, C.byref(p), C.byref(n)))
            return p.value
        if block:
            def gateup():
                _lib.check(lib.bwmoe_gateup_swiglu_block(view(8), view(13), view(1), W["q_gate"].data_ptr(),
                                                         W["q_up"].data_ptr(), W["s_gate"].data_ptr(),
                                                         W["s_up"].data_ptr(), M, D, H, E, view(9), view(14), view(0),
                                                         stream.cuda_stream))
            kernel_name = "block_gemm_kernel<GATE_UP>"
            out_bytes = 1.0 * M * H + 4.0 * M * ((H + 127) // 128)
        else:
            amax_h = torch.zeros(E, device=dev, dtype=torch.float32)
            scratch = torch.empty(max(256, lib.bwmoe_gemm_scratch_bytes(M, D, H, E)), device=dev, dtype=torch.uint8)

            def gateup():
                _lib.check(lib.bwmoe_gateup_swiglu(view(8), view(1), view(6), W["q_gate"].data_ptr(),
                                                   W["q_up"].data_ptr(), W["s_gate"].data_ptr(), W["s_up"].data_ptr(),
                                                   M, D, H, E, view(10), amax_h.data_ptr(), view(0), scratch.data_ptr(),
                                                   stream.cuda_stream))
            kernel_name = "grouped_gemm_kernel<GATE_UP>"
            out_bytes = 2.0 * M * H
        for _ in range(3):
            gateup()
        torch.cuda.synchronize(dev)
        k_secs = time_region(gateup, args.steps, stream) / args.steps
        flops = 4.0 * M * D * H
        off = bw.moe_stage_views(dev, T, D, H, E, K, block=block)["offsets"].cpu()
        used = int(((off[1:] - off[:-1]) > 0).sum())
        algo_bytes = used * 2.0 * D * H + 1.0 * M * D + out_bytes       # weights of the selected experts + rows in + rows out
        peak = 2.0 * pk["bf16_tflops"]
        achieved = flops / k_secs / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": None, "algorithmic_bytes": algo_bytes, "kernel": kernel_name,
                    "kernel_ms": k_secs * 1e3, "flops_per_launch": flops,
                    "peak_basis": f"2 x bf16_tflops (burst: the kernel is timed alone) = {peak:.0f} TFLOP/s {pk['of']}; the "
                                  "peaks file has no FP8 entry and dense FP8 is nominally 2 x bf16"}
        if fp8 and "fp8_tflops_burst" in fp8:
            roofline["frac_of_fp8_scaled_mm_burst"] = achieved / fp8["fp8_tflops_burst"]
            roofline["frac_of_fp8_scaled_mm_sustained"] = achieved / fp8["fp8_tflops_sustained"]
        if pk.get("bf16_tflops_sustained"):
            roofline["frac_of_2x_bf16_sustained"] = achieved / (2.0 * pk["bf16_tflops_sustained"])
        # decode sizes stream weights: the same launch against the HBM roofline (gate+up weights of the experts
        # that were selected; the loop above re-reads them from L2 when they fit, so these launches are flushed)
        if M <= 128 * E:      # at most 128 rows per expert on average: the weights, not the math, set the time
            kflush = flush if flush is not None else torch.empty(512 << 20, dtype=torch.uint8, device=dev)
            k_secs = time_region(gateup, args.steps, stream, kflush) / args.steps
            hbm = pk["hbm_gbs"]
            wbytes = used * 2.0 * D * H
            roofline = {"bound": "hbm", "achieved": wbytes / k_secs / 1e9, "peak": hbm, "unit": "GB/s",
                        "frac": wbytes / k_secs / 1e9 / hbm, "traffic": None, "algorithmic_bytes": wbytes,
                        "kernel": kernel_name, "kernel_ms": k_secs * 1e3, "bytes_per_launch": wbytes,
                        "peak_basis": f"hbm_gbs = {hbm:.0f} GB/s {pk['of']}"}

    if world == 1:
        E, K = E - blk.n_shared, K - blk.n_shared
    graph_ms = None
    if world == 1 and args.graph:
        g = graph_of(step, dev, stream)
        graph_ms = median(time_region(g.replay, args.steps, stream, flush, each=True)) * 1e3
        del g

    sweep = None
    if world == 1 and not args.no_sweep:
        sflush = flush if flush is not None else torch.empty(512 << 20, dtype=torch.uint8, device=dev)
        sweep = sweep_rows(dev, stream, pk, sflush, have=blk)

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        tps, dt, n = cpu_bf16_tokens_per_s(args.workload, T, steps=2, warmup=1, budget_s=60.0)
        cpu = {"value": tps, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
               "sample": f"all {T} tokens, {n} timed passes ({dt:.2f} s each) of the bf16 path restated from reference.py:9-39"}

    line = {
        "metric": "MoE-block tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": f"{args.workload} D={D} H={H} E={E} top_k={K} T={T} per GPU"
                               + (f" + shared experts H_s={Hs}" if Hs else ""),
                   "parallelism": "single GPU" if world == 1 else
                   f"ep{world} (experts sharded, tokens per rank fixed, exchange: "
                   f"{exchange})",
                   "l2": ("inputs larger than L2 (weights %.0f MB per step)" % (3.0 * E * D * H / world / 1e6)
                          if flush is None else "flushed: a 512 MiB buffer is rewritten before every timed step")},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": T * D * 2 * world,
                "d2h_bytes_per_step": T * D * 2 * world, "ms_per_step": e2e_secs / args.steps * 1e3, "api": e2e_api,
                "sync_call_value": tokens_total / e2e_sync_secs, "sync_call_ms_per_step": e2e_sync_secs / args.steps * 1e3},
        # counted by the library itself (bwmoe_launch_count) around the timed region of `value`, on rank 0
        "gpu_launches": int(launches),
        "clocks": clocks.summary(),
    }
    if graph_ms is not None:
        line["graph_ms_per_step"] = graph_ms
    if roofline is not None:
        line["roofline"] = roofline
    if fp8 is not None:
        line["fp8_peak_measured"] = fp8
    if cpu is not None:
        line["cpu_baseline"] = cpu
    if sweep is not None:
        line["sweep"] = sweep
    if extra is not None:
        line["extra"] = extra
    if ep_load is not None:
        line["ep_load"] = ep_load
    if ep_parity is not None:
        line["ep_parity"] = {"bit_exact": all(p["bit_exact"] for p in ep_parity), "tokens": sum(p["tokens"] for p in ep_parity),
                             "cases": ep_parity}
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def E_ok(world, workload):
    return WORKLOADS[workload][2] % world == 0


def make_ep(workload, w_gate, dev, dist, rank, world, transport):
    from blackwell_moe_b200.ep import ExpertParallelMoE
    D, H, E, K, _, _ = WORKLOADS[workload]
    assert E % world == 0, f"E={E} experts do not shard over {world} ranks"
    mine = range(rank * (E // world), (rank + 1) * (E // world))
    W = synth_weights(D, H, E, dev, seed=7, experts=mine, block=workload in BLOCK_SCALE)
    ep = ExpertParallelMoE(w_gate, W["q_gate"], W["q_up"], W["q_down"], W["s_gate"], W["s_up"], W["s_down"],
                           num_experts=E, top_k=K, group=dist.group.WORLD)
    if transport:
        ep.transport = transport
    return ep, W


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
