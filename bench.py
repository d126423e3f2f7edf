"""MoE-block forward benchmark (tokens/s) on 1..8 B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--tokens T]
    python bench.py --impl reference ...        # the bf16 CPU path on the host cores

One "step" is one forward of the MoE block over one batch of T synthetic tokens
per GPU.  Default workload: the Mixtral-8x7B-shape block (hidden 4096,
intermediate 14336, 8 experts, top-2, per-tensor E4M3 weights) at T=16384
prefill tokens.  With N > 1 the experts are sharded over the ranks (expert
parallel, all-to-all over NCCL) and every rank brings its own T tokens, so the
job is weak-scaled.  Rank 0 prints ONE JSON line.
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
    # name: (D, H, E, K, default T)
    "mixtral-8x7b": (4096, 14336, 8, 2, 16384),
    "deepseek-v2-lite": (2048, 1408, 64, 6, 4096),
    "toy": (1024, 2048, 16, 2, 256),
    "qwen3-30b-a3b": (2048, 768, 128, 8, 8192),        # 128x128 block-scale weights, Zipf(1.1) expert popularity
    "qwen3.6-35b-a3b": (2048, 512, 256, 8, 32768),     # 128x128 block-scale weights
}
BLOCK_SCALE = {"qwen3-30b-a3b", "qwen3.6-35b-a3b"}
ZIPF = {"qwen3-30b-a3b"}


# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) of one gate+up GEMM launch from the ncu capture
# summarised in profiles/grouped_gemm_mixtral_T2048_ncu_full.md: workload -> (T of the capture, bytes).
NCU_GATEUP_TRAFFIC = {"mixtral-8x7b": (2048, 956.4e6 + 108.8e6)}


def gateup_traffic_bytes(workload, T, D, H, E, K):
    """Measured traffic of the small capture scaled to T tokens: the weight bytes are read once whatever
    T is; the rest (FP8 activations in, bf16 h out) grows in proportion to the rows processed."""
    if workload not in NCU_GATEUP_TRAFFIC:
        return None
    t0, measured = NCU_GATEUP_TRAFFIC[workload]
    weights = 2.0 * E * D * H
    return weights + (measured - weights) * (T / t0)


def kernels_per_forward(M: int, T: int = 0, D: int = 0, E: int = 0, K: int = 0) -> int:
    """Kernels of ours launched by one single-GPU forward (per-tensor recipe) of M = T*K permuted rows."""
    tc_router = T >= 1024 and 8 <= E <= 256 and E % 8 == 0 and K <= 8 and K < E and D % 64 == 0
    router = 4 if tc_router else 1   # transpose, tensor-core logits, refine, all-expert fallback | one SIMT kernel
    if M > 1024:   # + 3 plan passes, segment scales, scatter+quant, gate/up GEMM, requant, down GEMM, combine
        return router + 9
    if M > 64:     # + one-block plan, scatter+quant, gate/up GEMM, requant, down GEMM, combine
        return router + 6
    # split-K: + plan, scatter+quant, gate/up GEMM, slab sum + SwiGLU, requant, down GEMM, slab sum + combine
    return router + 7


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="mixtral-8x7b", choices=sorted(WORKLOADS))
    ap.add_argument("--tokens", type=int, default=0, help="tokens per GPU (default: the workload's prefill size)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--graph", action="store_true",
                    help="one GPU: also time the forward captured once in a CUDA graph and replayed")
    ap.add_argument("--ep-transport", default=None, choices=["auto", "nccl", "peer"],
                    help="expert-parallel exchange (N > 1): NCCL all-to-all or stores/loads over peer memory")
    return ap.parse_args()


# --------------------------------------------------------------------------- inputs
def synth_weights(D, H, E, dev, seed, experts=None, keep_bf16=False, block=False):
    """Random-init weights of the workload's architecture: bf16 ~N(0, 0.02^2), quantised per
    expert matrix to E4M3 (scale 448/amax) exactly as the reference's bench does
    (src/blackwell_moe/bench/cli.py:39-70).  Generated expert by expert on the device."""
    import blackwell_moe_b200 as bw
    experts = range(E) if experts is None else experts
    g = torch.Generator(device=dev)
    out = {"q_gate": [], "q_up": [], "q_down": [], "s_gate": [], "s_up": [], "s_down": []}
    bf = {"gate": [], "up": [], "down": []}
    for e in experts:
        for name, shape in (("gate", (D, H)), ("up", (D, H)), ("down", (H, D))):
            g.manual_seed(seed * 100003 + e * 7 + {"gate": 0, "up": 1, "down": 2}[name])
            w = (torch.randn(shape, generator=g, device=dev) * 0.02).to(torch.bfloat16)
            q, s = bw.quant_fp8_block_128(w) if block else bw.quant_fp8_e4m3(w)
            out["q_" + name].append(q), out["s_" + name].append(s)
            if keep_bf16:
                bf[name].append(w.cpu())
    res = {k: torch.stack(v).contiguous() for k, v in out.items()}
    for k in ("s_gate", "s_up", "s_down"):
        res[k] = res[k].to(torch.float32)
    if keep_bf16:
        res.update({"bf_" + k: torch.stack(v) for k, v in bf.items()})
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
def cpu_bf16_tokens_per_s(D, H, E, K, sample_tokens, steps, warmup, seed=0):
    """The bf16 MoE forward restated from the reference (src/blackwell_moe/kernels/reference.py:9-39)
    on the host cores, on `sample_tokens` tokens of the workload."""
    import oracle
    torch.set_num_threads(os.cpu_count() or 1)
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(sample_tokens, D, generator=g).to(torch.bfloat16)
    w_gate = (torch.randn(D, E, generator=g) * 0.02).to(torch.bfloat16)
    ws = [(torch.randn(E, a, b, generator=g) * 0.02).to(torch.bfloat16) for a, b in ((D, H), (D, H), (H, D))]
    for _ in range(warmup):
        oracle.moe_forward_bf16(x, w_gate, *ws, top_k=K)
    t0 = time.perf_counter()
    for _ in range(steps):
        oracle.moe_forward_bf16(x, w_gate, *ws, top_k=K)
    dt = (time.perf_counter() - t0) / steps
    return sample_tokens / dt, dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    D, H, E, K, T_default = WORKLOADS[args.workload]
    T = args.tokens or T_default
    sample = min(T, 256)
    tps, dt = cpu_bf16_tokens_per_s(D, H, E, K, sample, max(1, args.steps), max(1, min(args.warmup, 2)))
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "MoE-block tokens/s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{args.workload} D={D} H={H} E={E} top_k={K} T={T}"},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                         "sample": f"{sample} of {T} tokens per step, bf16 path restated from reference.py:9-39"},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------- GPU arm
def time_region(fn, steps, stream, flush=None):
    """CUDA-event time of `steps` calls on the current stream, in seconds.  With `flush` (a buffer
    larger than L2) every call is timed on its own and the buffer is rewritten before it, so that
    nothing of the previous call is still L2-resident."""
    if flush is not None:
        total = 0.0
        for i in range(steps):
            flush.fill_(i & 0x7f)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            fn()
            b.record(stream)
            b.synchronize()
            total += a.elapsed_time(b) / 1e3
        return total
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(steps):
        fn()
    stop.record(stream)
    stop.synchronize()
    return start.elapsed_time(stop) / 1e3


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

    D, H, E, K, T_default = WORKLOADS[args.workload]
    T = args.tokens or T_default
    stream = torch.cuda.current_stream(dev)
    block, zipf = args.workload in BLOCK_SCALE, args.workload in ZIPF
    x, w_gate = synth_activations(T, D, E, dev, seed=1234 + rank, zipf=zipf, gate_seed=1234)   # router replicated

    if world == 1:
        W = synth_weights(D, H, E, dev, seed=7, block=block)
        wargs = (w_gate, W["q_gate"], W["q_up"], W["q_down"], W["s_gate"], W["s_up"], W["s_down"])
        step = lambda: bw.fp8_moe_forward(x, *wargs, top_k=K)            # noqa: E731
    else:
        from blackwell_moe_b200.ep import ExpertParallelMoE
        assert E % world == 0, f"E={E} experts do not shard over {world} ranks"
        mine = range(rank * (E // world), (rank + 1) * (E // world))
        W = synth_weights(D, H, E, dev, seed=7, experts=mine, block=block)
        ep = ExpertParallelMoE(w_gate, W["q_gate"], W["q_up"], W["q_down"], W["s_gate"], W["s_up"], W["s_down"],
                               num_experts=E, top_k=K, group=dist.group.WORLD)
        if args.ep_transport:
            ep.transport = args.ep_transport
        step = lambda: ep.forward(x)                                     # noqa: E731

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # L2 hygiene: when one step touches less than ~4x the 126 MB L2 (decode sizes), flush between steps
    # (weights of the experts a step can reach, plus the permuted activation rows it writes and re-reads)
    touched = min(E, T * K) * 3.0 * D * H / world + 3.0 * T * K * D
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev) if touched < 4 * 126e6 else None
    for _ in range(max(3, args.warmup)):
        step()
    barrier()
    with ClockSampler(local) as clocks:
        secs = time_region(step, args.steps, stream, flush)
        barrier()
    if dist is not None:
        t = torch.tensor([secs], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = float(t)
    tokens_total = T * world * args.steps
    value = tokens_total / secs

    # ---- end to end through the public API with host buffers (pinned), copies inside the region ----
    # (a) synchronous call per step: copy in, compute, copy out, wait
    x_host = x.cpu().pin_memory()
    if world == 1:
        e2e_step = lambda: bw.fp8_moe_forward(x_host, *wargs, top_k=K)   # noqa: E731
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
    if world == 1:
        pipe = bw.HostPipeline(*wargs, top_k=K, max_tokens=T, depth=2)
        for _ in range(3):
            pipe.result(pipe.submit(x_host))
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        tickets = []
        for i in range(args.steps):
            tickets.append(pipe.submit(x_host))
            if i >= 1:
                pipe.result(tickets[i - 1])         # the step's result is read on the host
        pipe.result(tickets[-1])
        torch.cuda.synchronize(dev)
        e2e_secs = time.perf_counter() - t0
        e2e_api = "HostPipeline.submit/result, depth 2 (H2D, compute, D2H of neighbouring steps overlap)"
    if dist is not None:
        t = torch.tensor([e2e_secs, e2e_sync_secs], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_secs, e2e_sync_secs = float(t[0]), float(t[1])
    e2e_value = tokens_total / e2e_secs

    if rank != 0:
        if dist is not None:
            dist.destroy_process_group()
        return

    # ---- dominant kernel alone: grouped gate+up GEMM, timed with events on its stream ----
    roofline = None
    if world == 1:
        lib = bw.lib()
        step()
        M = T * K
        ws = bw.moe._workspaces[(dev.index, stream.cuda_stream)]

        def view(sel):
            p, n = C.c_void_p(), C.c_size_t()
            _lib.check(lib.bwmoe_workspace_view(ws.data_ptr(), T, D, H, E, K, sel, C.byref(p), C.byref(n)))
            return p.value
        if block:
            def view(sel):                                                            # noqa: F811
                p, n = C.c_void_p(), C.c_size_t()
                _lib.check(lib.bwmoe_workspace_view_block(ws.data_ptr(), T, D, H, E, K, sel, C.byref(p), C.byref(n)))
                return p.value

            def gateup():
                _lib.check(lib.bwmoe_gateup_swiglu_block(view(8), view(13), view(1), W["q_gate"].data_ptr(),
                                                         W["q_up"].data_ptr(), W["s_gate"].data_ptr(),
                                                         W["s_up"].data_ptr(), M, D, H, E, view(9), view(14), view(0),
                                                         stream.cuda_stream))
            kernel_name = "block_gemm_kernel<GATE_UP>"
        else:
            amax_h = torch.zeros(E, device=dev, dtype=torch.float32)
            scratch = torch.empty(max(256, lib.bwmoe_gemm_scratch_bytes(M, D, H, E)), device=dev, dtype=torch.uint8)

            def gateup():
                _lib.check(lib.bwmoe_gateup_swiglu(view(8), view(1), view(6), W["q_gate"].data_ptr(),
                                                   W["q_up"].data_ptr(), W["s_gate"].data_ptr(), W["s_up"].data_ptr(),
                                                   M, D, H, E, view(10), amax_h.data_ptr(), view(0), scratch.data_ptr(),
                                                   stream.cuda_stream))
            kernel_name = "grouped_gemm_kernel<GATE_UP>"
        for _ in range(3):
            gateup()
        torch.cuda.synchronize(dev)
        k_secs = time_region(gateup, args.steps, stream) / args.steps
        flops = 4.0 * M * D * H
        peaks = {}
        pk = ROOT / "MEASURED_PEAKS.json"
        if pk.exists():
            peaks = json.loads(pk.read_text())
        bf16_sus = peaks.get("bf16_tflops_sustained")
        peak = 2.0 * bf16_sus if bf16_sus else 2.0 * 1400.0
        achieved = flops / k_secs / 1e12
        roofline = {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                    "traffic": gateup_traffic_bytes(args.workload, T, D, H, E, K), "kernel": kernel_name,
                    "kernel_ms": k_secs * 1e3, "flops_per_launch": flops,
                    "peak_basis": ("2 x bf16_tflops_sustained of MEASURED_PEAKS.json (it has no FP8 entry)"
                                   if bf16_sus else "2 x 1400 TFLOP/s fallback (sustained bf16 of the profiling recipe)")}
        # decode sizes stream weights: the same launch against the HBM roofline (gate+up weights of the experts
        # that were selected; the loop above re-reads them from L2 when they fit, so these launches are flushed)
        if M <= 128 * E:      # at most 128 rows per expert on average: the weights, not the math, set the time
            off = bw.moe_stage_views(dev, T, D, H, E, K, block=block)["offsets"].cpu()
            used = int(((off[1:] - off[:-1]) > 0).sum())
            kflush = flush if flush is not None else torch.empty(512 << 20, dtype=torch.uint8, device=dev)
            k_secs = time_region(gateup, args.steps, stream, kflush) / args.steps
            hbm = peaks.get("hbm_gbs")
            wbytes = used * 2.0 * D * H
            roofline = {"bound": "hbm", "achieved": wbytes / k_secs / 1e9, "peak": hbm or 6650.0, "unit": "GB/s",
                        "frac": wbytes / k_secs / 1e9 / (hbm or 6650.0), "traffic": None, "kernel": kernel_name,
                        "kernel_ms": k_secs * 1e3, "bytes_per_launch": wbytes,
                        "peak_basis": ("hbm_gbs of MEASURED_PEAKS.json" if hbm else "6.65 TB/s fallback of the profiling recipe")}

    graph_ms = None
    if world == 1 and args.graph:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            for _ in range(2):
                step()
        stream.wait_stream(side)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize(dev)
        gflush = flush if flush is not None else None
        graph_ms = time_region(g.replay, args.steps, stream, gflush) / args.steps * 1e3

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        sample = min(T, 256)
        tps, dt = cpu_bf16_tokens_per_s(D, H, E, K, sample, steps=3, warmup=1)
        cpu = {"value": tps, "unit": "tokens/s", "cores": os.cpu_count() or 1, "kind": "port",
               "sample": f"{sample} of {T} tokens, 3 timed passes of the bf16 path restated from reference.py:9-39"}

    line = {
        "metric": "MoE-block tokens/s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(3, args.warmup), "ms_per_step": secs / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3", "data": "synthetic",
        "config": {"workload": f"{args.workload} D={D} H={H} E={E} top_k={K} T={T} per GPU",
                   "parallelism": "single GPU" if world == 1 else
                   f"ep{world} (experts sharded, tokens per rank fixed, exchange: "
                   f"{'peer memory' if getattr(ep, '_peer', None) else 'NCCL all-to-all'})",
                   "l2": ("inputs larger than L2 (weights %.0f MB per step)" % (3.0 * E * D * H / world / 1e6)
                          if flush is None else "flushed: a 512 MiB buffer is rewritten before every timed step")},
        "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": T * D * 2 * world,
                "d2h_bytes_per_step": T * D * 2 * world, "ms_per_step": e2e_secs / args.steps * 1e3, "api": e2e_api,
                "sync_call_value": tokens_total / e2e_sync_secs, "sync_call_ms_per_step": e2e_sync_secs / args.steps * 1e3},
        # expert parallel: the same kernels plus one more segment-scale launch (the library's; NCCL's are not counted)
        "gpu_launches": ((9 if block and T * K > 1024 else 6 if block else kernels_per_forward(T * K, T, D, E, K))
                         + (1 if world > 1 and not block else 0)) * args.steps,
        "clocks": clocks.summary(),
    }
    if graph_ms is not None:
        line["graph_ms_per_step"] = graph_ms
    if roofline is not None:
        line["roofline"] = roofline
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    else:
        run_ours(a)
