"""Generate the golden fixtures in this directory from the reference package.

Run once, on a machine where the reference checkout is available:

    REFERENCE_SRC=/path/to/blackwell-moe/src python tests/golden/make_golden.py

The reference is imported unmodified and executed on CPU; inputs and outputs
are stored bit-exactly (bf16 as uint16, e4m3 as uint8) in ``*.npz`` files so
that the tests never need the reference checkout.  Nothing at test or run
time imports this script.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

sys.dont_write_bytecode = True
REF = os.environ.get("REFERENCE_SRC")          # the `src` directory of a blackwell-moe checkout
if not REF:
    sys.exit("set REFERENCE_SRC to the src/ directory of the reference checkout")
sys.path.insert(0, REF)
OUT = Path(__file__).resolve().parent


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    if t.dtype == torch.float8_e4m3fn:
        return t.contiguous().view(torch.uint8).numpy()
    return t.contiguous().numpy()


def gen(seed: int):
    return torch.Generator().manual_seed(seed)


def router_cases():
    from blackwell_moe.kernels.routing import top_k_router_ref
    out = {}
    # shapes of tests/test_router.py:7 and tests/test_correctness.py:13-14
    for i, (T, D, E, K) in enumerate([(32, 256, 8, 2), (128, 512, 16, 4), (64, 256, 16, 4), (48, 384, 64, 6)]):
        g = gen(100 + i)
        x = torch.randn(T, D, generator=g).to(torch.bfloat16)
        w = (torch.randn(D, E, generator=g) * 0.05).to(torch.bfloat16)
        wt, idx = top_k_router_ref(x, w, K)
        out.update({f"x{i}": bits(x), f"w{i}": bits(w), f"weights{i}": wt.numpy(), f"indices{i}": idx.numpy(),
                    f"k{i}": np.int32(K)})
    out["n"] = np.int32(4)
    np.savez_compressed(OUT / "router.npz", **out)


def quant_cases():
    from blackwell_moe.kernels.fp8_quant import quant_fp8_e4m3, dequant_fp8_e4m3
    from blackwell_moe.kernels.fp8_moe import to_fp8_e4m3
    from blackwell_moe.kernels.permute import permute_tokens
    g = gen(200)
    x = (torch.randn(64, 256, generator=g) * 0.2).to(torch.bfloat16)
    q, s = quant_fp8_e4m3(x)
    q2, s2 = to_fp8_e4m3(x)
    assert torch.equal(q.view(torch.uint8), q2.view(torch.uint8)) and float(s) == float(s2)
    dq = dequant_fp8_e4m3(q, s)
    tiny = torch.full((4, 16), 1e-6).to(torch.bfloat16)          # exercises the 1e-4 amax clamp
    qt, st = quant_fp8_e4m3(tiny)
    ids = torch.randint(0, 16, (96 * 4,), generator=g).to(torch.int32)
    xp = torch.randn(96, 32, generator=g).to(torch.bfloat16)
    x_perm, offsets, inverse_idx = permute_tokens(xp, ids, 16)
    np.savez_compressed(OUT / "quant_permute.npz", x=bits(x), q=bits(q), scale=s.numpy(), dq=bits(dq),
                        tiny=bits(tiny), qt=bits(qt), st=st.numpy(),
                        ids=ids.numpy(), xp=bits(xp), x_perm=bits(x_perm), offsets=offsets.numpy(),
                        inverse_idx=inverse_idx.numpy())


def forward_cases():
    from blackwell_moe.kernels.reference import moe_forward_bf16
    from blackwell_moe.kernels.fp8_quant import quant_fp8_e4m3
    from blackwell_moe.kernels.fp8_moe_torch import fp8_moe_forward_torch
    # (T, D, E, K, H): scripts/verify_v3.py:12 shape, and a top-6 / non-power-of-two-H shape
    for name, (T, D, E, K, H), xs in [("fwd_a", (64, 256, 8, 2, 128), 1.0), ("fwd_b", (40, 128, 12, 6, 176), 0.1)]:
        g = gen(300 + len(name) + T)
        x = (torch.randn(T, D, generator=g) * xs).to(torch.bfloat16)
        wg = (torch.randn(D, E, generator=g) * 0.02).to(torch.bfloat16)
        eg = (torch.randn(E, D, H, generator=g) * 0.02).to(torch.bfloat16)
        eu = (torch.randn(E, D, H, generator=g) * 0.02).to(torch.bfloat16)
        ed = (torch.randn(E, H, D, generator=g) * 0.02).to(torch.bfloat16)
        y_bf16 = moe_forward_bf16(x, wg, eg, eu, ed, K)
        qs = [[quant_fp8_e4m3(w[i]) for i in range(E)] for w in (eg, eu, ed)]
        eg8, eu8, ed8 = (torch.stack([q for q, _ in row]) for row in qs)
        sg, su, sd = (torch.stack([s for _, s in row]) for row in qs)
        y_fp8 = fp8_moe_forward_torch(x, wg, eg8, eu8, ed8, sg, su, sd, K)
        np.savez_compressed(OUT / f"{name}.npz", x=bits(x), wg=bits(wg), eg=bits(eg), eu=bits(eu), ed=bits(ed),
                            eg8=bits(eg8), eu8=bits(eu8), ed8=bits(ed8), sg=sg.numpy(), su=su.numpy(),
                            sd=sd.numpy(), y_bf16=bits(y_bf16), y_fp8=bits(y_fp8), k=np.int32(K))


def block_and_shared_cases():
    from blackwell_moe.runtime.qwen_patch import _dequant_block_fp8
    from blackwell_moe.runtime.shared_expert_fp8 import FP8SharedExpert
    g = gen(400)
    w = (torch.randn(256, 384, generator=g) * 0.5).clamp(-448, 448).to(torch.float8_e4m3fn)
    s = (torch.rand(2, 3, generator=g) * 1e-3 + 1e-4).to(torch.float32)
    deq = _dequant_block_fp8(w, s)
    w2 = (torch.randn(200, 130, generator=g) * 0.5).to(torch.float8_e4m3fn)      # ragged edges
    s2 = (torch.rand(2, 2, generator=g) * 1e-3 + 1e-4).to(torch.float32)
    deq2 = _dequant_block_fp8(w2, s2)

    D, Hs, T = 128, 192, 24

    class MLP(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.gate_proj = torch.nn.Linear(D, Hs, bias=False)
            self.up_proj = torch.nn.Linear(D, Hs, bias=False)
            self.down_proj = torch.nn.Linear(Hs, D, bias=False)

    torch.manual_seed(401)
    mlp = MLP()
    with torch.no_grad():
        for p in mlp.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    sh = FP8SharedExpert(mlp)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    y = sh(x)
    np.savez_compressed(
        OUT / "block_shared.npz", w=bits(w), s=s.numpy(), deq=bits(deq), w2=bits(w2), s2=s2.numpy(), deq2=bits(deq2),
        sx=bits(x), sy=bits(y),
        s_wg=bits(sh.w_gate.contiguous()), s_wu=bits(sh.w_up.contiguous()), s_wd=bits(sh.w_down.contiguous()),
        s_sg=sh.s_gate.numpy(), s_su=sh.s_up.numpy(), s_sd=sh.s_down.numpy())


def expert_file_cases():
    """Per-expert files written by the reference's own save_expert_to_disk
    (src/blackwell_moe/runtime/disk_expert_pool.py:38-56), with the tensors that went in and the
    reference's FP8 forward over them, for the weight-format adapter tests."""
    from blackwell_moe.runtime.disk_expert_pool import save_expert_to_disk
    from blackwell_moe.kernels.fp8_quant import quant_fp8_e4m3
    from blackwell_moe.kernels.fp8_moe_torch import fp8_moe_forward_torch
    T, D, E, K, H, layer = 48, 128, 4, 2, 96, 2
    g = gen(500)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    wg = (torch.randn(D, E, generator=g) * 0.02).to(torch.bfloat16)
    qs = {"g": [], "u": [], "d": []}
    ss = {"g": [], "u": [], "d": []}
    root = OUT / "expert_files"
    for e in range(E):
        for key, shape in (("g", (D, H)), ("u", (D, H)), ("d", (H, D))):
            q, s = quant_fp8_e4m3((torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16))
            qs[key].append(q), ss[key].append(s)
        save_expert_to_disk(root, layer, e, qs["g"][e], qs["u"][e], qs["d"][e], ss["g"][e], ss["u"][e], ss["d"][e])
    stack = lambda xs: torch.stack(xs)                                          # noqa: E731
    eg8, eu8, ed8 = stack(qs["g"]), stack(qs["u"]), stack(qs["d"])
    sg, su, sd = stack(ss["g"]), stack(ss["u"]), stack(ss["d"])
    y_fp8 = fp8_moe_forward_torch(x, wg, eg8, eu8, ed8, sg, su, sd, K)
    np.savez_compressed(OUT / "expert_files.npz", x=bits(x), wg=bits(wg), eg8=bits(eg8), eu8=bits(eu8), ed8=bits(ed8),
                        sg=sg.numpy(), su=su.numpy(), sd=sd.numpy(), y_fp8=bits(y_fp8), k=np.int32(K),
                        layer=np.int32(layer))


def streaming_qwen_case():
    """The reference's block-FP8 MoE block itself: StreamingQwenMoE.forward
    (src/blackwell_moe/runtime/qwen_patch.py:98-134) run unmodified on CPU.  The module asks its reader
    for an expert's raw FP8 weights and 128x128 inverse scales, dequantises them to bf16 and applies
    F.linear per expert; here the reader serves seeded tensors from memory, the gate is the reference's
    own top_k_router_ref, and the shared expert contributes zero.  Stored: inputs, HF-layout weights
    ([out, in] codes, [out/128, in/128] scales), routing, and the block output."""
    from blackwell_moe.kernels.routing import top_k_router_ref
    from blackwell_moe.runtime.qwen_patch import StreamingQwenMoE
    T, D, E, K, H = 96, 256, 16, 4, 384
    g = gen(600)
    x = torch.randn(T, D, generator=g).to(torch.bfloat16)
    w_gate = (torch.randn(D, E, generator=g) * 0.05).to(torch.bfloat16)

    def block_quant(w):                        # [out, in] bf16 -> HF block FP8 (codes, weight_scale_inv)
        o, i = w.shape
        wf = w.float().view(o // 128, 128, i // 128, 128)
        inv = (wf.abs().amax(dim=(1, 3)).clamp(min=1e-4) / 448.0).to(torch.float32)
        q = (wf / inv[:, None, :, None]).clamp(-448, 448).view(o, i).to(torch.float8_e4m3fn)
        return q, inv

    store = {}
    for e in range(E):
        store[e] = {
            "gate_proj": block_quant((torch.randn(H, D, generator=g) * 0.02).to(torch.bfloat16)),
            "up_proj": block_quant((torch.randn(H, D, generator=g) * 0.02).to(torch.bfloat16)),
            "down_proj": block_quant((torch.randn(D, H, generator=g) * 0.02).to(torch.bfloat16)),
        }

    class Reader:
        def load_expert_fp8(self, expert_id, device="cuda"):
            return store[int(expert_id)]

    class Gate(torch.nn.Module):
        def forward(self, h):
            weights, indices = top_k_router_ref(h, w_gate, K)
            return None, weights, indices.long()

    class Zero(torch.nn.Module):
        def __init__(self, width):
            super().__init__()
            self.width = width

        def forward(self, h):
            return torch.zeros(h.shape[0], self.width, dtype=h.dtype)

    class Experts:
        num_experts, hidden_dim = E, D

    class Original(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.gate, self.shared_expert, self.shared_expert_gate = Gate(), Zero(D), Zero(1)
            self.experts = Experts()

    block = StreamingQwenMoE(Original(), layer_idx=0, reader=Reader(), cache_size=E)
    with torch.no_grad():
        y = block(x.view(1, T, D)).view(T, D)
        weights, indices = top_k_router_ref(x, w_gate, K)
    out = dict(x=bits(x), wg=bits(w_gate), y=bits(y), weights=weights.numpy(), indices=indices.numpy().astype(np.int32),
               k=np.int32(K))
    for name in ("gate_proj", "up_proj", "down_proj"):
        out[name + "_q"] = np.stack([bits(store[e][name][0]) for e in range(E)])
        out[name + "_inv"] = np.stack([store[e][name][1].numpy() for e in range(E)])
    np.savez_compressed(OUT / "streaming_qwen.npz", **out)


if __name__ == "__main__":
    import blackwell_moe
    print("reference version", blackwell_moe.__version__, "torch", torch.__version__)
    router_cases()
    quant_cases()
    forward_cases()
    block_and_shared_cases()
    expert_file_cases()
    streaming_qwen_case()
    for f in sorted(OUT.glob("*.npz")):
        print(f.name, f.stat().st_size)
