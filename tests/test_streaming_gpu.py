"""The pre-routed entry points an expert-residency cache uses: expert ids of the whole model, a
device-side id -> slot lookup, experts taken from a pool of resident slots.

The cache here is a stand-in with the interface of the reference's ThreeTierExpertCache
(src/blackwell_moe/runtime/disk_expert_pool.py:89-268: ``gpu``, ``gpu_slots``, ``n_experts``,
``fetch``, ``prefetch_layer``); it keeps every expert "on disk" in host memory and copies the
requested ones into arbitrary free slots, evicting the least recently used."""

from collections import OrderedDict

import pytest
import torch

from helpers import make_inputs, to_cuda

pytestmark = pytest.mark.gpu


class FakeExpertCache:
    def __init__(self, inp, gpu_slots, dev="cuda:0", first_slot=0):
        E, D, H = inp["q_gate"].shape
        self.host = inp
        self.n_experts, self.gpu_slots = E, gpu_slots
        f8 = inp["q_gate"].dtype
        self.gpu = {"gate_q": torch.zeros(gpu_slots, D, H, dtype=torch.uint8, device=dev).view(f8),
                    "up_q": torch.zeros(gpu_slots, D, H, dtype=torch.uint8, device=dev).view(f8),
                    "down_q": torch.zeros(gpu_slots, H, D, dtype=torch.uint8, device=dev).view(f8),
                    "scale_g": torch.ones(gpu_slots, device=dev), "scale_u": torch.ones(gpu_slots, device=dev),
                    "scale_d": torch.ones(gpu_slots, device=dev)}
        self.map = OrderedDict()
        self.free = [(first_slot + 3 * i) % gpu_slots for i in range(gpu_slots)]     # a scrambled slot order
        assert len(set(self.free)) == gpu_slots
        self.prefetched = []

    def prefetch_layer(self, layer_idx):
        self.prefetched.append(layer_idx)

    def fetch(self, layer_idx, expert_ids):
        slots = []
        for e in expert_ids:
            key = (layer_idx, e)
            if key in self.map:
                self.map.move_to_end(key)
            else:
                slot = self.free.pop(0) if self.free else self.map.popitem(last=False)[1]
                for dst, src in (("gate_q", "q_gate"), ("up_q", "q_up"), ("down_q", "q_down"),
                                 ("scale_g", "s_gate"), ("scale_u", "s_up"), ("scale_d", "s_down")):
                    self.gpu[dst][slot].copy_(self.host[src][e])
                self.map[key] = slot
            slots.append(self.map[key])
        return torch.tensor(slots, dtype=torch.int32, device=self.gpu["scale_g"].device)


def test_streaming_forward_over_a_slot_pool_equals_the_resident_forward():
    import blackwell_moe_b200 as bw
    T, D, E, K, H = 48, 256, 16, 2, 128
    inp = make_inputs(T, D, E, K, H, seed=51, keep_bf16=False)
    c = to_cuda(inp)
    full = bw.fp8_moe_forward(c["x"], c["w_gate"], c["q_gate"], c["q_up"], c["q_down"],
                              c["s_gate"], c["s_up"], c["s_down"], top_k=K)
    cache = FakeExpertCache(inp, gpu_slots=20, first_slot=7)           # more slots than experts: nothing is evicted
    out = bw.streaming_moe_forward(c["x"], c["w_gate"], cache, layer_idx=3, top_k=K, prefetch_next_layer=4)
    assert cache.prefetched == [4]
    assert torch.equal(out, full)
    v = bw.moe_stage_views("cuda:0", T, D, H, cache.gpu_slots, K)
    assert int(v["status"][0]) == 0
    # a second batch re-uses resident experts and loads the missing ones into other slots
    x2 = torch.randn(T, D, generator=torch.Generator().manual_seed(52)).to(torch.bfloat16).cuda()
    full2 = bw.fp8_moe_forward(x2, c["w_gate"], c["q_gate"], c["q_up"], c["q_down"],
                               c["s_gate"], c["s_up"], c["s_down"], top_k=K)
    assert torch.equal(bw.streaming_moe_forward(x2, c["w_gate"], cache, layer_idx=3, top_k=K), full2)


def test_fastcache_signature_and_non_resident_experts():
    """remap = -1 for an expert that is not resident: its slots are skipped, BAD_EXPERT is raised, nothing traps."""
    import blackwell_moe_b200 as bw
    T, D, E, K, H = 40, 256, 8, 2, 128
    inp = make_inputs(T, D, E, K, H, seed=53, keep_bf16=False)
    c = to_cuda(inp)
    w, idx = bw.top_k_router(c["x"], c["w_gate"], K)
    perm = torch.tensor([5, 2, 7, 0, 3, 6, 1, 4], dtype=torch.int32, device="cuda:0")      # expert id -> slot
    inv = torch.argsort(perm.long())
    pool = [c[k][inv].contiguous() for k in ("q_gate", "q_up", "q_down", "s_gate", "s_up", "s_down")]
    full = bw.fp8_moe_forward(c["x"], c["w_gate"], c["q_gate"], c["q_up"], c["q_down"],
                              c["s_gate"], c["s_up"], c["s_down"], top_k=K)
    out = bw.fp8_moe_forward_fastcache(c["x"], w, idx, perm, *pool, n_slots=E, top_k=K)
    assert torch.equal(out, full)
    missing = int(idx[0, 0])
    holes = perm.clone()
    holes[missing] = -1
    out2 = bw.fp8_moe_forward_fastcache(c["x"], w, idx, holes, *pool, n_slots=E, top_k=K)
    v = bw.moe_stage_views("cuda:0", T, D, H, E, K)
    assert int(v["status"][0]) & 2, "BAD_EXPERT bit not set"
    assert torch.isfinite(out2.float()).all()
    untouched = ~(idx == missing).any(dim=1)
    assert untouched.any() and torch.isfinite(out2[untouched].float()).all()


def test_block_recipe_routed_form():
    import blackwell_moe_b200 as bw
    import oracle
    g = torch.Generator().manual_seed(54)
    T, D, E, K, H = 64, 256, 8, 2, 256
    x = torch.randn(T, D, generator=g).to(torch.bfloat16).cuda()
    w_gate = (torch.randn(D, E, generator=g) * 0.02).to(torch.bfloat16).cuda()
    q, s = {}, {}
    for name, shape in (("gate", (D, H)), ("up", (D, H)), ("down", (H, D))):
        pairs = [oracle.quant_block_128((torch.randn(shape, generator=g) * 0.02).to(torch.bfloat16)) for _ in range(E)]
        q[name] = torch.stack([p[0] for p in pairs]).cuda()
        s[name] = torch.stack([p[1] for p in pairs]).cuda()
    full = bw.fp8_moe_forward(x, w_gate, q["gate"], q["up"], q["down"], s["gate"], s["up"], s["down"], top_k=K)
    w, idx = bw.top_k_router(x, w_gate, K)
    routed = bw.fp8_moe_forward_routed(x, w, idx, q["gate"], q["up"], q["down"], s["gate"], s["up"], s["down"])
    assert torch.equal(routed, full)
    perm = torch.tensor([3, 0, 6, 1, 7, 2, 5, 4], dtype=torch.int32, device="cuda:0")
    inv = torch.argsort(perm.long())
    remapped = bw.fp8_moe_forward_routed(x, w, idx, q["gate"][inv].contiguous(), q["up"][inv].contiguous(),
                                         q["down"][inv].contiguous(), s["gate"][inv].contiguous(),
                                         s["up"][inv].contiguous(), s["down"][inv].contiguous(), remap=perm)
    # other slots hold the same experts, so rows meet the same weights; the per-token group scales do not
    # depend on the segment a row sits in, hence the result is identical
    assert torch.equal(remapped, full)


def test_forward_on_experts_loaded_from_reference_written_files(golden):
    """Per-expert files written by the reference's save_expert_to_disk -> formats.load_layer_experts ->
    one forward on the GPU, against the reference's own FP8 forward over the same experts."""
    import blackwell_moe_b200 as bw
    import oracle
    from blackwell_moe_b200 import formats
    from conftest import GOLDEN, from_bits
    g = golden("expert_files")
    E, K = g["eg8"].shape[0], int(g["k"])
    W = formats.load_layer_experts(GOLDEN / "expert_files", int(g["layer"]), E, device="cuda:0")
    x, wg = from_bits(g["x"], torch.bfloat16), from_bits(g["wg"], torch.bfloat16)
    out = bw.fp8_moe_forward(x.cuda(), wg.cuda(), *W, top_k=K).cpu()
    assert oracle.rel_l1(out, from_bits(g["y_fp8"], torch.bfloat16)) < 1e-2
