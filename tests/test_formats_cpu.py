"""Weight-format adapters: the reference's per-expert safetensors files and HF block-FP8 layout."""

import torch

import oracle
from blackwell_moe_b200 import formats

FP8 = torch.float8_e4m3fn


def test_per_expert_files_round_trip(tmp_path):
    g = torch.Generator().manual_seed(2)
    E, D, H = 3, 32, 48
    qs = [(torch.randn(E, a, b, generator=g) * 50).clamp(-448, 448).to(FP8) for a, b in ((D, H), (D, H), (H, D))]
    ss = [torch.rand(E, generator=g) * 100 + 1 for _ in range(3)]
    paths = formats.save_layer_experts(tmp_path, 7, *qs, *ss)
    assert paths[1].name == "expert_L007_E001.safetensors"      # naming of disk_expert_pool.py:47,66
    back = formats.load_layer_experts(tmp_path, 7, E)
    for a, b in zip(qs, back[:3]):
        assert torch.equal(a.view(torch.uint8), b.view(torch.uint8))
    for a, b in zip(ss, back[3:]):
        assert torch.equal(a.float(), b)


def test_hf_block_fp8_transposition_preserves_the_dequantised_weight(golden):
    from conftest import from_bits
    g = golden("block_shared")                                   # w [256,384] = [out,in], s [2,3]
    w, s = from_bits(g["w"], FP8), torch.from_numpy(g["s"])
    codes, inv = formats.from_hf_block_fp8([w, w], [s, s])
    assert codes.shape == (2, 384, 256) and inv.shape == (2, 3, 2)
    deq = oracle.dequant_block_128(codes[1], inv[1])             # [in, out]
    ref = from_bits(g["deq"], torch.bfloat16)                    # reference _dequant_block_fp8, [out, in]
    assert torch.equal(deq.t().contiguous().view(torch.int16), ref.view(torch.int16))


def test_files_written_by_the_reference_load_into_stacked_tensors(golden):
    """tests/golden/expert_files/ was written by the reference's own save_expert_to_disk
    (src/blackwell_moe/runtime/disk_expert_pool.py:38-56); the adapter must return exactly the tensors
    that went in (stored beside the files by the same script)."""
    from conftest import GOLDEN, from_bits
    g = golden("expert_files")
    E = g["eg8"].shape[0]
    got = formats.load_layer_experts(GOLDEN / "expert_files", int(g["layer"]), E)
    for a, key in zip(got[:3], ("eg8", "eu8", "ed8")):
        assert a.dtype == FP8 and torch.equal(a.view(torch.uint8), from_bits(g[key], FP8).view(torch.uint8))
    for a, key in zip(got[3:], ("sg", "su", "sd")):
        assert a.dtype == torch.float32 and torch.equal(a, torch.from_numpy(g[key]))
