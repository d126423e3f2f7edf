"""Host-side checks that need no GPU: the shared library loads, exports every
symbol the header declares, sizes workspaces sanely and rejects bad arguments
before touching the device."""

import ctypes as C
import re
from pathlib import Path

import pytest
import torch

import blackwell_moe_b200 as bw
from blackwell_moe_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "bwmoe.h").read_text()
    declared = set(re.findall(r"\b(bwmoe_[a-z_]+)\s*\(", header))
    assert declared, "no declarations found"
    handle = C.CDLL(str(bw.library_path()))
    for name in sorted(declared):
        assert hasattr(handle, name), f"{name} is declared in bwmoe.h but not exported"
    assert declared == set(_lib.SIGNATURES), declared ^ set(_lib.SIGNATURES)
    assert bw.lib().bwmoe_version() == 100


def test_workspace_sizes():
    lib = bw.lib()
    T, D, H, E, K = 256, 1024, 2048, 16, 2
    n = lib.bwmoe_workspace_bytes(T, D, H, E, K)
    M = T * K
    assert n >= M * D + 3 * M * H + 2 * M * D
    assert n < 2 * (M * D + 3 * M * H + 2 * M * D) + (1 << 20)
    assert lib.bwmoe_workspace_bytes_host(T, D, H, E, K) >= n + 4 * T * D
    # bad shapes: 0 bytes, never a crash
    assert lib.bwmoe_workspace_bytes(0, D, H, E, K) == 0
    assert lib.bwmoe_workspace_bytes(T, D + 8, H, E, K) == 0      # D % 16
    assert lib.bwmoe_workspace_bytes(T, D, H, 512, K) == 0        # E > 256
    assert lib.bwmoe_workspace_bytes(T, D, H, 4, 5) == 0          # K > E


def test_errors_are_reported_before_any_device_work():
    lib = bw.lib()
    rc = lib.bwmoe_router(None, None, 0, 16, 8, 2, None, None, None, None, 0, None)
    assert rc == -1 and "router" in _lib.last_error()
    rc = lib.bwmoe_router(None, None, 4, 16, 8, 2, None, None, None, None, 0, None)
    assert rc == -6
    rc = lib.bwmoe_router(None, None, 4, 16, 300, 2, None, None, None, None, 0, None)
    assert rc == -4
    rc = lib.bwmoe_moe_forward(*([None] * 8), 4, 20, 32, 8, 2, None, None, 0, None)
    assert rc == -1
    with pytest.raises(ValueError):
        _lib.check(rc)


def test_python_api_rejects_cpu_weights_and_bad_shapes():
    x = torch.zeros(4, 32, dtype=torch.bfloat16)
    wg = torch.zeros(32, 4, dtype=torch.bfloat16)
    q = torch.zeros(4, 32, 16, dtype=torch.float8_e4m3fn)
    qd = torch.zeros(4, 16, 32, dtype=torch.float8_e4m3fn)
    s = torch.ones(4)
    with pytest.raises(ValueError):
        bw.fp8_moe_forward(x, wg, q, q, qd, s, s, s, top_k=2)     # no CPU path
    with pytest.raises(AssertionError):
        bw.fp8_moe_forward(x, wg, q, q, q, s, s, s, top_k=2)      # down has the wrong shape
    with pytest.raises(ValueError):
        bw.top_k_router(x, wg, 2)


def test_weight_quantiser_matches_oracle():
    import oracle
    g = torch.Generator().manual_seed(5)
    w = (torch.randn(3, 64, 48, generator=g) * 0.02).to(torch.bfloat16)
    q, s = bw.quantize_expert_weights(w)
    for e in range(3):
        qo, so = oracle.quant_fp8_e4m3(w[e])
        assert torch.equal(q[e].view(torch.uint8), qo.view(torch.uint8)) and float(s[e]) == float(so)
