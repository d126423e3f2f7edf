"""The allocation-free permutation plan (bwmoe_permute_plan_static).

Some callers cannot give the library a scratch buffer because they cannot
allocate device memory where they call from (an allocator callback, a plugin
that only receives its inputs and outputs, a loop that has frozen its memory
pool).  For them the library carries a fixed 64 KiB scratch array of its own.
This test drives that entry point through the C ABI and requires exactly the
results of the regular entry point, three times in a row with different expert
counts and block counts, every call large enough to take the multi-pass plan
that uses the array, so that whatever one call left in the shared array cannot
leak into the next.  The file sorts last on purpose: a run that stops at the first failure
has then already executed every other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _plan(lib, check, fn_static, indices, row_amax, E):
    dev = indices.device
    T, K = indices.shape
    M = T * K
    stream = torch.cuda.current_stream(dev).cuda_stream
    outs = [torch.full((n,), -7, dtype=torch.int32, device=dev) for n in (E + 1, M, M, M)]
    seg_amax = torch.full((E,), -1.0, device=dev)
    status = torch.zeros(4, dtype=torch.int32, device=dev)
    ptrs = [t.data_ptr() for t in outs]
    if fn_static:
        check(lib.bwmoe_permute_plan_static(indices.data_ptr(), row_amax.data_ptr(), T, E, K, *ptrs,
                                            seg_amax.data_ptr(), status.data_ptr(), stream))
    else:
        scratch = torch.empty(lib.bwmoe_plan_scratch_bytes(T, E, K), dtype=torch.uint8, device=dev)
        check(lib.bwmoe_permute_plan(indices.data_ptr(), row_amax.data_ptr(), T, E, K, *ptrs,
                                     seg_amax.data_ptr(), status.data_ptr(), scratch.data_ptr(), stream))
    torch.cuda.synchronize(dev)
    assert int(status[0]) == 0
    return [t.cpu() for t in outs] + [seg_amax.cpu()]


def test_static_scratch_plan_matches_regular_plan_twice():
    import blackwell_moe_b200 as bw
    from blackwell_moe_b200 import _lib
    lib = bw.lib()
    dev = torch.device("cuda:0")
    g = torch.Generator().manual_seed(21)
    # Three calls in a row, each with more than 1024 slots (smaller plans run in one block and never touch
    # the array): 14 blocks x 64 experts, then 3 blocks x 200 experts over the same words, then the first
    # shape again over what the second left behind.
    for T, E, K in ((9000, 64, 6), (3000, 200, 3), (9000, 64, 6)):
        scores = torch.rand(T, E, generator=g)
        indices = scores.topk(K, dim=-1).indices.to(torch.int32).to(dev).contiguous()
        row_amax = torch.rand(T, generator=g).to(dev)
        ref = _plan(lib, _lib.check, False, indices, row_amax, E)
        got = _plan(lib, _lib.check, True, indices, row_amax, E)
        for name, a, b in zip(("offsets", "pos", "row_slot", "row_expert", "seg_amax"), got, ref):
            assert torch.equal(a, b), f"{name} differs between the static-scratch and regular plan"
        # and the plan itself is the stable sort by expert
        flat = indices.cpu().reshape(-1)
        order = torch.sort(flat, stable=True).indices
        assert torch.equal(got[2].long(), order)


def test_static_scratch_plan_rejects_oversized_requests():
    import blackwell_moe_b200 as bw
    from blackwell_moe_b200 import _lib
    lib = bw.lib()
    dev = torch.device("cuda:0")
    dummy = torch.zeros(8, dtype=torch.int32, device=dev)
    rc = lib.bwmoe_permute_plan_static(dummy.data_ptr(), None, 100000, 8, 8, dummy.data_ptr(), dummy.data_ptr(),
                                       dummy.data_ptr(), dummy.data_ptr(), None, dummy.data_ptr(), None)
    assert rc == -4
    msg = _lib.last_error()
    assert "262144" in msg and "bwmoe_permute_plan" in msg
