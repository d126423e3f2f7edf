"""CPU oracle for the FP8 MoE-block forward.  TEST INFRASTRUCTURE ONLY.

This package restates, with plain torch-on-CPU / numpy arithmetic, the
algorithm of the reference's MoE-block forward so that the CUDA kernels can
be checked against it.  It is imported only by the test-suite, by the smoke
check and by the CPU-baseline leg of the benchmark.  Nothing in the shipped
package imports it, and the shipped package has no CPU code path.

Parity pin: every function here is checked against outputs of the reference
package itself (imported unmodified on CPU) that are stored as fixtures
under ``tests/golden`` together with the script that generated them.  The
one exception is the 128x128 block-scale recipe (``oracle.block``): the
reference has no FP8 block-scale GEMM and no test for one, so that part is
"parity unpinned" beyond what the reference does compute for such
checkpoints - ``_dequant_block_fp8`` (pinned bit for bit) and the bf16 block
output of its ``StreamingQwenMoE.forward`` (pinned by a fixture; the FP8
recipe is held to the reference's ~7 % FP8-versus-bf16 bound against it).
"""

from .recipe import (  # noqa: F401
    FP8_MAX,
    quant_fp8_e4m3,
    dequant_fp8_e4m3,
    router_literal,
    router_canonical,
    permutation,
    moe_forward_bf16,
    moe_forward_fp8_recipe,
    shared_expert_fp8,
    rel_l1,
)
from .block import (  # noqa: F401
    quant_block_128,
    dequant_block_128,
    quant_act_group_128,
    moe_forward_block_recipe,
    streaming_qwen_forward,
)
