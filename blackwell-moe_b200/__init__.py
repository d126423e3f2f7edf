"""B200-native FP8 MoE-block forward behind the reference's Python API.

``fp8_moe_forward`` / ``top_k_router`` keep the signatures of
``blackwell_moe.kernels.fp8_moe.fp8_moe_forward`` and
``blackwell_moe.kernels.routing.top_k_router``; the work is done by
hand-written sm_100a CUDA kernels in ``libbwmoe.so`` reached through a C ABI
(``include/bwmoe.h``).  There is no CPU or PyTorch fallback: if the library is
missing or no B200 is present the calls raise.
"""

from .quant import (FP8_MAX_E4M3, dequant_fp8_e4m3, quant_fp8_block_128, quant_fp8_e4m3, quantize_expert_weights,
                    quantize_expert_weights_block)
from .moe import (
    HostPipeline,
    fp8_moe_forward,
    fp8_moe_forward_fastcache,
    fp8_moe_forward_routed,
    fp8_moe_forward_shared,
    moe_stage_views,
    stack_shared_experts,
    streaming_moe_forward,
    top_k_router,
)
from ._lib import lib, library_path, BwmoeError
from .modules import (FP8MixtralSparseMoeBlock, FP8MoELayer, FP8SharedExpert, fp8_dense_mlp,
                      patch_deepseek_moe_with_store, patch_shared_experts)

# The reference exports the same forward under several version names
# (src/blackwell_moe/__init__.py:14-15); all of them map to the one CUDA path.
fp8_moe_forward_v3 = fp8_moe_forward
fp8_moe_forward_v4 = fp8_moe_forward
fp8_moe_forward_small_e = fp8_moe_forward

__version__ = "0.1.0"

__all__ = [
    "FP8_MAX_E4M3", "BwmoeError", "HostPipeline", "FP8MixtralSparseMoeBlock", "FP8MoELayer", "FP8SharedExpert", "fp8_dense_mlp",
    "patch_deepseek_moe_with_store", "patch_shared_experts", "dequant_fp8_e4m3", "fp8_moe_forward", "fp8_moe_forward_fastcache",
    "fp8_moe_forward_routed", "fp8_moe_forward_shared", "stack_shared_experts", "streaming_moe_forward",
    "fp8_moe_forward_small_e", "fp8_moe_forward_v3", "fp8_moe_forward_v4", "lib", "library_path",
    "moe_stage_views", "quant_fp8_block_128", "quant_fp8_e4m3", "quantize_expert_weights",
    "quantize_expert_weights_block", "top_k_router",
]
