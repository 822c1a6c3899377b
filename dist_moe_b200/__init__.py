"""dist_moe_b200: the routed-expert hot path of dist_moe, rebuilt for B200 (sm_100a).

Drop-in surface (same names as ``dist_moe``); the CUDA library behind it is loaded
lazily on the first device call and there is no fallback path without it.
"""

from ._execution import ExecutionOptions, PreparedWeight, RMSNormPostprocess
from .api import (
    Bf16GroupedGemmPreset,
    BlockScaledConfig,
    BlockScaledKernelConfig,
    Config,
    Context,
    MemoryPlan,
    VmmConfig,
    create_context,
    plan_memory,
    prepare_block_scaled_weight,
    routed_experts,
    supports_fused_post_expert_rmsnorm,
)
from .formats import BlockScaledFormat
from . import _ops as _ops

# torch.ops.dist_moe.* (operator schemas and fake implementations for tracing); no device work happens here
_ops.register()

__all__ = [
    "Bf16GroupedGemmPreset",
    "BlockScaledConfig",
    "BlockScaledFormat",
    "BlockScaledKernelConfig",
    "Config",
    "Context",
    "ExecutionOptions",
    "MemoryPlan",
    "PreparedWeight",
    "RMSNormPostprocess",
    "VmmConfig",
    "create_context",
    "plan_memory",
    "prepare_block_scaled_weight",
    "routed_experts",
    "supports_fused_post_expert_rmsnorm",
]
