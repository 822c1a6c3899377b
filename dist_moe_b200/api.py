"""Public surface: configuration, memory planning, contexts and ``routed_experts``.

Names, argument meaning and error behaviour follow the reference's public API
(dist_moe/api.py: ``Config`` 332-515, ``MemoryPlan`` 517-691, ``plan_memory`` 875-1049,
``Context`` 1194-1388, ``create_context`` 1555-1706, ``routed_experts`` 3856-4112,
``prepare_block_scaled_weight`` 4115-4155).  Underneath, every device operation is a
hand-written sm_100a kernel reached through the C ABI in ``include/dist_moe_b200.h``.
"""

from __future__ import annotations

import dataclasses
import logging
import math
import threading
import uuid
from typing import Any, Literal, get_args

import torch
import torch.distributed as dist

from . import _planning
from ._execution import DEFAULT_OPTIONS, ExecutionOptions, PreparedWeight, RMSNormPostprocess
from .formats import (
    NVFP4_DIM_MULTIPLE,
    NVFP4_HIDDEN_DIM_MAX,
    NVFP4_INTERMEDIATE_DIM_MAX,
    SWIGLU_CLAMP_ALPHA_DEFAULT,
    SWIGLU_CLAMP_LIMIT_DEFAULT,
    BlockScaledFormat,
    format_constants,
)

logger = logging.getLogger(__name__)

Bf16GroupedGemmPreset = Literal[
    "1cta1mma_bm64_bn128",
    "1cta1mma_bm64_bn256",
    "1cta1mma_bm128_bn128",
    "1cta1mma_bm128_bn256",
    "1cta2mma_bm256_bn256",
    "2cta1mma_bm256_bn256",
    "2cta2mma_bm512_bn256",
]
_PRESETS = frozenset(get_args(Bf16GroupedGemmPreset))


# ---------------------------------------------------------------------------
# Configuration dataclasses
# ---------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class VmmConfig:
    """Host-backed overflow-scratch policy (accepted for planning; see ``create_context``)."""

    total_scratch_capacity_factor: float = 16.0
    prefetch: bool = True

    def __post_init__(self) -> None:
        if not math.isfinite(self.total_scratch_capacity_factor) or self.total_scratch_capacity_factor <= 0:
            raise ValueError("total_scratch_capacity_factor must be finite and positive")
        if not isinstance(self.prefetch, bool):
            raise TypeError("prefetch must be a bool")


@dataclasses.dataclass(frozen=True)
class BlockScaledKernelConfig:
    """Tile/pipeline override of the reference's CuTe kernels.

    Accepted and validated structurally for drop-in compatibility; the sm_100a kernels
    in this library choose their own tiles and ignore the values.
    """

    num_ctas: int
    block_m: int
    block_n: int
    block_k: int
    num_smem_buffers: int
    num_c_stages: int
    num_tmem_buffers: int
    num_tile_buffers: int
    epilogue_subtile: int
    overlapping_accum: bool
    swap_ab: bool
    kloop_unroll: int
    num_warps: int = 8
    static_scheduler: bool = False

    def __post_init__(self) -> None:
        positive = (self.num_ctas, self.block_m, self.block_n, self.block_k, self.num_smem_buffers, self.num_c_stages,
                    self.num_tmem_buffers, self.num_tile_buffers, self.epilogue_subtile, self.kloop_unroll,
                    self.num_warps)
        if any(v <= 0 for v in positive):
            raise ValueError("block-scaled kernel dimensions must be positive")
        if self.num_ctas not in (1, 2):
            raise ValueError("num_ctas must be 1 or 2")
        if self.block_n % self.epilogue_subtile:
            raise ValueError("epilogue_subtile must divide block_n")


@dataclasses.dataclass(frozen=True)
class BlockScaledConfig:
    """Block-scaled compute policy: MXFP8 E4M3 (training/inference) or NVFP4 (inference)."""

    format: BlockScaledFormat = BlockScaledFormat.MXFP8_E4M3
    fast_math: bool = False
    pipeline: Literal["staged", "mega"] = "staged"
    kernel_config: BlockScaledKernelConfig | None = None

    def __post_init__(self) -> None:
        if self.format not in (BlockScaledFormat.MXFP8_E4M3, BlockScaledFormat.NVFP4):
            raise ValueError(f"unsupported DistMoE block-scaled format {self.format}")
        if self.fast_math and self.format is BlockScaledFormat.NVFP4:
            raise ValueError("fast_math is supported only by the MXFP8 fused path")
        if self.pipeline not in ("staged", "mega"):
            raise ValueError("block-scaled pipeline must be 'staged' or 'mega'")
        if self.kernel_config is not None and self.kernel_config.block_k != 128:
            raise ValueError(f"{self.format.value} requires block_k=128, got {self.kernel_config.block_k}")


@dataclasses.dataclass(frozen=True)
class Config:
    """Static execution configuration of one MoE shape (dist_moe/api.py:332-515)."""

    max_num_local_input_tokens: int
    hidden_dim: int
    intermediate_dim: int
    top_k: int
    num_experts: int
    max_moe_layers_per_activation_slot: int
    device_scratch_capacity_factor: float = 1.0
    activation_slot_bytes: int | None = None
    activation_slot_capacity_factor: float | None = None
    num_activation_slots: int = 1
    vmm: VmmConfig | None = None
    num_sms: int | None = None
    bf16_grouped_gemm_preset: Bf16GroupedGemmPreset | None = None
    block_scaled: BlockScaledConfig | None = None
    activation: Literal["swiglu", "swiglu_clamped"] = "swiglu"
    swiglu_alpha: float = SWIGLU_CLAMP_ALPHA_DEFAULT
    swiglu_limit: float = SWIGLU_CLAMP_LIMIT_DEFAULT
    wgrad_dtype: torch.dtype | None = None
    inference: bool = False

    def __post_init__(self) -> None:  # noqa: C901
        if min(self.max_num_local_input_tokens, self.hidden_dim, self.intermediate_dim, self.top_k) <= 0:
            raise ValueError(
                "max_num_local_input_tokens, hidden_dim, intermediate_dim, and top_k must be positive"
            )
        if self.hidden_dim % 64 != 0:
            raise ValueError("hidden_dim must be a multiple of 64 BF16 elements")
        if self.num_experts <= 0:
            raise ValueError("num_experts must be positive")
        if self.top_k > self.num_experts:
            raise ValueError("top_k cannot exceed num_experts")
        if self.max_moe_layers_per_activation_slot <= 0:
            raise ValueError("max_moe_layers_per_activation_slot must be positive")
        if self.activation_slot_bytes is not None:
            if isinstance(self.activation_slot_bytes, bool) or not isinstance(self.activation_slot_bytes, int):
                raise TypeError("activation_slot_bytes must be an integer")
            if self.activation_slot_bytes < 0:
                raise ValueError("activation_slot_bytes cannot be negative")
        factor = self.activation_slot_capacity_factor
        if factor is not None:
            if isinstance(factor, bool) or not isinstance(factor, (int, float)):
                raise TypeError("activation_slot_capacity_factor must be a real number")
            if not math.isfinite(factor) or factor < 0:
                raise ValueError("activation_slot_capacity_factor must be finite and nonnegative")
        if self.activation_slot_bytes is not None and factor is not None:
            raise ValueError("activation_slot_bytes and activation_slot_capacity_factor are mutually exclusive")
        if not self.inference and self.num_activation_slots <= 0:
            raise ValueError("training requires at least one activation slot")
        if self.inference and self.num_activation_slots < 0:
            raise ValueError("num_activation_slots cannot be negative")
        if self.inference and (self.activation_slot_bytes is not None or factor is not None):
            raise ValueError(
                "inference does not retain saved activations; activation slot capacity controls must be None"
            )
        if not math.isfinite(self.device_scratch_capacity_factor) or self.device_scratch_capacity_factor <= 0:
            raise ValueError("device_scratch_capacity_factor must be finite and positive")
        if self.num_sms is not None and self.num_sms <= 0:
            raise ValueError("num_sms must be positive when specified")
        if self.bf16_grouped_gemm_preset is not None and self.bf16_grouped_gemm_preset not in _PRESETS:
            raise ValueError(
                f"bf16_grouped_gemm_preset must name a supported BF16 preset; got {self.bf16_grouped_gemm_preset!r}"
            )
        if self.wgrad_dtype is not None and self.wgrad_dtype not in (torch.bfloat16, torch.float32):
            raise TypeError(f"wgrad_dtype must be None, torch.bfloat16, or torch.float32, got {self.wgrad_dtype}")
        if self.activation not in ("swiglu", "swiglu_clamped"):
            raise ValueError(f"activation must be 'swiglu' or 'swiglu_clamped', got {self.activation!r}")
        if self.activation == "swiglu_clamped" and (
            not math.isfinite(self.swiglu_alpha) or not math.isfinite(self.swiglu_limit)
            or self.swiglu_alpha <= 0 or self.swiglu_limit <= 0
        ):
            raise ValueError("clamped SwiGLU requires finite positive swiglu_alpha and swiglu_limit")
        if self.block_scaled is not None:
            _validate_block_scaled(self)


def _validate_block_scaled(config: Config) -> None:
    policy = config.block_scaled
    assert policy is not None
    vec = format_constants(policy.format)[3]
    if config.hidden_dim % vec or config.intermediate_dim % vec:
        raise ValueError(
            f"block-scaled hidden_dim and intermediate_dim must be divisible by the format vector size {vec}"
        )
    if policy.format is BlockScaledFormat.NVFP4:
        if not config.inference:
            raise ValueError("NVFP4 DistMoE is inference-only")
        if (config.hidden_dim % NVFP4_DIM_MULTIPLE or config.intermediate_dim % NVFP4_DIM_MULTIPLE
                or config.hidden_dim > NVFP4_HIDDEN_DIM_MAX or config.intermediate_dim > NVFP4_INTERMEDIATE_DIM_MAX):
            raise ValueError(
                f"NVFP4 requires hidden_dim to be a multiple of {NVFP4_DIM_MULTIPLE} and at most "
                f"{NVFP4_HIDDEN_DIM_MAX}, and intermediate_dim to be a multiple of {NVFP4_DIM_MULTIPLE} and at most "
                f"{NVFP4_INTERMEDIATE_DIM_MAX}"
            )


# ---------------------------------------------------------------------------
# Memory plan
# ---------------------------------------------------------------------------
@dataclasses.dataclass(frozen=True)
class MemoryPlan:
    """Resolved allocation sizes (bytes, except the row counts and factors)."""

    balanced_recv_rows: int
    device_scratch_capacity_rows: int
    total_scratch_capacity_rows: int
    device_scratch_capacity_factor: float
    total_scratch_capacity_factor: float
    saved_input_bytes_per_layer: int
    device_scratch_bytes: int
    host_scratch_bytes: int
    minimum_activation_slot_bytes: int
    balanced_full_save_activation_slot_bytes: int
    maximum_useful_activation_slot_bytes: int
    activation_slot_bytes: int
    activation_slot_capacity_factor: float | None
    total_activation_bytes: int
    total_device_buffer_bytes: int
    total_virtual_bytes: int
    num_activation_slots: int
    inference: bool
    vmm_granularity_bytes: int | None
    vmm_device_prefix_bytes: int | None
    vmm_host_section_bytes: int | None
    vmm_device_scratch_section_bytes: int | None
    vmm_padding_bytes: int
    inference_operand_bytes: int | None = None

    @property
    def uses_host_scratch(self) -> bool:
        return self.host_scratch_bytes > 0

    def explain(self) -> str:
        """Log-friendly description; the text matches the reference's line for line."""

        def size(n: int) -> str:
            return f"{n / 1024**3:.3f} GiB ({n:,} bytes)"

        if self.inference:
            slots = "  activation slots: 0 slot(s)"
            recompute = "scratch-only inference; no saved activations"
            boundary = "  inference has no activation slots; total scratch capacity is a hard limit"
        else:
            if self.activation_slot_capacity_factor is not None:
                policy = f"balanced capacity factor {self.activation_slot_capacity_factor:g}"
            elif self.activation_slot_bytes == self.minimum_activation_slot_bytes:
                policy = "minimum all-recompute"
            else:
                policy = "exact per-slot bytes"
            slots = (f"  activation slots: {self.num_activation_slots} x {size(self.activation_slot_bytes)} = "
                     f"{size(self.total_activation_bytes)} ({policy})")
            if self.activation_slot_bytes == self.minimum_activation_slot_bytes:
                recompute = "all layers recompute at the minimum budget"
            elif self.activation_slot_bytes >= self.maximum_useful_activation_slot_bytes:
                recompute = "all executable routing fits without recompute"
            elif self.activation_slot_bytes >= self.balanced_full_save_activation_slot_bytes:
                recompute = "balanced routing fits without recompute; larger saved-state usage may recompute"
            else:
                recompute = "the activation budget may avoid recompute for some layers"
            boundary = ("  activation slots are a soft limit (recompute on exhaustion); "
                        "total scratch capacity is a hard limit")
        lines = [
            "Distributed MoE memory plan:",
            f"  balanced/device/total rows: {self.balanced_recv_rows}/"
            f"{self.device_scratch_capacity_rows}/{self.total_scratch_capacity_rows}",
            f"  device/total scratch capacity factors: {self.device_scratch_capacity_factor:g}/"
            f"{self.total_scratch_capacity_factor:g}",
            slots,
            f"  device scratch: {size(self.device_scratch_bytes)}",
            f"  host overflow scratch: {size(self.host_scratch_bytes)}",
            f"  total device buffer: {size(self.total_device_buffer_bytes)}",
            f"  activation slot minimum/balanced full-save/maximum useful: "
            f"{size(self.minimum_activation_slot_bytes)} / {size(self.balanced_full_save_activation_slot_bytes)} / "
            f"{size(self.maximum_useful_activation_slot_bytes)}",
            f"  virtual address range: {size(self.total_virtual_bytes)}; {recompute}",
            boundary,
        ]
        if self.inference_operand_bytes is not None:
            lines.append(f"  physical Mega inference operands: {size(self.inference_operand_bytes)} (within device scratch)")
        if self.vmm_granularity_bytes is not None:
            lines.extend((
                f"  VMM section granularity: {size(self.vmm_granularity_bytes)}",
                f"  mapped device/host/device sections: {size(self.vmm_device_prefix_bytes)} / "
                f"{size(self.vmm_host_section_bytes)} / {size(self.vmm_device_scratch_section_bytes)}",
                f"  VMM/allocator padding: {size(self.vmm_padding_bytes)}",
            ))
        return "\n".join(lines)


def _arena_sizing(config: Config, ep_size: int | None, factor: float | None = None) -> _planning.ArenaSizing:
    storage = None
    if config.block_scaled is not None:
        if ep_size is None:
            raise ValueError("ep_size is required for block-scaled memory planning")
        ob, vpe, sb, vec, gs = format_constants(config.block_scaled.format)
        storage = _planning.QuantStorage(ob, vpe, sb, vec, gs)
    return _planning.ArenaSizing(
        num_tokens=config.max_num_local_input_tokens,
        hidden=config.hidden_dim,
        inter=config.intermediate_dim,
        top_k=config.top_k,
        factor=config.device_scratch_capacity_factor if factor is None else factor,
        num_layers=config.max_moe_layers_per_activation_slot,
        num_local_experts=1 if ep_size is None else config.num_experts // ep_size,
        ep_size=ep_size,
        storage=storage,
        mega=config.block_scaled is not None and config.block_scaled.pipeline == "mega",
    )


def plan_memory(config: Config, ep_size: int, *, device: torch.device | str | int | None = None) -> MemoryPlan:
    """Resolve activation-slot, device-scratch and host-scratch sizes (dist_moe/api.py:875-1049).

    ``inference_operand_bytes`` is resolved under the reference's conditions (inference, block-scaled "mega"
    pipeline, no VMM, a device or ``num_sms`` given; dist_moe/api.py:962-981) as the size of this library's static
    operand carve, and the device scratch is raised to hold it.  With ``Config.vmm``, host scratch and a device the
    physical section sizes are resolved at the driver's granularity (dist_moe/api.py:1047-1109).
    """
    if ep_size <= 0:
        raise ValueError("ep_size must be positive")
    device_factor = min(config.device_scratch_capacity_factor, float(ep_size))
    if device_factor != config.device_scratch_capacity_factor:
        logger.warning(
            "Capping device_scratch_capacity_factor from %g to %g for ep_size=%d; routing topology cannot deliver "
            "a larger imbalance", config.device_scratch_capacity_factor, device_factor, ep_size)
    sizing = _arena_sizing(config, ep_size, device_factor)
    layers = config.max_moe_layers_per_activation_slot
    num_slots = 0 if config.inference else config.num_activation_slots
    if config.inference:
        device_scratch = _planning.align(sizing.inference_scratch_bytes)
        min_slot = full_slot = 0
    else:
        device_scratch = sizing.training_scratch_bytes
        min_slot = _planning.align(layers * sizing.saved_bytes(0, True))
        full_slot = _planning.align(layers * sizing.saved_bytes(sizing.rows_at(1.0), False))
        if full_slot < min_slot:
            raise RuntimeError("balanced full-save activation state is smaller than mandatory layer inputs")
    total_factor = device_factor
    host_scratch = 0
    if config.vmm is not None:
        total_factor = min(config.vmm.total_scratch_capacity_factor, float(ep_size))
        if total_factor < device_factor:
            raise ValueError(
                "total_scratch_capacity_factor must cover at least the device_scratch_capacity_factor after "
                "EP-size clamping")
        if config.inference:
            host_scratch = sizing.host_inference_scratch_bytes(total_factor)
        else:
            host_scratch = sizing.host_scratch_bytes(total_factor)
    if config.inference:
        max_slot = slot = 0
    else:
        max_slot = _planning.align(layers * sizing.saved_bytes(sizing.rows_at(total_factor), False))
        if config.activation_slot_bytes is not None:
            if config.activation_slot_bytes < min_slot:
                raise ValueError(
                    f"activation_slot_bytes={config.activation_slot_bytes} is below the minimum required "
                    f"{min_slot} bytes")
            slot = _planning.align(config.activation_slot_bytes)
        elif config.activation_slot_capacity_factor is not None:
            slot = _planning.align(
                min_slot + math.ceil(config.activation_slot_capacity_factor * (full_slot - min_slot)))
        else:
            slot = min_slot
        if slot > max_slot:
            logger.warning("activation_slot_bytes=%d exceeds the maximum useful %d bytes for this context", slot,
                           max_slot)
    inference_operand_bytes = None
    if (config.inference and config.block_scaled is not None and config.block_scaled.pipeline == "mega"
            and config.vmm is None and (device is not None or config.num_sms is not None)):
        from ._blockscaled import inference_layout

        inference_operand_bytes = inference_layout(config.block_scaled.format, config.hidden_dim,
                                                   config.intermediate_dim, sizing.capacity_rows)["total"]
        device_scratch = max(device_scratch, _planning.align(inference_operand_bytes))
    total_act = num_slots * slot
    total_dev = total_act + device_scratch
    plan = MemoryPlan(
        balanced_recv_rows=config.max_num_local_input_tokens * config.top_k,
        device_scratch_capacity_rows=sizing.capacity_rows,
        total_scratch_capacity_rows=sizing.rows_at(total_factor),
        device_scratch_capacity_factor=device_factor,
        total_scratch_capacity_factor=total_factor,
        saved_input_bytes_per_layer=sizing.saved_bytes(0, True),
        device_scratch_bytes=device_scratch,
        host_scratch_bytes=host_scratch,
        minimum_activation_slot_bytes=min_slot,
        balanced_full_save_activation_slot_bytes=full_slot,
        maximum_useful_activation_slot_bytes=max_slot,
        activation_slot_bytes=slot,
        activation_slot_capacity_factor=config.activation_slot_capacity_factor,
        total_activation_bytes=total_act,
        total_device_buffer_bytes=total_dev,
        total_virtual_bytes=total_dev + host_scratch,
        num_activation_slots=num_slots,
        inference=config.inference,
        vmm_granularity_bytes=None,
        vmm_device_prefix_bytes=None,
        vmm_host_section_bytes=None,
        vmm_device_scratch_section_bytes=None,
        vmm_padding_bytes=0,
        inference_operand_bytes=inference_operand_bytes,
    )
    if config.vmm is not None and host_scratch > 0 and device is not None:
        from . import _vmm

        dev = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        if dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        return _vmm.resolve_physical_plan(plan, _vmm.granularity(dev))
    return plan


# ---------------------------------------------------------------------------
# Context
# ---------------------------------------------------------------------------
_CONTEXTS: dict[str, "Context"] = {}
_CONTEXT_LOCK = threading.Lock()


@dataclasses.dataclass(init=False)
class Context:
    """Pre-allocated per-process state for one MoE shape; build with :func:`create_context`.

    Owns the symmetric routing/dispatch/combine buffers, the activation arena and the
    device-side planner state.  One call at a time: not re-entrant, single stream.
    """

    group: Any
    config: Config
    memory_plan: MemoryPlan
    _context_id: str
    _closed: bool = False

    def __init__(self) -> None:
        raise TypeError("use create_context()")

    @property
    def max_num_local_input_tokens(self) -> int:
        return self.config.max_num_local_input_tokens

    @property
    def hidden_dim(self) -> int:
        return self.config.hidden_dim

    @property
    def top_k(self) -> int:
        return self.config.top_k

    @property
    def context_id(self) -> str:
        if self._closed:
            raise RuntimeError("distributed MoE context is closed")
        return self._context_id

    def reset(self) -> None:
        """Rewind activation-slot state for a new execution schedule."""
        if self._closed:
            raise RuntimeError("distributed MoE context is closed")
        self._state.reset()

    def select_activation_slot(self, activation_slot: int, num_moe_layers_in_slot: int) -> None:
        """Select the activation slot (and its layer depth) used by the following calls."""
        if self._closed:
            raise RuntimeError("distributed MoE context is closed")
        self._state.select_slot(activation_slot, num_moe_layers_in_slot)

    def check_status(self) -> None:
        """Synchronise and raise if a kernel reported a contract violation.

        The reference traps the device in these cases; here the kernels record a code,
        turn the rest of the call into no-ops and leave the CUDA context usable.
        """
        self._state.check_status()

    def check_overflow(self):
        """Peak scratch / slot usage since the last ``reset`` (blocking); raises on overflow.  The asynchronous pair
        is ``begin_check_overflow`` / ``finish_check_overflow`` (dist_moe/_activation_buffer.py:690-760)."""
        return self._state.check_overflow()

    def begin_check_overflow(self):
        return self._state.begin_check_overflow()

    def finish_check_overflow(self, pending):
        return self._state.finish_check_overflow(pending)

    def close(self) -> None:
        with _CONTEXT_LOCK:
            _CONTEXTS.pop(self._context_id, None)
        if self._closed:
            return
        self._closed = True
        self._state.close()


def create_context(*, group: Any, config: Config, device: torch.device | str | int | None = None,
                   memory_plan: MemoryPlan | None = None) -> Context:
    """Collectively allocate the buffers of one MoE shape (dist_moe/api.py:1555-1706)."""
    from ._runtime import ContextState

    ep_size = dist.get_world_size(group) if group is not None else 1
    if config.num_experts % ep_size != 0:
        raise ValueError(
            f"num_experts={config.num_experts} must be divisible by the expert-parallel group size {ep_size}")
    if device is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    else:
        dev = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
    if dev.type != "cuda":
        raise ValueError(f"device must be CUDA, got {dev}")
    plan = memory_plan if memory_plan is not None else plan_memory(config, ep_size, device=dev)
    if config.vmm is not None and plan.host_scratch_bytes > 0 and plan.vmm_granularity_bytes is None:
        raise ValueError("a memory plan with host scratch must be resolved for the device: plan_memory(..., device=...)")
    logger.info("%s", plan.explain())
    ctx = object.__new__(Context)
    ctx.group = group
    ctx.config = config
    ctx.memory_plan = plan
    ctx._context_id = f"dist_moe_b200:{uuid.uuid4().hex}"
    ctx._closed = False
    ctx._state = ContextState(group=group, ep_size=ep_size, config=config, plan=plan, device=dev)
    with _CONTEXT_LOCK:
        _CONTEXTS[ctx._context_id] = ctx
    return ctx


# ---------------------------------------------------------------------------
# routed_experts
# ---------------------------------------------------------------------------
def _reshape_weights(w13: torch.Tensor, w2: torch.Tensor, e_local: int, config: Config):
    """Normalise the accepted weight layouts to [E_local, 2F, D] and [E_local, D, F]."""
    D, F = config.hidden_dim, config.intermediate_dim
    if w13.ndim == 4:
        w13 = w13.reshape(w13.shape[0], w13.shape[1] * w13.shape[2], w13.shape[3])
    elif w13.ndim == 2:
        w13 = w13.reshape(e_local, -1, w13.shape[1])
    if w2.ndim == 2:
        w2 = w2.reshape(e_local, -1, w2.shape[1])
    if w13.ndim != 3 or w2.ndim != 3:
        raise ValueError("w13_EFD and w2_EDF must be three-dimensional expert weights")
    if w13.shape[0] != e_local or w2.shape[0] != e_local:
        raise ValueError(f"weights must contain {e_local} local experts")
    if w13.shape[1] != 2 * w2.shape[2]:
        raise ValueError("w13_EFD output dimension must be twice w2_EDF's input dimension")
    if w2.shape[2] != F:
        raise ValueError(f"weight intermediate dimension does not match config.intermediate_dim={F}")
    if w13.shape[2] != D or w2.shape[1] != D:
        raise ValueError("weight hidden dimensions do not match the context")
    return w13, w2


def _validate_inputs(x, ids, scores, w13, w2, context: Context, *, prepared: bool) -> None:
    if x.dtype != torch.bfloat16:
        raise TypeError("x_TD must use torch.bfloat16")
    if not prepared and (w13.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16):
        raise TypeError("w13_EFD and w2_EDF compute weights must use torch.bfloat16")
    if ids.dtype not in (torch.int32, torch.int64):
        raise TypeError("topk_expert_ids_TK must use torch.int32 or torch.int64")
    if scores.dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("topk_scores_TK must use torch.bfloat16 or torch.float32")
    if x.ndim != 2 or x.shape[1] != context.hidden_dim:
        raise ValueError(f"x_TD must have shape [T, {context.hidden_dim}]")
    T = x.shape[0]
    if not 1 <= T <= context.max_num_local_input_tokens:
        raise ValueError(
            f"x_TD has {T} tokens; the context accepts 1..{context.max_num_local_input_tokens} local tokens")
    if tuple(ids.shape) != (T, context.top_k) or tuple(scores.shape) != (T, context.top_k):
        raise ValueError(f"topk_expert_ids_TK and topk_scores_TK must have shape {(T, context.top_k)}")
    tensors = (x, ids, scores) if prepared else (x, ids, scores, w13, w2)
    if any(t.device != x.device for t in tensors) or x.device.type != "cuda":
        raise ValueError("all operation tensors must reside on the same CUDA device")
    if any(not t.is_contiguous() for t in tensors):
        raise ValueError("all operation tensors must be contiguous")


def routed_experts(x_TD: torch.Tensor, topk_expert_ids_TK: torch.Tensor, topk_scores_TK: torch.Tensor,
                   w13_weight: torch.Tensor | PreparedWeight, w2_weight: torch.Tensor | PreparedWeight,
                   context: Context, *, options: ExecutionOptions | None = None) -> torch.Tensor:
    """Apply the routed experts ``W2 . SwiGLU(W13 . x)`` to the local tokens.

    Collective over ``context.group``: every rank calls in the same order with the same
    ``T``.  Returns a fresh bf16 ``[T, D]`` tensor.  See dist_moe/api.py:3856-4112.
    """
    if not isinstance(context, Context):
        raise TypeError("context must come from create_context()")
    if context._closed:
        raise RuntimeError("distributed MoE context is closed")
    options = DEFAULT_OPTIONS if options is None else options
    if not isinstance(options, ExecutionOptions):
        raise TypeError("options must be an ExecutionOptions")
    prepared13, prepared2 = isinstance(w13_weight, PreparedWeight), isinstance(w2_weight, PreparedWeight)
    if prepared13 != prepared2:
        raise TypeError("w13_weight and w2_weight must both be tensors or both be PreparedWeight")
    prepared = prepared13
    state = context._state
    src13 = w13_weight.source if prepared else w13_weight
    src2 = w2_weight.source if prepared else w2_weight
    if options.weights_preprocess_fn is not None:
        if prepared:
            raise ValueError("prepared weights cannot be combined with weights_preprocess_fn")
        # compact source weights: the callback produces the BF16 compute weights (shape-checked there)
        w13_EFD, w2_EDF = src13, src2
        _validate_inputs(x_TD, topk_expert_ids_TK, topk_scores_TK, None, None, context, prepared=True)
    else:
        w13_EFD, w2_EDF = _reshape_weights(src13, src2, state.e_local, context.config)
        _validate_inputs(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_EFD, w2_EDF, context, prepared=prepared)
    if x_TD.device != state.device:
        raise ValueError(f"x_TD is on {x_TD.device} but the context was created on {state.device}")
    post = options.experts_output_postprocess
    norm_weight = post.weight if isinstance(post, RMSNormPostprocess) else None
    grads = [t for t in (x_TD, topk_scores_TK, w13_EFD, w2_EDF, norm_weight) if t is not None and t.requires_grad]
    if context.config.inference and grads:
        raise RuntimeError("inference contexts do not support autograd")
    save_for_backward = torch.is_grad_enabled() and bool(grads)
    # every launch below goes to the context's device and to that device's current stream
    with torch.cuda.device(state.device):
        if context.config.block_scaled is not None:
            from ._blockscaled import run_block_scaled

            return run_block_scaled(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_weight, w2_weight, context, options,
                                    save_for_backward=save_for_backward)
        if prepared:
            raise ValueError("prepared weights require block-scaled execution")
        from ._bf16 import run_bf16

        return run_bf16(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_weight, w2_weight, w13_EFD, w2_EDF, context,
                        options, save_for_backward=save_for_backward)


def prepare_block_scaled_weight(weight: torch.Tensor, config: Config, *, fuse_swiglu: bool = False,
                                inference: bool = False, out: PreparedWeight | None = None) -> PreparedWeight:
    """Quantise one expert projection into caller-owned block-scaled operands."""
    from ._blockscaled import prepare_weight

    return prepare_weight(weight, config, fuse_swiglu=fuse_swiglu, inference=inference, out=out)


def supports_fused_post_expert_rmsnorm(*, input_dtype: torch.dtype, score_dtype: torch.dtype,
                                       norm_output_dtype: torch.dtype, output_dtype: torch.dtype, topk: int,
                                       dim: int) -> bool:
    """Whether the fused RMSNorm + top-k reduction accepts this tensor contract."""
    if output_dtype != input_dtype or input_dtype != torch.bfloat16:
        return False
    if score_dtype not in (torch.float32, torch.bfloat16):
        return False
    if norm_output_dtype not in (torch.float32, torch.bfloat16):
        return False
    return 1 <= topk <= 64 and dim % 8 == 0 and 8 <= dim <= 131072
