"""Per-call options, prepared weights and the post-expert RMSNorm policy.

Host-side policy objects only; they mirror the reference's public dataclasses
(dist_moe/_execution.py:92-382, dist_moe/_postprocess.py:21-91) field for field so
that caller code is unchanged.
"""

from __future__ import annotations

import dataclasses
import math
from typing import Any, Callable

import torch

from .formats import BlockScaledFormat


@dataclasses.dataclass(frozen=True)
class RMSNormPostprocess:
    """Fused post-expert RMSNorm + score-weighted top-k reduction.

    ``out[t] = sum_k s[t,k] * h3[t,k] / sqrt(mean_d(h3[t,k]^2) + eps)``; with ``weight``
    (inference only) ``h3`` is first multiplied by ``weight + gain_center``.
    """

    eps: float
    norm_output_dtype: torch.dtype
    output_dtype: torch.dtype
    require_bitwise: bool = True
    weight: torch.Tensor | None = None
    gain_center: float = 0.0
    use_kahan: bool = False
    observe_expert_output_fn: Callable[[torch.Tensor], None] | None = None
    observe_expert_output_grad_fn: Callable[[torch.Tensor, torch.Tensor], None] | None = None
    recompute_rstd: bool = False


def _postprocess_requires_eager(postprocess: Any) -> bool:
    if postprocess is None:
        return False
    if isinstance(postprocess, RMSNormPostprocess):
        return postprocess.observe_expert_output_fn is not None or postprocess.observe_expert_output_grad_fn is not None
    return True


@dataclasses.dataclass(frozen=True)
class ExecutionOptions:
    """Per-invocation controls (dist_moe/_execution.py:92-245)."""

    inplace_wgrad_accum: bool = False
    wgrad_parameter_owners: tuple[torch.Tensor, torch.Tensor] | None = dataclasses.field(
        default=None, repr=False, compare=False
    )
    weights_preprocess_fn: Callable | None = None
    experts_output_postprocess: Callable[[torch.Tensor], torch.Tensor] | RMSNormPostprocess | None = None
    wgrad_postprocess_fn: Callable | None = None
    swiglu_clip_stats_out_3: torch.Tensor | None = None
    swiglu_clip_limit: float = 7.0
    wgrad_destination_fn: Callable | None = None
    validate_expert_ids: bool = False
    zero_out_padded_callback_inputs: bool = False

    def __post_init__(self) -> None:
        out = self.swiglu_clip_stats_out_3
        if out is not None:
            if not isinstance(out, torch.Tensor):
                raise TypeError("swiglu_clip_stats_out_3 must be a tensor")
            if out.dtype is not torch.float32:
                raise TypeError("swiglu_clip_stats_out_3 must have dtype float32")
            if out.shape != (3,) or not out.is_contiguous():
                raise ValueError("swiglu_clip_stats_out_3 must be contiguous with shape [3]")
            if out.device.type != "cuda":
                raise ValueError("swiglu_clip_stats_out_3 must be a CUDA tensor")
        if not isinstance(self.swiglu_clip_limit, (int, float)) or isinstance(self.swiglu_clip_limit, bool):
            raise TypeError("swiglu_clip_limit must be a real number")
        if not math.isfinite(self.swiglu_clip_limit):
            raise ValueError("swiglu_clip_limit must be finite")
        if not isinstance(self.inplace_wgrad_accum, bool):
            raise TypeError("inplace_wgrad_accum must be a bool")
        if self.inplace_wgrad_accum and self.wgrad_postprocess_fn is not None:
            raise ValueError("inplace_wgrad_accum cannot be combined with wgrad_postprocess_fn")
        if self.wgrad_destination_fn is not None and (self.inplace_wgrad_accum or self.wgrad_postprocess_fn is not None):
            raise ValueError(
                "wgrad_destination_fn cannot be combined with inplace_wgrad_accum or wgrad_postprocess_fn"
            )
        if self.wgrad_destination_fn is not None and not callable(self.wgrad_destination_fn):
            raise TypeError("wgrad_destination_fn must be callable")
        if self.wgrad_parameter_owners is not None:
            if not self.inplace_wgrad_accum:
                raise ValueError("wgrad_parameter_owners requires inplace_wgrad_accum=True")
            owners = self.wgrad_parameter_owners
            if not isinstance(owners, tuple) or len(owners) != 2 or not all(isinstance(o, torch.Tensor) for o in owners):
                raise TypeError("wgrad_parameter_owners must be a pair of W13 and W2 tensors")
        for name in ("validate_expert_ids", "zero_out_padded_callback_inputs"):
            if not isinstance(getattr(self, name), bool):
                raise TypeError(f"{name} must be a bool")

    @property
    def requires_eager(self) -> bool:
        """Whether a Python callback has to run inside the kernel schedule."""
        return (
            self.weights_preprocess_fn is not None
            or _postprocess_requires_eager(self.experts_output_postprocess)
            or self.wgrad_postprocess_fn is not None
            or self.wgrad_destination_fn is not None
        )


DEFAULT_OPTIONS = ExecutionOptions()


@dataclasses.dataclass(frozen=True, init=False)
class PreparedWeight:
    """Caller-owned block-scaled operands of one expert projection.

    Built only by ``prepare_block_scaled_weight`` (dist_moe/_execution.py:248-382):
    MXFP8 keeps one E4M3 qdata tensor shared by forward and input-gradient GEMMs with
    two scale orientations; NVFP4 keeps packed E2M1 qdata, E4M3 block scales and the
    per-expert fp32 global scale with its reciprocal.
    """

    source: torch.Tensor
    format: BlockScaledFormat
    fprop_data: torch.Tensor
    fprop_scale: torch.Tensor
    dgrad_data: torch.Tensor | None
    dgrad_scale: torch.Tensor | None
    global_scale: torch.Tensor | None = None
    global_scale_inv: torch.Tensor | None = None
    _interleaved_fc13: bool = False

    def __init__(self) -> None:
        raise TypeError("use prepare_block_scaled_weight()")

    @classmethod
    def _create(cls, **fields: Any) -> "PreparedWeight":
        obj = object.__new__(cls)
        names = {f.name for f in dataclasses.fields(cls)}
        if "interleaved_fc13" in fields:
            fields["_interleaved_fc13"] = fields.pop("interleaved_fc13")
        for f in dataclasses.fields(cls):
            if f.name in fields:
                value = fields[f.name]
            elif f.default is not dataclasses.MISSING:
                value = f.default
            else:
                raise TypeError(f"missing prepared-weight field {f.name}")
            object.__setattr__(obj, f.name, value)
        unknown = set(fields) - names
        if unknown:
            raise TypeError(f"unknown prepared-weight fields {sorted(unknown)}")
        return obj

    def storage_tensors(self) -> tuple[torch.Tensor, ...]:
        """One representative tensor per distinct owned storage."""
        seen: list[torch.UntypedStorage] = []
        out: list[torch.Tensor] = []
        for t in (self.fprop_data, self.fprop_scale, self.dgrad_data, self.dgrad_scale, self.global_scale,
                  self.global_scale_inv):
            if t is None:
                continue
            st = t.untyped_storage()
            if any(st is s for s in seen):
                continue
            seen.append(st)
            out.append(t)
        return tuple(out)

    def _with_source(self, source: torch.Tensor) -> "PreparedWeight":
        fields = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}
        fields["source"] = source
        return self._create(**fields)
