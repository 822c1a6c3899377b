"""Typed post-expert processing: fused RMSNorm + score-weighted top-k reduction.

Host-side validation and launch of ``dm_rmsnorm_combine_fwd/bwd``; mirrors the contract of the
reference's ``RMSNormPostprocess`` path (dist_moe/_postprocess.py:648-719 validation,
dist_moe/kernels/norm/fused_rmsnorm_combine.py:326-348 tensor contract).
"""

from __future__ import annotations

import math

import torch

from . import _native as nat
from ._execution import RMSNormPostprocess


def validate_rmsnorm(post: RMSNormPostprocess, *, config, training: bool, x_dtype: torch.dtype,
                     observers_allowed: bool = False) -> None:
    if not isinstance(post.eps, (int, float)) or not math.isfinite(post.eps) or post.eps <= 0:
        raise ValueError("RMSNormPostprocess.eps must be finite and positive")
    if post.output_dtype != x_dtype:
        raise ValueError("RMSNormPostprocess.output_dtype must equal the input dtype")
    if post.norm_output_dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("RMSNormPostprocess.norm_output_dtype must be float32 or bfloat16")
    if post.use_kahan and post.weight is not None:
        raise ValueError("input-scale weight is not supported with Kahan summation")
    if (post.observe_expert_output_fn is not None or post.observe_expert_output_grad_fn is not None) \
            and not observers_allowed:
        raise NotImplementedError("expert-output observers run on BF16 contexts only (the eager callback path)")
    if post.weight is not None:
        if training:
            raise ValueError("RMSNormPostprocess.weight is supported for inference only")
        w = post.weight
        if w.dtype != x_dtype or w.shape != (config.hidden_dim,) or not w.is_contiguous() or w.device.type != "cuda":
            raise ValueError("RMSNormPostprocess.weight must be a contiguous CUDA tensor of shape [hidden_dim] "
                             "with the input dtype")


def rmsnorm_combine_forward(state, call, post: RMSNormPostprocess, scores, ids, out, *, save: bool,
                            save_to: torch.Tensor | None = None, observers_allowed: bool = False):
    """Normalise and reduce the expert outputs in the local combine buffer.  ``save`` keeps a copy of them for the
    backward: in the planner's slot (device-predicated on the call's save/recompute decision) or, when ``save_to``
    is given, unconditionally in that tensor."""
    cfg = state.config
    T, K, D = out.shape[0], cfg.top_k, cfg.hidden_dim
    validate_rmsnorm(post, config=cfg, training=save, x_dtype=out.dtype, observers_allowed=observers_allowed)
    rstd = None
    if save and not post.recompute_rstd:
        rstd = torch.empty(T, K, dtype=torch.float32, device=out.device)
    if save_to is not None:
        base, offset, cond = save_to.data_ptr(), None, None
    elif save:
        base, offset, cond = state.arena.data_ptr(), call.fwd_state[4:5].data_ptr(), call.cond.data_ptr()
    else:
        base = offset = cond = None
    nat.check(nat.lib.dm_rmsnorm_combine_fwd(
        state.combine.local().data_ptr(), scores.data_ptr(), int(scores.dtype == torch.bfloat16), ids.data_ptr(),
        int(ids.dtype == torch.int64), nat.ptr(post.weight), float(post.gain_center), float(post.eps),
        int(post.norm_output_dtype == torch.bfloat16), int(bool(post.use_kahan)), out.data_ptr(), nat.ptr(rstd), T, K,
        D, base, offset, cond, 0, nat.stream_ptr()), "dm_rmsnorm_combine_fwd")
    return rstd


def rmsnorm_combine_backward(state, call, post: RMSNormPostprocess, grad_out, scores, ids, grad_scores,
                             h3: torch.Tensor | None = None) -> None:
    """Gradient with respect to the expert outputs, written to the local combine buffer.  The expert outputs are
    read from ``h3`` when given, else from the combine buffer itself (restored there by the caller), in place."""
    cfg = state.config
    T, K, D = grad_out.shape[0], cfg.top_k, cfg.hidden_dim
    combine = state.combine.local().data_ptr()
    nat.check(nat.lib.dm_rmsnorm_combine_bwd(
        grad_out.data_ptr(), scores.data_ptr(), int(scores.dtype == torch.bfloat16), ids.data_ptr(),
        int(ids.dtype == torch.int64), combine if h3 is None else h3.data_ptr(), None, nat.ptr(call.rstd),
        float(post.eps), int(post.norm_output_dtype == torch.bfloat16), int(bool(post.use_kahan)), combine,
        nat.ptr(grad_scores), T, K, D, nat.stream_ptr()), "dm_rmsnorm_combine_bwd")
