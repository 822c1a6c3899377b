"""Calls that run Python callbacks inside the kernel schedule (dist_moe/_execution.py:93-245).

``ExecutionOptions`` with ``weights_preprocess_fn``, a callable ``experts_output_postprocess``,
``wgrad_postprocess_fn`` or ``wgrad_destination_fn`` cannot go through the registered operators: the callbacks are
Python code that has to run between two launches.  The launch sequence itself is the one of ``_bf16.py``; this module
supplies the callback hooks and the autograd function that re-materialises the compute weights before the backward
(dist_moe/api.py:1891-1893, 2252-2254).

* ``weights_preprocess_fn(source) -> bf16 weight``: called on both weights in the forward and again right before the
  backward; the weight gradients are returned in the SOURCE tensors' shapes.
* callable ``experts_output_postprocess(h3[T, K, D]) -> y[T, K, D]``: applied to the per-route expert outputs before the
  score-weighted top-k sum; its backward runs through PyTorch autograd on the saved graph, so parameters the callable
  closes over accumulate their own gradients.  With ``zero_out_padded_callback_inputs`` the rows of dropped routes are
  zeroed first (``dm_zero_padded_rows``).
* ``RMSNormPostprocess.observe_expert_output_fn(h3[T*K, D])`` sees the pre-norm expert outputs in every forward and in
  the backward's replay of a recomputed layer; ``observe_expert_output_grad_fn(h3, grad_h3)`` sees the saved or
  recomputed expert outputs together with their gradient.  Both are read-only taps for statistics.
* ``wgrad_postprocess_fn(name, grad) -> grad | None``: called as soon as each weight gradient exists; ``None`` means the
  callback took ownership.
* ``wgrad_destination_fn(name, shape, dtype, device) -> (tensor, accumulate)``: names the tensor a weight gradient is
  written (or added) into; nothing is returned to autograd for that weight.
"""

from __future__ import annotations

from typing import Any

import torch

from . import _native as nat
from ._execution import ExecutionOptions


class CallbackHooks:
    """Callback points of one call; ``forward_impl`` / ``backward_impl`` invoke them where the reference does."""

    def __init__(self, options: ExecutionOptions):
        self.options = options

    # ---- callable post-process -----------------------------------------------------------------------------
    def postprocess_forward(self, state, call, post, scores, ids, out, *, save: bool) -> None:
        cfg = state.config
        T, K, D = out.shape[0], cfg.top_k, cfg.hidden_dim
        st = nat.stream_ptr()
        routes = state.combine.local()[: T * K * D * 2].view(torch.bfloat16).view(T, K, D)
        if self.options.zero_out_padded_callback_inputs:
            nat.check(nat.lib.dm_zero_padded_rows(routes.data_ptr(), ids.data_ptr(), int(ids.dtype == torch.int64), T, K, D,
                                                  st), "dm_zero_padded_rows")
        source = routes.clone()  # the callback never sees the communication buffer itself
        if save:
            source.requires_grad_(True)
        with torch.enable_grad() if save else torch.no_grad():
            y = post(source)
        if not isinstance(y, torch.Tensor) or y.shape != source.shape or y.dtype != source.dtype \
                or y.device != source.device or not y.is_contiguous():
            raise ValueError("experts_output_postprocess must preserve shape, dtype, device and contiguity")
        nat.check(nat.lib.dm_scale_and_sum(y.data_ptr(), scores.data_ptr(), int(scores.dtype == torch.bfloat16),
                                           ids.data_ptr(), int(ids.dtype == torch.int64), out.data_ptr(), T, K, D, None,
                                           None, None, 0, st), "dm_scale_and_sum(callback)")
        call.callback_state = (source, y) if save else None

    def postprocess_backward(self, state, call, grad_out, scores, ids, grad_scores) -> None:
        source, y = call.callback_state
        T, K, D = y.shape
        grad_y = torch.empty_like(y)
        nat.check(nat.lib.dm_broadcast_and_scale(grad_out.data_ptr(), scores.data_ptr(), int(scores.dtype == torch.bfloat16),
                                                 ids.data_ptr(), int(ids.dtype == torch.int64), y.data_ptr(), None,
                                                 grad_y.data_ptr(), nat.ptr(grad_scores), T, K, D, nat.stream_ptr()),
                  "dm_broadcast_and_scale(callback)")
        torch.autograd.backward(y, grad_y)  # nested backward: fills source.grad and the callable's own parameters
        grad_routes = source.grad if source.grad is not None else torch.zeros_like(source)
        state.combine.local()[: T * K * D * 2].view(torch.bfloat16).view(T, K, D).copy_(grad_routes)
        call.callback_state = None

    # ---- observers of the fused RMSNorm post-process (dist_moe/_postprocess.py:1245-1256, 1385-1412) --------
    def _routes(self, state, T):
        cfg = state.config
        K, D = cfg.top_k, cfg.hidden_dim
        return state.combine.local()[: T * K * D * 2].view(torch.bfloat16).view(T * K, D)

    def observe_expert_output(self, state, post, ids, T) -> None:
        """The pre-norm expert outputs [T*K, D], as they sit in the combine buffer (read-only for the observer)."""
        fn = post.observe_expert_output_fn
        if fn is None:
            return
        routes = self._routes(state, T)
        if self.options.zero_out_padded_callback_inputs:
            cfg = state.config
            nat.check(nat.lib.dm_zero_padded_rows(routes.data_ptr(), ids.data_ptr(), int(ids.dtype == torch.int64), T,
                                                  cfg.top_k, cfg.hidden_dim, nat.stream_ptr()), "dm_zero_padded_rows")
        fn(routes)

    def preserved_expert_output(self, state, post, ids, T):
        """A copy of the expert outputs for the gradient observer: the fused backward then reads it and writes the
        gradient to the combine buffer instead of working in place.  None when there is no such observer."""
        if post.observe_expert_output_grad_fn is None:
            return None
        kept = self._routes(state, T).clone()
        if self.options.zero_out_padded_callback_inputs:
            cfg = state.config
            nat.check(nat.lib.dm_zero_padded_rows(kept.data_ptr(), ids.data_ptr(), int(ids.dtype == torch.int64), T,
                                                  cfg.top_k, cfg.hidden_dim, nat.stream_ptr()), "dm_zero_padded_rows")
        return kept

    def observe_expert_output_grad(self, state, post, kept, T) -> None:
        post.observe_expert_output_grad_fn(kept, self._routes(state, T))

    # ---- weight gradients --------------------------------------------------------------------------------------
    def wgrad_destination(self, name: str, shape, dtype: torch.dtype, device):
        """(tensor, accumulate) from ``wgrad_destination_fn``, validated; None when there is no such callback."""
        fn = self.options.wgrad_destination_fn
        if fn is None:
            return None
        dst, accumulate = fn(name, tuple(shape), dtype, device)
        if not isinstance(dst, torch.Tensor) or tuple(dst.shape) != tuple(shape) or dst.dtype != dtype \
                or dst.device != device or not dst.is_contiguous():
            raise ValueError("wgrad_destination_fn must return a contiguous tensor of the requested shape, dtype and device")
        return dst, bool(accumulate)

    def wgrad_postprocess(self, name: str, grad):
        fn = self.options.wgrad_postprocess_fn
        if fn is None or grad is None:
            return grad
        out = fn(name, grad)
        if out is None:
            return None
        if not isinstance(out, torch.Tensor) or out.shape != grad.shape or out.device != grad.device \
                or not out.is_contiguous() or out.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("wgrad_postprocess_fn must return None or a contiguous BF16/FP32 tensor of the same shape "
                             "and device")
        return out


def _compute_weights(options: ExecutionOptions, w13_source, w2_source, state):
    cfg = state.config
    fn = options.weights_preprocess_fn
    with torch.no_grad():
        w13 = fn(w13_source) if fn is not None else w13_source.detach()
        w2 = fn(w2_source) if fn is not None else w2_source.detach()
    for name, w in (("w13", w13), ("w2", w2)):
        if not isinstance(w, torch.Tensor) or w.dtype != torch.bfloat16 or w.device.type != "cuda" or not w.is_contiguous():
            raise ValueError(f"weights_preprocess_fn must return a contiguous CUDA bfloat16 tensor ({name})")
    w13 = w13.reshape(state.e_local, 2 * cfg.intermediate_dim, cfg.hidden_dim)
    w2 = w2.reshape(state.e_local, cfg.hidden_dim, cfg.intermediate_dim)
    return w13, w2


class _EagerBf16Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ids, scores, w13_source, w2_source, state, options):
        from ._bf16 import forward_impl

        hooks = CallbackHooks(options)
        w13, w2 = _compute_weights(options, w13_source, w2_source, state)
        out, call = forward_impl(state, x.detach().contiguous(), ids, scores.detach(), w13, w2, options, True, hooks=hooks)
        ctx.state, ctx.call, ctx.options, ctx.hooks, ctx.x_shape = state, call, options, hooks, x.shape
        ctx.save_for_backward(ids, scores, w13_source, w2_source)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from ._bf16 import backward_impl

        ids, scores, w13_source, w2_source = ctx.saved_tensors
        state, options = ctx.state, ctx.options
        w13, w2 = _compute_weights(options, w13_source, w2_source, state)  # materialised again, as in the forward
        needs = (ctx.needs_input_grad[0], ctx.needs_input_grad[2], ctx.needs_input_grad[3], ctx.needs_input_grad[4])
        with torch.cuda.device(state.device):
            gx, gs, g13, g2 = backward_impl(state, ctx.call, ctx.x_shape, ids, scores.detach(), w13, w2, w13, w2,
                                            grad_out.contiguous(), options, needs, hooks=ctx.hooks)
        if g13 is not None:
            g13 = g13.reshape(w13_source.shape)
        if g2 is not None:
            g2 = g2.reshape(w2_source.shape)
        return gx, None, gs, g13, g2, None, None


def run_bf16_eager(x, ids, scores, w13_source, w2_source, context: Any, options: ExecutionOptions, *,
                   save_for_backward: bool) -> torch.Tensor:
    from ._bf16 import forward_impl

    state = context._state
    if options.inplace_wgrad_accum and options.weights_preprocess_fn is not None:
        raise ValueError("inplace_wgrad_accum needs compute weights that own their gradient; it cannot be combined with "
                         "weights_preprocess_fn")
    if save_for_backward:
        return _EagerBf16Function.apply(x, ids, scores, w13_source, w2_source, state, options)
    w13, w2 = _compute_weights(options, w13_source, w2_source, state)
    out, _ = forward_impl(state, x.detach().contiguous(), ids, scores.detach(), w13, w2, options, False,
                          hooks=CallbackHooks(options))
    return out
