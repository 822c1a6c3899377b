"""BF16 routed-expert forward and backward: kernel sequencing and autograd glue.

Launch order follows the reference's BF16 orchestration
(dist_moe/api.py:1844-2188 forward, 2205-2609 backward):

forward   publish -> barrier -> route -> plan -> [save x] -> gather -> W13 (+SwiGLU) ->
          W2 + scatter -> barrier -> weighted top-k reduce (+ save h3)
backward  plan -> [recompute: republish, barrier, gather, W13, SwiGLU, W2 + scatter] ->
          grad_h3 / grad_scores -> barrier -> gather grad_h3 + W2 dgrad -> W2 wgrad ->
          SwiGLU bwd -> W13 dgrad + scatter -> W13 wgrad -> barrier -> reduce

Every data-dependent decision (row counts, arena offsets, save-versus-recompute) stays
on the device: the host never reads a device value, so the sequence can be captured in a
CUDA graph.  Bracketed steps are device-predicated on the planner's decision.
"""

from __future__ import annotations

from typing import Any

import torch
from torch.profiler import record_function

from . import _native as nat
from ._execution import ExecutionOptions, RMSNormPostprocess


# When set to a list, every grouped-GEMM launch is bracketed by CUDA events on the launching
# stream and (name, start, end) is appended; benchmarks use it to time the kernels in place.
PROFILE: list | None = None


def _profiled(fn):
    def call(*args, what: str):
        if PROFILE is None:
            nat.check(fn(*args), what)
            return
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        nat.check(fn(*args), what)
        end.record()
        PROFILE.append((what, start, end))

    return call


_gemm_fprop = _profiled(nat.lib.dm_gemm_fprop)
_gemm_dgrad = _profiled(nat.lib.dm_gemm_dgrad)
_gemm_fprop_dispatch = _profiled(nat.lib.dm_gemm_fprop_dispatch)
_gemm_dgrad_dispatch = _profiled(nat.lib.dm_gemm_dgrad_dispatch)
_gemm_wgrad = _profiled(nat.lib.dm_gemm_wgrad)


# Fused dispatch pulls the routed rows inside the W13 / W2-dgrad GEMM launches (gather warps overlap the peer
# transfer with the tensor cores).  With False the rows are gathered by a separate kernel first.
FUSED_DISPATCH = True
# The plain backward reads saved expert outputs where they were saved (chosen on the device) instead of copying
# them back into the communication buffer first.  False restores the copy.
READ_SAVED_H3_IN_PLACE = True


def _dispatch_fprop(state, ptrs, a_op_off, w, c_op, h2_op, c, N, Kd, fuse, act, condp, what):
    clamped, alpha, limit = act
    st, status = nat.stream_ptr(), state.status.data_ptr()
    if FUSED_DISPATCH:
        _gemm_fprop_dispatch(ptrs.data_ptr(), state.gather_flags.data_ptr(), _op(state, a_op_off), w.data_ptr(), c_op,
                             h2_op, c.offsets.data_ptr(), state.e_local, c.max_rows, N, Kd, int(fuse), clamped, alpha,
                             limit, condp, state.num_sms, status, st, what=what)
        return
    nat.check(nat.lib.dm_gather_rows(ptrs.data_ptr(), c.recv_rows.data_ptr(), state.arena.data_ptr(),
                                     a_op_off.data_ptr(), Kd * 2, c.max_rows, condp, st), "dm_gather_rows")
    _gemm_fprop(_op(state, a_op_off), w.data_ptr(), c_op, h2_op, None, c.offsets.data_ptr(), state.e_local,
                c.max_rows, N, Kd, int(fuse), clamped, alpha, limit, condp, state.num_sms, status, st, what=what)


class _Call:
    """Per-call device tensors produced by routing and planning."""

    __slots__ = ("T", "counts", "per_rank", "offsets", "recv_rows", "fwd", "bwd", "sct", "need", "cond", "fwd_state",
                 "max_rows", "rstd", "callback_state")


def _op(state, t: torch.Tensor | None) -> nat.Operand:
    return state.arena_operand(t)


def _none() -> nat.Operand:
    return nat.Operand(None, 0, None)


def _act(config) -> tuple[int, float, float]:
    return (1 if config.activation == "swiglu_clamped" else 0, float(config.swiglu_alpha), float(config.swiglu_limit))


def _route_and_plan(state, x, ids, scratch_only: bool, validate: bool) -> _Call:
    cfg = state.config
    T, D, K, E = x.shape[0], cfg.hidden_dim, cfg.top_k, cfg.num_experts
    dev, st = x.device, nat.stream_ptr()
    el, ep = state.e_local, state.ep
    with record_function("dist_moe_preprocess"):  # publish ids and rows, then the barrier every peer waits on
        nat.check(nat.lib.dm_publish(x.data_ptr(), ids.data_ptr(), int(ids.dtype == torch.int64),
                                     state.dispatch.local().data_ptr(), state.routing.local().data_ptr(), T, D, K, E,
                                     int(validate), state.status.data_ptr(), st), "dm_publish")
        state.barrier(state.dispatch)
    c = _Call()
    c.T = T
    size = ep * el * T
    c.counts = torch.empty(el, dtype=torch.int32, device=dev)
    c.per_rank = torch.empty(ep, dtype=torch.int32, device=dev)
    c.offsets = torch.empty(el + 1, dtype=torch.int32, device=dev)
    c.fwd = torch.empty(size, dtype=torch.int64, device=dev)
    c.bwd = None if scratch_only else torch.empty(size, dtype=torch.int64, device=dev)
    c.sct = torch.empty(size, dtype=torch.int64, device=dev)
    c.max_rows = min(size, state.capacity_rows)
    stride = D * 2
    nat.check(nat.lib.dm_route(state.routing.peer_ptrs.data_ptr(), state.dispatch.peer_ptrs.data_ptr(),
                               state.combine.peer_ptrs.data_ptr(), state.rank, ep, T, K, E, stride, stride, stride, 0,
                               state.capacity_rows, size, c.counts.data_ptr(), c.per_rank.data_ptr(),
                               c.offsets.data_ptr(), c.fwd.data_ptr(), nat.ptr(c.bwd), c.sct.data_ptr(),
                               state.route_workspace.data_ptr(), state.route_workspace_words,
                               state.status.data_ptr(), st), nat.route_call_name(ep, T, el))
    c.recv_rows = c.offsets[el:]
    c.need = torch.empty(1, dtype=torch.uint8, device=dev)
    c.cond = torch.empty(1, dtype=torch.int32, device=dev)
    c.fwd_state = torch.empty(6, dtype=torch.int64, device=dev)
    nat.check(nat.lib.dm_plan_fwd_bf16(c.recv_rows.data_ptr(), c.per_rank.data_ptr(), state.saved_bytes.data_ptr(),
                                       state.buffer_offsets.data_ptr(), state.peak_min_free.data_ptr(),
                                       c.need.data_ptr(), c.cond.data_ptr(), c.fwd_state.data_ptr(),
                                       state.slot_selector.data_ptr(), state.moe_layer_id.data_ptr(), ep,
                                       cfg.max_num_local_input_tokens, K, D, cfg.intermediate_dim,
                                       state.slot_bytes, state.num_slots, state.num_layers_in_slot,
                                       int(scratch_only), state.status.data_ptr(), st), "dm_plan_fwd_bf16")
    c.rstd = None
    c.callback_state = None
    state.last_call = c
    return c


def _expert_forward(state, c: _Call, w13, w2, xg_off, h1_off, h2_off, *, fuse: bool, cond, clip, clip_limit) -> None:
    """gather -> W13 (+SwiGLU) -> W2 + scatter into the owners' combine buffers."""
    cfg = state.config
    D, F, el = cfg.hidden_dim, cfg.intermediate_dim, state.e_local
    st, status = nat.stream_ptr(), state.status.data_ptr()
    clamped, alpha, limit = _act(cfg)
    condp = nat.ptr(cond)
    # dispatch + W13: gather warps pull the routed rows (peer loads) while the tensor cores run
    _dispatch_fprop(state, c.fwd, xg_off, w13, _op(state, h1_off), _op(state, h2_off) if fuse else _none(), c, 2 * F, D,
                    fuse, (clamped, alpha, limit), condp, "gemm_fprop_dispatch(w13)")
    if not fuse:
        nat.check(nat.lib.dm_swiglu_fwd(state.arena.data_ptr(), h1_off.data_ptr(), state.arena.data_ptr(),
                                        h2_off.data_ptr(), c.recv_rows.data_ptr(), c.max_rows, F, clamped, alpha,
                                        limit, nat.ptr(clip), float(clip_limit), None, st), "dm_swiglu_fwd")
    _gemm_fprop(_op(state, h2_off), w2.data_ptr(), _none(), _none(), c.sct.data_ptr(),
                                    c.offsets.data_ptr(), el, c.max_rows, D, F, 0, 0, 1.0, 0.0, condp, state.num_sms,
                                    status, st, what="gemm_fprop(w2)")


def forward_impl(state, x, ids, scores, w13, w2, options: ExecutionOptions, save_for_backward: bool, hooks=None):
    cfg = state.config
    T, D, K, F = x.shape[0], cfg.hidden_dim, cfg.top_k, cfg.intermediate_dim
    st = nat.stream_ptr()
    scratch_only = (not save_for_backward) or cfg.inference or state.num_slots == 0
    with record_function("dist_moe_routing"):  # the reference's profiler range names (dist_moe/api.py:1979-2072)
        c = _route_and_plan(state, x, ids, scratch_only, options.validate_expert_ids)
    fs = c.fwd_state
    if not scratch_only:
        nat.check(nat.lib.dm_cond_copy(x.data_ptr(), None, state.arena.data_ptr(), fs[0:1].data_ptr(), T * D * 2,
                                       c.cond.data_ptr(), 1, st), "dm_cond_copy(save x)")
    clip = options.swiglu_clip_stats_out_3
    if clip is not None:
        clip.zero_()
    fuse = clip is None and F % 128 == 0
    with record_function("dist_moe_forward"):
        _expert_forward(state, c, w13, w2, fs[1:2], fs[2:3], fs[3:4], fuse=fuse, cond=None, clip=clip,
                        clip_limit=options.swiglu_clip_limit)
    state.barrier(state.combine)
    out = torch.empty(T, D, dtype=torch.bfloat16, device=x.device)
    post = options.experts_output_postprocess
    if isinstance(post, RMSNormPostprocess):
        from ._postprocess import rmsnorm_combine_forward

        if hooks is not None:
            hooks.observe_expert_output(state, post, ids, T)
        c.rstd = rmsnorm_combine_forward(state, c, post, scores, ids, out, save=not scratch_only,
                                         observers_allowed=hooks is not None)
    elif post is not None:
        if hooks is None:
            raise RuntimeError("a callable expert-output post-process runs on the eager path only")
        hooks.postprocess_forward(state, c, post, scores, ids, out, save=not scratch_only)
    else:
        nat.check(nat.lib.dm_scale_and_sum(state.combine.local().data_ptr(), scores.data_ptr(),
                                           int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                           int(ids.dtype == torch.int64), out.data_ptr(), T, K, D,
                                           None if scratch_only else state.arena.data_ptr(),
                                           None if scratch_only else fs[4:5].data_ptr(),
                                           None if scratch_only else c.cond.data_ptr(), 0, st), "dm_scale_and_sum")
    return out, c


def _wgrad_destination(param: torch.Tensor, shape, options: ExecutionOptions, cfg, owner: torch.Tensor | None,
                       explicit=None, hooks=None, name: str = ""):
    """Return (tensor, accumulate, returned_to_autograd).

    ``explicit`` is used by the registered operators: a tensor to accumulate into, or a dtype for a fresh result.
    ``hooks`` (eager path) may name the destination through ``wgrad_destination_fn``.
    """
    if hooks is not None:
        named = hooks.wgrad_destination(name, shape, cfg.wgrad_dtype or param.dtype, param.device)
        if named is not None:
            return named[0], int(named[1]), False
    if isinstance(explicit, torch.Tensor):
        if not explicit.is_contiguous() or explicit.dtype not in (torch.bfloat16, torch.float32) \
                or explicit.numel() != param.numel():
            raise ValueError("WGRAD accumulators must be contiguous BF16 or FP32 tensors of the weight's size")
        return explicit, 1, False
    if isinstance(explicit, torch.dtype):
        if explicit not in (torch.bfloat16, torch.float32):
            raise ValueError("wgrad_output_dtype must be torch.bfloat16 or torch.float32")
        return torch.empty(shape, dtype=explicit, device=param.device), 0, True
    if options.inplace_wgrad_accum:
        target = owner if owner is not None else param
        if target.grad is None:
            dtype = cfg.wgrad_dtype or getattr(target, "grad_dtype", None) or target.dtype
            if dtype != target.dtype and hasattr(target, "grad_dtype"):
                target.grad_dtype = dtype
            target.grad = torch.zeros_like(target, dtype=dtype)
        grad = target.grad
        if not grad.is_contiguous() or grad.dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("in-place WGRAD accumulation needs a contiguous BF16 or FP32 parameter.grad")
        if grad.numel() != param.numel():
            raise ValueError("WGRAD owner gradient does not match the compute weight size")
        return grad, 1, False
    dtype = cfg.wgrad_dtype or param.dtype
    return torch.empty(shape, dtype=dtype, device=param.device), 0, True


def backward_impl(state, c: _Call, x_shape, ids, scores, w13, w2, w13_param, w2_param, grad_out,
                  options: ExecutionOptions, needs, wgrad_explicit=(None, None), hooks=None):
    cfg = state.config
    T, D, K, F, el = c.T, cfg.hidden_dim, cfg.top_k, cfg.intermediate_dim, state.e_local
    dev, st, status = grad_out.device, nat.stream_ptr(), state.status.data_ptr()
    clamped, alpha, limit = _act(cfg)
    need_x, need_scores, need_w13, need_w2 = needs
    bo = torch.empty(6, dtype=torch.int64, device=dev)  # [xg, h1, h2, grad_h2, grad_h3_gathered, grad_h1]
    nat.check(nat.lib.dm_plan_bwd_bf16(c.recv_rows.data_ptr(), c.per_rank.data_ptr(), state.saved_bytes.data_ptr(),
                                       state.buffer_offsets.data_ptr(), state.peak_min_free.data_ptr(),
                                       c.need.data_ptr(), c.fwd_state.data_ptr(), bo.data_ptr(),
                                       state.moe_layer_id.data_ptr(), state.ep, cfg.max_num_local_input_tokens, K, D,
                                       F, state.slot_bytes, state.num_slots, status, st), "dm_plan_bwd_bf16")
    fs, cond = c.fwd_state, c.cond
    arena = state.arena.data_ptr()
    post = options.experts_output_postprocess
    is_norm = isinstance(post, RMSNormPostprocess)
    is_callback = post is not None and not is_norm  # the callable kept its own input and output (eager path)
    # ---- recompute block (device-predicated on need_recompute) ----------------
    span = record_function("dist_moe_recompute")
    span.__enter__()
    nat.check(nat.lib.dm_cond_copy(arena, fs[0:1].data_ptr(), state.dispatch.local().data_ptr(), None, T * D * 2,
                                   cond.data_ptr(), 1, st), "dm_cond_copy(republish x)")
    state.barrier(state.dispatch, cond)
    _dispatch_fprop(state, c.fwd, bo[0:1], w13, _op(state, bo[1:2]), _none(), c, 2 * F, D, False,
                    (clamped, alpha, limit), cond.data_ptr(), "gemm_fprop_dispatch(w13 recompute)")
    # h2 is always rebuilt from h1: only x_gathered, h1 and h3 are ever saved.
    nat.check(nat.lib.dm_swiglu_fwd(arena, bo[1:2].data_ptr(), arena, bo[2:3].data_ptr(), c.recv_rows.data_ptr(),
                                    c.max_rows, F, clamped, alpha, limit, None, 0.0, None, st), "dm_swiglu_fwd(bwd)")
    need_h3 = (need_scores or is_norm) and not is_callback
    if need_h3:
        _gemm_fprop(_op(state, bo[2:3]), w2.data_ptr(), _none(), _none(), c.sct.data_ptr(),
                                        c.offsets.data_ptr(), el, c.max_rows, D, F, 0, 0, 1.0, 0.0, cond.data_ptr(),
                                        state.num_sms, status, st, what="gemm_fprop(w2 recompute)")
        # Saved path: the fused RMSNorm backward works on the expert outputs in place in the communication buffer,
        # so they are copied back there; the plain backward reads them where they were saved (selected on the device).
        if is_norm or not READ_SAVED_H3_IN_PLACE:
            nat.check(nat.lib.dm_cond_copy(arena, fs[4:5].data_ptr(), state.combine.local().data_ptr(), None,
                                           T * K * D * 2, cond.data_ptr(), 0, st), "dm_cond_copy(load h3)")
        state.barrier(state.combine, cond)
    span.__exit__(None, None, None)
    span = record_function("dist_moe_backward")
    span.__enter__()
    # ---- grad wrt expert outputs and scores ------------------------------------
    grad_scores = torch.empty(T, K, dtype=torch.float32, device=dev) if need_scores else None
    combine = state.combine.local().data_ptr()
    if is_norm:
        from ._postprocess import rmsnorm_combine_backward

        kept = None
        if hooks is not None:
            # the replay of a recomputed layer shows its expert outputs to the forward observer again; whether the
            # layer was recomputed is a device-side decision, read here because observers run on the host anyway
            if post.observe_expert_output_fn is not None and bool(c.need.item()):
                hooks.observe_expert_output(state, post, ids, T)
            kept = hooks.preserved_expert_output(state, post, ids, T)
        rmsnorm_combine_backward(state, c, post, grad_out, scores, ids, grad_scores, h3=kept)
        if kept is not None:
            hooks.observe_expert_output_grad(state, post, kept, T)
    elif is_callback:
        hooks.postprocess_backward(state, c, grad_out, scores, ids, grad_scores)
    else:
        if need_scores and READ_SAVED_H3_IN_PLACE:
            nat.check(nat.lib.dm_broadcast_and_scale_select(grad_out.data_ptr(), scores.data_ptr(),
                                                            int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                                            int(ids.dtype == torch.int64), arena, fs[4:5].data_ptr(),
                                                            combine, cond.data_ptr(), combine, nat.ptr(grad_scores), T,
                                                            K, D, st), "dm_broadcast_and_scale")
        else:
            nat.check(nat.lib.dm_broadcast_and_scale(grad_out.data_ptr(), scores.data_ptr(),
                                                     int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                                     int(ids.dtype == torch.int64), combine if need_scores else None,
                                                     None, combine, nat.ptr(grad_scores), T, K, D, st),
                      "dm_broadcast_and_scale")
    state.barrier(state.combine)
    # ---- W2: input gradient and weight gradient ----------------------------------
    if FUSED_DISPATCH:
        _gemm_dgrad_dispatch(c.sct.data_ptr(), state.gather_flags.data_ptr(), _op(state, bo[4:5]), w2.data_ptr(),
                             _op(state, bo[3:4]), c.offsets.data_ptr(), el, c.max_rows, F, D, None, state.num_sms,
                             status, st, what="gemm_dgrad_dispatch(w2)")
    else:
        nat.check(nat.lib.dm_gather_rows(c.sct.data_ptr(), c.recv_rows.data_ptr(), arena, bo[4:5].data_ptr(), D * 2,
                                         c.max_rows, None, st), "dm_gather_rows(grad_h3)")
        _gemm_dgrad(_op(state, bo[4:5]), w2.data_ptr(), _op(state, bo[3:4]), None, c.offsets.data_ptr(), el,
                    c.max_rows, F, D, None, state.num_sms, status, st, what="gemm_dgrad(w2)")
    grad_w13 = grad_w2 = None
    owners = options.wgrad_parameter_owners or (None, None)
    if need_w2:
        dst, acc, ret = _wgrad_destination(w2_param, (el, D, F), options, cfg, owners[1], wgrad_explicit[1], hooks, "w2")
        _gemm_wgrad(_op(state, bo[4:5]), _op(state, bo[2:3]), dst.data_ptr(),
                                        int(dst.dtype == torch.float32), acc, c.offsets.data_ptr(), el, c.max_rows,
                                        D, F, state.num_sms, status, st, what="gemm_wgrad(w2)")
        grad_w2 = dst.view(w2_param.shape) if ret else None
        if hooks is not None:
            grad_w2 = hooks.wgrad_postprocess("w2", grad_w2)
    # ---- SwiGLU backward, W13 input gradient (scattered to the owners) and weight gradient
    nat.check(nat.lib.dm_swiglu_bwd(arena, bo[1:2].data_ptr(), arena, bo[3:4].data_ptr(), arena, bo[5:6].data_ptr(),
                                    c.recv_rows.data_ptr(), c.max_rows, F, clamped, alpha, limit, st),
              "dm_swiglu_bwd")
    if need_x:
        _gemm_dgrad(_op(state, bo[5:6]), w13.data_ptr(), _none(), c.bwd.data_ptr(),
                                        c.offsets.data_ptr(), el, c.max_rows, D, 2 * F, None, state.num_sms, status,
                                        st, what="gemm_dgrad(w13)")
    if need_w13:
        dst, acc, ret = _wgrad_destination(w13_param, (el, 2 * F, D), options, cfg, owners[0], wgrad_explicit[0], hooks,
                                           "w13")
        _gemm_wgrad(_op(state, bo[5:6]), _op(state, bo[0:1]), dst.data_ptr(),
                                        int(dst.dtype == torch.float32), acc, c.offsets.data_ptr(), el, c.max_rows,
                                        2 * F, D, state.num_sms, status, st, what="gemm_wgrad(w13)")
        grad_w13 = dst.view(w13_param.shape) if ret else None
        if hooks is not None:
            grad_w13 = hooks.wgrad_postprocess("w13", grad_w13)
    grad_x = None
    # The closing barrier is unconditional (dist_moe/api.py:2580): peers may still be pulling grad_h3 out of this
    # rank's combine buffer, and the next call on this context overwrites it.
    state.barrier(state.dispatch)
    if need_x:
        grad_x = torch.empty(x_shape, dtype=torch.bfloat16, device=dev)
        nat.check(nat.lib.dm_scale_and_sum(state.dispatch.local().data_ptr(), None, 0, ids.data_ptr(),
                                           int(ids.dtype == torch.int64), grad_x.data_ptr(), T, K, D, None, None,
                                           None, 0, st), "dm_scale_and_sum(reduce_from_topk)")
    if grad_scores is not None and scores.dtype != torch.float32:
        grad_scores = grad_scores.to(scores.dtype)
    span.__exit__(None, None, None)
    return grad_x, grad_scores, grad_w13, grad_w2


class _Bf16Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ids, scores, w13_param, w2_param, state, options):
        cfg = state.config
        w13 = w13_param.detach().reshape(state.e_local, 2 * cfg.intermediate_dim, cfg.hidden_dim)
        w2 = w2_param.detach().reshape(state.e_local, cfg.hidden_dim, cfg.intermediate_dim)
        out, call = forward_impl(state, x.detach(), ids, scores.detach(), w13, w2, options, True)
        ctx.state, ctx.call, ctx.options = state, call, options
        ctx.x_shape = x.shape
        ctx.save_for_backward(ids, scores, w13_param, w2_param)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        ids, scores, w13_param, w2_param = ctx.saved_tensors
        state, cfg = ctx.state, ctx.state.config
        w13 = w13_param.detach().reshape(state.e_local, 2 * cfg.intermediate_dim, cfg.hidden_dim)
        w2 = w2_param.detach().reshape(state.e_local, cfg.hidden_dim, cfg.intermediate_dim)
        needs = (ctx.needs_input_grad[0], ctx.needs_input_grad[2], ctx.needs_input_grad[3], ctx.needs_input_grad[4])
        with torch.cuda.device(state.device):
            gx, gs, gw13, gw2 = backward_impl(state, ctx.call, ctx.x_shape, ids, scores.detach(), w13, w2, w13_param,
                                              w2_param, grad_out.contiguous(), ctx.options, needs)
        return gx, None, gs, gw13, gw2, None, None


def _rmsnorm_args(post):
    """The RMSNorm arguments of the registered operators (weight, enabled, eps, norm dtype, output dtype, bitwise,
    gain centre, Kahan, recompute rstd); disabled values when there is no RMSNorm post-process."""
    if isinstance(post, RMSNormPostprocess):
        return (post.weight, True, float(post.eps), post.norm_output_dtype, post.output_dtype, bool(post.require_bitwise),
                float(post.gain_center), bool(post.use_kahan), bool(post.recompute_rstd))
    return (None, False, 1e-6, torch.float32, torch.bfloat16, False, 0.0, False, False)


class _RegisteredBf16Function(torch.autograd.Function):
    """Training call through the registered operators ``dist_moe::bf16_forward`` (``..._with_clip_stats``) and
    ``dist_moe::bf16_backward`` / ``bf16_backward_accumulate_`` (dist_moe/api.py:4027-4042 applies its
    ``_RegisteredBf16Autograd`` the same way), so that FakeTensor propagation, ``make_fx`` and ``torch.compile`` of
    the caller's code see operator nodes with the reference's names and schemas."""

    @staticmethod
    def forward(ctx, x, ids, scores, w13_param, w2_param, context, options):
        state = context._state
        rms = _rmsnorm_args(options.experts_output_postprocess)
        head = (x.detach().contiguous(), ids, scores.detach(), w13_param.detach(), w2_param.detach(), *rms,
                state.slot_selector, state.num_layers_in_slot, bool(options.validate_expert_ids))
        clip = options.swiglu_clip_stats_out_3
        if clip is None:
            out, st = torch.ops.dist_moe.bf16_forward(*head, context._context_id)
        else:
            out, st, counters = torch.ops.dist_moe.bf16_forward_with_clip_stats(*head, float(options.swiglu_clip_limit),
                                                                                  context._context_id)
            clip.copy_(counters)  # graph-visible copy into the caller's tensor
        ctx.context, ctx.options, ctx.n_state = context, options, len(st)
        ctx.save_for_backward(ids, scores, w13_param, w2_param, *st)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        from . import _ops

        ids, scores, w13_param, w2_param, *st = ctx.saved_tensors
        context, options = ctx.context, ctx.options
        cfg = context.config
        rms = _rmsnorm_args(options.experts_output_postprocess)
        tail = (rms[1], rms[2], rms[3], rms[4], rms[5], rms[7], rms[8])
        needs = (ctx.needs_input_grad[0], ctx.needs_input_grad[2], ctx.needs_input_grad[3], ctx.needs_input_grad[4])
        e_local = context._state.e_local
        D, F = cfg.hidden_dim, cfg.intermediate_dim
        _ops.NEEDS_HINT.append(needs)
        try:
            if options.inplace_wgrad_accum:
                owners = options.wgrad_parameter_owners or (None, None)
                acc13, _, _ = _wgrad_destination(w13_param, (e_local, 2 * F, D), options, cfg, owners[0])
                acc2, _, _ = _wgrad_destination(w2_param, (e_local, D, F), options, cfg, owners[1])
                gx, gs = torch.ops.dist_moe.bf16_backward_accumulate_(
                    grad_out.contiguous(), w13_param.detach(), w2_param.detach(), acc13, acc2, ids, scores.detach(), st,
                    *tail, acc13.dtype, context._context_id)
                g13 = g2 = None
            else:
                dtype = cfg.wgrad_dtype or w13_param.dtype
                gx, gs, g13, g2 = torch.ops.dist_moe.bf16_backward(
                    grad_out.contiguous(), w13_param.detach(), w2_param.detach(), ids, scores.detach(), st, *tail, dtype,
                    context._context_id)
        finally:
            _ops.NEEDS_HINT.clear()
        if gs is not None and needs[1] and gs.dtype != scores.dtype:
            gs = gs.to(scores.dtype)
        return (gx if needs[0] else None, None, gs if needs[1] else None, g13 if needs[2] else None,
                g2 if needs[3] else None, None, None)


def _registered_ops_are_ours() -> bool:
    from . import _ops

    return "bf16_forward" in _ops.REGISTERED


def run_bf16(x, ids, scores, w13_weight, w2_weight, w13_EFD, w2_EDF, context: Any, options: ExecutionOptions, *,
             save_for_backward: bool) -> torch.Tensor:
    state = context._state
    if options.requires_eager:
        from ._eager import run_bf16_eager

        return run_bf16_eager(x, ids, scores, w13_weight, w2_weight, context, options, save_for_backward=save_for_backward)
    if save_for_backward:
        if _registered_ops_are_ours():
            return _RegisteredBf16Function.apply(x, ids, scores, w13_weight, w2_weight, context, options)
        return _Bf16Function.apply(x, ids, scores, w13_weight, w2_weight, state, options)
    out, _ = forward_impl(state, x.detach(), ids, scores.detach(), w13_EFD.detach(), w2_EDF.detach(), options, False)
    return out
