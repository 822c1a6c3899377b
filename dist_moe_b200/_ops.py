"""Registered ``dist_moe::*`` operators: what FakeTensor propagation, ``make_fx`` and CUDA-graph capture see.

Same operator names, argument names, argument order and mutation annotations as the reference
(dist_moe/api.py:2614-2626 ``bf16``; 2898-2922 ``bf16_forward``; 3100-3125 ``bf16_forward_with_clip_stats``;
3358-3379 ``bf16_backward``; 3401-3424 ``bf16_backward_accumulate_``; dist_moe/_blockscaled.py:140-144
``prepare_nvfp4_weight``; 2870-2882 ``prepare_mxfp8_weight``; 3421-3448 ``block_scaled_forward``; 3807-3828
``block_scaled_backward``; 3850-3873 ``block_scaled_backward_accumulate_``).  The context travels as a string
id that is resolved in a process-local table (dist_moe/_context.py:20-58).

The training forwards return ``(output, state)``; ``state`` is a fixed-length tensor list that the backward
operators take back.  BF16 state (9 tensors, the reference's order, dist_moe/api.py:3273-3285):
rows per local expert ``int32[E_local]``, backward gather pointers, forward gather pointers, scatter pointers
(``int64[P]`` each), rows per rank ``int32[EP]``, rows received ``int32[1]``, recompute flag ``uint8[1]``,
planner state ``int64[6]``, rstd ``fp32[T, K]`` (empty without RMSNorm).

Importing this module registers the operators once per process; if another library already defined an
operator of the same name (the reference imported next to this package) that definition is left alone.
"""

from __future__ import annotations

import torch

from ._execution import ExecutionOptions, PreparedWeight, RMSNormPostprocess
from .formats import BlockScaledFormat

_NS = "dist_moe"
REGISTERED: list[str] = []


def _context(context_id: str):
    from .api import _CONTEXTS

    ctx = _CONTEXTS.get(context_id)
    if ctx is None or ctx._closed:
        raise RuntimeError(f"distributed MoE context {context_id} is not live")
    return ctx


def _rmsnorm(weight, enabled, eps, norm_dtype, out_dtype, require_bitwise, gain_center, use_kahan, recompute_rstd):
    if not enabled:
        return None
    return RMSNormPostprocess(eps=eps, norm_output_dtype=norm_dtype, output_dtype=out_dtype,
                              require_bitwise=require_bitwise, weight=weight, gain_center=gain_center,
                              use_kahan=use_kahan, recompute_rstd=recompute_rstd)


def _select_slot(state, activation_slot_id_1: torch.Tensor, num_moe_layers_in_slot: int) -> None:
    if state.num_slots:
        state.slot_selector.copy_(activation_slot_id_1.reshape(1).to(torch.int64))
        state.num_layers_in_slot = int(num_moe_layers_in_slot)


# ---------------------------------------------------------------------------------------------
# BF16
# ---------------------------------------------------------------------------------------------
# Eager calls hand the forward's per-call record to the matching backward through this table (keyed by the address
# of the call's planner-state tensor), so the backward does not rebuild offsets and predicates with extra launches.
# A backward that finds no entry (a traced graph replayed later, another process) rebuilds them from the state list.
_LIVE_CALLS: dict[int, object] = {}
_LIVE_CALLS_MAX = 256
# Which of (x, scores, w13, w2) need gradients in the backward about to run; set by the autograd function that
# dispatches to the operator, consumed once.  Absent means all four.
NEEDS_HINT: list = []


def _pack_bf16_state(call, device) -> list[torch.Tensor]:
    rstd = call.rstd if call.rstd is not None else torch.empty(0, dtype=torch.float32, device=device)
    if len(_LIVE_CALLS) >= _LIVE_CALLS_MAX:
        _LIVE_CALLS.pop(next(iter(_LIVE_CALLS)))
    _LIVE_CALLS[call.fwd_state.data_ptr()] = call
    return [call.counts, call.bwd, call.fwd, call.sct, call.per_rank, call.recv_rows.clone(), call.need,
            call.fwd_state, rstd]


def _unpack_bf16_state(state, tensors, T: int):
    from ._bf16 import _Call

    if len(tensors) != 9:
        raise RuntimeError(f"BF16 backward received {len(tensors)} state tensors")
    live = _LIVE_CALLS.pop(tensors[7].data_ptr(), None)
    if live is not None and live.T == T and live.fwd.data_ptr() == tensors[2].data_ptr():
        rstd = tensors[8]
        live.rstd = rstd if rstd.numel() else None
        return live
    c = _Call()
    c.counts, c.bwd, c.fwd, c.sct, c.per_rank, recv, c.need, c.fwd_state, rstd = tensors
    c.T = T
    # expert offsets are the exclusive prefix of the per-expert rows; rebuilt on the device
    c.offsets = torch.zeros(state.e_local + 1, dtype=torch.int32, device=c.counts.device)
    c.offsets[1:] = torch.cumsum(c.counts, 0)
    c.recv_rows = recv
    c.cond = c.need.to(torch.int32)
    c.max_rows = min(c.fwd.numel(), state.capacity_rows)
    c.rstd = rstd if rstd.numel() else None
    return c


def _bf16_forward_common(x, ids, scores, w13, w2, post, slot_id, num_layers, validate, context_id, clip, clip_limit):
    from ._bf16 import forward_impl

    ctx = _context(context_id)
    state, cfg = ctx._state, ctx.config
    _select_slot(state, slot_id, num_layers)
    options = ExecutionOptions(validate_expert_ids=validate, experts_output_postprocess=post,
                               swiglu_clip_stats_out_3=clip, swiglu_clip_limit=clip_limit)
    w13 = w13.reshape(state.e_local, 2 * cfg.intermediate_dim, cfg.hidden_dim)
    w2 = w2.reshape(state.e_local, cfg.hidden_dim, cfg.intermediate_dim)
    out, call = forward_impl(state, x.contiguous(), ids, scores, w13, w2, options, True)
    return out, _pack_bf16_state(call, x.device)


def _fake_bf16_state(x, ids, context_id, rmsnorm_enabled):
    ctx = _context(context_id)
    state = ctx._state
    T, K = ids.shape
    P = state.ep * state.e_local * T
    i32, i64 = torch.int32, torch.int64
    return [x.new_empty(state.e_local, dtype=i32), x.new_empty(P, dtype=i64), x.new_empty(P, dtype=i64),
            x.new_empty(P, dtype=i64), x.new_empty(state.ep, dtype=i32), x.new_empty(1, dtype=i32),
            x.new_empty(1, dtype=torch.uint8), x.new_empty(6, dtype=i64),
            x.new_empty((T, K) if rmsnorm_enabled else (0,), dtype=torch.float32)]


def _or_empty(t, like):
    """An operator output cannot be None: a gradient that was not asked for comes back as an (unused) empty-like."""
    return t if t is not None else torch.empty_like(like)


def _register_bf16() -> None:
    @torch.library.custom_op(f"{_NS}::bf16_forward", mutates_args=(), device_types="cuda")
    def bf16_forward(x_TD: torch.Tensor, topk_expert_ids_TK: torch.Tensor, topk_scores_TK: torch.Tensor,
                     w13_EFD: torch.Tensor, w2_EDF: torch.Tensor, rmsnorm_weight_D: torch.Tensor | None,
                     rmsnorm_enabled: bool, rmsnorm_eps: float, rmsnorm_norm_output_dtype: torch.dtype,
                     rmsnorm_output_dtype: torch.dtype, rmsnorm_require_bitwise: bool, rmsnorm_gain_center: float,
                     rmsnorm_use_kahan: bool, rmsnorm_recompute_rstd: bool, activation_slot_id_1: torch.Tensor,
                     num_moe_layers_in_slot: int, validate_expert_ids: bool,
                     context_id: str) -> tuple[torch.Tensor, list[torch.Tensor]]:
        post = _rmsnorm(rmsnorm_weight_D, rmsnorm_enabled, rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype,
                        rmsnorm_require_bitwise, rmsnorm_gain_center, rmsnorm_use_kahan, rmsnorm_recompute_rstd)
        return _bf16_forward_common(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_EFD, w2_EDF, post,
                                    activation_slot_id_1, num_moe_layers_in_slot, validate_expert_ids, context_id,
                                    None, 7.0)

    @bf16_forward.register_fake
    def _(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_EFD, w2_EDF, rmsnorm_weight_D, rmsnorm_enabled, rmsnorm_eps,
          rmsnorm_norm_output_dtype, rmsnorm_output_dtype, rmsnorm_require_bitwise, rmsnorm_gain_center,
          rmsnorm_use_kahan, rmsnorm_recompute_rstd, activation_slot_id_1, num_moe_layers_in_slot,
          validate_expert_ids, context_id):
        return torch.empty_like(x_TD), _fake_bf16_state(x_TD, topk_expert_ids_TK, context_id, rmsnorm_enabled)

    @torch.library.custom_op(f"{_NS}::bf16_forward_with_clip_stats", mutates_args=(), device_types="cuda")
    def bf16_forward_with_clip_stats(x_TD: torch.Tensor, topk_expert_ids_TK: torch.Tensor, topk_scores_TK: torch.Tensor,
                                     w13_EFD: torch.Tensor, w2_EDF: torch.Tensor,
                                     rmsnorm_weight_D: torch.Tensor | None, rmsnorm_enabled: bool, rmsnorm_eps: float,
                                     rmsnorm_norm_output_dtype: torch.dtype, rmsnorm_output_dtype: torch.dtype,
                                     rmsnorm_require_bitwise: bool, rmsnorm_gain_center: float,
                                     rmsnorm_use_kahan: bool, rmsnorm_recompute_rstd: bool,
                                     activation_slot_id_1: torch.Tensor, num_moe_layers_in_slot: int,
                                     validate_expert_ids: bool, swiglu_clip_limit: float,
                                     context_id: str) -> tuple[torch.Tensor, list[torch.Tensor], torch.Tensor]:
        post = _rmsnorm(rmsnorm_weight_D, rmsnorm_enabled, rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype,
                        rmsnorm_require_bitwise, rmsnorm_gain_center, rmsnorm_use_kahan, rmsnorm_recompute_rstd)
        clip = torch.zeros(3, dtype=torch.float32, device=x_TD.device)
        out, st = _bf16_forward_common(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_EFD, w2_EDF, post,
                                       activation_slot_id_1, num_moe_layers_in_slot, validate_expert_ids, context_id,
                                       clip, swiglu_clip_limit)
        return out, st, clip

    @bf16_forward_with_clip_stats.register_fake
    def _(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_EFD, w2_EDF, rmsnorm_weight_D, rmsnorm_enabled, rmsnorm_eps,
          rmsnorm_norm_output_dtype, rmsnorm_output_dtype, rmsnorm_require_bitwise, rmsnorm_gain_center,
          rmsnorm_use_kahan, rmsnorm_recompute_rstd, activation_slot_id_1, num_moe_layers_in_slot,
          validate_expert_ids, swiglu_clip_limit, context_id):
        return (torch.empty_like(x_TD), _fake_bf16_state(x_TD, topk_expert_ids_TK, context_id, rmsnorm_enabled),
                x_TD.new_empty(3, dtype=torch.float32))

    def run_backward(grad_out, w13, w2, ids, scores, state_tensors, post, context_id, explicit):
        from ._bf16 import backward_impl

        ctx = _context(context_id)
        state, cfg = ctx._state, ctx.config
        c = _unpack_bf16_state(state, list(state_tensors), ids.shape[0])
        w13v = w13.reshape(state.e_local, 2 * cfg.intermediate_dim, cfg.hidden_dim)
        w2v = w2.reshape(state.e_local, cfg.hidden_dim, cfg.intermediate_dim)
        options = ExecutionOptions(experts_output_postprocess=post)
        needs = NEEDS_HINT.pop() if NEEDS_HINT else (True, True, True, True)
        return backward_impl(state, c, grad_out.shape, ids, scores, w13v, w2v, w13, w2, grad_out.contiguous(), options,
                             needs, wgrad_explicit=explicit)

    @torch.library.custom_op(f"{_NS}::bf16_backward", mutates_args=(), device_types="cuda")
    def bf16_backward(grad_output_TD: torch.Tensor, w13_EFD: torch.Tensor, w2_EDF: torch.Tensor,
                      topk_expert_ids_TK: torch.Tensor, topk_scores_TK: torch.Tensor,
                      state_tensors: list[torch.Tensor], rmsnorm_enabled: bool, rmsnorm_eps: float,
                      rmsnorm_norm_output_dtype: torch.dtype, rmsnorm_output_dtype: torch.dtype,
                      rmsnorm_require_bitwise: bool, rmsnorm_use_kahan: bool, rmsnorm_recompute_rstd: bool,
                      wgrad_output_dtype: torch.dtype,
                      context_id: str) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        post = _rmsnorm(None, rmsnorm_enabled, rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype,
                        rmsnorm_require_bitwise, 0.0, rmsnorm_use_kahan, rmsnorm_recompute_rstd)
        gx, gs, g13, g2 = run_backward(grad_output_TD, w13_EFD, w2_EDF, topk_expert_ids_TK, topk_scores_TK,
                                       state_tensors, post, context_id, (wgrad_output_dtype, wgrad_output_dtype))
        return (_or_empty(gx, grad_output_TD), _or_empty(gs, topk_scores_TK),
                _or_empty(g13, w13_EFD).reshape(w13_EFD.shape), _or_empty(g2, w2_EDF).reshape(w2_EDF.shape))

    @bf16_backward.register_fake
    def _(grad_output_TD, w13_EFD, w2_EDF, topk_expert_ids_TK, topk_scores_TK, state_tensors, rmsnorm_enabled,
          rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype, rmsnorm_require_bitwise, rmsnorm_use_kahan,
          rmsnorm_recompute_rstd, wgrad_output_dtype, context_id):
        return (torch.empty_like(grad_output_TD), torch.empty_like(topk_scores_TK),
                torch.empty_like(w13_EFD, dtype=wgrad_output_dtype), torch.empty_like(w2_EDF, dtype=wgrad_output_dtype))

    @torch.library.custom_op(f"{_NS}::bf16_backward_accumulate_",
                             mutates_args=("accumulator_grad_w13_EFD", "accumulator_grad_w2_EDF"), device_types="cuda")
    def bf16_backward_accumulate_(grad_output_TD: torch.Tensor, w13_EFD: torch.Tensor, w2_EDF: torch.Tensor,
                                  accumulator_grad_w13_EFD: torch.Tensor, accumulator_grad_w2_EDF: torch.Tensor,
                                  topk_expert_ids_TK: torch.Tensor, topk_scores_TK: torch.Tensor,
                                  state_tensors: list[torch.Tensor], rmsnorm_enabled: bool, rmsnorm_eps: float,
                                  rmsnorm_norm_output_dtype: torch.dtype, rmsnorm_output_dtype: torch.dtype,
                                  rmsnorm_require_bitwise: bool, rmsnorm_use_kahan: bool, rmsnorm_recompute_rstd: bool,
                                  wgrad_output_dtype: torch.dtype, context_id: str) -> tuple[torch.Tensor, torch.Tensor]:
        post = _rmsnorm(None, rmsnorm_enabled, rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype,
                        rmsnorm_require_bitwise, 0.0, rmsnorm_use_kahan, rmsnorm_recompute_rstd)
        gx, gs, _, _ = run_backward(grad_output_TD, w13_EFD, w2_EDF, topk_expert_ids_TK, topk_scores_TK, state_tensors,
                                    post, context_id, (accumulator_grad_w13_EFD, accumulator_grad_w2_EDF))
        return _or_empty(gx, grad_output_TD), _or_empty(gs, topk_scores_TK)

    @bf16_backward_accumulate_.register_fake
    def _(grad_output_TD, w13_EFD, w2_EDF, accumulator_grad_w13_EFD, accumulator_grad_w2_EDF, topk_expert_ids_TK,
          topk_scores_TK, state_tensors, rmsnorm_enabled, rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype,
          rmsnorm_require_bitwise, rmsnorm_use_kahan, rmsnorm_recompute_rstd, wgrad_output_dtype, context_id):
        return torch.empty_like(grad_output_TD), torch.empty_like(topk_scores_TK)

    for op in (bf16_forward, bf16_forward_with_clip_stats, bf16_backward):
        # the device-side activation planner is pushed and popped in call order: keep these ordered
        if hasattr(op, "register_effect") and hasattr(torch.library, "EffectType"):
            op.register_effect(torch.library.EffectType.ORDERED)
    REGISTERED.extend(["bf16_forward", "bf16_forward_with_clip_stats", "bf16_backward", "bf16_backward_accumulate_"])

    # inference operator with explicit storage mutation (schema text of dist_moe/api.py:2615-2626)
    lib = torch.library.Library(_NS, "FRAGMENT")
    lib.define(
        "bf16(Tensor x_TD, Tensor topk_expert_ids_TK, Tensor topk_scores_TK, Tensor w13_EFD, Tensor w2_EDF, "
        "Tensor? rmsnorm_weight_D, bool rmsnorm_enabled, float rmsnorm_eps, "
        "ScalarType rmsnorm_norm_output_dtype, ScalarType rmsnorm_output_dtype, "
        "bool rmsnorm_require_bitwise, float rmsnorm_gain_center, bool rmsnorm_use_kahan, bool rmsnorm_recompute_rstd, "
        "Tensor(a!) activation_storage, Tensor activation_slot_id_1, int num_moe_layers_in_slot, "
        "Tensor(b!) routing_storage, "
        "Tensor(c!) dispatch_storage, Tensor(d!) combine_storage, "
        "Tensor(e!)? swiglu_clip_stats_out_3, float swiglu_clip_limit, "
        "bool validate_expert_ids, str context_id) "
        "-> Tensor")

    def bf16_cuda(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_EFD, w2_EDF, rmsnorm_weight_D, rmsnorm_enabled,
                  rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype, rmsnorm_require_bitwise,
                  rmsnorm_gain_center, rmsnorm_use_kahan, rmsnorm_recompute_rstd, activation_storage,
                  activation_slot_id_1, num_moe_layers_in_slot, routing_storage, dispatch_storage, combine_storage,
                  swiglu_clip_stats_out_3, swiglu_clip_limit, validate_expert_ids, context_id):
        from ._bf16 import forward_impl

        ctx = _context(context_id)
        state, cfg = ctx._state, ctx.config
        post = _rmsnorm(rmsnorm_weight_D, rmsnorm_enabled, rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype,
                        rmsnorm_require_bitwise, rmsnorm_gain_center, rmsnorm_use_kahan, rmsnorm_recompute_rstd)
        options = ExecutionOptions(validate_expert_ids=validate_expert_ids, experts_output_postprocess=post,
                                   swiglu_clip_stats_out_3=swiglu_clip_stats_out_3, swiglu_clip_limit=swiglu_clip_limit)
        w13 = w13_EFD.reshape(state.e_local, 2 * cfg.intermediate_dim, cfg.hidden_dim)
        w2 = w2_EDF.reshape(state.e_local, cfg.hidden_dim, cfg.intermediate_dim)
        out, _ = forward_impl(state, x_TD.contiguous(), topk_expert_ids_TK, topk_scores_TK, w13, w2, options, False)
        return out

    def bf16_meta(x_TD, *args):
        return torch.empty_like(x_TD)

    lib.impl("bf16", bf16_cuda, "CUDA")
    lib.impl("bf16", bf16_meta, "Meta")
    _LIBS.append(lib)
    REGISTERED.append("bf16")


_LIBS: list = []


def inference_storage(context) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """(activation, slot id, routing, dispatch, combine) tensors to pass to ``dist_moe::bf16``."""
    st = context._state
    return st.arena, st.slot_selector, st.routing.local(), st.dispatch.local(), st.combine.local()


# ---------------------------------------------------------------------------------------------
# Block-scaled
# ---------------------------------------------------------------------------------------------
_PREPARED_FIELDS = ("fprop_data", "fprop_scale", "dgrad_data", "dgrad_scale", "global_scale", "global_scale_inv")


def pack_prepared(p13: PreparedWeight | None, p2: PreparedWeight | None) -> list[torch.Tensor | None]:
    """The 12-slot ``prepared`` argument of ``dist_moe::block_scaled_forward``: six operand tensors per weight
    (forward data, forward scales, input-gradient data, input-gradient scales, global scale and its inverse);
    all ``None`` when the weights are quantised inside the call."""
    out: list[torch.Tensor | None] = []
    for p in (p13, p2):
        out.extend([None] * 6 if p is None else [getattr(p, f) for f in _PREPARED_FIELDS])
    return out


def _unpack_prepared(prepared, fmt, sources, interleaved):
    if len(prepared) != 12:
        raise RuntimeError(f"block_scaled_forward received {len(prepared)} prepared slots, expected 12")
    out = []
    for i, src in enumerate(sources):
        slots = prepared[6 * i: 6 * i + 6]
        if slots[0] is None:
            out.append(None)
            continue
        out.append(PreparedWeight._create(source=src, format=fmt, fprop_data=slots[0], fprop_scale=slots[1],
                                          dgrad_data=slots[2], dgrad_scale=slots[3], global_scale=slots[4],
                                          global_scale_inv=slots[5], interleaved_fc13=bool(interleaved and i == 0)))
    return out


_TRAIN_STATE = ("offsets", "fwd", "bwd", "sct", "h1", "x_col", "x_col_sf", "h2_col", "h2_col_sf", "h3")


def _register_block_scaled() -> None:
    from . import _blockscaled as bs

    @torch.library.custom_op(f"{_NS}::prepare_mxfp8_weight", mutates_args=())
    def prepare_mxfp8_weight(weight: torch.Tensor, inference: bool,
                             fuse_swiglu: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        q, s0, s1 = bs.quantize_mxfp8_weight(weight, inference=inference, fuse_swiglu=fuse_swiglu)
        return q, s0, s1 if s1 is not None else weight.new_empty(0, dtype=torch.uint8)

    @prepare_mxfp8_weight.register_fake
    def _(weight, inference, fuse_swiglu):
        E, N, K = weight.shape
        grp = bs._blocked_group_bytes(N, K // 32)
        grp_d = 0 if inference else bs._blocked_group_bytes(K, N // 32)
        u8 = torch.uint8
        return (weight.new_empty((E, N, K), dtype=u8), weight.new_empty(E * grp, dtype=u8),
                weight.new_empty(E * grp_d, dtype=u8))

    @torch.library.custom_op(f"{_NS}::prepare_nvfp4_weight", mutates_args=())
    def prepare_nvfp4_weight(weight_ENK: torch.Tensor,
                             fuse_swiglu: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        return bs.quantize_nvfp4_weight(weight_ENK, fuse_swiglu=fuse_swiglu)

    @prepare_nvfp4_weight.register_fake
    def _(weight_ENK, fuse_swiglu):
        E, N, K = weight_ENK.shape
        grp = bs._blocked_group_bytes(N, K // 16)
        return (weight_ENK.new_empty((E, N, K // 2), dtype=torch.uint8), weight_ENK.new_empty(E * grp, dtype=torch.uint8),
                weight_ENK.new_empty(E, dtype=torch.float32), weight_ENK.new_empty(E, dtype=torch.float32))

    @torch.library.custom_op(f"{_NS}::block_scaled_forward", mutates_args=(), device_types="cuda")
    def block_scaled_forward(x_TD: torch.Tensor, topk_expert_ids_TK: torch.Tensor, topk_scores_TK: torch.Tensor,
                             w13_EFD: torch.Tensor, w2_EDF: torch.Tensor, prepared: list[torch.Tensor | None],
                             rmsnorm_weight_D: torch.Tensor | None, rmsnorm_enabled: bool, rmsnorm_eps: float,
                             rmsnorm_norm_output_dtype: torch.dtype, rmsnorm_output_dtype: torch.dtype,
                             rmsnorm_require_bitwise: bool, rmsnorm_gain_center: float, rmsnorm_use_kahan: bool,
                             rmsnorm_recompute_rstd: bool, activation_slot_id_1: torch.Tensor,
                             num_moe_layers_in_slot: int, save_for_backward: bool, validate_expert_ids: bool,
                             context_id: str, interleaved_fc13: bool) -> tuple[torch.Tensor, list[torch.Tensor]]:
        ctx = _context(context_id)
        state, cfg = ctx._state, ctx.config
        fmt = cfg.block_scaled.format
        post = _rmsnorm(rmsnorm_weight_D, rmsnorm_enabled, rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype,
                        rmsnorm_require_bitwise, rmsnorm_gain_center, rmsnorm_use_kahan, rmsnorm_recompute_rstd)
        options = ExecutionOptions(validate_expert_ids=validate_expert_ids, experts_output_postprocess=post)
        p13, p2 = _unpack_prepared(prepared, fmt, (w13_EFD, w2_EDF), interleaved_fc13)
        if not save_for_backward:
            w13 = p13 if p13 is not None else w13_EFD
            w2 = p2 if p2 is not None else w2_EDF
            out = bs.run_block_scaled(x_TD, topk_expert_ids_TK, topk_scores_TK, w13, w2, ctx, options,
                                      save_for_backward=False)
            return out, []
        if fmt is BlockScaledFormat.NVFP4:
            raise RuntimeError("NVFP4 is inference-only: it has no backward")
        t13, t2 = bs._training_weights(w13_EFD, w2_EDF, p13, p2, cfg)
        out, c = bs._mxfp8_forward(state, x_TD.contiguous(), topk_expert_ids_TK, topk_scores_TK, t13, t2, options,
                                   need_h3=True)
        saved = [getattr(c, name) for name in _TRAIN_STATE]
        # operator outputs may not alias operator inputs: operands that came in through `prepared` are copied
        own = (lambda t: t.clone()) if p13 is not None else (lambda t: t)
        saved += [own(t13.fprop_data), own(t13.dgrad_scale), own(t2.fprop_data), own(t2.dgrad_scale)]
        return out, saved

    @block_scaled_forward.register_fake
    def _(x_TD, topk_expert_ids_TK, topk_scores_TK, w13_EFD, w2_EDF, prepared, rmsnorm_weight_D, rmsnorm_enabled,
          rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype, rmsnorm_require_bitwise, rmsnorm_gain_center,
          rmsnorm_use_kahan, rmsnorm_recompute_rstd, activation_slot_id_1, num_moe_layers_in_slot, save_for_backward,
          validate_expert_ids, context_id, interleaved_fc13):
        out = torch.empty_like(x_TD)
        if not save_for_backward:
            return out, []
        ctx = _context(context_id)
        state, cfg = ctx._state, ctx.config
        T, K = topk_expert_ids_TK.shape
        D, F, el, ep = cfg.hidden_dim, cfg.intermediate_dim, state.e_local, state.ep
        size = max((ep * T * min(K, el) + el * 127 + 127) // 128 * 128, 128)
        R = min(size, state.capacity_rows // 128 * 128)
        u8, i64 = torch.uint8, torch.int64
        ne = x_TD.new_empty
        st = [ne(el + 1, dtype=torch.int32), ne(size, dtype=i64), ne(size, dtype=i64), ne(size, dtype=i64),
              ne((R, 2 * F), dtype=torch.bfloat16), ne((R, D), dtype=u8), ne(bs._sf_cols_bytes(R, D), dtype=u8),
              ne((R, F), dtype=u8), ne(bs._sf_cols_bytes(R, F), dtype=u8), ne(T * K * D, dtype=torch.bfloat16),
              ne((el, 2 * F, D), dtype=u8), ne(el * bs._blocked_group_bytes(D, 2 * F // 32), dtype=u8),
              ne((el, D, F), dtype=u8), ne(el * bs._blocked_group_bytes(F, D // 32), dtype=u8)]
        return out, st

    def run_backward(grad_out, w13, w2, ids, scores, st, context_id, explicit):
        ctx = _context(context_id)
        state, cfg = ctx._state, ctx.config
        if len(st) != len(_TRAIN_STATE) + 4:
            raise RuntimeError(f"block-scaled backward received {len(st)} state tensors")
        c = bs._TrainCall()
        for name, t in zip(_TRAIN_STATE, st):
            setattr(c, name, t)
        c.T = ids.shape[0]
        c.R = c.h1.shape[0]
        c.recv = c.offsets[state.e_local:]
        fmt = cfg.block_scaled.format
        mk = lambda src, q, sd: PreparedWeight._create(source=src, format=fmt, fprop_data=q, fprop_scale=q,  # noqa: E731
                                                        dgrad_data=q, dgrad_scale=sd)
        c.p13, c.p2 = mk(w13, st[-4], st[-3]), mk(w2, st[-2], st[-1])
        return bs._mxfp8_backward(state, c, grad_out.shape, ids, scores, w13, w2, grad_out.contiguous(),
                                  ExecutionOptions(), (True, True, True, True), wgrad_explicit=explicit)

    @torch.library.custom_op(f"{_NS}::block_scaled_backward", mutates_args=(), device_types="cuda")
    def block_scaled_backward(grad_output_TD: torch.Tensor, w13_EFD: torch.Tensor, w2_EDF: torch.Tensor,
                              topk_expert_ids_TK: torch.Tensor, topk_scores_TK: torch.Tensor,
                              state: list[torch.Tensor], rmsnorm_enabled: bool, rmsnorm_eps: float,
                              rmsnorm_norm_output_dtype: torch.dtype, rmsnorm_output_dtype: torch.dtype,
                              rmsnorm_require_bitwise: bool, rmsnorm_use_kahan: bool, rmsnorm_recompute_rstd: bool,
                              wgrad_output_dtype: torch.dtype,
                              context_id: str) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
        if rmsnorm_enabled:
            raise NotImplementedError("expert-output postprocessing is not available on the MXFP8 training path")
        gx, gs, g13, g2 = run_backward(grad_output_TD, w13_EFD, w2_EDF, topk_expert_ids_TK, topk_scores_TK, state,
                                       context_id, (wgrad_output_dtype, wgrad_output_dtype))
        return gx, gs, g13.reshape(w13_EFD.shape), g2.reshape(w2_EDF.shape)

    @block_scaled_backward.register_fake
    def _(grad_output_TD, w13_EFD, w2_EDF, topk_expert_ids_TK, topk_scores_TK, state, rmsnorm_enabled, rmsnorm_eps,
          rmsnorm_norm_output_dtype, rmsnorm_output_dtype, rmsnorm_require_bitwise, rmsnorm_use_kahan,
          rmsnorm_recompute_rstd, wgrad_output_dtype, context_id):
        return (torch.empty_like(grad_output_TD), torch.empty_like(topk_scores_TK),
                torch.empty_like(w13_EFD, dtype=wgrad_output_dtype), torch.empty_like(w2_EDF, dtype=wgrad_output_dtype))

    @torch.library.custom_op(f"{_NS}::block_scaled_backward_accumulate_",
                             mutates_args=("accumulator_grad_w13_EFD", "accumulator_grad_w2_EDF"), device_types="cuda")
    def block_scaled_backward_accumulate_(grad_output_TD: torch.Tensor, w13_EFD: torch.Tensor, w2_EDF: torch.Tensor,
                                          accumulator_grad_w13_EFD: torch.Tensor, accumulator_grad_w2_EDF: torch.Tensor,
                                          topk_expert_ids_TK: torch.Tensor, topk_scores_TK: torch.Tensor,
                                          state: list[torch.Tensor], rmsnorm_enabled: bool, rmsnorm_eps: float,
                                          rmsnorm_norm_output_dtype: torch.dtype, rmsnorm_output_dtype: torch.dtype,
                                          rmsnorm_require_bitwise: bool, rmsnorm_use_kahan: bool,
                                          rmsnorm_recompute_rstd: bool, wgrad_output_dtype: torch.dtype,
                                          context_id: str) -> tuple[torch.Tensor, torch.Tensor]:
        if rmsnorm_enabled:
            raise NotImplementedError("expert-output postprocessing is not available on the MXFP8 training path")
        gx, gs, _, _ = run_backward(grad_output_TD, w13_EFD, w2_EDF, topk_expert_ids_TK, topk_scores_TK, state,
                                    context_id, (accumulator_grad_w13_EFD, accumulator_grad_w2_EDF))
        return gx, gs

    @block_scaled_backward_accumulate_.register_fake
    def _(grad_output_TD, w13_EFD, w2_EDF, accumulator_grad_w13_EFD, accumulator_grad_w2_EDF, topk_expert_ids_TK,
          topk_scores_TK, state, rmsnorm_enabled, rmsnorm_eps, rmsnorm_norm_output_dtype, rmsnorm_output_dtype,
          rmsnorm_require_bitwise, rmsnorm_use_kahan, rmsnorm_recompute_rstd, wgrad_output_dtype, context_id):
        return torch.empty_like(grad_output_TD), torch.empty_like(topk_scores_TK)

    for op in (block_scaled_forward, block_scaled_backward):
        if hasattr(op, "register_effect") and hasattr(torch.library, "EffectType"):
            op.register_effect(torch.library.EffectType.ORDERED)
    REGISTERED.extend(["prepare_mxfp8_weight", "prepare_nvfp4_weight", "block_scaled_forward", "block_scaled_backward",
                       "block_scaled_backward_accumulate_"])


def register() -> list[str]:
    """Define the operators (idempotent).  Returns the names this package registered."""
    if REGISTERED:
        return list(REGISTERED)
    existing = getattr(torch.ops, _NS)
    if hasattr(existing, "bf16_forward"):
        # another package (the reference) owns the namespace in this process
        return []
    _register_bf16()
    _register_block_scaled()
    return list(REGISTERED)
