"""Activation checkpointing around ``routed_experts``: the backward pops the slot its own forward used, also when
the recomputation of a selective-checkpoint region selects another slot in between, and clip counters survive a
recomputed forward.  Mirrors tests/test_dist_moe.py:3304-3500 of the reference (bit-exact comparisons as there)."""

import pytest
import torch
from torch.utils.checkpoint import CheckpointPolicy, checkpoint, create_selective_checkpoint_contexts

from tests.test_bf16_layer_gpu import make_case

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _context(dm, T, D, F, K, E, layers=1, **kw):
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=layers, activation_slot_capacity_factor=1.0, **kw)
    return dm.create_context(group=None, config=cfg, device=0)


def _leaves(*tensors):
    return tuple(t.detach().clone().to(DEV).requires_grad_() for t in tensors)


def _planner_is_rewound(ctx):
    st = ctx._state
    n = st.num_slots
    offs = st.buffer_offsets.tolist()
    assert offs[:n] == [i * st.slot_bytes for i in range(n)], offs
    assert not st.saved_bytes.any().item()
    assert not st.moe_layer_id.any().item()


def test_backward_pops_the_slot_its_forward_selected():
    import dist_moe_b200 as dm

    T, D, F, K, E = 64, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=31, w_scale=D**-0.5)
    ctx = _context(dm, T, D, F, K, E, num_activation_slots=2)
    try:
        ids_d = ids.to(DEV)
        ctx.select_activation_slot(0, 1)
        ref_in = _leaves(x, scores, w13, w2)
        ref = dm.routed_experts(ref_in[0], ids_d, ref_in[1], ref_in[2], ref_in[3], ctx)
        g = torch.randn_like(ref)
        ref.backward(g)
        ctx.select_activation_slot(1, 1)
        got_in = _leaves(x, scores, w13, w2)
        got = dm.routed_experts(got_in[0], ids_d, got_in[1], got_in[2], got_in[3], ctx)
        assert ctx._state.buffer_offsets[1].item() > ctx._state.slot_bytes  # slot 1 holds this call's activations
        ctx.select_activation_slot(0, 1)  # a later microbatch selects another slot before this backward runs
        got.backward(g)
        ctx.check_status()
        assert torch.equal(got, ref)
        for a, b in zip(got_in, ref_in):
            assert torch.equal(a.grad, b.grad)
        _planner_is_rewound(ctx)
    finally:
        ctx.close()


def test_selective_checkpoint_keeps_the_forward_slot():
    """The registered forward is an ordered-effect operator: a selective-checkpoint policy saves it, the region's
    recomputation (which selects slot 1) does not run it again, and the backward unwinds slot 0."""
    import dist_moe_b200 as dm
    from torch._higher_order_ops.effects import has_effects

    T, D, F, K, E = 48, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=32, w_scale=D**-0.5)
    ctx = _context(dm, T, D, F, K, E, num_activation_slots=2)
    try:
        ids_d = ids.to(DEV)

        def layer(a, s, p, q):
            return dm.routed_experts(a, ids_d, s, p, q, ctx)

        ctx.select_activation_slot(0, 1)
        ref_in = _leaves(x, scores, w13, w2)
        ref = layer(*ref_in)
        g = torch.randn_like(ref)
        ref.backward(g)
        _planner_is_rewound(ctx)
        ctx.reset()

        calls, saved_ops = [0], []

        def region(*values):
            ctx.select_activation_slot(min(calls[0], 1), 1)
            calls[0] += 1
            return layer(*values)

        def policy(_ctx, op, *_a, **_k):
            if has_effects(op):
                saved_ops.append(op)
                return CheckpointPolicy.MUST_SAVE
            return CheckpointPolicy.PREFER_RECOMPUTE

        got_in = _leaves(x, scores, w13, w2)
        got = checkpoint(region, *got_in, use_reentrant=False,
                         context_fn=lambda: create_selective_checkpoint_contexts(policy), early_stop=False)
        assert calls[0] == 1
        got.backward(g)
        assert calls[0] == 2
        ctx.check_status()
        assert torch.equal(got, ref)
        for a, b in zip(got_in, ref_in):
            assert torch.equal(a.grad, b.grad)
        assert torch.ops.dist_moe.bf16_forward.default in saved_ops
        _planner_is_rewound(ctx)
    finally:
        ctx.close()


def test_clip_counters_survive_a_recomputed_forward():
    """A plain (non-selective) checkpoint runs the forward twice and the backward once: the slot needs room for two
    pushes, one stays on the stack afterwards and ``reset`` rewinds it."""
    import dist_moe_b200 as dm

    T, D, F, K, E = 64, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=33)
    ctx = _context(dm, T, D, F, K, E, layers=2)
    try:
        ids_d = ids.to(DEV)
        stats = torch.zeros(3, dtype=torch.float32, device=DEV)
        opts = dm.ExecutionOptions(swiglu_clip_stats_out_3=stats, swiglu_clip_limit=0.0)

        def run(a, s, p, q):
            return dm.routed_experts(a, ids_d, s, p, q, ctx, options=opts)

        ref_in = _leaves(x, scores, w13, w2)
        ref = run(*ref_in)
        g = torch.randn_like(ref)
        ref.backward(g)
        expect = stats.clone()
        assert expect[2].item() > 0
        ctx.reset()
        stats.zero_()
        got_in = _leaves(x, scores, w13, w2)
        got = checkpoint(run, *got_in, use_reentrant=False)
        got.backward(g)
        ctx.check_status()
        assert torch.equal(got, ref) and torch.equal(stats, expect)
        for a, b in zip(got_in, ref_in):
            assert torch.equal(a.grad, b.grad)
        assert ctx._state.moe_layer_id[0].item() == 1  # the first, discarded forward is still on the stack
        ctx.reset()
        _planner_is_rewound(ctx)
    finally:
        ctx.close()


def test_mxfp8_training_under_plain_checkpoint():
    import dist_moe_b200 as dm

    T, D, F, K, E = 128, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=34, w_scale=D**-0.5)
    ctx = _context(dm, T, D, F, K, E,
                   block_scaled=dm.BlockScaledConfig(format=dm.BlockScaledFormat.MXFP8_E4M3, pipeline="staged"))
    try:
        ids_d = ids.to(DEV)

        def run(a, s, p, q):
            return dm.routed_experts(a, ids_d, s, p, q, ctx)

        ref_in = _leaves(x, scores, w13, w2)
        ref = run(*ref_in)
        g = torch.randn_like(ref)
        ref.backward(g)
        got_in = _leaves(x, scores, w13, w2)
        got = checkpoint(run, *got_in, use_reentrant=False)
        got.backward(g)
        ctx.check_status()
        assert torch.equal(got, ref)
        for a, b in zip(got_in, ref_in):
            assert torch.equal(a.grad, b.grad)
    finally:
        ctx.close()
