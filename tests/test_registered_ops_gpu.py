"""The registered operators on a GPU: ``bf16_forward`` + ``bf16_backward`` (and the accumulating form) reproduce
``routed_experts`` under autograd bit for bit (they run the same kernels), the mutating inference operator equals
the no-grad call, and the MXFP8 operators round-trip their state list."""

import pytest
import torch

from tests.test_bf16_layer_gpu import make_case

pytestmark = pytest.mark.gpu


def _cfg(dm, T, D, F, K, E, **kw):
    return dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                     max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=1.0, **kw)


def test_bf16_operators_match_routed_experts():
    import dist_moe_b200 as dm

    dev = torch.device("cuda", 0)
    T, D, F, K, E = 96, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=3, w_scale=D**-0.5)
    x, ids, scores = x.to(dev), ids.to(dev), scores.to(dev)
    w13, w2 = w13.to(dev).reshape(E, 2 * F, D), w2.to(dev)
    go = torch.randn(T, D, device=dev).bfloat16()
    ctx = dm.create_context(group=None, config=_cfg(dm, T, D, F, K, E), device=dev)
    try:
        xs, ss = x.clone().requires_grad_(True), scores.clone().requires_grad_(True)
        a, b = w13.clone().requires_grad_(True), w2.clone().requires_grad_(True)
        ref = dm.routed_experts(xs, ids, ss, a, b, ctx)
        ref.backward(go)
        ctx.check_status()
        f32, bf16 = torch.float32, torch.bfloat16
        slot = torch.zeros(1, dtype=torch.int64, device=dev)
        cid = ctx.context_id
        out, state = torch.ops.dist_moe.bf16_forward(x, ids, scores, w13, w2, None, False, 1e-6, f32, bf16, True, 0.0,
                                                     False, False, slot, 1, False, cid)
        assert len(state) == 9 and torch.equal(out, ref)
        gx, gs, g13, g2 = torch.ops.dist_moe.bf16_backward(go, w13, w2, ids, scores, state, False, 1e-6, f32, bf16,
                                                           True, False, False, bf16, cid)
        ctx.check_status()
        assert torch.equal(gx, xs.grad) and torch.equal(gs, ss.grad)
        assert torch.equal(g13, a.grad) and torch.equal(g2, b.grad)
        # accumulating form: fp32 accumulators receive the same gradients on top of their content
        out, state = torch.ops.dist_moe.bf16_forward(x, ids, scores, w13, w2, None, False, 1e-6, f32, bf16, True, 0.0,
                                                     False, False, slot, 1, False, cid)
        acc13 = torch.full((E, 2 * F, D), 0.5, dtype=f32, device=dev)
        acc2 = torch.full((E, D, F), -0.25, dtype=f32, device=dev)
        gx2, gs2 = torch.ops.dist_moe.bf16_backward_accumulate_(go, w13, w2, acc13, acc2, ids, scores, state, False,
                                                                1e-6, f32, bf16, True, False, False, f32, cid)
        ctx.check_status()
        assert torch.equal(gx2, gx) and torch.equal(gs2, gs)
        torch.testing.assert_close(acc13 - 0.5, a.grad.float(), rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(acc2 + 0.25, b.grad.float(), rtol=2e-2, atol=2e-2)
        # clip statistics variant returns the counters as a third output
        out3, state3, clip = torch.ops.dist_moe.bf16_forward_with_clip_stats(
            x, ids, scores, w13, w2, None, False, 1e-6, f32, bf16, True, 0.0, False, False, slot, 1, False, 7.0, cid)
        assert clip.shape == (3,) and clip[2].item() == float((ids >= 0).sum().item() * F)
        torch.ops.dist_moe.bf16_backward(go, w13, w2, ids, scores, state3, False, 1e-6, f32, bf16, True, False, False,
                                         bf16, cid)  # unwinds the slot
        ctx.check_status()
    finally:
        ctx.close()


def test_bf16_inference_operator_with_storage_arguments():
    import dist_moe_b200 as dm
    from dist_moe_b200 import _ops

    dev = torch.device("cuda", 0)
    T, D, F, K, E = 64, 256, 128, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=4, w_scale=D**-0.5)
    x, ids, scores, w13, w2 = x.to(dev), ids.to(dev), scores.to(dev), w13.to(dev).reshape(E, 2 * F, D), w2.to(dev)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0)
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        with torch.no_grad():
            ref = dm.routed_experts(x, ids, scores, w13, w2, ctx)
        act, slot, routing, dispatch, combine = _ops.inference_storage(ctx)
        clip = torch.zeros(3, dtype=torch.float32, device=dev)
        out = torch.ops.dist_moe.bf16(x, ids, scores, w13, w2, None, False, 1e-6, torch.float32, torch.bfloat16, True,
                                      0.0, False, False, act, slot, 1, routing, dispatch, combine, clip, 7.0, True,
                                      ctx.context_id)
        ctx.check_status()
        assert torch.equal(out, ref) and clip[2].item() > 0
    finally:
        ctx.close()


def test_mxfp8_operators_round_trip_state():
    import dist_moe_b200 as dm
    from dist_moe_b200 import _ops

    dev = torch.device("cuda", 0)
    T, D, F, K, E = 96, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=5, w_scale=D**-0.5)
    x = (x.float() * 0.1).bfloat16().to(dev)
    ids, scores, w13, w2 = ids.to(dev), scores.to(dev), w13.to(dev).reshape(E, 2 * F, D), w2.to(dev)
    go = torch.randn(T, D, device=dev).bfloat16()
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        xs, ss = x.clone().requires_grad_(True), scores.clone().requires_grad_(True)
        a, b = w13.clone().requires_grad_(True), w2.clone().requires_grad_(True)
        ref = dm.routed_experts(xs, ids, ss, a, b, ctx)
        ref.backward(go)
        ctx.check_status()
        f32, bf16 = torch.float32, torch.bfloat16
        slot = torch.zeros(1, dtype=torch.int64, device=dev)
        cid = ctx.context_id
        # weights quantised inside the call, and the same through prepare_mxfp8_weight + the 12-slot list
        q13, s13, d13 = torch.ops.dist_moe.prepare_mxfp8_weight(w13, False, False)
        q2, s2, d2 = torch.ops.dist_moe.prepare_mxfp8_weight(w2, False, False)
        prepared = [q13, s13, q13, d13, None, None, q2, s2, q2, d2, None, None]
        for slots in ([None] * 12, prepared):
            out, state = torch.ops.dist_moe.block_scaled_forward(x, ids, scores, w13, w2, slots, None, False, 1e-6, f32,
                                                                 bf16, True, 0.0, False, False, slot, 1, True, False,
                                                                 cid, False)
            assert torch.equal(out, ref) and len(state) == 14
            gx, gs, g13, g2 = torch.ops.dist_moe.block_scaled_backward(go, w13, w2, ids, scores, state, False, 1e-6,
                                                                       f32, bf16, True, False, False, bf16, cid)
            ctx.check_status()
            assert torch.equal(gx, xs.grad) and torch.equal(gs, ss.grad)
            assert torch.equal(g13, a.grad) and torch.equal(g2, b.grad)
        acc13 = torch.zeros(E, 2 * F, D, dtype=f32, device=dev)
        acc2 = torch.zeros(E, D, F, dtype=f32, device=dev)
        torch.ops.dist_moe.block_scaled_backward_accumulate_(go, w13, w2, acc13, acc2, ids, scores, state, False, 1e-6,
                                                             f32, bf16, True, False, False, f32, cid)
        ctx.check_status()
        torch.testing.assert_close(acc13, a.grad.float(), rtol=2e-2, atol=2e-3)
        # inference through the operator: no state
        out_i, none = torch.ops.dist_moe.block_scaled_forward(x, ids, scores, w13, w2, [None] * 12, None, False, 1e-6,
                                                              f32, bf16, True, 0.0, False, False, slot, 1, False, False,
                                                              cid, False)
        assert none == [] and out_i.shape == ref.shape
        assert _ops.pack_prepared(None, None) == [None] * 12
    finally:
        ctx.close()
