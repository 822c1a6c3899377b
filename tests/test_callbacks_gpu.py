"""Python callbacks inside the kernel schedule (the reference's eager extension points, dist_moe/_execution.py:93-245;
its tests: tests/test_dist_moe.py "weights_preprocess_fn", "wgrad_postprocess_fn", "wgrad_destination_fn", callable
post-process) and the registered-operator route of the plain training call, all against the CPU oracle."""

import pytest
import torch

from oracle import moe as oracle_moe
from tests.helpers import BF16_FWD, BF16_GRAD, BF16_WGRAD, assert_close
from tests.test_bf16_layer_gpu import make_case, run_oracle

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
T, D, F, K, E = 96, 256, 256, 2, 4


def _ctx(dm, **kw):
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=1.0, **kw)
    return dm.create_context(group=None, config=cfg, device=DEV)


def test_weights_preprocess_fn_and_gradients_in_source_shape():
    """Compute weights are materialised from fp32 'master' weights of another shape, in the forward and again before
    the backward; weight gradients come back in the source tensors' shapes."""
    import dist_moe_b200 as dm

    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=3, w_scale=D**-0.5)
    ref = run_oracle(x, ids, scores, w13, w2)
    ctx = _ctx(dm)
    try:
        calls = []

        def preprocess(w):
            calls.append(tuple(w.shape))
            return w.to(torch.bfloat16).contiguous()

        src13 = w13.float().reshape(E * 2 * F, D).to(DEV).requires_grad_(True)   # flattened fp32 source
        src2 = w2.float().to(DEV).requires_grad_(True)
        xs, ss = x.to(DEV).requires_grad_(True), scores.to(DEV).requires_grad_(True)
        out = dm.routed_experts(xs, ids.to(DEV), ss, src13, src2, ctx,
                                options=dm.ExecutionOptions(weights_preprocess_fn=preprocess))
        out.float().sum().backward()
        ctx.check_status()
        assert len(calls) == 4 and calls[0] == (E * 2 * F, D)          # twice in the forward, twice before the backward
        assert src13.grad.shape == src13.shape and src2.grad.shape == src2.shape
        assert_close(out, ref[0], what="output", **BF16_FWD)
        assert_close(xs.grad, ref[1].grad, what="grad x", **BF16_GRAD)
        assert_close(src13.grad.reshape(E, 2, F, D), ref[3].grad, what="grad w13", **BF16_WGRAD)
        assert_close(src2.grad, ref[4].grad, what="grad w2", **BF16_WGRAD)
    finally:
        ctx.close()


def test_callable_postprocess_with_dropped_routes_and_closure_parameter():
    """``y = post(h3)`` before the weighted top-k sum; the callable's own parameter gets its gradient through the nested
    backward; rows of dropped routes are zeroed before the callable sees them."""
    import dist_moe_b200 as dm

    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=4, drop=0.2, w_scale=D**-0.5)
    gain = torch.full((D,), 1.5, device=DEV, requires_grad=True)
    seen = {}

    def post(h3):
        seen["dropped_rows_max"] = h3.detach()[(ids < 0).to(DEV)].abs().max().item() if (ids < 0).any() else 0.0
        return (torch.tanh(h3.float()) * gain).to(h3.dtype).contiguous()

    # oracle: the same function on the oracle's per-route outputs
    xr, sr = x.clone().requires_grad_(True), scores.clone().requires_grad_(True)
    a, b = w13.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    gain_ref = torch.full((D,), 1.5, requires_grad=True)
    h3 = oracle_moe.expert_outputs(xr, ids, a.reshape(E, 2 * F, D), b)
    y = (torch.tanh(h3.float()) * gain_ref).to(h3.dtype)
    ref = oracle_moe.combine(y, sr, torch.bfloat16)
    ref.float().sum().backward()

    ctx = _ctx(dm)
    try:
        xs, ss = x.to(DEV).requires_grad_(True), scores.to(DEV).requires_grad_(True)
        wa, wb = w13.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
        opts = dm.ExecutionOptions(experts_output_postprocess=post, zero_out_padded_callback_inputs=True)
        out = dm.routed_experts(xs, ids.to(DEV), ss, wa, wb, ctx, options=opts)
        out.float().sum().backward()
        ctx.check_status()
        assert seen["dropped_rows_max"] == 0.0
        assert_close(out, ref, what="output", **BF16_FWD)
        assert_close(xs.grad, xr.grad, what="grad x", **BF16_GRAD)
        assert_close(ss.grad, sr.grad, what="grad scores", **BF16_GRAD)
        assert_close(wa.grad, a.grad, what="grad w13", **BF16_WGRAD)
        assert_close(wb.grad, b.grad, what="grad w2", **BF16_WGRAD)
        assert_close(gain.grad, gain_ref.grad, what="closure parameter", rtol=3e-2, atol=0.5, rel_l2=1.5e-2, cosine=0.995)
        # no-grad call through the same callback path
        with torch.no_grad():
            again = dm.routed_experts(x.to(DEV), ids.to(DEV), scores.to(DEV), wa, wb, ctx, options=opts)
        assert torch.equal(again, out)
    finally:
        ctx.close()


def test_wgrad_postprocess_and_destination_callbacks():
    import dist_moe_b200 as dm

    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=5, w_scale=D**-0.5)
    ref = run_oracle(x, ids, scores, w13, w2)
    ctx = _ctx(dm)
    try:
        # postprocess: w2's gradient is replaced by twice itself, w13's is taken over (None goes back to autograd)
        taken = {}

        def postprocess(name, grad):
            if name == "w13":
                taken[name] = grad.clone()
                return None
            return (grad.float() * 2).to(grad.dtype)

        xs, ss = x.to(DEV).requires_grad_(True), scores.to(DEV).requires_grad_(True)
        wa, wb = w13.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
        out = dm.routed_experts(xs, ids.to(DEV), ss, wa, wb, ctx, options=dm.ExecutionOptions(wgrad_postprocess_fn=postprocess))
        out.float().sum().backward()
        ctx.check_status()
        assert wa.grad is None
        assert_close(taken["w13"].reshape(E, 2, F, D), ref[3].grad, what="w13 handed to the callback", **BF16_WGRAD)
        assert_close(wb.grad.float() / 2, ref[4].grad, what="grad w2 / 2", **BF16_WGRAD)

        # destination: the kernel accumulates into tensors the callback names; autograd gets nothing for the weights
        dst = {"w13": torch.ones(E, 2 * F, D, dtype=torch.bfloat16, device=DEV),
               "w2": torch.zeros(E, D, F, dtype=torch.bfloat16, device=DEV)}
        asked = []

        def destination(name, shape, dtype, device):
            asked.append((name, tuple(shape), dtype))
            return dst[name], name == "w13"      # w13: add to the ones; w2: overwrite

        xs, ss = x.to(DEV).requires_grad_(True), scores.to(DEV).requires_grad_(True)
        wa, wb = w13.to(DEV).requires_grad_(True), w2.to(DEV).requires_grad_(True)
        out = dm.routed_experts(xs, ids.to(DEV), ss, wa, wb, ctx, options=dm.ExecutionOptions(wgrad_destination_fn=destination))
        out.float().sum().backward()
        ctx.check_status()
        assert wa.grad is None and wb.grad is None
        assert sorted(asked) == [("w13", (E, 2 * F, D), torch.bfloat16), ("w2", (E, D, F), torch.bfloat16)]
        assert_close(dst["w13"].float() - 1.0, ref[3].grad.reshape(E, 2 * F, D), what="accumulated w13", **BF16_WGRAD)
        assert_close(dst["w2"], ref[4].grad, what="overwritten w2", **BF16_WGRAD)
        assert_close(xs.grad, ref[1].grad, what="grad x", **BF16_GRAD)
    finally:
        ctx.close()


def test_training_call_dispatches_through_the_registered_operators():
    """``make_fx`` of caller code sees ``dist_moe::bf16_forward`` and ``dist_moe::bf16_backward`` nodes (the reference
    applies its registered autograd the same way, dist_moe/api.py:4027-4042), and the traced graph computes what the
    eager call computes."""
    import dist_moe_b200 as dm
    from torch.fx.experimental.proxy_tensor import make_fx

    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=6, w_scale=D**-0.5)
    ref = run_oracle(x, ids, scores, w13, w2)
    ctx = _ctx(dm)
    try:
        idd = ids.to(DEV)

        def fn(xs, ss, wa, wb):
            out = dm.routed_experts(xs, idd, ss, wa, wb, ctx)
            gx, gs, g13, g2 = torch.autograd.grad(out.float().sum(), (xs, ss, wa, wb))
            return out, gx, gs, g13, g2

        args = [t.to(DEV).requires_grad_(True) for t in (x, scores, w13, w2)]
        eager = fn(*args)
        ctx.check_status()
        graph = make_fx(fn)(*args)
        targets = {str(n.target) for n in graph.graph.nodes if n.op == "call_function"}
        assert "dist_moe.bf16_forward.default" in targets and "dist_moe.bf16_backward.default" in targets, targets
        traced = graph(*args)
        ctx.check_status()
        for name, got, want in zip(("out", "gx", "gs", "g13", "g2"), traced, eager):
            assert torch.equal(got, want), name
        assert_close(eager[0], ref[0], what="output", **BF16_FWD)
        assert_close(eager[1], ref[1].grad, what="grad x", **BF16_GRAD)
        assert_close(eager[3], ref[3].grad, what="grad w13", **BF16_WGRAD)
    finally:
        ctx.close()


@pytest.mark.parametrize("recompute", [False, True])
def test_rmsnorm_observers_see_expert_outputs_and_their_gradient(recompute):
    """``observe_expert_output_fn`` sees the pre-norm expert outputs in the forward (and again in the replay of a
    recomputed layer), ``observe_expert_output_grad_fn`` the same outputs with their gradient; both are read-only
    taps, so results are bit-identical to the run without them (dist_moe/_postprocess.py:1245-1256, 1385-1412)."""
    import dist_moe_b200 as dm

    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=12, drop=0.15, w_scale=D**-0.5)
    sizing = dict(activation_slot_bytes=(T * D * 2 + 127) // 128 * 128) if recompute else \
        dict(activation_slot_capacity_factor=1.0)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, **sizing)
    ctx = dm.create_context(group=None, config=cfg, device=DEV)
    try:
        seen_fwd, seen_bwd = [], []
        plain = dm.RMSNormPostprocess(eps=1e-5, norm_output_dtype=torch.float32, output_dtype=torch.bfloat16)
        tapped = dm.RMSNormPostprocess(eps=1e-5, norm_output_dtype=torch.float32, output_dtype=torch.bfloat16,
                                       observe_expert_output_fn=lambda h3: seen_fwd.append(h3.clone()),
                                       observe_expert_output_grad_fn=lambda h3, g: seen_bwd.append((h3.clone(), g.clone())))
        g = torch.randn(T, D, generator=torch.Generator().manual_seed(8)).bfloat16().to(DEV)
        results = []
        for post in (plain, tapped):
            leaves = [t.detach().clone().to(DEV).requires_grad_() for t in (x, scores, w13, w2)]
            out = dm.routed_experts(leaves[0], ids.to(DEV), leaves[1], leaves[2], leaves[3], ctx,
                                    options=dm.ExecutionOptions(experts_output_postprocess=post,
                                                                zero_out_padded_callback_inputs=True))
            out.backward(g)
            ctx.check_status()
            results.append([out.detach()] + [leaf.grad for leaf in leaves])
        for a, b in zip(*results):
            assert torch.equal(a, b)
        assert len(seen_fwd) == (2 if recompute else 1) and len(seen_bwd) == 1
        h3 = seen_fwd[0]
        assert h3.shape == (T * K, D) and h3.dtype == torch.bfloat16
        assert torch.equal(seen_fwd[-1], h3)                     # the replay rebuilt the same expert outputs
        dropped = (ids.reshape(-1) < 0).to(DEV)
        assert dropped.any() and not h3[dropped].any()            # rows of dropped routes were zeroed first
        kept, grad = seen_bwd[0]
        assert torch.equal(kept, h3) and grad.shape == h3.shape and torch.isfinite(grad.float()).all()
        # the observed outputs reproduce the layer's result through the same normalise-and-reduce arithmetic
        h = h3.float().view(T, K, D)
        y = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-5)
        ref = (y * scores.to(DEV).float().masked_fill(ids.to(DEV) < 0, 0.0).unsqueeze(-1)).sum(1)
        assert_close(results[1][0], ref.cpu(), what="output from the observed expert outputs", **BF16_FWD)
    finally:
        ctx.close()


def test_observers_are_refused_on_block_scaled_contexts():
    import dist_moe_b200 as dm

    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=DEV)
    try:
        x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=13, w_scale=D**-0.5)
        post = dm.RMSNormPostprocess(eps=1e-5, norm_output_dtype=torch.float32, output_dtype=torch.bfloat16,
                                     observe_expert_output_fn=lambda h3: None)
        with pytest.raises(NotImplementedError):
            dm.routed_experts(x.to(DEV).requires_grad_(True), ids.to(DEV), scores.to(DEV), w13.to(DEV), w2.to(DEV), ctx,
                              options=dm.ExecutionOptions(experts_output_postprocess=post))
    finally:
        ctx.close()
