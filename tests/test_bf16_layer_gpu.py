"""``routed_experts`` (BF16, one rank) against the CPU oracle: forward, input/score/weight
gradients, save versus recompute, in-place weight-gradient accumulation, repeatability.

Tolerances are the reference's own for the BF16 path (tests/test_dist_moe.py:4228-4259,
4677-4678, 4750-4756): forward rtol/atol 2e-2, relative L2 < 5e-3, cosine > 0.999; input and
score gradients 3e-2 / 3e-2 / 1e-2 / 0.995; weight gradients rtol 3e-2, atol 1.0, 1.5e-2, 0.995."""

import pytest
import torch

from oracle import moe as oracle_moe
from tests.helpers import BF16_FWD, BF16_GRAD, BF16_WGRAD, assert_close

pytestmark = pytest.mark.gpu


def make_case(T, D, F, K, E, seed=0, drop=0.0, w_scale=None, dev="cuda"):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).bfloat16()
    w13 = torch.randn(E, 2, F, D, generator=g)
    w2 = torch.randn(E, D, F, generator=g)
    if w_scale is not None:
        w13, w2 = w13 * w_scale, w2 * w_scale
    w13, w2 = w13.bfloat16(), w2.bfloat16()
    logits = torch.randn(T, E, generator=g)
    top = torch.topk(torch.softmax(logits, -1), K)
    scores = (top.values / top.values.sum(-1, keepdim=True)).float()
    ids = top.indices.clone()
    if drop:
        mask = torch.rand(T, K, generator=g) < drop
        ids[mask] = -1
        scores = scores * (~mask)
    return x, ids, scores, w13, w2


def run_ours(dm, ctx, x, ids, scores, w13, w2, options=None, grad=True):
    dev = torch.device("cuda", 0)
    xs = x.to(dev).requires_grad_(grad)
    ss = scores.to(dev).requires_grad_(grad)
    a = w13.to(dev).requires_grad_(grad)
    b = w2.to(dev).requires_grad_(grad)
    out = dm.routed_experts(xs, ids.to(dev), ss, a, b, ctx, options=options)
    if grad:
        out.float().sum().backward()
    ctx.check_status()
    return out, xs, ss, a, b


def run_oracle(x, ids, scores, w13, w2, clamped=False):
    xs = x.clone().requires_grad_(True)
    ss = scores.clone().requires_grad_(True)
    a = w13.clone().requires_grad_(True)
    b = w2.clone().requires_grad_(True)
    out = oracle_moe.moe_forward(xs, ids, ss, a, b, clamped=clamped)
    out.float().sum().backward()
    return out, xs, ss, a, b


@pytest.mark.parametrize(
    "T,D,F,K,E,clamped,slot_factor,drop",
    [
        (16, 256, 256, 2, 8, False, None, 0.0),   # quickstart shape, all-recompute slot
        (16, 256, 256, 2, 8, True, 1.0, 0.0),     # clamped SwiGLU, everything saved
        (200, 512, 384, 4, 16, False, 1.0, 0.1),  # ragged experts, dropped routes, F % 128 != 0 path
        (130, 1024, 1024, 2, 4, False, None, 0.0),
    ],
)
def test_forward_backward_match_oracle(T, D, F, K, E, clamped, slot_factor, drop):
    import dist_moe_b200 as dm

    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=T, drop=drop, w_scale=D**-0.5)
    cfg = dm.Config(max_num_local_input_tokens=T + 3, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=slot_factor,
                    activation="swiglu_clamped" if clamped else "swiglu")
    ctx = dm.create_context(group=None, config=cfg, device=0)
    try:
        ref = run_oracle(x, ids, scores, w13, w2, clamped)
        for attempt in range(2):  # second pass: the LIFO slot state must have unwound
            got = run_ours(dm, ctx, x, ids, scores, w13, w2)
            assert_close(got[0], ref[0], what=f"output #{attempt}", **BF16_FWD)
            assert_close(got[1].grad, ref[1].grad, what="grad x", **BF16_GRAD)
            assert_close(got[2].grad, ref[2].grad, what="grad scores", **BF16_GRAD)
            assert_close(got[3].grad, ref[3].grad, what="grad w13", **BF16_WGRAD)
            assert_close(got[4].grad, ref[4].grad, what="grad w2", **BF16_WGRAD)
        # no-grad forward on the training context: scratch only, bit-identical output
        with torch.no_grad():
            again = run_ours(dm, ctx, x, ids, scores, w13, w2, grad=False)[0]
        assert torch.equal(again, got[0]), "no-grad forward differs from the grad-enabled one"
    finally:
        ctx.close()


def test_inplace_wgrad_accumulation_and_repeatability():
    import dist_moe_b200 as dm

    T, D, F, K, E = 96, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=5, w_scale=D**-0.5)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=1.0,
                    wgrad_dtype=torch.float32)
    ctx = dm.create_context(group=None, config=cfg, device=0)
    try:
        dev = torch.device("cuda", 0)
        a = w13.to(dev).requires_grad_(True)
        b = w2.to(dev).requires_grad_(True)
        opts = dm.ExecutionOptions(inplace_wgrad_accum=True)
        outs = []
        for _ in range(2):
            xs = x.to(dev).requires_grad_(True)
            out = dm.routed_experts(xs, ids.to(dev), scores.to(dev), a, b, ctx, options=opts)
            out.float().sum().backward()
            outs.append((out.detach().clone(), xs.grad.clone()))
            if len(outs) == 1:
                first = (a.grad.clone(), b.grad.clone())
        ctx.check_status()
        assert a.grad.dtype == torch.float32
        assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1]), "repeat run not bit-identical"
        torch.testing.assert_close(a.grad, 2 * first[0], rtol=5e-2, atol=2e-2)
        torch.testing.assert_close(b.grad, 2 * first[1], rtol=5e-2, atol=2e-2)
    finally:
        ctx.close()


def test_clip_stats_and_inference_context():
    import dist_moe_b200 as dm

    T, D, F, K, E = 64, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=9)  # unscaled weights: large pre-activations
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0)
    ctx = dm.create_context(group=None, config=cfg, device=0)
    try:
        dev = torch.device("cuda", 0)
        clip = torch.empty(3, dtype=torch.float32, device=dev)
        out = dm.routed_experts(x.to(dev), ids.to(dev), scores.to(dev), w13.to(dev), w2.to(dev), ctx,
                                options=dm.ExecutionOptions(swiglu_clip_stats_out_3=clip, swiglu_clip_limit=7.0))
        ctx.check_status()
        ref = oracle_moe.moe_forward(x, ids, scores, w13, w2)
        assert_close(out, ref, what="inference output", **BF16_FWD)
        expect = oracle_moe.clip_stats(x, ids, w13, 7.0)
        # counts may differ only where a bf16 pre-activation sits within rounding of the limit
        assert clip[2].item() == expect[2].item()
        assert abs(clip[0].item() - expect[0].item()) <= 0.002 * expect[2].item()
        assert abs(clip[1].item() - expect[1].item()) <= 0.002 * expect[2].item()
        with pytest.raises(RuntimeError):
            dm.routed_experts(x.to(dev).requires_grad_(True), ids.to(dev), scores.to(dev), w13.to(dev), w2.to(dev), ctx)
    finally:
        ctx.close()


@pytest.mark.parametrize("norm_dtype,recompute_rstd,slot_factor", [(torch.float32, False, 1.0), (torch.bfloat16, True, None)])
def test_fused_rmsnorm_postprocess_forward_backward(norm_dtype, recompute_rstd, slot_factor):
    import dist_moe_b200 as dm

    T, D, F, K, E = 100, 512, 256, 2, 8
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=21, drop=0.05, w_scale=D**-0.5)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=slot_factor)
    ctx = dm.create_context(group=None, config=cfg, device=0)
    try:
        post = dm.RMSNormPostprocess(eps=1e-6, norm_output_dtype=norm_dtype, output_dtype=torch.bfloat16,
                                     require_bitwise=False, recompute_rstd=recompute_rstd)
        got = run_ours(dm, ctx, x, ids, scores, w13, w2, options=dm.ExecutionOptions(experts_output_postprocess=post))
        xs = x.clone().requires_grad_(True)
        ss = scores.clone().requires_grad_(True)
        a = w13.clone().requires_grad_(True)
        b = w2.clone().requires_grad_(True)
        h3 = oracle_moe.expert_outputs(xs, ids, a.reshape(E, 2 * F, D), b)
        h3 = torch.where((ids >= 0)[:, :, None], h3, torch.zeros_like(h3))
        hf = h3.float()
        rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * (ids >= 0)[:, :, None]
        y = (hf * rstd).to(norm_dtype).float()
        ref = (y * ss[:, :, None]).sum(1).to(torch.bfloat16)
        ref.float().sum().backward()
        assert_close(got[0], ref, what="rmsnorm output", **BF16_FWD)
        assert_close(got[1].grad, xs.grad, what="rmsnorm grad x", **BF16_GRAD)
        assert_close(got[2].grad, ss.grad, what="rmsnorm grad scores", **BF16_GRAD)
        assert_close(got[3].grad, a.grad, what="rmsnorm grad w13", **BF16_WGRAD)
        assert_close(got[4].grad, b.grad, what="rmsnorm grad w2", **BF16_WGRAD)
    finally:
        ctx.close()


def test_rmsnorm_gamma_inference():
    import dist_moe_b200 as dm

    T, D, F, K, E = 40, 256, 256, 8, 16
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=22, w_scale=D**-0.5)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0)
    ctx = dm.create_context(group=None, config=cfg, device=0)
    try:
        dev = torch.device("cuda", 0)
        gamma = (torch.randn(D) * 0.1).bfloat16()
        post = dm.RMSNormPostprocess(eps=1e-5, norm_output_dtype=torch.float32, output_dtype=torch.bfloat16,
                                     weight=gamma.to(dev), gain_center=1.0)
        out = dm.routed_experts(x.to(dev), ids.to(dev), scores.to(dev), w13.to(dev), w2.to(dev), ctx,
                                options=dm.ExecutionOptions(experts_output_postprocess=post))
        ctx.check_status()
        h3 = oracle_moe.expert_outputs(x, ids, w13.reshape(E, 2 * F, D), w2)
        ref = oracle_moe.rmsnorm_combine(h3, scores, 1e-5, torch.bfloat16, weight=gamma, gain_center=1.0)
        assert_close(out, ref, what="gamma rmsnorm", **BF16_FWD)
    finally:
        ctx.close()
