"""``routed_experts`` with block-scaled contexts (MXFP8 training and inference, NVFP4 inference; one rank) against the
dense CPU oracle.  Bounds are the reference's own for these formats (tests/test_dist_moe.py:317-325,
applied there as relative L2 and cosine similarity): MXFP8 forward rel-L2 < 0.075, cosine > 0.9975;
NVFP4 forward rel-L2 < 0.29, cosine > 0.955.  Inputs follow its block-scaled tests: x * 0.1,
weights * dim^-0.5 (tests/test_dist_moe.py:4551-4552, 4582-4583)."""

import pytest
import torch

from oracle import moe as oracle_moe

pytestmark = pytest.mark.gpu
BOUNDS = {"MXFP8_E4M3": (0.075, 0.9975), "NVFP4": (0.29, 0.955)}


def _case(T, D, F, K, E, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, D, generator=g) * 0.1).bfloat16()
    w13 = (torch.randn(E, 2, F, D, generator=g) * D**-0.5).bfloat16()
    w2 = (torch.randn(E, D, F, generator=g) * F**-0.5).bfloat16()
    top = torch.topk(torch.softmax(torch.randn(T, E, generator=g), -1), K)
    scores = (top.values / top.values.sum(-1, keepdim=True)).float()
    ids = top.indices.clone()
    ids[torch.rand(T, K, generator=g) < 0.05] = -1
    scores = scores * (ids >= 0)
    return x, ids, scores, w13, w2


def _check(out, ref, fmt):
    out, ref = out.float().cpu(), ref.float()
    assert torch.isfinite(out).all()
    l2 = ((out - ref).norm() / ref.norm()).item()
    cos = torch.nn.functional.cosine_similarity(out.flatten(), ref.flatten(), dim=0).item()
    bound_l2, bound_cos = BOUNDS[fmt]
    assert l2 < bound_l2 and cos > bound_cos, (fmt, l2, cos)
    return l2, cos


@pytest.mark.parametrize("fmt,fuse,clamped,T,D,F,K,E", [
    ("MXFP8_E4M3", True, False, 200, 512, 256, 4, 8),
    ("MXFP8_E4M3", False, True, 64, 256, 384, 2, 4),
    ("NVFP4", True, False, 200, 512, 256, 8, 16),
    ("NVFP4", False, False, 33, 256, 512, 2, 4),
    ("MXFP8_E4M3", True, False, 1, 256, 128, 1, 2),
    ("NVFP4", True, False, 24, 512, 256, 8, 16),        # few rows per expert: the swapped-operand GEMMs
    ("MXFP8_E4M3", True, True, 40, 256, 384, 2, 8),
])
def test_inference_forward_with_prepared_weights(fmt, fuse, clamped, T, D, F, K, E):
    import dist_moe_b200 as dm

    dev = torch.device("cuda", 0)
    x, ids, scores, w13, w2 = _case(T, D, F, K, E, seed=T + D)
    cfg = dm.Config(max_num_local_input_tokens=T + 5, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0,
                    activation="swiglu_clamped" if clamped else "swiglu",
                    block_scaled=dm.BlockScaledConfig(format=getattr(dm.BlockScaledFormat, fmt)))
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        p13 = dm.prepare_block_scaled_weight(w13.to(dev), cfg, fuse_swiglu=fuse, inference=True)
        p2 = dm.prepare_block_scaled_weight(w2.to(dev), cfg, inference=True)
        assert p13.format is cfg.block_scaled.format and p13._interleaved_fc13 == fuse
        ref = oracle_moe.moe_forward(x, ids, scores, w13, w2, clamped=clamped)
        outs = []
        for _ in range(2):
            out = dm.routed_experts(x.to(dev), ids.to(dev), scores.to(dev), p13, p2, ctx)
            ctx.check_status()
            _check(out, ref, fmt)
            outs.append(out.clone())
        assert torch.equal(outs[0], outs[1]), "repeat execution is not bit-identical"
        if fuse:
            # the two GEMM orientations accumulate the same K steps in the same order: forcing either gives equal bits
            from dist_moe_b200 import _blockscaled as bs

            saved = bs.SWAPPED_MAX_ROWS_PER_EXPERT
            try:
                for threshold in (0, 10**9):
                    bs.SWAPPED_MAX_ROWS_PER_EXPERT = threshold
                    forced = dm.routed_experts(x.to(dev), ids.to(dev), scores.to(dev), p13, p2, ctx)
                    ctx.check_status()
                    assert torch.equal(forced, outs[0]), f"orientation threshold {threshold} changes the output"
            finally:
                bs.SWAPPED_MAX_ROWS_PER_EXPERT = saved
        with pytest.raises(TypeError):
            dm.routed_experts(x.to(dev), ids.to(dev), scores.to(dev), p13, w2.to(dev), ctx)
    finally:
        ctx.close()


def test_mxfp8_dynamic_weights_and_refill():
    import dist_moe_b200 as dm

    dev = torch.device("cuda", 0)
    T, D, F, K, E = 96, 256, 256, 2, 4
    x, ids, scores, w13, w2 = _case(T, D, F, K, E, seed=5)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0,
                    block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        ref = oracle_moe.moe_forward(x, ids, scores, w13, w2)
        out = dm.routed_experts(x.to(dev), ids.to(dev), scores.to(dev), w13.to(dev), w2.to(dev), ctx)  # raw bf16 weights
        ctx.check_status()
        _check(out, ref, "MXFP8_E4M3")
        # training-layout preparation (32x32 tiles, shared qdata, two scale orientations) and in-place refill
        t13 = dm.prepare_block_scaled_weight(w13.to(dev), dm.Config(**{**cfg.__dict__, "inference": False,
                                                                       "num_activation_slots": 1}))
        assert t13.dgrad_data is t13.fprop_data and t13.dgrad_scale is not None
        before = (t13.fprop_data.clone(), t13.fprop_scale.clone(), t13.fprop_data.data_ptr())
        again = dm.prepare_block_scaled_weight(w13.to(dev), dm.Config(**{**cfg.__dict__, "inference": False,
                                                                         "num_activation_slots": 1}), out=t13)
        assert again is t13 and t13.fprop_data.data_ptr() == before[2]
        assert torch.equal(t13.fprop_data, before[0]) and torch.equal(t13.fprop_scale, before[1])
    finally:
        ctx.close()


# ---------------------------------------------------------------------------------------------
# MXFP8 training: forward + all four gradients against autograd through the dense oracle.
# Bounds (tests/test_dist_moe.py:317-322): forward / grad / wgrad = (rtol, atol, rel-L2, cosine)
# (0.05, 0.002, 0.075, 0.9975) / (0.05, 0.04, ...) / (0.05, 0.025, ...).  The reference applies the
# aggregate pair everywhere and the elementwise pair on its D = F = 1024 plain-SwiGLU case only,
# because the dense reference does not fake-quantise intermediates (4682-4688).
# ---------------------------------------------------------------------------------------------
MX_FWD = dict(rtol=0.05, atol=0.002, rel_l2=0.075, cosine=0.9975)
MX_GRAD = dict(rtol=0.05, atol=0.04, rel_l2=0.075, cosine=0.9975)
MX_WGRAD = dict(rtol=0.05, atol=0.025, rel_l2=0.075, cosine=0.9975)


def _aggregate(got, ref, bounds, what):
    got, ref = got.detach().float().cpu(), ref.detach().float()
    assert torch.isfinite(got).all(), what
    l2 = ((got - ref).norm() / ref.norm().clamp_min(1e-12)).item()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    assert l2 < bounds["rel_l2"] and cos > bounds["cosine"], (what, l2, cos)


def _grad_out(T, D):
    """Upstream gradient of the reference's tests: ``randn_like(output)`` (tests/test_dist_moe.py:2283)."""
    return torch.randn(T, D, generator=torch.Generator().manual_seed(1)).bfloat16()


def _oracle_grads(x, ids, scores, w13, w2, clamped):
    xs, ss = x.clone().requires_grad_(True), scores.clone().requires_grad_(True)
    a, b = w13.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    out = oracle_moe.moe_forward(xs, ids, ss, a, b, clamped=clamped)
    out.backward(_grad_out(*out.shape))
    return out, xs.grad, ss.grad, a.grad, b.grad


@pytest.mark.parametrize("T,D,F,K,E,clamped,elementwise", [
    (384, 1024, 1024, 2, 4, False, True),
    (200, 512, 384, 4, 8, False, False),
    (64, 256, 256, 2, 4, True, False),
    (16, 256, 128, 2, 8, False, False),      # experts with no rows
])
def test_mxfp8_training_forward_backward(T, D, F, K, E, clamped, elementwise):
    import dist_moe_b200 as dm
    from tests.helpers import assert_close

    dev = torch.device("cuda", 0)
    x, ids, scores, w13, w2 = _case(T, D, F, K, E, seed=T + F)
    cfg = dm.Config(max_num_local_input_tokens=T + 3, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, activation="swiglu_clamped" if clamped else "swiglu",
                    block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        ref = _oracle_grads(x, ids, scores, w13, w2, clamped)
        names = ("output", "grad x", "grad scores", "grad w13", "grad w2")
        bounds = (MX_FWD, MX_GRAD, MX_GRAD, MX_WGRAD, MX_WGRAD)
        runs = []
        for _ in range(2):
            xs, ss = x.to(dev).requires_grad_(True), scores.to(dev).requires_grad_(True)
            a, b = w13.to(dev).requires_grad_(True), w2.to(dev).requires_grad_(True)
            out = dm.routed_experts(xs, ids.to(dev), ss, a, b, ctx)
            out.backward(_grad_out(T, D).to(dev))
            ctx.check_status()
            got = (out, xs.grad, ss.grad, a.grad, b.grad)
            for g, r, n, bd in zip(got, ref, names, bounds):
                assert g.shape == r.shape, n
                if elementwise:
                    assert_close(g, r, what=n, **bd)
                else:
                    _aggregate(g, r, bd, n)
            runs.append([t.detach().clone() for t in got])
        for first, second, n in zip(runs[0], runs[1], names):
            assert torch.equal(first, second), f"{n}: repeat execution is not bit-identical"
        with torch.no_grad():
            again = dm.routed_experts(x.to(dev), ids.to(dev), scores.to(dev), w13.to(dev), w2.to(dev), ctx)
        ctx.check_status()
        _aggregate(again, ref[0], MX_FWD, "no-grad output")
    finally:
        ctx.close()


def test_mxfp8_training_prepared_weights_and_inplace_wgrad():
    import dist_moe_b200 as dm

    dev = torch.device("cuda", 0)
    T, D, F, K, E = 96, 256, 256, 2, 4
    x, ids, scores, w13, w2 = _case(T, D, F, K, E, seed=21)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, wgrad_dtype=torch.float32,
                    block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        a, b = w13.to(dev).requires_grad_(True), w2.to(dev).requires_grad_(True)
        p13, p2 = dm.prepare_block_scaled_weight(a, cfg), dm.prepare_block_scaled_weight(b, cfg)
        opts = dm.ExecutionOptions(inplace_wgrad_accum=True)
        ref = _oracle_grads(x, ids, scores, w13, w2, False)
        for it in range(2):
            xs = x.to(dev).requires_grad_(True)
            out = dm.routed_experts(xs, ids.to(dev), scores.to(dev), p13, p2, ctx, options=opts)
            out.backward(_grad_out(T, D).to(dev))
            ctx.check_status()
            _aggregate(out, ref[0], MX_FWD, "output")
            _aggregate(xs.grad, ref[1], MX_GRAD, "grad x")
            if it == 0:
                first = (a.grad.clone(), b.grad.clone())
        assert a.grad.dtype == torch.float32 and b.grad.dtype == torch.float32
        _aggregate(first[0], ref[3], MX_WGRAD, "grad w13")
        _aggregate(first[1], ref[4], MX_WGRAD, "grad w2")
        # the second pass accumulated in place: twice the first (tests/test_dist_moe.py:4815-4826)
        torch.testing.assert_close(a.grad, 2 * first[0], rtol=5e-2, atol=2e-2)
        torch.testing.assert_close(b.grad, 2 * first[1], rtol=5e-2, atol=2e-2)
        # inference-prepared weights cannot train
        i13 = dm.prepare_block_scaled_weight(w13.to(dev), cfg, inference=True)._with_source(a)
        i2 = dm.prepare_block_scaled_weight(w2.to(dev), cfg, inference=True)._with_source(b)
        with pytest.raises(ValueError):
            dm.routed_experts(x.to(dev).requires_grad_(True), ids.to(dev), scores.to(dev), i13, i2, ctx)
    finally:
        ctx.close()
