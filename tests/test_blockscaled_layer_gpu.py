"""``routed_experts`` with block-scaled contexts (MXFP8 and NVFP4 inference, one rank) against the
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
        with pytest.raises(NotImplementedError):
            tcfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                             max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig())
            tctx = dm.create_context(group=None, config=tcfg, device=dev)
            try:
                dm.routed_experts(x.to(dev).requires_grad_(True), ids.to(dev), scores.to(dev), w13.to(dev), w2.to(dev), tctx)
            finally:
                tctx.close()
    finally:
        ctx.close()
