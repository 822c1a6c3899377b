"""``routed_experts`` at the shapes the reference's benchmark configurations name, checked on token samples.

An output row (and a row of the input gradient) depends only on that token's K experts, so a few dozen sampled
tokens are compared against the dense CPU oracle run on those tokens alone; a weight gradient depends on every row
routed to the expert, so one lightly loaded expert per case is compared against the oracle run on exactly its rows.
Bounds are the reference's own for each format (tests/test_dist_moe.py:317-325, 4228-4259, 4677-4756), applied as
relative L2 and cosine over the sample.  What these catch and the small-shape tests cannot: tiles past the fourth
column block, byte offsets above 2^31, descriptors at K = 7168, F not a multiple of 256.
"""

import pytest
import torch

from oracle import moe as oracle_moe
from tests.test_blockscaled_layer_gpu import BOUNDS, MX_FWD, MX_GRAD, MX_WGRAD, _aggregate

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
BF16_FWD = dict(rel_l2=5e-3, cosine=0.999)
BF16_GRAD = dict(rel_l2=1e-2, cosine=0.995)
BF16_WGRAD = dict(rel_l2=1.5e-2, cosine=0.995)


def _weights(E, D, F, std, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    w13 = (torch.randn(E, 2, F, D, device=DEV, generator=g) * std).bfloat16()
    w2 = (torch.randn(E, D, F, device=DEV, generator=g) * std).bfloat16()
    return w13, w2


def _router(T, E, K, seed, *, bias=None, sigmoid=False):
    g = torch.Generator().manual_seed(seed)
    logits = torch.randn(T, E, generator=g)
    if bias is not None:
        logits = logits + bias
    if sigmoid:  # sigmoid scores of the top-k logits, not renormalised
        top = torch.topk(logits, K)
        return top.indices, torch.sigmoid(top.values).float()
    top = torch.topk(torch.softmax(logits, -1), K)
    return top.indices, (top.values / top.values.sum(-1, keepdim=True)).float()


def _sample_tokens(T, n, seed):
    return torch.randperm(T, generator=torch.Generator().manual_seed(seed))[:n].sort().values


def _oracle_rows(x, ids, scores, w13, w2, tokens, clamped, grad_out=None):
    """Output (and input / score gradients) of the sampled tokens from the dense oracle run on them alone."""
    xs = x[tokens].cpu().clone().requires_grad_(grad_out is not None)
    ss = scores[tokens].cpu().clone().requires_grad_(grad_out is not None)
    E = w13.shape[0]
    out = oracle_moe.moe_forward(xs, ids[tokens].cpu(), ss, w13.cpu().reshape(E, -1, w13.shape[-1]), w2.cpu(),
                                 clamped=clamped)
    if grad_out is None:
        return out.detach(), None, None
    out.backward(grad_out[tokens].cpu())
    return out.detach(), xs.grad, ss.grad


def _oracle_expert_wgrad(x, ids, scores, w13, w2, e, clamped, grad_out):
    """Weight gradients of expert ``e``: the oracle on every token routed to it, with the other routes masked out."""
    rows = torch.nonzero((ids == e).any(-1)).flatten()
    only = torch.where(ids[rows] == e, torch.zeros_like(ids[rows]), torch.full_like(ids[rows], -1))
    a = w13[e:e + 1].cpu().reshape(1, -1, w13.shape[-1]).clone().requires_grad_(True)
    b = w2[e:e + 1].cpu().clone().requires_grad_(True)
    out = oracle_moe.moe_forward(x[rows].cpu(), only.cpu(), scores[rows].cpu(), a, b, clamped=clamped)
    out.backward(grad_out[rows].cpu())
    return a.grad[0], b.grad[0], len(rows)


def _lightest_expert(ids, E, at_least=8):
    load = torch.bincount(ids.flatten().clamp_min(0), minlength=E)
    load[load < at_least] = 1 << 30
    return int(load.argmin())


def test_bf16_training_layer_at_the_headline_shape():
    """T=4096, D=2048, F=1408 (not a multiple of 256), E=64, K=6, plain SwiGLU, forward + backward with in-place
    fp32 weight-gradient accumulation: the configuration the headline metric is quoted on, at EP=1."""
    import dist_moe_b200 as dm

    T, D, F, E, K = 4096, 2048, 1408, 64, 6
    w13, w2 = _weights(E, D, F, 0.02, 7)
    ids, scores = _router(T, E, K, 8)
    g = torch.Generator().manual_seed(9)
    x = torch.randn(T, D, generator=g).bfloat16()
    grad_out = torch.randn(T, D, generator=g).bfloat16()
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, wgrad_dtype=torch.float32)
    ctx = dm.create_context(group=None, config=cfg, device=DEV)
    try:
        xs, ss = x.to(DEV).requires_grad_(), scores.to(DEV).requires_grad_()
        a, b = w13.clone().requires_grad_(), w2.clone().requires_grad_()
        out = dm.routed_experts(xs, ids.to(DEV), ss, a, b, ctx, options=dm.ExecutionOptions(inplace_wgrad_accum=True))
        out.backward(grad_out.to(DEV))
        ctx.check_status()
        tokens = _sample_tokens(T, 48, 10)
        ref_out, ref_gx, ref_gs = _oracle_rows(x, ids, scores, w13, w2, tokens, False, grad_out)
        _aggregate(out[tokens.to(DEV)], ref_out, BF16_FWD, "output rows")
        _aggregate(xs.grad[tokens.to(DEV)], ref_gx, BF16_GRAD, "grad x rows")
        _aggregate(ss.grad[tokens.to(DEV)], ref_gs, BF16_GRAD, "grad score rows")
        e = _lightest_expert(ids, E)
        ga, gb, n = _oracle_expert_wgrad(x, ids, scores, w13, w2, e, False, grad_out)
        assert n > 0 and a.grad.dtype == torch.float32
        _aggregate(a.grad[e].reshape(2 * F, D), ga, BF16_WGRAD, f"grad w13[{e}]")
        _aggregate(b.grad[e], gb, BF16_WGRAD, f"grad w2[{e}]")
    finally:
        ctx.close()


def test_mxfp8_training_layer_on_one_ranks_expert_share_with_skewed_load():
    """D=4096, F=1536, K=8, the 16 experts one rank owns at EP=8, router logits N(0,1) plus a Zipf(1.1) bias, the
    scratch capacity sized on the host from the routed rows."""
    import numpy as np

    import dist_moe_b200 as dm

    T, D, F, E, K = 2048, 4096, 1536, 16, 8
    w13, w2 = _weights(E, D, F, 0.02, 17)
    bias = torch.from_numpy(np.random.default_rng(2027).zipf(1.1, E).clip(max=64).astype("float32")).log()
    ids, scores = _router(T, E, K, 18, bias=bias)
    g = torch.Generator().manual_seed(19)
    x = torch.randn(T, D, generator=g).bfloat16()
    grad_out = torch.randn(T, D, generator=g).bfloat16()
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=DEV)
    try:
        xs, ss = x.to(DEV).requires_grad_(), scores.to(DEV).requires_grad_()
        a, b = w13.clone().requires_grad_(), w2.clone().requires_grad_()
        out = dm.routed_experts(xs, ids.to(DEV), ss, a, b, ctx)
        out.backward(grad_out.to(DEV))
        ctx.check_status()
        tokens = _sample_tokens(T, 32, 20)
        ref_out, ref_gx, ref_gs = _oracle_rows(x, ids, scores, w13, w2, tokens, False, grad_out)
        _aggregate(out[tokens.to(DEV)], ref_out, MX_FWD, "output rows")
        _aggregate(xs.grad[tokens.to(DEV)], ref_gx, MX_GRAD, "grad x rows")
        _aggregate(ss.grad[tokens.to(DEV)], ref_gs, MX_GRAD, "grad score rows")
        e = _lightest_expert(ids, E)
        ga, gb, n = _oracle_expert_wgrad(x, ids, scores, w13, w2, e, False, grad_out)
        assert n > 0
        _aggregate(a.grad[e].reshape(2 * F, D), ga, MX_WGRAD, f"grad w13[{e}]")
        _aggregate(b.grad[e], gb, MX_WGRAD, f"grad w2[{e}]")
    finally:
        ctx.close()


@pytest.mark.parametrize("T", [128, 1024])
def test_nvfp4_inference_at_the_decode_and_prefill_shapes(T):
    """D=7168, F=2048, K=8, the 32 experts one rank owns at EP=8, sigmoid top-8 routing, prepared weights, CUDA-graph
    replay.  T=128 takes the swapped-operand GEMMs (about 32 rows per expert), T=1024 the 128 x 256 tiles."""
    import dist_moe_b200 as dm

    D, F, E, K = 7168, 2048, 32, 8
    w13, w2 = _weights(E, D, F, 0.02, 27)
    ids, scores = _router(T, E, K, 28, sigmoid=True)
    x = torch.randn(T, D, generator=torch.Generator().manual_seed(29)).bfloat16()
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0,
                    block_scaled=dm.BlockScaledConfig(format=dm.BlockScaledFormat.NVFP4))
    ctx = dm.create_context(group=None, config=cfg, device=DEV)
    try:
        p13 = dm.prepare_block_scaled_weight(w13, cfg, fuse_swiglu=True, inference=True)
        p2 = dm.prepare_block_scaled_weight(w2, cfg, inference=True)
        xs, idd, sd = x.to(DEV), ids.to(DEV), scores.to(DEV)
        eager = dm.routed_experts(xs, idd, sd, p13, p2, ctx)
        ctx.check_status()
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            dm.routed_experts(xs, idd, sd, p13, p2, ctx)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                captured = dm.routed_experts(xs, idd, sd, p13, p2, ctx)
        torch.cuda.current_stream().wait_stream(stream)
        graph.replay()
        torch.cuda.synchronize()
        ctx.check_status()
        assert torch.equal(captured, eager), "graph replay differs from the eager call"
        tokens = _sample_tokens(T, 24, 30)
        ref_out, _, _ = _oracle_rows(x, ids, scores, w13, w2, tokens, False)
        bound_l2, bound_cos = BOUNDS["NVFP4"]
        _aggregate(captured[tokens.to(DEV)], ref_out, dict(rel_l2=bound_l2, cosine=bound_cos), "output rows")
    finally:
        ctx.close()


@pytest.mark.parametrize("hot", [False, True])
def test_mxfp8_inference_clamped_swiglu_with_fused_rmsnorm(hot):
    """D=F=2816 (the legal shape nearest the named 2880), K=4, the 16 experts one rank owns at EP=8, clamped SwiGLU
    (limit 7) and the fused post-expert RMSNorm; uniform routing, and a stress where half of the assignments go to
    two experts."""
    import dist_moe_b200 as dm

    T, D, F, E, K = 1024, 2816, 2816, 16, 4
    w13, w2 = _weights(E, D, F, 0.02, 37)
    bias = None
    if hot:
        bias = torch.zeros(E)
        bias[:2] = 4.0
    ids, scores = _router(T, E, K, 38, bias=bias)
    x = torch.randn(T, D, generator=torch.Generator().manual_seed(39)).bfloat16()
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0,
                    activation="swiglu_clamped", swiglu_limit=7.0, block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=DEV)
    try:
        p13 = dm.prepare_block_scaled_weight(w13, cfg, fuse_swiglu=True, inference=True)
        p2 = dm.prepare_block_scaled_weight(w2, cfg, inference=True)
        post = dm.RMSNormPostprocess(eps=1e-6, norm_output_dtype=torch.float32, output_dtype=torch.bfloat16)
        out = dm.routed_experts(x.to(DEV), ids.to(DEV), scores.to(DEV), p13, p2, ctx,
                                options=dm.ExecutionOptions(experts_output_postprocess=post))
        ctx.check_status()
        tokens = _sample_tokens(T, 32, 40)
        h3 = oracle_moe.expert_outputs(x[tokens], ids[tokens], w13.cpu().reshape(E, 2 * F, D), w2.cpu(), clamped=True,
                                       limit=7.0)
        ref = oracle_moe.rmsnorm_combine(h3, scores[tokens], 1e-6, torch.bfloat16)
        _aggregate(out[tokens.to(DEV)], ref, MX_FWD, "normalised output rows")
    finally:
        ctx.close()
