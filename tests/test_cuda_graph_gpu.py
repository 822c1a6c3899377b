"""CUDA-graph capture: the whole call (publication, routing, planning, GEMMs, reductions) is captured with
no host read of device data; replays on new input values are bit-identical to eager execution
(the reference makes the same claim for its BF16/MXFP8/NVFP4 paths, tests/test_dist_moe.py:2518-, 4068-4148)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(T, D, F, K, E, seed):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(T, D, generator=g) * 0.5).bfloat16()
    top = torch.topk(torch.randn(T, E, generator=g), K)
    ids = top.indices
    scores = torch.softmax(top.values, -1).float()
    return x, ids, scores


@pytest.mark.parametrize("fmt", [None, "MXFP8_E4M3", "NVFP4"])
def test_inference_forward_replay_equals_eager(fmt):
    import dist_moe_b200 as dm

    dev = torch.device("cuda", 0)
    T, D, F, K, E = 128, 512, 256, 4, 8
    g = torch.Generator().manual_seed(1)
    w13 = (torch.randn(E, 2, F, D, generator=g) * D**-0.5).bfloat16().to(dev)
    w2 = (torch.randn(E, D, F, generator=g) * F**-0.5).bfloat16().to(dev)
    bs = None if fmt is None else dm.BlockScaledConfig(format=getattr(dm.BlockScaledFormat, fmt))
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0, block_scaled=bs)
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        if fmt is not None:
            w13 = dm.prepare_block_scaled_weight(w13, cfg, fuse_swiglu=True, inference=True)
            w2 = dm.prepare_block_scaled_weight(w2, cfg, inference=True)
        x0, ids0, s0 = _inputs(T, D, F, K, E, 2)
        x, ids, scores = x0.to(dev), ids0.to(dev), s0.to(dev)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(3):
                dm.routed_experts(x, ids, scores, w13, w2, ctx)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.no_grad(), torch.cuda.graph(graph):
            out = dm.routed_experts(x, ids, scores, w13, w2, ctx)
        for seed in (3, 4):
            x1, ids1, s1 = _inputs(T, D, F, K, E, seed)
            x.copy_(x1)
            ids.copy_(ids1)
            scores.copy_(s1)
            graph.replay()
            replayed = out.clone()
            with torch.no_grad():
                eager = dm.routed_experts(x, ids, scores, w13, w2, ctx)
            assert torch.equal(replayed, eager), f"{fmt}: replay differs from eager"
        ctx.check_status()
    finally:
        ctx.close()


def test_training_step_capture_with_two_activation_slots():
    import dist_moe_b200 as dm

    dev = torch.device("cuda", 0)
    T, D, F, K, E = 64, 256, 256, 2, 4
    g = torch.Generator().manual_seed(5)
    w13 = (torch.randn(E, 2, F, D, generator=g) * D**-0.5).bfloat16().to(dev).requires_grad_(True)
    w2 = (torch.randn(E, D, F, generator=g) * F**-0.5).bfloat16().to(dev).requires_grad_(True)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, num_activation_slots=2, activation_slot_capacity_factor=1.0)
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        x0, ids0, s0 = _inputs(T, D, F, K, E, 6)
        x = x0.to(dev).requires_grad_(True)
        ids, scores = ids0.to(dev), s0.to(dev).requires_grad_(True)

        def step():
            # two microbatches in flight, one per activation slot, backward in reverse order
            outs = []
            for slot in (0, 1):
                ctx.select_activation_slot(slot, 1)
                outs.append(dm.routed_experts(x, ids, scores, w13, w2, ctx))
            (outs[1].float().sum() * 2.0).backward()
            outs[0].float().sum().backward()
            return outs

        def zero():
            for t in (x, scores, w13, w2):
                t.grad = None

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                zero()
                step()
        torch.cuda.current_stream().wait_stream(side)
        eager = [t.grad.clone() for t in (x, scores, w13, w2)]
        zero()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        captured = (x.grad, scores.grad, w13.grad, w2.grad)
        for _ in range(2):
            graph.replay()
            for got, want, name in zip(captured, eager, ("x", "scores", "w13", "w2")):
                assert torch.equal(got, want), f"grad {name}: replay differs from eager"
        ctx.check_status()
    finally:
        ctx.close()


def test_mxfp8_training_step_capture():
    """MXFP8 forward + backward captured in one CUDA graph: replays give the gradients of the eager step bit for bit
    (per-call temporaries come from the graph's private pool, every decision is taken on the device)."""
    import dist_moe_b200 as dm

    dev = torch.device("cuda", 0)
    T, D, F, K, E = 128, 256, 256, 2, 4
    g = torch.Generator().manual_seed(9)
    w13 = (torch.randn(E, 2, F, D, generator=g) * D**-0.5).bfloat16().to(dev).requires_grad_(True)
    w2 = (torch.randn(E, D, F, generator=g) * F**-0.5).bfloat16().to(dev).requires_grad_(True)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=1.0,
                    block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        x0, ids0, s0 = _inputs(T, D, F, K, E, 10)
        x = (x0 * 0.1).to(dev).requires_grad_(True)
        ids, scores = ids0.to(dev), s0.to(dev).requires_grad_(True)
        p13, p2 = dm.prepare_block_scaled_weight(w13, cfg), dm.prepare_block_scaled_weight(w2, cfg)

        def step():
            dm.routed_experts(x, ids, scores, p13, p2, ctx).float().sum().backward()

        def zero():
            for t in (x, scores, w13, w2):
                t.grad = None

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                zero()
                step()
        torch.cuda.current_stream().wait_stream(side)
        eager = [t.grad.clone() for t in (x, scores, w13, w2)]
        zero()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        captured = (x.grad, scores.grad, w13.grad, w2.grad)
        for _ in range(2):
            graph.replay()
            for got, want, name in zip(captured, eager, ("x", "scores", "w13", "w2")):
                assert torch.equal(got, want), f"grad {name}: replay differs from eager"
        ctx.check_status()
    finally:
        ctx.close()
