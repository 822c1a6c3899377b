"""Profiler ranges and peak-usage counters of a training call (dist_moe/api.py:1979-2443 range names;
dist_moe/_activation_buffer.py:690-800 ``check_overflow`` and its asynchronous pair)."""

import pytest
import torch

from tests.test_bf16_layer_gpu import make_case

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _step(dm, ctx, case):
    x, ids, scores, w13, w2 = case
    leaves = [t.to(DEV).requires_grad_() for t in (x, scores, w13, w2)]
    out = dm.routed_experts(leaves[0], ids.to(DEV), leaves[1], leaves[2], leaves[3], ctx)
    out.float().sum().backward()
    ctx.check_status()


def test_profiler_ranges_carry_the_reference_names():
    import dist_moe_b200 as dm
    from torch.profiler import ProfilerActivity, profile

    T, D, F, K, E = 64, 256, 256, 2, 4
    case = make_case(T, D, F, K, E, seed=41, w_scale=D**-0.5)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1)
    ctx = dm.create_context(group=None, config=cfg, device=0)
    try:
        _step(dm, ctx, case)
        with profile(activities=[ProfilerActivity.CPU]) as prof:
            _step(dm, ctx, case)
        names = {e.name for e in prof.events()}
        for want in ("dist_moe_preprocess", "dist_moe_routing", "dist_moe_forward", "dist_moe_recompute", "dist_moe_backward"):
            assert want in names, (want, sorted(n for n in names if n.startswith("dist_moe")))
    finally:
        ctx.close()


@pytest.mark.parametrize("slot_factor", [None, 1.0])
def test_peak_counters_report_scratch_and_slot_use(slot_factor):
    import dist_moe_b200 as dm

    T, D, F, K, E = 96, 256, 512, 2, 4
    case = make_case(T, D, F, K, E, seed=42, w_scale=D**-0.5)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=slot_factor)
    ctx = dm.create_context(group=None, config=cfg, device=0)
    try:
        fresh = ctx.check_overflow()
        assert fresh.scratch_max_used == 0 and fresh.slot_max_used == [0.0]
        _step(dm, ctx, case)
        info = ctx.check_overflow()
        R = T * K
        h2 = R * F * 2
        assert info.scratch_size > 0 and 0 <= info.scratch_min_free < info.scratch_size
        assert info.scratch_max_used >= h2  # at least the SwiGLU output of every routed row lived in scratch
        assert info.scratch_max_used + info.scratch_min_free == info.scratch_size
        # the slot held x alone (recompute) or the gathered rows, h1 and the expert outputs (save)
        expect_slot = T * D * 2 if slot_factor is None else R * D * 2 + R * 2 * F * 2 + T * K * D * 2
        assert info.slot_max_used == [float(expect_slot)]
        pending = ctx.begin_check_overflow()
        again = ctx.finish_check_overflow(pending)
        assert again == info
        ctx.reset()
        assert ctx.check_overflow().scratch_max_used == 0
    finally:
        ctx.close()
