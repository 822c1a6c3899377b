"""Host-backed overflow scratch (``Config.vmm``): the arena is one virtual range laid out as
[device slots | host overflow scratch | device hot scratch]; a step whose scratch use exceeds the hot section runs
through host memory and still matches the oracle (dist_moe/_vmm.py:149-427, dist_moe/api.py:1052-1143)."""

import pytest
import torch

from tests.test_config_shapes_gpu import BF16_FWD, BF16_GRAD, _oracle_rows, _router, _sample_tokens, _weights
from tests.test_blockscaled_layer_gpu import _aggregate

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def test_training_step_through_host_backed_scratch():
    import dist_moe_b200 as dm

    T, D, F, E, K = 4096, 1024, 1024, 4, 2
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=1.0,
                    device_scratch_capacity_factor=0.25, vmm=dm.VmmConfig(total_scratch_capacity_factor=1.0))
    logical = dm.plan_memory(cfg, 1)
    assert logical.uses_host_scratch and logical.vmm_granularity_bytes is None
    plan = dm.plan_memory(cfg, 1, device=DEV)
    g = plan.vmm_granularity_bytes
    assert g and g % (64 * 1024) == 0
    for section in (plan.vmm_device_prefix_bytes, plan.vmm_host_section_bytes, plan.vmm_device_scratch_section_bytes):
        assert section % g == 0
    assert plan.vmm_host_section_bytes >= plan.host_scratch_bytes > 0
    assert plan.total_virtual_bytes == (plan.vmm_device_prefix_bytes + plan.vmm_host_section_bytes
                                        + plan.vmm_device_scratch_section_bytes)
    assert "mapped device/host/device sections" in plan.explain()

    w13, w2 = _weights(E, D, F, D**-0.5, 51)
    ids, scores = _router(T, E, K, 52)
    gen = torch.Generator().manual_seed(53)
    x = torch.randn(T, D, generator=gen).bfloat16()
    grad_out = torch.randn(T, D, generator=gen).bfloat16()
    free_before = torch.cuda.mem_get_info(DEV)[0]
    ctx = dm.create_context(group=None, config=cfg, device=DEV)
    try:
        assert ctx.memory_plan.vmm_granularity_bytes == g
        held = free_before - torch.cuda.mem_get_info(DEV)[0]
        assert held < plan.total_virtual_bytes  # the host section takes no device memory
        for _ in range(2):
            xs, ss = x.to(DEV).requires_grad_(), scores.to(DEV).requires_grad_()
            a, b = w13.clone().requires_grad_(), w2.clone().requires_grad_()
            out = dm.routed_experts(xs, ids.to(DEV), ss, a, b, ctx)
            out.backward(grad_out.to(DEV))
            ctx.check_status()
        tokens = _sample_tokens(T, 32, 54)
        ref_out, ref_gx, ref_gs = _oracle_rows(x, ids, scores, w13, w2, tokens, False, grad_out)
        _aggregate(out[tokens.to(DEV)], ref_out, BF16_FWD, "output rows")
        _aggregate(xs.grad[tokens.to(DEV)], ref_gx, BF16_GRAD, "grad x rows")
        _aggregate(ss.grad[tokens.to(DEV)], ref_gs, BF16_GRAD, "grad score rows")
        info = ctx.check_overflow()
        assert info.host_scratch_size == plan.vmm_host_section_bytes
        assert info.host_scratch_used > 0, info  # every routed row arrives: four times the hot section's rows
        assert info.device_scratch_used >= plan.vmm_device_scratch_section_bytes
    finally:
        ctx.close()
    assert ctx._state.vmm_arena is None  # unmapped and released
    again = dm.create_context(group=None, config=cfg, device=DEV)  # the range can be mapped anew
    again.close()
    # a context without host scratch (the factors coincide) takes the plain allocation
    same = dm.Config(max_num_local_input_tokens=64, hidden_dim=256, intermediate_dim=256, top_k=2, num_experts=4,
                     max_moe_layers_per_activation_slot=1, vmm=dm.VmmConfig(total_scratch_capacity_factor=1.0))
    ctx = dm.create_context(group=None, config=same, device=DEV)
    try:
        assert ctx.memory_plan.vmm_granularity_bytes is None and ctx._state.vmm_arena is None
    finally:
        ctx.close()
