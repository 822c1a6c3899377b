"""``plan_memory`` and ``Config`` validation against the reference (CPU).

``tests/golden/plan_memory.json`` holds the reference's own ``plan_memory`` outputs for
BF16, MXFP8 and NVFP4 configurations (written by ``tests/golden/gen_golden.py``); the
literal numbers below are the ones the reference's tests and README pin
(tests/test_dist_moe_vmm.py:146-167, README.md:435-446)."""

import dataclasses
import json
from pathlib import Path

import pytest
import torch

import dist_moe_b200 as dm

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "plan_memory.json").read_text())


def _config(spec):
    kw = dict(spec)
    bs = kw.pop("block_scaled", None)
    if bs is not None:
        kw["block_scaled"] = dm.BlockScaledConfig(format=getattr(dm.BlockScaledFormat, bs[0]), pipeline=bs[1])
    return dm.Config(**kw)


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_plan_memory_matches_reference_byte_for_byte(name):
    case = GOLDEN[name]
    plan = dm.plan_memory(_config(case["config"]), case["ep_size"])
    got = dataclasses.asdict(plan)
    assert got == case["plan"], {k: (got[k], case["plan"][k]) for k in got if got[k] != case["plan"][k]}
    assert plan.explain() == case["explain"]


def test_capacity_padding_example():
    """32 routed rows over 2 local experts pad to 256 rows of 128 (docs/mxfp8_execution.md:61-80)."""
    cfg = dm.Config(max_num_local_input_tokens=16, hidden_dim=256, intermediate_dim=256, top_k=2, num_experts=4,
                    max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig())
    plan = dm.plan_memory(cfg, 2)
    assert plan.balanced_recv_rows == 32 and plan.device_scratch_capacity_rows == 256


def test_config_validation_errors():
    base = dict(max_num_local_input_tokens=16, hidden_dim=256, intermediate_dim=256, top_k=2, num_experts=8,
                max_moe_layers_per_activation_slot=1)
    dm.Config(**base)
    for bad, exc in [
        (dict(hidden_dim=100), ValueError),
        (dict(top_k=9), ValueError),
        (dict(num_experts=0), ValueError),
        (dict(max_moe_layers_per_activation_slot=0), ValueError),
        (dict(activation_slot_bytes=1.5), TypeError),
        (dict(activation_slot_bytes=10, activation_slot_capacity_factor=1.0), ValueError),
        (dict(num_activation_slots=0), ValueError),
        (dict(device_scratch_capacity_factor=0.0), ValueError),
        (dict(wgrad_dtype=torch.float16), TypeError),
        (dict(activation="gelu"), ValueError),
        (dict(bf16_grouped_gemm_preset="nope"), ValueError),
        (dict(inference=True, activation_slot_capacity_factor=1.0), ValueError),
        (dict(block_scaled=dm.BlockScaledConfig(format=dm.BlockScaledFormat.NVFP4)), ValueError),  # NVFP4 => inference
    ]:
        with pytest.raises(exc):
            dm.Config(**{**base, **bad})
    with pytest.raises(ValueError):
        dm.BlockScaledConfig(format=dm.BlockScaledFormat.NVFP4, fast_math=True)
    with pytest.raises(ValueError):
        dm.plan_memory(dm.Config(**base), 0)
    with pytest.raises(ValueError):
        dm.plan_memory(dm.Config(**base, activation_slot_bytes=8), 2)
    with pytest.raises(TypeError):
        dm.Context()
    with pytest.raises(TypeError):
        dm.PreparedWeight()


def test_public_names_match_the_reference_surface():
    assert sorted(dm.__all__) == sorted([
        "Bf16GroupedGemmPreset", "BlockScaledConfig", "BlockScaledFormat", "BlockScaledKernelConfig", "Config",
        "Context", "ExecutionOptions", "MemoryPlan", "PreparedWeight", "RMSNormPostprocess", "VmmConfig",
        "create_context", "plan_memory", "prepare_block_scaled_weight", "routed_experts",
        "supports_fused_post_expert_rmsnorm",
    ])


def test_mega_inference_plan_reserves_the_static_operand_carve():
    """With a device or an SM count the plan of a Mega inference context names the bytes of the static operand
    carve and holds them inside the device scratch (dist_moe/api.py:962-981); without either it stays unresolved."""
    import dist_moe_b200 as dm
    from dist_moe_b200._blockscaled import inference_layout

    def cfg(**kw):
        return dm.Config(max_num_local_input_tokens=128, hidden_dim=7168, intermediate_dim=2048, top_k=8,
                         num_experts=256, max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0,
                         block_scaled=dm.BlockScaledConfig(format=dm.BlockScaledFormat.NVFP4, pipeline="mega"), **kw)

    assert dm.plan_memory(cfg(), 8).inference_operand_bytes is None
    plan = dm.plan_memory(cfg(num_sms=148), 8)
    want = inference_layout(dm.BlockScaledFormat.NVFP4, 7168, 2048, plan.device_scratch_capacity_rows)["total"]
    assert plan.inference_operand_bytes == want
    assert plan.device_scratch_bytes >= want and plan.total_device_buffer_bytes >= want
    assert "physical Mega inference operands" in plan.explain()
    staged = dm.Config(max_num_local_input_tokens=128, hidden_dim=7168, intermediate_dim=2048, top_k=8, num_experts=256,
                       max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0, num_sms=148,
                       block_scaled=dm.BlockScaledConfig(format=dm.BlockScaledFormat.NVFP4))
    assert dm.plan_memory(staged, 8).inference_operand_bytes is None


def test_vmm_physical_sections_follow_the_driver_granularity():
    """Section arithmetic of a host-backed plan (dist_moe/api.py:1052-1109), with the granularity given."""
    import dist_moe_b200 as dm
    from dist_moe_b200 import _vmm

    cfg = dm.Config(max_num_local_input_tokens=4096, hidden_dim=1024, intermediate_dim=1024, top_k=2, num_experts=8,
                    max_moe_layers_per_activation_slot=2, activation_slot_capacity_factor=1.0,
                    device_scratch_capacity_factor=1.0, vmm=dm.VmmConfig(total_scratch_capacity_factor=4.0))
    logical = dm.plan_memory(cfg, 8)
    assert logical.uses_host_scratch and logical.vmm_granularity_bytes is None
    g = 2 * 1024 * 1024
    plan = _vmm.resolve_physical_plan(logical, g)
    up = lambda v: (v + g - 1) // g * g  # noqa: E731
    assert plan.vmm_device_prefix_bytes == up(logical.total_activation_bytes)
    assert plan.vmm_host_section_bytes == up(logical.host_scratch_bytes)
    assert plan.vmm_device_scratch_section_bytes == up(logical.device_scratch_bytes)
    assert plan.total_virtual_bytes == (plan.vmm_device_prefix_bytes + plan.vmm_host_section_bytes
                                        + plan.vmm_device_scratch_section_bytes)
    assert plan.vmm_padding_bytes == plan.total_virtual_bytes - logical.total_activation_bytes \
        - logical.host_scratch_bytes - logical.device_scratch_bytes
    # a range below 10 MiB is planned as the allocator's 20 MiB block, the slack going to the hot device scratch
    small = dataclasses_replace(logical, total_activation_bytes=1 << 20, host_scratch_bytes=1 << 20,
                                device_scratch_bytes=1 << 20)
    tiny = _vmm.resolve_physical_plan(small, g)
    assert tiny.total_virtual_bytes == 20 * 1024 * 1024
    assert tiny.vmm_device_scratch_section_bytes == 20 * 1024 * 1024 - 2 * g


def dataclasses_replace(obj, **kw):
    import dataclasses

    return dataclasses.replace(obj, **kw)
