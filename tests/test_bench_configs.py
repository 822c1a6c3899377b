"""The workloads `bench.py` names are legal configurations of the public surface (host-side validation and the
memory plan only; nothing runs on a device)."""

import importlib.util
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("ep", [1, 2, 8])
def test_inference_workloads_are_legal_configs(ep):
    import dist_moe_b200 as dm

    bench = _bench()
    for name, (fmt, T, D, F, E, K, clamped, _routing, _rmsnorm) in bench.INFERENCE_WORKLOADS.items():
        extra = {"activation": "swiglu_clamped", "swiglu_limit": 7.0} if clamped else {}
        cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                        max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0,
                        block_scaled=dm.BlockScaledConfig(format=getattr(dm.BlockScaledFormat, fmt)), **extra)
        plan = dm.plan_memory(cfg, ep)
        assert plan.total_device_buffer_bytes > 0, name
        assert E % ep == 0, name


def test_training_workloads_are_legal_configs():
    import dist_moe_b200 as dm

    bench = _bench()
    bf16 = dm.Config(max_num_local_input_tokens=bench.T, hidden_dim=bench.D, intermediate_dim=bench.F, top_k=bench.K,
                     num_experts=bench.E, max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=1.25,
                     device_scratch_capacity_factor=1.25)
    mxfp8 = dm.Config(max_num_local_input_tokens=8192, hidden_dim=4096, intermediate_dim=1536, top_k=8, num_experts=128,
                      max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig())
    for cfg in (bf16, mxfp8):
        for ep in (1, 8):
            assert dm.plan_memory(cfg, ep).total_device_buffer_bytes > 0
