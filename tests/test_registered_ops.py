"""``torch.ops.dist_moe.*``: schemas as the reference's tests assert them (tests/test_dist_moe.py:401-411,
1256-1290) and FakeTensor propagation through the fake implementations (no GPU needed: the context table
gets a stand-in that only carries the shape facts the fake implementations read)."""

import types

import pytest
import torch

import dist_moe_b200 as dm
from dist_moe_b200 import _ops, api

OPS = ("bf16", "bf16_forward", "bf16_forward_with_clip_stats", "bf16_backward", "bf16_backward_accumulate_",
       "block_scaled_forward", "block_scaled_backward", "block_scaled_backward_accumulate_", "prepare_mxfp8_weight",
       "prepare_nvfp4_weight")


def test_all_ten_operators_are_registered():
    assert sorted(_ops.register()) == sorted(OPS)
    for name in OPS:
        assert hasattr(torch.ops.dist_moe, name), name


def test_bf16_schemas_expose_clip_statistics_mutation():
    inference = str(torch.ops.dist_moe.bf16.default._schema)
    training = str(torch.ops.dist_moe.bf16_forward.default._schema)
    clip_training = str(torch.ops.dist_moe.bf16_forward_with_clip_stats.default._schema)
    assert "Tensor(e!)? swiglu_clip_stats_out_3" in inference
    assert "Tensor(a!) activation_storage" in inference and "str context_id" in inference
    assert "!" not in training
    assert "float swiglu_clip_limit" in clip_training and "!" not in clip_training


@pytest.mark.parametrize("family", ["bf16", "block_scaled"])
def test_backward_schemas_separate_wgrad_ownership(family):
    functional = getattr(torch.ops.dist_moe, f"{family}_backward").default
    accumulate = getattr(torch.ops.dist_moe, f"{family}_backward_accumulate_").default
    assert all(a.alias_info is None for a in functional._schema.arguments)
    args = accumulate._schema.arguments
    assert [a.name for a in args[3:5]] == ["accumulator_grad_w13_EFD", "accumulator_grad_w2_EDF"]
    assert all(a.alias_info is not None and a.alias_info.is_write for a in args[3:5])
    assert all(r.alias_info is None for r in accumulate._schema.returns)


def test_argument_names_follow_the_reference():
    names = [a.name for a in torch.ops.dist_moe.block_scaled_forward.default._schema.arguments]
    assert names[:6] == ["x_TD", "topk_expert_ids_TK", "topk_scores_TK", "w13_EFD", "w2_EDF", "prepared"]
    assert names[-4:] == ["save_for_backward", "validate_expert_ids", "context_id", "interleaved_fc13"]
    names = [a.name for a in torch.ops.dist_moe.bf16_forward.default._schema.arguments]
    assert names[-4:] == ["activation_slot_id_1", "num_moe_layers_in_slot", "validate_expert_ids", "context_id"]
    assert [a.name for a in torch.ops.dist_moe.prepare_mxfp8_weight.default._schema.arguments] == \
        ["weight", "inference", "fuse_swiglu"]


@pytest.fixture
def fake_context():
    cfg = dm.Config(max_num_local_input_tokens=16, hidden_dim=256, intermediate_dim=256, top_k=2, num_experts=8,
                    max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig())
    state = types.SimpleNamespace(e_local=4, ep=2, capacity_rows=1024)
    ctx = types.SimpleNamespace(_closed=False, _state=state, config=cfg)
    api._CONTEXTS["test-fake"] = ctx
    yield "test-fake"
    api._CONTEXTS.pop("test-fake", None)


def test_fake_tensor_propagation(fake_context):
    from torch._subclasses.fake_tensor import FakeTensorMode

    T, D, F, K, el = 16, 256, 256, 2, 4
    bf16, f32 = torch.bfloat16, torch.float32
    with FakeTensorMode():
        x = torch.empty(T, D, dtype=bf16, device="cuda")
        ids = torch.empty(T, K, dtype=torch.int64, device="cuda")
        scores = torch.empty(T, K, dtype=f32, device="cuda")
        w13 = torch.empty(el, 2 * F, D, dtype=bf16, device="cuda")
        w2 = torch.empty(el, D, F, dtype=bf16, device="cuda")
        slot = torch.empty(1, dtype=torch.int64, device="cuda")
        out, state = torch.ops.dist_moe.bf16_forward(x, ids, scores, w13, w2, None, False, 1e-6, f32, bf16, True, 0.0,
                                                     False, False, slot, 1, False, fake_context)
        assert out.shape == (T, D) and out.dtype == bf16 and len(state) == 9
        assert state[0].shape == (el,) and state[1].shape == (2 * el * T,) and state[7].shape == (6,)
        gx, gs, g13, g2 = torch.ops.dist_moe.bf16_backward(out, w13, w2, ids, scores, state, False, 1e-6, f32, bf16,
                                                           True, False, False, f32, fake_context)
        assert gx.shape == x.shape and gs.shape == scores.shape
        assert g13.shape == w13.shape and g13.dtype == f32 and g2.shape == w2.shape
        out2, st2 = torch.ops.dist_moe.block_scaled_forward(x, ids, scores, w13, w2, [None] * 12, None, False, 1e-6,
                                                            f32, bf16, True, 0.0, False, False, slot, 1, True, False,
                                                            fake_context, False)
        assert out2.shape == (T, D) and len(st2) == 14 and st2[4].shape[1] == 2 * F
        q, s0, s1 = torch.ops.dist_moe.prepare_mxfp8_weight(w13, False, False)
        assert q.shape == (el, 2 * F, D) and q.dtype == torch.uint8 and s1.numel() > 0
        q4, s4, gs4, gsi4 = torch.ops.dist_moe.prepare_nvfp4_weight(w13, False)
        assert q4.shape == (el, 2 * F, D // 2) and gs4.shape == (el,)


def test_missing_context_is_reported():
    with pytest.raises(RuntimeError, match="not live"):
        _ops._context("no-such-context")
