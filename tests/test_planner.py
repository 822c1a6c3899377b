"""Arena planner (BF16): the CPU oracle and the CUDA planner kernels against scenarios
recorded from the reference's own planner kernels (``tests/golden/planner_bf16.json``):
multi-layer LIFO save/recompute decisions, two slots, a scratch-only (no-grad) forward."""

import json
from pathlib import Path

import pytest
import torch

from oracle import planner as oracle_planner

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "planner_bf16.json").read_text())


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_planner_oracle_matches_reference_kernels(name):
    c = GOLDEN[name]
    st = oracle_planner.PlannerState(c["slots"], c["EP"], c["slot_bytes"], c["arena_bytes"])
    dims = dict(T=c["T"], K=c["K"], D=c["D"], F=c["F"])
    fwd = []
    for step in c["steps"]:
        if step["op"] == "f":
            got = oracle_planner.plan_forward(st, step["R"], step["per_rank"], step["slot"], num_layers=c["layers"],
                                              scratch_only=step["scratch_only"], **dims)
            assert got["need"] == step["need"] and got["fwd_state"] == step["fwd_state"], (name, step, got)
            fwd.append(step)
        else:
            f = fwd[step["of"]]
            got = oracle_planner.plan_backward(st, f["R"], f["per_rank"], f["need"], f["fwd_state"], **dims)
            assert got == step["bwd_offsets"], (name, step, got)
        assert st.snapshot() == step["state"], (name, step["op"], st.snapshot(), step["state"])


def test_scenarios_cover_both_decisions():
    needs = {s["need"] for c in GOLDEN.values() for s in c["steps"] if s["op"] == "f" and not s["scratch_only"]}
    assert needs == {True, False}


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_planner_kernels_match_reference_kernels(name):
    from dist_moe_b200 import _native as nat

    c = GOLDEN[name]
    dev = torch.device("cuda", 0)
    n, ep = c["slots"], c["EP"]
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
    offs = i64([i * c["slot_bytes"] for i in range(n)] + [c["arena_bytes"]])
    saved = torch.zeros(n * ep, dtype=torch.int64, device=dev)
    peak = i64([c["slot_bytes"]] * n + [c["arena_bytes"] - n * c["slot_bytes"]])
    layer = torch.zeros(n, dtype=torch.int64, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    fwd = []
    for step in c["steps"]:
        if step["op"] == "f":
            rows = torch.tensor([step["R"]], dtype=torch.int32, device=dev)
            per_rank = torch.tensor(step["per_rank"], dtype=torch.int32, device=dev)
            need = torch.zeros(1, dtype=torch.uint8, device=dev)
            cond = torch.zeros(1, dtype=torch.int32, device=dev)
            fs = torch.zeros(6, dtype=torch.int64, device=dev)
            sel = i64([step["slot"]])
            nat.check(nat.lib.dm_plan_fwd_bf16(rows.data_ptr(), per_rank.data_ptr(), saved.data_ptr(), offs.data_ptr(),
                                               peak.data_ptr(), need.data_ptr(), cond.data_ptr(), fs.data_ptr(),
                                               sel.data_ptr(), layer.data_ptr(), ep, c["T"], c["K"], c["D"], c["F"],
                                               c["slot_bytes"], n, c["layers"], int(step["scratch_only"]),
                                               status.data_ptr(), nat.stream_ptr()), "plan_fwd")
            assert bool(need.item()) == step["need"] and cond.item() == int(step["need"])
            assert fs.tolist() == step["fwd_state"], (fs.tolist(), step["fwd_state"])
            fwd.append((rows, per_rank, need, fs))
        else:
            rows, per_rank, need, fs = fwd[step["of"]]
            bo = torch.zeros(6, dtype=torch.int64, device=dev)
            nat.check(nat.lib.dm_plan_bwd_bf16(rows.data_ptr(), per_rank.data_ptr(), saved.data_ptr(), offs.data_ptr(),
                                               peak.data_ptr(), need.data_ptr(), fs.data_ptr(), bo.data_ptr(),
                                               layer.data_ptr(), ep, c["T"], c["K"], c["D"], c["F"], c["slot_bytes"], n,
                                               status.data_ptr(), nat.stream_ptr()), "plan_bwd")
            assert bo.tolist() == step["bwd_offsets"]
        got = dict(buffer_offsets=offs.tolist(), saved=saved.tolist(), peak=peak.tolist(), layer=layer.tolist())
        assert got == step["state"], (step["op"], got, step["state"])
    assert status[0].item() == 0
