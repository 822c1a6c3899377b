"""Arena planner, block-scaled paths: the CPU oracle and the CUDA planner kernels against scenarios recorded from the
reference's own kernels (``tests/golden/planner_blockscaled.json``): MXFP8 saved / recomputed / mixed LIFO stacks, two
slots with a scratch-only forward, the mega and native-backward layouts, NVFP4 geometry, and the inference layouts
(with and without the interleaved W13 epilogue)."""

import json
from pathlib import Path

import pytest
import torch

from oracle import planner as oracle_planner
from oracle import planner_blockscaled as oracle_bs

GOLDEN = json.loads((Path(__file__).resolve().parent / "golden" / "planner_blockscaled.json").read_text())


def _flags(c):
    f = c["flags"]
    return dict(mega=bool(f.get("mega")), native=bool(f.get("native_backward"))), \
        dict(inference=bool(f.get("inference_mode")), interleaved=bool(f.get("interleaved_fc13")))


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_oracle_matches_reference_kernels(name):
    c = GOLDEN[name]
    st = oracle_planner.PlannerState(c["slots"], c["EP"], c["slot_bytes"], c["arena_bytes"])
    if c["slots"] == 0:
        st.saved, st.layer = [0], [0]  # the recorded state keeps one placeholder entry
    both, fwd_only = _flags(c)
    dims = dict(T=c["T"], K=c["K"], D=c["D"], F=c["F"], storage=oracle_bs.Storage(*c["storage"]))
    fwd = []
    for step in c["steps"]:
        if step["op"] == "f":
            got = oracle_bs.plan_forward(st, step["R"], step["per_rank"], step["slot"], num_layers=c["layers"],
                                         scratch_only=step["scratch_only"] and not fwd_only["inference"], **dims,
                                         **both, **fwd_only)
            assert got["need"] == step["need"], (name, step)
            assert got["offsets"][:9] == step["offsets"], (name, got["offsets"], step["offsets"])
            assert got["table"] == step["table"], (name, got["table"], step["table"])
            fwd.append(dict(step, offsets10=got["offsets"]))
        else:
            f = fwd[step["of"]]
            got = oracle_bs.plan_backward(st, f["R"], f["per_rank"], f["need"], f["offsets10"], **dims, **both)
            assert got["offsets"] == step["offsets"], (name, got["offsets"], step["offsets"])
            assert got["table"] == step["table"], (name, got["table"], step["table"])
        assert st.snapshot() == step["state"], (name, step["op"], st.snapshot(), step["state"])


def test_scenarios_cover_the_branches():
    needs = {(bool(c["flags"].get("native_backward")), s["need"]) for c in GOLDEN.values() for s in c["steps"]
             if s["op"] == "f" and not s["scratch_only"]}
    assert needs == {(False, False), (False, True), (True, False), (True, True)}
    assert any(c["flags"].get("mega") for c in GOLDEN.values())
    assert {c["format"] for c in GOLDEN.values()} == {"MXFP8_E4M3", "NVFP4"}


def test_storage_constants_match_the_format_table():
    from dist_moe_b200._blockscaled import planner_storage
    from dist_moe_b200.formats import BlockScaledFormat

    assert planner_storage(BlockScaledFormat.MXFP8_E4M3) == oracle_bs.MXFP8.as_list()
    assert planner_storage(BlockScaledFormat.NVFP4) == oracle_bs.NVFP4.as_list()


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_kernels_match_reference_kernels(name):
    import ctypes

    from dist_moe_b200 import _native as nat

    c = GOLDEN[name]
    dev = torch.device("cuda", 0)
    n, ep = c["slots"], c["EP"]
    both, fwd_only = _flags(c)
    storage = (ctypes.c_int * 6)(*c["storage"])
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
    offs = i64([i * c["slot_bytes"] for i in range(n)] + [c["arena_bytes"]])
    saved = torch.zeros(max(1, n * ep), dtype=torch.int64, device=dev)
    peak = i64([c["slot_bytes"]] * n + [c["arena_bytes"] - n * c["slot_bytes"]])
    layer = torch.zeros(max(1, n), dtype=torch.int64, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    fwd = []
    for step in c["steps"]:
        if step["op"] == "f":
            rows = torch.tensor([step["R"]], dtype=torch.int32, device=dev)
            per_rank = torch.tensor(step["per_rank"], dtype=torch.int32, device=dev)
            snapshot = torch.zeros(ep, dtype=torch.int32, device=dev)
            need = torch.zeros(1, dtype=torch.uint8, device=dev)
            cond = torch.zeros(1, dtype=torch.int32, device=dev)
            fo = torch.zeros(10, dtype=torch.int64, device=dev)
            table = torch.zeros(18, dtype=torch.int64, device=dev)
            sel = i64([step["slot"]])
            nat.check(nat.lib.dm_plan_fwd_blockscaled(
                rows.data_ptr(), per_rank.data_ptr(), snapshot.data_ptr(), saved.data_ptr(), offs.data_ptr(),
                peak.data_ptr(), need.data_ptr(), cond.data_ptr(), fo.data_ptr(), table.data_ptr(), sel.data_ptr(),
                layer.data_ptr(), ep, c["T"], c["K"], c["D"], c["F"], storage, c["capacity_rows"], c["slot_bytes"], n,
                c["layers"], int(both["mega"]), int(fwd_only["inference"]),
                int(step["scratch_only"] and not fwd_only["inference"]), int(both["native"]),
                int(fwd_only["interleaved"]), status.data_ptr(), nat.stream_ptr()), "plan_fwd_blockscaled")
            assert bool(need.item()) == step["need"] and cond.item() == step["cond"]
            assert fo.tolist()[:9] == step["offsets"] and fo[9].item() == step["slot"]
            assert table.tolist() == step["table"]
            assert snapshot.tolist() == step["per_rank"]
            fwd.append((rows, per_rank, need, fo))
        else:
            rows, per_rank, need, fo = fwd[step["of"]]
            bo = torch.zeros(16, dtype=torch.int64, device=dev)
            table = torch.zeros(54, dtype=torch.int64, device=dev)
            nat.check(nat.lib.dm_plan_bwd_blockscaled(
                rows.data_ptr(), per_rank.data_ptr(), saved.data_ptr(), offs.data_ptr(), peak.data_ptr(),
                need.data_ptr(), fo.data_ptr(), bo.data_ptr(), table.data_ptr(), layer.data_ptr(), ep, c["T"], c["K"],
                c["D"], c["F"], storage, c["capacity_rows"], c["slot_bytes"], n, int(both["mega"]),
                int(both["native"]), status.data_ptr(), nat.stream_ptr()), "plan_bwd_blockscaled")
            assert bo.tolist() == step["offsets"]
            assert table.tolist() == step["table"]
        got = dict(buffer_offsets=offs.tolist(), saved=saved.tolist(), peak=peak.tolist(), layer=layer.tolist())
        assert got == step["state"], (step["op"], got, step["state"])
    # two recorded scenarios run out of room (the reference's device assertion is inert under the interpreter): the
    # numbers still match, and the status word says so
    overflowed = min(min(step["state"]["peak"]) for step in c["steps"]) < 0
    assert nat.STATUS_NAMES[status[0].item()] == ("activation arena overflow" if overflowed else "ok")


@pytest.mark.gpu
def test_overflow_sets_the_status_word_instead_of_asserting():
    import ctypes

    from dist_moe_b200 import _native as nat

    dev = torch.device("cuda", 0)
    storage = (ctypes.c_int * 6)(*oracle_bs.MXFP8.as_list())
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
    slot_bytes, arena = 4096, 4096 + 8192  # far too small for 256 rows
    offs, saved, peak, layer = i64([0, arena]), i64([0]), i64([slot_bytes, arena - slot_bytes]), i64([0])
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    rows = torch.tensor([256], dtype=torch.int32, device=dev)
    need, sel = torch.zeros(1, dtype=torch.uint8, device=dev), i64([0])
    fo, table = torch.zeros(10, dtype=torch.int64, device=dev), torch.zeros(18, dtype=torch.int64, device=dev)
    nat.check(nat.lib.dm_plan_fwd_blockscaled(
        rows.data_ptr(), rows.data_ptr(), None, saved.data_ptr(), offs.data_ptr(), peak.data_ptr(), need.data_ptr(),
        None, fo.data_ptr(), table.data_ptr(), sel.data_ptr(), layer.data_ptr(), 1, 64, 2, 256, 128, storage,
        1024, slot_bytes, 1, 1, 0, 0, 0, 0, 0, status.data_ptr(), nat.stream_ptr()), "plan_fwd_blockscaled")
    torch.cuda.synchronize()
    assert nat.STATUS_NAMES[status[0].item()] == "activation arena overflow"
    assert peak[1].item() < 0  # the overflow is also visible in the peak counters
