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


# ---------------------------------------------------------------------------------------------------------------
# Size-independent properties on seeded random scenarios (sizes up to the MXFP8 training configuration and beyond
# 2**31 bytes), and the CUDA kernels against the oracle on the same scenarios.
# ---------------------------------------------------------------------------------------------------------------
def _random_scenarios(count=24, seed=1234):
    import random

    rng = random.Random(seed)
    out = []
    for i in range(count):
        big = i % 6 == 0
        ep = rng.choice([1, 2, 4, 8])
        T = rng.choice([8192, 4096]) if big else rng.choice([16, 64, 200, 512])
        K = rng.choice([2, 4, 8])
        D = rng.choice([4096, 7168]) if big else rng.choice([128, 256, 512, 1024])
        F = rng.choice([1536, 2048]) if big else rng.choice([128, 384, 512])
        layers = rng.choice([1, 2, 3])
        native, mega = rng.random() < 0.3, rng.random() < 0.3
        storage = oracle_bs.NVFP4 if rng.random() < 0.3 else oracle_bs.MXFP8
        calls = []
        for _ in range(layers):
            per_rank = [max(0, int(T * K * rng.uniform(0.2, 1.8))) for _ in range(ep)]
            rows = (per_rank[0] + rng.randrange(0, 16) * 128 + 127) // 128 * 128
            calls.append((rows, per_rank))
        worst_rows = max(r for r, _ in calls)
        x_mem = oracle_bs.packed_dispatch_size(T, D, storage) if native else oracle_planner.align(T * D * 2)
        full = max(oracle_bs._saved_cost(max(p), oracle_planner.align(T * K * D * 2), D, F, storage, native)
                   for _, p in calls)
        # slot between "inputs only" and "everything saved", so that both decisions occur across scenarios
        slot = oracle_planner.align(int(layers * x_mem + rng.uniform(0.0, 1.2) * layers * full) + 128 * 1024)
        scratch = 8 * worst_rows * (D + 6 * F + 64) + (1 << 20)
        out.append(dict(ep=ep, T=T, K=K, D=D, F=F, layers=layers, native=native, mega=mega, storage=storage,
                        calls=calls, slot=slot, arena=slot + oracle_planner.align(scratch)))
    return out


def _live_ranges(fwd, bwd, sc, rows):
    """(name, start, size) of what the backward reads or writes at the same time, from the two plans."""
    s, D, F = sc["storage"], sc["D"], sc["F"]
    xc = sum(oracle_bs.col_sizes(rows, D, s))
    hc = sum(oracle_bs.col_sizes(rows, F, s))
    dc = sum(oracle_bs.col_sizes(rows, 2 * F, s))
    h1, g2 = oracle_planner.align(rows * 2 * F * 2), oracle_planner.align(rows * F * 2)
    o = bwd["offsets"]
    return [("x_col", o[7], xc), ("h1", o[1], h1), ("h2_col", o[9], hc), ("grad_h3_col", o[11], xc), ("grad_h2", o[3], g2),
            ("dxy_col", o[13], dc)]


def test_oracle_properties_on_random_scenarios():
    decisions = set()
    for sc in _random_scenarios():
        st = oracle_planner.PlannerState(1, sc["ep"], sc["slot"], sc["arena"])
        initial = st.snapshot()
        kw = dict(T=sc["T"], K=sc["K"], D=sc["D"], F=sc["F"], storage=sc["storage"])
        plans = []
        for rows, per_rank in sc["calls"]:
            f = oracle_bs.plan_forward(st, rows, per_rank, 0, num_layers=sc["layers"], mega=sc["mega"],
                                       native=sc["native"], **kw)
            decisions.add(f["need"])
            assert all(v % 128 == 0 for v in f["offsets"][:9]), f
            assert all(v == oracle_bs.MISSING or v % 128 == 0 for v in f["table"] if v != f["table"][15]), f
            plans.append((rows, per_rank, f))
        fits = min(st.peak) >= 0
        for rows, per_rank, f in reversed(plans):
            b = oracle_bs.plan_backward(st, rows, per_rank, f["need"], f["offsets"], mega=sc["mega"],
                                        native=sc["native"], **kw)
            assert all(v % 128 == 0 for v in b["offsets"][:14]), b
            if not sc["native"] and fits and min(st.peak) >= 0:
                live = sorted(_live_ranges(f, b, sc, rows), key=lambda r: r[1])
                for (na, a0, an), (nb, b0, _) in zip(live, live[1:]):
                    assert a0 + an <= b0, (na, nb, a0, an, b0)          # no two live tensors share a byte
                assert live[-1][1] + live[-1][2] <= sc["arena"]
        after = st.snapshot()
        assert after["buffer_offsets"] == initial["buffer_offsets"] and after["saved"] == initial["saved"] \
            and after["layer"] == initial["layer"]                       # LIFO: the slot is exactly rewound
    assert decisions == {True, False}


@pytest.mark.gpu
def test_kernels_match_the_oracle_on_random_scenarios():
    import ctypes

    from dist_moe_b200 import _native as nat

    dev = torch.device("cuda", 0)
    i64 = lambda v: torch.tensor(v, dtype=torch.int64, device=dev)  # noqa: E731
    for sc in _random_scenarios():
        ep = sc["ep"]
        st = oracle_planner.PlannerState(1, ep, sc["slot"], sc["arena"])
        storage = (ctypes.c_int * 6)(*sc["storage"].as_list())
        offs, saved = i64(st.buffer_offsets), torch.zeros(ep, dtype=torch.int64, device=dev)
        peak, layer, sel = i64(st.peak), torch.zeros(1, dtype=torch.int64, device=dev), i64([0])
        status = torch.zeros(8, dtype=torch.int32, device=dev)
        kw = dict(T=sc["T"], K=sc["K"], D=sc["D"], F=sc["F"], storage=sc["storage"])
        dims = (ep, sc["T"], sc["K"], sc["D"], sc["F"], storage, 1 << 40, sc["slot"], 1)
        held = []
        for rows, per_rank in sc["calls"]:
            want = oracle_bs.plan_forward(st, rows, per_rank, 0, num_layers=sc["layers"], mega=sc["mega"],
                                          native=sc["native"], **kw)
            r = torch.tensor([rows], dtype=torch.int32, device=dev)
            pr = torch.tensor(per_rank, dtype=torch.int32, device=dev)
            need = torch.zeros(1, dtype=torch.uint8, device=dev)
            fo, ft = torch.zeros(10, dtype=torch.int64, device=dev), torch.zeros(18, dtype=torch.int64, device=dev)
            nat.check(nat.lib.dm_plan_fwd_blockscaled(
                r.data_ptr(), pr.data_ptr(), None, saved.data_ptr(), offs.data_ptr(), peak.data_ptr(), need.data_ptr(),
                None, fo.data_ptr(), ft.data_ptr(), sel.data_ptr(), layer.data_ptr(), *dims, sc["layers"],
                int(sc["mega"]), 0, 0, int(sc["native"]), 0, status.data_ptr(), nat.stream_ptr()), "plan_fwd_blockscaled")
            assert bool(need.item()) == want["need"] and fo.tolist() == want["offsets"] and ft.tolist() == want["table"]
            held.append((r, pr, need, fo, rows, per_rank, want))
        for r, pr, need, fo, rows, per_rank, f in reversed(held):
            want = oracle_bs.plan_backward(st, rows, per_rank, f["need"], f["offsets"], mega=sc["mega"],
                                           native=sc["native"], **kw)
            bo, bt = torch.zeros(16, dtype=torch.int64, device=dev), torch.zeros(54, dtype=torch.int64, device=dev)
            nat.check(nat.lib.dm_plan_bwd_blockscaled(
                r.data_ptr(), pr.data_ptr(), saved.data_ptr(), offs.data_ptr(), peak.data_ptr(), need.data_ptr(),
                fo.data_ptr(), bo.data_ptr(), bt.data_ptr(), layer.data_ptr(), *dims, int(sc["mega"]), int(sc["native"]),
                status.data_ptr(), nat.stream_ptr()), "plan_bwd_blockscaled")
            assert bo.tolist() == want["offsets"] and bt.tolist() == want["table"]
        assert dict(buffer_offsets=offs.tolist(), saved=saved.tolist(), peak=peak.tolist(), layer=layer.tolist()) \
            == st.snapshot()
