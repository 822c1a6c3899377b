"""The CPU oracle against golden vectors produced by the reference's own code
(``tests/golden/gen_golden.py``: reference Triton kernels under the CPU interpreter,
reference ``plan_memory`` in plain Python)."""

from pathlib import Path

import numpy as np
import pytest

from oracle import routing as oracle_routing

GOLDEN = Path(__file__).resolve().parent / "golden"
ROUTING_CASES = sorted(p.stem[len("routing_"):] for p in GOLDEN.glob("routing_*.npz"))


def load_routing(name):
    return np.load(GOLDEN / f"routing_{name}.npz")


def check_tables_against_golden(g, rank, counts, per_rank, fwd, bwd, sct, what):
    """Compare one rank's tables with the golden ones.  Only rows below the sum of the
    (padded) counts are defined; the reference leaves the tail of its tables unwritten."""
    g_counts = g[f"r{rank}_counts"]
    np.testing.assert_array_equal(np.asarray(counts), g_counts, err_msg=f"{what}: counts")
    np.testing.assert_array_equal(np.asarray(per_rank), g[f"r{rank}_per_rank"], err_msg=f"{what}: per_rank")
    rows = int(g_counts.sum())
    np.testing.assert_array_equal(np.asarray(fwd)[:rows], g[f"r{rank}_fwd"][:rows], err_msg=f"{what}: fwd")
    np.testing.assert_array_equal(np.asarray(sct)[:rows], g[f"r{rank}_sct"][:rows], err_msg=f"{what}: scatter")
    if f"r{rank}_bwd" in g.files and bwd is not None:
        np.testing.assert_array_equal(np.asarray(bwd)[:rows], g[f"r{rank}_bwd"][:rows], err_msg=f"{what}: bwd")
    return rows


@pytest.mark.parametrize("name", ROUTING_CASES)
def test_routing_oracle_matches_reference_kernels(name):
    g = load_routing(name)
    ids = g["ids"].astype(np.int64)
    ep = ids.shape[0]
    for rank in range(ep):
        t = oracle_routing.route(
            ids, rank, int(g["num_experts"]), g["r0_disp_base"], g["r0_comb_base"], int(g["gather_stride"]),
            int(g["bwd_stride"]) or int(g["gather_stride"]), int(g["scatter_stride"]), int(g["m_multiple_of"]),
        )
        rows = check_tables_against_golden(g, rank, t.counts, t.per_rank, t.fwd, t.bwd, t.sct, f"{name} rank {rank}")
        assert rows == int(t.expert_offsets[-1])


def test_routing_cases_cover_the_edge_cases():
    assert {"quickstart", "random_ep4", "skew_pad128", "single_rank", "multi_chunk"} <= set(ROUTING_CASES)
    g = load_routing("random_ep4")
    assert (g["ids"] < 0).any(), "dropped routes (-1) must be covered"
