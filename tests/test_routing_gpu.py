"""Publication + routing metadata on the GPU, bit-exact against the golden tables made by
the reference's kernels and against the CPU oracle on larger seeded cases."""

import numpy as np
import pytest
import torch

from oracle import routing as oracle_routing
from tests.test_oracle_golden import ROUTING_CASES, check_tables_against_golden, load_routing

pytestmark = pytest.mark.gpu
HEADER = 128


def _native():
    from dist_moe_b200 import _native

    return _native


def run_route(ids_all, rank, num_experts, disp_base, comb_base, gs, bs, ss, m_mult, bwd=True, capacity=None,
              ids_dtype=torch.int32):
    """Publish every rank's ids into its own routing buffer on one GPU, then route for `rank`."""
    nat = _native()
    dev = torch.device("cuda", 0)
    ep, T, K = ids_all.shape
    el = num_experts // ep
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    bufs = []
    for s in range(ep):
        buf = torch.zeros(HEADER + T * K * 2, dtype=torch.uint8, device=dev)
        ids = torch.from_numpy(ids_all[s].astype(np.int64)).to(dev).to(ids_dtype).contiguous()
        nat.check(nat.lib.dm_publish(None, ids.data_ptr(), int(ids_dtype == torch.int64), None, buf.data_ptr(), T, 0, K,
                                     num_experts, 1, status.data_ptr(), nat.stream_ptr()), "dm_publish")
        bufs.append(buf)
    routing_ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    dptr = torch.from_numpy(np.asarray(disp_base, dtype=np.int64)).to(dev)
    cptr = torch.from_numpy(np.asarray(comb_base, dtype=np.int64)).to(dev)
    if m_mult:
        size = (ep * T * min(K, el) + el * (m_mult - 1) + m_mult - 1) // m_mult * m_mult
    else:
        size = ep * el * T
    cap = size if capacity is None else capacity
    counts = torch.full((el,), -1, dtype=torch.int32, device=dev)
    per_rank = torch.full((ep,), -1, dtype=torch.int32, device=dev)
    offsets = torch.full((el + 1,), -1, dtype=torch.int32, device=dev)
    fwd = torch.full((size,), -5, dtype=torch.int64, device=dev)
    bwd_t = torch.full((size,), -5, dtype=torch.int64, device=dev) if bwd else None
    sct = torch.full((size,), -5, dtype=torch.int64, device=dev)
    words = nat.lib.dm_route_workspace_words(T, ep, num_experts)
    ws = torch.empty(words, dtype=torch.int32, device=dev)
    rc = nat.lib.dm_route(routing_ptrs.data_ptr(), dptr.data_ptr(), cptr.data_ptr(), rank, ep, T, K, num_experts, gs,
                          bs, ss, m_mult, cap, size, counts.data_ptr(), per_rank.data_ptr(), offsets.data_ptr(),
                          fwd.data_ptr(), nat.ptr(bwd_t), sct.data_ptr(), ws.data_ptr(), words, status.data_ptr(),
                          nat.stream_ptr())
    nat.check(rc, "dm_route")
    torch.cuda.synchronize()
    return dict(status=status.cpu().numpy(), counts=counts.cpu().numpy(), per_rank=per_rank.cpu().numpy(),
                offsets=offsets.cpu().numpy(), fwd=fwd.cpu().numpy(), sct=sct.cpu().numpy(),
                bwd=None if bwd_t is None else bwd_t.cpu().numpy())


@pytest.mark.parametrize("name", ROUTING_CASES)
def test_route_matches_reference_golden(name):
    g = load_routing(name)
    ids = g["ids"].astype(np.int64)
    has_bwd = "r0_bwd" in g.files
    for rank in range(ids.shape[0]):
        out = run_route(ids, rank, int(g["num_experts"]), g["r0_disp_base"], g["r0_comb_base"], int(g["gather_stride"]),
                        int(g["bwd_stride"]) or int(g["gather_stride"]), int(g["scatter_stride"]),
                        int(g["m_multiple_of"]), bwd=has_bwd)
        assert out["status"][0] == 0, out["status"]
        rows = check_tables_against_golden(g, rank, out["counts"], out["per_rank"], out["fwd"], out["bwd"], out["sct"],
                                           f"{name} rank {rank}")
        assert out["offsets"][-1] == rows
        np.testing.assert_array_equal(out["offsets"], np.concatenate([[0], np.cumsum(out["counts"])]))


@pytest.mark.parametrize(
    "ep,T,K,E,m_mult,ids_dtype",
    [(8, 4096, 6, 64, 0, torch.int64), (8, 1024, 8, 128, 128, torch.int32), (1, 4096, 6, 64, 0, torch.int64),
     (2, 1, 1, 2, 0, torch.int32), (4, 257, 8, 256, 128, torch.int32)],
)
def test_route_matches_oracle_at_full_size(ep, T, K, E, m_mult, ids_dtype):
    rng = np.random.default_rng(1000 + ep + T)
    logits = rng.standard_normal((ep, T, E))
    ids = np.argsort(-logits, axis=-1)[..., :K].astype(np.int64)
    if T > 4:
        ids[rng.random(ids.shape) < 0.02] = -1
    disp = [(s + 1) << 40 for s in range(ep)]
    comb = [((s + 1) << 40) | (1 << 39) for s in range(ep)]
    D = 2048
    for rank in sorted({0, ep - 1}):
        out = run_route(ids, rank, E, disp, comb, D * 2, D * 2, D * 2, m_mult, ids_dtype=ids_dtype)
        assert out["status"][0] == 0, out["status"]
        t = oracle_routing.route(ids, rank, E, disp, comb, D * 2, D * 2, D * 2, m_mult)
        rows = int(t.expert_offsets[-1])
        np.testing.assert_array_equal(out["counts"], t.counts)
        np.testing.assert_array_equal(out["per_rank"], t.per_rank)
        np.testing.assert_array_equal(out["offsets"], t.expert_offsets)
        np.testing.assert_array_equal(out["fwd"][:rows], t.fwd)
        np.testing.assert_array_equal(out["bwd"][:rows], t.bwd)
        np.testing.assert_array_equal(out["sct"][:rows], t.sct)


def test_route_reports_capacity_and_invalid_ids_without_trapping():
    rng = np.random.default_rng(7)
    ids = rng.integers(0, 8, size=(2, 64, 2)).astype(np.int64)
    ids[:, :, 1] = (ids[:, :, 0] + 1) % 8
    disp, comb = [1 << 40, 2 << 40], [3 << 40, 4 << 40]
    out = run_route(ids, 0, 8, disp, comb, 512, 512, 512, 0, capacity=4)
    assert out["status"][0] == 2, out["status"]  # capacity exceeded
    assert out["offsets"][-1] == 0 and not out["counts"].any()
    bad = ids.copy()
    bad[0, 0, 0] = 99
    out = run_route(bad, 0, 8, disp, comb, 512, 512, 512, 0)
    assert out["status"][0] == 3, out["status"]  # invalid expert id, reported by the publication check


@pytest.mark.parametrize("ep,T,K,E,m_mult", [(8, 128, 8, 256, 128), (1, 128, 8, 256, 128), (2, 512, 4, 64, 0),
                                             (4, 256, 8, 32, 128), (1, 1, 1, 4, 0), (8, 100, 6, 64, 0)])
def test_single_launch_decode_routing_equals_the_general_path_and_the_oracle(ep, T, K, E, m_mult):
    """ep * T <= 1024 takes the one-CTA kernel; its tables are those of the three general kernels and of the oracle."""
    nat = _native()
    rng = np.random.default_rng(77 + ep + T)
    ids = np.argsort(-rng.standard_normal((ep, T, E)), axis=-1)[..., :K].astype(np.int64)
    if T > 4:
        ids[rng.random(ids.shape) < 0.03] = -1
    disp = [(s + 1) << 40 for s in range(ep)]
    comb = [((s + 1) << 40) | (1 << 39) for s in range(ep)]
    stride = 7168
    for rank in sorted({0, ep - 1}):
        outs = {}
        for decode in (0, 1):
            previous = nat.lib.dm_set_route_decode_kernel(decode)
            try:
                outs[decode] = run_route(ids, rank, E, disp, comb, stride, stride, stride, m_mult)
            finally:
                nat.lib.dm_set_route_decode_kernel(previous)
            assert outs[decode]["status"][0] == 0, outs[decode]["status"]
        t = oracle_routing.route(ids, rank, E, disp, comb, stride, stride, stride, m_mult)
        rows = int(t.expert_offsets[-1])
        for key in ("counts", "per_rank", "offsets"):
            np.testing.assert_array_equal(outs[1][key], outs[0][key])
        for key in ("fwd", "bwd", "sct"):
            np.testing.assert_array_equal(outs[1][key][:rows], outs[0][key][:rows])
        np.testing.assert_array_equal(outs[1]["counts"], t.counts)
        np.testing.assert_array_equal(outs[1]["per_rank"], t.per_rank)
        np.testing.assert_array_equal(outs[1]["fwd"][:rows], t.fwd)
        np.testing.assert_array_equal(outs[1]["sct"][:rows], t.sct)
