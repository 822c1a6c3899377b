"""Failure paths that report through the status words instead of trapping or hanging.

Every failure is made on the host: a peer that published another token count, a barrier partner that never
signals.  The waits involved are bounded (a millisecond here), the kernels return, the CUDA context stays usable
and the same entry points work again afterwards.  The reference traps the device in the first case and spins
without a bound in the second (dist_moe/kernels/triton/dist_dispatch_routing_kernel.py:452-470,
dist_moe/kernels/triton/comm_utils.py:70-110).
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
HEADER = 128
TOKEN_COUNT_MISMATCH, BARRIER_TIMEOUT = 1, 4


def _nat():
    from dist_moe_b200 import _native

    return _native


def _route_two_local_ranks(T_published, T_routed, K=2, E=8):
    """Rank 0 routes over two routing buffers of this GPU whose headers hold ``T_published``."""
    nat = _nat()
    ep, el = 2, E // 2
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    bufs = []
    rng = np.random.default_rng(5)
    for s in range(ep):
        t = T_published[s]
        ids = torch.from_numpy(np.argsort(-rng.standard_normal((t, E)), axis=-1)[:, :K].astype(np.int32)).to(DEV)
        buf = torch.zeros(HEADER + max(T_published + [T_routed]) * K * 2, dtype=torch.uint8, device=DEV)
        nat.check(nat.lib.dm_publish(None, ids.data_ptr(), 0, None, buf.data_ptr(), t, 0, K, E, 1, status.data_ptr(),
                                     nat.stream_ptr()), "dm_publish")
        bufs.append(buf)
    T = T_routed
    size = ep * el * T
    routing = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=DEV)
    disp = torch.tensor([1 << 40, 2 << 40], dtype=torch.int64, device=DEV)
    comb = torch.tensor([3 << 40, 4 << 40], dtype=torch.int64, device=DEV)
    counts = torch.full((el,), -1, dtype=torch.int32, device=DEV)
    per_rank = torch.full((ep,), -1, dtype=torch.int32, device=DEV)
    offsets = torch.full((el + 1,), -1, dtype=torch.int32, device=DEV)
    tables = [torch.full((size,), -5, dtype=torch.int64, device=DEV) for _ in range(3)]
    words = nat.lib.dm_route_workspace_words(T, ep, E)
    ws = torch.empty(words, dtype=torch.int32, device=DEV)
    nat.check(nat.lib.dm_route(routing.data_ptr(), disp.data_ptr(), comb.data_ptr(), 0, ep, T, K, E, 512, 512, 512, 0, size,
                               size, counts.data_ptr(), per_rank.data_ptr(), offsets.data_ptr(), tables[0].data_ptr(),
                               tables[1].data_ptr(), tables[2].data_ptr(), ws.data_ptr(), words, status.data_ptr(),
                               nat.stream_ptr()), "dm_route")
    torch.cuda.synchronize()
    return status.cpu().numpy(), counts.cpu().numpy(), offsets.cpu().numpy()


@pytest.mark.parametrize("T,decode", [(64, 1), (64, 0), (2000, 0)])
def test_token_count_mismatch_is_reported_and_routes_nothing(T, decode):
    """A peer whose header holds another T: status 1 with (source rank, its T, my T); zero rows, so the kernels
    that follow do no work.  Covers the single-launch decode kernel and the three general kernels."""
    nat = _nat()
    previous = nat.lib.dm_set_route_decode_kernel(decode)
    try:
        status, counts, offsets = _route_two_local_ranks([T, T + 1], T)
        assert status[0] == TOKEN_COUNT_MISMATCH, status
        assert list(status[1:4]) == [1, T + 1, T]
        assert not counts.any() and offsets[-1] == 0
        # the same entry point, agreeing peers: clean status and real rows
        status, counts, offsets = _route_two_local_ranks([T, T], T)
        assert status[0] == 0 and counts.sum() > 0 and offsets[-1] == counts.sum()
    finally:
        nat.lib.dm_set_route_decode_kernel(previous)


def test_barrier_wait_runs_out_and_reports_instead_of_hanging():
    """Two signal pads on this GPU stand in for two ranks; nobody plays rank 1.  Rank 0 raises its flag in the
    peer's pad, waits one millisecond for the peer's flag in its own pad, gives up with status 4 and returns.
    Then the peer's signal is written by the host and the same call completes normally."""
    nat = _nat()
    pads = [torch.zeros(128, dtype=torch.int32, device=DEV) for _ in range(2)]
    table = torch.tensor([p.data_ptr() for p in pads], dtype=torch.int64, device=DEV)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    nat.check(nat.lib.dm_barrier(table.data_ptr(), 0, 2, 0, None, 1_000_000, status.data_ptr(), nat.stream_ptr()),
              "dm_barrier")
    end.record()
    torch.cuda.synchronize()
    assert status.tolist()[:4] == [BARRIER_TIMEOUT, 1, 0, 1]  # code, silent peer, channel, phase 1 = waiting for its flag
    assert start.elapsed_time(end) < 500.0  # milliseconds: bounded by the limit, not by a watchdog
    assert pads[1][0].item() == 1 and pads[0][1].item() == 0  # own flag was raised, the peer's never came
    # recovery: clear the pads (a real group recreates its context), let the "peer" signal, call again
    for p in pads:
        p.zero_()
    status.zero_()
    pads[0][1] = 1
    nat.check(nat.lib.dm_barrier(table.data_ptr(), 0, 2, 0, None, 1_000_000, status.data_ptr(), nat.stream_ptr()),
              "dm_barrier")
    torch.cuda.synchronize()
    assert status[0].item() == 0
    assert pads[0][1].item() == 0 and pads[1][0].item() == 1  # consumed the peer's flag, left its own for the peer
    # a device-side predicate of zero skips the barrier altogether
    cond = torch.zeros(1, dtype=torch.int32, device=DEV)
    pads[1].zero_()
    nat.check(nat.lib.dm_barrier(table.data_ptr(), 0, 2, 0, cond.data_ptr(), 1_000_000, status.data_ptr(),
                                 nat.stream_ptr()), "dm_barrier")
    torch.cuda.synchronize()
    assert status[0].item() == 0 and pads[1][0].item() == 0


def test_inputs_on_another_device_than_the_context_are_refused():
    """Launches go to the context's device; tensors of another device are refused on the host before any launch."""
    import dist_moe_b200 as dm

    dev = torch.device(DEV)
    cfg = dm.Config(max_num_local_input_tokens=8, hidden_dim=128, intermediate_dim=128, top_k=1, num_experts=2,
                    max_moe_layers_per_activation_slot=1)
    ctx = dm.create_context(group=None, config=cfg, device=dev)
    try:
        x = torch.zeros(8, 128, dtype=torch.bfloat16, device=dev)
        ids = torch.zeros(8, 1, dtype=torch.int32, device=dev)
        sc = torch.ones(8, 1, device=dev)
        w13 = torch.zeros(2, 256, 128, dtype=torch.bfloat16, device=dev)
        w2 = torch.zeros(2, 128, 128, dtype=torch.bfloat16, device=dev)
        dm.routed_experts(x, ids, sc, w13, w2, ctx)
        ctx.check_status()
        real = ctx._state.device
        ctx._state.device = torch.device("cuda", 1)  # pretend the context lives on the next GPU
        try:
            with pytest.raises(ValueError, match="context was created on"):
                dm.routed_experts(x, ids, sc, w13, w2, ctx)
        finally:
            ctx._state.device = real
    finally:
        ctx.close()
