"""``dm_route_static``: routing metadata for hosts that must not allocate device memory.

A serving loop that has given all free HBM to its KV cache, or a plugin that may not touch
its host framework's allocator, cannot hand ``dm_route`` a workspace.  The static entry
point keeps the intermediate counters in an array inside the library instead.  This file
calls it through the C ABI twice in a row (the array keeps the previous call's contents,
so the second call proves the clearing is right) and requires bit-identical tables to
``dm_route``.  It is collected last on purpose: a stop-at-first-failure run has then
already exercised everything else.
"""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
HEADER = 128


def _publish_all(nat, ids_all, num_experts, dev, status):
    ep, T, K = ids_all.shape
    bufs = []
    for s in range(ep):
        buf = torch.zeros(HEADER + T * K * 2, dtype=torch.uint8, device=dev)
        ids = torch.from_numpy(ids_all[s]).to(dev).to(torch.int32).contiguous()
        nat.check(nat.lib.dm_publish(None, ids.data_ptr(), 0, None, buf.data_ptr(), T, 0, K, num_experts, 0,
                                     status.data_ptr(), nat.stream_ptr()), "dm_publish")
        bufs.append(buf)
    return bufs


def _route(nat, static, bufs, ids_shape, rank, E, m_mult, dev, status):
    ep, T, K = ids_shape
    el = E // ep
    size = (ep * T * min(K, el) + el * (m_mult - 1) + m_mult - 1) // m_mult * m_mult if m_mult else ep * el * T
    routing_ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device=dev)
    disp = torch.tensor([(s + 1) << 40 for s in range(ep)], dtype=torch.int64, device=dev)
    comb = torch.tensor([((s + 1) << 40) | (1 << 39) for s in range(ep)], dtype=torch.int64, device=dev)
    out = dict(counts=torch.full((el,), -1, dtype=torch.int32, device=dev),
               per_rank=torch.full((ep,), -1, dtype=torch.int32, device=dev),
               offsets=torch.full((el + 1,), -1, dtype=torch.int32, device=dev),
               fwd=torch.zeros(size, dtype=torch.int64, device=dev),
               bwd=torch.zeros(size, dtype=torch.int64, device=dev),
               sct=torch.zeros(size, dtype=torch.int64, device=dev))
    head = (routing_ptrs.data_ptr(), disp.data_ptr(), comb.data_ptr(), rank, ep, T, K, E, 4096, 4096, 4096, m_mult,
            size, size, out["counts"].data_ptr(), out["per_rank"].data_ptr(), out["offsets"].data_ptr(),
            out["fwd"].data_ptr(), out["bwd"].data_ptr(), out["sct"].data_ptr())
    if static:
        rc = nat.lib.dm_route_static(*head, status.data_ptr(), nat.stream_ptr())
        nat.check(rc, nat.route_call_name(ep, T, el))
    else:
        words = nat.lib.dm_route_workspace_words(T, ep, E)
        ws = torch.empty(words, dtype=torch.int32, device=dev)
        rc = nat.lib.dm_route(*head, ws.data_ptr(), words, status.data_ptr(), nat.stream_ptr())
        nat.check(rc, nat.route_call_name(ep, T, el))
    torch.cuda.synchronize()
    rows = int(out["offsets"][-1])
    return {k: (v[:rows] if k in ("fwd", "bwd", "sct") else v).cpu().numpy() for k, v in out.items()}


def test_static_routing_matches_workspace_routing_on_two_calls_in_a_row():
    from dist_moe_b200 import _native as nat

    dev = torch.device("cuda", 0)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    rng = np.random.default_rng(11)
    # Different shapes back to back.  The first two have ep * T > 1024, so they run the three general kernels, the
    # only ones that use the array: the second of them (other chunk counts, padded expert segments) starts from the
    # first one's leftovers.  The third is in the single-launch decode regime, which keeps its counters in shared
    # memory and must give the same tables through this entry point too.
    shapes = [(4, 1000, 6, 64, 0), (2, 700, 4, 16, 128), (2, 300, 4, 16, 128)]
    for ep, T, K, E, m_mult in shapes:
        general = ep * T > 1024
        assert nat.route_call_name(ep, T, E // ep) == ("dm_route" if general else "dm_route(single launch)")
        ids = np.argsort(-rng.standard_normal((ep, T, E)), axis=-1)[..., :K].astype(np.int64)
        ids[rng.random(ids.shape) < 0.05] = -1
        bufs = _publish_all(nat, ids, E, dev, status)
        want = _route(nat, False, bufs, ids.shape, ep - 1, E, m_mult, dev, status)
        for attempt in range(2):
            got = _route(nat, True, bufs, ids.shape, ep - 1, E, m_mult, dev, status)
            for key in want:
                np.testing.assert_array_equal(got[key], want[key], err_msg=f"{key}, call {attempt}, shape {(ep, T, K, E)}")
    assert status[0].item() == 0, status.tolist()


def test_static_routing_rejects_shapes_beyond_the_fixed_array():
    from dist_moe_b200 import _native as nat

    dev = torch.device("cuda", 0)
    dummy = torch.zeros(16, dtype=torch.int64, device=dev)
    d = dummy.data_ptr()
    # 8 ranks x 256 chunks x 32 local experts x 2 + 256 words > 65536
    rc = nat.lib.dm_route_static(d, d, d, 0, 8, 65536, 8, 256, 512, 512, 512, 0, 1, 1, d, d, d, d, d, d, d,
                                 nat.stream_ptr())
    assert rc == -3  # DM_RC_TOO_LARGE, nothing launched
    torch.cuda.synchronize()
