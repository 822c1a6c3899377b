"""Expert-parallel execution of the routed-expert layer on CPU ranks (gloo), built from the oracle pieces.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Each rank owns ``E / world`` experts and its own tokens.  The data flow is the reference's
(dist_moe/api.py:1844-2188): every rank publishes its expert ids (all-gather), the routing tables of
``oracle/routing.py`` say which (source rank, token, route) rows each rank receives and in which order,
rows travel to the expert's rank (dispatch), the local experts run, and every output row travels back to
the (token, route) slot of its source rank (combine), where the score-weighted reduction happens.
Used by the world_size-2 CPU tests and as the quick-start CPU baseline.
"""

from __future__ import annotations

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import moe as oracle_moe
from . import routing as oracle_routing


def _all_to_all(recv, send, group):
    """List all-to-all built from point-to-point messages (gloo has no native all_to_all)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    recv[rank].copy_(send[rank])
    ops = []
    for peer in range(world):
        if peer == rank:
            continue
        ops.append(dist.P2POp(dist.isend, send[peer], peer, group))
        ops.append(dist.P2POp(dist.irecv, recv[peer], peer, group))
    if ops:
        for work in dist.batch_isend_irecv(ops):
            work.wait()


def moe_forward_ep(x, ids, scores, w13_local, w2_local, num_experts, group=None, *, clamped=False):
    """x [T, D] local tokens, ids/scores [T, K], w13_local [E_local, 2F, D], w2_local [E_local, D, F]."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    T, D = x.shape
    K = ids.shape[1]
    e_local = num_experts // world
    inter = w2_local.shape[2]
    w13_local = w13_local.reshape(e_local, 2 * inter, D)
    all_ids = [torch.empty_like(ids) for _ in range(world)]
    dist.all_gather(all_ids, ids.contiguous(), group=group)
    ids_all = torch.stack(all_ids).numpy()
    zeros = [0] * world
    # tables of every destination rank, computed locally from the gathered ids (deterministic)
    tables = [oracle_routing.route(ids_all, q, num_experts, zeros, zeros, 1, 1, 1) for q in range(world)]
    # ---- dispatch: rows this rank sends to rank q, in q's receive order restricted to this source
    send = []
    for q in range(world):
        mine = tables[q].src == rank
        send.append(x[torch.from_numpy(tables[q].token[mine].astype(np.int64))].contiguous())
    recv = [torch.empty(int((tables[rank].src == s).sum()), D, dtype=x.dtype) for s in range(world)]
    _all_to_all(recv, send, group)
    t = tables[rank]
    rows = int(t.expert_offsets[-1])
    xg = torch.empty(rows, D, dtype=x.dtype)
    for s in range(world):
        xg[torch.from_numpy(np.nonzero(t.src == s)[0])] = recv[s]
    # ---- local experts
    h3 = torch.empty(rows, D, dtype=x.dtype)
    for e in range(e_local):
        lo, hi = int(t.expert_offsets[e]), int(t.expert_offsets[e + 1])
        if hi == lo:
            continue
        h13 = F.linear(xg[lo:hi], w13_local[e])
        gate, up = h13.split(inter, dim=-1)
        h2 = oracle_moe.swiglu(gate, up, clamped=clamped).to(x.dtype)
        h3[lo:hi] = F.linear(h2, w2_local[e])
    # ---- combine: send every row back to its source rank's (token, route) slot
    back = [h3[torch.from_numpy(np.nonzero(t.src == s)[0])].contiguous() for s in range(world)]
    got = [torch.empty(int((tables[q].src == rank).sum()), D, dtype=x.dtype) for q in range(world)]
    _all_to_all(got, back, group)
    combine = torch.zeros(T, K, D, dtype=x.dtype)
    for q in range(world):
        mine = tables[q].src == rank
        tok = torch.from_numpy(tables[q].token[mine].astype(np.int64))
        slot = torch.from_numpy(tables[q].slot[mine].astype(np.int64))
        combine[tok, slot] = got[q]
    return oracle_moe.combine(combine, scores, x.dtype)
