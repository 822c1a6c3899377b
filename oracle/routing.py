"""Routing metadata, restated on the CPU (numpy, integer-exact).

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows the reference's general three-phase path
(dist_moe/kernels/triton/dist_dispatch_routing_kernel.py:420-956, launcher
dist_moe/_routing_metadata.py:886-1102):

* expert ``e`` lives on rank ``e // E_local`` (``_routing_metadata.py:1001-1007``);
* a route ``(src, token, k)`` with ``ids[src, token, k] == rank*E_local + el`` becomes one
  output row of local expert ``el``; ids outside ``[0, E)`` are ignored (kernel 556-561, 662-667);
* rows are ordered by (local expert, source rank, token) -- workers own contiguous token
  ranges and are compacted in worker order (kernel 575-580, 657, 772-777, 893-900);
* ``fwd = dispatch_base[src] + token*gather_stride``,
  ``bwd = dispatch_base[src] + (token*K + k)*bwd_stride``,
  ``sct = combine_base[src] + (token*K + k)*scatter_stride`` (kernel 592-644);
* with ``m_multiple_of`` every expert segment is rounded up and the tail holds pointer 0
  (kernel 936-956); ``num_tokens_per_rank[q]`` sums the rounded *global* counts of rank q's
  experts (kernel 659-678, 758-770).

Pinned against the reference's own Triton kernels executed by the Triton CPU
interpreter: ``tests/golden/gen_golden.py`` writes ``tests/golden/routing_*.npz`` and
``tests/test_oracle_golden.py`` compares this module with them.
"""

from __future__ import annotations

import dataclasses

import numpy as np


@dataclasses.dataclass
class RoutingTables:
    counts: np.ndarray  # int32 [E_local], rounded up when m_multiple_of
    per_rank: np.ndarray  # int32 [EP]
    expert_offsets: np.ndarray  # int32 [E_local + 1]
    fwd: np.ndarray  # int64 [rows]
    bwd: np.ndarray  # int64 [rows]
    sct: np.ndarray  # int64 [rows]
    src: np.ndarray  # int32 [rows] source rank (-1 on padding rows)
    token: np.ndarray  # int32 [rows]
    slot: np.ndarray  # int32 [rows] k index


def pad_to(n, m):
    return n if not m else (n + m - 1) // m * m


def route(ids_all, rank, num_experts, dispatch_base, combine_base, gather_stride, bwd_stride, scatter_stride,
          m_multiple_of=0) -> RoutingTables:
    """ids_all: int array [EP, T, K] of every rank's published expert ids."""
    ids_all = np.asarray(ids_all).astype(np.int64)
    ep, T, K = ids_all.shape
    el_n = num_experts // ep
    first = rank * el_n
    valid = (ids_all >= 0) & (ids_all < num_experts)
    hist = np.bincount(ids_all[valid].ravel(), minlength=num_experts).astype(np.int64)
    per_rank = np.array(
        [sum(pad_to(int(hist[q * el_n + el]), m_multiple_of) for el in range(el_n)) for q in range(ep)], dtype=np.int32
    )
    s_idx, t_idx, k_idx = np.nonzero(valid & (ids_all >= first) & (ids_all < first + el_n))
    el = ids_all[s_idx, t_idx, k_idx] - first
    # (expert, source rank, token): nonzero() already yields (s, t, k) ascending, a stable sort by expert keeps it.
    order = np.argsort(el, kind="stable")
    s_idx, t_idx, k_idx, el = s_idx[order], t_idx[order], k_idx[order], el[order]
    real = np.bincount(el, minlength=el_n).astype(np.int64)
    stored = np.array([pad_to(int(c), m_multiple_of) for c in real], dtype=np.int64)
    offsets = np.concatenate([[0], np.cumsum(stored)])
    rows = int(offsets[-1])
    fwd = np.zeros(rows, dtype=np.int64)
    bwd = np.zeros(rows, dtype=np.int64)
    sct = np.zeros(rows, dtype=np.int64)
    src = np.full(rows, -1, dtype=np.int32)
    tok = np.full(rows, -1, dtype=np.int32)
    slot = np.full(rows, -1, dtype=np.int32)
    real_start = np.concatenate([[0], np.cumsum(real)])
    dispatch_base = np.asarray(dispatch_base, dtype=np.int64)
    combine_base = np.asarray(combine_base, dtype=np.int64)
    for e in range(el_n):
        lo, hi = int(real_start[e]), int(real_start[e + 1])
        dst = slice(int(offsets[e]), int(offsets[e]) + hi - lo)
        s, t, k = s_idx[lo:hi], t_idx[lo:hi], k_idx[lo:hi]
        fwd[dst] = dispatch_base[s] + t * gather_stride
        bwd[dst] = dispatch_base[s] + (t * K + k) * bwd_stride
        sct[dst] = combine_base[s] + (t * K + k) * scatter_stride
        src[dst], tok[dst], slot[dst] = s, t, k
    return RoutingTables(stored.astype(np.int32), per_rank, offsets.astype(np.int32), fwd, bwd, sct, src, tok, slot)
