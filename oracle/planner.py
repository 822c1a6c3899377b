"""Activation-arena planner (BF16), restated with Python integers.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows dist_moe/_activation_buffer_planner_kernel.py:1068-1275 (forward) and 1278-1477
(backward).  State: ``buffer_offsets[N+1]`` (slot bump pointers, entry N = scratch end),
``saved[N*EP]``, ``peak[N+1]``, ``layer[N]``.  Pinned by ``tests/golden/planner_bf16.json``,
which records the reference kernels (run under the Triton CPU interpreter) on the same
scenarios.
"""

from __future__ import annotations


def align(v: int) -> int:
    return (v + 127) // 128 * 128


class PlannerState:
    def __init__(self, num_slots: int, ep: int, slot_bytes: int, arena_bytes: int):
        self.n, self.ep, self.slot_bytes = num_slots, ep, slot_bytes
        self.buffer_offsets = [i * slot_bytes for i in range(num_slots)] + [arena_bytes]
        self.saved = [0] * (num_slots * ep)
        self.peak = [slot_bytes] * num_slots + [arena_bytes - num_slots * slot_bytes]
        self.layer = [0] * num_slots

    def snapshot(self):
        return dict(buffer_offsets=list(self.buffer_offsets), saved=list(self.saved), peak=list(self.peak),
                    layer=list(self.layer))


def _full(rr, D, F, h3_mem):
    return align(rr * D * 2) + align(rr * 2 * F * 2) + h3_mem


def plan_forward(st: PlannerState, R, per_rank, selector, *, T, K, D, F, num_layers, scratch_only):
    es, N = 2, st.n
    xg, h1, h2 = align(R * D * es), align(R * 2 * F * es), align(R * F * es)
    end = st.buffer_offsets[N]
    s_h2 = end - h2
    s_h1 = s_h2 - h1
    s_xg = s_h1 - xg
    x_mem, h3_mem = align(T * D * es), align(T * K * D * es)
    need, x_off, xg_off, h1_off, h2_off, h3_off = True, 0, s_xg, s_h1, s_h2, 0
    if not scratch_only:
        m = selector % N
        free = st.buffer_offsets[m]
        slot_end = (m + 1) * st.slot_bytes
        layer = st.layer[m]
        worst = max(st.saved[m * st.ep + r] + _full(per_rank[r], D, F, h3_mem) for r in range(st.ep))
        need = worst + (num_layers - 1 - layer) * x_mem > st.slot_bytes
        if need:
            x_off, new_free = free, free + x_mem
        else:
            xg_off, h1_off = free, free + xg
            h3_off = h1_off + h1
            new_free, x_off = h3_off + h3_mem, 0
    bottom = xg_off if need else h2_off
    st.peak[N] = min(st.peak[N], bottom - N * st.slot_bytes)
    if not scratch_only:
        st.peak[m] = min(st.peak[m], slot_end - new_free)
        st.buffer_offsets[m] = new_free
        st.layer[m] = layer + 1
        for r in range(st.ep):
            st.saved[m * st.ep + r] += x_mem if need else _full(per_rank[r], D, F, h3_mem)
    return dict(need=bool(need), fwd_state=[x_off, xg_off, h1_off, h2_off, h3_off, selector])


def plan_backward(st: PlannerState, R, per_rank, need, fwd_state, *, T, K, D, F):
    es, N = 2, st.n
    m = fwd_state[5] % N
    free, slot_end, end = st.buffer_offsets[m], (m + 1) * st.slot_bytes, st.buffer_offsets[N]
    xg, h1, h2 = align(R * D * es), align(R * 2 * F * es), align(R * F * es)
    g_h1 = end - h1
    g_h2 = g_h1 - h2
    h2_off = end - h2
    g_h3g = (h2_off - xg) if D * es <= F * es else (g_h2 - xg)
    grad_bottom = min(g_h2, g_h3g)
    if need:
        h1_off = grad_bottom - h1
        xg_off = h1_off - xg
        bottom = xg_off
    else:
        xg_off, h1_off, bottom = fwd_state[1], fwd_state[2], grad_bottom
    st.peak[m] = min(st.peak[m], slot_end - free)
    st.peak[N] = min(st.peak[N], bottom - N * st.slot_bytes)
    st.buffer_offsets[m] = fwd_state[0] if need else fwd_state[1]
    x_mem, h3_mem = align(T * D * es), align(T * K * D * es)
    for r in range(st.ep):
        st.saved[m * st.ep + r] -= x_mem if need else _full(per_rank[r], D, F, h3_mem)
    st.layer[m] -= 1
    return [xg_off, h1_off, h2_off, g_h2, g_h3g, g_h1]
