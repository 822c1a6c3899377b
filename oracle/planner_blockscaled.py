"""Activation-arena planner for the block-scaled paths, restated with Python integers.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Follows dist_moe/_activation_buffer_planner_kernel.py:293-647 (forward), 651-1065 (backward) and the size helpers at
82-289.  State is the BF16 planner's (``oracle.planner.PlannerState``).  Pinned by
``tests/golden/planner_blockscaled.json``, which records the reference kernels (run under the Triton CPU
interpreter) on the same scenarios.
"""

from __future__ import annotations

from dataclasses import dataclass

from .planner import PlannerState, align

MISSING = -1


@dataclass(frozen=True)
class Storage:
    """dist_moe/_activation_buffer.py:958-1075 ``BlockscaledStorageConfig``."""

    operand_element_size: int
    values_per_element: int
    scale_element_size: int
    row_scale_multiple: int
    row_global_scale_size: int
    sf_vec: int

    def as_list(self):
        return [self.operand_element_size, self.values_per_element, self.scale_element_size, self.row_scale_multiple,
                self.row_global_scale_size, self.sf_vec]


MXFP8 = Storage(1, 1, 1, 4, 0, 32)
NVFP4 = Storage(1, 2, 1, 4, 4, 16)


def _cdiv(a, b):
    return -(-a // b)


def row_sizes(rows, dim, s: Storage):
    q = align(rows * _cdiv(dim, s.values_per_element) * s.operand_element_size)
    sc = align(rows * s.row_scale_multiple * _cdiv(dim, s.sf_vec) * s.scale_element_size
               + rows * s.row_global_scale_size)
    return q, sc


def col_sizes(rows, dim, s: Storage):
    q = align(dim * _cdiv(rows, s.values_per_element) * s.operand_element_size)
    sc = align(dim * _cdiv(rows, s.sf_vec) * s.scale_element_size)
    return q, sc


def packed_dispatch_size(rows, dim, s: Storage):
    row = _cdiv(dim, s.values_per_element) * s.operand_element_size + _cdiv(dim, s.sf_vec) * s.scale_element_size \
        + s.row_global_scale_size
    return align(rows * _cdiv(row, 16) * 16)


def _saved_cost(rr, h3_mem, D, F, s, native):
    sizes = row_sizes if native else col_sizes
    return sum(sizes(rr, D, s)) + align(rr * 2 * F * 2) + sum(sizes(rr, F, s)) + h3_mem


def _group(a_q=MISSING, b_q=MISSING, c=MISSING, a_scale=MISSING, b_scale=MISSING, source_x=MISSING, source_y=MISSING,
           col_q=MISSING, col_scale=MISSING):
    return [a_q, b_q, c, a_scale, b_scale, source_x, source_y, col_q, col_scale]


def plan_forward(st: PlannerState, rows, per_rank, selector, *, T, K, D, F, storage: Storage, num_layers,
                 mega=False, inference=False, scratch_only=False, native=False, interleaved=False):
    """Returns dict(need, offsets[10], table[18]); updates ``st`` in place."""
    s, N, es = storage, st.n, 2
    h1 = align(rows * 2 * F * es)
    xr_q, xr_s = row_sizes(rows, D, s)
    hr_q, hr_s = row_sizes(rows, F, s)
    xc_q, xc_s = col_sizes(rows, D, s)
    hc_q, hc_s = col_sizes(rows, F, s)
    xr, hr = xr_q + xr_s, hr_q + hr_s
    end = st.buffer_offsets[N]
    x_row = end - xr
    if mega:
        h2_row, row_slot = x_row - hr, xr + hr
    else:
        h2_row, row_slot = end - hr, max(xr, hr)
    slot_off = end - row_slot
    x_off = h1_off = h3_off = x_col = h2_col = staging = 0
    base = 0 if inference else N * st.slot_bytes
    need = True
    if inference or scratch_only:
        if interleaved:
            staging = slot_off - (align(rows * F * es) if s.row_global_scale_size > 0 else 0)
            bottom = staging
        else:
            h1_off = slot_off - h1
            bottom = h1_off
    else:
        m = selector % N
        free = st.buffer_offsets[m]
        x_mem = packed_dispatch_size(T, D, s) if native else align(T * D * es)
        h3_mem = align(T * K * D * es)
        layer = st.layer[m]
        cost = [_saved_cost(per_rank[r], h3_mem, D, F, s, native) for r in range(st.ep)]
        worst = max(st.saved[m * st.ep + r] + cost[r] for r in range(st.ep))
        need = worst + (num_layers - 1 - layer) * x_mem > st.slot_bytes
        if need and native:
            x_off, new_free = free, free + x_mem
            h1_off = slot_off - h1
            bottom = h1_off
        elif need:
            x_off, new_free = free, free + x_mem
            x_col = slot_off - xc_q - xc_s
            h1_off = x_col - h1
            h2_col = h1_off - hc_q - hc_s
            bottom = h2_col
        elif native:
            x_row = free
            h1_off = x_row + xr
            h2_row = h1_off + h1
            h3_off = h2_row + hr
            new_free, bottom = h3_off + h3_mem, end
        else:
            x_col = free
            h1_off = x_col + xc_q + xc_s
            h2_col = h1_off + h1
            h3_off = h2_col + hc_q + hc_s
            new_free, bottom = h3_off + h3_mem, slot_off
        st.peak[m] = min(st.peak[m], (m + 1) * st.slot_bytes - new_free)
        st.buffer_offsets[m] = new_free
        st.layer[m] = layer + 1
        for r in range(st.ep):
            st.saved[m * st.ep + r] += x_mem if need else cost[r]
    st.peak[N] = min(st.peak[N], bottom - base)
    if native:
        x_col, h2_col = x_row, h2_row
    offsets = [x_off, 0, h1_off, 0, h3_off, x_row, x_col, h2_row, h2_col, selector]
    if native:
        d_col, c_col = (x_row, x_row + xr_q), (h2_row, h2_row + hr_q)
    else:
        d_col, c_col = (x_col, x_col + xc_q), (h2_col, h2_col + hc_q)
    disp_c, sx, sy = h1_off, h1_off, h1_off + F * es
    if interleaved:
        disp_c = MISSING
        sx = sy = staging if s.row_global_scale_size > 0 else MISSING
    table = _group(a_q=x_row, c=disp_c, a_scale=x_row + xr_q, col_q=d_col[0], col_scale=d_col[1]) \
        + _group(a_q=h2_row, a_scale=h2_row + hr_q, source_x=sx, source_y=sy, col_q=c_col[0], col_scale=c_col[1])
    return dict(need=need, offsets=offsets, table=table)


def plan_backward(st: PlannerState, rows, per_rank, need, fwd_offsets, *, T, K, D, F, storage: Storage, mega=False,
                  native=False):
    """Returns dict(offsets[16], table[54]); updates ``st`` in place."""
    s, N, es = storage, st.n, 2
    m = fwd_offsets[9] % N
    end, free = st.buffer_offsets[N], st.buffer_offsets[m]
    fwd_x, fwd_h1, fwd_x_row, fwd_x_col, fwd_h2_row, fwd_h2_col = (fwd_offsets[i] for i in (0, 2, 5, 6, 7, 8))
    xr_q, xr_s = row_sizes(rows, D, s)
    hr_q, hr_s = row_sizes(rows, F, s)
    dr_q, dr_s = row_sizes(rows, 2 * F, s)
    xr, hr, dr = xr_q + xr_s, hr_q + hr_s, dr_q + dr_s
    x_row = end - xr
    if mega or native:
        re_h2_row, re_slot = x_row - hr, max(xr + hr, dr)
    else:
        re_h2_row, re_slot = end - hr, max(xr, hr, dr)
    dxy_row = end - dr
    h2_row = re_h2_row if need else dxy_row
    slot_off = end - (re_slot if need else max(xr, dr))
    g3_row = x_row
    xc_q, xc_s = col_sizes(rows, D, s)
    hc_q, hc_s = col_sizes(rows, F, s)
    dc_q, dc_s = col_sizes(rows, 2 * F, s)
    h1, g2, xg = align(rows * 2 * F * es), align(rows * F * es), align(rows * D * es)
    xg_off = h2_off = g3g_off = g1_off = 0
    cursor = slot_off
    if native:
        if need:
            h1_off = cursor - h1
            cursor = h1_off
            h2_row = re_h2_row
        else:
            h1_off, x_row, h2_row, cursor = fwd_h1, fwd_x_row, fwd_h2_row, end
        xg_off = cursor - xg
        h2_off = xg_off - g2
        g3g_off = h2_off - xg
        g2_off = g3g_off - g2
        g1_off = g2_off - h1
        x_col, h2_col, g3_col, dxy_col = x_row, h2_row, g3_row, dxy_row
        bottom = g1_off
    else:
        if need:
            x_col = cursor - xc_q - xc_s
            h1_off = x_col - h1
            h2_col = h1_off - hc_q - hc_s
            cursor = h2_col
        else:
            x_col, h1_off, h2_col = fwd_x_col, fwd_h1, fwd_h2_col
        g3_col = cursor - xc_q - xc_s
        g2_off = g3_col - g2
        dxy_col = g2_off - dc_q - dc_s
        bottom = dxy_col
    st.peak[N] = min(st.peak[N], bottom - N * st.slot_bytes)
    st.peak[m] = min(st.peak[m], (m + 1) * st.slot_bytes - free)
    offsets = [xg_off, h1_off, h2_off, g2_off, g3g_off, g1_off, x_row, x_col, h2_row, h2_col, g3_row, g3_col, dxy_row,
               dxy_col,
               x_row + xr_q + rows * s.row_scale_multiple * _cdiv(D, s.sf_vec) * s.scale_element_size,
               h2_row + hr_q + rows * s.row_scale_multiple * _cdiv(F, s.sf_vec) * s.scale_element_size]
    if native:
        xcs, hcs, g3cs, dcs = x_row + xr_q, h2_row + hr_q, g3_row + xr_q, dxy_row + dr_q
    else:
        xcs, hcs, g3cs, dcs = x_col + xc_q, h2_col + hc_q, g3_col + xc_q, dxy_col + dc_q
    table = (
        _group(a_q=x_row, c=h1_off, a_scale=x_row + xr_q, col_q=x_col, col_scale=xcs)
        + _group(a_q=h2_row, a_scale=h2_row + hr_q, source_x=h1_off, source_y=h1_off + F * es, col_q=h2_col,
                 col_scale=hcs)
        + _group(a_q=g3_row, c=g2_off, a_scale=g3_row + xr_q, col_q=g3_col, col_scale=g3cs)
        + _group(a_q=g3_col, b_q=h2_col, a_scale=g3cs, b_scale=hcs)
        + _group(a_q=dxy_row, a_scale=dxy_row + dr_q, source_x=g2_off, source_y=h1_off, col_q=dxy_col, col_scale=dcs)
        + _group(a_q=dxy_col, b_q=x_col, a_scale=dcs, b_scale=xcs))
    st.buffer_offsets[m] = fwd_x if need else (fwd_x_row if native else x_col)
    x_mem = packed_dispatch_size(T, D, s) if native else align(T * D * es)
    h3_mem = align(T * K * D * es)
    for r in range(st.ep):
        st.saved[m * st.ep + r] -= x_mem if need else _saved_cost(per_rank[r], h3_mem, D, F, s, native)
    st.layer[m] -= 1
    return dict(offsets=offsets, table=table)
