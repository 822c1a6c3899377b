"""Host-side byte arithmetic of the activation arena.

The arena is ``num_slots`` activation slots followed by shared scratch.  This
module sizes both for the worst case the configuration admits; the device-side
planner (``csrc/planner.cu``) then places tensors for the actual routed row
counts.  Every size is 128-byte aligned.  The formulas restate the reference's
``ModelConfig`` / ``BlockscaledStorageConfig`` (dist_moe/_activation_buffer.py:
957-1149, 1152-1189, 1192-1835) and must produce identical integers.
"""

from __future__ import annotations

import dataclasses

from .formats import DISPATCH_ROW_ALIGNMENT_BYTES, MEMORY_ALIGNMENT, ROW_SCALE_STORAGE_MULTIPLE


def align(nbytes: int) -> int:
    return (nbytes + MEMORY_ALIGNMENT - 1) // MEMORY_ALIGNMENT * MEMORY_ALIGNMENT


def ceil_div(a: int, b: int) -> int:
    return (a + b - 1) // b


def max_recv_rows(*, num_tokens: int, top_k: int, factor: float, num_local_experts: int, ep_size: int | None,
                  m_multiple_of: int | None) -> int:
    """Rows a rank may receive: imbalance-scaled, clamped by topology, padded per expert.

    dist_moe/_activation_buffer.py:1152-1189.
    """
    rows = int(num_tokens * top_k * factor + 0.5)
    if ep_size is not None:
        rows = min(rows, num_tokens * ep_size * min(top_k, num_local_experts))
    if m_multiple_of is not None:
        rows = (rows + num_local_experts * (m_multiple_of - 1)) // m_multiple_of * m_multiple_of
    return rows


@dataclasses.dataclass(frozen=True)
class QuantStorage:
    """Geometry of a block-scaled operand bundle (quantised data followed by its scales)."""

    operand_bytes: int
    values_per_element: int
    scale_bytes: int
    vec: int
    row_global_scale_bytes: int = 0

    def _q_cols(self, n: int) -> int:
        return ceil_div(n, self.values_per_element)

    def row_bundle(self, rows: int, dim: int) -> int:
        q = align(rows * self._q_cols(dim) * self.operand_bytes)
        s = align(rows * ROW_SCALE_STORAGE_MULTIPLE * ceil_div(dim, self.vec) * self.scale_bytes
                  + rows * self.row_global_scale_bytes)
        return q + s

    def col_bundle(self, rows: int, dim: int) -> int:
        q = align(dim * self._q_cols(rows) * self.operand_bytes)
        s = align(dim * ceil_div(rows, self.vec) * self.scale_bytes)
        return q + s

    def packed_row_stride(self, dim: int) -> int:
        raw = self._q_cols(dim) * self.operand_bytes + ceil_div(dim, self.vec) * self.scale_bytes + self.row_global_scale_bytes
        return ceil_div(raw, DISPATCH_ROW_ALIGNMENT_BYTES) * DISPATCH_ROW_ALIGNMENT_BYTES


@dataclasses.dataclass(frozen=True)
class ArenaSizing:
    """Worst-case sizes for one (config, ep_size)."""

    num_tokens: int
    hidden: int
    inter: int
    top_k: int
    factor: float
    num_layers: int
    num_local_experts: int
    ep_size: int | None
    storage: QuantStorage | None = None
    mega: bool = False
    es: int = 2  # bf16

    # ---- row capacity -----------------------------------------------------
    def rows_at(self, factor: float) -> int:
        return max_recv_rows(
            num_tokens=self.num_tokens, top_k=self.top_k, factor=factor, num_local_experts=self.num_local_experts,
            ep_size=self.ep_size, m_multiple_of=128 if self.storage is not None else None,
        )

    @property
    def capacity_rows(self) -> int:
        return self.rows_at(self.factor)

    # ---- dense pieces -----------------------------------------------------
    def _xg(self, r: int) -> int:
        return align(r * self.hidden * self.es)

    def _h1(self, r: int) -> int:
        return align(r * 2 * self.inter * self.es)

    def _h2(self, r: int) -> int:
        return align(r * self.inter * self.es)

    @property
    def x_bytes(self) -> int:
        return align(self.num_tokens * self.hidden * self.es)

    @property
    def h3_bytes(self) -> int:
        return align(self.num_tokens * self.top_k * self.hidden * self.es)

    # ---- saved state ------------------------------------------------------
    def saved_bytes(self, r: int, recompute: bool) -> int:
        if recompute:
            return self.x_bytes
        if self.storage is None:
            return self._xg(r) + self._h1(r) + self.h3_bytes
        s = self.storage
        return s.col_bundle(r, self.hidden) + self._h1(r) + s.col_bundle(r, self.inter) + self.h3_bytes

    # ---- scratch ----------------------------------------------------------
    def _fwd_row_scratch(self, r: int) -> int:
        s = self.storage
        x_row, h2_row = s.row_bundle(r, self.hidden), s.row_bundle(r, self.inter)
        return x_row + h2_row if self.mega else max(x_row, h2_row)

    def _bwd_row_scratch(self, r: int, recompute: bool) -> int:
        s = self.storage
        x_row, dxy_row = s.row_bundle(r, self.hidden), s.row_bundle(r, 2 * self.inter)
        if not recompute:
            return max(x_row, dxy_row)
        h2_row = s.row_bundle(r, self.inter)
        return max(x_row + h2_row, dxy_row) if self.mega else max(x_row, h2_row, dxy_row)

    def fwd_bytes(self, r: int, recompute: bool) -> int:
        if self.storage is None:
            if recompute:
                return self.x_bytes + self._xg(r) + self._h1(r) + self._h2(r)
            return self._xg(r) + self._h1(r) + self.h3_bytes + self._h2(r)
        s = self.storage
        if recompute:
            return (self.x_bytes + self._h1(r) + s.col_bundle(r, self.hidden) + s.col_bundle(r, self.inter)
                    + self._fwd_row_scratch(r))
        return self.saved_bytes(r, False) + self._fwd_row_scratch(r)

    def bwd_bytes(self, r: int, recompute: bool) -> int:
        if self.storage is None:
            grads = self._h1(r) + self._h2(r)
            if self.hidden > self.inter:
                grads += self._xg(r)
            return grads + (self._xg(r) + self._h1(r) if recompute else 0)
        s = self.storage
        live = (self._bwd_row_scratch(r, recompute) + s.col_bundle(r, self.hidden) + self._h2(r)
                + s.col_bundle(r, 2 * self.inter))
        if recompute:
            live += s.col_bundle(r, self.hidden) + self._h1(r) + s.col_bundle(r, self.inter)
        return live

    @property
    def training_scratch_bytes(self) -> int:
        return self.bwd_bytes(self.capacity_rows, True)

    @property
    def inference_scratch_bytes(self) -> int:
        r = self.capacity_rows
        if self.storage is not None:
            return self._fwd_row_scratch(r) + self._h1(r)
        return self.fwd_bytes(r, True) - self.x_bytes

    def host_scratch_bytes(self, total_factor: float) -> int:
        return max(0, self.bwd_bytes(self.rows_at(total_factor), True) - self.training_scratch_bytes)

    def host_inference_scratch_bytes(self, total_factor: float) -> int:
        other = dataclasses.replace(self, factor=total_factor)
        return max(0, align(other.inference_scratch_bytes) - align(self.inference_scratch_bytes))
