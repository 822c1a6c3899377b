"""Device-resident state of a context: symmetric buffers, arena, planner state.

Layout in HBM (per rank):
* routing buffer   int16[64 + Tmax*K]   128-byte header (int32 T) + published expert ids
* dispatch buffer  bf16[Tmax, K, D]     forward: first T*D elements hold x; backward: per-route input grads
* combine buffer   bf16[Tmax, K, D]     forward: per-route expert outputs; backward: per-route output grads
  (dist_moe/_buffers.py:574-629 allocates the same three symmetric buffers)
* arena            uint8[total_device_buffer_bytes + guard]  activation slots then shared scratch
* planner state    int64 vectors updated in place by the planner kernels
  (dist_moe/_activation_buffer.py:242-307)
Peers are reached through raw addresses obtained from torch's symmetric-memory
rendezvous; all traffic is issued by this library's own kernels.
"""

from __future__ import annotations

import dataclasses
import os
from typing import Any

import torch

from . import _native as nat
from .formats import BlockScaledFormat, format_constants


@dataclasses.dataclass
class ScratchInfo:
    """Peak use of the shared scratch region and of every activation slot since the last ``reset``
    (dist_moe/_activation_buffer.py:179-207 ``ScratchInfo``; the per-slot list is this library's addition)."""

    scratch_min_free: float      # smallest free byte count seen; negative = overflow by that many bytes
    scratch_size: float
    scratch_max_used: float
    device_scratch_size: float
    device_scratch_used: float
    host_scratch_size: float | None
    host_scratch_used: float | None
    slot_max_used: list


@dataclasses.dataclass
class PendingOverflowCheck:
    """A device-to-host copy of the planner's peak counters in flight (dist_moe/_activation_buffer.py:210-221)."""

    host_peaks: torch.Tensor
    ready: Any


ROUTING_HEADER_BYTES = 128
GUARD_ROWS = 256
BARRIER_TIMEOUT_NS = 5_000_000_000


class SymmetricBuffer:
    """One buffer that every rank of the group can address."""

    def __init__(self, nbytes: int, device: torch.device, group: Any, ep_size: int, rank: int):
        self.nbytes = nbytes
        self.ep_size = ep_size
        self.rank = rank
        n = (nbytes + 15) // 16 * 16
        if ep_size == 1:
            self.tensor = torch.zeros(n, dtype=torch.uint8, device=device)
            self.pad = torch.zeros(512, dtype=torch.uint8, device=device)
            ptrs, pads = [self.tensor.data_ptr()], [self.pad.data_ptr()]
            self._handle = None
        else:
            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
            import torch.distributed._symmetric_memory as symm_mem

            self.tensor = symm_mem.empty(n, dtype=torch.uint8, device=device)
            self.tensor.zero_()
            self._handle = symm_mem.rendezvous(self.tensor, group)
            ptrs, pads = list(self._handle.buffer_ptrs), list(self._handle.signal_pad_ptrs)
            if self._handle.signal_pad_size < 4 * ep_size:
                raise RuntimeError("symmetric-memory signal pad is too small for the expert-parallel barrier")
        self.peer_ptrs = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.peer_pads = torch.tensor(pads, dtype=torch.int64, device=device)
        self.peer_ptrs_host = ptrs

    def local(self) -> torch.Tensor:
        return self.tensor


class ContextState:
    def __init__(self, *, group: Any, ep_size: int, config, plan, device: torch.device):
        import torch.distributed as dist

        self.group = group
        self.ep = ep_size
        self.rank = dist.get_rank(group) if (group is not None and ep_size > 1) else 0
        self.config = config
        self.plan = plan
        self.device = device
        self.e_local = config.num_experts // ep_size
        T, K, D, F = config.max_num_local_input_tokens, config.top_k, config.hidden_dim, config.intermediate_dim
        self.block_scaled = config.block_scaled is not None
        self.m_multiple = 128 if self.block_scaled else 0
        self.capacity_rows = plan.total_scratch_capacity_rows
        # static inference operands reserve scratch without going through the planner (dist_moe/api.py:1686-1693)
        self.reserved_scratch_bytes = plan.inference_operand_bytes or 0
        with torch.cuda.device(device):
            self.routing = SymmetricBuffer(ROUTING_HEADER_BYTES + T * K * 2, device, group, ep_size, self.rank)
            self.dispatch = SymmetricBuffer(T * K * D * 2, device, group, ep_size, self.rank)
            self.combine = SymmetricBuffer(T * K * D * 2, device, group, ep_size, self.rank)
            guard = GUARD_ROWS * max(D, 2 * F) * 2
            self.vmm_arena = None
            if plan.vmm_granularity_bytes is not None:
                # [device: slots | host: overflow scratch | device: hot scratch] in one virtual range
                from ._vmm import VmmArena

                self.vmm_arena = VmmArena(plan, device, guard)
                self.arena_bytes = plan.total_virtual_bytes
                self.arena = self.vmm_arena.tensor
                self.hot_scratch_bytes = plan.vmm_device_scratch_section_bytes
                self.host_scratch_bytes = plan.vmm_host_section_bytes
            else:
                self.arena_bytes = plan.total_device_buffer_bytes
                self.arena = torch.zeros(self.arena_bytes + guard, dtype=torch.uint8, device=device)
                self.hot_scratch_bytes = self.host_scratch_bytes = None
            n = plan.num_activation_slots
            self.num_slots = n
            self.slot_bytes = plan.activation_slot_bytes
            self.buffer_offsets = torch.zeros(n + 1, dtype=torch.int64, device=device)
            self.saved_bytes = torch.zeros(max(1, n * ep_size), dtype=torch.int64, device=device)
            self.peak_min_free = torch.zeros(n + 1, dtype=torch.int64, device=device)
            self.moe_layer_id = torch.zeros(max(1, n), dtype=torch.int64, device=device)
            self.slot_selector = torch.zeros(1, dtype=torch.int64, device=device)
            self.status = torch.zeros(8, dtype=torch.int32, device=device)
            self.num_layers_in_slot = config.max_moe_layers_per_activation_slot
            words = nat.lib.dm_route_workspace_words(T, ep_size, config.num_experts)
            self.route_workspace = torch.zeros(max(1, words), dtype=torch.int32, device=device)
            self.route_workspace_words = words
            self.gather_flags = torch.zeros(self.capacity_rows // 128 + 8 + ep_size * self.e_local * T // 128,
                                            dtype=torch.int32, device=device)
            self.reset()
        if config.block_scaled is not None:
            ob, vpe, sb, vec, gs = format_constants(config.block_scaled.format)
            self.format = config.block_scaled.format
        else:
            self.format = None
        self.num_sms = config.num_sms or 0

    # ---- planner state -------------------------------------------------------
    def reset(self) -> None:
        n = self.num_slots
        offs = [i * self.slot_bytes for i in range(n)] + [self.arena_bytes]
        self.buffer_offsets.copy_(torch.tensor(offs, dtype=torch.int64))
        self.saved_bytes.zero_()
        peak = [self.slot_bytes] * n + [self.arena_bytes - n * self.slot_bytes - self.reserved_scratch_bytes]
        self.peak_min_free.copy_(torch.tensor(peak, dtype=torch.int64))
        self.moe_layer_id.zero_()

    def select_slot(self, slot: int, num_layers: int) -> None:
        if self.num_slots == 0:
            return
        if not 0 <= slot < self.num_slots:
            raise ValueError(f"activation_slot must be in [0, {self.num_slots})")
        if not 1 <= num_layers <= self.config.max_moe_layers_per_activation_slot:
            raise ValueError(
                "num_moe_layers_in_slot must be in [1, max_moe_layers_per_activation_slot="
                f"{self.config.max_moe_layers_per_activation_slot}]")
        self.slot_selector.fill_(slot)
        self.num_layers_in_slot = num_layers

    def last_recv_rows(self) -> int:
        """Rows this rank received in the most recent call (reads the device; not for hot paths)."""
        call = getattr(self, "last_call", None)
        return int(call.recv_rows.item()) if call is not None else 0

    # ---- status --------------------------------------------------------------
    def check_status(self) -> None:
        torch.cuda.synchronize(self.device)
        words = self.status.tolist()
        if words[0] != 0:
            self.status.zero_()
            raise RuntimeError(
                f"dist_moe_b200 device contract violation: {nat.STATUS_NAMES.get(words[0], words[0])} "
                f"(details {words[1:4]})")

    # ---- peak-usage metrics (dist_moe/_activation_buffer.py:690-800) --------------------
    def _scratch_info(self, peaks: list) -> ScratchInfo:
        n = self.num_slots
        scratch_size = float(self.arena_bytes - n * self.slot_bytes)
        min_free = float(peaks[n])
        slots = [float(self.slot_bytes - peaks[i]) for i in range(n)]
        overflow = min_free < 0 or any(peaks[i] < 0 for i in range(n))
        used = scratch_size - min_free
        if self.hot_scratch_bytes is not None:
            # scratch fills from the top: hot device section, then the host section, then the device bytes below it
            hot, host = float(self.hot_scratch_bytes), float(self.host_scratch_bytes)
            lower = max(0.0, scratch_size - hot - host)
            device_size = hot + lower
            device_used = min(used, hot) + max(0.0, used - hot - host)
            host_size, host_used = host, min(max(0.0, used - hot), host)
        else:
            device_size, device_used, host_size, host_used = scratch_size, used, None, None
        info = ScratchInfo(scratch_min_free=min_free, scratch_size=scratch_size, scratch_max_used=used,
                           device_scratch_size=device_size, device_scratch_used=device_used,
                           host_scratch_size=host_size, host_scratch_used=host_used, slot_max_used=slots)
        if overflow:
            raise RuntimeError(f"dist_moe_b200 activation buffer overflow: {info}")
        return info

    def check_overflow(self) -> ScratchInfo:
        """Blocking read of the planner's peak counters; raises if a slot or the scratch region overflowed."""
        return self._scratch_info(self.peak_min_free.tolist())

    def begin_check_overflow(self) -> PendingOverflowCheck:
        """Start the device-to-host copy of the counters on the current stream without draining the GPU."""
        staging = getattr(self, "_overflow_staging", None)
        if staging is None:
            staging = torch.empty_like(self.peak_min_free, device="cpu", pin_memory=True)
            self._overflow_staging = staging
        with torch.cuda.device(self.device):
            staging.copy_(self.peak_min_free, non_blocking=True)
            ready = torch.cuda.Event()
            ready.record()
        return PendingOverflowCheck(host_peaks=staging, ready=ready)

    def finish_check_overflow(self, pending: PendingOverflowCheck) -> ScratchInfo:
        pending.ready.synchronize()
        return self._scratch_info(pending.host_peaks.tolist())

    def close(self) -> None:
        torch.cuda.synchronize(self.device)
        self._bs_workspace = None  # a view of the arena's scratch region (block-scaled forward-only calls)
        if getattr(self, "vmm_arena", None) is not None:
            self.arena = None
            self.vmm_arena.close()
            self.vmm_arena = None
        self.arena = torch.empty(0, dtype=torch.uint8, device=self.device)

    # ---- barrier -------------------------------------------------------------
    def barrier(self, buf: SymmetricBuffer, cond: torch.Tensor | None = None) -> None:
        if self.ep == 1:
            return
        nat.check(nat.lib.dm_barrier(buf.peer_pads.data_ptr(), self.rank, self.ep, 0, nat.ptr(cond),
                                     BARRIER_TIMEOUT_NS, self.status.data_ptr(), nat.stream_ptr()), "dm_barrier")

    def arena_operand(self, offset_tensor: torch.Tensor | None) -> nat.Operand:
        return nat.Operand(self.arena.data_ptr(), self.arena.numel(),
                           None if offset_tensor is None else offset_tensor.data_ptr())
