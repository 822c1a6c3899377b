"""Host-backed overflow scratch: the arena of a context with ``Config.vmm`` is one virtual range laid out as
``[device: activation slots | host: overflow scratch | device: hot scratch]`` (dist_moe/_vmm.py:149-427,
dist_moe/api.py:1052-1143).  The device planner carves scratch from the top of the range downwards, so only a step
whose routing overflows the hot section reaches host memory.

The range is created by the C ABI (``dm_vmm_create``: driver virtual-memory calls); this module sizes the sections
and wraps the range in a tensor that does not own it.
"""

from __future__ import annotations

import ctypes
import dataclasses

import torch

from . import _native as nat

# torch's caching allocator hands out a 20 MiB block for large-pool requests below 10 MiB; the reference allocates
# its range through a torch memory pool and therefore plans with that rounding (dist_moe/api.py:1084-1094).  The
# numbers are kept so that plans agree, although this library maps the range itself.
LARGE_POOL_BUFFER_BYTES = 20 * 1024 * 1024
LARGE_POOL_MIN_ALLOC_BYTES = 10 * 1024 * 1024


def _align_to(value: int, granularity: int) -> int:
    return (value + granularity - 1) // granularity * granularity


def granularity(device: torch.device) -> int:
    out = ctypes.c_int64(0)
    with torch.cuda.device(device):
        torch.cuda.current_stream()  # a current context for the driver call
        nat.check(nat.lib.dm_vmm_granularity(device.index, ctypes.byref(out)), "dm_vmm_granularity")
    return int(out.value)


def resolve_physical_plan(plan, granularity_bytes: int):
    """Section sizes at the driver's granularity (dist_moe/api.py:1052-1109): activations keep their logical size,
    the padding at the end of the first device mapping becomes lower device scratch, allocator rounding goes to the
    hot device scratch."""
    g = granularity_bytes
    device_prefix = _align_to(plan.total_activation_bytes, g) if plan.total_activation_bytes else 0
    host_section = _align_to(plan.host_scratch_bytes, g)
    device_scratch_section = _align_to(plan.device_scratch_bytes, g)
    section_total = device_prefix + host_section + device_scratch_section
    allocator_total = LARGE_POOL_BUFFER_BYTES if section_total < LARGE_POOL_MIN_ALLOC_BYTES else section_total
    device_scratch_section += allocator_total - section_total
    return dataclasses.replace(
        plan,
        total_virtual_bytes=allocator_total,
        vmm_granularity_bytes=g,
        vmm_device_prefix_bytes=device_prefix,
        vmm_host_section_bytes=host_section,
        vmm_device_scratch_section_bytes=device_scratch_section,
        vmm_padding_bytes=allocator_total - plan.total_activation_bytes - plan.host_scratch_bytes
        - plan.device_scratch_bytes,
    )


class _Span:
    """Describes foreign device memory to ``torch.as_tensor``."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 3}


class VmmArena:
    """The mapped range and a ``uint8`` tensor over it.  ``guard_bytes`` extends the hot device section: edge tiles
    of the GEMMs read a few rows past an operand that ends at the top of the range."""

    def __init__(self, plan, device: torch.device, guard_bytes: int):
        g = plan.vmm_granularity_bytes
        sections = [(plan.vmm_device_prefix_bytes, 0), (plan.vmm_host_section_bytes, 1),
                    (plan.vmm_device_scratch_section_bytes + _align_to(guard_bytes, g), 0)]
        sections = [(size, host) for size, host in sections if size > 0]
        sizes = (ctypes.c_int64 * len(sections))(*[s for s, _ in sections])
        hosts = (ctypes.c_int * len(sections))(*[h for _, h in sections])
        base, handle = ctypes.c_uint64(0), ctypes.c_void_p(None)
        with torch.cuda.device(device):
            torch.cuda.current_stream()
            nat.check(nat.lib.dm_vmm_create(device.index, len(sections), sizes, hosts, ctypes.byref(base),
                                            ctypes.byref(handle)), "dm_vmm_create")
        self.device = device
        self.handle = handle
        self.base = int(base.value)
        self.nbytes = sum(s for s, _ in sections)
        self.host_bytes = sum(s for s, h in sections if h)
        with torch.cuda.device(device):
            self.tensor = torch.as_tensor(_Span(self.base, self.nbytes), device=device)
            self.tensor.zero_()

    def close(self) -> None:
        if self.handle is None:
            return
        torch.cuda.synchronize(self.device)
        self.tensor = None
        with torch.cuda.device(self.device):
            nat.check(nat.lib.dm_vmm_destroy(self.handle), "dm_vmm_destroy")
        self.handle = None
