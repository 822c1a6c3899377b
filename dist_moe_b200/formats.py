"""Block-scaled operand formats and shared numeric constants.

Mirrors the public vocabulary of the reference (dist_moe/formats.py:108-109,
133-175, 316-415; dist_moe/_execution.py ``BlockScaledFormat``): MXFP8 E4M3 with
E8M0 scales over 32 elements, NVFP4 (E2M1) with E4M3 scales over 16 elements and
an fp32 global scale.
"""

from __future__ import annotations

import enum

SWIGLU_CLAMP_ALPHA_DEFAULT = 1.702
SWIGLU_CLAMP_LIMIT_DEFAULT = 7.0

NVFP4_DIM_MULTIPLE = 256
NVFP4_HIDDEN_DIM_MAX = 16384
NVFP4_INTERMEDIATE_DIM_MAX = 8192

MEMORY_ALIGNMENT = 128
ROUTING_M_MULTIPLE = 128  # per-expert row padding of the block-scaled paths
ROW_SCALE_STORAGE_MULTIPLE = 4  # row-scale columns are stored in multiples of 4 (one blocked atom)
DISPATCH_ROW_ALIGNMENT_BYTES = 16  # packed inference dispatch rows


class BlockScaledFormat(enum.StrEnum):
    """Operand precision of a block-scaled context."""

    MXFP8_E4M3 = enum.auto()
    NVFP4 = enum.auto()


def format_constants(fmt: BlockScaledFormat) -> tuple[int, int, int, int, int]:
    """Return (operand element bytes, values per storage element, scale bytes, scale vector, row global scale bytes)."""
    if fmt is BlockScaledFormat.MXFP8_E4M3:
        return 1, 1, 1, 32, 0
    if fmt is BlockScaledFormat.NVFP4:
        return 1, 2, 1, 16, 4
    raise ValueError(f"unsupported block-scaled format {fmt}")
