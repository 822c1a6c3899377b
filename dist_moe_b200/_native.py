"""ctypes binding of the C-ABI library (``include/dist_moe_b200.h``).

The CUDA library is the only compute path.  If it cannot be loaded the import
of this module raises: there is no CPU or eager fallback behind it.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, c_float, c_int, c_int32, c_int64, c_uint64, c_void_p
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "_lib" / "libdist_moe_b200.so"

RC_NAMES = {0: "ok", -1: "bad argument", -2: "unsupported shape", -3: "too large", -4: "CUDA driver entry point unavailable"}
STATUS_NAMES = {
    0: "ok",
    1: "expert-parallel ranks published different token counts",
    2: "DistMoE scratch capacity exceeded",
    3: "expert id outside [-1, num_experts)",
    4: "barrier timed out waiting for a peer",
    5: "GEMM pipeline wait timed out",
    6: "activation arena overflow",
}


class Operand(ctypes.Structure):
    """``dm_operand``: (allocation base, allocation bytes, device offset pointer)."""

    _fields_ = [("base", c_void_p), ("bytes", c_int64), ("offset", c_void_p)]


class NativeError(RuntimeError):
    pass


def _load() -> ctypes.CDLL:
    override = os.environ.get("DIST_MOE_B200_LIB")
    if override:  # an alternative build of the same library (A/B timing of kernel variants)
        return ctypes.CDLL(override)
    # build() compares a digest of the sources with the one the library was built from and returns at once when they
    # agree, so a library left over from older sources is never loaded silently.
    from .build import build, find_nvcc

    try:
        find_nvcc()
        have_nvcc = True
    except RuntimeError:
        have_nvcc = False
    if have_nvcc or not _LIB_PATH.exists():
        build()
    if not _LIB_PATH.exists():
        raise ImportError(f"dist_moe_b200: CUDA library missing at {_LIB_PATH}; run python -m dist_moe_b200.build")
    return ctypes.CDLL(str(_LIB_PATH))


lib = _load()

_P = c_void_p
_SIGNATURES = {
    "dm_version": (c_int, []),
    "dm_publish": (c_int, [_P, _P, c_int, _P, _P, c_int64, c_int64, c_int, c_int, c_int, _P, _P]),
    "dm_barrier": (c_int, [_P, c_int, c_int, c_int, _P, c_uint64, _P, _P]),
    "dm_route_workspace_words": (c_int64, [c_int64, c_int, c_int]),
    "dm_route": (
        c_int,
        [_P, _P, _P, c_int, c_int, c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int64, c_int64]
        + [_P] * 7
        + [c_int64, _P, _P],
    ),
    "dm_route_counted": (
        c_int,
        [_P, _P, _P, c_int, c_int, c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int64, c_int64]
        + [_P] * 8
        + [c_int64, _P, _P],
    ),
    "dm_route_static": (
        c_int,
        [_P, _P, _P, c_int, c_int, c_int64, c_int, c_int, c_int64, c_int64, c_int64, c_int, c_int64, c_int64]
        + [_P] * 6
        + [_P, _P],
    ),
    "dm_plan_fwd_bf16": (
        c_int,
        [_P] * 10 + [c_int, c_int64, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_int, _P, _P],
    ),
    "dm_plan_bwd_bf16": (c_int, [_P] * 9 + [c_int, c_int64, c_int, c_int64, c_int64, c_int64, c_int, _P, _P]),
    "dm_plan_fwd_blockscaled": (
        c_int,
        [_P] * 12 + [c_int, c_int64, c_int, c_int64, c_int64, _P, c_int64, c_int64, c_int, c_int, c_int, c_int, c_int,
                     c_int, c_int, _P, _P],
    ),
    "dm_plan_bwd_blockscaled": (
        c_int,
        [_P] * 10 + [c_int, c_int64, c_int, c_int64, c_int64, _P, c_int64, c_int64, c_int, c_int, c_int, _P, _P],
    ),
    "dm_gather_rows": (c_int, [_P, _P, _P, _P, c_int64, c_int64, _P, _P]),
    "dm_cond_copy": (c_int, [_P, _P, _P, _P, c_int64, _P, c_int, _P]),
    "dm_swiglu_fwd": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_float, c_float, _P, c_float, _P, _P]),
    "dm_swiglu_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int64, c_int, c_float, c_float, _P]),
    "dm_scale_and_sum": (c_int, [_P, _P, c_int, _P, c_int, _P, c_int64, c_int, c_int64, _P, _P, _P, c_int, _P]),
    "dm_broadcast_and_scale": (c_int, [_P, _P, c_int, _P, c_int, _P, _P, _P, _P, c_int64, c_int, c_int64, _P]),
    "dm_broadcast_and_scale_select": (c_int, [_P, _P, c_int, _P, c_int, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int64, _P]),
    "dm_zero_padded_rows": (c_int, [_P, _P, c_int, c_int64, c_int, c_int64, _P]),
    "dm_gemm_blockscaled": (
        c_int,
        [c_int, Operand, Operand, _P, _P, Operand, Operand, _P, Operand, _P, _P, c_int, c_int64, c_int64, c_int64,
         c_int, c_int, c_float, c_float, _P, c_int, _P, _P],
    ),
    "dm_gemm_blockscaled_swapped": (
        c_int,
        [c_int, Operand, Operand, _P, _P, Operand, Operand, _P, Operand, _P, _P, _P, c_int, c_int64, c_int64, c_int64,
         c_int, c_int, c_float, c_float, _P, c_int, _P, _P],
    ),
    "dm_vmm_granularity": (c_int, [c_int, _P]),
    "dm_vmm_create": (c_int, [c_int, c_int, _P, _P, _P, _P]),
    "dm_vmm_destroy": (c_int, [_P]),
    "dm_set_route_decode_kernel": (c_int, [c_int]),
    "dm_route_decode_kernel_enabled": (c_int, []),
    "dm_gemm_blockscaled_swiglu_mxfp8": (
        c_int,
        [Operand, Operand, _P, _P, Operand, Operand, _P, c_int, c_int64, c_int64, c_int64, c_int, c_float, c_float, _P,
         c_int, _P, _P],
    ),
    "dm_gemm_blockscaled_dgrad": (
        c_int,
        [Operand, Operand, _P, _P, Operand, _P, _P, c_int, c_int64, c_int64, c_int64, _P, c_int, _P, _P],
    ),
    "dm_gemm_blockscaled_wgrad": (
        c_int,
        [Operand, Operand, Operand, Operand, _P, c_int, c_int, _P, c_int, c_int64, c_int64, c_int64, _P, c_int, _P, _P],
    ),
    "dm_gemm_blockscaled_wgrad_compact": (
        c_int,
        [Operand, Operand, Operand, Operand, _P, c_int, c_int, _P, c_int, c_int64, c_int64, c_int64, _P, c_int, _P, _P],
    ),
    "dm_quant_mxfp8_rowcol_gather_at": (c_int, [_P, _P, c_int64, c_int64, Operand, Operand, Operand, Operand, _P, _P]),
    "dm_swiglu_fwd_quant_mxfp8_rowcol_at": (
        c_int, [Operand, _P, c_int64, c_int64, c_int, c_float, c_float, Operand, Operand, Operand, Operand, _P, _P]),
    "dm_swiglu_bwd_quant_mxfp8_at": (
        c_int, [Operand, Operand, _P, c_int64, c_int64, c_int, c_float, c_float, Operand, Operand, Operand, Operand, _P]),
    "dm_rmsnorm_combine_fwd": (
        c_int,
        [_P, _P, c_int, _P, c_int, _P, c_float, c_float, c_int, c_int, _P, _P, c_int64, c_int, c_int64, _P, _P, _P, c_int,
         _P],
    ),
    "dm_rmsnorm_combine_bwd": (
        c_int,
        [_P, _P, c_int, _P, c_int, _P, _P, _P, c_float, c_int, c_int, _P, _P, c_int64, c_int, c_int64, _P],
    ),
    "dm_quant_mxfp8_row": (c_int, [_P, _P, c_int64, c_int64, _P, c_int64, _P, c_int64, c_int, _P]),
    "dm_quant_mxfp8_col": (c_int, [_P, _P, c_int64, c_int64, _P, _P, c_int, _P]),
    "dm_quant_mxfp8_rowcol": (c_int, [_P, _P, c_int64, c_int64, _P, _P, _P, _P, _P]),
    "dm_quant_mxfp8_rowcol_gather": (c_int, [_P, _P, c_int64, c_int64, _P, _P, _P, _P, _P]),
    "dm_swiglu_fwd_quant_mxfp8_rowcol": (c_int, [_P, _P, c_int64, c_int64, c_int, c_float, c_float, _P, _P, _P, _P, _P]),
    "dm_swiglu_bwd_quant_mxfp8": (c_int, [_P, _P, _P, c_int64, c_int64, c_int, c_float, c_float, _P, _P, _P, _P, _P]),
    "dm_quant_mxfp8_tile32": (c_int, [_P, c_int64, c_int64, c_int64, _P, _P, _P, c_int, _P]),
    "dm_quant_nvfp4_token": (c_int, [_P, _P, c_int64, c_int64, _P, c_int64, _P, c_int64, c_int, _P, c_int64, _P]),
    "dm_quant_nvfp4_token_live": (c_int, [_P, _P, _P, c_int64, c_int64, _P, c_int64, _P, c_int64, c_int, _P, c_int64, _P]),
    "dm_gather_packed_rows": (c_int, [_P, _P, c_int64, c_int64, c_int64, c_int, Operand, Operand, Operand, _P, _P]),
    "dm_quant_nvfp4_weight": (c_int, [_P, _P, c_int64, c_int64, c_int64, _P, _P, c_int, _P]),
    "dm_sf_swizzle": (c_int, [_P, _P, c_int64, c_int64, _P]),
    "dm_gemm_fprop": (
        c_int,
        [Operand, _P, Operand, Operand, _P, _P, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_float, c_float, _P, c_int, _P, _P],
    ),
    "dm_gemm_fprop_dispatch": (
        c_int,
        [_P, _P, Operand, _P, Operand, Operand, _P, c_int, c_int64, c_int64, c_int64, c_int, c_int, c_float, c_float, _P,
         c_int, _P, _P],
    ),
    "dm_gemm_dgrad_dispatch": (c_int, [_P, _P, Operand, _P, Operand, _P, c_int, c_int64, c_int64, c_int64, _P, c_int, _P, _P]),
    "dm_gemm_dgrad": (c_int, [Operand, _P, Operand, _P, _P, c_int, c_int64, c_int64, c_int64, _P, c_int, _P, _P]),
    "dm_gemm_wgrad": (c_int, [Operand, Operand, _P, c_int, c_int, _P, c_int, c_int64, c_int64, c_int64, c_int, _P, _P]),
}

EXPORTS = tuple(_SIGNATURES)

for _name, (_res, _args) in _SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


# Kernel launches issued through this binding (benchmarks report the count).
LAUNCHES = [0]
_LAUNCHES_PER_CALL = {"dm_route": 3, "dm_route_counted": 3}


def route_call_name(ep: int, tokens: int, e_local: int) -> str:
    """Name under which a ``dm_route`` call is counted: the decode regime runs one launch instead of three."""
    single = ep * tokens <= 1024 and e_local <= 512 and lib.dm_route_decode_kernel_enabled()
    return "dm_route(single launch)" if single else "dm_route"


def check(rc: int, what: str) -> None:
    """Raise on a non-zero return code of an entry point."""
    if rc == 0:
        LAUNCHES[0] += _LAUNCHES_PER_CALL.get(what, 1)
        return
    if rc < 0:
        raise NativeError(f"{what}: {RC_NAMES.get(rc, rc)}")
    if rc >= 1000:
        raise NativeError(f"{what}: a CUDA driver call failed with CUresult {rc - 1000}")
    raise NativeError(f"{what}: CUDA error {rc}")


def ptr(t) -> int | None:
    """Device (or pinned host) address of a tensor, ``None`` for ``None``."""
    return None if t is None else t.data_ptr()


def operand(t, offset=None, nbytes: int | None = None) -> Operand:
    """Build a ``dm_operand`` from an allocation tensor and an optional device int64 offset tensor."""
    if t is None:
        return Operand(None, 0, None)
    size = t.numel() * t.element_size() if nbytes is None else nbytes
    return Operand(t.data_ptr(), size, None if offset is None else offset.data_ptr())


def stream_ptr() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream
