"""Block-scaled quantisation (MXFP8 E4M3, NVFP4), restated with numpy integer/float32 arithmetic.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

MXFP8 (dist_moe/kernels/blockscaled_quantization_common.py:120-147,
dist_moe/kernels/triton_quantization/blockscaled_quantize.py:296-365, 585-615):
  amax over a 32-element block in fp32 (NaN -> inf); ``s = amax * fl(1/448)``;
  scale byte = ``s`` rounded UP to a power of two (E8M0, ``cvt.rp.ue8m0x2.f32``, inf -> 0xFF);
  ``recip = bitcast((254 - byte) << 23)`` (NaN for byte 0xFF); ``q = e4m3_rn_satfinite(x * recip)``.
NVFP4 (same file 179-257, 739-752; triton twin 368-493; global_scale.py:37-72):
  per token ``row_scale = 2688 * rcp_rn(max(row_amax, 1e-8))``, ``token_scale_inv = rcp_rn(row_scale)``;
  per expert weight ``gs = 2688 * reciprocal(clamp(amax, 1e-12))``;
  per 16-block ``raw = (amax * scale) * fl(1/6)`` clamped to [2^-9, 448], scale byte = e4m3_rn(raw),
  ``mult = div_rn(scale, f32(scale byte))``, codes = e2m1_rn_satfinite(x * mult), two per byte with the
  even element in the low nibble.
Scale storage: natural row-major, or the 128x4 blocked atom
``atom*512 + (row%32)*16 + (row//32 % 4)*4 + col%4`` with atoms ordered (row atom, column atom)
(blockscaled_quantize.py:1012-1043).

Pin status: every function here is pinned, byte for byte with nothing masked out, against outputs of the
reference's own quantisers executed on a B200 (``tests/golden/*_gpu.npz``, produced by
``tests/golden/gen_golden_gpu.py``): the Triton quantiser for MXFP8 rows / columns / 32x32 tiles and NVFP4 rows
and weights, the CuTe-DSL quantisers for the same MXFP8 modes and for per-token NVFP4, and the two
weight-preparation operators (``tests/test_quant_oracle.py``).
"""

from __future__ import annotations

import numpy as np
import torch

F32 = np.float32
FP8_MAX, FP4_MAX = F32(448.0), F32(6.0)
RECIP_448 = F32(1.0) / F32(448.0)
RECIP_6 = F32(1.0 / 6.0)
NVFP4_NUMERATOR = F32(2688.0)
E4M3_MIN_SUBNORMAL = F32(0.001953125)


def e8m0_round_up(s):
    """Smallest power of two >= s as an E8M0 byte (cvt.rp.ue8m0x2.f32): 0 -> 0, inf/NaN -> 0xFF."""
    s = np.asarray(s, dtype=F32)
    bits = s.view(np.uint32)
    exp = ((bits >> 23) & 0xFF).astype(np.int64)
    mant = (bits & 0x7FFFFF).astype(np.int64)
    byte = exp + (mant != 0)
    denorm = exp == 0
    byte = np.where(denorm, np.where(mant > 0x400000, 1, 0), byte)
    byte = np.where(exp == 255, 255, np.minimum(byte, 255))
    return byte.astype(np.uint8)


def e8m0_recip(byte):
    byte = np.asarray(byte, dtype=np.int64)
    bits = ((254 - byte) << 23).astype(np.uint32)
    out = bits.view(F32).copy()
    out[byte == 255] = np.nan
    return out


def e4m3_rn_satfinite(v):
    """fp32 -> E4M3 byte, round to nearest even, saturate to +-448, NaN -> 0x7F."""
    v = np.asarray(v, dtype=F32)
    nan = np.isnan(v)
    c = np.clip(np.where(nan, 0, v), -448.0, 448.0).astype(F32)
    b = torch.from_numpy(c).to(torch.float8_e4m3fn).view(torch.uint8).numpy().copy()
    b[nan] = 0x7F
    return b


def e4m3_to_f32(b):
    return torch.from_numpy(np.asarray(b, dtype=np.uint8)).view(torch.float8_e4m3fn).float().numpy()


def e2m1_rn_satfinite(v):
    """fp32 -> 4-bit E2M1 code (sign << 3 | magnitude index), RN-even, saturate to 6, NaN -> +6."""
    v = np.asarray(v, dtype=F32)
    a = np.abs(v)
    idx = ((a > 0.25).astype(np.uint8) + (a >= 0.75) + (a > 1.25) + (a >= 1.75) + (a > 2.5) + (a >= 3.5) + (a > 5.0))
    code = idx.astype(np.uint8) | (np.signbit(v).astype(np.uint8) << 3)
    return np.where(np.isnan(v), np.uint8(7), code).astype(np.uint8)


E2M1_VALUES = np.array([0, 0.5, 1, 1.5, 2, 3, 4, 6], dtype=F32)


def e2m1_to_f32(code):
    code = np.asarray(code, dtype=np.uint8)
    return np.where(code & 8, -1.0, 1.0).astype(F32) * E2M1_VALUES[code & 7]


def blocked_scale_offset(row, col, n_col_atoms):
    row, col = np.asarray(row, dtype=np.int64), np.asarray(col, dtype=np.int64)
    atom = (row // 128) * n_col_atoms + col // 4
    return atom * 512 + (row % 32) * 16 + ((row % 128) // 32) * 4 + col % 4


def to_blocked(scales):
    """[rows, cols] natural scale bytes -> flat blocked storage (rows padded to 128, cols to 4, pad = 0)."""
    rows, cols = scales.shape
    pr, pc = (rows + 127) // 128 * 128, (cols + 3) // 4 * 4
    out = np.zeros(pr * pc, dtype=scales.dtype)
    r, c = np.meshgrid(np.arange(rows), np.arange(cols), indexing="ij")
    out[blocked_scale_offset(r, c, pc // 4)] = scales
    return out


def _amax_nonfinite(xb):
    a = np.abs(xb)
    a = np.where(np.isnan(a), np.inf, a)
    return a.max(axis=-1).astype(F32)


def mxfp8_quantize_blocks(xb):
    """xb: float32 [..., 32] blocks -> (q uint8 [..., 32], scale byte [...])."""
    amax = _amax_nonfinite(xb)
    byte = e8m0_round_up(amax * RECIP_448)
    recip = e8m0_recip(byte)
    q = e4m3_rn_satfinite(xb.astype(F32) * recip[..., None])
    return q, byte


def mxfp8_row(x):
    """x: bf16 torch tensor [R, C] -> (q [R, C] u8, scales [R, C/32] u8), 1x32 blocks along C."""
    xf = x.float().numpy()
    R, C = xf.shape
    q, s = mxfp8_quantize_blocks(xf.reshape(R, C // 32, 32))
    return q.reshape(R, C), s


def mxfp8_col(x):
    """32x1 blocks along the rows: (q [R, C], scales [C, ceil(R/32)]); missing rows count as zeros."""
    xf = x.float().numpy()
    R, C = xf.shape
    Rp = (R + 31) // 32 * 32
    xp = np.zeros((Rp, C), dtype=F32)
    xp[:R] = xf
    blocks = xp.reshape(Rp // 32, 32, C).transpose(2, 0, 1)  # [C, R/32, 32]
    q, s = mxfp8_quantize_blocks(blocks)
    return q.transpose(1, 2, 0).reshape(Rp, C)[:R], s


def mxfp8_tile32(w):
    """32x32 tiles: one scale per tile; returns (q [N, K], scales [N/32, K/32])."""
    wf = w.float().numpy()
    N, K = wf.shape
    t = wf.reshape(N // 32, 32, K // 32, 32).transpose(0, 2, 1, 3).reshape(N // 32, K // 32, 1024)
    amax = _amax_nonfinite(t)
    byte = e8m0_round_up(amax * RECIP_448)
    recip = e8m0_recip(byte)
    q = e4m3_rn_satfinite(t * recip[..., None]).reshape(N // 32, K // 32, 32, 32).transpose(0, 2, 1, 3).reshape(N, K)
    return q, byte


def mxfp8_dequant_row(q, s):
    scale = np.exp2(s.astype(np.float64) - 127.0)
    return e4m3_to_f32(q).reshape(q.shape[0], -1, 32) * scale[..., None]


def _nvfp4_blocks(xb, scale):
    """xb [..., nb, 16] float32, scale [...] (per row/expert) -> (codes [..., nb, 16], scale bytes [..., nb])."""
    amax = _amax_nonfinite(xb)
    amax = np.where(np.isinf(amax), np.nan, amax).astype(F32)
    raw = ((amax * scale[..., None]).astype(F32) * RECIP_6).astype(F32)
    raw = np.where(np.isnan(raw), raw, np.clip(raw, E4M3_MIN_SUBNORMAL, FP8_MAX)).astype(F32)
    sb = e4m3_rn_satfinite(raw)
    sf = e4m3_to_f32(sb)
    mult = (scale[..., None].astype(F32) / sf).astype(F32)  # one correctly rounded fp32 division
    codes = e2m1_rn_satfinite((xb.astype(F32) * mult[..., None]).astype(F32))
    return codes, sb


def pack_e2m1(codes):
    codes = codes.reshape(*codes.shape[:-2], -1)
    return (codes[..., 0::2] | (codes[..., 1::2] << 4)).astype(np.uint8)


def nvfp4_token_rows(x):
    """Per-token NVFP4: x bf16 [R, C] -> (packed [R, C/2], scale bytes [R, C/16], token_scale_inv f32 [R])."""
    xf = x.float().numpy()
    R, C = xf.shape
    row_amax = np.abs(xf).max(axis=1).astype(F32)
    row_scale = (NVFP4_NUMERATOR * (F32(1.0) / np.maximum(row_amax, F32(1e-8))).astype(F32)).astype(F32)
    inv = (F32(1.0) / row_scale).astype(F32)
    codes, sb = _nvfp4_blocks(xf.reshape(R, C // 16, 16), row_scale)
    return pack_e2m1(codes), sb, inv


def nvfp4_weight(w):
    """Per-expert NVFP4: w bf16 [E, N, K] -> (packed [E, N, K/2], scale bytes [E, N, K/16], gs [E], 1/gs [E])."""
    wf = w.float().numpy()
    E, N, K = wf.shape
    amax = np.maximum(np.abs(wf).reshape(E, -1).max(axis=1).astype(F32), F32(1e-12))
    gs = (NVFP4_NUMERATOR * (F32(1.0) / amax).astype(F32)).astype(F32)
    codes, sb = _nvfp4_blocks(wf.reshape(E, N, K // 16, 16), np.broadcast_to(gs[:, None], (E, N)).copy())
    return pack_e2m1(codes), sb, gs, (F32(1.0) / gs).astype(F32)


def nvfp4_dequant(packed, sb, inv_scale):
    lo, hi = packed & 0xF, packed >> 4
    codes = np.stack([lo, hi], axis=-1).reshape(*packed.shape[:-1], -1)
    vals = e2m1_to_f32(codes).reshape(*sb.shape, 16) * e4m3_to_f32(sb)[..., None]
    return vals.reshape(*packed.shape[:-1], -1) * np.asarray(inv_scale, dtype=F32)[..., None]
