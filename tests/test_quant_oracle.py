"""Quantisation oracle (CPU): MXFP8 against bytes produced by the reference's Triton quantiser
(``tests/golden/quant_mxfp8.npz``); NVFP4 (parity unpinned by any reference execution) against the
properties its definition implies."""

from pathlib import Path

import numpy as np
import torch

from oracle import quant as Q

G = np.load(Path(__file__).resolve().parent / "golden" / "quant_mxfp8.npz")


def _bf16(arr):
    return torch.from_numpy(arr.copy()).view(torch.bfloat16)


def _assert_bytes_equal_up_to_ties(x, q, s, ref_q):
    """Data bytes must equal the reference kernel's wherever the Triton CPU interpreter's *software*
    fp32->e4m3 cast is faithful to the instruction the reference names
    (``cvt.rn.satfinite.e4m3x2.f32``, round to nearest even).  That emulation is wrong in three
    value-determined situations, which are excluded by a rule computed from the scaled value alone:
    exact rounding ties (it rounds them away from zero) and values that round *up* into the next
    binade (it drops the exponent carry), and results in the E4M3 subnormal range (it truncates).  Everywhere else the bytes must be identical."""
    v = (x.float().numpy() * np.repeat(Q.e8m0_recip(s), 32, axis=1)).astype(np.float64)
    mine = Q.e4m3_to_f32(q).astype(np.float64)
    mag = np.abs(mine)
    is_pow2 = (mag > 0) & (np.exp2(np.floor(np.log2(np.where(mag > 0, mag, 1)))) == mag)
    carry = is_pow2 & (mag > np.abs(v))
    below = Q.e4m3_to_f32(np.where(q & 0x7F, q - 1, q).astype(np.uint8)).astype(np.float64)
    above = Q.e4m3_to_f32(np.where((q & 0x7F) < 0x7E, q + 1, q).astype(np.uint8)).astype(np.float64)
    tie = (np.abs(v - mine) == np.abs(below - v)) | (np.abs(v - mine) == np.abs(above - v))
    tie &= v != mine
    subnormal = (mag < 2.0**-6) & (mag > 0)  # the emulation truncates in the E4M3 subnormal range
    excluded = carry | tie | subnormal
    np.testing.assert_array_equal(q[~excluded], ref_q[~excluded])
    assert excluded.mean() < 0.15
    assert ((q[tie] & 1) == 0).all(), "ties go to the even code"


def test_mxfp8_row_bytes_and_scales_match_reference_kernel():
    a = _bf16(G["a"])
    q, s = Q.mxfp8_row(a)
    np.testing.assert_array_equal(s, G["a_s"])
    finite_blocks = np.repeat(G["a_s"] != 255, 32, axis=1)
    qa, ra = q.copy(), G["a_q"].copy()
    qa[~finite_blocks] = 0
    ra[~finite_blocks] = 0
    _assert_bytes_equal_up_to_ties(a, qa, np.where(G["a_s"] == 255, 127, s).astype(np.uint8), ra)
    # non-finite blocks: the scale byte is 0xFF and every data byte is a NaN encoding
    assert ((q[~finite_blocks] & 0x7F) == 0x7F).all()
    assert (~finite_blocks).any()


def test_mxfp8_blocked_scale_layout_matches_reference_kernel():
    b = _bf16(G["b"])
    q, s = Q.mxfp8_row(b)
    _assert_bytes_equal_up_to_ties(b, q, s, G["b_q"])
    ref = G["b_s_blocked"]
    rows, cols = s.shape
    r, c = np.meshgrid(np.arange(rows), np.arange(cols), indexing="ij")
    np.testing.assert_array_equal(ref[Q.blocked_scale_offset(r, c, (cols + 3) // 4)], s)
    mine = Q.to_blocked(s)
    written = np.zeros(ref.shape, dtype=bool)
    written[Q.blocked_scale_offset(r, c, (cols + 3) // 4)] = True
    np.testing.assert_array_equal(mine[written], ref[written])


def test_mxfp8_scale_is_minimal_power_of_two():
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(64, 256, generator=g) * torch.logspace(-3, 3, 64)[:, None]).bfloat16()
    q, s = Q.mxfp8_row(x)
    amax = x.float().abs().reshape(64, 8, 32).amax(-1).numpy().astype(np.float64)
    scale = np.exp2(s.astype(np.float64) - 127)
    assert (amax / scale <= 448 * (1 + 2**-20)).all()
    assert ((amax / (scale / 2) > 448 * (1 - 2**-20)) | (s == 0)).all()
    deq = Q.mxfp8_dequant_row(q, s).reshape(64, 256)
    err = np.abs(deq - x.float().numpy())
    assert (err <= np.repeat(scale, 32, axis=1) * 448 * 2.0**-4 + 1e-30).all()  # half an E4M3 ulp at the block top


def test_col_and_tile_modes_share_the_row_arithmetic():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(96, 64, generator=g).bfloat16()
    qc, sc = Q.mxfp8_col(x)
    qr, sr = Q.mxfp8_row(x.t().contiguous())
    np.testing.assert_array_equal(qc, qr.T)
    np.testing.assert_array_equal(sc, sr)
    qt, st = Q.mxfp8_tile32(x)
    assert st.shape == (3, 2)
    amax = x.float().abs().reshape(3, 32, 2, 32).amax(dim=(1, 3)).numpy()
    np.testing.assert_array_equal(st, Q.e8m0_round_up(amax.astype(np.float32) * Q.RECIP_448))


def test_e2m1_and_e4m3_codecs():
    vals = np.array([0, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 6, 7, 100, -0.75, -6.5, np.nan], np.float32)
    codes = Q.e2m1_rn_satfinite(vals)
    np.testing.assert_array_equal(codes, [0, 0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 7, 7, 10, 15, 7])
    np.testing.assert_array_equal(Q.e4m3_rn_satfinite(np.array([448, 1000, -1000, 0.001953125, np.nan], np.float32)),
                                  [0x7E, 0x7E, 0xFE, 0x01, 0x7F])
    np.testing.assert_array_equal(Q.e8m0_round_up(np.array([0, 1, 1.0001, 2.0**-127, 2.0**-126, np.inf], np.float32)),
                                  [0, 127, 128, 0, 1, 255])


def test_nvfp4_token_and_weight_properties():
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(33, 256, generator=g) * torch.logspace(-2, 2, 33)[:, None]).bfloat16()
    packed, sb, inv = Q.nvfp4_token_rows(x)
    assert packed.shape == (33, 128) and sb.shape == (33, 16) and inv.shape == (33,)
    deq = Q.nvfp4_dequant(packed, sb, inv)
    ref = x.float().numpy()
    rel = np.linalg.norm(deq - ref) / np.linalg.norm(ref)
    assert rel < 0.12, rel
    # the largest element of every row maps to the top of the format: |x|max * row_scale == 2688
    assert np.allclose(np.abs(ref).max(1) / inv, 2688.0, rtol=1e-5)
    w = (torch.randn(3, 64, 128, generator=g) * 0.02).bfloat16()
    wp, ws, gs, gsi = Q.nvfp4_weight(w)
    wd = Q.nvfp4_dequant(wp.reshape(3 * 64, 64), ws.reshape(3 * 64, 8), np.repeat(gsi, 64))
    relw = np.linalg.norm(wd - w.float().numpy().reshape(192, 128)) / np.linalg.norm(w.float().numpy())
    assert relw < 0.12, relw
    assert np.allclose(gs * gsi, 1.0, rtol=1e-6)
