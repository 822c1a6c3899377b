"""Quantisation oracle (CPU) against bytes the reference's own quantisers produced on a B200
(``tests/golden/*_gpu.npz``, written by ``tests/golden/gen_golden_gpu.py``): the Triton quantiser
(dist_moe/kernels/triton_quantization/blockscaled_quantize.py), the CuTe-DSL quantisers
(dist_moe/kernels/blockscaled_quantize.py) and the weight-preparation operators.  Every byte is
compared -- ties, exponent carries, subnormals, infinities and NaNs included; nothing is masked out."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import quant as Q

GOLDEN = Path(__file__).resolve().parent / "golden"


def load(name):
    return np.load(GOLDEN / name)


def bf16(arr):
    return torch.from_numpy(arr.copy()).view(torch.bfloat16)


def blocked_groups(scales_ENS):
    """Blocked scale storage of a grouped [E, N, S] scale tensor: one padded 128-row group per expert."""
    return np.concatenate([Q.to_blocked(s) for s in scales_ENS])


def interleave_rows(F):
    g = np.arange(F).reshape(-1, 8)
    return np.stack([g, g + F], axis=1).reshape(-1)


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_mxfp8_rows_equal_the_triton_quantiser(name):
    G = load("quant_mxfp8_gpu.npz")
    x = bf16(G[name])
    q, s = Q.mxfp8_row(x)
    np.testing.assert_array_equal(s, G[f"{name}_nat_s"])
    np.testing.assert_array_equal(q, G[f"{name}_nat_q"])  # includes the inf / NaN blocks of case "a"
    np.testing.assert_array_equal(Q.to_blocked(s), G[f"{name}_blk_s"].reshape(-1))  # padding bytes are zero


def test_mxfp8_special_blocks_are_present_in_the_golden_input():
    G = load("quant_mxfp8_gpu.npz")
    a = bf16(G["a"]).float()
    assert torch.isinf(a).any() and torch.isnan(a).any() and (a[0, :32] == 0).all()
    s = G["a_nat_s"]
    assert (s == 255).sum() == 2 and (s == 0).any()
    # ties and exponent carries occur in bulk in the random cases (about one value in sixteen is an exact tie)
    c = bf16(G["c"])
    q, sc = Q.mxfp8_row(c)
    v = c.float().numpy() * np.repeat(Q.e8m0_recip(sc), 32, axis=1)
    frac = np.abs(v) / np.exp2(np.floor(np.log2(np.maximum(np.abs(v), 2.0**-9))) - 3)
    assert (np.abs(frac - np.round(frac)) == 0.5).mean() > 0.02


def test_mxfp8_columns_and_tiles_equal_the_triton_quantiser():
    G = load("quant_mxfp8_axes_gpu.npz")
    x = bf16(G["x"])
    qc, sc = Q.mxfp8_col(x)
    np.testing.assert_array_equal(qc.T, G["col_nat_q"])   # the reference stores the column copy transposed
    np.testing.assert_array_equal(sc.T, G["col_nat_s"])
    np.testing.assert_array_equal(Q.to_blocked(sc), G["col_blk_s"].reshape(-1))
    qt, st = Q.mxfp8_tile32(x)
    np.testing.assert_array_equal(qt, G["tile_nat_q"])
    np.testing.assert_array_equal(qt, G["tile_blk_q"])
    row_s, col_s = np.repeat(st, 32, axis=0), np.repeat(st.T, 32, axis=0)
    np.testing.assert_array_equal(row_s, G["tile_nat_s_row"])
    np.testing.assert_array_equal(Q.to_blocked(row_s), G["tile_blk_s_row"].reshape(-1))
    np.testing.assert_array_equal(Q.to_blocked(col_s), G["tile_blk_s_col"].reshape(-1))


def test_mxfp8_all_modes_equal_the_cute_quantisers():
    G = load("quant_mxfp8_cute_gpu.npz")
    x = bf16(G["x"])
    q, s = Q.mxfp8_row(x)
    qc, sc = Q.mxfp8_col(x)
    qt, st = Q.mxfp8_tile32(x)
    np.testing.assert_array_equal(q, G["row_q"])
    np.testing.assert_array_equal(Q.to_blocked(s), G["row_s"].reshape(-1))
    np.testing.assert_array_equal(qc.T, G["col_q"])  # returned as the transposed view of [R, C] storage
    np.testing.assert_array_equal(Q.to_blocked(sc), G["col_s"].reshape(-1))
    np.testing.assert_array_equal(q, G["both_row_q"])
    np.testing.assert_array_equal(qc.T if G["both_col_q"].shape != qc.shape else qc, G["both_col_q"])
    np.testing.assert_array_equal(Q.to_blocked(s), G["both_row_s"].reshape(-1))
    np.testing.assert_array_equal(Q.to_blocked(sc), G["both_col_s"].reshape(-1))
    np.testing.assert_array_equal(qt, G["tile_q"])
    np.testing.assert_array_equal(Q.to_blocked(np.repeat(st, 32, axis=0)), G["tile_s_row"].reshape(-1))
    np.testing.assert_array_equal(Q.to_blocked(np.repeat(st.T, 32, axis=0)), G["tile_s_col"].reshape(-1))


def test_mxfp8_weight_preparation_equals_the_reference_operator():
    """``dist_moe::prepare_mxfp8_weight``: training (32x32 tiles, one qdata, two scale orientations), inference rows,
    inference rows with the fused-SwiGLU interleave."""
    G = load("prep_mxfp8_weight_gpu.npz")
    w = bf16(G["w"])
    E, N, K = w.shape
    tiles = [Q.mxfp8_tile32(w[e]) for e in range(E)]
    np.testing.assert_array_equal(np.stack([t[0] for t in tiles]), G["train_q"])
    np.testing.assert_array_equal(blocked_groups([np.repeat(t[1], 32, axis=0) for t in tiles]), G["train_sf"].reshape(-1))
    np.testing.assert_array_equal(blocked_groups([np.repeat(t[1].T, 32, axis=0) for t in tiles]),
                                  G["train_sd"].reshape(-1))
    rows = [Q.mxfp8_row(w[e]) for e in range(E)]
    np.testing.assert_array_equal(np.stack([r[0] for r in rows]), G["infer_q"])
    np.testing.assert_array_equal(blocked_groups([r[1] for r in rows]), G["infer_sf"].reshape(-1))
    assert G["infer_sd"].size == 0
    idx = interleave_rows(N // 2)
    np.testing.assert_array_equal(np.stack([r[0][idx] for r in rows]), G["infer_fused_q"])
    np.testing.assert_array_equal(blocked_groups([r[1][idx] for r in rows]), G["infer_fused_sf"].reshape(-1))


@pytest.mark.parametrize("name", ["w", "w13plain"])
def test_nvfp4_weights_equal_the_reference_operator(name):
    """``dist_moe::prepare_nvfp4_weight``: packed codes, E4M3 block scales (blocked), global scale and its inverse."""
    G = load("quant_nvfp4_gpu.npz")
    w = bf16(G[name])
    packed, sb, gs, gsi = Q.nvfp4_weight(w)
    np.testing.assert_array_equal(gs.view(np.uint32), G[f"{name}_gs"].view(np.uint32))
    np.testing.assert_array_equal(gsi.view(np.uint32), G[f"{name}_gsi"].view(np.uint32))
    np.testing.assert_array_equal(packed, G[f"{name}_q"])
    np.testing.assert_array_equal(blocked_groups(sb), G[f"{name}_s"].reshape(-1))


def test_nvfp4_interleaved_w13_equals_the_reference_operator():
    G = load("quant_nvfp4_gpu.npz")
    w = bf16(G["w13"])
    packed, sb, gs, _ = Q.nvfp4_weight(w)
    idx = interleave_rows(w.shape[1] // 2)
    np.testing.assert_array_equal(packed[:, idx], G["w13_q"])
    np.testing.assert_array_equal(blocked_groups(sb[:, idx]), G["w13_s"].reshape(-1))
    np.testing.assert_array_equal(gs.view(np.uint32), G["w13_gs"].view(np.uint32))


@pytest.mark.parametrize("file,names", [("quant_nvfp4_token_cute_gpu.npz", "tuv"), ("quant_nvfp4_gpu.npz", "tu")])
def test_nvfp4_token_rows_equal_the_reference_quantisers(file, names):
    """Per-token NVFP4: the CuTe quantiser (``_quantize_nvfp4_per_token``) computes the row scale itself; the Triton
    quantiser is given ``2688 * reciprocal(max(row amax, 1e-8))`` as its per-token global scale.  Both give the same
    codes, block scales and inverse row scales as the oracle."""
    G = load(file)
    for n in names:
        x = bf16(G[n])
        packed, sb, inv = Q.nvfp4_token_rows(x)
        np.testing.assert_array_equal(inv.view(np.uint32), G[f"{n}_inv"].view(np.uint32))
        np.testing.assert_array_equal(sb, G[f"{n}_s"])
        np.testing.assert_array_equal(packed, G[f"{n}_q"])


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


def test_e2m1_and_e4m3_codecs():
    vals = np.array([0, 0.25, 0.26, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 5.01, 6, 7, 100, -0.75, -6.5, np.nan], np.float32)
    codes = Q.e2m1_rn_satfinite(vals)
    np.testing.assert_array_equal(codes, [0, 0, 1, 2, 2, 4, 4, 6, 6, 7, 7, 7, 7, 10, 15, 7])
    np.testing.assert_array_equal(Q.e4m3_rn_satfinite(np.array([448, 1000, -1000, 0.001953125, np.nan], np.float32)),
                                  [0x7E, 0x7E, 0xFE, 0x01, 0x7F])
    np.testing.assert_array_equal(Q.e8m0_round_up(np.array([0, 1, 1.0001, 2.0**-127, 2.0**-126, np.inf], np.float32)),
                                  [0, 127, 128, 0, 1, 255])


def test_nvfp4_round_trip_error():
    g = torch.Generator().manual_seed(5)
    x = (torch.randn(33, 256, generator=g) * torch.logspace(-2, 2, 33)[:, None]).bfloat16()
    packed, sb, inv = Q.nvfp4_token_rows(x)
    deq = Q.nvfp4_dequant(packed, sb, inv)
    ref = x.float().numpy()
    assert np.linalg.norm(deq - ref) / np.linalg.norm(ref) < 0.12
    assert np.allclose(np.abs(ref).max(1) / inv, 2688.0, rtol=1e-5)
