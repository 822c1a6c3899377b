"""Shared numeric checks for the parity tests."""

import torch


def assert_close(got, ref, *, rtol, atol, rel_l2, cosine, what):
    """The four-part bound the reference's tests use: elementwise rtol/atol, relative L2
    error below ``rel_l2`` and cosine similarity above ``cosine``."""
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err = (got - ref).abs()
    bad = err > atol + rtol * ref.abs()
    l2 = (got - ref).norm() / ref.norm().clamp_min(1e-12)
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0)
    assert not bad.any(), f"{what}: {int(bad.sum())}/{bad.numel()} elements exceed rtol={rtol} atol={atol}; max err {err.max():.4g}"
    assert l2 < rel_l2, f"{what}: relative L2 {l2:.4g} >= {rel_l2}"
    assert cos > cosine, f"{what}: cosine {cos:.6f} <= {cosine}"


BF16_FWD = dict(rtol=2e-2, atol=2e-2, rel_l2=5e-3, cosine=0.999)
BF16_GRAD = dict(rtol=3e-2, atol=3e-2, rel_l2=1e-2, cosine=0.995)
BF16_WGRAD = dict(rtol=3e-2, atol=1.0, rel_l2=1.5e-2, cosine=0.995)
