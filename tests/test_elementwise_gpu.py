"""Row kernels (gather, SwiGLU fwd/bwd, top-k reduce and its backward) through the C ABI
against plain torch fp32 references.  Tolerance: outputs are bf16, so one bf16 ulp of the
reference value (2^-7 relative) plus a small absolute term."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _native():
    from dist_moe_b200 import _native

    return _native


def _close(got, ref, what, rel=2.0**-7, abs_=1e-3):
    got, ref = got.float(), ref.float()
    scale = ref.pow(2).mean().sqrt().item() + 1e-6
    err = (got - ref).abs()
    bad = err > ref.abs() * rel + abs_ * scale
    assert not bool(bad.any()), f"{what}: {int(bad.sum())}/{bad.numel()} bad, max err {err.max().item():.4g}"


def _swiglu_ref(g, u, clamped):
    if clamped:
        g = g.clamp(max=7.0)
        u = u.clamp(-7.0, 7.0)
        return g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return g * torch.sigmoid(g) * u


@pytest.mark.parametrize("clamped", [0, 1])
def test_swiglu_fwd_bwd_and_clip_stats(clamped):
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    R, F = 777, 1408
    h1 = (torch.randn(R + 10, 2 * F, device=dev) * 4).bfloat16()
    h2 = torch.zeros(R + 10, F, device=dev, dtype=torch.bfloat16)
    rows = torch.tensor([R], dtype=torch.int32, device=dev)
    clip = torch.zeros(3, dtype=torch.float32, device=dev)
    nat.check(nat.lib.dm_swiglu_fwd(h1.data_ptr(), None, h2.data_ptr(), None, rows.data_ptr(), R + 10, F, clamped,
                                    1.702, 7.0, clip.data_ptr(), 7.0, None, nat.stream_ptr()), "swiglu_fwd")
    g, u = h1[:R, :F].float(), h1[:R, F:].float()
    _close(h2[:R], _swiglu_ref(g, u, clamped), "swiglu fwd")
    assert not h2[R:].any(), "rows past num_rows were written"
    expect = torch.tensor([(g > 7.0).sum(), (u.abs() > 7.0).sum(), R * F], dtype=torch.float32, device=dev)
    assert torch.equal(clip, expect), (clip, expect)

    dz = torch.randn(R, F, device=dev).bfloat16()
    gh1 = torch.zeros(R, 2 * F, device=dev, dtype=torch.bfloat16)
    nat.check(nat.lib.dm_swiglu_bwd(h1.data_ptr(), None, dz.data_ptr(), None, gh1.data_ptr(), None, rows.data_ptr(), R,
                                    F, clamped, 1.702, 7.0, nat.stream_ptr()), "swiglu_bwd")
    gx = g.clone().requires_grad_(True)
    ux = u.clone().requires_grad_(True)
    _swiglu_ref(gx, ux, clamped).backward(dz.float())
    dgx, dux = gx.grad, ux.grad
    if clamped:
        # The explicit backward keeps the gradient at exactly +-limit; autograd's clamp does too for
        # max/min ties, so only the strict outside is zero in both.
        pass
    _close(gh1[:, :F], dgx, "swiglu bwd gate", abs_=2e-3)
    _close(gh1[:, F:], dux, "swiglu bwd up", abs_=2e-3)


@pytest.mark.parametrize("ids_dtype,score_dtype", [(torch.int64, torch.float32), (torch.int32, torch.bfloat16)])
def test_scale_and_sum_and_backward(ids_dtype, score_dtype):
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    T, K, D = 333, 6, 2048
    h3 = torch.randn(T, K, D, device=dev).bfloat16()
    scores = torch.rand(T, K, device=dev).to(score_dtype)
    ids = torch.randint(0, 64, (T, K), device=dev).to(ids_dtype)
    ids[torch.rand(T, K, device=dev) < 0.1] = -1
    h3_poison = h3.clone()
    h3_poison[ids < 0] = float("nan")  # skipped routes must not be read into the sum
    out = torch.zeros(T, D, device=dev, dtype=torch.bfloat16)
    save = torch.zeros(T * K * D + 64, device=dev, dtype=torch.bfloat16)
    save_off = torch.tensor([128], dtype=torch.int64, device=dev)
    cond = torch.tensor([0], dtype=torch.int32, device=dev)
    nat.check(nat.lib.dm_scale_and_sum(h3_poison.data_ptr(), scores.data_ptr(), int(score_dtype == torch.bfloat16),
                                       ids.data_ptr(), int(ids_dtype == torch.int64), out.data_ptr(), T, K, D,
                                       save.data_ptr(), save_off.data_ptr(), cond.data_ptr(), 0, nat.stream_ptr()),
              "scale_and_sum")
    w = scores.float() * (ids >= 0)
    _close(out, (h3.float() * w[:, :, None]).sum(1), "scale_and_sum")
    saved = save[64 : 64 + T * K * D].view(T, K, D)
    assert torch.equal(saved.view(torch.int16), h3_poison.view(torch.int16)), "conditional save copy differs"

    # reduce_from_topk: unit weights
    out2 = torch.zeros(T, D, device=dev, dtype=torch.bfloat16)
    nat.check(nat.lib.dm_scale_and_sum(h3_poison.data_ptr(), None, 0, ids.data_ptr(), int(ids_dtype == torch.int64),
                                       out2.data_ptr(), T, K, D, None, None, None, 0, nat.stream_ptr()), "reduce")
    _close(out2, (h3.float() * (ids >= 0)[:, :, None]).sum(1), "reduce_from_topk")

    go = torch.randn(T, D, device=dev).bfloat16()
    buf = h3.clone()  # in place: h3 is read and grad_h3 written at the same addresses
    gs = torch.full((T, K), 9.0, device=dev)
    nat.check(nat.lib.dm_broadcast_and_scale(go.data_ptr(), scores.data_ptr(), int(score_dtype == torch.bfloat16),
                                             ids.data_ptr(), int(ids_dtype == torch.int64), buf.data_ptr(), None,
                                             buf.data_ptr(), gs.data_ptr(), T, K, D, nat.stream_ptr()), "bcast")
    _close(buf, w[:, :, None] * go.float()[:, None, :], "grad_h3")
    ref_gs = (h3.float() * go.float()[:, None, :]).sum(-1) * (ids >= 0)
    assert torch.allclose(gs, ref_gs, rtol=1e-3, atol=1e-2), (gs - ref_gs).abs().max()


def test_gather_rows_and_cond_copy():
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(2)
    src = torch.randn(500, 256, device=dev).bfloat16()
    R = 321
    idx = torch.randint(0, 500, (R + 7,), device=dev)
    ptrs = src.data_ptr() + idx.to(torch.int64) * 512
    ptrs[5] = 0
    arena = torch.full((128 * 3 + (R + 7) * 512,), 0x11, dtype=torch.uint8, device=dev)
    off = torch.tensor([384], dtype=torch.int64, device=dev)
    rows = torch.tensor([R], dtype=torch.int32, device=dev)
    nat.check(nat.lib.dm_gather_rows(ptrs.data_ptr(), rows.data_ptr(), arena.data_ptr(), off.data_ptr(), 512, R + 7,
                                     None, nat.stream_ptr()), "gather")
    got = arena[384:].view(torch.bfloat16).view(R + 7, 256)
    ref = src[idx[:R]].clone()
    ref[5] = 0
    assert torch.equal(got[:R].view(torch.int16), ref.view(torch.int16))
    assert bool((arena[384 + R * 512 :] == 0x11).all()), "rows past num_rows were written"
    for flag, expect_copy in ((1, True), (0, False)):
        dst = torch.zeros(4096, dtype=torch.uint8, device=dev)
        cond = torch.tensor([flag], dtype=torch.int32, device=dev)
        nat.check(nat.lib.dm_cond_copy(arena.data_ptr(), off.data_ptr(), dst.data_ptr(), None, 4096, cond.data_ptr(), 1,
                                       nat.stream_ptr()), "cond_copy")
        assert torch.equal(dst, arena[384 : 384 + 4096]) == expect_copy
