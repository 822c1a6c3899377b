"""Fused post-expert RMSNorm kernels through the C ABI: compensated (Kahan) sum of squares against float64, and
the fused RMSNorm on the MXFP8 training path against autograd through the dense oracle.

The reference offers ``use_kahan`` for "near-FP64 accuracy in FP32" of the normalisation's sum of squares
(dist_moe/kernels/norm/fused_rmsnorm_combine.py:16, dist_moe/_postprocess.py:44-46); the check here is exactly that:
with it the reciprocal RMS stays within the rounding of ``rsqrtf`` of the float64 value, on rows built so that the
plain fp32 sum is visibly off."""

import pytest
import torch

from oracle import moe as oracle_moe
from tests.test_blockscaled_layer_gpu import MX_FWD, MX_GRAD, MX_WGRAD, _aggregate, _case, _grad_out

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _nat():
    from dist_moe_b200 import _native

    return _native


def _rstd(nat, h3, ids, scores, eps, kahan):
    T, K, D = h3.shape
    out = torch.empty(T, D, dtype=torch.bfloat16, device=DEV)
    rstd = torch.empty(T, K, dtype=torch.float32, device=DEV)
    nat.check(nat.lib.dm_rmsnorm_combine_fwd(h3.data_ptr(), scores.data_ptr(), 0, ids.data_ptr(), 0, None, 0.0, eps, 0,
                                             int(kahan), out.data_ptr(), rstd.data_ptr(), T, K, D, None, None, None, 0,
                                             nat.stream_ptr()), "dm_rmsnorm_combine_fwd")
    torch.cuda.synchronize()
    return out, rstd


def test_kahan_sum_of_squares_matches_float64():
    nat = _nat()
    T, K, D = 64, 2, 8192
    g = torch.Generator().manual_seed(3)
    # one huge element followed by thousands of small ones: a plain fp32 running sum drops most of the small squares
    h3 = (torch.rand(T, K, D, generator=g) * 0.25 + 0.25).bfloat16()
    h3[:, :, 0] = 2048.0
    ids = torch.zeros(T, K, dtype=torch.int32)
    scores = torch.full((T, K), 0.5)
    eps = 1e-6
    exact = torch.rsqrt(h3.double().pow(2).mean(-1) + eps)
    _, plain = _rstd(nat, h3.to(DEV), ids.to(DEV), scores.to(DEV), eps, kahan=False)
    _, comp = _rstd(nat, h3.to(DEV), ids.to(DEV), scores.to(DEV), eps, kahan=True)
    ulp = torch.finfo(torch.float32).eps * exact.float().abs()
    err_plain = (plain.cpu().double() - exact).abs()
    err_comp = (comp.cpu().double() - exact).abs()
    # rsqrtf itself may be off by two units in the last place; the compensated sum adds less than one
    assert bool((err_comp <= 3.0 * ulp.double()).all()), (err_comp / ulp.double()).max()
    assert err_comp.max() <= err_plain.max() and err_comp.mean() < err_plain.mean()


@pytest.mark.parametrize("kahan,recompute_rstd", [(False, False), (True, True)])
def test_kahan_backward_matches_the_plain_backward(kahan, recompute_rstd):
    """The compensated backward (which may recompute rstd) agrees with float64 autograd of the same composition."""
    nat = _nat()
    T, K, D = 48, 3, 1024
    g = torch.Generator().manual_seed(5)
    h3 = torch.randn(T, K, D, generator=g).bfloat16()
    go = torch.randn(T, D, generator=g).bfloat16()
    ids = torch.zeros(T, K, dtype=torch.int32)
    ids[3, 1] = -1
    scores = torch.rand(T, K, generator=g)
    eps = 1e-5
    hd = h3.double().requires_grad_()
    sd = scores.double().requires_grad_()
    valid = (ids >= 0)[:, :, None]
    y = hd * torch.rsqrt(hd.pow(2).mean(-1, keepdim=True) + eps) * valid
    (y * sd[:, :, None]).sum(1).mul(go.double()).sum().backward()
    _, rstd = _rstd(nat, h3.to(DEV), ids.to(DEV), scores.to(DEV), eps, kahan)
    grad_h3 = torch.empty(T, K, D, dtype=torch.bfloat16, device=DEV)
    grad_s = torch.empty(T, K, dtype=torch.float32, device=DEV)
    h3d, god, sdev, idev = h3.to(DEV), go.to(DEV), scores.to(DEV), ids.to(DEV)
    nat.check(nat.lib.dm_rmsnorm_combine_bwd(god.data_ptr(), sdev.data_ptr(), 0, idev.data_ptr(),
                                             0, h3d.data_ptr(), None, None if recompute_rstd else rstd.data_ptr(), eps,
                                             0, int(kahan), grad_h3.data_ptr(), grad_s.data_ptr(), T, K, D,
                                             nat.stream_ptr()), "dm_rmsnorm_combine_bwd")
    torch.cuda.synchronize()
    torch.testing.assert_close(grad_h3.float().cpu(), hd.grad.float(), rtol=2e-2, atol=2e-2)
    torch.testing.assert_close(grad_s.cpu(), (sd.grad * (ids >= 0)).float(), rtol=1e-3, atol=1e-3)


@pytest.mark.parametrize("norm_dtype,recompute_rstd,kahan", [(torch.float32, False, False), (torch.bfloat16, True, True)])
def test_mxfp8_training_with_fused_rmsnorm(norm_dtype, recompute_rstd, kahan):
    import dist_moe_b200 as dm

    T, D, F, K, E = 200, 512, 384, 4, 8
    x, ids, scores, w13, w2 = _case(T, D, F, K, E, seed=77)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=DEV)
    try:
        eps = 1e-6
        post = dm.RMSNormPostprocess(eps=eps, norm_output_dtype=norm_dtype, output_dtype=torch.bfloat16,
                                     require_bitwise=False, recompute_rstd=recompute_rstd, use_kahan=kahan)
        xs, ss = x.to(DEV).requires_grad_(), scores.to(DEV).requires_grad_()
        a, b = w13.to(DEV).requires_grad_(), w2.to(DEV).requires_grad_()
        out = dm.routed_experts(xs, ids.to(DEV), ss, a, b, ctx, options=dm.ExecutionOptions(experts_output_postprocess=post))
        go = _grad_out(T, D)
        out.backward(go.to(DEV))
        ctx.check_status()
        xr, sr = x.clone().requires_grad_(), scores.clone().requires_grad_()
        ar, br = w13.clone().requires_grad_(), w2.clone().requires_grad_()
        h3 = oracle_moe.expert_outputs(xr, ids, ar.reshape(E, 2 * F, D), br)
        hf = h3.float()
        rstd = torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * (ids >= 0)[:, :, None]
        ref = ((hf * rstd).to(norm_dtype).float() * sr[:, :, None]).sum(1).to(torch.bfloat16)
        ref.backward(go)
        _aggregate(out, ref, MX_FWD, "normalised output")
        _aggregate(xs.grad, xr.grad, MX_GRAD, "grad x")
        _aggregate(ss.grad, sr.grad, MX_GRAD, "grad scores")
        _aggregate(a.grad, ar.grad, MX_WGRAD, "grad w13")
        _aggregate(b.grad, br.grad, MX_WGRAD, "grad w2")
    finally:
        ctx.close()
