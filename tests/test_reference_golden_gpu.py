"""The CUDA kernels against outputs of the reference's own GPU kernels, recorded on a B200 by
``tests/golden/gen_golden_gpu.py`` (``tests/golden/*_gpu.npz``).

Quantised bytes, scale bytes, global scales and the element-wise kernels are compared bit for bit with no mask.
Layer outputs and gradients (grouped GEMMs in between, whose fp32 accumulation order is free) are compared with the
reference's own tolerances (tests/test_dist_moe.py:317-325) and, more tightly, by the share of bit-identical bf16
values, which is what two correct implementations of the same rounding points give."""

from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import quant as Q
from tests.test_quant_oracle import bf16, blocked_groups, interleave_rows, load

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _nat():
    from dist_moe_b200 import _native

    return _native


def _dm():
    import dist_moe_b200 as dm

    return dm


# ---------------------------------------------------------------------------------------------------------------
# quantisers
# ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_mxfp8_row_kernel_equals_the_reference_bytes(name):
    nat, G = _nat(), load("quant_mxfp8_gpu.npz")
    x = bf16(G[name]).to(DEV)
    rows, cols = x.shape
    sc = cols // 32
    cnt = torch.tensor([rows], dtype=torch.int32, device=DEV)
    q = torch.zeros(rows, cols, dtype=torch.uint8, device=DEV)
    s = torch.zeros(rows, sc, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_row(x.data_ptr(), cnt.data_ptr(), rows, cols, q.data_ptr(), 0, s.data_ptr(), 0, 0,
                                         nat.stream_ptr()), "row")
    sb = torch.zeros(G[f"{name}_blk_s"].size, dtype=torch.uint8, device=DEV)
    q2 = torch.zeros_like(q)
    nat.check(nat.lib.dm_quant_mxfp8_row(x.data_ptr(), cnt.data_ptr(), rows, cols, q2.data_ptr(), 0, sb.data_ptr(), 0, 1,
                                         nat.stream_ptr()), "row blocked")
    torch.cuda.synchronize()
    np.testing.assert_array_equal(s.cpu().numpy(), G[f"{name}_nat_s"])
    np.testing.assert_array_equal(q.cpu().numpy(), G[f"{name}_nat_q"])  # NaN / inf blocks included
    np.testing.assert_array_equal(q2.cpu().numpy(), G[f"{name}_nat_q"])
    np.testing.assert_array_equal(sb.cpu().numpy(), G[f"{name}_blk_s"].reshape(-1))


def test_mxfp8_column_and_both_axes_kernels_equal_the_reference_bytes():
    nat, G = _nat(), load("quant_mxfp8_cute_gpu.npz")
    x = bf16(G["x"]).to(DEV)
    rows, cols = x.shape
    cnt = torch.tensor([rows], dtype=torch.int32, device=DEV)
    q = torch.zeros(rows, cols, dtype=torch.uint8, device=DEV)
    s = torch.zeros(G["col_s"].size, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_col(x.data_ptr(), cnt.data_ptr(), rows, cols, q.data_ptr(), s.data_ptr(), 1,
                                         nat.stream_ptr()), "col")
    outs = [torch.zeros(rows, cols, dtype=torch.uint8, device=DEV), torch.zeros(G["both_row_s"].size, dtype=torch.uint8, device=DEV),
            torch.zeros(rows, cols, dtype=torch.uint8, device=DEV), torch.zeros(G["both_col_s"].size, dtype=torch.uint8, device=DEV)]
    nat.check(nat.lib.dm_quant_mxfp8_rowcol(x.data_ptr(), cnt.data_ptr(), rows, cols, *[t.data_ptr() for t in outs],
                                            nat.stream_ptr()), "rowcol")
    torch.cuda.synchronize()
    np.testing.assert_array_equal(q.cpu().numpy().T, G["col_q"])  # the reference returns the column copy transposed
    np.testing.assert_array_equal(s.cpu().numpy(), G["col_s"].reshape(-1))
    np.testing.assert_array_equal(outs[0].cpu().numpy(), G["both_row_q"])
    np.testing.assert_array_equal(outs[1].cpu().numpy(), G["both_row_s"].reshape(-1))
    both_col = G["both_col_q"]
    np.testing.assert_array_equal(outs[2].cpu().numpy() if both_col.shape == (rows, cols) else outs[2].cpu().numpy().T, both_col)
    np.testing.assert_array_equal(outs[3].cpu().numpy(), G["both_col_s"].reshape(-1))


def test_weight_preparation_equals_the_reference_operators():
    """The bodies of ``dist_moe::prepare_mxfp8_weight`` and ``dist_moe::prepare_nvfp4_weight`` (shape-only contract,
    as in the reference) against what the reference's operators returned for the same weights."""
    from dist_moe_b200._blockscaled import quantize_mxfp8_weight, quantize_nvfp4_weight

    G = load("prep_mxfp8_weight_gpu.npz")
    w = bf16(G["w"]).to(DEV)
    q, sf, sd = quantize_mxfp8_weight(w, inference=False, fuse_swiglu=False)
    np.testing.assert_array_equal(q.cpu().numpy(), G["train_q"])
    np.testing.assert_array_equal(sf.cpu().numpy(), G["train_sf"].reshape(-1))
    np.testing.assert_array_equal(sd.cpu().numpy(), G["train_sd"].reshape(-1))
    q, sf, sd = quantize_mxfp8_weight(w, inference=True, fuse_swiglu=False)
    assert sd is None
    np.testing.assert_array_equal(q.cpu().numpy(), G["infer_q"])
    np.testing.assert_array_equal(sf.cpu().numpy(), G["infer_sf"].reshape(-1))
    q, sf, _ = quantize_mxfp8_weight(w, inference=True, fuse_swiglu=True)
    np.testing.assert_array_equal(q.cpu().numpy(), G["infer_fused_q"])
    np.testing.assert_array_equal(sf.cpu().numpy(), G["infer_fused_sf"].reshape(-1))

    G = load("quant_nvfp4_gpu.npz")
    for name, fuse in (("w13plain", False), ("w13", True)):
        q, s, gs, gsi = quantize_nvfp4_weight(bf16(G[name]).to(DEV), fuse_swiglu=fuse)
        np.testing.assert_array_equal(gs.cpu().numpy().view(np.uint32), G[f"{name}_gs"].view(np.uint32))
        np.testing.assert_array_equal(gsi.cpu().numpy().view(np.uint32), G[f"{name}_gsi"].view(np.uint32))
        np.testing.assert_array_equal(q.cpu().numpy(), G[f"{name}_q"])
        np.testing.assert_array_equal(s.cpu().numpy(), G[f"{name}_s"].reshape(-1))
    # [3, 160, 256]: rows not a multiple of 128, so through the kernel entry point with the recorded global scales
    nat = _nat()
    w = bf16(G["w"]).to(DEV)
    E, N, K = w.shape
    gs = torch.from_numpy(G["w_gs"]).to(DEV)
    q = torch.zeros(E, N, K // 2, dtype=torch.uint8, device=DEV)
    s = torch.zeros(G["w_s"].size, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_nvfp4_weight(w.data_ptr(), gs.data_ptr(), E, N, K, q.data_ptr(), s.data_ptr(), 1,
                                            nat.stream_ptr()), "nvfp4_weight")
    torch.cuda.synchronize()
    np.testing.assert_array_equal(q.cpu().numpy(), G["w_q"])
    np.testing.assert_array_equal(s.cpu().numpy(), G["w_s"].reshape(-1))


@pytest.mark.parametrize("file,names", [("quant_nvfp4_token_cute_gpu.npz", "tuv"), ("quant_nvfp4_gpu.npz", "tu")])
def test_nvfp4_token_kernel_equals_the_reference_bytes(file, names):
    nat, G = _nat(), load(file)
    for n in names:
        x = bf16(G[n]).to(DEV)
        rows, cols = x.shape
        q = torch.zeros(rows, cols // 2, dtype=torch.uint8, device=DEV)
        s = torch.zeros(rows, cols // 16, dtype=torch.uint8, device=DEV)
        inv = torch.zeros(rows, dtype=torch.float32, device=DEV)
        nat.check(nat.lib.dm_quant_nvfp4_token(x.data_ptr(), None, rows, cols, q.data_ptr(), cols // 2, s.data_ptr(),
                                               cols // 16, 0, inv.data_ptr(), 4, nat.stream_ptr()), "nvfp4_token")
        torch.cuda.synchronize()
        np.testing.assert_array_equal(inv.cpu().numpy().view(np.uint32), G[f"{n}_inv"].view(np.uint32))
        np.testing.assert_array_equal(s.cpu().numpy(), G[f"{n}_s"])
        np.testing.assert_array_equal(q.cpu().numpy(), G[f"{n}_q"])


# ---------------------------------------------------------------------------------------------------------------
# element-wise kernels: identical rounding points, so identical bf16 bits
# ---------------------------------------------------------------------------------------------------------------
def test_swiglu_and_topk_kernels_equal_the_reference_kernels():
    nat, G = _nat(), load("elementwise_gpu.npz")
    st = nat.stream_ptr()
    h1, dz = bf16(G["h1"]).to(DEV), bf16(G["dz"]).to(DEV)
    rows, F = dz.shape
    cnt = torch.tensor([rows], dtype=torch.int32, device=DEV)
    for name, clamped in (("plain", 0), ("clamped", 1)):
        z = torch.zeros(rows, F, dtype=torch.bfloat16, device=DEV)
        dxy = torch.zeros(rows, 2 * F, dtype=torch.bfloat16, device=DEV)
        nat.check(nat.lib.dm_swiglu_fwd(h1.data_ptr(), None, z.data_ptr(), None, cnt.data_ptr(), rows, F, clamped, 1.702, 7.0,
                                        None, 0.0, None, st), "swiglu_fwd")
        nat.check(nat.lib.dm_swiglu_bwd(h1.data_ptr(), None, dz.data_ptr(), None, dxy.data_ptr(), None, cnt.data_ptr(), rows,
                                        F, clamped, 1.702, 7.0, st), "swiglu_bwd")
        torch.cuda.synchronize()
        assert torch.equal(z.cpu(), bf16(G[f"z_{name}"])), name
        assert torch.equal(dxy.cpu(), bf16(G[f"dxy_{name}"])), name
    x, dy = bf16(G["x"]).to(DEV), bf16(G["dy"]).to(DEV)
    sc, ids = torch.from_numpy(G["scale"]).to(DEV), torch.from_numpy(G["ids"]).to(DEV)
    T, K, D = x.shape
    y = torch.zeros(T, D, dtype=torch.bfloat16, device=DEV)
    r = torch.zeros(T, D, dtype=torch.bfloat16, device=DEV)
    nat.check(nat.lib.dm_scale_and_sum(x.data_ptr(), sc.data_ptr(), 0, ids.data_ptr(), 1, y.data_ptr(), T, K, D, None, None,
                                       None, 0, st), "scale_and_sum")
    nat.check(nat.lib.dm_scale_and_sum(x.data_ptr(), None, 0, ids.data_ptr(), 1, r.data_ptr(), T, K, D, None, None, None, 0,
                                       st), "reduce_from_topk")
    dx = torch.full((T, K, D), 7.0, dtype=torch.bfloat16, device=DEV)
    ds = torch.zeros(T, K, dtype=torch.float32, device=DEV)
    nat.check(nat.lib.dm_broadcast_and_scale(dy.data_ptr(), sc.data_ptr(), 0, ids.data_ptr(), 1, x.data_ptr(), None,
                                             dx.data_ptr(), ds.data_ptr(), T, K, D, st), "broadcast_and_scale")
    torch.cuda.synchronize()
    assert torch.equal(y.cpu(), bf16(G["y"]))
    assert torch.equal(r.cpu(), bf16(G["r"]))
    valid = (ids >= 0).cpu()
    assert torch.equal(dx.cpu()[valid], bf16(G["dx"])[valid])
    ref_ds = torch.from_numpy(G["dscale"])
    assert (ds.cpu()[~valid] == 0).all() and (ref_ds[~valid] == 0).all()
    torch.testing.assert_close(ds.cpu(), ref_ds, rtol=1e-5, atol=1e-4)  # fp32 sum over D in another order


# ---------------------------------------------------------------------------------------------------------------
# whole layer
# ---------------------------------------------------------------------------------------------------------------
def layer_inputs(T, D, F, E, K, seed, w_std):
    """Inputs of the recorded end-to-end runs (the generator's ``_e2e_inputs``; CPU generator, so reproducible)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g)
    top = torch.topk(torch.softmax(logits, -1), K, dim=-1)
    scores = (top.values / top.values.sum(-1, keepdim=True)).float()
    ids = top.indices.to(torch.int64)
    w13 = (torch.randn(E, 2 * F, D, generator=g) * w_std).bfloat16()
    w2 = (torch.randn(E, D, F, generator=g) * w_std).bfloat16()
    return x, ids, scores, w13, w2


def closeness(got, ref):
    got, ref = got.detach().float().cpu(), ref.detach().float().cpu()
    l2 = ((got - ref).norm() / ref.norm().clamp_min(1e-30)).item()
    cos = torch.nn.functional.cosine_similarity(got.flatten(), ref.flatten(), dim=0).item()
    same = (got == ref).float().mean().item()
    return l2, cos, same


def _bf16_layer(T, D, F, E, K, w_std):
    dm = _dm()
    x, ids, scores, w13, w2 = [t.to(DEV) for t in layer_inputs(T, D, F, E, K, 1000, w_std)]
    for t in (x, scores, w13, w2):
        t.requires_grad_(True)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, device_scratch_capacity_factor=1.0,
                    activation_slot_capacity_factor=1.0, num_activation_slots=1)
    ctx = dm.create_context(group=None, config=cfg, device=torch.device(DEV))
    try:
        out = dm.routed_experts(x, ids, scores, w13, w2, ctx)
        out.float().sum().backward()
        ctx.check_status()
    finally:
        ctx.close()
    return out, x, scores, w13, w2


@pytest.mark.parametrize("tag,T,D,F,E,K,w_std", [("small", 192, 256, 256, 4, 2, 1.0), ("c2", 4096, 2048, 1408, 64, 6, 0.02)])
def test_bf16_layer_equals_the_reference_layer(tag, T, D, F, E, K, w_std):
    """Forward + backward of ``routed_experts`` against the reference's own ``routed_experts`` on the same seeded
    inputs (one rank): the small case in full, the BF16 training configuration (T=4096, D=2048, F=1408, E=64, K=6) on
    the recorded sample (64 tokens; 64 rows of two experts' weight gradients)."""
    G = load(f"e2e_bf16_{tag}_gpu.npz")
    assert list(G["shape"]) == [T, D, F, E, K]
    if "x" in G.files:  # the generator's inputs really are what this test regenerates
        assert torch.equal(bf16(G["x"]), layer_inputs(T, D, F, E, K, 1000, w_std)[0])
    out, x, scores, w13, w2 = _bf16_layer(T, D, F, E, K, w_std)
    n = G["out"].shape[0]
    pairs = [("out", out[:n], bf16(G["out"]), 2e-2, 0.999), ("grad_x", x.grad[:n], bf16(G["gx"]), 3e-2, 0.995),
             ("grad_scores", scores.grad[:n], torch.from_numpy(G["gs"]), 3e-2, 0.995),
             ("grad_w13[0]", w13.grad[0, :64], bf16(G["gw13_e0"]), 1.5e-2, 0.995),
             ("grad_w2[0]", w2.grad[0, :64], bf16(G["gw2_e0"]), 1.5e-2, 0.995),
             ("grad_w13[-1]", w13.grad[E - 1, -64:], bf16(G["gw13_last"]), 1.5e-2, 0.995),
             ("grad_w2[-1]", w2.grad[E - 1, -64:], bf16(G["gw2_last"]), 1.5e-2, 0.995)]
    for name, got, ref, bound_l2, bound_cos in pairs:
        l2, cos, same = closeness(got, ref)
        assert l2 < bound_l2 and cos > bound_cos, (tag, name, l2, cos)
        # two implementations of the same rounding points differ by fp32 summation order only
        assert l2 < 4e-3, (tag, name, l2)
        if name != "grad_scores":
            assert same > 0.5, (tag, name, same)


def test_mxfp8_training_layer_equals_the_reference_layer():
    """MXFP8 forward + backward against the reference's staged MXFP8 path on the recorded inputs.  Both quantise to the
    same bytes, so the difference is accumulation order inside the block-scaled GEMMs."""
    dm = _dm()
    G = load("e2e_mxfp8_train_gpu.npz")
    T, D, F, E, K = [int(v) for v in G["shape"]]
    x, w13, w2 = bf16(G["x"]).to(DEV), bf16(G["w13"]).to(DEV), bf16(G["w2"]).to(DEV)
    ids, scores = torch.from_numpy(G["ids"]).to(DEV), torch.from_numpy(G["scores"]).to(DEV)
    for t in (x, scores, w13, w2):
        t.requires_grad_(True)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, device_scratch_capacity_factor=1.0,
                    activation_slot_capacity_factor=1.0, num_activation_slots=1, block_scaled=dm.BlockScaledConfig())
    ctx = dm.create_context(group=None, config=cfg, device=torch.device(DEV))
    try:
        out = dm.routed_experts(x, ids, scores, w13, w2, ctx)
        out.float().sum().backward()
        ctx.check_status()
    finally:
        ctx.close()
    for name, got, ref in (("out", out, bf16(G["out"])), ("grad_x", x.grad, bf16(G["gx"])),
                           ("grad_w13", w13.grad, bf16(G["gw13"])), ("grad_w2", w2.grad, bf16(G["gw2"]))):
        l2, cos, same = closeness(got, ref)
        assert l2 < 0.02 and cos > 0.9995, (name, l2, cos, same)


def test_nvfp4_inference_layer_equals_the_reference_layer():
    dm = _dm()
    G = load("e2e_nvfp4_infer_gpu.npz")
    T, D, F, E, K = [int(v) for v in G["shape"]]
    x, w13, w2 = bf16(G["x"]).to(DEV), bf16(G["w13"]).to(DEV), bf16(G["w2"]).to(DEV)
    ids, scores = torch.from_numpy(G["ids"]).to(DEV), torch.from_numpy(G["scores"]).to(DEV)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0,
                    block_scaled=dm.BlockScaledConfig(format=dm.BlockScaledFormat.NVFP4))
    ctx = dm.create_context(group=None, config=cfg, device=torch.device(DEV))
    try:
        for fuse in (False, True):
            p13 = dm.prepare_block_scaled_weight(w13, cfg, inference=True, fuse_swiglu=fuse)
            p2 = dm.prepare_block_scaled_weight(w2, cfg, inference=True)
            with torch.no_grad():
                out = dm.routed_experts(x, ids, scores, p13, p2, ctx)
            ctx.check_status()
            l2, cos, same = closeness(out, bf16(G["out"]))
            assert l2 < 0.02 and cos > 0.9995, (fuse, l2, cos, same)
    finally:
        ctx.close()
