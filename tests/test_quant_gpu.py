"""CUDA quantisers through the C ABI, bit-exact against the CPU oracle (`oracle/quant.py`), which
is itself held to the reference's Triton quantiser for MXFP8.  Sizes up to the full C3 row width."""

import numpy as np
import pytest
import torch

from oracle import quant as Q

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _nat():
    from dist_moe_b200 import _native

    return _native


def _data(rows, cols, seed, spread=True, specials=True):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(rows, cols, generator=g)
    if spread:
        x = x * torch.logspace(-4, 3, rows)[:, None]
    x = x.bfloat16()
    if specials and rows > 4:
        x[0, :32] = 0
        x[1, 7] = float("inf")
        x[2, 40] = float("nan")
        x[3, :32] = 448.0
    return x


@pytest.mark.parametrize("rows,cols,blocked", [(37, 256, 0), (200, 384, 1), (1000, 4096, 1), (1, 32, 0)])
def test_mxfp8_row(rows, cols, blocked):
    nat = _nat()
    x = _data(rows, cols, rows)
    xd = x.to(DEV)
    q = torch.zeros(rows, cols, dtype=torch.uint8, device=DEV)
    sc = cols // 32
    atoms = (sc + 3) // 4
    n_s = ((rows + 127) // 128 * 128) * atoms * 4 if blocked else rows * sc
    s = torch.full((n_s,), 0xEE, dtype=torch.uint8, device=DEV)
    cnt = torch.tensor([rows], dtype=torch.int32, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_row(xd.data_ptr(), cnt.data_ptr(), rows, cols, q.data_ptr(), 0, s.data_ptr(), 0, blocked,
                                         nat.stream_ptr()), "mxfp8_row")
    torch.cuda.synchronize()
    rq, rs = Q.mxfp8_row(x)
    got_s = s.cpu().numpy()
    if blocked:
        r, c = np.meshgrid(np.arange(rows), np.arange(sc), indexing="ij")
        got_s = got_s[Q.blocked_scale_offset(r, c, atoms)]
    else:
        got_s = got_s.reshape(rows, sc)
    np.testing.assert_array_equal(got_s, rs)
    finite = np.repeat(rs != 255, 32, axis=1)
    gq = q.cpu().numpy()
    np.testing.assert_array_equal(gq[finite], rq[finite])
    assert ((gq[~finite] & 0x7F) == 0x7F).all()


@pytest.mark.parametrize("rows,cols", [(96, 64), (333, 520), (4096, 1536)])
def test_mxfp8_col(rows, cols):
    nat = _nat()
    x = _data(rows, cols, rows + 1, specials=False)
    q = torch.zeros(rows, cols, dtype=torch.uint8, device=DEV)
    rb = (rows + 31) // 32
    s = torch.zeros(cols * rb, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_col(x.to(DEV).data_ptr(), None, rows, cols, q.data_ptr(), s.data_ptr(), 0,
                                         nat.stream_ptr()), "mxfp8_col")
    torch.cuda.synchronize()
    rq, rs = Q.mxfp8_col(x)
    np.testing.assert_array_equal(s.cpu().numpy().reshape(cols, rb), rs)
    np.testing.assert_array_equal(q.cpu().numpy(), rq)


@pytest.mark.parametrize("experts,n,k,blocked", [(2, 64, 96, 0), (3, 256, 512, 1)])
def test_mxfp8_tile32_weights(experts, n, k, blocked):
    nat = _nat()
    w = _data(experts * n, k, 11, spread=False, specials=False) * 0.02
    w = w.bfloat16()
    q = torch.zeros(experts * n, k, dtype=torch.uint8, device=DEV)
    a0, a1 = (k // 32 + 3) // 4, (n // 32 + 3) // 4
    g0 = (n + 127) // 128 * 128 * a0 * 4 if blocked else n * (k // 32)
    g1 = (k + 127) // 128 * 128 * a1 * 4 if blocked else k * (n // 32)
    s0 = torch.zeros(experts * g0, dtype=torch.uint8, device=DEV)
    s1 = torch.zeros(experts * g1, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_tile32(w.to(DEV).data_ptr(), experts, n, k, q.data_ptr(), s0.data_ptr(),
                                            s1.data_ptr(), blocked, nat.stream_ptr()), "tile32")
    torch.cuda.synchronize()
    gq, g0s, g1s = q.cpu().numpy(), s0.cpu().numpy().reshape(experts, -1), s1.cpu().numpy().reshape(experts, -1)
    for e in range(experts):
        rq, rs = Q.mxfp8_tile32(w[e * n:(e + 1) * n])
        np.testing.assert_array_equal(gq[e * n:(e + 1) * n], rq)
        row_s = np.repeat(rs, 32, axis=0)            # [n, k/32]
        col_s = np.repeat(rs.T, 32, axis=0)          # [k, n/32]
        if blocked:
            r, c = np.meshgrid(np.arange(n), np.arange(k // 32), indexing="ij")
            np.testing.assert_array_equal(g0s[e][Q.blocked_scale_offset(r, c, a0)], row_s)
            r, c = np.meshgrid(np.arange(k), np.arange(n // 32), indexing="ij")
            np.testing.assert_array_equal(g1s[e][Q.blocked_scale_offset(r, c, a1)], col_s)
        else:
            np.testing.assert_array_equal(g0s[e].reshape(n, k // 32), row_s)
            np.testing.assert_array_equal(g1s[e].reshape(k, n // 32), col_s)


@pytest.mark.parametrize("rows,cols", [(33, 256), (128, 7168), (5, 2880 - 2880 % 16)])
def test_nvfp4_token_dense_and_packed_rows(rows, cols):
    nat = _nat()
    x = _data(rows, cols, rows + 2, specials=False)
    xd = x.to(DEV)
    rp, rs, rinv = Q.nvfp4_token_rows(x)
    # dense outputs
    q = torch.zeros(rows, cols // 2, dtype=torch.uint8, device=DEV)
    s = torch.zeros(rows, cols // 16, dtype=torch.uint8, device=DEV)
    inv = torch.zeros(rows, dtype=torch.float32, device=DEV)
    nat.check(nat.lib.dm_quant_nvfp4_token(xd.data_ptr(), None, rows, cols, q.data_ptr(), cols // 2, s.data_ptr(),
                                           cols // 16, 0, inv.data_ptr(), 4, nat.stream_ptr()), "nvfp4_token")
    torch.cuda.synchronize()
    np.testing.assert_array_equal(inv.cpu().numpy().view(np.uint32), rinv.view(np.uint32))
    np.testing.assert_array_equal(s.cpu().numpy(), rs)
    np.testing.assert_array_equal(q.cpu().numpy(), rp)
    # packed dispatch row [q | scales | inv | pad16]: bit-identical to the dense call
    stride = (cols // 2 + cols // 16 + 4 + 15) // 16 * 16
    packed = torch.zeros(rows, stride, dtype=torch.uint8, device=DEV)
    base = packed.data_ptr()
    nat.check(nat.lib.dm_quant_nvfp4_token(xd.data_ptr(), None, rows, cols, base, stride, base + cols // 2, stride, 0,
                                           base + cols // 2 + cols // 16, stride, nat.stream_ptr()), "nvfp4_token")
    torch.cuda.synchronize()
    p = packed.cpu().numpy()
    np.testing.assert_array_equal(p[:, : cols // 2], rp)
    np.testing.assert_array_equal(p[:, cols // 2 : cols // 2 + cols // 16], rs)
    got_inv = np.ascontiguousarray(p[:, cols // 2 + cols // 16 : cols // 2 + cols // 16 + 4]).view(np.uint32)[:, 0]
    np.testing.assert_array_equal(got_inv, rinv.view(np.uint32))


def test_nvfp4_weight_and_swizzle():
    nat = _nat()
    experts, n, k = 3, 160, 256
    g = torch.Generator().manual_seed(7)
    w = (torch.randn(experts, n, k, generator=g) * 0.02).bfloat16()
    rp, rs, gs, gsi = Q.nvfp4_weight(w)
    wd = w.to(DEV)
    amax = torch.linalg.vector_norm(wd, ord=float("inf"), dim=(-2, -1), dtype=torch.float32).clamp(min=1e-12)
    gsd = 2688.0 * torch.reciprocal(amax)
    np.testing.assert_array_equal(gsd.cpu().numpy().view(np.uint32), gs.view(np.uint32))
    q = torch.zeros(experts, n, k // 2, dtype=torch.uint8, device=DEV)
    s = torch.zeros(experts * n, k // 16, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_nvfp4_weight(wd.data_ptr(), gsd.data_ptr(), experts, n, k, q.data_ptr(), s.data_ptr(), 0,
                                            nat.stream_ptr()), "nvfp4_weight")
    torch.cuda.synchronize()
    np.testing.assert_array_equal(s.cpu().numpy().reshape(experts, n, k // 16), rs)
    np.testing.assert_array_equal(q.cpu().numpy(), rp)
    # swizzle natural -> blocked equals the oracle's layout, padding zeroed
    sw = torch.full(((n + 127) // 128 * 128 * 4 * 4,), 0xEE, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_sf_swizzle(s[:n].contiguous().data_ptr(), sw.data_ptr(), n, k // 16, nat.stream_ptr()), "swz")
    torch.cuda.synchronize()
    np.testing.assert_array_equal(sw.cpu().numpy(), Q.to_blocked(rs[0]))


@pytest.mark.parametrize("rows,cols,cap", [(96, 64, 128), (333, 512, 384), (4096, 1536, 4096)])
def test_mxfp8_rowcol_equals_the_separate_kernels(rows, cols, cap):
    """One pass producing both copies is bit-identical to the row kernel (blocked scales) and the column kernel
    (blocked scales), which are held to the oracle above."""
    nat = _nat()
    x = _data(rows, cols, rows + 3, specials=False).to(DEV)
    cnt = torch.tensor([rows], dtype=torch.int32, device=DEV)
    ra, ca = (cols // 32 + 3) // 4, ((cap + 31) // 32 + 3) // 4
    n_rs, n_cs = (cap + 127) // 128 * 128 * ra * 4, (cols + 127) // 128 * 128 * ca * 4
    st = nat.stream_ptr()
    q_r = torch.zeros(cap, cols, dtype=torch.uint8, device=DEV)
    s_r = torch.zeros(n_rs, dtype=torch.uint8, device=DEV)
    q_c = torch.zeros(cap, cols, dtype=torch.uint8, device=DEV)
    s_c = torch.zeros(n_cs, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_row(x.data_ptr(), cnt.data_ptr(), cap, cols, q_r.data_ptr(), 0, s_r.data_ptr(), 0, 1, st), "row")
    nat.check(nat.lib.dm_quant_mxfp8_col(x.data_ptr(), cnt.data_ptr(), cap, cols, q_c.data_ptr(), s_c.data_ptr(), 1, st), "col")
    f_r, fs_r, f_c, fs_c = (torch.zeros_like(t) for t in (q_r, s_r, q_c, s_c))
    nat.check(nat.lib.dm_quant_mxfp8_rowcol(x.data_ptr(), cnt.data_ptr(), cap, cols, f_r.data_ptr(), fs_r.data_ptr(),
                                            f_c.data_ptr(), fs_c.data_ptr(), st), "rowcol")
    torch.cuda.synchronize()
    assert torch.equal(f_r, q_r) and torch.equal(f_c, q_c)
    assert torch.equal(fs_c, s_c)
    # row scales: compare the entries of real rows (the row kernel leaves other positions untouched as well)
    r, c = np.meshgrid(np.arange(rows), np.arange(cols // 32), indexing="ij")
    idx = Q.blocked_scale_offset(r, c, ra)
    np.testing.assert_array_equal(fs_r.cpu().numpy()[idx], s_r.cpu().numpy()[idx])


@pytest.mark.parametrize("rows,cols,cap", [(96, 512, 128), (200, 1536, 256)])
def test_mxfp8_rowcol_with_gather_and_with_swiglu_equal_the_staged_forms(rows, cols, cap):
    """The quantiser that pulls rows through a pointer table, and the one that applies SwiGLU to h1 first, give the
    bytes of gather -> quantise and SwiGLU -> quantise run as separate kernels."""
    nat = _nat()
    st = nat.stream_ptr()
    cnt = torch.tensor([rows], dtype=torch.int32, device=DEV)
    ra, ca = (cols // 32 + 3) // 4, ((cap + 31) // 32 + 3) // 4
    n_rs, n_cs = (cap + 127) // 128 * 128 * ra * 4, (cols + 127) // 128 * 128 * ca * 4

    def outputs():
        return (torch.zeros(cap, cols, dtype=torch.uint8, device=DEV), torch.zeros(n_rs, dtype=torch.uint8, device=DEV),
                torch.zeros(cap, cols, dtype=torch.uint8, device=DEV), torch.zeros(n_cs, dtype=torch.uint8, device=DEV))

    # --- gather: a permutation of source rows with every seventh pointer null
    src = _data(rows, cols, rows + 11, specials=False).to(DEV)
    perm = torch.randperm(rows, generator=torch.Generator().manual_seed(rows))
    ptrs = torch.tensor([0 if i % 7 == 3 else src.data_ptr() + int(perm[i]) * cols * 2 for i in range(rows)],
                        dtype=torch.int64, device=DEV)
    dense = src[perm.to(DEV)].clone()
    dense[torch.arange(rows, device=DEV) % 7 == 3] = 0
    want = outputs()
    nat.check(nat.lib.dm_quant_mxfp8_rowcol(dense.data_ptr(), cnt.data_ptr(), cap, cols, want[0].data_ptr(),
                                            want[1].data_ptr(), want[2].data_ptr(), want[3].data_ptr(), st), "rowcol")
    got = outputs()
    nat.check(nat.lib.dm_quant_mxfp8_rowcol_gather(ptrs.data_ptr(), cnt.data_ptr(), cap, cols, got[0].data_ptr(),
                                                   got[1].data_ptr(), got[2].data_ptr(), got[3].data_ptr(), st), "gather")
    torch.cuda.synchronize()
    for g, w in zip(got, want):
        assert torch.equal(g, w)

    # --- SwiGLU (plain and clamped) of h1 = [gate | up]
    for clamped in (0, 1):
        h1 = (torch.randn(rows, 2 * cols, generator=torch.Generator().manual_seed(5 + clamped)) * 3).bfloat16().to(DEV)
        h2 = torch.zeros(rows, cols, dtype=torch.bfloat16, device=DEV)
        nat.check(nat.lib.dm_swiglu_fwd(h1.data_ptr(), None, h2.data_ptr(), None, cnt.data_ptr(), rows, cols, clamped, 1.702,
                                        7.0, None, 0.0, None, st), "swiglu")
        want = outputs()
        nat.check(nat.lib.dm_quant_mxfp8_rowcol(h2.data_ptr(), cnt.data_ptr(), cap, cols, want[0].data_ptr(),
                                                want[1].data_ptr(), want[2].data_ptr(), want[3].data_ptr(), st), "rowcol")
        got = outputs()
        nat.check(nat.lib.dm_swiglu_fwd_quant_mxfp8_rowcol(h1.data_ptr(), cnt.data_ptr(), cap, cols, clamped, 1.702, 7.0,
                                                           got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(),
                                                           got[3].data_ptr(), st), "swiglu+quant")
        torch.cuda.synchronize()
        for g, w in zip(got, want):
            assert torch.equal(g, w)


@pytest.mark.parametrize("rows,F,cap,clamped", [(96, 512, 128, 0), (200, 1536, 256, 1), (70, 96, 128, 0)])
def test_swiglu_backward_fused_into_the_quantiser_equals_the_staged_form(rows, F, cap, clamped):
    """dm_swiglu_bwd_quant_mxfp8 gives the bytes of dm_swiglu_bwd followed by the row+column quantiser, and leaves
    out the copy that is not asked for."""
    nat = _nat()
    st = nat.stream_ptr()
    cnt = torch.tensor([rows], dtype=torch.int32, device=DEV)
    C = 2 * F
    ra, ca = (C // 32 + 3) // 4, ((cap + 31) // 32 + 3) // 4
    n_rs, n_cs = (cap + 127) // 128 * 128 * ra * 4, (C + 127) // 128 * 128 * ca * 4

    def outputs():
        return (torch.zeros(cap, C, dtype=torch.uint8, device=DEV), torch.zeros(n_rs, dtype=torch.uint8, device=DEV),
                torch.zeros(cap, C, dtype=torch.uint8, device=DEV), torch.zeros(n_cs, dtype=torch.uint8, device=DEV))

    g = torch.Generator().manual_seed(31 + rows)
    h1 = (torch.randn(rows, C, generator=g) * 4).bfloat16().to(DEV)
    dz = (torch.randn(rows, F, generator=g) * torch.logspace(-3, 2, rows)[:, None]).bfloat16().to(DEV)
    dh1 = torch.zeros(rows, C, dtype=torch.bfloat16, device=DEV)
    nat.check(nat.lib.dm_swiglu_bwd(h1.data_ptr(), None, dz.data_ptr(), None, dh1.data_ptr(), None, cnt.data_ptr(), rows, F,
                                    clamped, 1.702, 7.0, st), "swiglu_bwd")
    want = outputs()
    nat.check(nat.lib.dm_quant_mxfp8_rowcol(dh1.data_ptr(), cnt.data_ptr(), cap, C, want[0].data_ptr(), want[1].data_ptr(),
                                            want[2].data_ptr(), want[3].data_ptr(), st), "rowcol")
    got = outputs()
    nat.check(nat.lib.dm_swiglu_bwd_quant_mxfp8(h1.data_ptr(), dz.data_ptr(), cnt.data_ptr(), cap, F, clamped, 1.702, 7.0,
                                                got[0].data_ptr(), got[1].data_ptr(), got[2].data_ptr(), got[3].data_ptr(),
                                                st), "fused")
    only_row, only_col = outputs(), outputs()
    nat.check(nat.lib.dm_swiglu_bwd_quant_mxfp8(h1.data_ptr(), dz.data_ptr(), cnt.data_ptr(), cap, F, clamped, 1.702, 7.0,
                                                only_row[0].data_ptr(), only_row[1].data_ptr(), None, None, st), "row only")
    nat.check(nat.lib.dm_swiglu_bwd_quant_mxfp8(h1.data_ptr(), dz.data_ptr(), cnt.data_ptr(), cap, F, clamped, 1.702, 7.0,
                                                None, None, only_col[2].data_ptr(), only_col[3].data_ptr(), st), "col only")
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a, b)
    assert torch.equal(only_row[0], want[0]) and torch.equal(only_row[1], want[1]) and not only_row[2].any()
    assert torch.equal(only_col[2], want[2]) and torch.equal(only_col[3], want[3]) and not only_col[0].any()


@pytest.mark.parametrize("rows,cols", [(96, 2048), (40, 7168)])
def test_nvfp4_token_live_rows_only(rows, cols):
    """dm_quant_nvfp4_token_live quantises the rows whose table entry is non-zero exactly as the plain call does
    and leaves the others untouched."""
    nat = _nat()
    st = nat.stream_ptr()
    x = _data(rows, cols, rows + 5, specials=False).to(DEV)
    live = torch.tensor([0 if r % 3 == 1 else 1000 + r for r in range(rows)], dtype=torch.int64, device=DEV)

    def outputs(fill):
        return (torch.full((rows, cols // 2), fill, dtype=torch.uint8, device=DEV),
                torch.full((rows, cols // 16), fill, dtype=torch.uint8, device=DEV),
                torch.full((rows,), float(fill), dtype=torch.float32, device=DEV))

    want, got = outputs(0), outputs(0xAB)
    nat.check(nat.lib.dm_quant_nvfp4_token(x.data_ptr(), None, rows, cols, want[0].data_ptr(), cols // 2, want[1].data_ptr(),
                                           cols // 16, 0, want[2].data_ptr(), 4, st), "plain")
    nat.check(nat.lib.dm_quant_nvfp4_token_live(live.data_ptr(), x.data_ptr(), None, rows, cols, got[0].data_ptr(), cols // 2,
                                                got[1].data_ptr(), cols // 16, 0, got[2].data_ptr(), 4, st), "live")
    torch.cuda.synchronize()
    keep = live != 0
    for g, w in zip(got, want):
        assert torch.equal(g[keep], w[keep])
    assert bool((got[0][~keep] == 0xAB).all()) and bool((got[1][~keep] == 0xAB).all())
    assert bool((got[2][~keep] == float(0xAB)).all())
