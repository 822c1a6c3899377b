"""Grouped BF16 GEMMs (tcgen05) through the C ABI against torch fp32 matmuls.

Tolerance: the kernels accumulate in fp32 and round once to bf16, so a result
may differ from the fp32 reference by bf16 rounding of the reference value:
|diff| <= 2^-7 * |ref| + 1e-3 * scale (scale = rms of the reference).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _native():
    from dist_moe_b200 import _native

    return _native


def _close(got, ref, what):
    got = got.float()
    ref = ref.float()
    scale = ref.pow(2).mean().sqrt().item() + 1e-6
    err = (got - ref).abs()
    bound = ref.abs() * 2.0**-7 + 2e-3 * scale
    bad = err > bound
    assert not bool(bad.any()), (
        f"{what}: {int(bad.sum())} of {bad.numel()} elements out of tolerance; "
        f"max err {err.max().item():.4g}, scale {scale:.4g}, first bad idx {bad.nonzero()[:4].tolist()}"
    )


def _arena(nbytes, dev):
    return torch.zeros(nbytes, dtype=torch.uint8, device=dev)


def _place(arena, offset, t):
    flat = t.contiguous().view(torch.uint8).reshape(-1)
    arena[offset : offset + flat.numel()] = flat


def _view(arena, offset, shape, dtype=torch.bfloat16):
    n = 1
    for s in shape:
        n *= s
    nbytes = n * torch.tensor([], dtype=dtype).element_size()
    return arena[offset : offset + nbytes].view(dtype).reshape(shape)


def _offsets(counts, dev):
    off = [0]
    for c in counts:
        off.append(off[-1] + c)
    return torch.tensor(off, dtype=torch.int32, device=dev), off


CASES = [
    # counts per expert, Kd, N
    ([200, 0, 333], 256, 512),
    ([1, 127, 128, 129], 64, 256),
    ([700], 512, 768),
    ([513, 31, 0, 260], 256, 320),   # feature count a multiple of 64 only; chunks of 192 / 32 / 160 rows
    ([40, 1000], 128, 1408),         # 5.5 feature blocks of 256
]


@pytest.mark.parametrize("counts,kd,n", CASES)
def test_fprop_matches_torch(counts, kd, n):
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(1)
    e = len(counts)
    offs_t, off = _offsets(counts, dev)
    rows = off[-1]
    a = torch.randn(rows, kd, device=dev).bfloat16()
    w = (torch.randn(e, n, kd, device=dev) * 0.1).bfloat16()
    a_off, c_off = 128 * 5, 128 * 5 + ((rows + 300) * kd * 2 + 127) // 128 * 128 + 384
    total = c_off + (rows + 300) * n * 2 + 4096
    arena = _arena(total, dev)
    _place(arena, a_off, a)
    sentinel = torch.full((rows + 16, n), 7.0, device=dev).bfloat16()
    _place(arena, c_off, sentinel)
    offs_dev = torch.tensor([a_off, c_off], dtype=torch.int64, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    none = nat.Operand(None, 0, None)
    rc = nat.lib.dm_gemm_fprop(
        nat.Operand(arena.data_ptr(), arena.numel(), offs_dev[0:1].data_ptr()),
        w.data_ptr(),
        nat.Operand(arena.data_ptr(), arena.numel(), offs_dev[1:2].data_ptr()),
        none, None, offs_t.data_ptr(), e, rows, n, kd, 0, 0, 1.0, 0.0, None, 0, status.data_ptr(), nat.stream_ptr(),
    )
    nat.check(rc, "dm_gemm_fprop")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    got = _view(arena, c_off, (rows + 16, n))
    for ei in range(e):
        lo, hi = off[ei], off[ei + 1]
        if hi > lo:
            _close(got[lo:hi], a[lo:hi].float() @ w[ei].float().T, f"fprop expert {ei}")
    assert torch.equal(got[rows:], sentinel[rows:]), "rows past the last expert were overwritten"


@pytest.mark.parametrize("counts,kd,n", [([200, 0, 333], 256, 512), ([90, 300], 128, 256)])
def test_fprop_fused_swiglu(counts, kd, n):
    """n is 2F; W13 = [e, 2, F, kd]; writes h1 and h2 = bf16(swiglu(bf16 gate, bf16 up))."""
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(2)
    e = len(counts)
    f = n // 2
    offs_t, off = _offsets(counts, dev)
    rows = off[-1]
    a = torch.randn(rows, kd, device=dev).bfloat16()
    w = (torch.randn(e, n, kd, device=dev) * 0.1).bfloat16()
    a_off = 256
    c_off = a_off + ((rows + 300) * kd * 2 + 127) // 128 * 128
    h2_off = c_off + ((rows + 300) * n * 2 + 127) // 128 * 128
    arena = _arena(h2_off + (rows + 300) * f * 2, dev)
    _place(arena, a_off, a)
    offs_dev = torch.tensor([a_off, c_off, h2_off], dtype=torch.int64, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    for clamped in (0, 1):
        rc = nat.lib.dm_gemm_fprop(
            nat.Operand(arena.data_ptr(), arena.numel(), offs_dev[0:1].data_ptr()),
            w.data_ptr(),
            nat.Operand(arena.data_ptr(), arena.numel(), offs_dev[1:2].data_ptr()),
            nat.Operand(arena.data_ptr(), arena.numel(), offs_dev[2:3].data_ptr()),
            None, offs_t.data_ptr(), e, rows, n, kd, 1, clamped, 1.702, 7.0, None, 0, status.data_ptr(), nat.stream_ptr(),
        )
        nat.check(rc, "dm_gemm_fprop fused")
        torch.cuda.synchronize()
        assert status[0].item() == 0, status.tolist()
        h1 = _view(arena, c_off, (rows, n))
        h2 = _view(arena, h2_off, (rows, f))
        for ei in range(e):
            lo, hi = off[ei], off[ei + 1]
            if hi == lo:
                continue
            _close(h1[lo:hi], a[lo:hi].float() @ w[ei].float().T, f"h1 expert {ei}")
            g, u = h1[lo:hi, :f].float(), h1[lo:hi, f:].float()
            if clamped:
                g = g.clamp(max=7.0)
                u = u.clamp(-7.0, 7.0)
                ref = g * torch.sigmoid(1.702 * g) * (u + 1.0)
            else:
                ref = g * torch.sigmoid(g) * u
            _close(h2[lo:hi], ref, f"h2 expert {ei} clamped={clamped}")


@pytest.mark.parametrize("counts,kd,n", CASES)
def test_dgrad_matches_torch(counts, kd, n):
    """C[r, n] = sum_k A[r, k] W[e][k][n] with W stored [e, kd, n]."""
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    e = len(counts)
    offs_t, off = _offsets(counts, dev)
    rows = off[-1]
    a = torch.randn(rows, kd, device=dev).bfloat16()
    w = (torch.randn(e, kd, n, device=dev) * 0.1).bfloat16()
    arena = _arena(128 + (rows + 300) * kd * 2, dev)
    _place(arena, 128, a)
    a_off = torch.tensor([128], dtype=torch.int64, device=dev)
    out = torch.zeros(rows, n, device=dev, dtype=torch.bfloat16)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    rc = nat.lib.dm_gemm_dgrad(
        nat.Operand(arena.data_ptr(), arena.numel(), a_off.data_ptr()),
        w.data_ptr(),
        nat.Operand(out.data_ptr(), out.numel() * 2, None),
        None, offs_t.data_ptr(), e, rows, n, kd, None, 0, status.data_ptr(), nat.stream_ptr(),
    )
    nat.check(rc, "dm_gemm_dgrad")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    for ei in range(e):
        lo, hi = off[ei], off[ei + 1]
        if hi > lo:
            _close(out[lo:hi], a[lo:hi].float() @ w[ei].float(), f"dgrad expert {ei}")


@pytest.mark.parametrize("counts,kd,n", [([200, 0, 333], 256, 384), ([1, 63, 64, 65], 64, 128), ([700], 512, 256)])
@pytest.mark.parametrize("fp32_out", [0, 1])
def test_wgrad_matches_torch(counts, kd, n, fp32_out):
    """dW[e][n][k] (+)= sum_r dY[r, n] X[r, k]; ragged row counts, empty experts, accumulation."""
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(4)
    e = len(counts)
    offs_t, off = _offsets(counts, dev)
    rows = off[-1]
    dy = torch.randn(rows, n, device=dev).bfloat16()
    x = torch.randn(rows, kd, device=dev).bfloat16()
    dy_off = 384
    x_off = dy_off + ((rows + 300) * n * 2 + 127) // 128 * 128
    arena = _arena(x_off + (rows + 300) * kd * 2, dev)
    # Poison everything (NaN bit patterns) so that a chunk row leaking in from a neighbour shows up.
    arena.view(torch.int16).fill_(0x7FC0)
    _place(arena, dy_off, dy)
    _place(arena, x_off, x)
    offs_dev = torch.tensor([dy_off, x_off], dtype=torch.int64, device=dev)
    out_dtype = torch.float32 if fp32_out else torch.bfloat16
    dw = torch.full((e, n, kd), 3.0, device=dev, dtype=out_dtype)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    ref = torch.stack(
        [dy[off[i] : off[i + 1]].float().T @ x[off[i] : off[i + 1]].float() for i in range(e)]
    )
    for accumulate in (0, 1):
        rc = nat.lib.dm_gemm_wgrad(
            nat.Operand(arena.data_ptr(), arena.numel(), offs_dev[0:1].data_ptr()),
            nat.Operand(arena.data_ptr(), arena.numel(), offs_dev[1:2].data_ptr()),
            dw.data_ptr(), fp32_out, accumulate, offs_t.data_ptr(), e, rows, n, kd, 0, status.data_ptr(), nat.stream_ptr(),
        )
        nat.check(rc, "dm_gemm_wgrad")
        torch.cuda.synchronize()
        assert status[0].item() == 0, status.tolist()
        expect = ref if not accumulate else ref + dw_prev.float()
        _close(dw, expect, f"wgrad accumulate={accumulate} fp32={fp32_out}")
        dw_prev = dw.clone()


def test_fprop_scatter_rows():
    """Rows of C go to per-row destinations (the combine scatter), null pointers are skipped."""
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    counts, kd, n = [150, 77], 128, 256
    e = len(counts)
    offs_t, off = _offsets(counts, dev)
    rows = off[-1]
    a = torch.randn(rows, kd, device=dev).bfloat16()
    w = (torch.randn(e, n, kd, device=dev) * 0.1).bfloat16()
    dest = torch.zeros(rows, n, device=dev, dtype=torch.bfloat16)
    perm = torch.randperm(rows, device=dev)
    ptrs = dest.data_ptr() + perm.to(torch.int64) * n * 2
    ptrs[3] = 0
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    pad = torch.zeros(300 * kd, device=dev, dtype=torch.bfloat16)
    a_full = torch.cat([a.reshape(-1), pad])
    rc = nat.lib.dm_gemm_fprop(
        nat.Operand(a_full.data_ptr(), a_full.numel() * 2, None),
        w.data_ptr(), nat.Operand(None, 0, None), nat.Operand(None, 0, None), ptrs.data_ptr(),
        offs_t.data_ptr(), e, rows, n, kd, 0, 0, 1.0, 0.0, None, 0, status.data_ptr(), nat.stream_ptr(),
    )
    nat.check(rc, "dm_gemm_fprop scatter")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    ref = torch.zeros(rows, n, device=dev)
    for ei in range(e):
        lo, hi = off[ei], off[ei + 1]
        ref[perm[lo:hi]] = a[lo:hi].float() @ w[ei].float().T
    ref[perm[3]] = 0
    _close(dest, ref, "scatter")


@pytest.mark.parametrize("mode", ["fprop", "dgrad"])
def test_fused_dispatch_gathers_rows_inside_the_gemm(mode):
    """Rows of A are pulled through a pointer table by the kernel's gather warps (null pointer = zero row);
    the pulled copy must also be left in the A operand for the later weight-gradient GEMM."""
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.manual_seed(6)
    counts, kd, n = [300, 0, 45, 500], 256, 512
    e = len(counts)
    offs_t, off = _offsets(counts, dev)
    rows = off[-1]
    src = torch.randn(2000, kd, device=dev).bfloat16()
    idx = torch.randint(0, 2000, (rows,), device=dev)
    ptrs = src.data_ptr() + idx.to(torch.int64) * kd * 2
    ptrs[17] = 0
    a_ref = src[idx].clone()
    a_ref[17] = 0
    w = (torch.randn(e, n, kd, device=dev) * 0.1).bfloat16() if mode == "fprop" else \
        (torch.randn(e, kd, n, device=dev) * 0.1).bfloat16()
    a_buf = torch.full(((rows + 300) * kd,), 9.0, device=dev, dtype=torch.bfloat16)
    out = torch.zeros(rows, n, device=dev, dtype=torch.bfloat16)
    flags = torch.full((rows // 128 + 8,), 77, dtype=torch.int32, device=dev)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    a_op = nat.Operand(a_buf.data_ptr(), a_buf.numel() * 2, None)
    c_op = nat.Operand(out.data_ptr(), out.numel() * 2, None)
    none = nat.Operand(None, 0, None)
    for _ in range(2):
        if mode == "fprop":
            rc = nat.lib.dm_gemm_fprop_dispatch(ptrs.data_ptr(), flags.data_ptr(), a_op, w.data_ptr(), c_op, none,
                                                offs_t.data_ptr(), e, rows, n, kd, 0, 0, 1.0, 0.0, None, 0,
                                                status.data_ptr(), nat.stream_ptr())
        else:
            rc = nat.lib.dm_gemm_dgrad_dispatch(ptrs.data_ptr(), flags.data_ptr(), a_op, w.data_ptr(), c_op,
                                                offs_t.data_ptr(), e, rows, n, kd, None, 0, status.data_ptr(),
                                                nat.stream_ptr())
        nat.check(rc, "dispatch gemm")
        torch.cuda.synchronize()
        assert status[0].item() == 0, status.tolist()
        got_a = a_buf[: rows * kd].view(rows, kd)
        assert torch.equal(got_a.view(torch.int16), a_ref.view(torch.int16)), "gathered rows differ"
        for ei in range(e):
            lo, hi = off[ei], off[ei + 1]
            if hi > lo:
                wt = w[ei].float().T if mode == "fprop" else w[ei].float()
                _close(out[lo:hi], a_ref[lo:hi].float() @ wt, f"{mode} dispatch expert {ei}")
