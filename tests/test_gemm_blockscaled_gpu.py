"""Block-scaled grouped GEMM (tcgen05 with TMEM scale factors) through the C ABI.

Operands are produced by this library's quantisers (bit-exact against the oracle elsewhere) and the
reference result is the fp32 matmul of the *dequantised* operands, so the comparison isolates the GEMM:
only fp32 accumulation order and the final bf16 rounding may differ (|diff| <= 2^-7 |ref| + 2e-3 rms)."""

import numpy as np
import pytest
import torch

from oracle import quant as Q

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _nat():
    from dist_moe_b200 import _native

    return _native


def _close(got, ref, what):
    got, ref = got.float(), ref.float()
    scale = ref.pow(2).mean().sqrt().item() + 1e-9
    err = (got - ref).abs()
    bad = err > ref.abs() * 2.0**-7 + 2e-3 * scale
    assert not bool(bad.any()), f"{what}: {int(bad.sum())}/{bad.numel()} bad, max err {err.max().item():.4g}, rms {scale:.4g}"


def _quant_act(nat, x, fmt):
    """x bf16 [R, K] on device -> (q, blocked scales, dequantised fp32, row_inv or None)."""
    R, K = x.shape
    if fmt == 0:
        q = torch.zeros(R + 256, K, dtype=torch.uint8, device=DEV)
        atoms = (K // 32 + 3) // 4
        s = torch.zeros((R + 127) // 128 * 128 * atoms * 4, dtype=torch.uint8, device=DEV)
        nat.check(nat.lib.dm_quant_mxfp8_row(x.data_ptr(), None, R, K, q.data_ptr(), 0, s.data_ptr(), 0, 1, nat.stream_ptr()), "q")
        qn, sn = Q.mxfp8_row(x.cpu())
        deq = torch.from_numpy(Q.mxfp8_dequant_row(qn, sn).reshape(R, K).astype(np.float32))
        return q, s, deq, None
    q = torch.zeros(R + 256, K // 2, dtype=torch.uint8, device=DEV)
    nat_s = torch.zeros(R, K // 16, dtype=torch.uint8, device=DEV)
    inv = torch.zeros(R, dtype=torch.float32, device=DEV)
    nat.check(nat.lib.dm_quant_nvfp4_token(x.data_ptr(), None, R, K, q.data_ptr(), K // 2, nat_s.data_ptr(), K // 16, 0,
                                           inv.data_ptr(), 4, nat.stream_ptr()), "q")
    atoms = (K // 16 + 3) // 4
    s = torch.zeros((R + 127) // 128 * 128 * atoms * 4, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_sf_swizzle(nat_s.data_ptr(), s.data_ptr(), R, K // 16, nat.stream_ptr()), "swz")
    pk, sb, iv = Q.nvfp4_token_rows(x.cpu())
    deq = torch.from_numpy(Q.nvfp4_dequant(pk, sb, iv).astype(np.float32))
    return q, s, deq, inv


def _quant_w(nat, w, fmt):
    """w bf16 [E, N, K] on device -> (q, blocked scales per expert, dequantised fp32 [E,N,K], expert_inv or None)."""
    E, N, K = w.shape
    if fmt == 0:
        q = torch.zeros(E * N, K, dtype=torch.uint8, device=DEV)
        atoms = (K // 32 + 3) // 4
        s = torch.zeros(E * ((N + 127) // 128 * 128) * atoms * 4, dtype=torch.uint8, device=DEV)
        for e in range(E):  # row mode per expert so that every expert is its own blocked group
            grp = (N + 127) // 128 * 128 * atoms * 4
            nat.check(nat.lib.dm_quant_mxfp8_row(w[e].data_ptr(), None, N, K, q[e * N:].data_ptr(), 0,
                                                 s[e * grp:].data_ptr(), 0, 1, nat.stream_ptr()), "qw")
        qn, sn = Q.mxfp8_row(w.reshape(E * N, K).cpu())
        deq = torch.from_numpy(Q.mxfp8_dequant_row(qn, sn).reshape(E, N, K).astype(np.float32))
        return q, s, deq, None
    amax = torch.linalg.vector_norm(w, ord=float("inf"), dim=(-2, -1), dtype=torch.float32).clamp(min=1e-12)
    gs = 2688.0 * torch.reciprocal(amax)
    q = torch.zeros(E * N, K // 2, dtype=torch.uint8, device=DEV)
    atoms = (K // 16 + 3) // 4
    s = torch.zeros(E * ((N + 127) // 128 * 128) * atoms * 4, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_nvfp4_weight(w.data_ptr(), gs.data_ptr(), E, N, K, q.data_ptr(), s.data_ptr(), 1,
                                            nat.stream_ptr()), "qw")
    pk, sb, g, gi = Q.nvfp4_weight(w.cpu())
    deq = torch.from_numpy(Q.nvfp4_dequant(pk.reshape(E * N, K // 2), sb.reshape(E * N, K // 16),
                                           np.repeat(gi, N)).reshape(E, N, K).astype(np.float32))
    return q, s, deq, torch.reciprocal(gs)


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("counts,K,N", [([128, 0, 256], 256, 256), ([384], 512, 128), ([128, 128, 128, 128], 1024, 384)])
def test_blockscaled_gemm_plain_and_scatter(fmt, counts, K, N):
    nat = _nat()
    torch.manual_seed(fmt * 7 + K)
    E = len(counts)
    off = [0]
    for c in counts:
        off.append(off[-1] + c)
    R = off[-1]
    offs = torch.tensor(off, dtype=torch.int32, device=DEV)
    x = torch.randn(R, K, device=DEV).bfloat16()
    w = (torch.randn(E, N, K, device=DEV) * 0.05).bfloat16()
    qa, sa, da, inv = _quant_act(nat, x, fmt)
    qw, sw, dw, einv = _quant_w(nat, w, fmt)
    out = torch.full((R + 8, N), 5.0, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    op = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    none = nat.Operand(None, 0, None)
    rc = nat.lib.dm_gemm_blockscaled(fmt, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), op(out), none, None,
                                     op(inv) if inv is not None else none, nat.ptr(einv), offs.data_ptr(), E, R, N, K,
                                     0, 0, 1.0, 0.0, None, 0, status.data_ptr(), nat.stream_ptr())
    nat.check(rc, "dm_gemm_blockscaled")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    for e in range(E):
        lo, hi = off[e], off[e + 1]
        if hi > lo:
            _close(out[lo:hi].cpu(), da[lo:hi] @ dw[e].T, f"fmt {fmt} expert {e}")
    assert bool((out[R:] == 5.0).all())


@pytest.mark.parametrize("fmt", [0, 1])
def test_blockscaled_gemm_interleaved_swiglu(fmt):
    nat = _nat()
    torch.manual_seed(3 + fmt)
    counts, K, F = [128, 256], 512, 192
    E, N = len(counts), 2 * F
    off = [0, 128, 384]
    R = off[-1]
    offs = torch.tensor(off, dtype=torch.int32, device=DEV)
    x = torch.randn(R, K, device=DEV).bfloat16()
    w = (torch.randn(E, N, K, device=DEV) * 0.05).bfloat16()  # canonical rows: [gate F | up F]
    # interleave rows in groups of 8: gate[0:8], up[0:8], gate[8:16], ...
    idx = torch.stack([torch.arange(F).reshape(-1, 8), torch.arange(F).reshape(-1, 8) + F], dim=1).reshape(-1)
    wi = w[:, idx.to(DEV), :].contiguous()
    qa, sa, da, inv = _quant_act(nat, x, fmt)
    qw, sw, dwi, einv = _quant_w(nat, wi, fmt)
    h1 = torch.zeros(R, N, device=DEV, dtype=torch.bfloat16)
    h2 = torch.zeros(R, F, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    op = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    none = nat.Operand(None, 0, None)
    rc = nat.lib.dm_gemm_blockscaled(fmt, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), op(h1), op(h2), None,
                                     op(inv) if inv is not None else none, nat.ptr(einv), offs.data_ptr(), E, R, N, K,
                                     1, 0, 1.702, 7.0, None, 0, status.data_ptr(), nat.stream_ptr())
    nat.check(rc, "dm_gemm_blockscaled swiglu")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    inv_idx = torch.empty_like(idx)
    inv_idx[idx] = torch.arange(N)
    for e in range(E):
        lo, hi = off[e], off[e + 1]
        ref_i = da[lo:hi] @ dwi[e].T                 # interleaved columns
        ref = ref_i[:, inv_idx]                      # canonical [gate | up]
        _close(h1[lo:hi].cpu(), ref, f"h1 fmt {fmt} expert {e}")
        g, u = h1[lo:hi, :F].float().cpu(), h1[lo:hi, F:].float().cpu()
        _close(h2[lo:hi].cpu(), g * torch.sigmoid(g) * u, f"h2 fmt {fmt} expert {e}")


# ---------------------------------------------------------------------------------------------
# MXFP8 training backward: input gradient (W read N-major) and weight gradient (both operands
# quantised along the row dimension).  Same rule as above: reference = fp32 matmul of dequantised
# operands, so only accumulation order and the final rounding differ.
# ---------------------------------------------------------------------------------------------
def _e8m0(s):
    return np.exp2(s.astype(np.float32) - 127.0)


def _tile32_weight(nat, w):
    """w bf16 [E, N, K] -> (shared qdata, fprop scales, dgrad scales, dequantised fp32 [E, N, K])."""
    E, N, K = w.shape
    q = torch.zeros(E * N, K, dtype=torch.uint8, device=DEV)
    a0, a1 = (K // 32 + 3) // 4, (N // 32 + 3) // 4
    s0 = torch.zeros(E * ((N + 127) // 128 * 128) * a0 * 4, dtype=torch.uint8, device=DEV)
    s1 = torch.zeros(E * ((K + 127) // 128 * 128) * a1 * 4, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_tile32(w.data_ptr(), E, N, K, q.data_ptr(), s0.data_ptr(), s1.data_ptr(), 1,
                                            nat.stream_ptr()), "tile32")
    deq = []
    for e in range(E):
        qn, sn = Q.mxfp8_tile32(w[e].cpu())
        full = np.repeat(np.repeat(_e8m0(sn), 32, axis=0), 32, axis=1)
        deq.append(torch.from_numpy(Q.e4m3_to_f32(qn).astype(np.float32) * full))
    return q, s0, s1, torch.stack(deq)


def _quant_col(nat, x, max_rows):
    """x bf16 [R, C] -> (q [max_rows, C], blocked scales (feature, row block), dequantised fp32 [R, C])."""
    R, C = x.shape
    q = torch.zeros(max_rows, C, dtype=torch.uint8, device=DEV)
    atoms = ((max_rows + 31) // 32 + 3) // 4
    s = torch.zeros((C + 127) // 128 * 128 * atoms * 4, dtype=torch.uint8, device=DEV)
    cnt = torch.tensor([R], dtype=torch.int32, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_col(x.data_ptr(), cnt.data_ptr(), max_rows, C, q.data_ptr(), s.data_ptr(), 1,
                                         nat.stream_ptr()), "qcol")
    qn, sn = Q.mxfp8_col(x.cpu())                       # scales [C, R/32]
    deq = Q.e4m3_to_f32(qn).astype(np.float32) * np.repeat(_e8m0(sn).T, 32, axis=0)[:R]
    return q, s, torch.from_numpy(deq)


def _offsets(counts):
    off = [0]
    for c in counts:
        off.append(off[-1] + c)
    return off


@pytest.mark.parametrize("counts,K,N", [([128, 0, 256], 256, 128), ([384], 128, 384), ([128, 256, 128], 512, 256)])
@pytest.mark.parametrize("scatter", [False, True])
def test_blockscaled_dgrad(counts, K, N, scatter):
    """C[r, n] = sum_k dY[r, k] W[e][k, n]; W stored [E, K, N] (the forward's [E, rows=K, cols=N])."""
    nat = _nat()
    torch.manual_seed(K + N)
    E, off = len(counts), _offsets(counts)
    R = off[-1]
    offs = torch.tensor(off, dtype=torch.int32, device=DEV)
    dy = torch.randn(R, K, device=DEV).bfloat16()
    w = (torch.randn(E, K, N, device=DEV) * 0.05).bfloat16()
    qa, sa, da, _ = _quant_act(nat, dy, 0)
    qw, _, s_dgrad, dw = _tile32_weight(nat, w)
    out = torch.full((R + 8, N), 5.0, device=DEV, dtype=torch.bfloat16)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    op = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    none = nat.Operand(None, 0, None)
    ptrs = None
    if scatter:
        perm = torch.randperm(R, device=DEV)
        ptrs = out.data_ptr() + perm.to(torch.int64) * (N * 2)
        ptrs[R - 1] = 0  # a padding row: skipped
    rc = nat.lib.dm_gemm_blockscaled_dgrad(op(qa), op(sa), qw.data_ptr(), s_dgrad.data_ptr(), none if scatter else op(out),
                                           nat.ptr(ptrs), offs.data_ptr(), E, R, N, K, None, 0, status.data_ptr(),
                                           nat.stream_ptr())
    nat.check(rc, "dm_gemm_blockscaled_dgrad")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    ref = torch.zeros(R, N)
    for e in range(E):
        ref[off[e]:off[e + 1]] = da[off[e]:off[e + 1]] @ dw[e]
    got = out[:R].cpu()
    if scatter:
        p = perm.cpu()
        _close(got[p[: R - 1]], ref[: R - 1], "dgrad scatter")
        assert bool((got[p[R - 1]] == 5.0).all())
    else:
        _close(got, ref, "dgrad")
    assert bool((out[R:] == 5.0).all())


@pytest.mark.parametrize("counts,M,N", [([128, 0, 256], 128, 256), ([384, 128], 256, 128), ([1024], 384, 128)])
@pytest.mark.parametrize("fp32,acc", [(1, 0), (1, 1), (0, 0), (0, 1)])
def test_blockscaled_wgrad(counts, M, N, fp32, acc):
    nat = _nat()
    torch.manual_seed(M + 3 * N + fp32)
    E, off = len(counts), _offsets(counts)
    R = off[-1]
    cap = R + 256                                        # capacity larger than the routed rows
    offs = torch.tensor(off, dtype=torch.int32, device=DEV)
    dy = torch.randn(R, M, device=DEV).bfloat16()
    x = torch.randn(R, N, device=DEV).bfloat16()
    qd, sd, dd = _quant_col(nat, dy, cap)
    qx, sx, dx = _quant_col(nat, x, cap)
    dtype = torch.float32 if fp32 else torch.bfloat16
    base = (torch.randn(E, M, N, device=DEV) * 4).to(dtype) if acc else torch.full((E, M, N), 7.0, device=DEV, dtype=dtype)
    dw = base.clone()
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    op = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    rc = nat.lib.dm_gemm_blockscaled_wgrad(op(qd), op(sd), op(qx), op(sx), dw.data_ptr(), fp32, acc, offs.data_ptr(), E,
                                           cap, M, N, None, 0, status.data_ptr(), nat.stream_ptr())
    nat.check(rc, "dm_gemm_blockscaled_wgrad")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    for e in range(E):
        lo, hi = off[e], off[e + 1]
        ref = dd[lo:hi].T @ dx[lo:hi]
        got = dw[e].float().cpu()
        if acc:
            ref = ref + base[e].float().cpu()
            if not fp32:  # one bf16 rounding of the sum
                ref = ref.bfloat16().float()
                assert (got - ref).abs().max().item() <= ref.abs().max().item() * 2.0**-7
                continue
        elif hi == lo:
            assert bool((got == 0).all())
            continue
        _close(got if fp32 else got.bfloat16(), ref, f"wgrad expert {e}")


def test_swiglu_epilogue_that_quantises_h2_equals_gemm_then_row_quantiser():
    """dm_gemm_blockscaled_swiglu_mxfp8 writes the E4M3 bytes and scales that dm_quant_mxfp8_row produces from the
    bf16 h2 of the plain SwiGLU call."""
    nat = _nat()
    torch.manual_seed(11)
    counts, K, F = [128, 384, 0, 256], 512, 320
    E, N = len(counts), 2 * F
    off = [0]
    for c in counts:
        off.append(off[-1] + c)
    R = off[-1]
    offs = torch.tensor(off, dtype=torch.int32, device=DEV)
    x = torch.randn(R, K, device=DEV).bfloat16()
    w = (torch.randn(E, N, K, device=DEV) * 0.05).bfloat16()
    qa, sa, _, _ = _quant_act(nat, x, 0)
    qw, sw, _, _ = _quant_w(nat, w, 0)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    op = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    none = nat.Operand(None, 0, None)
    st = nat.stream_ptr()
    h2 = torch.zeros(R, F, device=DEV, dtype=torch.bfloat16)
    nat.check(nat.lib.dm_gemm_blockscaled(0, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), none, op(h2), None, none, None,
                                          offs.data_ptr(), E, R, N, K, 1, 1, 1.702, 7.0, None, 0, status.data_ptr(), st),
              "gemm+swiglu")
    atoms = (F // 32 + 3) // 4
    want_q = torch.zeros(R, F, dtype=torch.uint8, device=DEV)
    want_s = torch.zeros(R * atoms * 4, dtype=torch.uint8, device=DEV)
    nat.check(nat.lib.dm_quant_mxfp8_row(h2.data_ptr(), None, R, F, want_q.data_ptr(), 0, want_s.data_ptr(), 0, 1, st), "row")
    got_q, got_s = torch.zeros_like(want_q), torch.zeros_like(want_s)
    nat.check(nat.lib.dm_gemm_blockscaled_swiglu_mxfp8(op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), op(got_q), op(got_s),
                                                       offs.data_ptr(), E, R, N, K, 1, 1.702, 7.0, None, 0,
                                                       status.data_ptr(), st), "gemm+swiglu+quant")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    assert torch.equal(got_q, want_q)
    assert torch.equal(got_s, want_s)
