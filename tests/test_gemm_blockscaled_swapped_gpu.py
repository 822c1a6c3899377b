"""Swapped-operand block-scaled GEMM (weights on the MMA's M side, few routed rows on the N side) through the C ABI.

Reference = fp32 matmul of the dequantised operands, as for the 128 x 256 kernel, plus an exact comparison with that
kernel on the same operands: both accumulate the same K steps in the same order, so their bf16 outputs are equal."""

import pytest
import torch

from tests.test_gemm_blockscaled_gpu import _close, _nat, _quant_act, _quant_w

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _layout(counts):
    """Row groups padded to 128 as the routing step lays them out: (padded offsets, row index of every real row)."""
    off, rows = [0], []
    for c in counts:
        rows.extend(range(off[-1], off[-1] + c))
        off.append(off[-1] + (c + 127) // 128 * 128)
    return off, torch.tensor(rows, dtype=torch.int64)


def _operands(nat, fmt, counts, K, N, seed, interleave_F=None):
    torch.manual_seed(seed)
    E = len(counts)
    off, real = _layout(counts)
    R = max(off[-1], 128)
    x = torch.zeros(R, K, device=DEV, dtype=torch.bfloat16)
    x[real.to(DEV)] = torch.randn(len(real), K, device=DEV).bfloat16()
    w = (torch.randn(E, N, K, device=DEV) * 0.05).bfloat16()
    if interleave_F is not None:
        F = interleave_F
        idx = torch.stack([torch.arange(F).reshape(-1, 8), torch.arange(F).reshape(-1, 8) + F], dim=1).reshape(-1)
        w = w[:, idx.to(DEV), :].contiguous()
    qa, sa, da, inv = _quant_act(nat, x, fmt)
    qw, sw, dw, einv = _quant_w(nat, w, fmt)
    offs = torch.tensor(off, dtype=torch.int32, device=DEV)
    cnts = torch.tensor(counts, dtype=torch.int32, device=DEV)
    return E, off, real, R, (qa, sa, da, inv), (qw, sw, dw, einv), offs, cnts


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("counts,K,N", [([5, 0, 33, 64], 256, 128), ([100, 128, 1], 512, 384), ([130, 17], 1024, 256),
                                         ([0, 0], 256, 128)])
@pytest.mark.parametrize("scatter", [False, True])
def test_swapped_plain_and_scatter(fmt, counts, K, N, scatter):
    nat = _nat()
    E, off, real, R, (qa, sa, da, inv), (qw, sw, dw, einv), offs, cnts = _operands(nat, fmt, counts, K, N, 11 * fmt + K + N)
    op = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    none = nat.Operand(None, 0, None)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    out = torch.full((R + 8, N), 5.0, device=DEV, dtype=torch.bfloat16)
    ptrs = None
    if scatter:
        # real rows go to shuffled rows of `out`; padding rows carry a null pointer
        perm = torch.randperm(R, device=DEV)
        ptrs = torch.zeros(R, dtype=torch.int64, device=DEV)
        ptrs[real.to(DEV)] = out.data_ptr() + perm[real.to(DEV)].to(torch.int64) * (N * 2)
    rc = nat.lib.dm_gemm_blockscaled_swapped(fmt, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), none if scatter else op(out),
                                             none, nat.ptr(ptrs), op(inv) if inv is not None else none, nat.ptr(einv),
                                             offs.data_ptr(), cnts.data_ptr(), E, R, N, K, 0, 0, 1.0, 0.0, None, 0,
                                             status.data_ptr(), nat.stream_ptr())
    nat.check(rc, "dm_gemm_blockscaled_swapped")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    wide = torch.full((R + 8, N), 5.0, device=DEV, dtype=torch.bfloat16)
    nat.check(nat.lib.dm_gemm_blockscaled(fmt, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), op(wide), none, None,
                                          op(inv) if inv is not None else none, nat.ptr(einv), offs.data_ptr(), E, R, N,
                                          K, 0, 0, 1.0, 0.0, None, 0, status.data_ptr(), nat.stream_ptr()), "wide")
    torch.cuda.synchronize()
    got = out.cpu()
    touched = torch.zeros(R + 8, dtype=torch.bool)
    for e in range(E):
        rows = torch.arange(off[e], off[e] + counts[e])
        if len(rows) == 0:
            continue
        dst = perm.cpu()[rows] if scatter else rows
        touched[dst] = True
        _close(got[dst], da[rows] @ dw[e].T, f"fmt {fmt} expert {e}")
        assert torch.equal(got[dst], wide.cpu()[rows]), f"expert {e}: differs from the 128 x 256 kernel"
    assert bool((got[~touched] == 5.0).all()), "rows past an expert's count were written"


@pytest.mark.parametrize("fmt", [0, 1])
@pytest.mark.parametrize("clamped", [0, 1])
def test_swapped_interleaved_swiglu(fmt, clamped):
    nat = _nat()
    counts, K, F = [40, 0, 7, 128, 65], 512, 192
    N = 2 * F
    E, off, real, R, (qa, sa, da, inv), (qw, sw, dw, einv), offs, cnts = _operands(nat, fmt, counts, K, N, 5 + fmt, F)
    op = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    none = nat.Operand(None, 0, None)
    status = torch.zeros(8, dtype=torch.int32, device=DEV)
    h2 = torch.full((R, F), 5.0, device=DEV, dtype=torch.bfloat16)
    nat.check(nat.lib.dm_gemm_blockscaled_swapped(fmt, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), none, op(h2), None,
                                                  op(inv) if inv is not None else none, nat.ptr(einv), offs.data_ptr(),
                                                  cnts.data_ptr(), E, R, N, K, 1, clamped, 1.702, 7.0, None, 0,
                                                  status.data_ptr(), nat.stream_ptr()), "swapped swiglu")
    wide = torch.zeros(R, F, device=DEV, dtype=torch.bfloat16)
    nat.check(nat.lib.dm_gemm_blockscaled(fmt, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), none, op(wide), None,
                                          op(inv) if inv is not None else none, nat.ptr(einv), offs.data_ptr(), E, R, N,
                                          K, 1, clamped, 1.702, 7.0, None, 0, status.data_ptr(), nat.stream_ptr()),
              "wide swiglu")
    torch.cuda.synchronize()
    assert status[0].item() == 0, status.tolist()
    got, ref = h2.cpu(), wide.cpu()
    assert torch.equal(got[real], ref[real]), "SwiGLU rows differ from the 128 x 256 kernel"
    pad = torch.ones(R, dtype=torch.bool)
    pad[real] = False
    assert bool((got[pad] == 5.0).all())
    if not clamped:
        idx = torch.stack([torch.arange(F).reshape(-1, 8), torch.arange(F).reshape(-1, 8) + F], dim=1).reshape(-1)
        inv_idx = torch.empty_like(idx)
        inv_idx[idx] = torch.arange(N)
        for e in range(E):
            rows = torch.arange(off[e], off[e] + counts[e])
            if len(rows) == 0:
                continue
            h1 = (da[rows] @ dw[e].T)[:, inv_idx].bfloat16().float()
            g, u = h1[:, :F], h1[:, F:]
            _close(got[rows], g * torch.sigmoid(g) * u, f"h2 fmt {fmt} expert {e}")
