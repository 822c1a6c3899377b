"""Routed-expert math, restated with plain eager PyTorch on the CPU.

TEST INFRASTRUCTURE ONLY (see ``oracle/__init__.py``).

Same rounding points as the oracle the reference's own tests use
(tests/test_dist_moe.py:179-243 ``_reference_moe``): ``h13 = linear(x, w13[e])`` in the
input dtype, SwiGLU in fp32 then cast back, ``linear(h2, w2[e])``, fp32 score-weighted
sum over the K routes, cast to the input dtype; routes with id -1 contribute zero rows.
Clamped SwiGLU: ``g = min(gate, L)``, ``u = clamp(up, -L, L)``, ``g * sigmoid(alpha*g) * (u + 1)``
(dist_moe/kernels/triton/swiglu.py:200-206).  Backward is autograd on this graph.

The per-expert batching below is only a reordering of the reference's per-token loop:
each (token, route) goes through exactly the same operations.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F


def swiglu(gate, up, *, clamped=False, alpha=1.702, limit=7.0):
    g, u = gate.float(), up.float()
    if clamped:
        g = torch.minimum(g, g.new_tensor(limit))
        u = torch.clamp(u, min=-limit, max=limit)
        return g * torch.sigmoid(alpha * g) * (u + 1.0)
    return g * torch.sigmoid(g) * u


def expert_outputs(x, ids, w13, w2, *, clamped=False, alpha=1.702, limit=7.0, expert_base=0):
    """Per-route expert outputs h3[T, K, D]; w13 = [E, 2F, D], w2 = [E, D, F] hold experts
    ``expert_base .. expert_base+E``; routes to other experts (or -1) stay zero."""
    T, K = ids.shape
    D = x.shape[1]
    inter = w2.shape[2]
    rows = []
    h3 = torch.zeros(T, K, D, dtype=x.dtype)
    pieces = []
    for e in range(w13.shape[0]):
        t_idx, k_idx = torch.nonzero(ids == e + expert_base, as_tuple=True)
        if t_idx.numel() == 0:
            continue
        h13 = F.linear(x[t_idx], w13[e])
        gate, up = h13.split(inter, dim=-1)
        h2 = swiglu(gate, up, clamped=clamped, alpha=alpha, limit=limit).to(x.dtype)
        pieces.append((t_idx, k_idx, F.linear(h2, w2[e])))
    if pieces:
        t_all = torch.cat([p[0] for p in pieces])
        k_all = torch.cat([p[1] for p in pieces])
        h3 = h3.index_put((t_all, k_all), torch.cat([p[2] for p in pieces]))
    del rows
    return h3


def combine(h3, scores, out_dtype):
    return torch.sum(h3.float() * scores.float()[:, :, None], dim=1).to(out_dtype)


def rmsnorm_combine(h3, scores, eps, out_dtype, weight=None, gain_center=0.0):
    """``sum_k s_k * h3_k / sqrt(mean(h3_k^2) + eps)`` in fp32
    (dist_moe/kernels/norm/fused_rmsnorm_combine.py:427-466 unfused composition)."""
    h = h3.float()
    if weight is not None:
        h = h * (weight.float() + gain_center)
    rstd = torch.rsqrt(h.pow(2).mean(dim=-1, keepdim=True) + eps)
    return torch.sum(h * rstd * scores.float()[:, :, None], dim=1).to(out_dtype)


def moe_forward(x, ids, scores, w13, w2, *, clamped=False, alpha=1.702, limit=7.0, rmsnorm_eps=None):
    """Single-process dense evaluation: x [T, D], w13 [E, 2F, D], w2 [E, D, F] (all experts)."""
    w13 = w13.reshape(w13.shape[0], -1, w13.shape[-1])
    h3 = expert_outputs(x, ids, w13, w2, clamped=clamped, alpha=alpha, limit=limit)
    if rmsnorm_eps is not None:
        return rmsnorm_combine(h3, scores, rmsnorm_eps, x.dtype)
    return combine(h3, scores, x.dtype)


def clip_stats(x, ids, w13, clip_limit):
    """[#gate > limit, #|up| > limit, #valid elements] (tests/test_dist_moe.py:246-290)."""
    w13 = w13.reshape(w13.shape[0], -1, w13.shape[-1])
    inter = w13.shape[1] // 2
    gate_n = up_n = total = 0
    for e in range(w13.shape[0]):
        t_idx, _ = torch.nonzero(ids == e, as_tuple=True)
        if t_idx.numel() == 0:
            continue
        h13 = F.linear(x[t_idx], w13[e])
        gate, up = h13.split(inter, dim=-1)
        gate_n += int((gate.float() > clip_limit).sum())
        up_n += int((up.float().abs() > clip_limit).sum())
        total += t_idx.numel() * inter
    return torch.tensor([gate_n, up_n, total], dtype=torch.float32)
