"""Block-scaled (MXFP8 E4M3 / NVFP4) execution: weight preparation and the forward path.

Launch order of the forward (mirrors the reference's staged block-scaled forward,
dist_moe/_blockscaled.py:1309-1931, with static inference storage):

  quantise x into the packed symmetric dispatch row [q | scales | inverse row scale | pad]
  -> publish ids -> barrier -> route (per-expert rows padded to 128, packed row stride)
  -> gather packed rows (peer loads) into dense q rows + blocked scales
  -> W13 block-scaled GEMM with fused SwiGLU (interleaved prepared W13) -> bf16 h2
  -> quantise h2 rows -> W2 block-scaled GEMM, rows scattered to the owners' combine buffers
  -> barrier -> weighted top-k reduction (or fused RMSNorm).

Weight preparation follows dist_moe/_blockscaled.py:798-882 (MXFP8) and 140-196 (NVFP4):
MXFP8 training weights use 32x32 tiles with one shared qdata and two scale orientations,
MXFP8 inference weights 1x32 rows, NVFP4 a per-expert fp32 global scale ``2688 / amax``.
``fuse_swiglu`` interleaves W13 rows in groups of 8 gate / 8 up rows
(dist_moe/_blockscaled_weight.py:16-39) so that one 128-row tile holds matching pairs.

MXFP8 training (autograd) follows the reference's staged sequence
(dist_moe/_blockscaled.py:1309-1931 forward, 1951-2541 backward):

  forward   publish bf16 x -> barrier -> route (128-padded) -> gather bf16 rows -> quantise rows (+ the
            column-quantised copy the weight gradient needs) -> W13 -> bf16 h1 (saved) -> SwiGLU ->
            quantise h2 rows + columns -> W2, rows scattered -> barrier -> weighted reduce (+ keep h3)
  backward  grad_h3 / grad_scores -> barrier -> gather grad_h3 -> quantise rows + columns ->
            W2 dgrad (same qdata, transposed scales) -> W2 wgrad -> SwiGLU bwd -> quantise ->
            W13 dgrad scattered to the owners -> W13 wgrad -> barrier -> reduce over top-k

Saved activations of the training path live in per-call torch allocations sized for the row capacity
(h1 in bf16, x and h2 as column-quantised E4M3); the device planner of the BF16 path is not used here.
NVFP4 has no backward (dist_moe/_blockscaled.py:245-321).
"""

from __future__ import annotations

from typing import Any

import torch
from torch.profiler import record_function

from . import _native as nat
from ._execution import ExecutionOptions, PreparedWeight, RMSNormPostprocess
from .formats import BlockScaledFormat, format_constants


def _fmt_id(fmt: BlockScaledFormat) -> int:
    return 1 if fmt is BlockScaledFormat.NVFP4 else 0


def _geometry(fmt: BlockScaledFormat, dim: int) -> tuple[int, int]:
    """(quantised bytes per row, scale columns per row) of a [*, dim] operand."""
    if fmt is BlockScaledFormat.NVFP4:
        return dim // 2, dim // 16
    return dim, dim // 32


def planner_storage(fmt: BlockScaledFormat) -> list[int]:
    """Storage geometry the arena planner sizes bundles with (dist_moe/_activation_buffer.py:958-1075
    ``BlockscaledStorageConfig``): [operand element bytes, values per element, scale bytes, row-scale storage
    multiple, per-row global-scale bytes, scale vector]."""
    ob, vpe, sb, vec, gs = format_constants(fmt)
    return [ob, vpe, sb, 4, gs, vec]


def packed_row_stride(fmt: BlockScaledFormat, dim: int) -> int:
    q, sc = _geometry(fmt, dim)
    raw = q + sc + (4 if fmt is BlockScaledFormat.NVFP4 else 0)
    return (raw + 15) // 16 * 16


def interleave_index(F: int, device) -> torch.Tensor:
    """Row order gate[0:8], up[0:8], gate[8:16], up[8:16], ... of a canonical [gate F | up F] W13."""
    g = torch.arange(F, device=device).reshape(-1, 8)
    return torch.stack([g, g + F], dim=1).reshape(-1)


def _blocked_group_bytes(rows: int, scale_cols: int) -> int:
    return (rows + 127) // 128 * 128 * ((scale_cols + 3) // 4) * 4


def prepare_weight(weight: torch.Tensor, config, *, fuse_swiglu: bool = False, inference: bool = False,
                   out: PreparedWeight | None = None) -> PreparedWeight:
    if config.block_scaled is None:
        raise ValueError("prepare_block_scaled_weight needs a config with a block_scaled policy")
    fmt = config.block_scaled.format
    if not isinstance(weight, torch.Tensor) or weight.device.type != "cuda" or weight.dtype != torch.bfloat16:
        raise TypeError("weight must be a CUDA bfloat16 tensor")
    if not weight.is_contiguous():
        raise ValueError("weight must be contiguous")
    if fmt is BlockScaledFormat.NVFP4 and not inference:
        raise ValueError("NVFP4 weights are inference-only; pass inference=True")
    D, F = config.hidden_dim, config.intermediate_dim
    w = weight.detach()
    if w.ndim == 4:
        w = w.reshape(w.shape[0], w.shape[1] * w.shape[2], w.shape[3])
    elif w.ndim == 2:
        if D == F:
            raise ValueError("a flattened 2-D weight is ambiguous when hidden_dim == intermediate_dim; pass it as 3-D")
        w = w.reshape(-1, 2 * F if w.shape[1] == D else D, w.shape[1])
    if w.ndim != 3:
        raise ValueError("weight must be [E_local, N, K] (or one of the accepted W13/W2 layouts)")
    E, N, K = w.shape
    is_w13 = (N, K) == (2 * F, D)
    if not is_w13 and (N, K) != (D, F):
        raise ValueError(f"weight shape {tuple(weight.shape)} matches neither W13 [E, 2F, D] nor W2 [E, D, F]")
    if fuse_swiglu:
        if not is_w13:
            raise ValueError("fuse_swiglu applies to the W13 projection only")
        if not inference:
            raise ValueError("fuse_swiglu (interleaved W13) is an inference-only layout")
        if F % 64 != 0:
            raise ValueError("fuse_swiglu needs intermediate_dim to be a multiple of 64")
        w = w.index_select(1, interleave_index(F, w.device)).contiguous()
    if out is not None:
        qfmt = "nvfp4" if fmt is BlockScaledFormat.NVFP4 else "mxfp8"
        _quantize_weight(w, qfmt, inference, out=out)
        return out
    if fmt is BlockScaledFormat.NVFP4:
        q, sc, gs, gsi = _quantize_weight(w, "nvfp4", True)
        return PreparedWeight._create(source=weight, format=fmt, fprop_data=q, fprop_scale=sc, dgrad_data=None,
                                      dgrad_scale=None, global_scale=gs, global_scale_inv=gsi,
                                      interleaved_fc13=bool(fuse_swiglu))
    q, s0, s1 = _quantize_weight(w, "mxfp8", inference)
    return PreparedWeight._create(source=weight, format=fmt, fprop_data=q, fprop_scale=s0,
                                  dgrad_data=None if inference else q, dgrad_scale=s1, global_scale=None,
                                  global_scale_inv=None, interleaved_fc13=bool(fuse_swiglu))


def _quantize_weight(w: torch.Tensor, kind: str, inference: bool, out: PreparedWeight | None = None):
    """Quantise a contiguous bf16 ``[E, N, K]`` weight (rows already interleaved if wanted).

    mxfp8: ``(qdata [E,N,K] u8, forward scales, input-gradient scales or None)``; training uses 32x32 tiles with
    one shared qdata and two scale orientations, inference 1x32 rows (dist_moe/_blockscaled.py:798-882).
    nvfp4: ``(packed qdata [E,N,K/2], E4M3 scales, global scale fp32[E], its inverse)`` with
    ``global scale = 2688 / amax`` per expert (dist_moe/_blockscaled.py:140-196).
    ``out`` refills the tensors of an existing PreparedWeight in place.
    """
    E, N, K = w.shape
    nvfp4 = kind == "nvfp4"
    if K % (256 if nvfp4 else 128) or N % 128:
        raise ValueError("block-scaled weights need N % 128 == 0 and K % 128 == 0 (K % 256 for NVFP4)")
    dev, st = w.device, nat.stream_ptr()
    qb, sc = (K // 2, K // 16) if nvfp4 else (K, K // 32)
    grp = _blocked_group_bytes(N, sc)

    def storage(name, shape, dtype):
        if out is not None:
            t = getattr(out, name)
            if t is None or tuple(t.shape) != tuple(shape) or t.dtype != dtype:
                raise ValueError(f"out.{name} does not match the prepared layout")
            return t
        return torch.zeros(shape, dtype=dtype, device=dev)

    fprop_data = storage("fprop_data", (E, N, qb), torch.uint8)
    fprop_scale = storage("fprop_scale", (E * grp,), torch.uint8)
    if nvfp4:
        amax = torch.linalg.vector_norm(w, ord=float("inf"), dim=(-2, -1), dtype=torch.float32).clamp(min=1e-12)
        gs_new = 2688.0 * torch.reciprocal(amax)
        gs = storage("global_scale", (E,), torch.float32)
        gsi = storage("global_scale_inv", (E,), torch.float32)
        gs.copy_(gs_new)
        gsi.copy_(torch.reciprocal(gs_new))
        nat.check(nat.lib.dm_quant_nvfp4_weight(w.data_ptr(), gs.data_ptr(), E, N, K, fprop_data.data_ptr(),
                                                fprop_scale.data_ptr(), 1, st), "dm_quant_nvfp4_weight")
        return fprop_data, fprop_scale, gs, gsi
    if inference:
        for e in range(E):
            nat.check(nat.lib.dm_quant_mxfp8_row(w[e].data_ptr(), None, N, K, fprop_data[e].data_ptr(), 0,
                                                 fprop_scale[e * grp:].data_ptr(), 0, 1, st), "dm_quant_mxfp8_row")
        return fprop_data, fprop_scale, None
    grp_d = _blocked_group_bytes(K, N // 32)
    dgrad_scale = storage("dgrad_scale", (E * grp_d,), torch.uint8)
    nat.check(nat.lib.dm_quant_mxfp8_tile32(w.data_ptr(), E, N, K, fprop_data.data_ptr(), fprop_scale.data_ptr(),
                                            dgrad_scale.data_ptr(), 1, st), "dm_quant_mxfp8_tile32")
    return fprop_data, fprop_scale, dgrad_scale


def _as_enk(weight: torch.Tensor, fuse_swiglu: bool) -> torch.Tensor:
    if weight.device.type != "cuda" or weight.dtype != torch.bfloat16:
        raise TypeError("weight must be a CUDA bfloat16 tensor")
    w = weight.detach()
    if w.ndim == 4:
        w = w.reshape(w.shape[0], w.shape[1] * w.shape[2], w.shape[3])
    if w.ndim != 3:
        raise ValueError("weight must be [E_local, N, K]")
    if fuse_swiglu:
        F = w.shape[1] // 2
        if F % 64:
            raise ValueError("fuse_swiglu needs intermediate_dim to be a multiple of 64")
        w = w.index_select(1, interleave_index(F, w.device))
    return w.contiguous()


def quantize_mxfp8_weight(weight: torch.Tensor, *, inference: bool, fuse_swiglu: bool):
    """Body of ``dist_moe::prepare_mxfp8_weight`` (dist_moe/_blockscaled.py:2870-2913): shape-only contract."""
    return _quantize_weight(_as_enk(weight, fuse_swiglu), "mxfp8", inference)


def quantize_nvfp4_weight(weight: torch.Tensor, *, fuse_swiglu: bool):
    """Body of ``dist_moe::prepare_nvfp4_weight`` (dist_moe/_blockscaled.py:140-196)."""
    return _quantize_weight(_as_enk(weight, fuse_swiglu), "nvfp4", True)


def inference_layout(fmt: BlockScaledFormat, D: int, F: int, rows: int) -> dict:
    """Byte offsets of the forward-only block-scaled operands for ``rows`` received rows, and their total: packed
    rows and blocked scales of x and of h2, the NVFP4 per-row scales, and the dense SwiGLU buffers.  A static carve:
    nothing in it depends on routing data, so the storage is fixed when the context is created (the role the
    reference's Mega-inference operand envelope plays, dist_moe/_inference_memory.py:24-110)."""
    a128 = lambda v: (v + 127) // 128 * 128  # noqa: E731
    xq, xs = _geometry(fmt, D)
    hq, hs = _geometry(fmt, F)
    R = rows
    out, off = {}, 0
    for name, nbytes in (("x_q", R * xq), ("x_sf", _blocked_group_bytes(R, xs)), ("x_inv", R * 4), ("h_q", R * hq),
                         ("h_sf", _blocked_group_bytes(R, hs)), ("h_inv", R * 4),
                         ("dense", R * 2 * F * 2),      # h1 [R, 2F] (unfused) or h2 [R, F] (fused)
                         ("h2_dense", R * F * 2)):      # only used by the unfused path
        out[name] = off
        off += a128(nbytes)
    out["total"] = off + 256 * max(D, 2 * F) * 2
    return out


class _Layout:
    """Static carve of the scratch arena for the forward-only block-scaled path (capacity rows)."""

    def __init__(self, state):
        cfg, fmt = state.config, state.config.block_scaled.format
        self.fp4 = fmt is BlockScaledFormat.NVFP4
        for name, value in inference_layout(fmt, cfg.hidden_dim, cfg.intermediate_dim, state.capacity_rows).items():
            setattr(self, name, value)


def _workspace(state):
    ws = getattr(state, "_bs_workspace", None)
    if ws is None:
        lay = _Layout(state)
        # only the shared scratch region may be used: on a training context the activation slots in front of it hold
        # what earlier forwards saved for their backward, and a no-grad call (an evaluation step, the first pass of a
        # checkpointed region) must leave them alone
        scratch = state.arena[state.num_slots * state.slot_bytes:]
        if lay.total <= scratch.numel():
            buf = scratch
        else:  # the reference aliases x and h2 row slots; this layout keeps them apart and may need more room
            buf = torch.zeros(lay.total, dtype=torch.uint8, device=state.device)
        ws = (lay, buf)
        state._bs_workspace = ws
    return ws


# Inference calls whose experts receive at most this many rows on average take the swapped-operand GEMMs (rows on
# the MMA's N side in steps of 32); above it a 128-row tile is mostly real rows and the 128 x 256 kernel wins.
# Measured crossovers (whole layer, one B200): NVFP4 wins at 32 rows per expert and loses at 64, MXFP8 wins at 16 and
# loses at 32 (its MMAs move twice the bytes per row).  ``None`` keeps the per-format value.
SWAPPED_MAX_ROWS_PER_EXPERT = None
_SWAPPED_MAX_ROWS = {BlockScaledFormat.NVFP4: 48, BlockScaledFormat.MXFP8_E4M3: 24}


def _view(buf: torch.Tensor, offset: int) -> nat.Operand:
    return nat.Operand(buf.data_ptr() + offset, buf.numel() - offset, None)


def _weights_for_call(w13, w2, state, cfg):
    """Prepared operands of this call; raw bf16 weights are quantised on the fly (row mode)."""
    if isinstance(w13, PreparedWeight):
        if w13.format is not cfg.block_scaled.format or w2.format is not cfg.block_scaled.format:
            raise ValueError("prepared weights use a different block-scaled format than the context")
        return w13, w2
    if cfg.block_scaled.format is BlockScaledFormat.NVFP4:
        raise ValueError("NVFP4 requires weights from prepare_block_scaled_weight()")
    p13 = prepare_weight(w13, cfg, fuse_swiglu=cfg.intermediate_dim % 64 == 0, inference=True)
    p2 = prepare_weight(w2, cfg, inference=True)
    return p13, p2


def run_block_scaled(x, ids, scores, w13_weight, w2_weight, context: Any, options: ExecutionOptions, *,
                     save_for_backward: bool) -> torch.Tensor:
    state = context._state
    cfg = state.config
    fmt = cfg.block_scaled.format
    D, F, K, E = cfg.hidden_dim, cfg.intermediate_dim, cfg.top_k, cfg.num_experts
    if D % 128 or F % 128:
        raise ValueError("block-scaled execution needs hidden_dim and intermediate_dim to be multiples of 128")
    if options.requires_eager:
        # Python callbacks between launches (dist_moe/_blockscaled.py:2596-2700 `_run_blockscaled_eager`): MXFP8
        # training calls on contexts with activation slots
        post = options.experts_output_postprocess
        if isinstance(post, RMSNormPostprocess):
            raise NotImplementedError("expert-output observers run on BF16 contexts only")
        if not save_for_backward or fmt is BlockScaledFormat.NVFP4 or state.num_slots == 0 \
                or options.swiglu_clip_stats_out_3 is not None or isinstance(w13_weight, PreparedWeight):
            raise NotImplementedError("Python callbacks on block-scaled contexts are supported for MXFP8 training calls "
                                      "with tensor weights only")
        return _EagerMxfp8Function.apply(x, ids, scores, w13_weight, w2_weight, state, options)
    if save_for_backward:
        if fmt is BlockScaledFormat.NVFP4:
            raise RuntimeError("NVFP4 is inference-only: it has no backward")
        prepared = isinstance(w13_weight, PreparedWeight)
        src13 = w13_weight.source if prepared else w13_weight
        src2 = w2_weight.source if prepared else w2_weight
        return _Mxfp8Function.apply(x, ids, scores, src13, src2, state, options,
                                    w13_weight if prepared else None, w2_weight if prepared else None)
    x, scores = x.detach(), scores.detach()
    T = x.shape[0]
    p13, p2 = _weights_for_call(w13_weight, w2_weight, state, cfg)
    lay, buf = _workspace(state)
    f, st, status = _fmt_id(fmt), nat.stream_ptr(), state.status.data_ptr()
    dev, el, ep = x.device, state.e_local, state.ep
    clamped = 1 if cfg.activation == "swiglu_clamped" else 0
    alpha, limit = float(cfg.swiglu_alpha), float(cfg.swiglu_limit)
    xq, xs = _geometry(fmt, D)
    hq, hs = _geometry(fmt, F)
    stride = packed_row_stride(fmt, D)
    dispatch = state.dispatch.local().data_ptr()
    # ---- publish: quantise straight into the packed symmetric dispatch rows ----------------
    if lay.fp4:
        nat.check(nat.lib.dm_quant_nvfp4_token(x.data_ptr(), None, T, D, dispatch, stride, dispatch + xq, stride, 0,
                                               dispatch + xq + xs, stride, st), "dm_quant_nvfp4_token")
    else:
        nat.check(nat.lib.dm_quant_mxfp8_row(x.data_ptr(), None, T, D, dispatch, stride, dispatch + xq, stride, 0, st),
                  "dm_quant_mxfp8_row")
    nat.check(nat.lib.dm_publish(None, ids.data_ptr(), int(ids.dtype == torch.int64), None,
                                 state.routing.local().data_ptr(), T, 0, K, E, int(options.validate_expert_ids),
                                 status, st), "dm_publish")
    state.barrier(state.dispatch)
    # ---- routing (rows of every expert padded to 128) -----------------------------------------
    size = (ep * T * min(K, el) + el * 127 + 127) // 128 * 128
    size = max(size, 128)
    counts = torch.empty(el, dtype=torch.int32, device=dev)
    per_rank = torch.empty(ep, dtype=torch.int32, device=dev)
    offsets = torch.empty(el + 1, dtype=torch.int32, device=dev)
    fwd = torch.empty(size, dtype=torch.int64, device=dev)
    sct = torch.empty(size, dtype=torch.int64, device=dev)
    max_rows = min(size, state.capacity_rows)
    real = torch.empty(el, dtype=torch.int32, device=dev)  # rows per expert before the padding to 128
    nat.check(nat.lib.dm_route_counted(state.routing.peer_ptrs.data_ptr(), state.dispatch.peer_ptrs.data_ptr(),
                                       state.combine.peer_ptrs.data_ptr(), state.rank, ep, T, K, E, stride, stride,
                                       D * 2, 128, state.capacity_rows, size, counts.data_ptr(), real.data_ptr(),
                                       per_rank.data_ptr(), offsets.data_ptr(), fwd.data_ptr(), None, sct.data_ptr(),
                                       state.route_workspace.data_ptr(), state.route_workspace_words, status, st),
              nat.route_call_name(ep, T, el))
    recv = offsets[el:]
    # ---- gather + unpack -----------------------------------------------------------------------
    none = nat.Operand(None, 0, None)
    nat.check(nat.lib.dm_gather_packed_rows(fwd.data_ptr(), recv.data_ptr(), max_rows, xq, xs, int(lay.fp4),
                                            _view(buf, lay.x_q), _view(buf, lay.x_sf),
                                            _view(buf, lay.x_inv) if lay.fp4 else none, None, st),
              "dm_gather_packed_rows")
    # ---- W13 (+SwiGLU) ---------------------------------------------------------------------------
    fused = bool(p13._interleaved_fc13)
    row_inv = _view(buf, lay.x_inv) if lay.fp4 else none
    h2_quantised = False
    # few rows per expert (decode): weights on the MMA's M side, the rows on its N side
    limit_rows = _SWAPPED_MAX_ROWS[fmt] if SWAPPED_MAX_ROWS_PER_EXPERT is None else SWAPPED_MAX_ROWS_PER_EXPERT
    swapped = fused and ep * T * K <= limit_rows * E
    if swapped:
        h2_dense = lay.dense
        nat.check(nat.lib.dm_gemm_blockscaled_swapped(f, _view(buf, lay.x_q), _view(buf, lay.x_sf),
                                                      p13.fprop_data.data_ptr(), p13.fprop_scale.data_ptr(), none,
                                                      _view(buf, h2_dense), None, row_inv,
                                                      nat.ptr(p13.global_scale_inv), offsets.data_ptr(),
                                                      real.data_ptr(), el, max_rows, 2 * F, D, 1, clamped, alpha,
                                                      limit, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled_swapped(w13+swiglu)")
    elif fused and not lay.fp4:
        # MXFP8: the SwiGLU epilogue writes h2 already row-quantised, the operand of the W2 GEMM
        h2_dense = lay.dense
        h2_quantised = True
        nat.check(nat.lib.dm_gemm_blockscaled_swiglu_mxfp8(_view(buf, lay.x_q), _view(buf, lay.x_sf),
                                                           p13.fprop_data.data_ptr(), p13.fprop_scale.data_ptr(),
                                                           _view(buf, lay.h_q), _view(buf, lay.h_sf),
                                                           offsets.data_ptr(), el, max_rows, 2 * F, D, clamped, alpha,
                                                           limit, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled_swiglu_mxfp8")
    elif fused:
        h2_dense = lay.dense
        nat.check(nat.lib.dm_gemm_blockscaled(f, _view(buf, lay.x_q), _view(buf, lay.x_sf), p13.fprop_data.data_ptr(),
                                              p13.fprop_scale.data_ptr(), none, _view(buf, h2_dense), None, row_inv,
                                              nat.ptr(p13.global_scale_inv), offsets.data_ptr(), el, max_rows, 2 * F,
                                              D, 1, clamped, alpha, limit, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled(w13+swiglu)")
    else:
        h2_dense = lay.h2_dense
        nat.check(nat.lib.dm_gemm_blockscaled(f, _view(buf, lay.x_q), _view(buf, lay.x_sf), p13.fprop_data.data_ptr(),
                                              p13.fprop_scale.data_ptr(), _view(buf, lay.dense), none, None, row_inv,
                                              nat.ptr(p13.global_scale_inv), offsets.data_ptr(), el, max_rows, 2 * F,
                                              D, 0, 0, 1.0, 0.0, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled(w13)")
        nat.check(nat.lib.dm_swiglu_fwd(buf.data_ptr() + lay.dense, None, buf.data_ptr() + h2_dense, None,
                                        recv.data_ptr(), max_rows, F, clamped, alpha, limit, None, 0.0, None, st),
                  "dm_swiglu_fwd")
    # ---- quantise h2 rows --------------------------------------------------------------------------
    h2_ptr = buf.data_ptr() + h2_dense
    if h2_quantised:
        pass
    elif lay.fp4:
        # padding rows of the 128-row-padded expert groups (null scatter pointer) are skipped
        nat.check(nat.lib.dm_quant_nvfp4_token_live(sct.data_ptr(), h2_ptr, recv.data_ptr(), max_rows, F,
                                                    buf.data_ptr() + lay.h_q, hq, buf.data_ptr() + lay.h_sf, 0, 1,
                                                    buf.data_ptr() + lay.h_inv, 4, st), "dm_quant_nvfp4_token_live(h2)")
    else:
        nat.check(nat.lib.dm_quant_mxfp8_row(h2_ptr, recv.data_ptr(), max_rows, F, buf.data_ptr() + lay.h_q, 0,
                                             buf.data_ptr() + lay.h_sf, 0, 1, st), "dm_quant_mxfp8_row(h2)")
    # ---- W2 + scatter to the owners' combine buffers ---------------------------------------------
    if swapped:
        nat.check(nat.lib.dm_gemm_blockscaled_swapped(f, _view(buf, lay.h_q), _view(buf, lay.h_sf),
                                                      p2.fprop_data.data_ptr(), p2.fprop_scale.data_ptr(), none, none,
                                                      sct.data_ptr(), _view(buf, lay.h_inv) if lay.fp4 else none,
                                                      nat.ptr(p2.global_scale_inv), offsets.data_ptr(),
                                                      real.data_ptr(), el, max_rows, D, F, 0, 0, 1.0, 0.0, None,
                                                      state.num_sms, status, st), "dm_gemm_blockscaled_swapped(w2)")
    else:
        nat.check(nat.lib.dm_gemm_blockscaled(f, _view(buf, lay.h_q), _view(buf, lay.h_sf), p2.fprop_data.data_ptr(),
                                              p2.fprop_scale.data_ptr(), none, none, sct.data_ptr(),
                                              _view(buf, lay.h_inv) if lay.fp4 else none,
                                              nat.ptr(p2.global_scale_inv), offsets.data_ptr(), el, max_rows, D, F, 0,
                                              0, 1.0, 0.0, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled(w2)")
    state.barrier(state.combine)
    out = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
    post = options.experts_output_postprocess
    if isinstance(post, RMSNormPostprocess):
        from ._postprocess import validate_rmsnorm

        validate_rmsnorm(post, config=cfg, training=False, x_dtype=out.dtype)
        nat.check(nat.lib.dm_rmsnorm_combine_fwd(
            state.combine.local().data_ptr(), scores.data_ptr(), int(scores.dtype == torch.bfloat16), ids.data_ptr(),
            int(ids.dtype == torch.int64), nat.ptr(post.weight), float(post.gain_center), float(post.eps),
            int(post.norm_output_dtype == torch.bfloat16), int(bool(post.use_kahan)), out.data_ptr(), None, T, K, D,
            None, None, None, 0, st), "dm_rmsnorm_combine_fwd")
    else:
        nat.check(nat.lib.dm_scale_and_sum(state.combine.local().data_ptr(), scores.data_ptr(),
                                           int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                           int(ids.dtype == torch.int64), out.data_ptr(), T, K, D, None, None, None, 0,
                                           st), "dm_scale_and_sum")
    state.last_recv = recv
    return out


# =============================================================================================
# MXFP8 training
# =============================================================================================
class _Bump:
    """Carves 256-byte aligned views out of one cached workspace tensor."""

    def __init__(self, buf: torch.Tensor):
        self.buf, self.off = buf, 0

    def take(self, nbytes: int) -> nat.Operand:
        start = self.off
        self.off = (start + nbytes + 255) // 256 * 256
        if self.off > self.buf.numel():
            raise RuntimeError("block-scaled training workspace is too small")
        return nat.Operand(self.buf.data_ptr() + start, self.buf.numel() - start, None)


def _sf_rows_bytes(rows: int, dim: int) -> int:
    """Blocked scales of a row-quantised [rows, dim] operand."""
    return _blocked_group_bytes(rows, dim // 32)


def _sf_cols_bytes(rows: int, dim: int) -> int:
    """Blocked scales of a column-quantised [rows, dim] operand (feature = row index, rows/32 = column index)."""
    return _blocked_group_bytes(dim, (rows + 31) // 32)


def _train_workspace(state, R: int) -> torch.Tensor:
    cfg = state.config
    D, F = cfg.hidden_dim, cfg.intermediate_dim
    need = R * (2 * D + D + D + 2 * F + 4 * F + 2 * F + 2 * F) \
        + _sf_rows_bytes(R, D) + _sf_cols_bytes(R, D) + _sf_rows_bytes(R, 2 * F) + _sf_cols_bytes(R, 2 * F) \
        + 256 * max(D, 2 * F) * 2 + 16 * 256
    ws = getattr(state, "_bs_train_ws", None)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=state.device)
        state._bs_train_ws = ws
    return ws


def _ptr(op: nat.Operand) -> int:
    return op.base


def _training_weights(w13_param, w2_param, p13, p2, cfg):
    """Training operands: one E4M3 qdata per weight (32x32 tiles) with forward and transposed scales."""
    if p13 is not None:
        if p13.dgrad_scale is None or p2.dgrad_scale is None or p13._interleaved_fc13:
            raise ValueError("training needs weights prepared without inference=True / fuse_swiglu")
        return p13, p2
    el = w13_param.numel() // (2 * cfg.intermediate_dim * cfg.hidden_dim)
    w13 = w13_param.detach().reshape(el, 2 * cfg.intermediate_dim, cfg.hidden_dim)
    w2 = w2_param.detach().reshape(el, cfg.hidden_dim, cfg.intermediate_dim)
    return prepare_weight(w13, cfg), prepare_weight(w2, cfg)


class _TrainCall:
    __slots__ = ("T", "R", "offsets", "recv", "fwd", "bwd", "sct", "h1", "x_col", "x_col_sf", "h2_col", "h2_col_sf",
                 "h3", "p13", "p2", "rstd", "planned", "per_rank", "need", "cond", "fwd_state", "fwd_table",
                 "callback_state")


# MXFP8 training keeps its activations in the context's arena, placed by the device planner (saved bundles in the
# selected activation slot, transient ones in the shared scratch, save-or-recompute decided on the device from every
# rank's row counts: dist_moe/_blockscaled.py:1150-1420, 2284-2512).  Contexts without activation slots and calls that
# ask for the SwiGLU clip counters (which need a dense h2 the plan has no room for) use per-call tensors instead.
PLANNED_ARENA = True

# groups of the planner's offset tables, nine entries each
_A_Q, _B_Q, _C, _A_SF, _B_SF, _SRC_X, _SRC_Y, _COL_Q, _COL_SF = range(9)


def _route_training(state, x, ids, options, c: "_TrainCall"):
    """publish -> barrier -> routing tables (rows of every expert padded to 128)."""
    cfg = state.config
    D, K, E = cfg.hidden_dim, cfg.top_k, cfg.num_experts
    T, dev, el, ep = x.shape[0], x.device, state.e_local, state.ep
    st, status = nat.stream_ptr(), state.status.data_ptr()
    nat.check(nat.lib.dm_publish(x.data_ptr(), ids.data_ptr(), int(ids.dtype == torch.int64),
                                 state.dispatch.local().data_ptr(), state.routing.local().data_ptr(), T, D, K, E,
                                 int(options.validate_expert_ids), status, st), "dm_publish")
    state.barrier(state.dispatch)
    size = max((ep * T * min(K, el) + el * 127 + 127) // 128 * 128, 128)
    c.T = T
    c.R = min(size, state.capacity_rows // 128 * 128)
    counts = torch.empty(el, dtype=torch.int32, device=dev)
    c.per_rank = torch.empty(ep, dtype=torch.int32, device=dev)
    c.offsets = torch.empty(el + 1, dtype=torch.int32, device=dev)
    c.fwd = torch.empty(size, dtype=torch.int64, device=dev)
    c.bwd = torch.empty(size, dtype=torch.int64, device=dev)
    c.sct = torch.empty(size, dtype=torch.int64, device=dev)
    stride = D * 2
    nat.check(nat.lib.dm_route(state.routing.peer_ptrs.data_ptr(), state.dispatch.peer_ptrs.data_ptr(),
                               state.combine.peer_ptrs.data_ptr(), state.rank, ep, T, K, E, stride, stride, stride, 128,
                               state.capacity_rows, size, counts.data_ptr(), c.per_rank.data_ptr(),
                               c.offsets.data_ptr(), c.fwd.data_ptr(), c.bwd.data_ptr(), c.sct.data_ptr(),
                               state.route_workspace.data_ptr(), state.route_workspace_words, status, st),
              nat.route_call_name(ep, T, el))
    c.recv = c.offsets[el:]


def _storage_array(state):
    import ctypes

    arr = getattr(state, "_planner_storage", None)
    if arr is None:
        arr = (ctypes.c_int * 6)(*planner_storage(state.config.block_scaled.format))
        state._planner_storage = arr
    return arr


def _mxfp8_forward_planned(state, x, ids, scores, p13, p2, options, need_h3: bool, hooks=None):
    cfg = state.config
    D, F, K = cfg.hidden_dim, cfg.intermediate_dim, cfg.top_k
    T, dev, el, ep = x.shape[0], x.device, state.e_local, state.ep
    st, status = nat.stream_ptr(), state.status.data_ptr()
    clamped = 1 if cfg.activation == "swiglu_clamped" else 0
    alpha, limit = float(cfg.swiglu_alpha), float(cfg.swiglu_limit)
    c = _TrainCall()
    c.planned, c.p13, c.p2 = True, p13, p2
    c.h1 = c.x_col = c.x_col_sf = c.h2_col = c.h2_col_sf = c.h3 = c.callback_state = None
    _route_training(state, x, ids, options, c)
    R, recv = c.R, c.recv.data_ptr()
    c.need = torch.empty(1, dtype=torch.uint8, device=dev)
    c.cond = torch.empty(1, dtype=torch.int32, device=dev)
    c.fwd_state = torch.empty(10, dtype=torch.int64, device=dev)  # [x, -, h1, -, h3, x_row, x_col, h2_row, h2_col, slot]
    c.fwd_table = torch.empty(18, dtype=torch.int64, device=dev)
    nat.check(nat.lib.dm_plan_fwd_blockscaled(
        recv, c.per_rank.data_ptr(), None, state.saved_bytes.data_ptr(), state.buffer_offsets.data_ptr(),
        state.peak_min_free.data_ptr(), c.need.data_ptr(), c.cond.data_ptr(), c.fwd_state.data_ptr(),
        c.fwd_table.data_ptr(), state.slot_selector.data_ptr(), state.moe_layer_id.data_ptr(), ep,
        cfg.max_num_local_input_tokens, K, D, F, _storage_array(state), state.capacity_rows, state.slot_bytes,
        state.num_slots, state.num_layers_in_slot, 0, 0, 0, 0, 0, status, st), "dm_plan_fwd_blockscaled")
    fs, ft = c.fwd_state, c.fwd_table
    A = lambda table, group, entry: state.arena_operand(table[group * 9 + entry:group * 9 + entry + 1])  # noqa: E731
    none = nat.Operand(None, 0, None)
    arena = state.arena.data_ptr()
    # a layer that will be recomputed keeps only its dense input
    nat.check(nat.lib.dm_cond_copy(x.data_ptr(), None, arena, fs[0:1].data_ptr(), T * D * 2, c.cond.data_ptr(), 1, st),
              "dm_cond_copy(save x)")
    # dispatch: the routed rows are pulled through the pointer table by the quantiser itself
    nat.check(nat.lib.dm_quant_mxfp8_rowcol_gather_at(c.fwd.data_ptr(), recv, R, D, A(ft, 0, _A_Q), A(ft, 0, _A_SF),
                                                      A(ft, 0, _COL_Q), A(ft, 0, _COL_SF), None, st),
              "dm_quant_mxfp8_rowcol_gather_at(x)")
    nat.check(nat.lib.dm_gemm_blockscaled(0, A(ft, 0, _A_Q), A(ft, 0, _A_SF), p13.fprop_data.data_ptr(),
                                          p13.fprop_scale.data_ptr(), A(ft, 0, _C), none, None, none, None,
                                          c.offsets.data_ptr(), el, R, 2 * F, D, 0, 0, 1.0, 0.0, None, state.num_sms,
                                          status, st), "dm_gemm_blockscaled(w13)")
    nat.check(nat.lib.dm_swiglu_fwd_quant_mxfp8_rowcol_at(A(ft, 1, _SRC_X), recv, R, F, clamped, alpha, limit,
                                                          A(ft, 1, _A_Q), A(ft, 1, _A_SF), A(ft, 1, _COL_Q),
                                                          A(ft, 1, _COL_SF), None, st),
              "dm_swiglu_fwd_quant_mxfp8_rowcol_at")
    nat.check(nat.lib.dm_gemm_blockscaled(0, A(ft, 1, _A_Q), A(ft, 1, _A_SF), p2.fprop_data.data_ptr(),
                                          p2.fprop_scale.data_ptr(), none, none, c.sct.data_ptr(), none, None,
                                          c.offsets.data_ptr(), el, R, D, F, 0, 0, 1.0, 0.0, None, state.num_sms, status,
                                          st), "dm_gemm_blockscaled(w2)")
    state.barrier(state.combine)
    out = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
    post = options.experts_output_postprocess
    is_norm = isinstance(post, RMSNormPostprocess)
    c.rstd = None
    if is_norm:
        from ._postprocess import rmsnorm_combine_forward

        c.rstd = rmsnorm_combine_forward(state, c, post, scores, ids, out, save=True)
    elif post is not None:
        if hooks is None:
            raise RuntimeError("a callable expert-output post-process runs on the eager path only")
        hooks.postprocess_forward(state, c, post, scores, ids, out, save=True)  # keeps its own input and output
    else:
        # the expert outputs go to the slot (when the layer is saved) only if the score gradient will read them
        nat.check(nat.lib.dm_scale_and_sum(state.combine.local().data_ptr(), scores.data_ptr(),
                                           int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                           int(ids.dtype == torch.int64), out.data_ptr(), T, K, D,
                                           arena if need_h3 else None, fs[4:5].data_ptr() if need_h3 else None,
                                           c.cond.data_ptr() if need_h3 else None, 0, st), "dm_scale_and_sum")
    state.last_recv = c.recv
    state.last_train_call = c
    return out, c


def _mxfp8_backward_planned(state, c: _TrainCall, x_shape, ids, scores, w13_param, w2_param, grad_out, options, needs,
                            wgrad_explicit=(None, None), hooks=None):
    from ._bf16 import _wgrad_destination

    cfg = state.config
    D, F, K = cfg.hidden_dim, cfg.intermediate_dim, cfg.top_k
    T, R, el, ep, dev = c.T, c.R, state.e_local, state.ep, grad_out.device
    st, status = nat.stream_ptr(), state.status.data_ptr()
    clamped = 1 if cfg.activation == "swiglu_clamped" else 0
    alpha, limit = float(cfg.swiglu_alpha), float(cfg.swiglu_limit)
    need_x, need_scores, need_w13, need_w2 = needs
    recv, offs = c.recv.data_ptr(), c.offsets.data_ptr()
    none = nat.Operand(None, 0, None)
    arena, combine = state.arena.data_ptr(), state.combine.local().data_ptr()
    bo = torch.empty(16, dtype=torch.int64, device=dev)
    bt = torch.empty(54, dtype=torch.int64, device=dev)
    nat.check(nat.lib.dm_plan_bwd_blockscaled(
        recv, c.per_rank.data_ptr(), state.saved_bytes.data_ptr(), state.buffer_offsets.data_ptr(),
        state.peak_min_free.data_ptr(), c.need.data_ptr(), c.fwd_state.data_ptr(), bo.data_ptr(), bt.data_ptr(),
        state.moe_layer_id.data_ptr(), ep, cfg.max_num_local_input_tokens, K, D, F, _storage_array(state),
        state.capacity_rows, state.slot_bytes, state.num_slots, 0, 0, status, st), "dm_plan_bwd_blockscaled")
    A = lambda group, entry: state.arena_operand(bt[group * 9 + entry:group * 9 + entry + 1])  # noqa: E731
    fs, cond = c.fwd_state, c.cond
    post = options.experts_output_postprocess
    is_norm = isinstance(post, RMSNormPostprocess)
    is_callback = post is not None and not is_norm  # the callable kept its own input and output (eager path)
    # ---- recompute block: every launch is a no-op unless the forward chose to recompute this layer ------------
    with record_function("dist_moe_recompute"):
        nat.check(nat.lib.dm_cond_copy(arena, fs[0:1].data_ptr(), state.dispatch.local().data_ptr(), None, T * D * 2,
                                       cond.data_ptr(), 1, st), "dm_cond_copy(republish x)")
        state.barrier(state.dispatch, cond)
        nat.check(nat.lib.dm_quant_mxfp8_rowcol_gather_at(c.fwd.data_ptr(), recv, R, D, A(0, _A_Q), A(0, _A_SF),
                                                          A(0, _COL_Q), A(0, _COL_SF), cond.data_ptr(), st),
                  "dm_quant_mxfp8_rowcol_gather_at(x recompute)")
        nat.check(nat.lib.dm_gemm_blockscaled(0, A(0, _A_Q), A(0, _A_SF), c.p13.fprop_data.data_ptr(),
                                              c.p13.fprop_scale.data_ptr(), A(0, _C), none, None, none, None, offs, el,
                                              R, 2 * F, D, 0, 0, 1.0, 0.0, cond.data_ptr(), state.num_sms, status, st),
                  "dm_gemm_blockscaled(w13 recompute)")
        nat.check(nat.lib.dm_swiglu_fwd_quant_mxfp8_rowcol_at(A(1, _SRC_X), recv, R, F, clamped, alpha, limit,
                                                              A(1, _A_Q), A(1, _A_SF), A(1, _COL_Q), A(1, _COL_SF),
                                                              cond.data_ptr(), st),
                  "dm_swiglu_fwd_quant_mxfp8_rowcol_at(recompute)")
        if (need_scores or is_norm) and not is_callback:
            # the expert outputs again, scattered to their owners' combine buffers
            nat.check(nat.lib.dm_gemm_blockscaled(0, A(1, _A_Q), A(1, _A_SF), c.p2.fprop_data.data_ptr(),
                                                  c.p2.fprop_scale.data_ptr(), none, none, c.sct.data_ptr(), none, None,
                                                  offs, el, R, D, F, 0, 0, 1.0, 0.0, cond.data_ptr(), state.num_sms,
                                                  status, st), "dm_gemm_blockscaled(w2 recompute)")
            if is_norm:  # the fused RMSNorm backward works on the expert outputs in place in the combine buffer
                nat.check(nat.lib.dm_cond_copy(arena, fs[4:5].data_ptr(), combine, None, T * K * D * 2,
                                               cond.data_ptr(), 0, st), "dm_cond_copy(load h3)")
            state.barrier(state.combine, cond)
    # ---- gradient with respect to the expert outputs and the scores ------------------------------------------
    grad_scores = torch.empty(T, K, dtype=torch.float32, device=dev) if need_scores else None
    if is_norm:
        from ._postprocess import rmsnorm_combine_backward

        rmsnorm_combine_backward(state, c, post, grad_out, scores, ids, grad_scores)
    elif is_callback:
        hooks.postprocess_backward(state, c, grad_out, scores, ids, grad_scores)
    elif need_scores:
        nat.check(nat.lib.dm_broadcast_and_scale_select(grad_out.data_ptr(), scores.data_ptr(),
                                                        int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                                        int(ids.dtype == torch.int64), arena, fs[4:5].data_ptr(),
                                                        combine, cond.data_ptr(), combine, nat.ptr(grad_scores), T, K,
                                                        D, st), "dm_broadcast_and_scale")
    else:
        nat.check(nat.lib.dm_broadcast_and_scale(grad_out.data_ptr(), scores.data_ptr(),
                                                 int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                                 int(ids.dtype == torch.int64), None, None, combine, None, T, K, D, st),
                  "dm_broadcast_and_scale")
    state.barrier(state.combine)
    # ---- W2 ----------------------------------------------------------------------------------------------------
    nat.check(nat.lib.dm_quant_mxfp8_rowcol_gather_at(c.sct.data_ptr(), recv, R, D, A(2, _A_Q), A(2, _A_SF),
                                                      A(2, _COL_Q) if need_w2 else none,
                                                      A(2, _COL_SF) if need_w2 else none, None, st),
              "dm_quant_mxfp8_rowcol_gather_at(grad_h3)")
    nat.check(nat.lib.dm_gemm_blockscaled_dgrad(A(2, _A_Q), A(2, _A_SF), c.p2.fprop_data.data_ptr(),
                                                c.p2.dgrad_scale.data_ptr(), A(2, _C), None, offs, el, R, F, D, None,
                                                state.num_sms, status, st), "dm_gemm_blockscaled_dgrad(w2)")
    grad_w13 = grad_w2 = None
    owners = options.wgrad_parameter_owners or (None, None)
    if need_w2:
        dst, acc, ret = _wgrad_destination(w2_param, (el, D, F), options, cfg, owners[1], wgrad_explicit[1], hooks, "w2")
        nat.check(nat.lib.dm_gemm_blockscaled_wgrad_compact(A(3, _A_Q), A(3, _A_SF), A(3, _B_Q), A(3, _B_SF),
                                                            dst.data_ptr(), int(dst.dtype == torch.float32), acc, offs,
                                                            el, R, D, F, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled_wgrad(w2)")
        grad_w2 = dst.view(w2_param.shape) if ret else None
        if hooks is not None:
            grad_w2 = hooks.wgrad_postprocess("w2", grad_w2)
    # ---- SwiGLU backward, W13 ---------------------------------------------------------------------------------
    if need_x or need_w13:
        nat.check(nat.lib.dm_swiglu_bwd_quant_mxfp8_at(A(4, _SRC_Y), A(4, _SRC_X), recv, R, F, clamped, alpha, limit,
                                                       A(4, _A_Q) if need_x else none, A(4, _A_SF) if need_x else none,
                                                       A(4, _COL_Q) if need_w13 else none,
                                                       A(4, _COL_SF) if need_w13 else none, st),
                  "dm_swiglu_bwd_quant_mxfp8_at")
    if need_x:
        nat.check(nat.lib.dm_gemm_blockscaled_dgrad(A(4, _A_Q), A(4, _A_SF), c.p13.fprop_data.data_ptr(),
                                                    c.p13.dgrad_scale.data_ptr(), none, c.bwd.data_ptr(), offs, el, R, D,
                                                    2 * F, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled_dgrad(w13)")
    if need_w13:
        dst, acc, ret = _wgrad_destination(w13_param, (el, 2 * F, D), options, cfg, owners[0], wgrad_explicit[0], hooks,
                                           "w13")
        nat.check(nat.lib.dm_gemm_blockscaled_wgrad_compact(A(5, _A_Q), A(5, _A_SF), A(5, _B_Q), A(5, _B_SF),
                                                            dst.data_ptr(), int(dst.dtype == torch.float32), acc, offs,
                                                            el, R, 2 * F, D, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled_wgrad(w13)")
        grad_w13 = dst.view(w13_param.shape) if ret else None
        if hooks is not None:
            grad_w13 = hooks.wgrad_postprocess("w13", grad_w13)
    grad_x = None
    # unconditional, as in the reference (dist_moe/api.py:2580): peers may still be reading this rank's combine buffer
    state.barrier(state.dispatch)
    if need_x:
        grad_x = torch.empty(x_shape, dtype=torch.bfloat16, device=dev)
        nat.check(nat.lib.dm_scale_and_sum(state.dispatch.local().data_ptr(), None, 0, ids.data_ptr(),
                                           int(ids.dtype == torch.int64), grad_x.data_ptr(), T, K, D, None, None, None,
                                           0, st), "dm_scale_and_sum(reduce_from_topk)")
    if grad_scores is not None and scores.dtype != torch.float32:
        grad_scores = grad_scores.to(scores.dtype)
    return grad_x, grad_scores, grad_w13, grad_w2


def _mxfp8_forward(state, x, ids, scores, p13, p2, options, need_h3: bool):
    cfg = state.config
    D, F, K, E = cfg.hidden_dim, cfg.intermediate_dim, cfg.top_k, cfg.num_experts
    T, dev, el, ep = x.shape[0], x.device, state.e_local, state.ep
    st, status = nat.stream_ptr(), state.status.data_ptr()
    clamped = 1 if cfg.activation == "swiglu_clamped" else 0
    alpha, limit = float(cfg.swiglu_alpha), float(cfg.swiglu_limit)
    nat.check(nat.lib.dm_publish(x.data_ptr(), ids.data_ptr(), int(ids.dtype == torch.int64),
                                 state.dispatch.local().data_ptr(), state.routing.local().data_ptr(), T, D, K, E,
                                 int(options.validate_expert_ids), status, st), "dm_publish")
    state.barrier(state.dispatch)
    size = max((ep * T * min(K, el) + el * 127 + 127) // 128 * 128, 128)
    c = _TrainCall()
    c.T, c.p13, c.p2, c.planned = T, p13, p2, False
    R = c.R = min(size, state.capacity_rows // 128 * 128)
    counts = torch.empty(el, dtype=torch.int32, device=dev)
    per_rank = torch.empty(ep, dtype=torch.int32, device=dev)
    c.offsets = torch.empty(el + 1, dtype=torch.int32, device=dev)
    c.fwd = torch.empty(size, dtype=torch.int64, device=dev)
    c.bwd = torch.empty(size, dtype=torch.int64, device=dev)
    c.sct = torch.empty(size, dtype=torch.int64, device=dev)
    stride = D * 2
    nat.check(nat.lib.dm_route(state.routing.peer_ptrs.data_ptr(), state.dispatch.peer_ptrs.data_ptr(),
                               state.combine.peer_ptrs.data_ptr(), state.rank, ep, T, K, E, stride, stride, stride, 128,
                               state.capacity_rows, size, counts.data_ptr(), per_rank.data_ptr(), c.offsets.data_ptr(),
                               c.fwd.data_ptr(), c.bwd.data_ptr(), c.sct.data_ptr(), state.route_workspace.data_ptr(),
                               state.route_workspace_words, status, st), nat.route_call_name(ep, T, el))
    c.recv = c.offsets[el:]
    recv = c.recv.data_ptr()
    ws = _Bump(_train_workspace(state, R))
    xg = ws.take(R * D * 2)
    xq, xsf = ws.take(R * D), ws.take(_sf_rows_bytes(R, D))
    h2 = ws.take(R * F * 2)
    hq, hsf = ws.take(R * F), ws.take(_sf_rows_bytes(R, F))
    # saved for the backward
    c.h1 = torch.empty(R, 2 * F, dtype=torch.bfloat16, device=dev)
    c.x_col = torch.empty(R, D, dtype=torch.uint8, device=dev)
    c.x_col_sf = torch.empty(_sf_cols_bytes(R, D), dtype=torch.uint8, device=dev)
    c.h2_col = torch.empty(R, F, dtype=torch.uint8, device=dev)
    c.h2_col_sf = torch.empty(_sf_cols_bytes(R, F), dtype=torch.uint8, device=dev)
    none = nat.Operand(None, 0, None)
    full = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    # dispatch: the routed rows are pulled through the pointer table by the quantiser itself
    nat.check(nat.lib.dm_quant_mxfp8_rowcol_gather(c.fwd.data_ptr(), recv, R, D, _ptr(xq), _ptr(xsf), c.x_col.data_ptr(),
                                                   c.x_col_sf.data_ptr(), st), "dm_quant_mxfp8_rowcol_gather(x)")
    nat.check(nat.lib.dm_gemm_blockscaled(0, xq, xsf, p13.fprop_data.data_ptr(), p13.fprop_scale.data_ptr(), full(c.h1),
                                          none, None, none, None, c.offsets.data_ptr(), el, R, 2 * F, D, 0, 0, 1.0, 0.0,
                                          None, state.num_sms, status, st), "dm_gemm_blockscaled(w13)")
    clip = options.swiglu_clip_stats_out_3
    if clip is not None:
        clip.zero_()
    if clip is None:
        nat.check(nat.lib.dm_swiglu_fwd_quant_mxfp8_rowcol(c.h1.data_ptr(), recv, R, F, clamped, alpha, limit, _ptr(hq),
                                                           _ptr(hsf), c.h2_col.data_ptr(), c.h2_col_sf.data_ptr(), st),
                  "dm_swiglu_fwd_quant_mxfp8_rowcol")
    else:  # the clip counters live in the standalone activation kernel
        nat.check(nat.lib.dm_swiglu_fwd(c.h1.data_ptr(), None, _ptr(h2), None, recv, R, F, clamped, alpha, limit,
                                        nat.ptr(clip), float(options.swiglu_clip_limit), None, st), "dm_swiglu_fwd")
        nat.check(nat.lib.dm_quant_mxfp8_rowcol(_ptr(h2), recv, R, F, _ptr(hq), _ptr(hsf), c.h2_col.data_ptr(),
                                                c.h2_col_sf.data_ptr(), st), "dm_quant_mxfp8_rowcol(h2)")
    nat.check(nat.lib.dm_gemm_blockscaled(0, hq, hsf, p2.fprop_data.data_ptr(), p2.fprop_scale.data_ptr(), none, none,
                                          c.sct.data_ptr(), none, None, c.offsets.data_ptr(), el, R, D, F, 0, 0, 1.0,
                                          0.0, None, state.num_sms, status, st), "dm_gemm_blockscaled(w2)")
    state.barrier(state.combine)
    out = torch.empty(T, D, dtype=torch.bfloat16, device=dev)
    post = options.experts_output_postprocess
    is_norm = isinstance(post, RMSNormPostprocess)
    # the expert outputs are kept for the score gradient, and always for the backward of the fused RMSNorm
    c.h3 = torch.empty(T * K * D, dtype=torch.bfloat16, device=dev) if (need_h3 or is_norm) else None
    c.rstd = None
    if is_norm:
        from ._postprocess import rmsnorm_combine_forward

        c.rstd = rmsnorm_combine_forward(state, c, post, scores, ids, out, save=True, save_to=c.h3)
    elif post is not None:
        raise NotImplementedError("callable expert-output post-processing runs on the BF16 eager path only")
    else:
        nat.check(nat.lib.dm_scale_and_sum(state.combine.local().data_ptr(), scores.data_ptr(),
                                           int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                           int(ids.dtype == torch.int64), out.data_ptr(), T, K, D, nat.ptr(c.h3), None,
                                           None, 0, st), "dm_scale_and_sum")
    state.last_recv = c.recv
    return out, c


def _mxfp8_backward(state, c: _TrainCall, x_shape, ids, scores, w13_param, w2_param, grad_out, options, needs,
                    wgrad_explicit=(None, None)):
    from ._bf16 import _wgrad_destination

    cfg = state.config
    D, F, K = cfg.hidden_dim, cfg.intermediate_dim, cfg.top_k
    T, R, el, dev = c.T, c.R, state.e_local, grad_out.device
    st, status = nat.stream_ptr(), state.status.data_ptr()
    clamped = 1 if cfg.activation == "swiglu_clamped" else 0
    alpha, limit = float(cfg.swiglu_alpha), float(cfg.swiglu_limit)
    need_x, need_scores, need_w13, need_w2 = needs
    recv, offs = c.recv.data_ptr(), c.offsets.data_ptr()
    none = nat.Operand(None, 0, None)
    full = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    ws = _Bump(_train_workspace(state, R))
    dyg = ws.take(R * D * 2)
    dyq, dysf = ws.take(R * D), ws.take(_sf_rows_bytes(R, D))
    dyc, dycsf = ws.take(R * D), ws.take(_sf_cols_bytes(R, D))
    dh2 = ws.take(R * F * 2)
    dh1 = ws.take(R * 2 * F * 2)
    d1q, d1sf = ws.take(R * 2 * F), ws.take(_sf_rows_bytes(R, 2 * F))
    d1c, d1csf = ws.take(R * 2 * F), ws.take(_sf_cols_bytes(R, 2 * F))
    combine = state.combine.local().data_ptr()
    grad_scores = torch.empty(T, K, dtype=torch.float32, device=dev) if need_scores else None
    post = options.experts_output_postprocess
    if isinstance(post, RMSNormPostprocess):
        from ._postprocess import rmsnorm_combine_backward

        rmsnorm_combine_backward(state, c, post, grad_out, scores, ids, grad_scores, h3=c.h3)
    else:
        nat.check(nat.lib.dm_broadcast_and_scale(grad_out.data_ptr(), scores.data_ptr(),
                                                 int(scores.dtype == torch.bfloat16), ids.data_ptr(),
                                                 int(ids.dtype == torch.int64),
                                                 c.h3.data_ptr() if need_scores else None, None, combine,
                                                 nat.ptr(grad_scores), T, K, D, st), "dm_broadcast_and_scale")
    state.barrier(state.combine)
    # ---- W2 ----------------------------------------------------------------------------------
    if need_w2:
        nat.check(nat.lib.dm_quant_mxfp8_rowcol_gather(c.sct.data_ptr(), recv, R, D, _ptr(dyq), _ptr(dysf), _ptr(dyc),
                                                       _ptr(dycsf), st), "dm_quant_mxfp8_rowcol_gather(dy)")
    else:
        nat.check(nat.lib.dm_gather_rows(c.sct.data_ptr(), recv, _ptr(dyg), None, D * 2, R, None, st),
                  "dm_gather_rows(grad_h3)")
        nat.check(nat.lib.dm_quant_mxfp8_row(_ptr(dyg), recv, R, D, _ptr(dyq), 0, _ptr(dysf), 0, 1, st),
                  "dm_quant_mxfp8_row(dy)")
    nat.check(nat.lib.dm_gemm_blockscaled_dgrad(dyq, dysf, c.p2.fprop_data.data_ptr(), c.p2.dgrad_scale.data_ptr(), dh2,
                                                None, offs, el, R, F, D, None, state.num_sms, status, st),
              "dm_gemm_blockscaled_dgrad(w2)")
    grad_w13 = grad_w2 = None
    owners = options.wgrad_parameter_owners or (None, None)
    if need_w2:
        dst, acc, ret = _wgrad_destination(w2_param, (el, D, F), options, cfg, owners[1], wgrad_explicit[1])
        nat.check(nat.lib.dm_gemm_blockscaled_wgrad(dyc, dycsf, full(c.h2_col), full(c.h2_col_sf), dst.data_ptr(),
                                                    int(dst.dtype == torch.float32), acc, offs, el, R, D, F, None,
                                                    state.num_sms, status, st), "dm_gemm_blockscaled_wgrad(w2)")
        grad_w2 = dst.view(w2_param.shape) if ret else None
    # ---- SwiGLU backward, W13 ---------------------------------------------------------------
    if need_x or need_w13:
        # grad_h1 goes straight from the SwiGLU backward arithmetic into its quantised copies
        nat.check(nat.lib.dm_swiglu_bwd_quant_mxfp8(c.h1.data_ptr(), _ptr(dh2), recv, R, F, clamped, alpha, limit,
                                                    _ptr(d1q) if need_x else None, _ptr(d1sf) if need_x else None,
                                                    _ptr(d1c) if need_w13 else None, _ptr(d1csf) if need_w13 else None,
                                                    st), "dm_swiglu_bwd_quant_mxfp8")
    if need_x:
        nat.check(nat.lib.dm_gemm_blockscaled_dgrad(d1q, d1sf, c.p13.fprop_data.data_ptr(),
                                                    c.p13.dgrad_scale.data_ptr(), none, c.bwd.data_ptr(), offs, el, R, D,
                                                    2 * F, None, state.num_sms, status, st),
                  "dm_gemm_blockscaled_dgrad(w13)")
    if need_w13:
        dst, acc, ret = _wgrad_destination(w13_param, (el, 2 * F, D), options, cfg, owners[0], wgrad_explicit[0])
        nat.check(nat.lib.dm_gemm_blockscaled_wgrad(d1c, d1csf, full(c.x_col), full(c.x_col_sf), dst.data_ptr(),
                                                    int(dst.dtype == torch.float32), acc, offs, el, R, 2 * F, D, None,
                                                    state.num_sms, status, st), "dm_gemm_blockscaled_wgrad(w13)")
        grad_w13 = dst.view(w13_param.shape) if ret else None
    grad_x = None
    # unconditional, as in the reference (dist_moe/api.py:2580): peers may still be reading this rank's combine buffer
    state.barrier(state.dispatch)
    if need_x:
        grad_x = torch.empty(x_shape, dtype=torch.bfloat16, device=dev)
        nat.check(nat.lib.dm_scale_and_sum(state.dispatch.local().data_ptr(), None, 0, ids.data_ptr(),
                                           int(ids.dtype == torch.int64), grad_x.data_ptr(), T, K, D, None, None, None,
                                           0, st), "dm_scale_and_sum(reduce_from_topk)")
    if grad_scores is not None and scores.dtype != torch.float32:
        grad_scores = grad_scores.to(scores.dtype)
    return grad_x, grad_scores, grad_w13, grad_w2


class _Mxfp8Function(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, ids, scores, w13_param, w2_param, state, options, p13, p2):
        p13, p2 = _training_weights(w13_param, w2_param, p13, p2, state.config)
        planned = PLANNED_ARENA and state.num_slots > 0 and options.swiglu_clip_stats_out_3 is None
        with record_function("dist_moe_forward"):
            forward = _mxfp8_forward_planned if planned else _mxfp8_forward
            out, call = forward(state, x.detach().contiguous(), ids, scores.detach(), p13, p2, options,
                                need_h3=scores.requires_grad)
        ctx.state, ctx.call, ctx.options, ctx.x_shape = state, call, options, x.shape
        ctx.save_for_backward(ids, scores, w13_param, w2_param)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        ids, scores, w13_param, w2_param = ctx.saved_tensors
        needs = (ctx.needs_input_grad[0], ctx.needs_input_grad[2], ctx.needs_input_grad[3], ctx.needs_input_grad[4])
        with torch.cuda.device(ctx.state.device), record_function("dist_moe_backward"):
            backward = _mxfp8_backward_planned if ctx.call.planned else _mxfp8_backward
            gx, gs, gw13, gw2 = backward(ctx.state, ctx.call, ctx.x_shape, ids, scores.detach(), w13_param, w2_param,
                                         grad_out.contiguous(), ctx.options, needs)
        return gx, None, gs, gw13, gw2, None, None, None, None


class _EagerMxfp8Function(torch.autograd.Function):
    """MXFP8 training with Python callbacks inside the launch sequence: compute weights materialised from their
    sources (and quantised) in the forward and again before the backward, a callable post-process on the expert
    outputs, named destinations and post-processing of the weight gradients."""

    @staticmethod
    def _weights(options, w13_source, w2_source, state):
        from ._eager import _compute_weights

        w13, w2 = _compute_weights(options, w13_source, w2_source, state)
        return w13, w2, prepare_weight(w13, state.config), prepare_weight(w2, state.config)

    @staticmethod
    def forward(ctx, x, ids, scores, w13_source, w2_source, state, options):
        from ._eager import CallbackHooks

        if options.inplace_wgrad_accum and options.weights_preprocess_fn is not None:
            raise ValueError("inplace_wgrad_accum needs compute weights that own their gradient; it cannot be combined "
                             "with weights_preprocess_fn")
        hooks = CallbackHooks(options)
        _, _, p13, p2 = _EagerMxfp8Function._weights(options, w13_source, w2_source, state)
        with record_function("dist_moe_forward"):
            out, call = _mxfp8_forward_planned(state, x.detach().contiguous(), ids, scores.detach(), p13, p2, options,
                                               need_h3=scores.requires_grad, hooks=hooks)
        call.p13 = call.p2 = None  # re-materialised before the backward, as the reference does
        ctx.state, ctx.call, ctx.options, ctx.hooks, ctx.x_shape = state, call, options, hooks, x.shape
        ctx.save_for_backward(ids, scores, w13_source, w2_source)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        ids, scores, w13_source, w2_source = ctx.saved_tensors
        state, options, call = ctx.state, ctx.options, ctx.call
        # compute weights are materialised again, as in the forward; the weight gradients take their shapes and are
        # handed back in the sources' shapes
        w13, w2, call.p13, call.p2 = _EagerMxfp8Function._weights(options, w13_source, w2_source, state)
        needs = (ctx.needs_input_grad[0], ctx.needs_input_grad[2], ctx.needs_input_grad[3], ctx.needs_input_grad[4])
        with torch.cuda.device(state.device), record_function("dist_moe_backward"):
            gx, gs, g13, g2 = _mxfp8_backward_planned(state, call, ctx.x_shape, ids, scores.detach(), w13, w2,
                                                      grad_out.contiguous(), options, needs, hooks=ctx.hooks)
        if g13 is not None:
            g13 = g13.reshape(w13_source.shape)
        if g2 is not None:
            g2 = g2.reshape(w2_source.shape)
        return gx, None, gs, g13, g2, None, None
