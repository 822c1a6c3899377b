"""Run the reference's own GPU code on a Blackwell GPU, stage by stage, and keep what it returns.

    python tests/golden/gen_golden_gpu.py --reference <dir holding the dist_moe package> --out <dir>

Every stage runs in a child process with a time limit, so a JIT failure of one stage (the reference pins
newer Triton / CuTe-DSL releases than this image carries) is recorded as text and the next stage still
runs; a stage that times out ends the whole run, nothing is retried.  ``<out>/ref_gpu_probe.json`` lists
stage -> "ok" or the exception; the ``*.npz`` files hold inputs and the reference's outputs byte for byte.

Nothing here spins on another rank: quantisers and element-wise kernels are single-launch; the end-to-end
stages use PyTorch's fake process group with one rank, for which the reference aliases peer buffers to
local memory and skips its signal-pad barriers (dist_moe/_triton_ops.py:79), and keep ``T*K`` above the
reference's cooperative decode-routing threshold so only its general routing kernels run.

Stages (reference entry point each one calls):
  triton_quant   dist_moe/kernels/triton_quantization/blockscaled_quantize.py:3471 quantize_block_scaled
                 (MXFP8 rows, natural + blocked scales; NVFP4 rows with a per-token global scale) and
                 dist_moe/_blockscaled.py:141 _prepare_nvfp4_weight_operands (plain and W13-interleaved)
  triton_axes    blockscaled_quantize.py:3785 quantize_block_scaled_axes (MXFP8 32x1 columns, 32x32 tiles)
  cute_quant     dist_moe/_quantization.py:66 quantize_for_format (MXFP8 row/col/both/tile, CuTe DSL)
  cute_nvfp4     dist_moe/kernels/blockscaled_quantize.py:5080 _quantize_nvfp4_per_token
  prep_mxfp8     dist_moe/_blockscaled.py:2874 _prepare_mxfp8_weight_op (training, inference, interleaved)
  elementwise    dist_moe/kernels/triton/swiglu.py:272/671, broadcast_n_reduction.py:70/386/723
  e2e_bf16       dist_moe.routed_experts, BF16 forward + backward, one rank, small shape (outputs kept)
  e2e_bf16_c2    the same at T=4096 D=2048 F=1408 E=64 K=6 (timed with CUDA events, sampled outputs kept)
  e2e_mxfp8 / e2e_nvfp4   block-scaled training / prepared-weight inference, small shapes
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import time
import traceback
from pathlib import Path

STAGES = ["triton_quant", "triton_axes", "cute_quant", "cute_nvfp4", "prep_mxfp8", "elementwise", "e2e_bf16",
          "e2e_bf16_c2", "e2e_mxfp8", "e2e_nvfp4"]


def _i16(t):
    return t.detach().cpu().contiguous().view(__import__("torch").int16).numpy()


def _u8(t):
    import torch

    t = t.detach().cpu().contiguous()
    return t.view(torch.uint8).numpy()


def _wide(rows, cols, seed, lo=-6, hi=4):
    import torch

    g = torch.Generator().manual_seed(seed)
    return (torch.randn(rows, cols, generator=g) * torch.logspace(lo, hi, rows)[:, None]).bfloat16()


def stage_triton_quant(out):
    import numpy as np
    import torch

    from dist_moe._blockscaled import _prepare_nvfp4_weight_operands
    from dist_moe.kernels.triton_quantization import blockscaled_quantize as TQ
    from dist_moe.kernels.triton_quantization.formats import BlockScaledFormatId as F, ScaleFactorLayoutId as L
    from dist_moe.kernels.triton_quantization.global_scale import (GlobalScaleGranularity, expand_global_scale_for_rows,
                                                                     wire_inverse)

    a = _wide(37, 256, 2027)
    a[0, :32] = 0
    a[1, 5] = float("inf")
    a[2, 70] = float("nan")
    a[3, :64] = torch.tensor(2.0**-120).bfloat16()
    a[4, :32] = 448.0
    a[5, :32] = 449.0
    a[6, :32] = torch.tensor([2.0**k for k in range(-16, 16)]).bfloat16()
    b = (torch.randn(200, 384, generator=torch.Generator().manual_seed(1)) * 0.02).bfloat16()
    c = _wide(256, 512, 3, -5, 3)
    blob = {"a": _i16(a), "b": _i16(b), "c": _i16(c)}
    for name, x in (("a", a), ("b", b), ("c", c)):
        for lname, lid in (("nat", L.NATURAL.value), ("blk", L.CUBLAS_BLOCKED.value)):
            q, s = TQ.quantize_block_scaled(x.cuda(), format_id=F.MXFP8_E4M3.value, layout_id=lid, is_a=True)
            blob[f"{name}_{lname}_q"], blob[f"{name}_{lname}_s"] = _u8(q), _u8(s)
    np.savez_compressed(out / "quant_mxfp8_gpu.npz", **blob)

    blob = {}
    # weights: plain and with the fused-SwiGLU row interleave (gate[0:8], up[0:8], gate[8:16], ...)
    w = (torch.randn(3, 160, 256, generator=torch.Generator().manual_seed(7)) * 0.02).bfloat16()
    w13 = (torch.randn(2, 256, 256, generator=torch.Generator().manual_seed(8)) * 0.02).bfloat16()
    w13[1] *= 37.0
    for name, t, fuse in (("w", w, False), ("w13", w13, True), ("w13plain", w13, False)):
        q, s, gs, gsi = _prepare_nvfp4_weight_operands(t.cuda(), fuse)
        blob[name] = _i16(t)
        blob[f"{name}_q"], blob[f"{name}_s"] = _u8(q), _u8(s)
        blob[f"{name}_gs"], blob[f"{name}_gsi"] = gs.cpu().numpy(), gsi.cpu().numpy()
    # activations: per-token global scale = 2688 * reciprocal(max(row amax, 1e-8)), natural scale layout
    for name, x in (("t", _wide(33, 256, 5, -2, 2)), ("u", _wide(128, 1024, 6, -3, 3))):
        xd = x.cuda()
        amax = torch.linalg.vector_norm(xd, ord=float("inf"), dim=-1, dtype=torch.float32).clamp(min=1e-8)
        row_scale = 2688.0 * torch.reciprocal(amax)
        gs_rows = expand_global_scale_for_rows(row_scale, xd.shape, device=xd.device,
                                               granularity=GlobalScaleGranularity.PER_TOKEN)
        q, s = TQ.quantize_block_scaled(xd, format_id=F.NVFP4.value, layout_id=L.NATURAL.value, is_a=True,
                                        global_scale=gs_rows)
        blob[name] = _i16(x)
        blob[f"{name}_q"], blob[f"{name}_s"] = _u8(q), _u8(s)
        blob[f"{name}_row_scale"], blob[f"{name}_inv"] = row_scale.cpu().numpy(), wire_inverse(row_scale).cpu().numpy()
    np.savez_compressed(out / "quant_nvfp4_gpu.npz", **blob)


def stage_triton_axes(out):
    import numpy as np
    import torch

    from dist_moe.kernels.triton_quantization import blockscaled_quantize as TQ
    from dist_moe.kernels.triton_quantization.formats import (AxisMask, BlockScaledFormatId as F,
                                                              ScaleFactorLayoutId as L, ScaleReduction)

    x = _wide(256, 384, 11, -4, 3)
    blob = {"x": _i16(x)}
    for lname, lid in (("nat", L.NATURAL.value), ("blk", L.CUBLAS_BLOCKED.value)):
        q, s = TQ.quantize_block_scaled_axes(x.cuda(), format_id=F.MXFP8_E4M3.value, axis_mask=AxisMask.M.value,
                                             scale_reduction_id=ScaleReduction.ONE_D.value, layout_id=lid)
        blob[f"col_{lname}_q"], blob[f"col_{lname}_s"] = _u8(q), _u8(s)
        blob[f"col_{lname}_q_shape"], blob[f"col_{lname}_q_stride"] = np.array(q.shape), np.array(q.stride())
        (qc, sc), (qr, sr) = TQ.quantize_block_scaled_axes(
            x.cuda(), format_id=F.MXFP8_E4M3.value, axis_mask=(AxisMask.M | AxisMask.K).value,
            scale_reduction_id=ScaleReduction.TWO_D.value, layout_id=lid)
        blob[f"tile_{lname}_q"], blob[f"tile_{lname}_s_row"], blob[f"tile_{lname}_s_col"] = _u8(qr), _u8(sr), _u8(sc)
    np.savez_compressed(out / "quant_mxfp8_axes_gpu.npz", **blob)


def stage_cute_quant(out):
    import numpy as np
    import torch

    from dist_moe._quantization import quantize_for_format
    from dist_moe.formats import BlockScaledFormat

    x = _wide(256, 512, 13, -4, 3)
    blob = {"x": _i16(x)}
    fmt = BlockScaledFormat.MXFP8_E4M3
    q, s = quantize_for_format(x.cuda(), fmt, block_size=((1, 32),))
    blob["row_q"], blob["row_s"] = _u8(q), _u8(s)
    q, s = quantize_for_format(x.cuda(), fmt, block_size=((32, 1),))
    blob["col_q"], blob["col_s"] = _u8(q), _u8(s)
    blob["col_q_shape"], blob["col_q_stride"] = np.array(q.shape), np.array(q.stride())
    (qc, sc), (qr, sr) = quantize_for_format(x.cuda(), fmt, block_size=((32, 1), (1, 32)))
    blob["both_col_q"], blob["both_col_s"], blob["both_row_q"], blob["both_row_s"] = _u8(qc), _u8(sc), _u8(qr), _u8(sr)
    (qc, sc), (qr, sr) = quantize_for_format(x.cuda(), fmt, block_size=((32, 32),))
    blob["tile_q"], blob["tile_s_col"], blob["tile_s_row"] = _u8(qr), _u8(sc), _u8(sr)
    np.savez_compressed(out / "quant_mxfp8_cute_gpu.npz", **blob)


def stage_cute_nvfp4(out):
    import numpy as np

    from dist_moe.formats import ScaleFactorLayout
    from dist_moe.kernels.blockscaled_quantize import _quantize_nvfp4_per_token

    blob = {}
    for name, x in (("t", _wide(33, 256, 5, -2, 2)), ("u", _wide(128, 1024, 6, -3, 3)), ("v", _wide(16, 7168, 9, -1, 1))):
        q, s, inv = _quantize_nvfp4_per_token(x.cuda(), layout=ScaleFactorLayout.NATURAL)
        blob[name] = _i16(x)
        blob[f"{name}_q"], blob[f"{name}_s"], blob[f"{name}_inv"] = _u8(q), _u8(s), inv.cpu().numpy()
    np.savez_compressed(out / "quant_nvfp4_token_cute_gpu.npz", **blob)


def stage_prep_mxfp8(out):
    import numpy as np
    import torch

    from dist_moe._blockscaled import _prepare_mxfp8_weight_op

    w = (torch.randn(2, 256, 384, generator=torch.Generator().manual_seed(21)) * 0.02).bfloat16()
    w[1] *= 11.0
    blob = {"w": _i16(w)}
    for name, inference, fuse in (("train", False, False), ("infer", True, False), ("infer_fused", True, True)):
        q, sf, sd = _prepare_mxfp8_weight_op(w.cuda(), inference, fuse)
        blob[f"{name}_q"], blob[f"{name}_sf"], blob[f"{name}_sd"] = _u8(q), _u8(sf), _u8(sd)
    np.savez_compressed(out / "prep_mxfp8_weight_gpu.npz", **blob)


def stage_elementwise(out):
    import numpy as np
    import torch

    from dist_moe.kernels.triton.broadcast_n_reduction import broadcast_and_scale, reduce_from_topk, scale_and_sum
    from dist_moe.kernels.triton.swiglu import swiglu_bwd, swiglu_fwd

    g = torch.Generator().manual_seed(33)
    h1 = (torch.randn(96, 512, generator=g) * 4).bfloat16()
    dz = (torch.randn(96, 256, generator=g)).bfloat16()
    blob = {"h1": _i16(h1), "dz": _i16(dz)}
    for name, kw in (("plain", {}), ("clamped", dict(clamped=True, alpha=1.702, limit=7.0))):
        z = swiglu_fwd(h1.cuda(), **kw)
        dxy = swiglu_bwd(dz.cuda(), h1.cuda(), **kw)
        blob[f"z_{name}"], blob[f"dxy_{name}"] = _i16(z), _i16(dxy)
    T, K, D = 40, 4, 256
    x = torch.randn(T, K, D, generator=g).bfloat16()
    sc = torch.rand(T, K, generator=g)
    ids = torch.randint(0, 8, (T, K), generator=g)
    ids[torch.rand(T, K, generator=g) < 0.15] = -1
    dy = torch.randn(T, D, generator=g).bfloat16()
    y, _ = scale_and_sum(x.cuda(), sc.cuda(), ids.cuda(), return_copy=False)
    r = reduce_from_topk(x.cuda(), ids.cuda())
    dx, dscale = broadcast_and_scale(dy.cuda(), sc.cuda(), x.cuda(), ids.cuda())
    blob.update(x=_i16(x), scale=sc.numpy(), ids=ids.numpy(), dy=_i16(dy), y=_i16(y), r=_i16(r), dx=_i16(dx),
                dscale=dscale.float().cpu().numpy())
    np.savez_compressed(out / "elementwise_gpu.npz", **blob)


def _fake_group():
    import torch.distributed as dist
    import torch.testing._internal.distributed.fake_pg  # noqa: F401  (registers the "fake" backend)

    if not dist.is_initialized():
        dist.init_process_group("fake", rank=0, world_size=1)
    return dist.group.WORLD


def _e2e_inputs(T, D, F, E, K, seed, w_std, device):
    import torch

    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, D, generator=g).bfloat16()
    logits = torch.randn(T, E, generator=g)
    top = torch.topk(torch.softmax(logits, -1), K, dim=-1)
    scores = (top.values / top.values.sum(-1, keepdim=True)).float()
    ids = top.indices.to(torch.int64)
    w13 = (torch.randn(E, 2 * F, D, generator=g) * w_std).bfloat16()
    w2 = (torch.randn(E, D, F, generator=g) * w_std).bfloat16()
    return [t.to(device) for t in (x, ids, scores, w13, w2)]


def _run_bf16(out, tag, T, D, F, E, K, w_std, timed_iters):
    import numpy as np
    import torch

    import dist_moe

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    group = _fake_group()
    cfg = dist_moe.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                          max_moe_layers_per_activation_slot=1, device_scratch_capacity_factor=1.0,
                          activation_slot_capacity_factor=1.0, num_activation_slots=1)
    ctx = dist_moe.create_context(group=group, config=cfg, device=dev, emulate_peer_buffers=True)
    try:
        x, ids, scores, w13, w2 = _e2e_inputs(T, D, F, E, K, 1000, w_std, dev)
        for t in (x, scores, w13, w2):
            t.requires_grad_(True)
        outp = dist_moe.routed_experts(x, ids, scores, w13, w2, ctx)
        outp.float().sum().backward()
        torch.cuda.synchronize()
        rows = slice(0, min(T, 64))
        blob = dict(shape=np.array([T, D, F, E, K]), w_std=np.float64(w_std), out=_i16(outp[rows]), gx=_i16(x.grad[rows]),
                    gs=scores.grad[rows].float().cpu().numpy(), gw13_e0=_i16(w13.grad[0, :64]), gw2_e0=_i16(w2.grad[0, :64]),
                    gw13_last=_i16(w13.grad[E - 1, -64:]), gw2_last=_i16(w2.grad[E - 1, -64:]))
        if T * D <= 1 << 16:
            blob.update(x=_i16(x), ids=ids.cpu().numpy(), scores=scores.detach().cpu().numpy(), w13=_i16(w13), w2=_i16(w2))
        np.savez_compressed(out / f"e2e_bf16_{tag}_gpu.npz", **blob)
        timing = None
        if timed_iters:
            opts = dist_moe.ExecutionOptions(inplace_wgrad_accum=True)
            for it in range(3 + timed_iters):
                if it == 3:
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                o = dist_moe.routed_experts(x, ids, scores, w13, w2, ctx, options=opts)
                o.float().sum().backward()
            e1.record()
            torch.cuda.synchronize()
            timing = e0.elapsed_time(e1) / timed_iters
        return {"ms_per_step_eager": timing}
    finally:
        ctx.close()


def stage_e2e_bf16(out):
    return _run_bf16(out, "small", 192, 256, 256, 4, 2, 1.0, 0)


def stage_e2e_bf16_c2(out):
    return _run_bf16(out, "c2", 4096, 2048, 1408, 64, 6, 0.02, 10)


def _run_blockscaled(out, tag, fmt_name, inference, T, D, F, E, K):
    import numpy as np
    import torch

    import dist_moe

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    group = _fake_group()
    fmt = getattr(dist_moe.BlockScaledFormat, fmt_name)
    cfg = dist_moe.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                          max_moe_layers_per_activation_slot=1, device_scratch_capacity_factor=1.0,
                          activation_slot_capacity_factor=None if inference else 1.0,
                          num_activation_slots=0 if inference else 1, inference=inference,
                          block_scaled=dist_moe.BlockScaledConfig(format=fmt, pipeline="staged"))
    ctx = dist_moe.create_context(group=group, config=cfg, device=dev, emulate_peer_buffers=True)
    try:
        x, ids, scores, w13, w2 = _e2e_inputs(T, D, F, E, K, 1000, 0.02, dev)
        blob = dict(shape=np.array([T, D, F, E, K]), x=_i16(x), ids=ids.cpu().numpy(), scores=scores.cpu().numpy(),
                    w13=_i16(w13), w2=_i16(w2))
        if inference:
            p13 = dist_moe.prepare_block_scaled_weight(w13, cfg.block_scaled, inference=True)
            p2 = dist_moe.prepare_block_scaled_weight(w2, cfg.block_scaled, inference=True)
            with torch.no_grad():
                outp = dist_moe.routed_experts(x, ids, scores, p13, p2, ctx)
            blob["out"] = _i16(outp)
        else:
            for t in (x, scores, w13, w2):
                t.requires_grad_(True)
            outp = dist_moe.routed_experts(x, ids, scores, w13, w2, ctx)
            outp.float().sum().backward()
            blob.update(out=_i16(outp), gx=_i16(x.grad), gw13=_i16(w13.grad), gw2=_i16(w2.grad))
        torch.cuda.synchronize()
        np.savez_compressed(out / f"e2e_{tag}_gpu.npz", **blob)
    finally:
        ctx.close()


def stage_e2e_mxfp8(out):
    _run_blockscaled(out, "mxfp8_train", "MXFP8_E4M3", False, 256, 256, 256, 4, 2)


def stage_e2e_nvfp4(out):
    _run_blockscaled(out, "nvfp4_infer", "NVFP4", True, 256, 256, 256, 4, 2)


def _child(stage, reference, out):
    sys.path.insert(0, reference)
    res = {"stage": stage}
    try:
        extra = globals()[f"stage_{stage}"](Path(out))
        res["status"] = "ok"
        if extra:
            res.update(extra)
    except BaseException as e:  # noqa: BLE001 -- the text of every failure is the result
        res["status"] = f"{type(e).__name__}: {str(e)[:600]}"
        res["trace_tail"] = traceback.format_exc()[-1500:]
    print("PROBE_RESULT " + json.dumps(res), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="baseline/_ref")
    ap.add_argument("--out", default=str(Path(__file__).resolve().parent))
    ap.add_argument("--stages", default=",".join(STAGES))
    ap.add_argument("--child", default="")
    ap.add_argument("--limit", type=int, default=240, help="seconds per stage")
    args = ap.parse_args()
    if args.child:
        _child(args.child, args.reference, args.out)
        return
    Path(args.out).mkdir(parents=True, exist_ok=True)
    results = {}
    import torch

    results["_stack"] = dict(torch=torch.__version__, gpu=torch.cuda.get_device_name(0))
    for mod in ("triton", "cutlass"):
        try:
            results["_stack"][mod] = __import__(mod).__version__
        except Exception as e:  # noqa: BLE001
            results["_stack"][mod] = f"missing: {e}"
    for stage in args.stages.split(","):
        t0 = time.time()
        try:
            p = subprocess.run([sys.executable, __file__, "--reference", args.reference, "--out", args.out, "--child", stage],
                               capture_output=True, text=True, timeout=args.limit, env=dict(os.environ, TRITON_INTERPRET="0"))
        except subprocess.TimeoutExpired:
            results[stage] = {"status": f"timed out after {args.limit} s; run ended here"}
            break
        line = [ln for ln in p.stdout.splitlines() if ln.startswith("PROBE_RESULT ")]
        results[stage] = json.loads(line[-1][13:]) if line else {"status": f"child exited {p.returncode}",
                                                                  "stderr_tail": p.stderr[-1500:]}
        results[stage]["seconds"] = round(time.time() - t0, 1)
        print(stage, "->", results[stage]["status"][:200], flush=True)
        (Path(args.out) / "ref_gpu_probe.json").write_text(json.dumps(results, indent=1))
    (Path(args.out) / "ref_gpu_probe.json").write_text(json.dumps(results, indent=1))


if __name__ == "__main__":
    main()
