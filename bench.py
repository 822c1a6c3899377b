"""Benchmark of the routed-expert layer (BF16 training layer, forward + backward).

Workload (the reference's EP8 BF16 training configuration): T=4096 tokens per rank, D=2048, F=1408, E=64 experts
sharded over the ranks (E_local = 64 / N), top-6 softmax routing renormalised to 1, plain
SwiGLU, weight gradients accumulated in place into ``parameter.grad``.  Inputs are seeded
synthetic data: x ~ N(0,1), weights ~ N(0,0.02), router logits ~ N(0,1).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

For N > 1 launch one process per GPU with ``python -m torch.distributed.run``.  Rank 0 prints
one JSON line.  ``--impl reference`` times the unmodified reference installed under ``baseline/_ref``
on one GPU through its own ``routed_experts`` (one-rank group, all experts local); if that is not
available it times the CPU restatement of the reference's math (``oracle/moe.py``; the reference has
no CPU path) on the host cores, on a bounded token sample.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

T, D, F, E, K = 4096, 2048, 1408, 64, 6
CPU_SAMPLE_TOKENS = int(os.environ.get("DIST_MOE_BENCH_CPU_TOKENS", "256"))  # bounded CPU sample
CPU_STEPS, CPU_WARMUP = 3, 1  # the same in both places that time the CPU restatement
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return json.loads(path.read_text()), "measured"
        except Exception:
            pass
    return FALLBACK_PEAKS, "fallback"


def kernel_source_digest() -> str:
    """Digest of the grouped-GEMM sources; a recorded ncu traffic figure is only reported for the sources it was
    captured on."""
    import hashlib

    h = hashlib.sha256()
    for name in ("gemm_bf16.cu", "gemm_common.cuh", "common.cuh"):
        h.update((ROOT / "dist_moe_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:16]


def recorded_dram_traffic():
    """(bytes per working GEMM launch, note) from profiles/grouped_gemm_dram_traffic.json, or (None, why)."""
    path = ROOT / "profiles" / "grouped_gemm_dram_traffic.json"
    try:
        rec = json.loads(path.read_text())
    except (OSError, ValueError):
        return None, "no ncu capture recorded"
    if rec.get("kernel_source_digest") != kernel_source_digest():
        return None, f"stale: captured on kernel sources {rec.get('kernel_source_digest')}, commit {rec.get('commit')}"
    return rec["dram_bytes_per_launch"], f"ncu dram read+write per launch, N=1 capture on commit {rec.get('commit')}"


def sampled_parity(dm, ctx, opts, x, ids, scores, w13, w2, grad_out, sample=64):
    """One forward + backward outside every timed region, checked on a token sample against the CPU oracle: an output
    row, and the gradients of that token's input and scores, depend only on the token's own K experts, so 64 tokens
    need 64 x K small products on the host.  Bounds are the reference's BF16 ones (tests/test_dist_moe.py:317-325)."""
    from oracle import moe as oracle_moe

    xs, ss = x.detach().clone().requires_grad_(True), scores.detach().clone().requires_grad_(True)
    out = dm.routed_experts(xs, ids, ss, w13, w2, ctx, options=opts)
    out.backward(grad_out)
    ctx.check_status()
    idx = torch.linspace(0, x.shape[0] - 1, sample).long()
    gw = torch.Generator().manual_seed(2027)
    w13_all = (torch.randn(E, 2, F, D, generator=gw) * 0.02).bfloat16().reshape(E, 2 * F, D)
    w2_all = (torch.randn(E, D, F, generator=gw) * 0.02).bfloat16()
    xr, sr = x[idx.to(x.device)].cpu().requires_grad_(True), scores[idx.to(x.device)].cpu().requires_grad_(True)
    ref = oracle_moe.moe_forward(xr, ids[idx.to(x.device)].cpu(), sr, w13_all, w2_all)
    ref.backward(grad_out[idx.to(x.device)].cpu())
    report, ok = {}, True
    for name, got, want, l2_max, cos_min in (("out", out[idx.to(x.device)], ref, 5e-3, 0.999),
                                             ("grad_x", xs.grad[idx.to(x.device)], xr.grad, 1e-2, 0.995),
                                             ("grad_scores", ss.grad[idx.to(x.device)], sr.grad, 1e-2, 0.995)):
        got, want = got.detach().float().cpu(), want.detach().float()
        l2 = ((got - want).norm() / want.norm().clamp_min(1e-30)).item()
        cos = torch.nn.functional.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
        report[name] = {"rel_l2": l2, "cosine": cos}
        ok = ok and l2 < l2_max and cos > cos_min
    return ok, report


def make_inputs(rank: int, world: int, device, tokens: int = T):
    """Seeded synthetic inputs: seed 1000+rank for tokens/router, 2027 for the weights."""
    g = torch.Generator().manual_seed(1000 + rank)
    x = torch.randn(tokens, D, generator=g).bfloat16()
    logits = torch.randn(tokens, E, generator=g)
    top = torch.topk(torch.softmax(logits, -1), K)
    scores = (top.values / top.values.sum(-1, keepdim=True)).float()
    ids = top.indices.to(torch.int64)
    e_local = E // world
    gw = torch.Generator().manual_seed(2027)
    w13_all = (torch.randn(E, 2, F, D, generator=gw) * 0.02).bfloat16()
    w2_all = (torch.randn(E, D, F, generator=gw) * 0.02).bfloat16()
    sl = slice(rank * e_local, (rank + 1) * e_local)
    return x, ids, scores, w13_all[sl].contiguous(), w2_all[sl].contiguous()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    PERIOD_MS = 20

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines: list = []
        self.marks: list[float] = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms",
                 str(self.PERIOD_MS), "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL,
                text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def mark(self):
        """Wall-clock bracket of a timed region: only samples taken between two marks are reported."""
        self.marks.append(time.time())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        windows = list(zip(self.marks[0::2], self.marks[1::2]))
        for stamp, line in self.lines:
            if windows and not any(a <= stamp <= b + 0.03 for a, b in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(steps: int, warmup: int, threads: int | None = None):
    """Forward + backward of a token sample through the eager CPU restatement (all 64 experts)."""
    from oracle import moe as oracle_moe

    cores = threads or os.cpu_count() or 1
    torch.set_num_threads(cores)
    x, ids, scores, w13, w2 = make_inputs(0, 1, "cpu", tokens=CPU_SAMPLE_TOKENS)
    w13 = w13.requires_grad_(True)
    w2 = w2.requires_grad_(True)
    times = []
    grad_out = torch.randn(CPU_SAMPLE_TOKENS, D, generator=torch.Generator().manual_seed(4000)).bfloat16()
    for i in range(warmup + steps):
        xs = x.clone().requires_grad_(True)
        ss = scores.clone().requires_grad_(True)
        t0 = time.perf_counter()
        out = oracle_moe.moe_forward(xs, ids, ss, w13, w2)
        out.backward(grad_out)
        dt = time.perf_counter() - t0
        if i >= warmup:
            times.append(dt)
    per_step = sum(times) / len(times)
    return {"value": CPU_SAMPLE_TOKENS / per_step, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{CPU_SAMPLE_TOKENS} of {T} tokens, all {E} experts, fwd+bwd, eager torch bf16 on CPU",
            "ms_per_step": per_step * 1e3}


def base_line(args, world):
    return {
        "metric": "MoE layer tokens/s (BF16 training layer, fwd+bwd), whole job",
        "unit": "tokens/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic (seeded N(0,1) tokens, N(0,0.02) weights, softmax top-6 routing)",
        "config": {
            "workload": f"BF16 training layer EP={world}: T={T} tokens/rank, D={D}, F={F}, E={E} (E_local={E // world}), "
                        f"K={K}, plain SwiGLU, fwd+bwd, in-place wgrad accumulation",
            "l2": "no flush: per-step working set (expert weights + routed activations, > 1 GB at N=1) exceeds the 126 MB L2",
        },
    }


REFERENCE_DIR = ROOT / "baseline" / "_ref"


def pipelined_e2e(dev, pinned, statics, run_step, out_host):
    """End-to-end step for either arm: every step copies its inputs from pinned host memory and its output back.
    Host->device and device->host copies run on a stream each (the link is full duplex) with two staging buffers,
    so the upload of step i+1 and the download of step i-1 overlap the kernels of step i.  Returns (step, drain)."""
    x_pin, ids_pin, scores_pin = pinned
    x_static, ids_static, scores_static = statics
    copy_stream = torch.cuda.Stream(device=dev)
    down_stream = torch.cuda.Stream(device=dev)
    stage_in = [(torch.empty_like(x_static), torch.empty_like(ids_static), torch.empty_like(scores_static))
                for _ in range(2)]
    stage_out = [torch.empty(out_host.shape, dtype=out_host.dtype, device=dev) for _ in range(2)]
    in_ready = [torch.cuda.Event() for _ in range(2)]
    in_free = [torch.cuda.Event() for _ in range(2)]
    out_free = [torch.cuda.Event() for _ in range(2)]
    state = {"k": 0, "primed": False}

    def upload(slot):
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(in_free[slot])  # the step that last read this staging buffer has finished
            xb, ib, sb = stage_in[slot]
            xb.copy_(x_pin, non_blocking=True)
            ib.copy_(ids_pin, non_blocking=True)
            sb.copy_(scores_pin, non_blocking=True)
            in_ready[slot].record(copy_stream)

    def step():
        main = torch.cuda.current_stream(dev)
        k = state["k"]
        slot = k & 1
        if not state["primed"]:
            for ev in in_free + out_free:
                ev.record(main)
            upload(slot)
            state["primed"] = True
        upload(slot ^ 1)                   # next step's inputs travel while this step computes
        main.wait_event(in_ready[slot])
        xb, ib, sb = stage_in[slot]
        x_static.copy_(xb, non_blocking=True)
        ids_static.copy_(ib, non_blocking=True)
        scores_static.copy_(sb, non_blocking=True)
        in_free[slot].record(main)
        out = run_step()
        main.wait_event(out_free[slot])    # the device->host copy that last read this output buffer is done
        stage_out[slot].copy_(out.detach(), non_blocking=True)
        done = torch.cuda.Event()
        done.record(main)
        with torch.cuda.stream(down_stream):
            down_stream.wait_event(done)
            out_host.copy_(stage_out[slot], non_blocking=True)
            out_free[slot].record(down_stream)
        state["k"] = k + 1

    def drain():
        torch.cuda.current_stream(dev).wait_stream(copy_stream)
        torch.cuda.current_stream(dev).wait_stream(down_stream)

    return step, drain



def reference_gpu_step_times(args):
    """Time the unmodified reference (installed under baseline/_ref) on GPU 0 through its own public API:
    ``dist_moe.routed_experts`` forward + backward on this benchmark's inputs with all 64 experts on one rank.

    The expert-parallel group is PyTorch's one-rank fake process group, for which the reference aliases its peer
    buffers to local memory and skips its signal-pad barriers (they spin without a bound); with one rank that is
    numerically the real thing.  Steps are CUDA-graph replays when the reference's step captures, eager calls
    otherwise.  Returns None when the reference is not installed or does not run (the caller falls back to the CPU
    restatement)."""
    if not (REFERENCE_DIR / "dist_moe" / "__init__.py").exists() or not torch.cuda.is_available():
        return None
    sys.path.insert(0, str(REFERENCE_DIR))
    try:
        import importlib

        ref = importlib.import_module("dist_moe")
        dist = importlib.import_module("torch.distributed")
        importlib.import_module("torch.testing._internal.distributed.fake_pg")  # registers the "fake" backend

        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        if not dist.is_initialized():
            dist.init_process_group("fake", rank=0, world_size=1)
        x_h, ids_h, scores_h, w13_h, w2_h = make_inputs(0, 1, dev)
        x_pin, ids_pin, scores_pin = x_h.pin_memory(), ids_h.pin_memory(), scores_h.pin_memory()
        out_host = torch.empty(T, D, dtype=torch.bfloat16).pin_memory()
        w13 = w13_h.reshape(E, 2 * F, D).to(dev).requires_grad_(True)
        w2 = w2_h.to(dev).requires_grad_(True)
        w13.grad, w2.grad = torch.zeros_like(w13), torch.zeros_like(w2)
        cfg = ref.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                         max_moe_layers_per_activation_slot=1, activation_slot_capacity_factor=1.0,
                         device_scratch_capacity_factor=1.0)
        ctx = ref.create_context(group=dist.group.WORLD, config=cfg, device=dev, emulate_peer_buffers=True)
        opts = ref.ExecutionOptions(inplace_wgrad_accum=True)
        x, ids, scores = x_h.to(dev), ids_h.to(dev), scores_h.to(dev)
        grad_out = torch.randn(T, D, generator=torch.Generator().manual_seed(4000)).bfloat16().to(dev)

        def step():
            xs, ss = x.detach().requires_grad_(True), scores.detach().requires_grad_(True)
            out = ref.routed_experts(xs, ids, ss, w13, w2, ctx, options=opts)
            out.backward(grad_out)
            return out

        warm = max(3, args.warmup)
        for _ in range(warm):
            step()
        torch.cuda.synchronize()
        graph, out_static = None, None
        if not args.no_graph:
            try:
                side = torch.cuda.Stream(device=dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    step()
                torch.cuda.current_stream(dev).wait_stream(side)
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out_static = step()
                graph.replay()
                torch.cuda.synchronize()
            except Exception as exc:  # noqa: BLE001 -- eager timing is still the reference's own code path
                print(f"[bench] reference step did not capture ({exc!r}); timing eager calls", file=sys.stderr, flush=True)
                graph = None
                torch.cuda.synchronize()

        def run_step():
            if graph is not None:
                graph.replay()
                return out_static
            return step()

        # the same pipelined harness as this repository's arm: copies on a second stream, two staging buffers
        run_e2e, drain_e2e = pipelined_e2e(dev, (x_pin, ids_pin, scores_pin), (x, ids, scores), run_step, out_host)

        def timed(fn, drain=None):
            for _ in range(2):
                fn()
            if drain is not None:
                drain()
            torch.cuda.synchronize()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            for _ in range(args.steps):
                fn()
            if drain is not None:
                drain()
            e.record()
            torch.cuda.synchronize()
            return s.elapsed_time(e) / args.steps

        sampler = ClockSampler(0)
        sampler.start()
        time.sleep(0.3)
        sampler.mark()
        ms = timed(run_step)
        e2e_ms = timed(run_e2e, drain_e2e)
        sampler.mark()
        clocks = sampler.stop()
        ctx.close()
        return {"ms": ms, "e2e_ms": e2e_ms, "warmup": warm, "mode": "cuda-graph replay" if graph is not None else "eager",
                "clocks": clocks,
                "h2d": x_pin.numel() * 2 + ids_pin.numel() * 8 + scores_pin.numel() * 4, "d2h": out_host.numel() * 2}
    except Exception as exc:  # noqa: BLE001
        print(f"[bench] the reference's GPU path did not run ({exc!r}); timing its CPU restatement", file=sys.stderr,
              flush=True)
        return None


def _reference_modules():
    import importlib

    sys.path.insert(0, str(REFERENCE_DIR))
    ref = importlib.import_module("dist_moe")
    dist = importlib.import_module("torch.distributed")
    importlib.import_module("torch.testing._internal.distributed.fake_pg")  # registers the "fake" backend
    if not dist.is_initialized():
        dist.init_process_group("fake", rank=0, world_size=1)
    return ref, dist


def _time_replays(fn, steps, warmup):
    """p50 / p90 / mean in milliseconds of ``steps`` calls, each bracketed by its own CUDA events."""
    for _ in range(max(3, warmup)):
        fn()
    torch.cuda.synchronize()
    pairs = []
    for _ in range(steps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        pairs.append((s, e))
    torch.cuda.synchronize()
    times = sorted(s.elapsed_time(e) for s, e in pairs)
    return times[len(times) // 2], times[min(len(times) - 1, (len(times) * 9) // 10)], sum(times) / len(times)


def _capture(step, dev, no_graph):
    """CUDA graph of ``step`` (or None when capture is off or fails) and its static result."""
    if no_graph:
        return None, None
    try:
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            step()
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = step()
        graph.replay()
        torch.cuda.synchronize()
        return graph, out
    except Exception as exc:  # noqa: BLE001
        print(f"[bench] step did not capture ({exc!r}); timing eager calls", file=sys.stderr, flush=True)
        torch.cuda.synchronize()
        return None, None


def reference_blockscaled(args):
    """The unmodified reference (baseline/_ref) on GPU 0 for the block-scaled workloads, one rank, same inputs as
    this repository's arm.  Both of its pipelines are tried ("mega" = its chunk-pipelined fused launch, "staged");
    the faster one that runs is the line's value, both are listed."""
    ref, dist = _reference_modules()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    tried = {}
    train = args.workload == "mxfp8-train"
    case = mxfp8_train_case(args, 0, 1, dev) if train else inference_case(args, 0, 1, dev)
    Tn, Dn, Fn, En, Kn = (case[k] for k in ("T", "D", "F", "E", "K"))
    x, ids, scores = case["x"], case["ids"], case["scores"]
    fmt = "MXFP8_E4M3" if train else case["fmt"]
    if train:
        padded = ((case["per_expert"] + 127) // 128 * 128).sum().item()
        factor = min(1.0, max(1.0, 1.02 * padded / float(Tn * Kn)))
        # leaves of their own (the reference resolves a view to its base to find the gradient's owner)
        w13 = case.pop("w13").reshape(En, 2 * Fn, Dn).clone().requires_grad_(True)
        w2 = case.pop("w2").clone().requires_grad_(True)
        w13.grad, w2.grad = torch.zeros_like(w13), torch.zeros_like(w2)
    else:
        factor = 1.0
        gen = case["weights"]()
        w13 = next(gen).reshape(En, 2 * Fn, Dn)
        w2 = next(gen)
    extra = {"activation": "swiglu_clamped", "swiglu_limit": 7.0} if (not train and case["clamped"]) else {}
    for pipeline in ("mega", "staged"):
        ctx = None
        try:
            policy = ref.BlockScaledConfig(format=getattr(ref.BlockScaledFormat, fmt), pipeline=pipeline)
            if train:
                cfg = ref.Config(max_num_local_input_tokens=Tn, hidden_dim=Dn, intermediate_dim=Fn, top_k=Kn, num_experts=En,
                                 max_moe_layers_per_activation_slot=1, block_scaled=policy,
                                 activation_slot_capacity_factor=1.0, device_scratch_capacity_factor=factor)
            else:
                cfg = ref.Config(max_num_local_input_tokens=Tn, hidden_dim=Dn, intermediate_dim=Fn, top_k=Kn, num_experts=En,
                                 max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0,
                                 block_scaled=policy, device_scratch_capacity_factor=factor, **extra)
            ctx = ref.create_context(group=dist.group.WORLD, config=cfg, device=dev, emulate_peer_buffers=True)
            if train:
                p13 = ref.prepare_block_scaled_weight(w13, policy)
                p2 = ref.prepare_block_scaled_weight(w2, policy)
                opts = ref.ExecutionOptions(inplace_wgrad_accum=True)
                grad_out = case["grad_out"]

                def step():
                    xs, ss = x.detach().requires_grad_(True), scores.detach().requires_grad_(True)
                    out = ref.routed_experts(xs, ids, ss, p13, p2, ctx, options=opts)
                    out.backward(grad_out)
                    return out
            else:
                p13 = ref.prepare_block_scaled_weight(w13, policy, inference=True, fuse_swiglu=pipeline == "mega")
                p2 = ref.prepare_block_scaled_weight(w2, policy, inference=True)

                ropts = rmsnorm_options(ref, case)
                if ropts is not None:
                    try:  # the reference admits its fused RMSNorm for top_k 2 and 8 only, and its norm kernels need
                        # a newer cutlass-dsl than some stacks carry
                        with torch.no_grad():
                            ref.routed_experts(x, ids, scores, p13, p2, ctx, options=ropts)
                    except Exception as exc:  # noqa: BLE001 -- whatever the reason, time the layer without it
                        tried.setdefault("notes", []).append(
                            f"{pipeline}: fused RMSNorm not available in the reference ({repr(exc)[:160]}); timed without it")
                        ropts = None

                def step():
                    with torch.no_grad():
                        return ref.routed_experts(x, ids, scores, p13, p2, ctx, options=ropts)
            for _ in range(3):
                step()
            torch.cuda.synchronize()
            graph, _out = _capture(step, dev, args.no_graph)
            p50, p90, mean = _time_replays(graph.replay if graph is not None else step, args.steps, args.warmup)
            tried[pipeline] = {"p50_ms": p50, "p90_ms": p90, "mean_ms": mean,
                               "step_mode": "cuda-graph replay" if graph is not None else "eager"}
            del graph, p13, p2
        except Exception as exc:  # noqa: BLE001 -- the other pipeline may still run
            tried[pipeline] = {"error": repr(exc)[:400]}
            torch.cuda.synchronize()
        finally:
            if ctx is not None:
                ctx.close()
            torch.cuda.empty_cache()
    ok = {k: v for k, v in tried.items() if isinstance(v, dict) and "mean_ms" in v}
    if not ok:
        return None, tried, case
    best = min(ok, key=lambda k: ok[k]["mean_ms"])
    return best, tried, case


def run_reference_blockscaled(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    best, tried, case = reference_blockscaled(args)
    Tn = case["T"]
    line = {"impl": "reference", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "n_gpus_used": 1, "steps": args.steps,
            "warmup": max(3, args.warmup), "unit": "tokens/s", "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "data": "synthetic, the same seeded inputs as this repository's arm",
            "metric": f"MoE layer tokens/s ({args.workload}), the reference's own kernels on one GPU",
            "config": {"workload": f"{args.workload}: T={Tn}, D={case['D']}, F={case['F']}, E={case['E']} (all local), "
                                   f"K={case['K']}; reference from baseline/_ref, one-rank fake group"},
            "pipelines": tried}
    if best is None:
        line["unavailable"] = "neither pipeline of the reference ran for this workload (errors under 'pipelines')"
    else:
        r = tried[best]
        line.update({"pipeline": best, "value": Tn / (r["mean_ms"] * 1e-3), "ms_per_step": r["mean_ms"],
                     "p50_us": r["p50_ms"] * 1e3, "p90_us": r["p90_ms"] * 1e3, "step_mode": r["step_mode"],
                     "e2e": {"value": Tn / (r["mean_ms"] * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 0,
                             "d2h_bytes_per_step": 0},
                     "cpu_baseline": {"value": Tn / (r["mean_ms"] * 1e-3), "unit": "tokens/s", "cores": 0, "kind": "reference",
                                      "sample": "not a CPU run: the unmodified reference on one B200, whole workload"}})
    print(json.dumps(line), flush=True)


def run_reference(args):
    """Reference arm: rank 0 alone works.  First choice is the reference's own GPU implementation on one GPU; if it is
    not installed or fails, the CPU restatement of its math on the host cores (a bounded token sample)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    line = base_line(args, world)
    line["impl"] = "reference"
    gpu = None if args.reference_on_cpu else reference_gpu_step_times(args)
    if gpu is not None:
        value = T / (gpu["ms"] * 1e-3)
        line["config"]["workload"] = (f"BF16 training layer, the reference's own kernels on ONE GPU (EP=1, fake one-rank group): "
                                      f"T={T} tokens, D={D}, F={F}, E={E} (all local), K={K}, plain SwiGLU, fwd+bwd, "
                                      f"in-place wgrad accumulation")
        line.update({
            "value": value, "ms_per_step": gpu["ms"], "warmup": gpu["warmup"], "n_gpus_used": 1,
            "step_mode": gpu["mode"], "clocks": gpu["clocks"],
            "e2e": {"value": T / (gpu["e2e_ms"] * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": gpu["h2d"],
                    "d2h_bytes_per_step": gpu["d2h"], "ms_per_step": gpu["e2e_ms"]},
            "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": 0, "kind": "reference",
                             "sample": "not a CPU run: the unmodified reference (baseline/_ref) on one B200, whole workload"},
            "note": "unmodified reference from baseline/_ref through dist_moe.routed_experts; its Triton and CuTe-DSL "
                    "kernels JIT on this image (torch 2.11 / triton 3.6 / cutlass-dsl 4.5)",
        })
        print(json.dumps(line), flush=True)
        return
    steps, warm = CPU_STEPS, CPU_WARMUP
    cb = cpu_baseline(steps, warm)
    line.update({
        "steps": steps, "warmup": warm,
        "value": cb["value"],
        # one step of the stated workload (T tokens) at the sample's rate; the sample itself took sample_ms_per_step
        "ms_per_step": T / cb["value"] * 1e3,
        "sample_ms_per_step": cb["ms_per_step"],
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference's math on the host cores (the reference has no CPU path); used "
                "because the reference's GPU path was not available to this run",
    })
    print(json.dumps(line), flush=True)


def bind_host_to_gpu_numa_node(dev):
    """Run this process on the cores of the NUMA node the GPU hangs off, so that the pinned staging buffers
    allocated afterwards are first-touched on that node and the copies do not cross the socket interconnect
    (eight ranks copying 34 MB per step from the wrong socket share one link).  Reads sysfs only; returns the
    node, or None when the topology is not visible or the node's cores are outside this process's cpuset."""
    try:
        p = torch.cuda.get_device_properties(dev)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except (OSError, ValueError, AttributeError):
        return None


def run_ours(args):
    import torch.distributed as dist

    import dist_moe_b200 as dm
    from dist_moe_b200 import _bf16, _native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    numa_node = bind_host_to_gpu_numa_node(dev)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")

    x_h, ids_h, scores_h, w13_h, w2_h = make_inputs(rank, world, dev)
    x_pin, ids_pin, scores_pin = x_h.pin_memory(), ids_h.pin_memory(), scores_h.pin_memory()
    w13 = w13_h.to(dev).requires_grad_(True)
    w2 = w2_h.to(dev).requires_grad_(True)
    w13.grad = torch.zeros_like(w13)
    w2.grad = torch.zeros_like(w2)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=1,
                    # slot and scratch sized 25 % above balanced routing so that random top-6 routing never
                    # forces the save-versus-recompute planner into recompute (it does at exactly 1.0 once
                    # some rank receives more than T*K rows)
                    activation_slot_capacity_factor=1.0 if world == 1 else 1.25,
                    device_scratch_capacity_factor=min(1.25, float(world)))
    ctx = dm.create_context(group=group, config=cfg, device=dev)
    opts = dm.ExecutionOptions(inplace_wgrad_accum=True)
    _bf16.FUSED_DISPATCH = not args.separate_gather
    x = x_h.to(dev)
    ids = ids_h.to(dev)
    scores = scores_h.to(dev)
    out_host = torch.empty(T, D, dtype=torch.bfloat16).pin_memory()
    # upstream gradient of the layer output: an input of the backward pass, as in a model step (seeded, resident)
    grad_out = torch.randn(T, D, generator=torch.Generator().manual_seed(4000 + rank)).bfloat16().to(dev)

    def step(xd, idd, sd):
        xs = xd.requires_grad_(True)
        ss = sd.requires_grad_(True)
        out = dm.routed_experts(xs, idd, ss, w13, w2, ctx, options=opts)
        out.backward(grad_out)
        return out

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, steps, drain=None):
        sync_all()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        if drain is not None:
            drain()                        # the end event waits for the copies still in flight
        e.record()
        sync_all()
        ms = torch.tensor([s.elapsed_time(e)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # started early: the first sample takes nvidia-smi a few hundred milliseconds
    for _ in range(max(3, args.warmup)):
        step(x.detach().clone(), ids, scores.detach().clone())
    ctx.check_status()

    # ---- one step = one CUDA-graph replay of routed_experts forward + backward (static input buffers) ----
    # The reference documents graph capture of the layer as the deployment mode; the kernels are the same as in
    # eager mode, every data-dependent decision is taken on the device.  --no-graph times the eager calls.
    x_static, ids_static, scores_static = x.clone(), ids.clone(), scores.clone()
    graph, out_static, launches_per_step = None, None, None
    l0 = _native.LAUNCHES[0]
    step(x_static.detach(), ids_static, scores_static.detach())
    launches_per_step = _native.LAUNCHES[0] - l0
    if not args.no_graph:
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                step(x_static.detach(), ids_static, scores_static.detach())
            torch.cuda.current_stream(dev).wait_stream(side)
            sync_all()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                out_static = step(x_static.detach(), ids_static, scores_static.detach())
        except Exception as exc:  # capture is an optimisation of the harness, not of the kernels
            print(f"[bench] CUDA-graph capture failed ({exc!r}); timing eager calls", file=sys.stderr, flush=True)
            graph = None
    sync_all()
    ctx.check_status()

    def run_step():
        if graph is not None:
            graph.replay()
            return out_static
        return step(x_static.detach(), ids_static, scores_static.detach())

    for _ in range(3):
        run_step()
    sampler.mark()
    total_ms = timed(run_step, args.steps)
    sampler.mark()
    launches = launches_per_step * args.steps
    ctx.check_status()

    # ---- end to end: every step copies its inputs from pinned host memory and its output back, all inside
    # the timed region (copies pipelined on a second stream; the reference arm uses the same harness)
    step_e2e, drain_e2e = pipelined_e2e(dev, (x_pin, ids_pin, scores_pin), (x_static, ids_static, scores_static),
                                        run_step, out_host)

    for _ in range(2):
        step_e2e()
    drain_e2e()
    sampler.mark()
    e2e_ms = timed(step_e2e, args.steps, drain_e2e)
    sampler.mark()
    clocks = sampler.stop() if rank == 0 else None  # samples of the two timed regions
    ctx.check_status()
    # the same copies with no layer step between them: what the host side alone sustains with all ranks copying
    idle_out = out_static if out_static is not None else torch.empty(T, D, dtype=torch.bfloat16, device=dev)
    copy_step, copy_drain = pipelined_e2e(dev, (x_pin, ids_pin, scores_pin), (x_static, ids_static, scores_static),
                                          lambda: idle_out, out_host)
    copies_ms = timed(copy_step, args.steps, copy_drain)

    # ---- GEMM timing pass: the same K steps once more, eager, every grouped-GEMM launch bracketed by CUDA events
    _bf16.PROFILE = []
    timed(lambda: step(x_static.detach(), ids_static, scores_static.detach()), args.steps)
    events, _bf16.PROFILE = _bf16.PROFILE, None
    ctx.check_status()

    # ---- roofline of the dominant kernel (the grouped tcgen05 GEMM, all launches of the timed region)
    torch.cuda.synchronize()
    gemm_ms = sum(s.elapsed_time(e) for name, s, e in events if name.startswith("gemm"))
    n_gemm = sum(1 for name, _, _ in events if name.startswith("gemm"))
    breakdown = {}
    for name, s_ev, e_ev in events:
        breakdown.setdefault(name, []).append(s_ev.elapsed_time(e_ev))
    breakdown = {k: round(1e3 * sum(v) / len(v), 1) for k, v in breakdown.items()}
    rows = int(ctx._state.last_recv_rows()) if hasattr(ctx._state, "last_recv_rows") else T * K
    flops_step = 18.0 * rows * D * F
    pk, pk_kind = peaks()
    peak_tf = pk.get("bf16_tflops_sustained") or pk["bf16_tflops"]
    achieved = flops_step * args.steps / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    roofline = {
        "kernel": "grouped_gemm_kernel<fprop|dgrad|wgrad> (tcgen05; 6 working launches per step, "
                  "recompute launches are predicated off)",
        "bound": "tensor",
        "achieved": achieved,
        "peak": peak_tf,
        "peak_source": f"{pk_kind} bf16_tflops_sustained",
        "unit": "TFLOP/s",
        "frac": achieved / peak_tf if achieved else None,
        "flops_per_launch": flops_step / 6.0,
        "avg_launch_ms": gemm_ms / n_gemm if n_gemm else None,
        "launches": n_gemm,
        "timing": "CUDA events around every grouped-GEMM launch in an eager pass of the same K steps",
    }
    traffic, traffic_note = recorded_dram_traffic() if world == 1 else (None, "not captured for N > 1")
    roofline["traffic"] = traffic
    roofline["traffic_unit"] = f"bytes per launch ({traffic_note})"

    # ---- NVLink: bytes this rank moves to or from peers inside the four GEMM launches that carry the exchange
    nvlink = None
    if world > 1:
        local_rows = int(((ids_h // (E // world)) == rank).sum().item())
        remote_bytes = max(0, rows - local_rows) * D * 2
        nvlink = {"remote_bytes_per_launch": remote_bytes, "peak": 900.0, "unit": "GB/s per direction",
                  "note": "remote rows x D x 2 bytes / CUDA-event time of the whole launch (GEMM included): a lower "
                          "bound on the link rate while it overlaps the tensor cores; rank 0"}
        for key, name in (("dispatch_pull_w13_fprop", "gemm_fprop_dispatch(w13)"), ("combine_push_w2_fprop", "gemm_fprop(w2)"),
                          ("dispatch_pull_w2_dgrad", "gemm_dgrad_dispatch(w2)"), ("combine_push_w13_dgrad", "gemm_dgrad(w13)")):
            if breakdown.get(name):
                nvlink[key] = {"us": breakdown[name], "GBps": remote_bytes / (breakdown[name] * 1e-6) / 1e9,
                               "frac": remote_bytes / (breakdown[name] * 1e-6) / 1e9 / 900.0}

    parity_ok, parity = sampled_parity(dm, ctx, opts, x, ids, scores, w13, w2, grad_out)

    if rank == 0:
        line = base_line(args, world)
        ms_step = total_ms / args.steps
        line.update({
            "value": world * T / (ms_step * 1e-3),
            "ms_per_step": ms_step,
            "e2e": {"value": world * T / (e2e_ms / args.steps * 1e-3), "unit": "tokens/s",
                    "h2d_bytes_per_step": x_pin.numel() * 2 + ids_pin.numel() * 8 + scores_pin.numel() * 4,
                    "d2h_bytes_per_step": out_host.numel() * 2, "ms_per_step": e2e_ms / args.steps,
                    "copies_only_ms_per_step": copies_ms / args.steps,
                    "copies_only_GBps_per_rank_each_way": (x_pin.numel() * 2 + ids_pin.numel() * 8
                                                           + scores_pin.numel() * 4) / (copies_ms / args.steps) / 1e6,
                    "host_numa_node_rank0": numa_node},
            "gpu_launches": launches,
            "step_mode": "cuda-graph replay" if graph is not None else "eager",
            "clocks": clocks,
            "roofline": roofline,
            "routed_rows_rank0": rows,
            "gemm_us_per_launch": breakdown,
            "parity_checked": bool(parity_ok),
            "parity": parity,
        })
        if nvlink is not None:
            line["nvlink"] = nvlink
        if world == 1 and not args.no_cpu_baseline:
            cb = cpu_baseline(CPU_STEPS, CPU_WARMUP)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
    ctx.close()
    del ctx, w13, w2
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and not args.no_extras:
        # the other configurations of the reference's benchmark table, one short run each, same process
        extras = {}
        for name, tokens, experts in (("mxfp8-train", 0, 0), ("nvfp4-decode", 0, 0), ("nvfp4-decode", 0, 32),
                                      ("nvfp4-prefill", 0, 32), ("mxfp8-infer", 0, 0)):
            sub = argparse.Namespace(**{**vars(args), "workload": name, "tokens": tokens, "experts": experts,
                                        "steps": 10 if name == "mxfp8-train" else 50, "warmup": 3})
            key = name + (f"-E{experts}" if experts else "")
            try:
                res = run_mxfp8_train(sub, emit=False) if name == "mxfp8-train" else run_inference(sub, emit=False)
                extras[key] = {k: res[k] for k in ("value", "unit", "ms_per_step", "p50_us", "p90_us", "steps", "step_mode",
                                                    "tflops_balanced", "achieved") if k in res}
                extras[key]["workload"] = res["config"]["workload"]
            except Exception as exc:  # noqa: BLE001 -- an extra must not cost the headline line
                extras[key] = {"error": repr(exc)[:300]}
        line["other_workloads"] = extras
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


INFERENCE_WORKLOADS = {
    # name: (format, T, D, F, E, K, clamped SwiGLU, routing, fused post-expert RMSNorm)
    "nvfp4-decode": ("NVFP4", 128, 7168, 2048, 256, 8, False, "sigmoid", False),
    "nvfp4-prefill": ("NVFP4", 8192, 7168, 2048, 256, 8, False, "sigmoid", False),
    # the reference rejects D = F = 2880 for MXFP8 (dimensions must be multiples of 128); 2816 is the nearest legal shape
    "mxfp8-infer": ("MXFP8_E4M3", 4096, 2816, 2816, 128, 4, True, "uniform", True),
}


def mxfp8_train_case(args, rank, world, dev):
    """Inputs of the MXFP8 training workload (shared by both arms): tokens, Zipf-skewed top-8 routing, bf16 weights
    and the scratch capacity factor the skew needs."""
    import numpy as np

    Tn, Dn, Fn, En, Kn = args.tokens or 8192, 4096, 1536, args.experts or 128, 8
    e_local = En // world
    g = torch.Generator().manual_seed(1000 + rank)
    x = torch.randn(Tn, Dn, generator=g).bfloat16().to(dev)
    bias = torch.from_numpy(np.random.default_rng(2027).zipf(1.1, En).clip(max=64).astype("float32")).log()
    logits = torch.randn(Tn, En, generator=g) + bias
    top = torch.topk(torch.softmax(logits, -1), Kn)
    scores = (top.values / top.values.sum(-1, keepdim=True)).float().to(dev)
    ids = top.indices.to(dev)
    per_expert = torch.bincount(top.indices.flatten(), minlength=En).float()
    grad_out = torch.randn(Tn, Dn, generator=g).bfloat16().to(dev)
    gw = torch.Generator(device=dev).manual_seed(2027 + rank)
    w13 = (torch.randn(e_local, 2, Fn, Dn, device=dev, generator=gw) * 0.02).bfloat16()
    w2 = (torch.randn(e_local, Dn, Fn, device=dev, generator=gw) * 0.02).bfloat16()
    return dict(T=Tn, D=Dn, F=Fn, E=En, K=Kn, e_local=e_local, x=x, ids=ids, scores=scores, per_expert=per_expert,
                grad_out=grad_out, w13=w13, w2=w2)


def inference_case(args, rank, world, dev):
    """Inputs of a forward-only inference workload (shared by both arms)."""
    fmt, Tn, Dn, Fn, En, Kn, clamped, routing, rmsnorm = INFERENCE_WORKLOADS[args.workload]
    if args.tokens:
        Tn = args.tokens
    if args.experts:
        En = args.experts  # e.g. E / 8: one rank's share of the experts of the EP=8 configuration on one GPU
    e_local = En // world
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    x = torch.randn(Tn, Dn, device=dev, generator=g).bfloat16()
    logits = torch.randn(Tn, En, device=dev, generator=g)
    if getattr(args, "routing", "config") == "hot":
        # stress: half of every token's assignments go to the experts rank 0 owns at EP=8 (the first E/8)
        hot, k_hot = max(Kn, En // 8), Kn // 2
        a, b = torch.topk(logits[:, :hot], k_hot), torch.topk(logits[:, hot:], Kn - k_hot)
        top_values, top_ids = torch.cat([a.values, b.values], 1), torch.cat([a.indices, b.indices + hot], 1)
    else:
        top_values, top_ids = torch.topk(logits, Kn)
    if routing == "sigmoid":   # sigmoid scores of the top-k logits, not renormalised
        scores, ids = torch.sigmoid(top_values).float(), top_ids
    else:                      # uniform random distinct experts, softmax-renormalised scores
        scores, ids = torch.softmax(top_values, -1).float(), top_ids
    gw = torch.Generator(device=dev).manual_seed(2027 + rank)

    def weights():
        """W13 then W2, generated one after the other so that only one bf16 weight is alive next to its quantised form."""
        yield (torch.randn(e_local, 2, Fn, Dn, device=dev, generator=gw) * 0.02).bfloat16()
        yield (torch.randn(e_local, Dn, Fn, device=dev, generator=gw) * 0.02).bfloat16()

    return dict(fmt=fmt, T=Tn, D=Dn, F=Fn, E=En, K=Kn, e_local=e_local, clamped=clamped, rmsnorm=rmsnorm, x=x, ids=ids,
                scores=scores, weights=weights,
                routing=f"{routing} top-{Kn}" + (", half of the assignments on the first E/8 experts"
                                                 if getattr(args, "routing", "config") == "hot" else ""))


def rmsnorm_options(module, case):
    """ExecutionOptions of an inference workload for either arm's package: the fused post-expert RMSNorm where the
    configuration names one."""
    if not case.get("rmsnorm"):
        return None
    post = module.RMSNormPostprocess(eps=1e-6, norm_output_dtype=torch.float32, output_dtype=torch.bfloat16)
    return module.ExecutionOptions(experts_output_postprocess=post)


def run_mxfp8_train(args, emit=True):
    """MXFP8 E4M3 training layer (forward + backward, prepared weights, in-place weight-gradient accumulation) at
    the reference's EP=8 MXFP8 configuration: T=8192 tokens/rank, D=4096, F=1536, E=128, K=8, router logits N(0,1)
    plus a per-expert bias drawn from Zipf(1.1).  Steps are eager calls timed with CUDA events; a second pass
    brackets every C-ABI call with events for the per-call breakdown."""
    import torch.distributed as dist

    import dist_moe_b200 as dm
    from dist_moe_b200 import _native

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    case = mxfp8_train_case(args, rank, world, dev)
    Tn, Dn, Fn, En, Kn, e_local = (case[k] for k in ("T", "D", "F", "E", "K", "e_local"))
    x, ids, scores, grad_out = case["x"], case["ids"], case["scores"], case["grad_out"]
    # rows the busiest rank receives (every expert's rows padded to 128), relative to T*K: the plan's capacity factor
    per_expert = case["per_expert"]
    if world > 1:
        t = per_expert.to(dev)
        dist.all_reduce(t)
        per_expert = t.cpu()
    padded = ((per_expert + 127) // 128 * 128).view(world, e_local).sum(1).max().item()
    factor = min(float(world), max(1.0, 1.02 * padded / float(Tn * Kn)))
    w13, w2 = case["w13"].requires_grad_(True), case["w2"].requires_grad_(True)
    w13.grad, w2.grad = torch.zeros_like(w13), torch.zeros_like(w2)
    cfg = dm.Config(max_num_local_input_tokens=Tn, hidden_dim=Dn, intermediate_dim=Fn, top_k=Kn, num_experts=En,
                    max_moe_layers_per_activation_slot=1, block_scaled=dm.BlockScaledConfig(),
                    activation_slot_capacity_factor=1.0 if world == 1 else min(float(world), 1.25),
                    device_scratch_capacity_factor=factor)
    ctx = dm.create_context(group=group, config=cfg, device=dev)
    opts = dm.ExecutionOptions(inplace_wgrad_accum=True)
    p13, p2 = dm.prepare_block_scaled_weight(w13, cfg), dm.prepare_block_scaled_weight(w2, cfg)

    def step():
        xs, ss = x.detach().requires_grad_(True), scores.detach().requires_grad_(True)
        dm.routed_experts(xs, ids, ss, p13, p2, ctx, options=opts).backward(grad_out)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for _ in range(max(3, args.warmup)):
        step()
    ctx.check_status()
    l0 = _native.LAUNCHES[0]
    step()
    launches_per_step = _native.LAUNCHES[0] - l0
    graph, _ = _capture(step, dev, args.no_graph)  # one step = one CUDA-graph replay, as in the BF16 workload
    run_step = graph.replay if graph is not None else step
    for _ in range(3):
        run_step()
    ctx.check_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sync_all()
    sampler.mark()
    s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s0.record()
    for _ in range(args.steps):
        run_step()
    s1.record()
    sync_all()
    sampler.mark()
    launches = launches_per_step * args.steps
    clocks = sampler.stop() if rank == 0 else None
    ctx.check_status()
    ms = torch.tensor([s0.elapsed_time(s1) / args.steps], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    ms = float(ms.item())
    # per-call breakdown of one more step (rank 0)
    events = []
    names = [n for n in _native.EXPORTS if n.startswith("dm_") and n not in ("dm_version", "dm_route_workspace_words")]
    saved = {n: getattr(_native.lib, n) for n in names}

    def bracket(fn, n):
        def call(*a):
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a0.record()
            r = fn(*a)
            a1.record()
            events.append((n, a0, a1))
            return r
        return call

    for n in names:
        setattr(_native.lib, n, bracket(saved[n], n))
    step()
    torch.cuda.synchronize()
    for n in names:
        setattr(_native.lib, n, saved[n])
    breakdown = [[n[3:], round(a0.elapsed_time(a1) * 1e3, 1)] for n, a0, a1 in events]
    rows = int(padded) if world == 1 else None
    last = getattr(ctx._state, "last_train_call", None)  # what the device planner decided for the layer
    decision = None if last is None else ("recompute" if bool(last.need.item()) else "saved")
    line = None
    if rank == 0:
        line = ({
            "metric": "MoE layer tokens/s (MXFP8 E4M3 training layer, fwd+bwd), whole job", "value": world * Tn / (ms * 1e-3),
            "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "e4m3 x e8m0 block scales",
            "data": "synthetic (seeded N(0,1) tokens, N(0,0.02) weights, softmax top-8 on N(0,1) logits + log Zipf(1.1) bias)",
            "config": {"workload": f"mxfp8-train: T={Tn} tokens/rank, D={Dn}, F={Fn}, E={En} (E_local={e_local}), K={Kn}, "
                                   f"plain SwiGLU, fwd+bwd, prepared weights, in-place wgrad accumulation",
                       "l2": "no flush: weights and routed activations exceed the 126 MB L2",
                       "capacity_factor": factor, "activation_slot_capacity_factor": cfg.activation_slot_capacity_factor,
                       "planner_decision": decision},
            "gpu_launches": launches, "step_mode": "cuda-graph replay" if graph is not None else "eager", "clocks": clocks,
            "padded_rows_busiest_rank": rows,
            "flops_per_step_rank0_balanced": 18.0 * Tn * Kn * Dn * Fn,
            "tflops_balanced": 18.0 * Tn * Kn * Dn * Fn / (ms * 1e-3) / 1e12, "us_per_call": breakdown})
        if emit:
            print(json.dumps(line), flush=True)
    ctx.close()
    del ctx, p13, p2, w13, w2
    torch.cuda.empty_cache()
    if world > 1 and emit:
        dist.barrier()
        dist.destroy_process_group()
    return line


def run_inference(args, emit=True):
    """Forward-only inference workloads with prepared block-scaled weights, timed as CUDA-graph replays.

    Every replay is bracketed by its own pair of CUDA events, so the line carries the median (p50) and the
    90th percentile of the layer time next to the whole-job tokens/s.  Experts are sharded over the ranks
    (E_local = E / N) and every rank contributes T tokens, as in the training workload.
    """
    import torch.distributed as dist

    import dist_moe_b200 as dm

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    case = inference_case(args, rank, world, dev)
    fmt, Tn, Dn, Fn, En, Kn, e_local, clamped = (case[k] for k in ("fmt", "T", "D", "F", "E", "K", "e_local", "clamped"))
    x, ids, scores = case["x"], case["ids"], case["scores"]
    bs = dm.BlockScaledConfig(format=getattr(dm.BlockScaledFormat, fmt))
    extra = {"activation": "swiglu_clamped", "swiglu_limit": 7.0} if clamped else {}
    rows_max = int(torch.bincount((ids // e_local).flatten(), minlength=world).max().item())
    if world > 1:
        t = torch.tensor([rows_max], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        rows_max = int(t.item())
    # the busiest rank's received rows relative to T*K (the plan adds the per-expert padding to 128 rows itself)
    factor = min(float(world), max(1.0, 1.05 * rows_max / float(Tn * Kn)))
    cfg = dm.Config(max_num_local_input_tokens=Tn, hidden_dim=Dn, intermediate_dim=Fn, top_k=Kn, num_experts=En,
                    max_moe_layers_per_activation_slot=1, inference=True, num_activation_slots=0, block_scaled=bs,
                    device_scratch_capacity_factor=factor, **extra)
    ctx = dm.create_context(group=group, config=cfg, device=dev)
    gen = case["weights"]()
    w13 = next(gen)
    p13 = dm.prepare_block_scaled_weight(w13, cfg, fuse_swiglu=True, inference=True)
    del w13
    w2 = next(gen)
    p2 = dm.prepare_block_scaled_weight(w2, cfg, inference=True)
    del w2
    torch.cuda.empty_cache()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    from dist_moe_b200 import _native

    opts = rmsnorm_options(dm, case)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side), torch.no_grad():
        for _ in range(3):
            l0 = _native.LAUNCHES[0]
            dm.routed_experts(x, ids, scores, p13, p2, ctx, options=opts)
            launches_per_step = _native.LAUNCHES[0] - l0
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.no_grad(), torch.cuda.graph(graph):
        out = dm.routed_experts(x, ids, scores, p13, p2, ctx, options=opts)
    for _ in range(max(3, args.warmup)):
        graph.replay()
    ctx.check_status()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    sync_all()
    sampler.mark()
    pairs = []
    for _ in range(args.steps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        graph.replay()
        e.record()
        pairs.append((s, e))
    sync_all()
    sampler.mark()
    clocks = sampler.stop() if rank == 0 else None
    ctx.check_status()
    times = sorted(s.elapsed_time(e) for s, e in pairs)
    stats = torch.tensor([times[len(times) // 2], times[min(len(times) - 1, (len(times) * 9) // 10)],
                          sum(times) / len(times)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    p50, p90, mean = (float(v) for v in stats.tolist())
    rows = int((ids // e_local == rank).sum().item()) if world > 1 else Tn * Kn
    bits = 4.5 if fmt == "NVFP4" else 8.25   # payload + block scales per weight element
    hit = int(torch.unique(ids[(ids // e_local) == rank]).numel()) if world > 1 else int(torch.unique(ids).numel())
    weight_bytes = hit * 3 * Dn * Fn * bits / 8
    flops = 6.0 * rows * Dn * Fn
    pk, src = peaks()
    line = None
    if rank == 0:
        line = {
            "metric": f"MoE layer tokens/s ({fmt} inference forward, prepared weights, CUDA-graph replay), whole job",
            "value": world * Tn / (mean * 1e-3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": mean, "p50_us": p50 * 1e3, "p90_us": p90 * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e2m1 x e4m3 block scales" if fmt == "NVFP4" else "e4m3 x e8m0 block scales",
            "data": "synthetic (seeded N(0,1) tokens, N(0,0.02) weights quantised once, top-k router on N(0,1) logits)",
            "config": {"workload": f"{args.workload}: T={Tn} tokens/rank, D={Dn}, F={Fn}, E={En} (E_local={e_local}), "
                                   f"K={Kn}, {'clamped' if clamped else 'plain'} SwiGLU"
                                   f"{', fused post-expert RMSNorm' if case['rmsnorm'] else ''}, routing {case['routing']}"
                                   ", forward only",
                       "l2": "no flush: the prepared weights of the experts hit exceed the 126 MB L2"
                       if weight_bytes > 126e6 else "weights of the experts hit fit in L2 between replays"},
            "gpu_launches": launches_per_step * args.steps, "step_mode": "cuda-graph replay", "clocks": clocks,
            "rows_rank0": rows, "experts_hit_rank0": hit,
            "achieved": {"weight_stream_GBps": weight_bytes / (p50 * 1e-3) / 1e9, "hbm_peak_GBps": pk["hbm_gbs"],
                         "tflops": flops / (p50 * 1e-3) / 1e12, "peak_source": src},
        }
        if emit:
            print(json.dumps(line), flush=True)
    _ = out
    ctx.close()
    del ctx, graph, p13, p2
    torch.cuda.empty_cache()
    if world > 1 and emit:
        dist.barrier()
        dist.destroy_process_group()
    return line


def run_micro(args):
    """A few launches of one grouped-GEMM arrangement on a reduced case (E_local=8, R=8192 rows):
    operands exceed L2 but stay small enough for a multi-pass profiler capture."""
    from dist_moe_b200 import _native as nat

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    e, rows = 8, 8192
    off = torch.arange(0, e + 1, dtype=torch.int32, device=dev) * (rows // e)
    status = torch.zeros(8, dtype=torch.int32, device=dev)
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(rows + 256, D, device=dev, generator=g).bfloat16()
    h1 = torch.randn(rows + 256, 2 * F, device=dev, generator=g).bfloat16()
    h2 = torch.zeros(rows + 256, F, device=dev, dtype=torch.bfloat16)
    w13 = (torch.randn(e, 2 * F, D, device=dev, generator=g) * 0.02).bfloat16()
    dw13 = torch.zeros(e, 2 * F, D, device=dev, dtype=torch.bfloat16)
    op = lambda t: nat.Operand(t.data_ptr(), t.numel() * t.element_size(), None)  # noqa: E731
    none, st = nat.Operand(None, 0, None), nat.stream_ptr()
    calls = {
        "fprop": lambda: nat.lib.dm_gemm_fprop(op(x), w13.data_ptr(), op(h1), op(h2), None, off.data_ptr(), e, rows,
                                               2 * F, D, 1, 0, 1.0, 0.0, None, 0, status.data_ptr(), st),
        "dgrad": lambda: nat.lib.dm_gemm_dgrad(op(h1), w13.data_ptr(), op(x), None, off.data_ptr(), e, rows, D, 2 * F,
                                               None, 0, status.data_ptr(), st),
        "wgrad": lambda: nat.lib.dm_gemm_wgrad(op(h1), op(x), dw13.data_ptr(), 0, 1, off.data_ptr(), e, rows, 2 * F, D,
                                               0, status.data_ptr(), st),
    }
    if args.micro == "quant-mxfp8":
        # row + column MXFP8 quantiser on a [16384, 4096] bf16 matrix (134 MB in, 134 MB + scales out)
        qr, qc_cols = 16384, 4096
        xq = torch.randn(qr, qc_cols, device=dev, generator=g).bfloat16()
        q_row = torch.empty(qr, qc_cols, dtype=torch.uint8, device=dev)
        q_col = torch.empty(qr, qc_cols, dtype=torch.uint8, device=dev)
        s_row = torch.empty(qr * (qc_cols // 32), dtype=torch.uint8, device=dev)
        s_col = torch.empty(qc_cols * (qr // 32), dtype=torch.uint8, device=dev)
        fnq = lambda: nat.lib.dm_quant_mxfp8_rowcol(xq.data_ptr(), None, qr, qc_cols, q_row.data_ptr(), s_row.data_ptr(),  # noqa: E731
                                                    q_col.data_ptr(), s_col.data_ptr(), st)
        for _ in range(2):
            nat.check(fnq(), args.micro)
        torch.cuda.synchronize()
        s0, t0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            nat.check(fnq(), args.micro)
        t0.record()
        torch.cuda.synchronize()
        ms = s0.elapsed_time(t0) / args.steps
        nbytes = qr * qc_cols * (2 + 2 * (1 + 1 / 32))
        print(json.dumps({"micro": args.micro, "rows": qr, "cols": qc_cols, "ms": ms, "algorithmic_GBps": nbytes / ms / 1e6}),
              flush=True)
        return
    if args.micro in ("bs-nvfp4", "bs-mxfp8"):
        # block-scaled forward GEMM (W13 with the SwiGLU epilogue) on synthetic quantised bytes: timing does not
        # depend on the values, scale bytes are 1.0 in their format
        fp4 = args.micro == "bs-nvfp4"
        n, k = (4096, 7168) if fp4 else (3072, 4096)
        rows = 8192
        off = torch.arange(0, e + 1, dtype=torch.int32, device=dev) * (rows // e)
        kb, per_scale = (k // 2, 16) if fp4 else (k, 32)
        atoms = (k // per_scale + 3) // 4
        qa = torch.randint(0, 120, (rows + 256, kb), dtype=torch.uint8, device=dev, generator=g)
        qw = torch.randint(0, 120, (e * n, kb), dtype=torch.uint8, device=dev, generator=g)
        sa = torch.full((rows * atoms * 4,), 0x38 if fp4 else 127, dtype=torch.uint8, device=dev)
        sw = torch.full((e * n * atoms * 4,), 0x38 if fp4 else 127, dtype=torch.uint8, device=dev)
        inv = torch.ones(rows, dtype=torch.float32, device=dev)
        einv = torch.ones(e, dtype=torch.float32, device=dev)
        hq = torch.zeros(rows + 8, n // 2, dtype=torch.bfloat16, device=dev)
        calls[args.micro] = lambda: nat.lib.dm_gemm_blockscaled(
            1 if fp4 else 0, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), none, op(hq), None, op(inv) if fp4 else none,
            einv.data_ptr() if fp4 else None, off.data_ptr(), e, rows, n, k, 1, 0, 1.0, 0.0, None, 0, status.data_ptr(), st)
        flops_bs = 2.0 * rows * n * k
    if args.micro == "bs-decode":
        # swapped-operand NVFP4 GEMM at a decode shape: 12 experts x 32 real rows inside 128-row groups, W13 of
        # D=7168, F=2048 (176 MB of weights + 22 MB of scales per launch: more than L2, streamed once)
        e, n, k, real = 12, 4096, 7168, 32
        rows = e * 128
        off = torch.arange(0, e + 1, dtype=torch.int32, device=dev) * 128
        cnt = torch.full((e,), real, dtype=torch.int32, device=dev)
        atoms = (k // 16 + 3) // 4
        qa = torch.randint(0, 120, (rows + 256, k // 2), dtype=torch.uint8, device=dev, generator=g)
        qw = torch.randint(0, 120, (e * n, k // 2), dtype=torch.uint8, device=dev, generator=g)
        sa = torch.full(((rows + 256) * atoms * 4,), 0x38, dtype=torch.uint8, device=dev)
        sw = torch.full((e * n * atoms * 4,), 0x38, dtype=torch.uint8, device=dev)
        inv = torch.ones(rows + 256, dtype=torch.float32, device=dev)
        einv = torch.ones(e, dtype=torch.float32, device=dev)
        hq = torch.zeros(rows + 8, n // 2, dtype=torch.bfloat16, device=dev)
        calls[args.micro] = lambda: nat.lib.dm_gemm_blockscaled_swapped(
            1, op(qa), op(sa), qw.data_ptr(), sw.data_ptr(), none, op(hq), None, op(inv), einv.data_ptr(), off.data_ptr(),
            cnt.data_ptr(), e, rows, n, k, 1, 0, 1.0, 0.0, None, 0, status.data_ptr(), st)
        flops_bs = 2.0 * e * real * n * k
        stream_bytes = qw.numel() + sw.numel()
    fn = calls[args.micro]
    flops = flops_bs if args.micro.startswith("bs-") else 2.0 * rows * D * 2 * F
    for _ in range(2):
        nat.check(fn(), args.micro)
    torch.cuda.synchronize()
    s, t = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(args.steps):
        nat.check(fn(), args.micro)
    t.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(t) / args.steps
    line = {"micro": args.micro, "rows": rows, "e_local": e, "D": D, "F": F, "ms": ms, "tflops": flops / ms / 1e9,
            "status": status.tolist()[:2]}
    if args.micro == "bs-decode":
        line["weight_stream_GBps"] = stream_bytes / ms / 1e6
    print(json.dumps(line), flush=True)
    _ = none


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="N=1: skip the short runs of the MXFP8 / NVFP4 workloads added to the line as other_workloads")
    ap.add_argument("--reference-on-cpu", action="store_true",
                    help="--impl reference: time the CPU restatement even when the reference's GPU build is installed")
    ap.add_argument("--separate-gather", action="store_true",
                    help="gather routed rows with a separate kernel instead of inside the GEMM launches")
    ap.add_argument("--no-graph", action="store_true",
                    help="time eager routed_experts calls instead of CUDA-graph replays of the same step")
    ap.add_argument("--micro", default=None, choices=["fprop", "dgrad", "wgrad", "bs-nvfp4", "bs-mxfp8", "bs-decode", "quant-mxfp8"],
                    help="time one grouped-GEMM arrangement alone on a reduced case (for profiler captures)")
    ap.add_argument("--workload", default="bf16-train", choices=["bf16-train", "mxfp8-train"] + sorted(INFERENCE_WORKLOADS),
                    help="bf16-train is the headline training layer; the others are forward-only inference layers")
    ap.add_argument("--tokens", type=int, default=0, help="tokens per rank of an inference workload (sweeps)")
    ap.add_argument("--routing", default="config", choices=["config", "hot"],
                    help="inference workloads: the configuration's router, or the stress where half of the assignments "
                         "go to the experts rank 0 owns at EP=8")
    ap.add_argument("--experts", type=int, default=0, help="total experts of an inference workload (default: the config's)")
    args = ap.parse_args()
    if args.micro:
        run_micro(args)
    elif args.impl == "reference" and args.workload != "bf16-train":
        run_reference_blockscaled(args)
    elif args.impl == "reference":
        run_reference(args)
    elif args.workload == "mxfp8-train":
        run_mxfp8_train(args)
    elif args.workload != "bf16-train":
        run_inference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
