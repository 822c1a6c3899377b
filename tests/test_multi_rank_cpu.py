"""world_size-2 runs on CPU (gloo): the expert-parallel composition of the oracle (id all-gather, routing
tables, dispatch and combine all-to-alls) equals the single-process dense oracle, and ``bench.py``'s
reference arm prints exactly one line from rank 0 under a multi-process launch."""

import json
import os
import subprocess
import sys
from pathlib import Path

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import distributed as oracle_dist
        from oracle import moe as oracle_moe

        T, D, F, K, E = 16, 64, 32, 2, 8  # quick-start routing: ids (global_token*K + k) % E, scores 1/K
        g = torch.Generator().manual_seed(17)
        xs = [torch.randn(T, D, generator=g).bfloat16() for _ in range(world)]
        w13 = torch.randn(E, 2 * F, D, generator=g).bfloat16() * 0.2
        w2 = torch.randn(E, D, F, generator=g).bfloat16() * 0.2
        el = E // world
        for case in ("quickstart", "random"):
            if case == "quickstart":
                tok = rank * T + torch.arange(T)
                ids = (tok[:, None] * K + torch.arange(K)[None, :]) % E
                scores = torch.full((T, K), 1.0 / K)
            else:
                gg = torch.Generator().manual_seed(100 + rank)
                ids = torch.stack([torch.randperm(E, generator=gg)[:K] for _ in range(T)])
                ids[torch.rand(T, K, generator=gg) < 0.2] = -1
                scores = torch.rand(T, K, generator=gg) * (ids >= 0)
            out = oracle_dist.moe_forward_ep(xs[rank], ids, scores, w13[rank * el:(rank + 1) * el],
                                             w2[rank * el:(rank + 1) * el], E)
            ref = oracle_moe.moe_forward(xs[rank], ids, scores, w13, w2)
            assert torch.equal(out, ref), (case, (out.float() - ref.float()).abs().max())
        results[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_expert_parallel_oracle_matches_dense_oracle_on_two_gloo_ranks():
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(_worker, args=(2, 29731, results), nprocs=2, join=True)
    assert dict(results) == {0: "ok", 1: "ok"}


def test_reference_arm_prints_one_line_from_rank_zero():
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29741", str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2",
           "--steps", "1", "--warmup", "1"]
    env = dict(os.environ, DIST_MOE_BENCH_CPU_TOKENS="16")
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert res.returncode == 0, res.stderr[-2000:]
    lines = [json.loads(l) for l in res.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = lines[0]
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["cpu_baseline"]["kind"] == "port"
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0
