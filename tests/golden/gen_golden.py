"""Generate golden vectors by executing the reference's own code on the CPU.

Run where a checkout of the reference is available and pass its location:

    python tests/golden/gen_golden.py --reference <path to the dist_moe checkout>

What runs, unmodified, from the reference:
* ``dist_moe.plan_memory`` (pure Python) -> ``plan_memory.json``;
* the Triton routing kernels (gather / split / prefix / combine,
  ``dist_moe/kernels/triton/dist_dispatch_routing_kernel.py``) and the BF16 and block-scaled
  planner kernels (``dist_moe/_activation_buffer_planner_kernel.py``) under Triton's CPU
  interpreter (``TRITON_INTERPRET=1``) -> ``routing_*.npz``, ``planner_bf16.json``,
  ``planner_blockscaled.json``.

Quantised bytes and floating-point outputs come from the reference's GPU kernels run on a B200 instead:
see ``gen_golden_gpu.py`` in this directory.

Three shims make the interpreter accept those kernels; none changes arithmetic:
``range`` inside the kernel module yields interpreter scalars (the kernels call
``.to(...)`` on loop indices), ``device_trap_if`` (inline PTX ``trap``) becomes a
Python assertion, and ``get_flat_tid`` (inline PTX read of %tid) returns 0.  Peer buffers are ordinary host arrays whose addresses are
passed where the kernels expect peer pointers.
"""

from __future__ import annotations

import argparse
import builtins
import json
import os
import sys
from pathlib import Path

os.environ["TRITON_INTERPRET"] = "1"
HERE = Path(__file__).resolve().parent


def _shim(module, np, tl, TensorHandle):
    def _range(*args):
        vals = [int(a.handle.data.item()) if hasattr(a, "handle") else int(a) for a in args]
        for i in builtins.range(*vals):
            yield tl.core.tensor(TensorHandle(np.array([i], dtype=np.int32), tl.int32), tl.int32)

    def _trap(cond):
        data = cond.handle.data if hasattr(cond, "handle") else np.asarray(cond)
        assert not bool(np.any(data)), "reference kernel would trap"

    def _flat_tid():
        return tl.core.tensor(TensorHandle(np.array([0], dtype=np.int32), tl.int32), tl.int32)

    module.range = _range
    if hasattr(module, "device_trap_if"):
        module.device_trap_if = _trap
    if hasattr(module, "get_flat_tid"):
        module.get_flat_tid = _flat_tid  # the reference reads %tid with inline PTX; one program = thread 0


def gen_plan_memory(ref):
    import dist_moe
    import torch

    F = dist_moe.BlockScaledFormat
    cases = {
        "tiny_bf16": (dict(max_num_local_input_tokens=16, hidden_dim=256, intermediate_dim=256, top_k=2, num_experts=8,
                           max_moe_layers_per_activation_slot=1), 2),
        "c2_bf16_ep8": (dict(max_num_local_input_tokens=4096, hidden_dim=2048, intermediate_dim=1408, top_k=6,
                             num_experts=64, max_moe_layers_per_activation_slot=1,
                             activation_slot_capacity_factor=1.0), 8),
        "c2_bf16_ep1": (dict(max_num_local_input_tokens=4096, hidden_dim=2048, intermediate_dim=1408, top_k=6,
                             num_experts=64, max_moe_layers_per_activation_slot=1,
                             activation_slot_capacity_factor=1.0), 1),
        "bf16_two_slots": (dict(max_num_local_input_tokens=512, hidden_dim=1024, intermediate_dim=2048, top_k=4,
                                num_experts=32, max_moe_layers_per_activation_slot=3, num_activation_slots=2,
                                device_scratch_capacity_factor=1.5, activation_slot_capacity_factor=0.5), 4),
        "bf16_exact_bytes": (dict(max_num_local_input_tokens=128, hidden_dim=512, intermediate_dim=384, top_k=2,
                                  num_experts=8, max_moe_layers_per_activation_slot=2,
                                  activation_slot_bytes=3_000_000), 2),
        "bf16_inference": (dict(max_num_local_input_tokens=1024, hidden_dim=2880, intermediate_dim=2880, top_k=4,
                                num_experts=128, max_moe_layers_per_activation_slot=1, inference=True,
                                num_activation_slots=0), 8),
        "c3_mxfp8_ep8": (dict(max_num_local_input_tokens=8192, hidden_dim=4096, intermediate_dim=1536, top_k=8,
                              num_experts=128, max_moe_layers_per_activation_slot=1,
                              device_scratch_capacity_factor=1.25,
                              block_scaled=("MXFP8_E4M3", "staged")), 8),
        "mxfp8_mega": (dict(max_num_local_input_tokens=256, hidden_dim=512, intermediate_dim=256, top_k=2,
                            num_experts=16, max_moe_layers_per_activation_slot=2,
                            activation_slot_capacity_factor=1.0, block_scaled=("MXFP8_E4M3", "mega")), 4),
        "c4_nvfp4_decode": (dict(max_num_local_input_tokens=128, hidden_dim=7168, intermediate_dim=2048, top_k=8,
                                 num_experts=256, max_moe_layers_per_activation_slot=1, inference=True,
                                 num_activation_slots=0, block_scaled=("NVFP4", "staged")), 8),
        "c4_nvfp4_prefill": (dict(max_num_local_input_tokens=8192, hidden_dim=7168, intermediate_dim=2048, top_k=8,
                                  num_experts=256, max_moe_layers_per_activation_slot=1, inference=True,
                                  num_activation_slots=0, block_scaled=("NVFP4", "staged")), 8),
        "mxfp8_inference": (dict(max_num_local_input_tokens=1024, hidden_dim=3072, intermediate_dim=3072, top_k=8,
                                 num_experts=128, max_moe_layers_per_activation_slot=1, inference=True,
                                 num_activation_slots=0, block_scaled=("MXFP8_E4M3", "staged")), 8),
    }
    out = {}
    for name, (kw, ep) in cases.items():
        kw = dict(kw)
        spec = dict(kw)
        bs = kw.pop("block_scaled", None)
        if bs is not None:
            kw["block_scaled"] = dist_moe.BlockScaledConfig(format=getattr(F, bs[0]), pipeline=bs[1])
        plan = dist_moe.plan_memory(dist_moe.Config(**kw), ep)
        fields = {k: v for k, v in plan.__dict__.items()}
        out[name] = {"config": spec, "ep_size": ep, "plan": fields, "explain": plan.explain()}
    (HERE / "plan_memory.json").write_text(json.dumps(out, indent=1, sort_keys=True))
    print("plan_memory.json:", len(out), "cases")


def _ref_route(np, torch, triton, tl, K, ids_all, rank, E, m_mult, bwd, gather_stride, bwd_stride, scatter_stride):
    """Run the reference's four routing kernels for one rank; mirrors the launcher
    dist_moe/_routing_metadata.py:886-1102 (grid and buffer shapes only)."""
    EP, T, topk = ids_all.shape
    EL = E // EP
    header = 128
    bufs = []
    for s in range(EP):
        b = np.zeros(header + T * topk * 2, dtype=np.uint8)
        b[:4] = np.frombuffer(np.int32(T).tobytes(), dtype=np.uint8)
        b[header:] = np.frombuffer(ids_all[s].astype(np.int16).tobytes(), dtype=np.uint8)
        bufs.append(torch.from_numpy(b))
    routing_ptrs = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64)
    disp_base = torch.tensor([(s + 1) << 40 for s in range(EP)], dtype=torch.int64)
    comb_base = torch.tensor([((s + 1) << 40) | (1 << 39) for s in range(EP)], dtype=torch.int64)

    block_size_k = triton.next_power_of_2(topk)
    block_size_t = max(1, 256 // block_size_k)
    max_workers = (512 if bwd else 256) // EP
    num_workers = max(1, min(max_workers, (T + block_size_t - 1) // block_size_t))
    num_workers = min(max_workers, triton.next_power_of_2(num_workers))
    tpw = (T + num_workers - 1) // num_workers
    cnts = torch.full((EP, EL, num_workers), 12345, dtype=torch.int32)
    per_rank = torch.full((E,), 777, dtype=torch.int32)
    gathered = torch.full((EP, T, topk), -7, dtype=torch.int16)
    gw = max(1, (T + 1023) // 1024)
    K._triton_dist_gather_metadata[(EP, gw, 1)](
        routing_buffer_ptrs=routing_ptrs, gathered_expert_ids_ptr=gathered, per_rank_token_cnts_ptr=cnts,
        num_tokens_per_rank_ptr=per_rank, world_size=EP, num_tokens=T, num_experts=E, topk=topk, block_size_t=1024,
        num_gather_workers=gw, split_num_workers=num_workers, index_ty=tl.int16, routing_header_size_bytes=header,
        BLOCK_K=block_size_k, BLOCK_WORLD_SIZE=triton.next_power_of_2(EP))
    shape = (EP, EL, num_workers, tpw)
    pr_bwd = torch.zeros(shape, dtype=torch.int64) if bwd else None
    pr_fwd = torch.zeros(shape, dtype=torch.int64)
    pr_sct = torch.zeros(shape, dtype=torch.int64)
    K._triton_dispatch_routing_split[(EP, num_workers, 1)](
        gathered_expert_ids_ptr=gathered, gather_buffer_ptrs=disp_base, scatter_buffer_ptrs=comb_base,
        per_rank_token_cnts_ptr=cnts, per_rank_bwd_gather_ptrs_ptr=pr_bwd, gather_stride_bytes=gather_stride,
        bwd_gather_stride_bytes=bwd_stride, per_rank_fwd_gather_ptrs_ptr=pr_fwd, per_rank_scatter_ptrs_ptr=pr_sct,
        scatter_stride_bytes=scatter_stride, num_tokens_per_rank_ptr=per_rank, expert_id_offset=rank * EL,
        dest_rank_base=0, world_size=EP, num_tokens=T, num_experts=E, topk=topk, block_size_t=block_size_t,
        BLOCK_EL=triton.next_power_of_2(EL), BLOCK_K=block_size_k)
    from dist_moe._routing_metadata import _routing_ptrs_capacity

    ptrs_size = _routing_ptrs_capacity(world_size=EP, num_tokens=T, topk=topk, num_local_experts=EL,
                                       m_multiple_of=m_mult, max_num_recv_tokens=None,
                                       pointer_capacity_multiple_of=1)
    sentinel = -(1 << 62)
    out_bwd = torch.full((ptrs_size,), sentinel, dtype=torch.int64) if bwd else None
    out_fwd = torch.full((ptrs_size,), sentinel, dtype=torch.int64)
    out_sct = torch.full((ptrs_size,), sentinel, dtype=torch.int64)
    counts = torch.zeros((EL,), dtype=torch.int32)
    max_compact = 16 * 148
    limit = max(1, max_compact // E)
    cpp = min(num_workers, 1 << (limit.bit_length() - 1))
    wpc = num_workers // cpp
    offs = torch.zeros((EP, EL, cpp), dtype=torch.int64)
    K._triton_dispatch_routing_prefix[(1, 1, 1)](
        per_rank_token_cnts_ptr=cnts, token_cnts_ptr=counts, num_tokens_per_rank_ptr=per_rank,
        compact_offsets_ptr=offs, world_size=EP, num_experts=E, num_workers=num_workers, compact_ctas_per_pair=cpp,
        workers_per_compact_cta=wpc, BLOCK_EL=triton.next_power_of_2(EL), m_multiple_of=m_mult,
        max_num_recv_tokens=0, has_max_num_recv_tokens=False)
    K._triton_dispatch_routing_combine[(EP * EL * cpp, 1, 1)](
        per_rank_token_cnts_ptr=cnts, per_rank_bwd_gather_ptrs_ptr=pr_bwd, per_rank_fwd_gather_ptrs_ptr=pr_fwd,
        per_rank_scatter_ptrs_ptr=pr_sct, token_cnts_ptr=counts, compact_offsets_ptr=offs,
        bwd_gather_ptrs_ptr=out_bwd, fwd_gather_ptrs_ptr=out_fwd, scatter_ptrs_ptr=out_sct, world_size=EP,
        num_experts=E, block_size_t=block_size_t, num_workers=num_workers, num_tokens_per_worker=tpw,
        compact_ctas_per_pair=cpp, workers_per_compact_cta=wpc, m_multiple_of=m_mult)
    res = dict(counts=counts.numpy(), per_rank=per_rank[:EP].numpy().copy(), fwd=out_fwd.numpy(),
               sct=out_sct.numpy(), disp_base=disp_base.numpy(), comb_base=comb_base.numpy(),
               sentinel=np.int64(sentinel))
    if bwd:
        res["bwd"] = out_bwd.numpy()
    return res


def gen_routing(ref):
    import numpy as np
    import torch
    import triton
    import triton.language as tl
    from triton.runtime.interpreter import TensorHandle

    from dist_moe.kernels.triton import dist_dispatch_routing_kernel as K

    _shim(K, np, tl, TensorHandle)
    rng = np.random.default_rng(2027)

    def random_ids(EP, T, topk, E, drop=0.0, skew=None):
        ids = np.empty((EP, T, topk), dtype=np.int64)
        p = None
        if skew is not None:
            p = 1.0 / np.arange(1, E + 1) ** skew
            p /= p.sum()
        for s in range(EP):
            for t in range(T):
                ids[s, t] = rng.choice(E, size=topk, replace=False, p=p)
        if drop:
            ids[rng.random(ids.shape) < drop] = -1
        return ids

    cases = {}
    EP, T, topk, E = 2, 16, 2, 8  # quickstart ids: (global_token*K + k) % E
    ids = np.stack([(((r * T + np.arange(T))[:, None] * topk + np.arange(topk)[None, :]) % E) for r in range(EP)])
    cases["quickstart"] = (ids, E, 0, True, 512, 512, 512)
    cases["random_ep4"] = (random_ids(4, 300, 3, 16, drop=0.1), 16, 0, True, 2048, 2048, 2048)
    cases["skew_pad128"] = (random_ids(2, 200, 4, 8, skew=1.1), 8, 128, True, 1024, 1024, 1024)
    cases["packed_stride_pad128_nobwd"] = (random_ids(4, 64, 2, 8, drop=0.05), 8, 128, False, 4048, 0, 14336)
    cases["single_rank"] = (random_ids(1, 130, 2, 4), 4, 0, True, 256, 256, 256)
    cases["multi_chunk"] = (random_ids(2, 600, 2, 4), 4, 0, True, 128, 128, 128)
    for name, (ids, E, m_mult, bwd, gs, bs, ss) in cases.items():
        EP = ids.shape[0]
        blob = {"ids": ids.astype(np.int16), "num_experts": np.int64(E), "m_multiple_of": np.int64(m_mult),
                "gather_stride": np.int64(gs), "bwd_stride": np.int64(bs), "scatter_stride": np.int64(ss)}
        for rank in range(EP):
            res = _ref_route(np, torch, triton, tl, K, ids, rank, E, m_mult, bwd, gs, bs if bwd else gs, ss)
            for k, v in res.items():
                blob[f"r{rank}_{k}"] = v
        np.savez_compressed(HERE / f"routing_{name}.npz", **blob)
        print("routing", name, "ok")


PLANNER_SCENARIOS = {
    # name: (EP, T, K, D, F, slots, layers, slot_factor, ops); ops: ("f", slot, R, per_rank, scratch_only) / ("b", index of f)
    "two_layers_saved": (2, 64, 2, 256, 256, 1, 2, 1.0,
                         [("f", 0, 120, [120, 136], False), ("f", 0, 100, [100, 156], False), ("b", 1), ("b", 0)]),
    "recompute_when_full": (2, 64, 2, 256, 512, 1, 3, 0.4,
                            [("f", 0, 128, [128, 128], False), ("f", 0, 200, [200, 56], False),
                             ("f", 0, 90, [90, 166], False), ("b", 2), ("b", 1), ("b", 0)]),
    "two_slots_and_no_grad": (4, 32, 4, 512, 128, 2, 1, None,
                              [("f", 0, 100, [100, 140, 160, 112], False), ("f", 1, 33, [33, 200, 150, 129], False),
                               ("f", 1, 64, [64, 64, 64, 64], True), ("b", 1), ("b", 0)]),
    "hidden_le_inter": (1, 16, 2, 128, 1024, 1, 1, 1.0, [("f", 0, 32, [32], False), ("b", 0)]),
}


def gen_planner(ref):
    import numpy as np
    import torch
    import triton.language as tl
    from triton.runtime.interpreter import TensorHandle

    import dist_moe
    from dist_moe import _activation_buffer_planner_kernel as P

    _shim(P, np, tl, TensorHandle)
    out = {}
    for name, (EP, T, K, D, F, slots, layers, factor, ops) in PLANNER_SCENARIOS.items():
        cfg = dist_moe.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K,
                              num_experts=4 * EP, max_moe_layers_per_activation_slot=layers,
                              num_activation_slots=slots, activation_slot_capacity_factor=factor,
                              device_scratch_capacity_factor=float(EP))
        plan = dist_moe.plan_memory(cfg, EP)
        slot_bytes, arena = plan.activation_slot_bytes, plan.total_device_buffer_bytes
        i64 = lambda v: torch.tensor(v, dtype=torch.int64)  # noqa: E731
        buffer_offsets = i64([i * slot_bytes for i in range(slots)] + [arena])
        saved = torch.zeros(slots * EP, dtype=torch.int64)
        peak = i64([slot_bytes] * slots + [arena - slots * slot_bytes])
        layer = torch.zeros(slots, dtype=torch.int64)
        steps, fwd_records = [], []
        for op in ops:
            if op[0] == "f":
                _, slot, R, per_rank, scratch_only = op
                need = torch.zeros(1, dtype=torch.bool)
                fwd_state = torch.zeros(6, dtype=torch.int64)
                sel = i64([slot])
                P._triton_get_forward_plan[(1,)](
                    torch.tensor([R], dtype=torch.int32), torch.tensor(per_rank, dtype=torch.int32), None, saved,
                    buffer_offsets, peak, need, fwd_state, EP=EP, num_tokens=T, topk=K, element_size=2, hidden_dim=D,
                    intermediate_dim=F, microbatch_id_ptr=sel, activation_slot_bytes=slot_bytes, buffer_size=arena,
                    num_activation_slots=slots, moe_layer_id_ptr=layer, num_moe_layers=layers,
                    scratch_only=scratch_only)
                rec = dict(op="f", slot=slot, R=R, per_rank=per_rank, scratch_only=scratch_only, need=bool(need[0]),
                           fwd_state=fwd_state.tolist())
                fwd_records.append(rec)
            else:
                f = [r for r in fwd_records][op[1]]
                bwd = torch.zeros(6, dtype=torch.int64)
                fs = i64(f["fwd_state"])
                P._triton_get_backward_plan[(1,)](
                    torch.tensor([f["R"]], dtype=torch.int32), buffer_offsets, peak, torch.tensor([f["need"]]),
                    fs[0:1], fs[1:2], fs[2:3], saved, torch.tensor(f["per_rank"], dtype=torch.int32), bwd, EP=EP,
                    num_tokens=T, topk=K, element_size=2, hidden_dim=D, intermediate_dim=F,
                    microbatch_id_ptr=fs[5:6], activation_slot_bytes=slot_bytes, buffer_size=arena,
                    num_activation_slots=slots, moe_layer_id_ptr=layer)
                rec = dict(op="b", of=op[1], bwd_offsets=bwd.tolist())
            rec["state"] = dict(buffer_offsets=buffer_offsets.tolist(), saved=saved.tolist(), peak=peak.tolist(),
                                layer=layer.tolist())
            steps.append(rec)
        out[name] = dict(EP=EP, T=T, K=K, D=D, F=F, slots=slots, layers=layers, slot_bytes=slot_bytes,
                         arena_bytes=arena, steps=steps)
    (HERE / "planner_bf16.json").write_text(json.dumps(out, indent=1, sort_keys=True))
    print("planner_bf16.json:", len(out), "scenarios")


# name: (format, EP, T, K, D, F, slots, layers, slot factor, flags, ops); ops as in PLANNER_SCENARIOS.  The slot
# factor decides which scenarios save (1.0) and which recompute (small); flags are the kernel's constexpr switches.
BLOCKSCALED_PLANNER_SCENARIOS = {
    "mxfp8_saved": ("MXFP8_E4M3", 2, 64, 2, 256, 128, 1, 1, 1.0, {},
                    [("f", 0, 256, [128, 128], False), ("b", 0)]),
    "mxfp8_recompute": ("MXFP8_E4M3", 2, 64, 2, 256, 128, 1, 1, 0.25, {},
                        [("f", 0, 256, [150, 106], False), ("b", 0)]),
    "mxfp8_mixed_stack": ("MXFP8_E4M3", 4, 32, 4, 512, 256, 1, 3, 0.3, {},
                          [("f", 0, 512, [100, 140, 160, 112], False), ("f", 0, 384, [33, 120, 150, 81], False),
                           ("f", 0, 640, [160, 160, 160, 160], False), ("b", 2), ("b", 1), ("b", 0)]),
    "mxfp8_two_slots_scratch_only": ("MXFP8_E4M3", 2, 48, 2, 384, 256, 2, 2, 1.0, {},
                                     [("f", 0, 256, [96, 96], False), ("f", 1, 128, [70, 26], False),
                                      ("f", 1, 256, [128, 100], True), ("f", 1, 256, [60, 130], False), ("b", 3),
                                      ("b", 1), ("b", 0)]),
    "mxfp8_mega": ("MXFP8_E4M3", 2, 64, 2, 256, 384, 1, 2, 0.22, {"mega": True},
                   [("f", 0, 256, [128, 100], False), ("f", 0, 384, [200, 150], False), ("b", 1), ("b", 0)]),
    "mxfp8_native_backward": ("MXFP8_E4M3", 2, 64, 2, 256, 128, 1, 2, 0.3, {"native_backward": True},
                              [("f", 0, 256, [128, 128], False), ("f", 0, 256, [90, 140], False), ("b", 1), ("b", 0)]),
    "nvfp4_saved_and_recompute": ("NVFP4", 2, 64, 4, 512, 256, 1, 2, 0.35, {},
                                  [("f", 0, 384, [180, 190], False), ("f", 0, 512, [256, 250], False), ("b", 1),
                                   ("b", 0)]),
    "nvfp4_inference": ("NVFP4", 2, 64, 4, 512, 256, 0, 1, None, {"inference_mode": True},
                        [("f", 0, 384, [180, 190], True)]),
    "nvfp4_inference_interleaved_mega": ("NVFP4", 2, 64, 4, 512, 256, 0, 1, None,
                                         {"inference_mode": True, "interleaved_fc13": True, "mega": True},
                                         [("f", 0, 256, [128, 120], True)]),
    "mxfp8_inference_interleaved_mega": ("MXFP8_E4M3", 2, 64, 4, 512, 256, 0, 1, None,
                                         {"inference_mode": True, "interleaved_fc13": True, "mega": True},
                                         [("f", 0, 256, [128, 120], True)]),
}


def gen_planner_blockscaled(ref):
    import numpy as np
    import torch
    import triton.language as tl
    from triton.runtime.interpreter import TensorHandle

    import dist_moe
    from dist_moe import _activation_buffer_planner_kernel as P

    _shim(P, np, tl, TensorHandle)
    storages = {"MXFP8_E4M3": [1, 1, 1, 4, 0, 32], "NVFP4": [1, 2, 1, 4, 4, 16]}
    out = {}
    for name, (fmt, EP, T, K, D, F, slots, layers, factor, flags, ops) in BLOCKSCALED_PLANNER_SCENARIOS.items():
        inference = bool(flags.get("inference_mode"))
        kw = dict(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=4 * EP,
                  max_moe_layers_per_activation_slot=layers, num_activation_slots=slots,
                  device_scratch_capacity_factor=float(EP), inference=inference,
                  # the reference's Config admits NVFP4 for inference only: a training scenario takes its slot and
                  # arena sizes from the MXFP8 plan and still runs the kernels with the NVFP4 storage geometry
                  block_scaled=dist_moe.BlockScaledConfig(format=getattr(dist_moe.BlockScaledFormat,
                                                                         fmt if inference else "MXFP8_E4M3"),
                                                          pipeline="mega" if flags.get("mega") else "staged"))
        if factor is not None:
            kw["activation_slot_capacity_factor"] = factor
        plan = dist_moe.plan_memory(dist_moe.Config(**kw), EP)
        slot_bytes, arena, capacity = plan.activation_slot_bytes, plan.total_device_buffer_bytes, \
            plan.total_scratch_capacity_rows
        st = storages[fmt]
        geometry = dict(element_size=2, operand_element_size=st[0], operand_values_per_storage_element=st[1],
                        scale_element_size=st[2], row_scale_storage_multiple=st[3],
                        row_global_scale_element_size=st[4], sf_vec_size=st[5])
        i64 = lambda v: torch.tensor(v, dtype=torch.int64)  # noqa: E731
        buffer_offsets = i64([i * slot_bytes for i in range(slots)] + [arena])
        saved = torch.zeros(max(1, slots * EP), dtype=torch.int64)
        peak = i64([slot_bytes] * slots + [arena - slots * slot_bytes])
        layer = torch.zeros(max(1, slots), dtype=torch.int64)
        mega, native = bool(flags.get("mega")), bool(flags.get("native_backward"))
        steps, fwd_records = [], []
        for op in ops:
            if op[0] == "f":
                _, slot, R, per_rank, scratch_only = op
                need = torch.zeros(1, dtype=torch.bool)
                cond = torch.zeros(1, dtype=torch.int32)
                offsets = torch.zeros(9, dtype=torch.int64)
                table = torch.zeros(18, dtype=torch.int64)
                sel = i64([slot])
                P._triton_get_blockscaled_forward_plan[(1,)](
                    torch.tensor([R], dtype=torch.int32), torch.tensor(per_rank, dtype=torch.int32), None, saved,
                    buffer_offsets, peak, need, cond, offsets, table, EP=EP, num_tokens=T, topk=K, **geometry,
                    hidden_dim=D, intermediate_dim=F, capacity_rows=capacity, microbatch_id_ptr=sel,
                    activation_slot_bytes=slot_bytes, num_activation_slots=slots, moe_layer_id_ptr=layer,
                    num_moe_layers=layers, mega=mega, inference_mode=inference,
                    scratch_only=bool(scratch_only) and not inference, native_backward=native,
                    interleaved_fc13=bool(flags.get("interleaved_fc13")))
                rec = dict(op="f", slot=slot, R=R, per_rank=per_rank, scratch_only=bool(scratch_only),
                           need=bool(need[0]), cond=int(cond[0]), offsets=offsets.tolist(), table=table.tolist())
                fwd_records.append(rec)
            else:
                f = fwd_records[op[1]]
                fo = i64(f["offsets"])
                offsets = torch.zeros(16, dtype=torch.int64)
                table = torch.zeros(54, dtype=torch.int64)
                P._triton_get_blockscaled_backward_plan[(1,)](
                    torch.tensor([f["R"]], dtype=torch.int32), torch.tensor(f["per_rank"], dtype=torch.int32),
                    buffer_offsets, peak, torch.tensor([f["need"]]), fo[0:1], fo[2:3], fo[6:7], fo[8:9], fo[5:6],
                    fo[7:8], saved, offsets, table, EP=EP, num_tokens=T, topk=K, **geometry, hidden_dim=D,
                    intermediate_dim=F, capacity_rows=capacity, microbatch_id_ptr=i64([f["slot"]]),
                    activation_slot_bytes=slot_bytes, num_activation_slots=slots, moe_layer_id_ptr=layer, mega=mega,
                    native_backward=native)
                rec = dict(op="b", of=op[1], offsets=offsets.tolist(), table=table.tolist())
            rec["state"] = dict(buffer_offsets=buffer_offsets.tolist(), saved=saved.tolist(), peak=peak.tolist(),
                                layer=layer.tolist())
            steps.append(rec)
        out[name] = dict(format=fmt, storage=st, EP=EP, T=T, K=K, D=D, F=F, slots=slots, layers=layers,
                         slot_bytes=slot_bytes, arena_bytes=arena, capacity_rows=capacity, flags=flags, steps=steps)
    (HERE / "planner_blockscaled.json").write_text(json.dumps(out, indent=1, sort_keys=True))
    print("planner_blockscaled.json:", len(out), "scenarios")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("DIST_MOE_REFERENCE", "reference"))
    ap.add_argument("--only", default="")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    steps = {"plan": gen_plan_memory, "routing": gen_routing, "planner": gen_planner,
             "planner_blockscaled": gen_planner_blockscaled}
    for name, fn in steps.items():
        if not args.only or name in args.only.split(","):
            fn(args.reference)


if __name__ == "__main__":
    main()
