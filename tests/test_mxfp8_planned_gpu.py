"""MXFP8 training with activations placed by the device planner (bundles in the context's arena) against the same
kernels run on per-call tensors: placement must not change a single bit of the output or of any gradient, whether the
planner saves the layer, recomputes it, or stacks two layers in one slot; afterwards the planner state is rewound and
the peak counters show the slot and the scratch region in use.  The column bundles use the compact scale layout
(sized by the device row count), which the weight-gradient GEMM must read back identically."""

import pytest
import torch

from tests.test_bf16_layer_gpu import make_case

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


def _align(v):
    return (v + 127) // 128 * 128


def _context(dm, T, D, F, K, E, layers=1, slot_bytes=None, **kw):
    sizing = dict(activation_slot_capacity_factor=1.0) if slot_bytes is None else dict(activation_slot_bytes=slot_bytes)
    cfg = dm.Config(max_num_local_input_tokens=T, hidden_dim=D, intermediate_dim=F, top_k=K, num_experts=E,
                    max_moe_layers_per_activation_slot=layers, block_scaled=dm.BlockScaledConfig(), **sizing, **kw)
    return dm.create_context(group=None, config=cfg, device=0)


def _leaves(*tensors):
    return tuple(t.detach().clone().to(DEV).requires_grad_() for t in tensors)


def _rewound(ctx):
    st = ctx._state
    n = st.num_slots
    assert st.buffer_offsets.tolist()[:n] == [i * st.slot_bytes for i in range(n)]
    assert not st.saved_bytes.any().item() and not st.moe_layer_id.any().item()


def _run(dm, ctx, case, planned, *, options=None, grads=(True, True, True, True), layers=1):
    """forward (+ second stacked layer) and backward; returns (outputs and grads, recompute decisions)."""
    import dist_moe_b200._blockscaled as bs

    x, ids, scores, w13, w2 = case
    bs.PLANNED_ARENA = planned
    try:
        leaves = _leaves(x, scores, w13, w2)
        for leaf, wanted in zip(leaves, grads):
            leaf.requires_grad_(wanted)
        ids_d = ids.to(DEV)
        kw = {} if options is None else dict(options=options)
        if layers > 1:
            ctx.select_activation_slot(0, layers)
        h, decisions = leaves[0], []
        for _ in range(layers):
            h = dm.routed_experts(h, ids_d, leaves[1], leaves[2], leaves[3], ctx, **kw)
            if planned:
                decisions.append(ctx._state.last_train_call.need)
        g = torch.randn(h.shape, generator=torch.Generator().manual_seed(5)).bfloat16().to(DEV)
        h.backward(g)
        ctx.check_status()
        got = [h.detach()] + [leaf.grad for leaf in leaves]
        return got, [bool(d.item()) for d in decisions]
    finally:
        bs.PLANNED_ARENA = True


def _same(a, b):
    for i, (p, q) in enumerate(zip(a, b)):
        assert (p is None) == (q is None), i
        if p is not None:
            assert torch.equal(p, q), f"tensor {i} differs between arena placement and per-call tensors"


@pytest.mark.parametrize("recompute", [False, True])
@pytest.mark.parametrize("T,D,F,K,E", [(200, 512, 384, 4, 8), (64, 256, 256, 2, 4), (16, 256, 128, 2, 8)])
def test_planned_placement_is_bit_identical(T, D, F, K, E, recompute):
    import dist_moe_b200 as dm

    case = make_case(T, D, F, K, E, seed=T + K, w_scale=D**-0.5)
    slot = _align(T * D * 2) + 256 if recompute else None  # room for the dense input only
    ctx = _context(dm, T, D, F, K, E, slot_bytes=slot)
    try:
        planned, decisions = _run(dm, ctx, case, True)
        assert decisions == [recompute]
        _rewound(ctx)
        info = ctx.check_overflow()
        assert info.scratch_max_used > 0 and info.slot_max_used[0] > 0
        again, _ = _run(dm, ctx, case, True)
        _same(planned, again)
        plain, _ = _run(dm, ctx, case, False)
        _same(planned, plain)
    finally:
        ctx.close()


@pytest.mark.parametrize("grads", [(True, False, True, True), (False, True, False, True), (True, True, True, False),
                                   (False, False, True, False)])
@pytest.mark.parametrize("recompute", [False, True])
def test_partial_gradients(grads, recompute):
    import dist_moe_b200 as dm

    T, D, F, K, E = 96, 256, 384, 2, 4
    case = make_case(T, D, F, K, E, seed=9, w_scale=D**-0.5)
    ctx = _context(dm, T, D, F, K, E, slot_bytes=_align(T * D * 2) if recompute else None)
    try:
        planned, decisions = _run(dm, ctx, case, True, grads=grads)
        assert decisions == [recompute]
        _rewound(ctx)
        plain, _ = _run(dm, ctx, case, False, grads=grads)
        _same(planned, plain)
    finally:
        ctx.close()


@pytest.mark.parametrize("slot_kind", ["both_saved", "second_recomputed", "both_recomputed"])
def test_two_layers_stacked_in_one_slot(slot_kind):
    import dist_moe_b200 as dm
    from oracle import planner_blockscaled as ob

    T, D, F, K, E = 512, 256, 256, 2, 4
    case = make_case(T, D, F, K, E, seed=3, w_scale=D**-0.5)
    ids = case[1]
    x_mem, h3_mem = _align(T * D * 2), _align(T * K * D * 2)
    # what the planner charges for a saved layer (unpadded rows) and what its bundles occupy (rows padded per expert)
    charged = ob._saved_cost(T * K, h3_mem, D, F, ob.MXFP8, False)
    padded = sum((int((ids == e).sum()) + 127) // 128 * 128 for e in range(E))
    placed = sum(ob.col_sizes(padded, D, ob.MXFP8)) + _align(padded * 2 * F * 2) + sum(ob.col_sizes(padded, F, ob.MXFP8)) \
        + h3_mem
    middle = max(charged, placed) + x_mem + 1024  # layer 1 fits with room for layer 2's input, layer 2 does not
    assert middle < 2 * charged
    slot = {"both_saved": 2 * placed + 4096, "second_recomputed": middle, "both_recomputed": 2 * x_mem}[slot_kind]
    ctx = _context(dm, T, D, F, K, E, layers=2, slot_bytes=slot)
    try:
        planned, decisions = _run(dm, ctx, case, True, layers=2)
        expect = {"both_saved": [False, False], "second_recomputed": [False, True], "both_recomputed": [True, True]}
        assert decisions == expect[slot_kind], (decisions, slot, charged, placed)
        _rewound(ctx)
        plain, _ = _run(dm, ctx, case, False, layers=2)
        _same(planned, plain)
    finally:
        ctx.close()


@pytest.mark.parametrize("recompute", [False, True])
def test_fused_rmsnorm_on_the_planned_path(recompute):
    import dist_moe_b200 as dm

    T, D, F, K, E = 64, 256, 256, 2, 4
    case = make_case(T, D, F, K, E, seed=17, w_scale=D**-0.5)
    ctx = _context(dm, T, D, F, K, E, slot_bytes=_align(T * D * 2) if recompute else None)
    try:
        post = dm.RMSNormPostprocess(eps=1e-5, norm_output_dtype=torch.float32, output_dtype=torch.bfloat16)
        opts = dm.ExecutionOptions(experts_output_postprocess=post)
        planned, decisions = _run(dm, ctx, case, True, options=opts)
        assert decisions == [recompute]
        _rewound(ctx)
        plain, _ = _run(dm, ctx, case, False, options=opts)
        _same(planned, plain)
    finally:
        ctx.close()


def test_slot_below_the_mandatory_inputs_is_refused_at_planning_time():
    import dist_moe_b200 as dm

    T, D = 64, 256
    with pytest.raises(ValueError, match="below the minimum"):
        _context(dm, T, D, 256, 2, 4, slot_bytes=_align(T * D * 2) - 128)


def test_no_grad_call_between_forward_and_backward_leaves_the_slot_alone():
    """An evaluation step (or the first pass of a checkpointed region) on the same context runs on the scratch region
    only; the activations an earlier forward saved in its slot survive it."""
    import dist_moe_b200 as dm

    T, D, F, K, E = 96, 256, 256, 2, 4
    x, ids, scores, w13, w2 = make_case(T, D, F, K, E, seed=41, w_scale=D**-0.5)
    ctx = _context(dm, T, D, F, K, E)
    try:
        ids_d = ids.to(DEV)
        g = torch.randn(T, D, generator=torch.Generator().manual_seed(6)).bfloat16().to(DEV)
        results = []
        for interleave in (False, True):
            leaves = _leaves(x, scores, w13, w2)
            out = dm.routed_experts(leaves[0], ids_d, leaves[1], leaves[2], leaves[3], ctx)
            assert not bool(ctx._state.last_train_call.need.item())  # saved in the slot
            if interleave:
                with torch.no_grad():
                    other = dm.routed_experts(torch.randn_like(leaves[0]), ids_d.flip(0), leaves[1], leaves[2],
                                              leaves[3], ctx)
                assert torch.isfinite(other.float()).all()
            out.backward(g)
            ctx.check_status()
            results.append([out.detach()] + [leaf.grad for leaf in leaves])
        _same(results[0], results[1])
        _rewound(ctx)
    finally:
        ctx.close()


def test_backward_rewinds_the_slot_its_forward_used():
    import dist_moe_b200 as dm

    T, D, F, K, E = 64, 256, 256, 2, 4
    case = make_case(T, D, F, K, E, seed=43, w_scale=D**-0.5)
    x, ids, scores, w13, w2 = case
    ctx = _context(dm, T, D, F, K, E, num_activation_slots=2)
    try:
        ids_d = ids.to(DEV)
        ctx.select_activation_slot(0, 1)
        ref_leaves = _leaves(x, scores, w13, w2)
        ref = dm.routed_experts(ref_leaves[0], ids_d, ref_leaves[1], ref_leaves[2], ref_leaves[3], ctx)
        g = torch.randn_like(ref)
        ref.backward(g)
        ctx.select_activation_slot(1, 1)
        leaves = _leaves(x, scores, w13, w2)
        out = dm.routed_experts(leaves[0], ids_d, leaves[1], leaves[2], leaves[3], ctx)
        assert ctx._state.buffer_offsets[1].item() > ctx._state.slot_bytes  # slot 1 holds this call's bundles
        ctx.select_activation_slot(0, 1)  # another microbatch selects slot 0 before this backward runs
        out.backward(g)
        ctx.check_status()
        _same([ref.detach()] + [leaf.grad for leaf in ref_leaves], [out.detach()] + [leaf.grad for leaf in leaves])
        _rewound(ctx)
    finally:
        ctx.close()


# ---------------------------------------------------------------------------------------------------------------
# Python callbacks on MXFP8 training calls (dist_moe/_blockscaled.py:2596-2700 `_run_blockscaled_eager`)
# ---------------------------------------------------------------------------------------------------------------
def _plain_run(dm, ctx, case, g):
    x, ids, scores, w13, w2 = case
    leaves = _leaves(x, scores, w13, w2)
    out = dm.routed_experts(leaves[0], ids.to(DEV), leaves[1], leaves[2], leaves[3], ctx)
    out.backward(g)
    ctx.check_status()
    return [out.detach()] + [leaf.grad for leaf in leaves]


def test_weights_preprocess_fn_on_an_mxfp8_context():
    """fp32 master weights of another shape are turned into bf16 compute weights (and quantised) in the forward and
    again before the backward; the weight gradients come back in the sources' shapes, bit-identical to a plain call."""
    import dist_moe_b200 as dm

    T, D, F, K, E = 96, 256, 256, 2, 4
    case = make_case(T, D, F, K, E, seed=51, w_scale=D**-0.5)
    x, ids, scores, w13, w2 = case
    ctx = _context(dm, T, D, F, K, E)
    try:
        g = torch.randn(T, D, generator=torch.Generator().manual_seed(7)).bfloat16().to(DEV)
        ref = _plain_run(dm, ctx, case, g)
        calls = []

        def preprocess(w):
            calls.append(tuple(w.shape))
            return w.to(torch.bfloat16).contiguous()

        src13 = w13.float().reshape(E * 2 * F, D).to(DEV).requires_grad_(True)
        src2 = w2.float().to(DEV).requires_grad_(True)
        xs, ss = x.to(DEV).requires_grad_(True), scores.to(DEV).requires_grad_(True)
        out = dm.routed_experts(xs, ids.to(DEV), ss, src13, src2, ctx,
                                options=dm.ExecutionOptions(weights_preprocess_fn=preprocess))
        out.backward(g)
        ctx.check_status()
        assert len(calls) == 4 and calls[0] == (E * 2 * F, D)
        assert src13.grad.shape == src13.shape and src2.grad.shape == src2.shape
        _same(ref, [out.detach(), xs.grad, ss.grad, src13.grad.reshape(ref[3].shape).to(ref[3].dtype),
                    src2.grad.reshape(ref[4].shape).to(ref[4].dtype)])
        _rewound(ctx)
    finally:
        ctx.close()


def test_wgrad_callbacks_on_an_mxfp8_context():
    import dist_moe_b200 as dm

    T, D, F, K, E = 96, 256, 256, 2, 4
    case = make_case(T, D, F, K, E, seed=52, w_scale=D**-0.5)
    x, ids, scores, w13, w2 = case
    ctx = _context(dm, T, D, F, K, E)
    try:
        g = torch.randn(T, D, generator=torch.Generator().manual_seed(7)).bfloat16().to(DEV)
        ref = _plain_run(dm, ctx, case, g)
        taken = {}

        def postprocess(name, grad):
            if name == "w13":
                taken[name] = grad.clone()
                return None
            return (grad.float() * 2).to(grad.dtype)

        leaves = _leaves(x, scores, w13, w2)
        out = dm.routed_experts(leaves[0], ids.to(DEV), leaves[1], leaves[2], leaves[3], ctx,
                                options=dm.ExecutionOptions(wgrad_postprocess_fn=postprocess))
        out.backward(g)
        ctx.check_status()
        assert leaves[2].grad is None and torch.equal(taken["w13"].reshape(ref[3].shape), ref[3])
        assert torch.equal(leaves[3].grad, (ref[4].float() * 2).to(ref[4].dtype))
        assert torch.equal(leaves[0].grad, ref[1])

        dst = {"w13": torch.zeros(E, 2 * F, D, dtype=torch.bfloat16, device=DEV),
               "w2": torch.full((E, D, F), 3.0, dtype=torch.bfloat16, device=DEV)}
        leaves = _leaves(x, scores, w13, w2)
        out = dm.routed_experts(leaves[0], ids.to(DEV), leaves[1], leaves[2], leaves[3], ctx,
                                options=dm.ExecutionOptions(wgrad_destination_fn=lambda n, s, dt, dev: (dst[n], n == "w13")))
        out.backward(g)
        ctx.check_status()
        assert leaves[2].grad is None and leaves[3].grad is None
        assert torch.equal(dst["w13"].reshape(ref[3].shape), ref[3])     # added to zeros
        assert torch.equal(dst["w2"].reshape(ref[4].shape), ref[4])      # overwritten
        _rewound(ctx)
    finally:
        ctx.close()


@pytest.mark.parametrize("recompute", [False, True])
def test_callable_postprocess_on_an_mxfp8_context(recompute):
    """``y = post(h3)`` before the weighted top-k sum; identity gives the plain call bit for bit, a scaling callable
    with a parameter of its own gets that parameter's gradient through the nested backward."""
    import dist_moe_b200 as dm

    T, D, F, K, E = 96, 256, 256, 2, 4
    case = make_case(T, D, F, K, E, seed=53, w_scale=D**-0.5)
    x, ids, scores, w13, w2 = case
    ctx = _context(dm, T, D, F, K, E, slot_bytes=_align(T * D * 2) if recompute else None)
    try:
        g = torch.randn(T, D, generator=torch.Generator().manual_seed(7)).bfloat16().to(DEV)
        ref = _plain_run(dm, ctx, case, g)
        leaves = _leaves(x, scores, w13, w2)
        out = dm.routed_experts(leaves[0], ids.to(DEV), leaves[1], leaves[2], leaves[3], ctx,
                                options=dm.ExecutionOptions(experts_output_postprocess=lambda h3: h3 * 1.0))
        assert bool(ctx._state.last_train_call.need.item()) == recompute
        out.backward(g)
        ctx.check_status()
        _same(ref, [out.detach()] + [leaf.grad for leaf in leaves])
        gain = torch.full((D,), 2.0, dtype=torch.bfloat16, device=DEV, requires_grad=True)
        leaves = _leaves(x, scores, w13, w2)
        out = dm.routed_experts(leaves[0], ids.to(DEV), leaves[1], leaves[2], leaves[3], ctx,
                                options=dm.ExecutionOptions(experts_output_postprocess=lambda h3: h3 * gain))
        out.backward(g)
        ctx.check_status()
        assert torch.allclose(out.float(), 2 * ref[0].float(), rtol=2e-2, atol=2e-2)
        assert gain.grad is not None and torch.isfinite(gain.grad.float()).all() and gain.grad.abs().sum() > 0
        assert torch.allclose(leaves[0].grad.float(), 2 * ref[1].float(), rtol=5e-2, atol=5e-2)
        _rewound(ctx)
    finally:
        ctx.close()
