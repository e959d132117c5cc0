"""GPU parity of the whole layer through `mok.functional` at EP = 1 (one process, one GPU): forward, backward,
context recomputation, the macrobatch ring, SwiGLU clamp, run-to-run bitwise reproducibility.  Checked against
the CPU oracle on the same seeded inputs: BF16 outputs and gradients within rel-L2 <= 1e-2 (the acceptance bound)
and inside the reference's own tolerance (max |diff| <= 0.5, sum|diff|/sum|ref| <= 0.01)."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu

FIELDS = ("d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
          "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")


def _to(dev, inp):
    return {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in vars(inp).items()}


def _run(dist_ctx, inp, E, config, limit=None, recompute=False):
    import torch.distributed as dist
    import mok
    F = mok.functional
    _, _, dev = dist_ctx
    d = _to(dev, inp)
    T, H = inp.x.shape
    K = inp.topk_experts.shape[1]
    ws = F.get_workspace(config, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
    sched = F.build_schedule(ws, config, d["topk_experts"], num_local_experts=E)
    weights = (d["w_shared_gate"], d["w_shared_up"], d["w_shared_down"], d["w_routed_gate"], d["w_routed_up"], d["w_routed_down"])
    out, ctx = F.forward(config, ws, sched, d["x"], d["router_weights"], *weights, swiglu_limit=limit)
    if recompute:
        ctx2 = F.recompute_forward_context(config, ws, sched, d["x"], weights[0], weights[1], weights[3], weights[4], swiglu_limit=limit)
        for name in ("x_routed", "gate_shared", "gate_routed", "up_shared", "up_routed", "hidden_shared", "hidden_routed"):
            n = int(sched.num_tokens.item())
            a, b = getattr(ctx, name), getattr(ctx2, name)
            rows = min(n, a.shape[0]) if "routed" in name else a.shape[0]
            assert torch.equal(a[:rows], b[:rows]), f"recomputed {name} differs from forward"
        ctx = ctx2
    grads = F.backward(config, ws, sched, ctx, d["d_output"], d["x"], d["router_weights"], *weights, swiglu_limit=limit)
    torch.cuda.synchronize()
    mok.ops.check_status(dev)
    return out, grads


def _compare(ref, out, grads, tag):
    problems = []
    for name, got in (("output", out),) + tuple(zip(FIELDS, grads)):
        r = getattr(ref, name).float()
        mx, l1, l2, cos = O.error_stats(r, got.float().cpu())
        if not (mx <= 0.5 and l1 <= 0.01 and l2 <= 0.01 and cos >= 0.9999):
            problems.append(f"{name}: max {mx:.3e} l1 {l1:.3e} l2 {l2:.3e} cos {cos:.6f}")
    assert not problems, tag + " | " + " ; ".join(problems)


CASES = [
    # name, E, H, I, K, T, config kwargs, swiglu limit
    ("all-minimums", 1, 256, 256, 1, 512, {}, None),
    ("small", 4, 256, 512, 2, 512, {}, None),
    ("clamped", 4, 512, 256, 2, 512, {}, 1.0),
    ("ring-2-windows", 4, 256, 256, 4, 512, dict(minibatch_size=256, macrobatch_size=2048), None),
    ("ring-min-window", 8, 256, 256, 2, 512, dict(minibatch_size=256, macrobatch_size=256), None),
    ("many-experts", 64, 256, 256, 8, 1024, {}, None),
]


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_layer_fwd_bwd_matches_oracle(dist_ctx, case):
    import mok
    name, E, H, I, K, T, cfg, limit = case
    config = mok.functional.MoKConfig(**cfg)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    ref = O.moe_layer_oracle([inp], swiglu_limit=limit)[0]
    out, grads = _run(dist_ctx, inp, E, config, limit)
    _compare(ref, out, grads, name)


SWEEP = [("topk-1", 4, 1), ("topk-6", 8, 6), ("local-experts-6", 6, 4), ("local-experts-12", 12, 4), ("local-experts-24", 24, 8),
         ("local-experts-32", 32, 8)]


@pytest.mark.parametrize("name,E,K", SWEEP, ids=[c[0] for c in SWEEP])
def test_topk_values_and_local_expert_counts(dist_ctx, name, E, K):
    """top-k values and local-expert counts of the reference's end-to-end sweeps (tests/test_misc.py:1852,1883), with
    its small ring (minibatch 256, macrobatch 512: every case runs several windows and the backward replay)."""
    import mok
    H, I, T = 512, 256, 512
    # capacity 3 x the routes: with 32 experts the padding to 256 rows per expert alone can double the row count
    config = mok.functional.MoKConfig(minibatch_size=256, macrobatch_size=512, schedule_capacity_multiplier=3.0)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    ref = O.moe_layer_oracle([inp])[0]
    out, grads = _run(dist_ctx, inp, E, config)
    _compare(ref, out, grads, name)


def test_workspace_cache_reuse_and_isolation(dist_ctx):
    """`get_workspace` returns the cached object for the same (group, device, sizes, capacity factor), a new one for a
    larger capacity multiplier or another process group, and `create_workspace` never touches the cache (reference
    tests/test_misc.py:577-645)."""
    import math
    import torch.distributed as dist
    import mok
    F = mok.functional
    _, world, dev = dist_ctx
    F.clear_workspace_cache()
    duplicate_world = dist.new_group(ranks=list(range(world)))
    kwargs = dict(device=dev, num_local_tokens=512, hidden_size=256, topk=1)
    default_config = F.MoKConfig(minibatch_size=256, macrobatch_size=512)
    larger_config = F.MoKConfig(minibatch_size=256, macrobatch_size=512, schedule_capacity_multiplier=2.5)
    try:
        created = F.create_workspace(default_config, dist.group.WORLD, **kwargs)
        default = F.get_workspace(default_config, dist.group.WORLD, **kwargs)
        reused = F.get_workspace(default_config, dist.group.WORLD, **kwargs)
        larger = F.get_workspace(larger_config, dist.group.WORLD, **kwargs)
        duplicate = F.get_workspace(default_config, duplicate_world, **kwargs)
        assert created is not default and reused is default and larger is not default and duplicate is not default
        assert default.schedule_capacity == 512 * max(2, math.ceil(world * 0.5))
        assert larger.schedule_capacity == 512 * max(2, math.ceil(world * 2.5))
        assert duplicate.group_name == duplicate_world.group_name != default.group_name
        assert created.x_buffer.data_ptr() != default.x_buffer.data_ptr()
    finally:
        F.clear_workspace_cache()
        dist.destroy_process_group(duplicate_world)


def test_cpu_plumbing_configuration_against_fp32_math(dist_ctx):
    """The small configuration of the acceptance list (2048 tokens, hidden 512, 8 experts of intermediate 1024, top-2,
    weights ~ N(0, 0.02), seed 0) against plain fp32 math of the same layer: rel-L2 <= 1e-2 for outputs and gradients."""
    import mok
    E, H, I, K, T = 8, 512, 1024, 2, 2048
    inp = O.make_rank_inputs(0, E, E, K, T, H, I, seed=0, weight_std=0.02)
    ref = O.moe_layer_oracle([inp], round_bf16=False)[0]
    out, grads = _run(dist_ctx, inp, E, mok.functional.MoKConfig())
    for name, got in (("output", out),) + tuple(zip(FIELDS, grads)):
        _, _, l2, _ = O.error_stats(getattr(ref, name).float(), got.float().cpu())
        assert l2 <= 1e-2, (name, l2)


@pytest.mark.parametrize("minibatch", [256, 512, 1024, 2048])
def test_imbalanced_routing_minibatch_sweep(dist_ctx, minibatch):
    """Mixtral-like proportions (8 experts, intermediate 3.5x hidden, top-2) with a Zipf(1.2) expert bias, so one expert
    takes the bulk of the routes, at schedule_capacity_multiplier 1.0 and every minibatch size of the sweep; the
    macrobatch equals the minibatch, so the ring and the backward replay are exercised on a skewed schedule."""
    import mok
    E, H, I, K, T = 8, 512, 1792, 2, 2048
    bias = 4.0 * torch.log(torch.arange(1, E + 1, dtype=torch.float32) ** -1.2)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I, seed=3, weight_std=0.02, expert_bias=bias)
    counts = torch.bincount(inp.topk_experts.flatten(), minlength=E).float()
    assert counts.max() / counts.sum() > 0.35                      # the skew is real
    ref = O.moe_layer_oracle([inp])[0]
    config = mok.functional.MoKConfig(minibatch_size=minibatch, macrobatch_size=minibatch, schedule_capacity_multiplier=1.0)
    out, grads = _run(dist_ctx, inp, E, config)
    _compare(ref, out, grads, f"imbalanced/minibatch={minibatch}")


def test_layer_with_recomputed_context_and_bitwise_repeat(dist_ctx):
    import mok
    E, H, I, K, T = 8, 256, 512, 2, 1024
    config = mok.functional.MoKConfig(minibatch_size=256, macrobatch_size=1024)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    ref = O.moe_layer_oracle([inp])[0]
    out1, grads1 = _run(dist_ctx, inp, E, config, recompute=True)
    _compare(ref, out1, grads1, "recompute")
    out2, grads2 = _run(dist_ctx, inp, E, config, recompute=False)
    assert torch.equal(out1, out2)
    for name, a, b in zip(FIELDS, grads1, grads2):
        assert torch.equal(a, b), f"{name} is not bitwise reproducible"


def test_dispatch_and_combine_permutations_are_bit_exact(dist_ctx):
    """x_routed[row] must be the token row the schedule names (zeros on padding rows) and combine_buffer[token*K+k] the
    expert output row of that route — copies, so bit for bit."""
    import torch.distributed as dist
    import mok
    F = mok.functional
    _, _, dev = dist_ctx
    E, H, I, K, T = 8, 256, 256, 4, 512
    config = F.MoKConfig(minibatch_size=256, macrobatch_size=4096)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    d = _to(dev, inp)
    ws = F.get_workspace(config, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
    sched = F.build_schedule(ws, config, d["topk_experts"], num_local_experts=E)
    ws.x_buffer.copy_(d["x"])
    outs = mok.ops.dispatch_mlp_swiglu_combine_fwd_bf16(
        ws.x_buffer, ws.x_buffer_ptrs, ws.combine_buffer, ws.combine_buffer_ptrs, d["w_shared_gate"], d["w_routed_gate"],
        d["w_shared_up"], d["w_routed_up"], d["w_shared_down"], d["w_routed_down"], sched.peer_rank, sched.peer_token_idx,
        sched.num_tokens, sched.tokens_per_expert, K, None, config.fwd_num_comm_sms, config.macrobatch_size, config.minibatch_size)
    x_routed, y_routed = outs[0], outs[8]
    torch.cuda.synchronize()
    n = int(sched.num_tokens.item())
    peer, route = sched.peer_rank[:n].long(), sched.peer_token_idx[:n].long()
    valid = peer >= 0
    expect = torch.zeros(n, H, dtype=torch.bfloat16, device=dev)
    expect[valid] = d["x"][route[valid] // K]
    assert torch.equal(x_routed[:n], expect)
    assert int(valid.sum()) == T * K                                  # every route scheduled exactly once
    assert torch.equal(ws.combine_buffer[route[valid]], y_routed[:n][valid])
    # the schedule the rows follow is the oracle's, bit for bit
    pr, pt, nt, _ = O.schedule_oracle(inp.topk_experts.to(torch.int32).unsqueeze(0).numpy(), E, ws.schedule_capacity, 0)
    assert (sched.peer_rank.cpu().numpy() == pr).all() and (sched.peer_token_idx.cpu().numpy() == pt).all() and n == int(nt[0])


@pytest.mark.parametrize("recompute", [False, True])
def test_autograd_wrapper_matches_functional_calls(dist_ctx, recompute):
    """`mok.moe_layer` under autograd gives exactly what the hand-written forward / backward sequence gives."""
    import mok
    _, _, dev = dist_ctx
    E, H, I, K, T = 4, 256, 256, 2, 512
    config = mok.functional.MoKConfig(minibatch_size=256, macrobatch_size=1024)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    out_ref, grads_ref = _run(dist_ctx, inp, E, config)
    d = _to(dev, inp)
    leaves = {k: d[k].clone().requires_grad_() for k in ("x", "router_weights", "w_shared_gate", "w_shared_up", "w_shared_down",
                                                           "w_routed_gate", "w_routed_up", "w_routed_down")}
    out = mok.moe_layer(leaves["x"], d["topk_experts"], leaves["router_weights"], leaves["w_shared_gate"], leaves["w_shared_up"],
                        leaves["w_shared_down"], leaves["w_routed_gate"], leaves["w_routed_up"], leaves["w_routed_down"],
                        config=config, recompute=recompute)
    out.backward(d["d_output"])
    torch.cuda.synchronize()
    assert torch.equal(out.detach(), out_ref)
    order = ("x", "router_weights", "w_routed_gate", "w_routed_up", "w_routed_down", "w_shared_gate", "w_shared_up", "w_shared_down")
    for name, ref in zip(order, grads_ref):
        assert torch.equal(leaves[name].grad, ref), name


def test_moe_module_trains_one_step(dist_ctx):
    import mok
    _, _, dev = dist_ctx
    torch.manual_seed(0)
    layer = mok.MoKMoE(256, 256, 8, 2, device=dev, config=mok.functional.MoKConfig(minibatch_size=256, macrobatch_size=2048))
    x = torch.randn(512, 256, device=dev, dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    y.float().square().mean().backward()
    torch.cuda.synchronize()
    mok.ops.check_status(dev)
    assert y.shape == x.shape and torch.isfinite(y.float()).all()
    for name, p in layer.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad.float()).all() and p.grad.float().abs().sum() > 0, name
    assert x.grad is not None and torch.isfinite(x.grad.float()).all()


def test_forward_backward_trace_as_one_graph(dist_ctx):
    """The ops are opaque custom ops with shape functions, so `torch.compile(fullgraph=True)` captures the whole
    forward + backward call sequence (the reference pins this, tests/test_misc.py:1262-1521); the compiled function
    returns what the eager one returns."""
    import torch.distributed as dist
    import mok
    F = mok.functional
    _, _, dev = dist_ctx
    E, H, I, K, T = 4, 256, 256, 2, 512
    config = F.MoKConfig(minibatch_size=256, macrobatch_size=1024)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    d = _to(dev, inp)
    ws = F.get_workspace(config, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
    weights = (d["w_shared_gate"], d["w_shared_up"], d["w_shared_down"], d["w_routed_gate"], d["w_routed_up"], d["w_routed_down"])

    def layer(x, top_experts, rw, d_out):
        sched = F.build_schedule(ws, config, top_experts, num_local_experts=E)
        out, ctx = F.forward(config, ws, sched, x, rw, *weights)
        grads = F.backward(config, ws, sched, ctx, d_out, x, rw, *weights)
        return out, grads[0], grads[1], grads[2]

    eager = layer(d["x"], d["topk_experts"], d["router_weights"], d["d_output"])
    compiled = torch.compile(layer, backend="eager", fullgraph=True)(d["x"], d["topk_experts"], d["router_weights"], d["d_output"])
    torch.cuda.synchronize()
    for a, b in zip(eager, compiled):
        assert torch.equal(a, b)


def test_chunked_two_stream_pipeline_equals_single_stream(dist_ctx, monkeypatch):
    """Dispatch / combine on the internal stream with many small chunks gives bit-identical results to the plain
    single-stream order (same kernels, same per-element arithmetic)."""
    import mok
    E, H, I, K, T = 8, 256, 256, 4, 1024
    config = mok.functional.MoKConfig(minibatch_size=256, macrobatch_size=2048)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    monkeypatch.setenv("MOK_NO_OVERLAP", "1")
    out_a, grads_a = _run(dist_ctx, inp, E, config)
    monkeypatch.delenv("MOK_NO_OVERLAP")
    monkeypatch.setenv("MOK_CHUNK_ROWS", "256")
    out_b, grads_b = _run(dist_ctx, inp, E, config)
    monkeypatch.delenv("MOK_CHUNK_ROWS")
    _compare(O.moe_layer_oracle([inp])[0], out_b, grads_b, "chunked")
    assert torch.equal(out_a, out_b)
    for name, a, b in zip(FIELDS, grads_a, grads_b):
        assert torch.equal(a, b), name


def test_degenerate_routing_all_tokens_pick_first_experts(dist_ctx):
    import mok
    E, H, I, K, T = 16, 256, 256, 8, 512
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    inp.topk_experts = torch.arange(K).expand(T, K).contiguous()
    ref = O.moe_layer_oracle([inp])[0]
    out, grads = _run(dist_ctx, inp, E, mok.functional.MoKConfig(minibatch_size=256, macrobatch_size=512))
    _compare(ref, out, grads, "degenerate")
    # experts 8..15 received nothing: their weight gradients are exactly zero
    for g in grads[2:5]:
        assert torch.count_nonzero(g[K:]) == 0


@pytest.mark.parametrize("limit", [None, 1.0])
def test_swiglu_in_the_gemm_epilogue_equals_the_separate_kernel(dist_ctx, monkeypatch, limit):
    """By default the forward gate / up GEMM forms hidden = silu(gate) * up in its epilogue from the bf16-rounded gate
    and up it stores; with MOK_NO_FUSED_SWIGLU=1 a separate kernel reads gate and up back.  Same arithmetic on the same
    values, so every output and gradient is bitwise equal (routed and shared expert, ring of two windows)."""
    import mok
    E, H, I, K, T = 8, 256, 768, 2, 1024
    config = mok.functional.MoKConfig(minibatch_size=256, macrobatch_size=2048)
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    monkeypatch.setenv("MOK_NO_FUSED_SWIGLU", "1")
    out_a, grads_a = _run(dist_ctx, inp, E, config, limit)
    monkeypatch.delenv("MOK_NO_FUSED_SWIGLU")
    out_b, grads_b = _run(dist_ctx, inp, E, config, limit, recompute=True)
    _compare(O.moe_layer_oracle([inp], swiglu_limit=limit)[0], out_b, grads_b, "fused swiglu")
    assert torch.equal(out_a, out_b)
    for name, a, b in zip(FIELDS, grads_a, grads_b):
        assert torch.equal(a, b), name
