"""Invalid-argument tables for the operators, in the style of the reference's own operator tests
(tests/test_ops.py:148-170, 228-247, 591-605): every op is first called with valid arguments on the GPU, then once per
row with one argument replaced, and must raise the listed exception type before anything is launched."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


def _expect_failures(fn, valid, table):
    for name, overrides, exc in table:
        with pytest.raises(exc):
            fn(**(valid | overrides))
            pytest.fail(f"{name} should have failed")


@pytest.fixture(scope="module")
def problem(dist_ctx):
    import torch.distributed as dist
    import mok
    F = mok.functional
    _, _, dev = dist_ctx
    E, H, I, K, T = 4, 256, 256, 2, 512
    inp = O.make_rank_inputs(0, E, E, K, T, H, I)
    d = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in vars(inp).items()}
    config = F.MoKConfig()
    ws = F.get_workspace(config, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
    sched = F.build_schedule(ws, config, d["topk_experts"], num_local_experts=E)
    return dict(d=d, ws=ws, sched=sched, config=config, dims=(E, H, I, K, T), dev=dev)


def test_all_gather_top_experts_rejects_bad_arguments(problem):
    import mok
    ws, d = problem["ws"], problem["d"]
    valid = dict(top_experts=d["topk_experts"].to(torch.int32).contiguous(),
                 all_gather_top_experts_buffer=ws.all_gather_top_experts_buffer,
                 all_gather_top_experts_buffer_multicast_ptr=ws.all_gather_top_experts_buffer_multicast_ptr,
                 rank=0, chunk_bytes=16)
    mok.ops.all_gather_top_experts(**valid)
    assert torch.equal(ws.all_gather_top_experts_buffer[0], valid["top_experts"])
    _expect_failures(mok.ops.all_gather_top_experts, valid, (
        ("top_experts dtype", {"top_experts": valid["top_experts"].to(torch.int64)}, ValueError),
        ("buffer dtype", {"all_gather_top_experts_buffer": ws.all_gather_top_experts_buffer.to(torch.int64)}, TypeError),
        ("multicast pointer", {"all_gather_top_experts_buffer_multicast_ptr": 0}, TypeError),
        ("rank", {"rank": ws.ep_size}, ValueError),
        ("chunk alignment", {"chunk_bytes": 15}, ValueError),
        ("chunk divisibility", {"chunk_bytes": 48}, ValueError),
    ))


def test_schedule_rejects_bad_arguments(problem):
    import mok
    ws = problem["ws"]
    E, H, I, K, T = problem["dims"]
    topk_all = ws.all_gather_top_experts_buffer
    valid = dict(topk_all=topk_all, num_local_experts=E, schedule_capacity=ws.schedule_capacity, rank=0)
    mok.ops.schedule(**valid)
    _expect_failures(mok.ops.schedule, valid, (
        ("topk_all rank", {"topk_all": topk_all[0]}, ValueError),
        ("topk_all dtype", {"topk_all": topk_all.to(torch.int64)}, ValueError),
        ("local experts", {"num_local_experts": 0}, ValueError),
        ("schedule capacity zero", {"schedule_capacity": 0}, ValueError),
        ("schedule capacity alignment", {"schedule_capacity": 128}, ValueError),
        ("schedule capacity size", {"schedule_capacity": 256}, ValueError),
        ("rank", {"rank": ws.ep_size}, ValueError),
    ))


def test_mxfp8_quantize_rejects_bad_arguments(problem):
    import mok
    x = torch.randn(256, 384, device=problem["dev"], dtype=torch.bfloat16)
    valid = dict(x_bf16=x, return_normal=True, return_transposed=True)
    mok.ops.mxfp8_quantize(**valid)
    _expect_failures(mok.ops.mxfp8_quantize, valid, (
        ("rank", {"x_bf16": x[0]}, ValueError),
        ("row alignment", {"x_bf16": x[:192].contiguous()}, ValueError),
        ("column alignment", {"x_bf16": x[:, :192].contiguous()}, ValueError),
        ("dtype", {"x_bf16": x.float()}, ValueError),
        ("non-contiguous", {"x_bf16": x.t()[:256, :256]}, ValueError),
        ("no layout", {"return_normal": False, "return_transposed": False}, ValueError),
    ))


def _fwd_kwargs(problem):
    ws, d, s = problem["ws"], problem["d"], problem["sched"]
    E, H, I, K, T = problem["dims"]
    ws.x_buffer.copy_(d["x"])
    return dict(
        x=ws.x_buffer, x_ptrs=ws.x_buffer_ptrs, combine_buffer=ws.combine_buffer, combine_buffer_ptrs=ws.combine_buffer_ptrs,
        w_shared_gate=d["w_shared_gate"], w_routed_gate=d["w_routed_gate"], w_shared_up=d["w_shared_up"],
        w_routed_up=d["w_routed_up"], w_shared_down=d["w_shared_down"], w_routed_down=d["w_routed_down"],
        schedule_peer_rank=s.peer_rank, schedule_peer_token_idx=s.peer_token_idx, num_tokens=s.num_tokens,
        tokens_per_expert=s.tokens_per_expert, topk=K, swiglu_limit=None, num_comm_sms=40, macrobatch_size=2048,
        minibatch_size=256)


def test_forward_bf16_rejects_bad_arguments(problem):
    import mok
    ws, d = problem["ws"], problem["d"]
    valid = _fwd_kwargs(problem)
    mok.ops.dispatch_mlp_swiglu_combine_fwd_bf16(**valid)
    torch.cuda.synchronize()
    mok.ops.check_status(problem["dev"])
    _expect_failures(mok.ops.dispatch_mlp_swiglu_combine_fwd_bf16, valid, (
        ("input rank", {"x": ws.x_buffer.unsqueeze(0)}, ValueError),
        ("input dtype", {"x": ws.x_buffer.float()}, TypeError),
        ("top-k", {"topk": 0}, ValueError),
        ("negative clamp", {"swiglu_limit": -1.0}, ValueError),
        ("communication SMs", {"num_comm_sms": 1}, ValueError),
        ("minibatch alignment", {"minibatch_size": 128}, ValueError),
        ("macrobatch multiple", {"macrobatch_size": 384}, ValueError),
        ("null pointer", {"x_ptrs": [0] * len(ws.x_buffer_ptrs)}, TypeError),
        ("pointer EP size", {"combine_buffer_ptrs": ws.combine_buffer_ptrs + ws.combine_buffer_ptrs}, ValueError),
        ("weight shape", {"w_routed_up": d["w_routed_up"][:, :128].contiguous()}, ValueError),
        ("weight dtype", {"w_shared_down": d["w_shared_down"].float()}, TypeError),
        ("schedule length", {"schedule_peer_token_idx": problem["sched"].peer_token_idx[:256]}, ValueError),
        ("combine buffer shape", {"combine_buffer": ws.combine_buffer[:256]}, ValueError),
    ))


def test_backward_bf16_and_recompute_reject_bad_arguments(problem):
    import mok
    F = mok.functional
    ws, d, s, config = problem["ws"], problem["d"], problem["sched"], problem["config"]
    weights = (d["w_shared_gate"], d["w_shared_up"], d["w_shared_down"], d["w_routed_gate"], d["w_routed_up"], d["w_routed_down"])
    out, ctx = F.forward(config, ws, s, d["x"], d["router_weights"], *weights)
    F.backward(config, ws, s, ctx, d["d_output"], d["x"], d["router_weights"], *weights)
    torch.cuda.synchronize()
    for name, kwargs, exc in (
        ("x dtype", dict(x=d["x"].float()), ValueError),
        ("x shape", dict(x=d["x"][:256]), ValueError),
        ("d_output shape", dict(d_output=d["d_output"][:, :128]), ValueError),
        ("router weights dtype", dict(router_weights=d["router_weights"].to(torch.bfloat16)), ValueError),
    ):
        call = dict(d_output=d["d_output"], x=d["x"], router_weights=d["router_weights"]) | kwargs
        with pytest.raises(exc):
            F.backward(config, ws, s, ctx, call["d_output"], call["x"], call["router_weights"], *weights)
            pytest.fail(f"{name} should have failed")
    with pytest.raises((ValueError, TypeError)):
        F.recompute_forward_context(config, ws, s, d["x"][:, :128], weights[0], weights[1], weights[3], weights[4])


def test_epilogues_reject_bad_arguments(problem):
    import mok
    E, H, I, K, T = problem["dims"]
    dev = problem["dev"]
    y = torch.randn(T, H, device=dev, dtype=torch.bfloat16)
    slots = torch.randn(T * K, H, device=dev, dtype=torch.bfloat16)
    w = torch.rand(T, K, device=dev)
    valid = dict(y_shared=y, combine_buffer=slots, topk_weights=w)
    mok.ops.fwd_epilogue(**valid)
    _expect_failures(mok.ops.fwd_epilogue, valid, (
        ("y rank", {"y_shared": y[0]}, ValueError),
        ("token alignment", {"y_shared": y[:384]}, ValueError),
        ("hidden alignment", {"y_shared": y[:, :128].contiguous()}, ValueError),
        ("weights shape", {"topk_weights": w[:256]}, ValueError),
        ("slot shape", {"combine_buffer": slots[:T]}, ValueError),
    ))
    valid = dict(d_x_shared=y, d_x_routed_buffer=slots)
    mok.ops.bwd_epilogue(**valid)
    _expect_failures(mok.ops.bwd_epilogue, valid, (
        ("rank", {"d_x_shared": y[0]}, ValueError),
        ("token alignment", {"d_x_shared": y[:384]}, ValueError),
        ("slot rows", {"d_x_routed_buffer": slots[:T + 256]}, ValueError),
        ("slot hidden", {"d_x_routed_buffer": slots[:, :128].contiguous()}, ValueError),
    ))


def test_workspace_and_schedule_validation(problem):
    import torch.distributed as dist
    import mok
    F = mok.functional
    dev = problem["dev"]
    E, H, I, K, T = problem["dims"]
    for kwargs, exc in (
        (dict(num_local_tokens=384, hidden_size=H, topk=K), ValueError),
        (dict(num_local_tokens=T, hidden_size=H + 64, topk=K), ValueError),
        (dict(num_local_tokens=T, hidden_size=H, topk=0), ValueError),
    ):
        with pytest.raises(exc):
            F.create_workspace(problem["config"], dist.group.WORLD, device=dev, **kwargs)
    with pytest.raises((ValueError, TypeError)):
        F.build_schedule(problem["ws"], problem["config"], problem["d"]["topk_experts"][:, :1], num_local_experts=E)
    with pytest.raises(ValueError):
        F.build_schedule(problem["ws"], problem["config"], problem["d"]["topk_experts"], num_local_experts=0)
