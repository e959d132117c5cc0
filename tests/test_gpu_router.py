"""GPU parity of the device router (logits GEMM with fp32 output, top-k + softmax kernel, backward) against the float64
restatement of the expression the reference's tests use for their routes (tests/utils.py:82-84).

Routing indices must equal `torch.topk` of the float64 logits except where two logits are closer than the fp32
accumulation noise of the device product (|gap| < 1e-4 here; such near-ties are counted and must be rare); weights
agree to 1e-5; logits to 2e-4 (bf16 x, fp32 weight carried as two bf16 terms, fp32 accumulation)."""
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import mok  # noqa: F401
    return torch.device("cuda", 0)


def _inputs(T, H, E, w_dtype, with_bias, seed=5):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(T, H, generator=g, dtype=torch.bfloat16)
    w = (torch.randn(E, H, generator=g) * H ** -0.5).to(w_dtype)
    b = torch.randn(E, generator=g) * 0.5 if with_bias else None
    return x, w, b


CASES = [
    # T, H, E, topk, weight dtype, bias
    (512, 256, 256, 8, torch.float32, False),      # DeepSeek-like expert count
    (1024, 512, 128, 8, torch.float32, True),      # experts padded to 256 columns, bias (Qwen3-like count)
    (512, 256, 8, 2, torch.bfloat16, False),       # Mixtral-like count, bf16 weight (single term)
    (768, 1024, 384, 6, torch.float32, True),      # two column tiles, 12 logits per lane
    (512, 256, 1024, 32, torch.float32, False),    # the limits: 1024 experts, top-32
]


@pytest.mark.parametrize("T,H,E,K,w_dtype,with_bias", CASES)
def test_router_forward_matches_float64_topk(dev, T, H, E, K, w_dtype, with_bias):
    import mok
    x, w, b = _inputs(T, H, E, w_dtype, with_bias)
    routes, weights, logits = mok.ops.router_fwd(x.to(dev), w.to(dev), b.to(dev) if with_bias else None, K)
    torch.cuda.synchronize()
    mok.ops.check_status(dev)
    ref_routes, ref_weights, ref_logits = O.router_oracle(x, w, b, K)
    assert routes.dtype == torch.int32 and weights.dtype == torch.float32 and tuple(logits.shape) == (T, E)
    assert (logits.cpu().double() - ref_logits).abs().max() <= 2e-4 * max(1.0, ref_logits.abs().max().item())
    got = routes.cpu().long()
    same = (got == ref_routes).all(dim=1)
    # tokens whose routes differ must be near-ties: the device's own choice has (almost) the same logits
    biased = ref_logits if b is None else ref_logits + b.double()
    if not same.all():
        bad = (~same).nonzero().flatten()
        assert bad.numel() <= max(1, T // 100)
        gap = (torch.gather(biased[bad], 1, got[bad]).sort(dim=1).values -
               torch.gather(biased[bad], 1, ref_routes[bad]).sort(dim=1).values).abs().max()
        assert gap < 1e-4
    assert (got.sort(dim=1).values[:, 1:] != got.sort(dim=1).values[:, :-1]).all()       # k distinct experts per token
    torch.testing.assert_close(weights.cpu().double()[same], ref_weights[same], rtol=1e-4, atol=1e-5)
    assert torch.allclose(weights.sum(dim=1).cpu(), torch.ones(T), atol=1e-5)
    assert (weights[:, :-1] >= weights[:, 1:]).all()                                         # descending, like torch.topk


@pytest.mark.parametrize("T,H,E,K,w_dtype,with_bias", CASES[:4])
def test_router_backward_matches_autograd(dev, T, H, E, K, w_dtype, with_bias):
    import mok
    x, w, b = _inputs(T, H, E, w_dtype, with_bias, seed=9)
    g = torch.Generator().manual_seed(10)
    d_weights = torch.randn(T, K, generator=g)
    routes, weights, _ = mok.ops.router_fwd(x.to(dev), w.to(dev), b.to(dev) if with_bias else None, K)
    d_x, d_w, d_b = mok.ops.router_bwd(x.to(dev), w.to(dev), routes, weights, d_weights.to(dev), with_bias)
    torch.cuda.synchronize()
    mok.ops.check_status(dev)
    rx, rw, rb = O.router_bwd_oracle(x, w, b, routes.cpu(), d_weights)
    # d_logits travels as bf16 (like every activation gradient of the layer): rel-L2 1e-2, the layer's own bound
    for name, got, ref in (("d_x", d_x, rx), ("d_w_router", d_w, rw)) + ((("d_bias", d_b, rb),) if with_bias else ()):
        _, _, l2, _ = O.error_stats(ref, got.cpu())
        assert l2 <= 1e-2, (name, l2)
    assert tuple(d_w.shape) == (E, H) and d_w.dtype == torch.float32
    if not with_bias:
        assert torch.count_nonzero(d_b) == 0


def test_route_function_trains_through_the_layer(dist_ctx):
    """mok.route feeds build_schedule / forward with int32 routes and carries the gradient of the router weights back to
    the router matrix and to x (the module does exactly this)."""
    import mok
    _, _, dev = dist_ctx
    torch.manual_seed(3)
    layer = mok.MoKMoE(256, 256, 8, 2, device=dev)
    x = torch.randn(512, 256, device=dev, dtype=torch.bfloat16, requires_grad=True)
    out = layer(x)
    out.float().square().mean().backward()
    torch.cuda.synchronize()
    mok.ops.check_status(dev)
    assert tuple(layer.router.shape) == (8, 256)
    for p in (layer.router, layer.w_routed_gate, layer.w_shared_down):
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0
    assert x.grad is not None and torch.isfinite(x.grad).all()


def test_router_rejects_bad_arguments(dev):
    import mok
    x, w, b = _inputs(512, 256, 16, torch.float32, True)
    x, w, b = x.to(dev), w.to(dev), b.to(dev)
    mok.ops.router_fwd(x, w, b, 2)
    for kwargs, exc in (
        (dict(x=x[:384]), ValueError), (dict(x=x.float()), TypeError), (dict(w_router=w[:, :128].contiguous()), ValueError),
        (dict(w_router=w.half()), TypeError), (dict(bias=b[:8]), ValueError), (dict(topk=0), ValueError), (dict(topk=17), ValueError),
    ):
        with pytest.raises(exc):
            mok.ops.router_fwd(**(dict(x=x, w_router=w, bias=b, topk=2) | kwargs))


def test_module_quantizes_its_weights_once_until_they_change(dist_ctx, monkeypatch):
    """MoKMoE(mxfp8=True) keeps the MXFP8 copies of its routed weights between calls and rebuilds them after an
    in-place update of a weight (what an optimizer step does)."""
    import mok
    _, _, dev = dist_ctx
    torch.manual_seed(4)
    layer = mok.MoKMoE(256, 256, 8, 2, device=dev, mxfp8=True)
    calls = []
    original = mok.ops.mxfp8_quantize
    monkeypatch.setattr(mok.ops, "mxfp8_quantize", lambda *a: (calls.append(1), original(*a))[1])
    x = torch.randn(512, 256, device=dev, dtype=torch.bfloat16)
    with torch.no_grad():
        out1 = layer(x)
        out2 = layer(x)
    assert len(calls) == 3 and torch.equal(out1, out2)          # gate, up, down: once
    with torch.no_grad():
        layer.w_routed_down.mul_(0.5)
        out3 = layer(x)
    assert len(calls) == 6 and not torch.equal(out1, out3)
    layer(x).float().sum().backward()                           # training path uses the cached copies too
    assert len(calls) == 6 and layer.w_routed_gate.grad is not None
    torch.cuda.synchronize()
    mok.ops.check_status(dev)
