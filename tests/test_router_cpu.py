"""CPU checks around the device router: the float64 oracle states the same expression the reference's tests use to draw
routes (tests/utils.py:82-84: top-k of the logits, softmax over the selected values), its backward equals autograd of
that expression, and the ops' shape functions match their documented outputs."""
import torch

from oracle import moe_oracle as O


def test_router_oracle_is_topk_then_softmax_of_selected_logits():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 32, generator=g, dtype=torch.bfloat16)
    w = torch.randn(16, 32, generator=g)
    b = torch.randn(16, generator=g)
    experts, weights, logits = O.router_oracle(x, w, b, 4)
    ref_logits = x.float() @ w.t() + b
    vals, idx = torch.topk(ref_logits, 4, dim=1)
    assert torch.equal(experts, idx)
    torch.testing.assert_close(weights.float(), torch.softmax(vals.float(), dim=-1), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(logits.float(), x.float() @ w.t(), rtol=1e-5, atol=1e-5)
    assert torch.allclose(weights.sum(1), torch.ones(64, dtype=torch.float64))


def test_router_backward_oracle_matches_the_closed_form():
    g = torch.Generator().manual_seed(1)
    x = torch.randn(32, 16, generator=g, dtype=torch.bfloat16)
    w = torch.randn(8, 16, generator=g)
    experts, weights, _ = O.router_oracle(x, w, None, 2)
    d_weights = torch.randn(32, 2, generator=g)
    d_x, d_w, d_b = O.router_bwd_oracle(x, w, None, experts, d_weights)
    assert d_b is None
    # softmax backward on the selected logits, scattered to a dense [T, E] gradient
    d_v = weights * (d_weights.double() - (weights * d_weights.double()).sum(1, keepdim=True))
    d_logits = torch.zeros(32, 8, dtype=torch.float64).scatter_(1, experts, d_v)
    torch.testing.assert_close(d_x, d_logits @ w.double())
    torch.testing.assert_close(d_w, d_logits.t() @ x.double())


def test_router_shape_functions():
    import mok  # noqa: F401
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        x = torch.empty(512, 256, dtype=torch.bfloat16)
        w = torch.empty(24, 256)
        routes, weights, logits = torch.ops.mok.router_fwd(x, w, None, 4)
        assert (routes.shape, routes.dtype) == ((512, 4), torch.int32)
        assert (weights.shape, weights.dtype) == ((512, 4), torch.float32)
        assert (logits.shape, logits.dtype) == ((512, 24), torch.float32)
        d_x, d_w, d_b = torch.ops.mok.router_bwd(x, w, routes, weights, weights, False)
        assert d_x.shape == x.shape and d_x.dtype == torch.bfloat16
        assert (d_w.shape, d_w.dtype, d_b.shape) == ((24, 256), torch.float32, (24,))


def test_two_bf16_terms_carry_an_fp32_router_matrix():
    """`hi + lo` (both bf16) reproduces an fp32 matrix to about 16 mantissa bits, which is what keeps the device logits
    within 2e-4 of the fp32 product; rows added as padding are zero."""
    from mok.ops import _router_terms
    g = torch.Generator().manual_seed(2)
    w = torch.randn(24, 256, generator=g)
    hi, lo = _router_terms(w, 256)
    assert hi.shape == (256, 256) and lo.shape == (256, 256) and hi.dtype == lo.dtype == torch.bfloat16
    assert torch.count_nonzero(hi[24:]) == 0 and torch.count_nonzero(lo[24:]) == 0
    err = (hi[:24].float() + lo[:24].float() - w).abs() / w.abs().clamp_min(1e-30)
    assert err.max() < 2.0 ** -15
    hi_only, none = _router_terms(w.to(torch.bfloat16), 256)
    assert none is None and torch.equal(hi_only[:24], w.to(torch.bfloat16))
