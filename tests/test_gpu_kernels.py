"""GPU parity tests of the individual kernels, called through the C ABI (via `mok.ops`) and checked against the
CPU oracle / golden fixtures.  Integer and byte results must match bit for bit; bf16 GEMM results within
rel-L2 <= 1e-2 of fp32 math on the same inputs (observed ~3e-3, the bf16 output rounding)."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import mok  # noqa: F401  (fails loudly when the native library is missing)
    return torch.device("cuda", 0)


def _rel_l2(ref, got):
    ref, got = ref.double(), got.double()
    return ((ref - got).norm() / ref.norm().clamp_min(1e-30)).item()


# ---------------------------------------------------------------------------------------------------------
# schedule
# ---------------------------------------------------------------------------------------------------------
def _check_schedule(dev, topk_all, e_loc, cap, rank):
    import mok
    got = mok.ops.schedule(topk_all.to(dev), e_loc, cap, rank)
    ref = O.schedule_oracle(topk_all.numpy(), e_loc, cap, rank)
    for name, r, g in zip(("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert"), ref, got):
        assert np.array_equal(r, g.cpu().numpy()), f"{name} differs (ep={topk_all.shape[0]} rank={rank})"
    mok.ops.check_status(dev)


@pytest.mark.parametrize("ep,E,K,T", [
    (1, 8, 2, 2048),      # CPU-plumbing configuration
    (1, 1, 1, 512),       # all minimums
    (2, 16, 3, 768),      # routes not a multiple of 1024
    (4, 32, 8, 1024),
    (8, 64, 6, 512),
    (8, 8, 8, 512),       # one local expert per rank
    (1, 256, 8, 4096),    # many local experts
])
def test_schedule_matches_oracle(dev, ep, E, K, T):
    g = torch.Generator().manual_seed(100 + ep + E)
    topk_all = torch.stack([torch.topk(torch.randn(T, E, generator=g), K, dim=1).indices for _ in range(ep)]).to(torch.int32)
    cap = T * K * max(2, math.ceil(ep * 1.5))
    for rank in sorted({0, ep - 1, ep // 2}):
        _check_schedule(dev, topk_all, E // ep, cap, rank)


def test_schedule_golden_and_exact_capacity(dev, golden_dir):
    import glob
    for path in sorted(glob.glob(os.path.join(golden_dir, "sched_*.npz"))):
        g = np.load(path)
        e_loc, cap, rank = (int(v) for v in g["meta"])
        import mok
        got = mok.ops.schedule(torch.from_numpy(g["topk_all"]).to(dev), e_loc, cap, rank)
        assert np.array_equal(got[0].cpu().numpy(), g["peer_rank"]), path
        valid = g["peer_rank"] >= 0
        assert np.array_equal(got[1].cpu().numpy()[valid], g["peer_token_idx"][valid]), path
        assert np.array_equal(got[2].cpu().numpy(), g["num_tokens"]), path
        assert np.array_equal(got[3].cpu().numpy(), g["tokens_per_expert"]), path


def test_schedule_imbalanced_and_empty_experts(dev):
    # every token picks experts 0..K-1 (the reference's degenerate-routing case) -> the other experts are empty
    T, K, E = 512, 4, 16
    topk = torch.arange(K, dtype=torch.int32).expand(T, K).contiguous()
    topk_all = torch.stack([topk, topk])
    _check_schedule(dev, topk_all, E // 2, T * K * 2, 0)
    _check_schedule(dev, topk_all, E // 2, T * K * 2, 1)


def test_schedule_overflow_sets_status_instead_of_trapping(dev):
    import mok
    T, K = 512, 1
    topk_all = torch.zeros(2, T, K, dtype=torch.int32)          # both ranks send everything to expert 0 of rank 0
    out = mok.ops.schedule(topk_all.to(dev), 1, T * K, 0)        # 1024 routes into a capacity of 512
    torch.cuda.synchronize()
    assert int(out[2].item()) == 1024
    # while the word holds an error bit the epilogues hand out NaN instead of sums over slots that may be stale
    shared = torch.ones(T, 256, device=dev, dtype=torch.bfloat16)
    routed = torch.ones(T * K, 256, device=dev, dtype=torch.bfloat16)
    w = torch.ones(T, K, device=dev)
    assert torch.isnan(mok.ops.fwd_epilogue(shared, routed, w).float()).all()
    assert torch.isnan(mok.ops.bwd_epilogue(shared, routed).float()).all()
    with pytest.raises(RuntimeError, match="schedule overflow"):
        mok.ops.check_status(dev)
    mok.ops.check_status(dev)   # the word was reset
    assert torch.all(mok.ops.fwd_epilogue(shared, routed, w) == 2.0)
    assert torch.all(mok.ops.bwd_epilogue(shared, routed) == 2.0)


def test_schedule_rejects_bad_arguments(dev):
    import mok
    topk_all = torch.zeros(1, 512, 1, dtype=torch.int32, device=dev)
    ok = dict(topk_all=topk_all, num_local_experts=1, schedule_capacity=512, rank=0)
    for bad in (dict(topk_all=topk_all.squeeze(-1)), dict(num_local_experts=0), dict(schedule_capacity=0),
                dict(schedule_capacity=128), dict(schedule_capacity=256), dict(rank=1)):
        with pytest.raises(ValueError):
            mok.ops.schedule(**(ok | bad))


# ---------------------------------------------------------------------------------------------------------
# epilogues
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,H,K", [(512, 256, 1), (512, 512, 8), (1024, 256, 55), (768, 1024, 3)])
def test_epilogues_match_oracle(dev, T, H, K):
    import mok
    g = torch.Generator().manual_seed(7)
    ys = torch.randn(T, H, generator=g, dtype=torch.bfloat16)
    cb = torch.randn(T * K, H, generator=g, dtype=torch.bfloat16)
    w = torch.softmax(torch.randn(T, K, generator=g), dim=-1)
    fwd = mok.ops.fwd_epilogue(ys.to(dev), cb.to(dev), w.to(dev)).cpu()
    bwd = mok.ops.bwd_epilogue(ys.to(dev), cb.to(dev)).cpu()
    rf, rb = O.fwd_epilogue_oracle(ys, cb, w), O.bwd_epilogue_oracle(ys, cb)
    # same order of additions; the device fuses w*r+acc into one rounding, so allow one bf16 ulp on rare elements
    for got, ref in ((fwd, rf), (bwd, rb)):
        assert (got.float() - ref.float()).abs().max() <= 2.0 ** -5
        assert (got == ref).float().mean() > 0.995
    assert torch.equal(bwd, rb)   # no multiplication: identical


def test_epilogue_known_answers_large_token_count(dev):
    import mok
    T = 2 * 65536
    shared = torch.full((T, 256), 1.0, device=dev, dtype=torch.bfloat16)
    routed = torch.full_like(shared, 2.0)
    w = torch.full((T, 1), 0.25, device=dev)
    assert torch.all(mok.ops.fwd_epilogue(shared, routed, w) == 1.5)
    assert torch.all(mok.ops.bwd_epilogue(shared, routed) == 3.0)


# ---------------------------------------------------------------------------------------------------------
# MXFP8 quantizer (bit-exact)
# ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(128, 128), (256, 384), (2, 128, 256), (3, 384, 128)])
def test_mxfp8_quantize_bit_exact(dev, shape):
    import mok
    g = torch.Generator().manual_seed(11)
    x = torch.randn(shape, generator=g, dtype=torch.bfloat16) * 3
    x.view(-1)[:64] = 0                       # an all-zero block and a block with a single non-zero
    x.view(-1)[40] = 448.0 * 2 ** -7          # amax / 448 exactly a power of two
    got = mok.ops.mxfp8_quantize(x.to(dev), True, True)
    ref = O.mxfp8_quantize_oracle(x, True, True)
    for name, r, q in zip(("x_fp8", "x_sc", "x_fp8_t", "x_sc_t"), ref, got):
        assert torch.equal(r.view(torch.uint8), q.cpu().view(torch.uint8)), name
    only_n = mok.ops.mxfp8_quantize(x.to(dev), True, False)
    only_t = mok.ops.mxfp8_quantize(x.to(dev), False, True)
    assert only_n[2] is None and only_n[3] is None and only_t[0] is None and only_t[1] is None
    assert torch.equal(only_n[0].view(torch.uint8), got[0].view(torch.uint8))
    assert torch.equal(only_t[3], got[3])


def test_mxfp8_quantize_golden(dev, golden_dir):
    import mok
    for tag in ("q2d", "q3d"):
        g = np.load(os.path.join(golden_dir, f"mxfp8_{tag}.npz"))
        x = torch.from_numpy(g["x"].copy()).view(torch.bfloat16)
        got = mok.ops.mxfp8_quantize(x.to(dev), True, True)
        for name, q in zip(("x_fp8", "x_sc", "x_fp8_t", "x_sc_t"), got):
            assert np.array_equal(q.cpu().view(torch.uint8).numpy(), g[name]), (tag, name)


def test_mxfp8_quantize_rejects_bad_arguments(dev):
    import mok
    x = torch.randn(128, 128, device=dev, dtype=torch.bfloat16)
    for bad in ((x.flatten(), True, True), (x[:127], True, True), (x[:, :127].contiguous(), True, True), (x, False, False)):
        with pytest.raises(ValueError):
            mok.ops.mxfp8_quantize(*bad)


# ---------------------------------------------------------------------------------------------------------
# grouped GEMM (tcgen05) through the C ABI
# ---------------------------------------------------------------------------------------------------------
def _gemm(dev, A, B, counts, N, K, b_is_kn):
    from mok import _native as nat
    rows = A.shape[0]
    D = torch.full((rows, N), float("nan"), device=dev, dtype=torch.bfloat16)
    status = nat.status_word(dev)
    if counts is None:
        tpe, nt, E = None, None, 1
    else:
        tpe = torch.tensor(counts, dtype=torch.int32, device=dev)
        nt = torch.tensor([sum(counts)], dtype=torch.int32, device=dev)
        E = len(counts)
    nat.check(nat.lib().mok_grouped_gemm_bf16(nat.ptr(A), nat.ptr(B), nat.ptr(D), nat.ptr(tpe), nat.ptr(nt), E, rows, N, K,
                                              int(b_is_kn), nat.ptr(status), nat.stream_ptr(dev)), "grouped_gemm")
    torch.cuda.synchronize()
    nat.check_status(dev)
    return D


@pytest.mark.parametrize("b_is_kn", [False, True])
@pytest.mark.parametrize("counts,N,K", [
    (None, 256, 64),                 # one tile, one K step
    (None, 256, 256),
    ([256, 512, 0, 256], 512, 320),  # uneven experts, an empty one, K not a multiple of 128
    ([1024, 256], 768, 1024),
])
def test_grouped_gemm_matches_fp32(dev, counts, N, K, b_is_kn):
    g = torch.Generator().manual_seed(3)
    rows = 256 if counts is None else sum(counts)
    E = 1 if counts is None else len(counts)
    A = (torch.randn(rows, K, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    B = (torch.randn(E, K, N, generator=g) if b_is_kn else torch.randn(E, N, K, generator=g)).mul(0.1).to(torch.bfloat16).to(dev)
    D = _gemm(dev, A, B, counts, N, K, b_is_kn)
    ref = torch.empty(rows, N, device=dev)
    off = 0
    for e, n in enumerate([rows] if counts is None else counts):
        w = B[e].float() if b_is_kn else B[e].float().T
        ref[off:off + n] = A[off:off + n].float() @ w
        off += n
    assert not torch.isnan(D.float()).any(), "unwritten output tile"
    err = _rel_l2(ref, D.float())
    assert err <= 1e-2, f"rel-L2 {err:.3e}"


@pytest.mark.parametrize("counts,M,N", [(None, 256, 256), ([256, 0, 768], 256, 512), ([512, 512], 512, 256)])
def test_grouped_wgrad_matches_fp32(dev, counts, M, N):
    from mok import _native as nat
    g = torch.Generator().manual_seed(5)
    rows = 512 if counts is None else sum(counts)
    E = 1 if counts is None else len(counts)
    A = (torch.randn(rows, M, generator=g) * 0.3).to(torch.bfloat16).to(dev)
    B = (torch.randn(rows, N, generator=g) * 0.3).to(torch.bfloat16).to(dev)
    D = torch.full((E, M, N), float("nan"), device=dev, dtype=torch.bfloat16)
    tpe = None if counts is None else torch.tensor(counts, dtype=torch.int32, device=dev)
    nt = None if counts is None else torch.tensor([rows], dtype=torch.int32, device=dev)
    nat.check(nat.lib().mok_grouped_wgrad_bf16(nat.ptr(A), nat.ptr(B), nat.ptr(D), nat.ptr(tpe), nat.ptr(nt), E, rows, M, N,
                                               nat.ptr(nat.status_word(dev)), nat.stream_ptr(dev)), "grouped_wgrad")
    torch.cuda.synchronize()
    nat.check_status(dev)
    off = 0
    for e, n in enumerate([rows] if counts is None else counts):
        if n == 0:
            assert torch.isnan(D[e].float()).all()   # empty experts are left to the zero-fill kernel
            continue
        ref = A[off:off + n].float().T @ B[off:off + n].float()
        err = _rel_l2(ref, D[e].float())
        assert err <= 1e-2, f"expert {e}: rel-L2 {err:.3e}"
        off += n
