"""De-duplicated dispatch on one GPU, through the C ABI: the index arrays that number every (source rank, token) a rank
serves against the numpy oracle (integers: bit-exact), and the two-step dispatch (stage each token once, fan out
locally) against the row-by-row dispatch (copies, and one multiply per element for the weighted form: bit-exact).  The
"peers" are separate buffers of this one GPU, which is all the kernels need: they only ever dereference the addresses
they are given."""
import math

import numpy as np
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


def _routes(ep, E, K, T, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.stack([torch.topk(torch.randn(T, E, generator=g), K, dim=1).indices for _ in range(ep)]).to(torch.int32)


@pytest.mark.parametrize("ep,E,K,T", [(2, 16, 3, 768), (4, 32, 8, 1024), (8, 64, 6, 512), (8, 8, 8, 512), (4, 8, 1, 512)])
def test_dedup_index_arrays_match_oracle(dev, ep, E, K, T):
    import mok
    topk_all = _routes(ep, E, K, T, 300 + ep + E)
    cap = T * K * max(2, math.ceil(ep * 1.5))
    for rank in sorted({0, ep - 1}):
        pr, pt, nt, _ = mok.ops.schedule(topk_all.to(dev), E // ep, cap, rank)
        got = mok.ops.schedule_dedup(topk_all.to(dev), pr, pt, nt, E // ep, rank)
        torch.cuda.synchronize()
        row_source, unique_peer, unique_token, unique_before, n = O.dedup_oracle(pr.cpu().numpy(), pt.cpu().numpy(), K, T)
        assert int(got[4].item()) == n
        assert np.array_equal(got[0].cpu().numpy(), row_source), "row_source"
        assert np.array_equal(got[1].cpu().numpy()[:n], unique_peer), "unique_peer"
        assert np.array_equal(got[2].cpu().numpy()[:n], unique_token), "unique_token"
        assert np.array_equal(got[3].cpu().numpy(), unique_before), "unique_before"
        valid = int((pr >= 0).sum().item())
        assert n <= valid and (K > 1 or n == valid)      # with one route per token there is nothing to merge
    mok.ops.check_status(dev)


@pytest.mark.parametrize("weighted", [False, True])
def test_staged_dispatch_equals_row_by_row_dispatch(dev, weighted):
    import mok
    from mok import _native as nat
    ep, E, K, T, H, rank = 4, 16, 6, 512, 512, 1
    topk_all = _routes(ep, E, K, T, 77).to(dev)
    cap = T * K * 2
    pr, pt, nt, _ = mok.ops.schedule(topk_all, E // ep, cap, rank)
    row_source, unique_peer, unique_token, unique_before, num_unique = mok.ops.schedule_dedup(topk_all, pr, pt, nt, E // ep, rank)
    g = torch.Generator(device=dev).manual_seed(5)
    xs = [torch.randn(T, H, generator=g, device=dev, dtype=torch.bfloat16) for _ in range(ep)]
    ws = [torch.rand(T, K, generator=g, device=dev) + 0.1 for _ in range(ep)]
    x_ptrs = nat.ptr_array([int(t.data_ptr()) for t in xs])
    w_ptrs = nat.ptr_array([int(t.data_ptr()) for t in ws]) if weighted else None
    L, st, stream = nat.lib(), nat.status_word(dev), nat.stream_ptr(dev)
    n = int(nt.item())

    ref = torch.full((cap, H), float("nan"), device=dev, dtype=torch.bfloat16)
    ref_w = torch.full((cap,), float("nan"), device=dev)
    nat.check(L.mok_dispatch_rows(x_ptrs, w_ptrs, ep, nat.ptr(pr), nat.ptr(pt), nat.ptr(nt), 0, cap, K, T, H, nat.ptr(ref),
                                  nat.ptr(ref_w) if weighted else None, 0, nat.ptr(st), stream), "dispatch_rows")

    staged_rows = unique_peer.numel()
    staged = torch.full((staged_rows, H), float("nan"), device=dev, dtype=torch.bfloat16)   # NaN: an unstaged read shows
    got = torch.full((cap, H), float("nan"), device=dev, dtype=torch.bfloat16)
    got_w = torch.full((cap,), float("nan"), device=dev)
    edges = [0, 1024, 2560, cap]          # three chunks, as the layer hands them over
    for lo, hi in zip(edges[:-1], edges[1:]):
        nat.check(L.mok_stage_unique_rows(x_ptrs, ep, rank, nat.ptr(unique_peer), nat.ptr(unique_token), nat.ptr(unique_before),
                                          nat.ptr(nt), lo, hi, T, H, nat.ptr(staged), staged_rows, 0, nat.ptr(st), stream),
                  "stage_unique_rows")
        nat.check(L.mok_dispatch_rows_staged(x_ptrs, w_ptrs, ep, rank, nat.ptr(pr), nat.ptr(pt), nat.ptr(nt), nat.ptr(row_source),
                                             nat.ptr(staged), staged_rows, lo, hi, K, T, H,
                                             nat.ptr(got[lo:]), nat.ptr(got_w[lo:]) if weighted else None, 0, nat.ptr(st), stream),
                  "dispatch_rows_staged")
    torch.cuda.synchronize()
    nat.check_status(dev)
    assert torch.equal(ref[:n].view(torch.int16), got[:n].view(torch.int16))
    if weighted:
        assert torch.equal(ref_w[:n], got_w[:n])
    # every other rank's token crossed once: the staged rows of remote tokens are exactly the distinct remote tokens
    u = int(num_unique.item())
    remote = unique_peer[:u] != rank
    assert not torch.isnan(staged[:u][remote].float()).any()
    assert torch.isnan(staged[:u][~remote].float()).all()          # this rank's own tokens are read in place, never staged
    remote_rows = int(((pr[:n] >= 0) & (pr[:n] != rank)).sum().item())
    assert int(remote.sum().item()) < remote_rows                   # fewer pulls than rows: the point of the exercise
