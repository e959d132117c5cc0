"""`mok_schedule_static`: the schedule builder for hosts that may not allocate device memory when they need a
schedule (a serving process with a frozen memory pool, a plugin called under another framework's allocator lock).
Its scratch is a fixed array inside the library, so it must give exactly what `mok_schedule` gives with
caller-provided scratch — also on a second call that finds the first call's leftovers in the array — and it must
refuse sizes that do not fit the array.  This file is collected last on purpose."""
import math

import pytest
import torch


def _native():
    from mok import _native as nat
    return nat


def _call(nat, dev, topk_all, e_loc, cap, rank, static):
    ep, T, K = topk_all.shape
    i32 = dict(dtype=torch.int32, device=dev)
    outs = [torch.full((cap,), -7, **i32), torch.full((cap,), -7, **i32), torch.full((1,), -7, **i32), torch.full((e_loc,), -7, **i32)]
    status = nat.status_word(dev)
    L = nat.lib()
    if static:
        rc = L.mok_schedule_static(nat.ptr(topk_all), ep, T, K, e_loc, cap, rank, *[nat.ptr(o) for o in outs], nat.ptr(status),
                                   nat.stream_ptr(dev))
    else:
        scratch = torch.empty(L.mok_schedule_scratch_bytes(ep, T, K, e_loc) // 4, **i32)
        rc = L.mok_schedule(nat.ptr(topk_all), ep, T, K, e_loc, cap, rank, *[nat.ptr(o) for o in outs], nat.ptr(scratch),
                            nat.ptr(status), nat.stream_ptr(dev))
    torch.cuda.synchronize()
    return rc, outs


@pytest.mark.gpu
def test_static_scratch_schedule_matches_regular_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    nat = _native()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator().manual_seed(2024)
    # two different problems back to back: the second call starts from the first call's scratch contents
    for ep, E, K, T in ((4, 32, 8, 1024), (2, 6, 3, 768)):
        topk_all = torch.stack([torch.topk(torch.randn(T, E, generator=g), K, dim=1).indices for _ in range(ep)])
        topk_all = topk_all.to(torch.int32).to(dev)
        cap = T * K * max(2, math.ceil(ep * 1.5))
        for rank in (0, ep - 1):
            rc_ref, ref = _call(nat, dev, topk_all, E // ep, cap, rank, static=False)
            rc_new, new = _call(nat, dev, topk_all, E // ep, cap, rank, static=True)
            assert rc_ref == 0 and rc_new == 0
            for name, a, b in zip(("peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert"), ref, new):
                assert torch.equal(a, b), f"{name} differs (ep={ep}, rank={rank})"   # integer work: bit-exact
    nat.check_status(dev)


def test_static_scratch_schedule_rejects_sizes_beyond_its_array():
    nat = _native()
    L = nat.lib()
    # 8 ranks x 1048576 tokens x top-8 with 256 local experts needs about 16 times the fixed 4 MiB array: clearly too
    # large whatever the exact layout of the counters, so the size check is what answers (not a later pointer check).
    T = 1 << 20
    assert L.mok_schedule_scratch_bytes(8, T, 8, 256) > 8 * 4 * 1024 * 1024
    rc = L.mok_schedule_static(None, 8, T, 8, 256, 256 * (T // 256) * 8 * 4, 0, None, None, None, None, None, None)
    assert rc == -4   # MOK_ERR_TOO_LARGE, decided before anything touches the GPU
