"""CPU checks of the de-duplicated dispatch bookkeeping: the numpy oracle's index arrays satisfy their definition on
schedules built by the schedule oracle (every row maps to its own source rank and token, tokens are numbered by first
row, the prefix counts match), and the rule that switches de-duplication on follows top-k against the EP size."""
import math
import types

import numpy as np
import torch

from oracle import moe_oracle as O


def _schedule(ep, E, K, T, rank, seed):
    g = torch.Generator().manual_seed(seed)
    topk_all = np.stack([torch.topk(torch.randn(T, E, generator=g), K, dim=1).indices.numpy().astype(np.int32) for _ in range(ep)])
    cap = T * K * max(2, math.ceil(ep * 1.5))
    pr, pt, nt, tpe = O.schedule_oracle(topk_all, E // ep, cap, rank)
    return pr, pt, int(nt[0]), cap


def test_dedup_oracle_satisfies_its_definition():
    for ep, E, K, T, rank in ((2, 16, 3, 768, 1), (4, 32, 8, 512, 0), (8, 64, 6, 512, 7), (4, 8, 1, 512, 2)):
        pr, pt, n, cap = _schedule(ep, E, K, T, rank, 40 + ep)
        row_source, unique_peer, unique_token, unique_before, u = O.dedup_oracle(pr, pt, K, T)
        valid = pr >= 0
        assert (row_source[~valid] == -1).all() and (row_source[valid] >= 0).all() and row_source.max() == u - 1
        # every row's number names the row's own (source rank, token)
        assert np.array_equal(unique_peer[row_source[valid]], pr[valid])
        assert np.array_equal(unique_token[row_source[valid]], pt[valid] // K)
        # distinct pairs, numbered in the order of their first row
        pairs = set(zip(pr[valid].tolist(), (pt[valid] // K).tolist()))
        assert len(pairs) == u == len(set(zip(unique_peer.tolist(), unique_token.tolist())))
        first_row = np.full(u, cap, dtype=np.int64)
        np.minimum.at(first_row, row_source[valid], np.nonzero(valid)[0])
        assert (np.diff(first_row) > 0).all()
        # unique_before[i] = tokens first used below row 256 * i: a prefix of the numbering
        assert unique_before[0] == 0 and unique_before[-1] == u and len(unique_before) == cap // 256 + 1
        for i in (1, len(unique_before) // 2, len(unique_before) - 1):
            assert unique_before[i] == int((first_row < 256 * i).sum())
            below = row_source[:256 * i]
            assert below.max(initial=-1) < unique_before[i]      # rows below the boundary need only that prefix
        if K == 1:
            assert u == int(valid.sum())                          # one route per token: nothing to merge
        else:
            assert u < int(valid.sum())


def test_dedup_is_switched_on_by_routes_per_rank(monkeypatch):
    import mok
    wanted = mok.functional._dedup_wanted
    monkeypatch.delenv("MOK_DEDUP", raising=False)
    ws = lambda ep, k: types.SimpleNamespace(ep_size=ep, topk=k)   # noqa: E731
    assert not wanted(ws(1, 8))                                     # one rank: every pull is local
    assert wanted(ws(2, 8)) and wanted(ws(4, 8)) and not wanted(ws(8, 8)) and not wanted(ws(4, 6)) and wanted(ws(2, 4))
    monkeypatch.setenv("MOK_DEDUP", "1")
    assert wanted(ws(8, 8)) and not wanted(ws(1, 8))
    monkeypatch.setenv("MOK_DEDUP", "0")
    assert not wanted(ws(2, 8))
