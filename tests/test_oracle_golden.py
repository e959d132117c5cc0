"""Pins the CPU oracle against fixtures produced by the reference project's own helpers
(`tests/golden/make_golden.py`): bit-exact for integer/byte work, tolerance for floating point."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import moe_oracle as O


def _bf16(a):
    return torch.from_numpy(a.copy()).view(torch.bfloat16) if a.dtype == np.uint16 else torch.from_numpy(a.copy())


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "sched_*.npz"))))
def test_schedule_matches_reference(path):
    g = np.load(path)
    e_loc, cap, rank = (int(v) for v in g["meta"])
    pr, pt, nt, tpe = O.schedule_oracle(g["topk_all"], e_loc, cap, rank)
    assert np.array_equal(pr, g["peer_rank"])
    assert np.array_equal(pt, g["peer_token_idx"])
    assert np.array_equal(nt, g["num_tokens"])
    assert np.array_equal(tpe, g["tokens_per_expert"])


@pytest.mark.parametrize("tag", ["q2d", "q3d"])
def test_mxfp8_bytes_match_reference(golden_dir, tag):
    g = np.load(os.path.join(golden_dir, f"mxfp8_{tag}.npz"))
    x = _bf16(g["x"])
    q = O.mxfp8_quantize_oracle(x, True, True)
    assert np.array_equal(q[0].view(torch.uint8).numpy(), g["x_fp8"])
    assert np.array_equal(q[1].numpy(), g["x_sc"])
    assert np.array_equal(q[2].view(torch.uint8).numpy(), g["x_fp8_t"])
    assert np.array_equal(q[3].numpy(), g["x_sc_t"])
    # round trip: dequantize(quantize(x)) is within one e4m3 step (2^-3 relative) of x
    back = O.mxfp8_dequantize_oracle(q[0], q[1])
    blockmax = x.float().reshape(-1, 32).abs().amax(-1, keepdim=True)
    assert ((back.reshape(-1, 32) - x.float().reshape(-1, 32)).abs() <= blockmax * 2.0 ** -3).all()


def test_mxfp8_zero_block_follows_device_code():
    x = torch.zeros(128, 128, dtype=torch.bfloat16)
    q, sc = O.mxfp8_quantize_rows_oracle(x)
    assert int(sc.max()) == int(sc.min()) == 88   # 2^-39 = round-up of 1e-12 (csrc/mxfp8.cuh:57)
    assert (q.view(torch.uint8) == 0).all()


def test_swiglu_matches_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "swiglu.npz"))
    gate, up = _bf16(g["gate"]), _bf16(g["up"])
    plain = O.swiglu_oracle(gate, up).to(torch.bfloat16)
    clamp = O.swiglu_oracle(gate, up, 4.0).to(torch.bfloat16)
    # the reference's unclamped form multiplies two bf16 tensors (double rounding): allow 1 bf16 ulp
    ref_plain, ref_clamp = _bf16(g["plain"]).float(), _bf16(g["clamp"]).float()
    assert ((plain.float() - ref_plain).abs() <= ref_plain.abs() * 2.0 ** -7 + 1e-30).all()
    assert torch.equal(clamp.float(), ref_clamp)


def test_epilogues_match_reference(golden_dir):
    g = np.load(os.path.join(golden_dir, "epilogues.npz"))
    ys, cb, w = _bf16(g["y_shared"]), _bf16(g["combine"]), torch.from_numpy(g["w"])
    fwd = O.fwd_epilogue_oracle(ys, cb, w)
    bwd = O.bwd_epilogue_oracle(ys, cb)
    # the reference sums over k with a tensor reduction; order may differ by one fp32 rounding
    assert (fwd.float() - _bf16(g["fwd"]).float()).abs().max() <= 2.0 ** -6
    assert (bwd.float() - _bf16(g["bwd"]).float()).abs().max() <= 2.0 ** -5
    assert (fwd == _bf16(g["fwd"])).float().mean() > 0.99
    assert (bwd == _bf16(g["bwd"])).float().mean() > 0.99


def test_epilogue_known_answers():
    # closed-form cases of the reference tests (tests/test_misc.py:1937-1955)
    shared = torch.full((512, 256), 1.0, dtype=torch.bfloat16)
    routed = torch.full_like(shared, 2.0)
    w = torch.full((512, 1), 0.25)
    assert torch.all(O.fwd_epilogue_oracle(shared, routed, w) == 1.5)
    assert torch.all(O.bwd_epilogue_oracle(shared, routed) == 3.0)


def _layer_case(golden_dir, name, ws, limit_tag):
    blobs = [np.load(os.path.join(golden_dir, f"layer_{name}_ws{ws}_r{r}_{limit_tag}.npz")) for r in range(ws)]
    E, H, I, K, T, _, _ = (int(v) for v in blobs[0]["shape"])
    limit = float(blobs[0]["limit"][0])
    limit = None if limit < 0 else limit
    ranks = [O.make_rank_inputs(r, E, E // ws, K, T, H, I) for r in range(ws)]
    for r, b in enumerate(blobs):   # the re-drawn inputs are the tensors the reference saw
        i = ranks[r]
        sums = [float(t.double().abs().sum()) for t in (i.x, i.topk_experts, i.router_weights, i.w_shared_gate,
                i.w_shared_up, i.w_shared_down, i.w_routed_gate, i.w_routed_up, i.w_routed_down, i.d_output)]
        assert np.allclose(sums, b["input_checksums"], rtol=0, atol=0)
    return blobs, ranks, limit


@pytest.mark.parametrize("name", ["tiny", "small"])
@pytest.mark.parametrize("ws", [1, 2])
@pytest.mark.parametrize("limit_tag", ["plain", "clamp"])
def test_layer_matches_reference(golden_dir, name, ws, limit_tag):
    blobs, ranks, limit = _layer_case(golden_dir, name, ws, limit_tag)
    outs = O.moe_layer_oracle(ranks, swiglu_limit=limit)
    for r in range(ws):
        for field in ("output", "d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
                      "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down", "combine_buffer", "y_shared"):
            ref = _bf16(blobs[r][field]).float()
            got = getattr(outs[r], field).float()
            mx, l1, l2, cos = O.error_stats(ref, got)
            # bf16 tolerance of the reference tests (tests/utils.py:7) and the rel-L2 <= 1e-2 acceptance bound
            assert mx <= 0.5 and l1 <= 0.01 and l2 <= 0.01 and cos >= 0.9999, (field, mx, l1, l2, cos)
