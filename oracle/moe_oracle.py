"""CPU oracle for the expert-parallel MoE layer (TEST INFRASTRUCTURE, not product code).

This file restates, on the CPU, the arithmetic that the reference project states in its own
PyTorch test helpers and CUDA scheduler.  It exists only to check the CUDA path: the test-suite,
the smoke entry and the CPU-baseline leg of the benchmark may import it; nothing in the shipped
package does.

Parity status: PINNED.  `tests/golden/` holds outputs of the reference's own helpers
(`tests/utils.py` of the reference, executed on CPU by `tests/golden/make_golden.py`), and
`tests/test_oracle_golden.py` checks every function below against them (bit-exact for the
schedule and the MXFP8 bytes, tolerance for floating point).

All EP ranks are emulated inside one process: "rank r" is index r of the per-rank input lists.

Reference statements followed (paths inside the reference project):
  schedule ordering ........ csrc/scheduler.cuh:78-147, tests/utils.py:122-176
  MXFP8 quantizer .......... csrc/mxfp8.cuh:45-72,181-184, tests/utils.py:179-221
  SwiGLU (+clamp) .......... csrc/megakernel/swiglu.cuh:1-36,135-165, tests/utils.py:224-235
  epilogues ................ csrc/utils.cuh:43-95,140-176, tests/utils.py:299-317
  full forward / backward .. tests/utils.py:238-296,320-432
  rounding points .......... csrc/megakernel/dispatch_combine.cuh:116-124
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np
import torch

EXPERT_ROW_PADDING = 256     # csrc/scheduler.cuh:14
SCHEDULER_THREADS = 1024     # csrc/scheduler.cuh:16


# --------------------------------------------------------------------------------------------
# Schedule (integer, bit-exact)
# --------------------------------------------------------------------------------------------
def visit_order(num_routes: int, threads: int = SCHEDULER_THREADS) -> np.ndarray:
    """Route indices in the order the reference scheduler visits them.

    A block of `threads` threads walks the routes of one peer with a thread stride
    (csrc/scheduler.cuh:106-109,130): thread t owns routes t, t+threads, ...; all matches of
    thread 0 come before those of thread 1 (the scan at :110-128 is over threads).
    """
    idx = np.arange(num_routes, dtype=np.int64)
    key = (idx % threads) * (num_routes // threads + 2) + idx // threads
    return idx[np.argsort(key, kind="stable")]


def schedule_oracle(topk_all: np.ndarray, num_local_experts: int, schedule_capacity: int, rank: int):
    """Padded per-expert receive schedule of `rank` (tests/utils.py:122-176).

    topk_all: int32 [ep, T, K].  Returns (peer_rank[cap], peer_token_idx[cap], num_tokens[1],
    tokens_per_expert[E_loc]); padding rows hold -1 in both index arrays.

    Row of the j-th route that peer p sends to local expert e (csrc/scheduler.cuh:134-139):
        base_e + sum_r min(n_r, j) + #{r < p : n_r > j}
    i.e. peers are interleaved round-robin and drop out when they run dry.
    """
    topk_all = np.asarray(topk_all)
    ep, num_tokens_local, topk = topk_all.shape
    routes = num_tokens_local * topk
    flat = topk_all.reshape(ep, routes)
    order = visit_order(routes)
    first = rank * num_local_experts

    peer_rank = np.full(schedule_capacity, -1, dtype=np.int32)
    peer_token = np.full(schedule_capacity, -1, dtype=np.int32)
    per_expert = np.zeros(num_local_experts, dtype=np.int32)

    base = 0
    for e in range(num_local_experts):
        lists = [order[flat[p, order] == first + e] for p in range(ep)]
        counts = np.array([len(l) for l in lists], dtype=np.int64)
        total = int(counts.sum())
        padded = (total + EXPERT_ROW_PADDING - 1) // EXPERT_ROW_PADDING * EXPERT_ROW_PADDING
        per_expert[e] = padded
        if base + padded > schedule_capacity:
            raise ValueError("schedule_capacity too small")
        for p in range(ep):
            if counts[p] == 0:
                continue
            j = np.arange(counts[p], dtype=np.int64)
            dst = base + np.minimum(counts[None, :], j[:, None]).sum(axis=1)
            dst += (counts[None, :p] > j[:, None]).sum(axis=1)
            peer_rank[dst] = p
            peer_token[dst] = lists[p].astype(np.int32)
        base += padded
    return peer_rank, peer_token, np.array([base], dtype=np.int32), per_expert


def dedup_oracle(peer_rank: np.ndarray, peer_token_idx: np.ndarray, topk: int, num_local_tokens: int):
    """Index arrays of the de-duplicated dispatch for a finished schedule (integer, bit-exact).

    The reference has no counterpart: its dispatch pulls one row per route (csrc/megakernel/dispatch_combine.cuh:74-77).
    Definition: the distinct (source rank, token) pairs among the non-padding rows are numbered 0, 1, ... in the order
    of their first row.  Returns (row_source[cap] = number of the row's pair, -1 on padding rows; unique_peer[U];
    unique_token[U]; unique_before[cap/256 + 1] = pairs whose first row lies below row 256*i; U)."""
    peer_rank = np.asarray(peer_rank)
    cap = peer_rank.shape[0]
    valid = np.nonzero(peer_rank >= 0)[0]
    keys = peer_rank[valid].astype(np.int64) * num_local_tokens + np.asarray(peer_token_idx)[valid] // topk
    uniq, first_pos, inverse = np.unique(keys, return_index=True, return_inverse=True)
    order = np.argsort(first_pos, kind="stable")            # unique keys by first row
    number_of = np.empty(len(uniq), dtype=np.int64)
    number_of[order] = np.arange(len(uniq))
    row_source = np.full(cap, -1, dtype=np.int32)
    row_source[valid] = number_of[inverse].astype(np.int32)
    unique_peer = (uniq[order] // num_local_tokens).astype(np.int32)
    unique_token = (uniq[order] % num_local_tokens).astype(np.int32)
    first_rows = np.sort(valid[first_pos])
    unique_before = np.searchsorted(first_rows, np.arange(0, cap + 1, 256), side="left").astype(np.int32)
    return row_source, unique_peer, unique_token, unique_before, len(uniq)


# --------------------------------------------------------------------------------------------
# MXFP8 quantizer (bytes are bit-exact)
# --------------------------------------------------------------------------------------------
def mxfp8_scale_layout(scale_bytes: torch.Tensor) -> torch.Tensor:
    """[R, C/32] uint8 row-major block scales -> [R/128, C/128, 32, 16] tensor-core layout.

    Byte position inside one 128x128 tile: (r % 32) * 16 + (r // 32) * 4 + kblock
    (csrc/mxfp8.cuh:181-184; tests/utils.py:197-200).
    """
    rows, kblocks = scale_bytes.shape
    t = scale_bytes.reshape(rows // 128, 4, 32, kblocks // 4, 4)   # [rt, r//32, r%32, ct, kb]
    t = t.permute(0, 3, 2, 1, 4)                                    # [rt, ct, r%32, r//32, kb]
    return t.reshape(rows // 128, kblocks // 4, 32, 16).contiguous()


def mxfp8_quantize_rows_oracle(x_bf16: torch.Tensor):
    """Quantize along the last dim in blocks of 32 (csrc/mxfp8.cuh:45-72).

    scale exponent = ceil(log2(amax / 448)) (round-up e8m0), floor -127; element = rn_e4m3(x / 2^exp).
    Returns (fp8 tensor of x's shape, scales [E*M/128, N/128, 32, 16] uint8).
    """
    squeeze = x_bf16.ndim == 2
    x3 = x_bf16.unsqueeze(0) if squeeze else x_bf16
    e, m, n = x3.shape
    xf = x3.float().reshape(e * m, n // 32, 32)
    amax = xf.abs().amax(dim=-1)
    # The CUDA quantizer computes scale = max(amax * fp32(1/448), 1e-12) in fp32 and rounds it UP to
    # a power of two (csrc/mxfp8.cuh:57-60); the Python helper of the reference instead floors the
    # exponent at -127 (tests/utils.py:192), which differs only for all-zero blocks (byte 88 vs 0).
    # The device code is followed here.  ceil(log2(.)) is taken exactly with frexp.
    scale = torch.clamp_min(amax * torch.tensor(0.002232142857, dtype=torch.float32), 1e-12)
    mant, expo = torch.frexp(scale)                       # scale = mant * 2^expo, mant in [0.5, 1)
    ceil_log2 = torch.where(mant == 0.5, expo - 1, expo).to(torch.float32)
    ceil_log2 = ceil_log2.clamp(min=-127.0, max=127.0)
    q = (xf / torch.pow(2.0, ceil_log2).unsqueeze(-1)).to(torch.float8_e4m3fn).reshape(e, m, n)
    sc = mxfp8_scale_layout((ceil_log2 + 127.0).to(torch.uint8).reshape(e * m, n // 32))
    return (q.squeeze(0) if squeeze else q), sc


def mxfp8_quantize_oracle(x_bf16: torch.Tensor, return_normal: bool, return_transposed: bool):
    """(x_fp8, x_sc, x_fp8_t, x_sc_t) as the `mxfp8_quantize` op returns them (tests/utils.py:204-221)."""
    out = [None, None, None, None]
    if return_normal:
        out[0], out[1] = mxfp8_quantize_rows_oracle(x_bf16)
    if return_transposed:
        out[2], out[3] = mxfp8_quantize_rows_oracle(x_bf16.transpose(-2, -1).contiguous())
    return tuple(out)


def mxfp8_dequantize_oracle(x_fp8: torch.Tensor, x_sc: torch.Tensor) -> torch.Tensor:
    """Inverse of `mxfp8_quantize_rows_oracle` (fp32 result), used by the MXFP8-emulating layer oracle."""
    squeeze = x_fp8.ndim == 2
    q3 = x_fp8.unsqueeze(0) if squeeze else x_fp8
    e, m, n = q3.shape
    t = x_sc.reshape(e * m // 128, n // 128, 32, 4, 4).permute(0, 3, 2, 1, 4)  # [rt, r//32, r%32, ct, kb]
    sc = t.reshape(e * m, n // 32).float() - 127.0
    out = (q3.float().reshape(e * m, n // 32, 32) * torch.pow(2.0, sc).unsqueeze(-1)).reshape(e, m, n)
    return out.squeeze(0) if squeeze else out


# --------------------------------------------------------------------------------------------
# Elementwise pieces
# --------------------------------------------------------------------------------------------
def _bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def swiglu_oracle(gate: torch.Tensor, up: torch.Tensor, limit: float | None = None) -> torch.Tensor:
    """hidden = silu(gate) * up in fp32 from the given values; gate <= L, |up| <= L when clamped
    (csrc/megakernel/swiglu.cuh:135-165)."""
    g, u = gate.float(), up.float()
    if limit is not None:
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    return g * torch.sigmoid(g) * u


def swiglu_bwd_oracle(gate, up, d_hidden, limit: float | None = None):
    """(d_gate, d_up, hidden_fp32) following csrc/megakernel/swiglu.cuh:1-36."""
    g, u, dh = gate.float(), up.float(), d_hidden.float()
    if limit is not None:
        g_ok = g <= limit
        u_ok = (u >= -limit) & (u <= limit)
        g = g.clamp(max=limit)
        u = u.clamp(min=-limit, max=limit)
    sig = torch.sigmoid(g)
    silu = g * sig
    dsilu = (1.0 - silu) * sig + silu
    d_gate = dsilu * u * dh
    d_up = silu * dh
    if limit is not None:
        d_gate = torch.where(g_ok, d_gate, torch.zeros_like(d_gate))
        d_up = torch.where(u_ok, d_up, torch.zeros_like(d_up))
    return d_gate, d_up, silu * u


def fwd_epilogue_oracle(y_shared, combine_buffer, topk_weights):
    """out[t] = bf16(y_shared[t] + sum_k w[t,k] * combine[t*K+k]), k ascending, fp32 accumulate
    (csrc/utils.cuh:43-95)."""
    t, h = y_shared.shape
    k = topk_weights.shape[1]
    acc = y_shared.float().clone()
    routed = combine_buffer.float().view(t, k, h)
    for i in range(k):
        acc += topk_weights[:, i:i + 1].float() * routed[:, i]
    return acc.to(torch.bfloat16)


def bwd_epilogue_oracle(d_x_shared, d_x_routed_buffer):
    """d_x[t] = bf16(d_x_shared[t] + sum_k d_x_routed[t*K+k]), k ascending (csrc/utils.cuh:140-176)."""
    t, h = d_x_shared.shape
    k = d_x_routed_buffer.shape[0] // t
    acc = d_x_shared.float().clone()
    routed = d_x_routed_buffer.float().view(t, k, h)
    for i in range(k):
        acc += routed[:, i]
    return acc.to(torch.bfloat16)


# --------------------------------------------------------------------------------------------
# Whole layer, all ranks in one process
# --------------------------------------------------------------------------------------------
@dataclass
class RankInputs:
    x: torch.Tensor               # [T, H]
    topk_experts: torch.Tensor    # [T, K] integer
    router_weights: torch.Tensor  # [T, K] fp32
    w_shared_gate: torch.Tensor   # [I, H]
    w_shared_up: torch.Tensor     # [I, H]
    w_shared_down: torch.Tensor   # [H, I]
    w_routed_gate: torch.Tensor   # [E_loc, I, H]
    w_routed_up: torch.Tensor     # [E_loc, I, H]
    w_routed_down: torch.Tensor   # [E_loc, H, I]
    d_output: torch.Tensor        # [T, H]


@dataclass
class RankOutputs:
    output: torch.Tensor
    d_x: torch.Tensor
    d_router_weights: torch.Tensor
    d_w_routed_gate: torch.Tensor
    d_w_routed_up: torch.Tensor
    d_w_routed_down: torch.Tensor
    d_w_shared_gate: torch.Tensor
    d_w_shared_up: torch.Tensor
    d_w_shared_down: torch.Tensor
    combine_buffer: torch.Tensor   # [T*K, H] per-route expert outputs as they land on the source rank
    y_shared: torch.Tensor


def _ffn_fwd(x, wg, wu, wd, limit, rnd):
    gate = rnd(x @ wg.float().T)
    up = rnd(x @ wu.float().T)
    hidden = rnd(swiglu_oracle(gate, up, limit))
    y = rnd(hidden @ wd.float().T)
    return gate, up, hidden, y


def _ffn_bwd(x, gate, up, hidden, d_y, wg, wu, wd, limit, rnd):
    d_hidden = rnd(d_y @ wd.float())
    d_gate, d_up, hidden_f = swiglu_bwd_oracle(gate, up, d_hidden, limit)
    d_gate, d_up = rnd(d_gate), rnd(d_up)
    d_x = rnd(d_gate @ wg.float() + d_up @ wu.float())
    d_wd = d_y.T @ hidden
    d_wg = d_gate.T @ x
    d_wu = d_up.T @ x
    return d_x, d_wg, d_wu, d_wd, d_hidden, hidden_f


def _qdq(t: torch.Tensor) -> torch.Tensor:
    """Value after an MXFP8 round trip with blocks of 32 along the last dimension (dims padded to 128 with zeros,
    which changes no block that holds data)."""
    r, c = t.shape
    rp, cp = -(-r // 128) * 128, -(-c // 128) * 128
    buf = torch.zeros(rp, cp, dtype=torch.bfloat16)
    buf[:r, :c] = t.to(torch.bfloat16)
    q, sc = mxfp8_quantize_rows_oracle(buf)
    return mxfp8_dequantize_oracle(q, sc)[:r, :c]


def _ffn_mxfp8(x, d_y, wg, wu, wd, limit):
    """Routed expert forward + backward with MXFP8 operands, quantized where the device path quantizes
    (csrc/megakernel/forward.cuh / backward.cuh of the reference: x after dispatch, gate / up after their GEMM,
    hidden after SwiGLU, d_y*w after dispatch, d_gate / d_up after SwiGLU backward; weights and their transposes are
    quantized separately; wgrad operands are quantized along the schedule rows).  Rows of x / d_y are in schedule order."""
    wg_q, wu_q, wd_q = _qdq(wg), _qdq(wu), _qdq(wd)                   # [I,H] [I,H] [H,I], blocks along K of the forward GEMMs
    wg_t, wu_t, wd_t = _qdq(wg.T.contiguous()), _qdq(wu.T.contiguous()), _qdq(wd.T.contiguous())   # [H,I] [H,I] [I,H]
    x_q = _qdq(x)
    gate, up = _bf16(x_q @ wg_q.T), _bf16(x_q @ wu_q.T)
    hidden = _bf16(swiglu_oracle(gate, up, limit))
    y = _bf16(_qdq(hidden) @ wd_q.T)
    gate_s, up_s = _qdq(gate), _qdq(up)                              # what backward reads back
    d_hidden = _bf16(_qdq(d_y) @ wd_t.T)
    d_gate, d_up, hidden_f = swiglu_bwd_oracle(gate_s, up_s, d_hidden, limit)
    d_gate, d_up = _bf16(d_gate), _bf16(d_up)
    d_x = _bf16(_qdq(d_gate) @ wg_t.T + _qdq(d_up) @ wu_t.T)
    x_t, hid_t = _qdq(x.T.contiguous()), _qdq(hidden.T.contiguous())  # blocks of 32 along the schedule rows
    d_wd = _qdq(d_y.T.contiguous()) @ hid_t.T
    d_wg = _qdq(d_gate.T.contiguous()) @ x_t.T
    d_wu = _qdq(d_up.T.contiguous()) @ x_t.T
    d_router = (d_hidden * hidden_f).sum(-1)                          # still to be divided by the router weight
    return y, d_x, d_wg, d_wu, d_wd, d_router


def moe_layer_oracle(ranks: list[RankInputs], swiglu_limit: float | None = None,
                     round_bf16: bool = True, mxfp8: bool = False) -> list[RankOutputs]:
    """Forward + backward of the EP MoE layer for every rank (tests/utils.py:320-432).

    round_bf16=True rounds to bf16 at the points where the CUDA path stores bf16 (gate, up,
    hidden, y, d_y*w, d_hidden, d_gate, d_up, d_x_routed, weight grads, final sums);
    round_bf16=False is plain fp32 math (used for the "fp32 reference math" configuration).
    d_router_weights[t,k] = sum_h d_out[t,h] * y_routed[t,k,h]  (tests/utils.py:420).
    """
    rnd = _bf16 if round_bf16 else (lambda t: t.float())
    ep = len(ranks)
    e_loc = ranks[0].w_routed_gate.shape[0]
    t_loc, h = ranks[0].x.shape
    k = ranks[0].topk_experts.shape[1]
    out_dtype = torch.bfloat16 if round_bf16 else torch.float32

    combine = [torch.zeros(t_loc * k, h) for _ in range(ep)]
    d_x_routed = [torch.zeros(t_loc * k, h) for _ in range(ep)]
    d_rw = [torch.zeros(t_loc * k) for _ in range(ep)]
    d_wg = [torch.zeros(e_loc, *ranks[0].w_routed_gate.shape[1:]) for _ in range(ep)]
    d_wu = [torch.zeros_like(d_wg[0]) for _ in range(ep)]
    d_wd = [torch.zeros(e_loc, *ranks[0].w_routed_down.shape[1:]) for _ in range(ep)]

    if mxfp8:
        topk_all = np.stack([r.topk_experts.to(torch.int32).numpy() for r in ranks])
        cap = (t_loc * k * ep // 256 + e_loc + 1) * 256
        x_all = torch.stack([r.x.float() for r in ranks])
        dy_all = torch.stack([r.d_output.float() for r in ranks])
        w_all = torch.stack([r.router_weights.reshape(-1).float() for r in ranks])
    for owner in range(ep if mxfp8 else 0):
        pr, pt, _, tpe = schedule_oracle(topk_all, e_loc, cap, owner)
        base = 0
        for e in range(e_loc):
            rows = np.arange(base, base + int(tpe[e]))
            rows = rows[pr[rows] >= 0]                                  # schedule order, padding dropped
            base += int(tpe[e])
            src = torch.from_numpy(pr[rows].astype(np.int64))
            route = torch.from_numpy(pt[rows].astype(np.int64))
            if rows.size == 0:
                continue
            xe = x_all[src, route // k]
            w = w_all[src, route]
            dye = _bf16(dy_all[src, route // k] * w[:, None])
            y, dxe, g_wg, g_wu, g_wd, d_router = _ffn_mxfp8(xe, dye, ranks[owner].w_routed_gate[e], ranks[owner].w_routed_up[e],
                                                            ranks[owner].w_routed_down[e], swiglu_limit)
            d_wg[owner][e], d_wu[owner][e], d_wd[owner][e] = g_wg, g_wu, g_wd
            for s in range(ep):
                m = src == s
                combine[s][route[m]] = y[m]
                d_x_routed[s][route[m]] = dxe[m]
                d_rw[s][route[m]] = torch.where(w[m] > 0, d_router[m] / w[m], torch.zeros_like(w[m]))

    for owner in range(0 if mxfp8 else ep):
        for e in range(e_loc):
            ge = owner * e_loc + e
            xs, dys, where = [], [], []
            for src in range(ep):
                routes = (ranks[src].topk_experts.reshape(-1) == ge).nonzero().flatten()
                tok = routes // k
                xs.append(ranks[src].x.float()[tok])
                w = ranks[src].router_weights.reshape(-1)[routes].float()
                dys.append(rnd(ranks[src].d_output.float()[tok] * w[:, None]))   # dispatch_combine.cuh:121-122
                where.append((src, routes))
            xe, dye = torch.cat(xs), torch.cat(dys)
            wg, wu, wd = (ranks[owner].w_routed_gate[e], ranks[owner].w_routed_up[e], ranks[owner].w_routed_down[e])
            gate, up, hidden, y = _ffn_fwd(xe, wg, wu, wd, swiglu_limit, rnd)
            dxe, g_wg, g_wu, g_wd, _, _ = _ffn_bwd(xe, gate, up, hidden, dye, wg, wu, wd, swiglu_limit, rnd)
            d_wg[owner][e], d_wu[owner][e], d_wd[owner][e] = g_wg, g_wu, g_wd
            off = 0
            for src, routes in where:
                n = routes.numel()
                combine[src][routes] = y[off:off + n]
                d_x_routed[src][routes] = dxe[off:off + n]
                off += n

    results = []
    for r, inp in enumerate(ranks):
        x = inp.x.float()
        gate_s, up_s, hidden_s, y_s = _ffn_fwd(x, inp.w_shared_gate, inp.w_shared_up, inp.w_shared_down, swiglu_limit, rnd)
        d_out = inp.d_output.float()
        dxs, gsg, gsu, gsd, _, _ = _ffn_bwd(x, gate_s, up_s, hidden_s, d_out, inp.w_shared_gate, inp.w_shared_up,
                                            inp.w_shared_down, swiglu_limit, rnd)
        routed = combine[r].view(t_loc, k, h)
        w = inp.router_weights.float()
        acc = y_s.clone()
        dacc = dxs.clone()
        dxr = d_x_routed[r].view(t_loc, k, h)
        for i in range(k):
            acc += w[:, i:i + 1] * routed[:, i]
            dacc += dxr[:, i]
        d_router = d_rw[r].view(t_loc, k) if mxfp8 else (d_out[:, None, :] * routed).sum(-1)
        results.append(RankOutputs(
            output=acc.to(out_dtype), d_x=dacc.to(out_dtype), d_router_weights=d_router,
            d_w_routed_gate=d_wg[r].to(out_dtype), d_w_routed_up=d_wu[r].to(out_dtype),
            d_w_routed_down=d_wd[r].to(out_dtype),
            d_w_shared_gate=gsg.to(out_dtype), d_w_shared_up=gsu.to(out_dtype), d_w_shared_down=gsd.to(out_dtype),
            combine_buffer=combine[r].to(out_dtype), y_shared=y_s.to(out_dtype)))
    return results


# --------------------------------------------------------------------------------------------
# Seeded synthetic inputs and the comparison metric
# --------------------------------------------------------------------------------------------
def make_rank_inputs(rank: int, num_experts: int, num_local_experts: int, topk: int, num_local_tokens: int,
                     hidden: int, intermediate: int, *, seed: int = 1234, weight_std: float | None = None,
                     dtype=torch.bfloat16, expert_bias: torch.Tensor | None = None) -> RankInputs:
    """Seeded inputs drawn the way the reference tests draw them (tests/utils.py:59-106): random
    logits -> top-k -> softmax over the selected logits; x ~ N(0,1); weights ~ N(0, fan_in^-1/2)
    unless `weight_std` is given; d_output ~ N(0, 1/H).  The draw order matches the reference so the
    same seed reproduces the same tensors on CPU."""
    g = torch.Generator(device="cpu").manual_seed(seed + rank)
    logits = torch.randn(num_local_tokens, num_experts, generator=g)
    if expert_bias is not None:
        logits = logits + expert_bias
    vals, experts = torch.topk(logits, topk, dim=1)
    weights = torch.softmax(vals.float(), dim=-1)

    def rn(*shape, scale):
        return torch.randn(*shape, generator=g, dtype=dtype) * scale
    sh = weight_std if weight_std is not None else hidden ** -0.5
    si = weight_std if weight_std is not None else intermediate ** -0.5
    x = torch.randn(num_local_tokens, hidden, generator=g, dtype=dtype)
    wsg = rn(intermediate, hidden, scale=sh)
    wsu = rn(intermediate, hidden, scale=sh)
    wsd = rn(hidden, intermediate, scale=si)
    wrg = rn(num_local_experts, intermediate, hidden, scale=sh)
    wru = rn(num_local_experts, intermediate, hidden, scale=sh)
    wrd = rn(num_local_experts, hidden, intermediate, scale=si)
    d_out = rn(num_local_tokens, hidden, scale=hidden ** -0.5)
    return RankInputs(x, experts, weights, wsg, wsu, wsd, wrg, wru, wrd, d_out)


def router_oracle(x: torch.Tensor, w_router: torch.Tensor, bias: torch.Tensor | None, topk: int):
    """The router expression of the reference's tests (tests/utils.py:82-84) with a weight matrix in front of it:
    logits = x @ w_router.T (+ bias), top-k, softmax over the selected logits.  float64 throughout, so that it can judge
    near-ties.  Returns (top_experts int64 [T, k], router_weights f64 [T, k], logits f64 [T, E] without the bias)."""
    logits = x.double() @ w_router.double().t()
    biased = logits if bias is None else logits + bias.double()
    values, experts = torch.topk(biased, topk, dim=-1)
    return experts, torch.softmax(values, dim=-1), logits


def router_bwd_oracle(x: torch.Tensor, w_router: torch.Tensor, bias: torch.Tensor | None, top_experts: torch.Tensor,
                      d_router_weights: torch.Tensor):
    """Gradients of router_oracle's weights for the given routes, by autograd in float64:
    (d_x [T, H], d_w_router [E, H], d_bias [E] or None)."""
    xd = x.double().requires_grad_(True)
    wd = w_router.double().requires_grad_(True)
    bd = bias.double().requires_grad_(True) if bias is not None else None
    logits = xd @ wd.t()
    if bd is not None:
        logits = logits + bd
    weights = torch.softmax(torch.gather(logits, 1, top_experts.long()), dim=-1)
    weights.backward(d_router_weights.double())
    return xd.grad, wd.grad, (bd.grad if bd is not None else None)


def error_stats(reference: torch.Tensor, actual: torch.Tensor):
    """(max |diff|, sum|diff| / sum|ref|, rel-L2, cosine) — the reference metric is the first two
    (tests/utils.py:435-476); rel-L2 is the bound the acceptance criteria state."""
    r, a = reference.double().flatten(), actual.double().flatten()
    d = (r - a).abs()
    l1 = (d.sum() / r.abs().sum().clamp_min(1e-30)).item()
    l2 = ((r - a).norm() / r.norm().clamp_min(1e-30)).item()
    cos = (torch.dot(r, a) / (r.norm() * a.norm()).clamp_min(1e-30)).item()
    return d.max().item(), l1, l2, cos
