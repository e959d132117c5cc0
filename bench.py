"""Benchmark of the expert-parallel MoE layer, forward + backward (tokens/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c4|c0|tiny]
                    [--dtype bf16|mxfp8] [--minibatch ROWS] [--macrobatch ROWS] [--single]

One step = build_schedule + forward + backward of one MoE layer over one batch of synthetic tokens through
`mok.functional`.  The default workload is the DeepSeek-V3-shaped layer (32768 tokens per rank, hidden 7168,
256 routed experts of intermediate 2048 sharded over the N ranks, top-8, one shared expert).  Rank 0 prints one
JSON line.  Under torchrun (N > 1) every rank runs one GPU; times are the maximum over ranks.

The line describes the BF16 step (`--dtype mxfp8`: the MXFP8 step) and carries, in the same run:
  * `parity`  — a sampled check of the full-size step against the CPU oracle, outside the timed region: rank 0's
                schedule bit for bit, a few tokens' output / d_x / d_router_weights rows recomputed from the experts
                they use, and the three weight gradients of one or two experts recomputed from their rows;
  * `mxfp8`   — the same step with the routed experts in MXFP8 (`bf16` when `--dtype mxfp8`), timed, with its own
                GEMM-form timings, end-to-end figure and parity sample (`--single` leaves it out);
  * `ring`    — the step at the reference's default macrobatch size (131072 rows), where backward replays the gate / up
                projections of the later windows; the headline sizes the ring buffers to hold every row in one window;
  * `roofline`, `cpu_baseline`, `e2e`, `clocks`, `comm`, `phases`.

`--impl reference` times the CPU restatement of the reference math (oracle/) on the host cores, on a bounded
sample of the same layer shape; that leg never touches the GPU library.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
import types

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

WORKLOADS = {
    # name: tokens/rank, hidden, experts (global), intermediate, topk, weight std, expert bias std, Zipf exponent of the
    # expert bias (0 = none), schedule_capacity_multiplier (None = library default), default macrobatch (None = one window)
    "c2": dict(T=32768, H=7168, E=256, I=2048, K=8, std=0.006, bias=0.0, zipf=0.0, cap_mult=None, macrobatch=None,
               label="deepseek-v3-shaped bf16"),
    # the benchmark's row shapes on a few GB of device memory: the case profiler captures of the bandwidth kernels use
    "c2s": dict(T=4096, H=7168, E=16, I=2048, K=8, std=0.006, bias=0.0, zipf=0.0, cap_mult=None, macrobatch=None,
                label="deepseek-v3-shaped bf16, 16 experts"),
    "c1": dict(T=16384, H=2048, E=128, I=768, K=8, std=0.02, bias=0.5, zipf=0.0, cap_mult=None, macrobatch=None,
               label="qwen3-moe-shaped bf16"),
    # imbalanced-routing stress: 8 experts, a Zipf(1.2) expert bias calibrated so that the busiest expert (= the busiest
    # rank at EP 8) takes about 45 % of the routes; capacity multiplier 1.0; the reference's default macrobatch
    "c4": dict(T=16384, H=4096, E=8, I=14336, K=2, std=0.02, bias=0.0, zipf=1.2, cap_mult=1.0, macrobatch=131072,
               label="mixtral-shaped bf16, zipf(1.2) routing"),
    "c0": dict(T=2048, H=512, E=8, I=1024, K=2, std=0.02, bias=0.0, zipf=0.0, cap_mult=None, macrobatch=None,
               label="cpu-plumbing shape"),
    "tiny": dict(T=512, H=256, E=8, I=256, K=2, std=0.02, bias=0.0, zipf=0.0, cap_mult=None, macrobatch=None, label="tiny"),
}
REFERENCE_DEFAULT_MACROBATCH = 131072      # mok/functional.py:24-31 of the reference
NVLINK_PEER_COPY_GBS = 770.0               # measured peer copy on this pool, per direction and GPU (900 nominal)


def flops_per_token(w) -> float:
    """Algorithmic FLOPs of forward + backward per token: 18*K*H*I for the routed experts (3 GEMMs forward, 6
    backward, 2*H*I each) plus 18*H*I for the shared expert.  Padding rows and replayed GEMMs are not counted."""
    return 18.0 * (w["K"] + 1) * w["H"] * w["I"]


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(burst=float(p["bf16_tflops"]), sustained=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    hbm=float(p["hbm_gbs"]), source="measured")
    return dict(burst=1590.0, sustained=1400.0, hbm=6650.0, source="fallback")


def host_threads() -> int:
    """Host cores this process may use.  torchrun exports OMP_NUM_THREADS=1 to its workers; the CPU legs set the
    thread count from the affinity mask instead, so that they use the cores the single-process run uses."""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.time(), [c.strip() for c in line.split(",")]))

    def window(self, t_begin: float, t_end: float):
        """Summary of the samples that arrived inside [t_begin, t_end] (wall clock)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        clocks, reasons, mx = [], set(), None
        inside = [s for t, s in self.samples if t_begin <= t <= t_end + 0.2]
        for s in inside or [s for _, s in self.samples[-2:]]:
            try:
                clocks.append(float(s[0]))
                mx = float(s[1])
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference math, timed on the host cores
# ------------------------------------------------------------------------------------------------------------
def cpu_sample(w, tokens: int, experts: int, steps: int, warmup: int):
    """Times fwd+bwd of a bounded sample: `tokens` tokens, `experts` experts, same H / I / K as the workload."""
    import torch
    from oracle import moe_oracle as O
    torch.set_num_threads(host_threads())
    inp = O.make_rank_inputs(0, experts, experts, min(w["K"], experts), tokens, w["H"], w["I"], seed=0, weight_std=w["std"])
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        O.moe_layer_oracle([inp])
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return tokens / sec, sec, torch.get_num_threads()


def cpu_sample_size(w):
    # about 2e11..6e11 FLOP per pass: seconds on a few host cores
    budget = 4e11
    tokens = int(max(64, min(2048, budget / flops_per_token(w))))
    tokens = max(64, tokens // 64 * 64)
    return tokens, min(w["E"], 8)


def cpu_sample_text(w, tokens, experts):
    return (f"{tokens} tokens, {experts} experts, H={w['H']} I={w['I']} top-{min(w['K'], experts)}, "
            "fp32 math with bf16 rounding points (CPU oracle)")


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tokens, experts = cpu_sample_size(w)
    tps, sec, cores = cpu_sample(w, tokens, experts, max(1, args.steps), min(args.warmup, 1))
    sample = cpu_sample_text(w, tokens, experts)
    line = {
        "impl": "reference", "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # what this arm timed: a bounded sample of the layer shape (same hidden / intermediate / top-k) on the host
        # cores of one process; `gpu_arm_workload` names the full-size configuration the GPU arm runs
        "config": {"workload": f"{w['label']}: bounded CPU sample ({tokens} tokens, {experts} experts)",
                   "tokens_per_rank": tokens, "hidden": w["H"], "experts": experts, "intermediate": w["I"],
                   "topk": min(w["K"], experts), "shared_expert": True, "ranks": 1, "host_threads": cores,
                   "gpu_arm_workload": {"tokens_per_rank": w["T"], "experts": w["E"], "topk": w["K"]}},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# GPU arm: inputs
# ------------------------------------------------------------------------------------------------------------
def router_parameters(w, dev):
    """Router matrix [H, E] and per-expert bias, the same on every rank.  With `zipf` > 0 the bias is c * log p_e with
    p_e proportional to e^-zipf (e = 1..E) and c calibrated on a seeded sample of tokens so that the busiest expert
    receives 45 % of the routes."""
    import torch
    gw = torch.Generator(device=dev).manual_seed(12345)
    H, E, K = w["H"], w["E"], w["K"]
    w_r = torch.randn(H, E, generator=gw, device=dev) * w["std"]
    bias = torch.zeros(E, device=dev)
    if w["bias"] > 0:
        bias = torch.randn(E, generator=gw, device=dev) * w["bias"]
    if w["zipf"] > 0:
        logp = -w["zipf"] * torch.log(torch.arange(1, E + 1, device=dev, dtype=torch.float32))
        logp = logp - torch.logsumexp(logp, 0)
        sample = torch.randn(8192, H, generator=torch.Generator(device=dev).manual_seed(999), device=dev, dtype=torch.bfloat16)
        logits = sample.float() @ w_r

        def share(c):
            top = torch.topk(logits + c * logp, K, dim=1).indices
            return (torch.bincount(top.flatten(), minlength=E).max().float() / top.numel()).item()
        lo, hi = 0.0, 64.0
        for _ in range(40):
            mid = 0.5 * (lo + hi)
            lo, hi = (mid, hi) if share(mid) < 0.45 else (lo, mid)
        bias = bias + 0.5 * (lo + hi) * logp
    return w_r, bias


def make_activations(w, rank: int, dev, router):
    """Seeded tokens of one rank: x, dy ~ N(0,1); logits = x W_r + bias; top-k routing with softmax over the selected
    logits (renormalised weights).  Any rank can redraw any other rank's tokens from the seed."""
    import torch
    g = torch.Generator(device=dev).manual_seed(0 + rank)
    T, H, K = w["T"], w["H"], w["K"]
    x = torch.randn(T, H, generator=g, device=dev, dtype=torch.bfloat16)
    dy = torch.randn(T, H, generator=g, device=dev, dtype=torch.bfloat16)
    w_r, bias = router
    vals, topk = torch.topk(x.float() @ w_r + bias, K, dim=1)
    return x, dy, topk.contiguous(), torch.softmax(vals, dim=-1).contiguous()


def make_weights(w, e_loc: int, rank: int, dev):
    """Seeded weights of one rank ~ N(0, std): shared gate / up / down, routed gate / up / down of its experts."""
    import torch
    g = torch.Generator(device=dev).manual_seed(1000 + rank)
    H, I = w["H"], w["I"]

    def wt(*shape):
        return torch.randn(*shape, generator=g, device=dev, dtype=torch.bfloat16).mul_(w["std"])
    return (wt(I, H), wt(I, H), wt(H, I), wt(e_loc, I, H), wt(e_loc, I, H), wt(e_loc, H, I))


# ------------------------------------------------------------------------------------------------------------
# GPU arm: single launches of the dominant kernels
# ------------------------------------------------------------------------------------------------------------
def _time_forms(named_fns, reps=5):
    """Average duration of single launches of each form, timed with one CUDA-event pair per launch and the forms taken
    in turn (a, b, c, a, b, c, ...): under the power cap the SM clock sinks within milliseconds of sustained load, so
    forms timed one after the other in blocks would be measured at different clocks; in turn they share the same state."""
    import torch
    from mok import _native as nat
    for name, fn in named_fns:
        for _ in range(2):
            nat.check(fn(), name)
    events = {name: [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(reps)]
              for name, _ in named_fns}
    torch.cuda.synchronize()
    for i in range(reps):
        for name, fn in named_fns:
            events[name][i][0].record()
            fn()
            events[name][i][1].record()
    torch.cuda.synchronize()
    return {name: sum(a.elapsed_time(b) for a, b in events[name]) / reps for name, _ in named_fns}


def time_gemm_forms(dev, w, e_loc, sched, weights, rows_buf):
    """Times single launches of the dominant kernel (tcgen05 grouped GEMM) on the layer's own shapes."""
    import torch
    from mok import _native as nat
    H, I = w["H"], w["I"]
    valid_rows = int((sched.peer_rank >= 0).sum().item())
    padded_rows = int(sched.num_tokens.item())
    rows_buf = min(rows_buf, (padded_rows + 255) // 256 * 256)
    a_h = torch.randn(rows_buf, H, device=dev, dtype=torch.bfloat16)
    a_i = torch.randn(rows_buf, I, device=dev, dtype=torch.bfloat16)
    d_i = torch.empty(rows_buf, I, device=dev, dtype=torch.bfloat16)
    d_w = torch.empty(e_loc, I, H, device=dev, dtype=torch.bfloat16)
    st = nat.status_word(dev)
    L = nat.lib()
    tpe, nt = nat.ptr(sched.tokens_per_expert), nat.ptr(sched.num_tokens)

    def fwd():
        return L.mok_grouped_gemm_bf16(nat.ptr(a_h), nat.ptr(weights[3]), nat.ptr(d_i), tpe, nt, e_loc, rows_buf, I, H, 0,
                                       nat.ptr(st), nat.stream_ptr(dev))

    def dgrad():
        return L.mok_grouped_gemm_bf16(nat.ptr(a_h), nat.ptr(weights[5]), nat.ptr(d_i), tpe, nt, e_loc, rows_buf, I, H, 1,
                                       nat.ptr(st), nat.stream_ptr(dev))

    def wgrad():
        return L.mok_grouped_wgrad_bf16(nat.ptr(a_i), nat.ptr(a_h), nat.ptr(d_w), tpe, nt, e_loc, rows_buf, I, H,
                                        nat.ptr(st), nat.stream_ptr(dev))
    out = {}
    rows_done = min(valid_rows, rows_buf)
    for name, ms in _time_forms((("fwd_gate", fwd), ("dgrad_down", dgrad), ("wgrad_gate", wgrad))).items():
        out[name] = {"ms": ms, "tflops": 2.0 * rows_done * H * I / (ms * 1e-3) / 1e12}
    nat.check_status(dev)
    return out, rows_done


def time_gemm_forms_mxfp8(dev, w, e_loc, sched, qg, rows_buf):
    """Single launches of the block-scaled MXFP8 GEMM on the layer's shapes (forward gate form, wgrad gate form)."""
    import torch
    import mok
    from mok import _native as nat
    H, I = w["H"], w["I"]
    valid_rows = int((sched.peer_rank >= 0).sum().item())
    padded_rows = int(sched.num_tokens.item())
    rows_buf = min(rows_buf, (padded_rows + 255) // 256 * 256)
    a = torch.randn(rows_buf, H, device=dev, dtype=torch.bfloat16)
    a_q, a_sc, a_t, a_t_sc = mok.ops.mxfp8_quantize(a, True, True)
    g = torch.randn(rows_buf, I, device=dev, dtype=torch.bfloat16)
    _, _, g_t, g_t_sc = mok.ops.mxfp8_quantize(g, False, True)
    del a, g
    d_i = torch.empty(rows_buf, I, device=dev, dtype=torch.bfloat16)
    d_w = torch.empty(e_loc, I, H, device=dev, dtype=torch.bfloat16)
    st = nat.status_word(dev)
    L = nat.lib()
    tpe, nt = nat.ptr(sched.tokens_per_expert), nat.ptr(sched.num_tokens)

    def fwd():
        return L.mok_grouped_gemm_mxfp8(nat.ptr(a_q), nat.ptr(a_sc), nat.ptr(qg[0]), nat.ptr(qg[1]), nat.ptr(d_i), tpe, nt, e_loc,
                                        rows_buf, I, H, nat.ptr(st), nat.stream_ptr(dev))

    def wgrad():
        return L.mok_grouped_wgrad_mxfp8(nat.ptr(g_t), nat.ptr(g_t_sc), nat.ptr(a_t), nat.ptr(a_t_sc), nat.ptr(d_w), tpe, nt, e_loc,
                                         rows_buf, I, H, nat.ptr(st), nat.stream_ptr(dev))
    out = {}
    rows_done = min(valid_rows, rows_buf)
    for name, ms in _time_forms((("fwd_gate", fwd), ("wgrad_gate", wgrad))).items():
        out[name] = {"ms": ms, "tflops": 2.0 * rows_done * H * I / (ms * 1e-3) / 1e12}
    nat.check_status(dev)
    return out, rows_done


def time_comm_kernels(dev, w, ws, sched, rows_buf, world, num_comm_ctas):
    """Dispatch (pull rows from the owning ranks) and combine (push rows into the owners' slot buffers) alone, timed
    with CUDA events while every rank does the same: GB/s of payload per rank and direction."""
    import torch
    import torch.distributed as dist
    from mok import _native as nat
    H, K, T = w["H"], w["K"], w["T"]
    valid_rows = int((sched.peer_rank >= 0).sum().item())
    padded_rows = int(sched.num_tokens.item())
    rows_buf = min(rows_buf, (padded_rows + 255) // 256 * 256)
    buf = torch.empty(rows_buf, H, device=dev, dtype=torch.bfloat16)
    L = nat.lib()
    st = nat.status_word(dev)
    xp, cp = nat.ptr_array(ws.x_buffer_ptrs), nat.ptr_array(ws.combine_buffer_ptrs)
    common = (nat.ptr(sched.peer_rank), nat.ptr(sched.peer_token_idx), nat.ptr(sched.num_tokens), 0, rows_buf, K, T, H)

    def dispatch(ctas):
        return L.mok_dispatch_rows(xp, None, world, *common, nat.ptr(buf), None, ctas, nat.ptr(st), nat.stream_ptr(dev))

    def combine(ctas):
        return L.mok_combine_rows(cp, None, world, *common, nat.ptr(buf), None, ctas, nat.ptr(st), nat.stream_ptr(dev))
    out = {}
    rows_done = min(valid_rows, rows_buf)
    for name, fn, ctas in (("dispatch_full_grid", dispatch, 0), ("combine_full_grid", combine, 0),
                           ("dispatch_comm_ctas", dispatch, num_comm_ctas), ("combine_comm_ctas", combine, num_comm_ctas)):
        nat.check(fn(ctas), name)
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            fn(ctas)
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / 3], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        gbs = rows_done * H * 2 / (ms.item() * 1e-3) / 1e9
        out[name] = {"ms": ms.item(), "payload_gbs": gbs, "nvlink_gbs": gbs * (world - 1) / world}
    dist.barrier()
    nat.check_status(dev)
    return out


# ------------------------------------------------------------------------------------------------------------
# GPU arm: sampled parity of the full-size step against the CPU oracle (outside the timed region)
# ------------------------------------------------------------------------------------------------------------
def sampled_parity(case, mxfp8: bool, sched, out, grads, n_tokens: int, max_expert_rows: int = 9000):
    """Rank 0 only.  Checks of the step that was just computed on the GPU:
      schedule   rank 0's schedule against the oracle's scheduler on the routes of all ranks, bit for bit;
      tokens     for `n_tokens` tokens of rank 0: output, d_x and d_router_weights rows recomputed on the CPU from the
                 token, its K experts' weights (other ranks' experts are redrawn from their seeds) and the shared expert;
      experts    for the first and the last local expert of rank 0 (as far as their rows number at most `max_expert_rows`
                 together): the three weight gradients recomputed on the CPU from the expert's rows in schedule order.
    BF16 compares with the oracle's bf16-rounding math at rel-L2 <= 1e-2; MXFP8 with the oracle that quantizes at the
    same points at rel-L2 <= 3e-2."""
    import numpy as np
    import torch
    from oracle import moe_oracle as O
    torch.set_num_threads(host_threads())
    w, dev, world, e_loc = case.w, case.dev, case.world, case.e_loc
    T, H, I, K = w["T"], w["H"], w["I"], w["K"]
    tol = 3e-2 if mxfp8 else 1e-2
    t_start = time.time()

    pr = sched.peer_rank.cpu().numpy()
    pt = sched.peer_token_idx.cpu().numpy()
    tpe = sched.tokens_per_expert.cpu().numpy()
    cum = np.concatenate([[0], np.cumsum(tpe)])
    # the first and the last local expert, as far as their rows stay within what the CPU recomputes in seconds
    experts, budget = [], max_expert_rows
    for e in ([0] if e_loc == 1 else [0, e_loc - 1]):
        if int(tpe[e]) <= budget:
            experts.append(e)
            budget -= int(tpe[e])
    expert_rows = {}
    for e in experts:
        rows = np.arange(cum[e], cum[e + 1])
        rows = rows[pr[rows] >= 0]
        expert_rows[e] = dict(src=pr[rows].astype(np.int64), route=pt[rows].astype(np.int64),
                              x=torch.empty(len(rows), H), dy=torch.empty(len(rows), H), w=torch.empty(len(rows)))

    # redraw every rank's tokens once: routes for the schedule check, rows for the expert checks
    topk_all = np.empty((world, T, K), dtype=np.int32)
    for r in range(world):
        x_r, dy_r, topk_r, rw_r = (case.x, case.dy, case.topk, case.rw) if r == 0 else make_activations(w, r, dev, case.router)
        topk_all[r] = topk_r.to(torch.int32).cpu().numpy()
        for e, rec in expert_rows.items():
            sel = np.nonzero(rec["src"] == r)[0]
            if sel.size == 0:
                continue
            route = torch.from_numpy(rec["route"][sel]).to(dev)
            rec["x"][sel] = x_r[route // K].float().cpu()
            rec["dy"][sel] = dy_r[route // K].float().cpu()
            rec["w"][sel] = rw_r.reshape(-1)[route].cpu()
        del x_r, dy_r, topk_r, rw_r
    ref_pr, ref_pt, ref_nt, ref_tpe = O.schedule_oracle(topk_all, e_loc, case.capacity, 0)
    valid = ref_pr >= 0
    schedule_exact = bool(np.array_equal(pr, ref_pr) and np.array_equal(pt[valid], ref_pt[valid])
                          and int(sched.num_tokens.item()) == int(ref_nt[0]) and np.array_equal(tpe, ref_tpe))

    def rel_l2(ref, got):
        ref, got = ref.double().flatten(), got.double().flatten()
        return ((ref - got).norm() / ref.norm().clamp_min(1e-30)).item()

    errors = {}
    # ---- experts: weight gradients from the expert's rows --------------------------------------------------------
    def rank_weights(owner):   # rank 0's own unless they were dropped for the measurement; other ranks' from their seed
        return case.weights if (owner == 0 and case.weights[3] is not None) else make_weights(w, e_loc, owner, dev)

    local_wts = rank_weights(0)
    local_expert_weights = {e: tuple(local_wts[i][e].cpu() for i in (3, 4, 5)) for e in expert_rows}
    for e, rec in expert_rows.items():
        if rec["x"].shape[0] == 0:
            continue
        wg, wu, wd = local_expert_weights[e]
        dye = O._bf16(rec["dy"] * rec["w"][:, None])
        if mxfp8:
            _, _, g_wg, g_wu, g_wd, _ = O._ffn_mxfp8(rec["x"], dye, wg, wu, wd, None)
        else:
            gate, up, hidden, _ = O._ffn_fwd(rec["x"], wg, wu, wd, None, O._bf16)
            _, g_wg, g_wu, g_wd, _, _ = O._ffn_bwd(rec["x"], gate, up, hidden, dye, wg, wu, wd, None, O._bf16)
        for name, ref, got in (("d_w_routed_gate", g_wg, grads[2][e]), ("d_w_routed_up", g_wu, grads[3][e]),
                               ("d_w_routed_down", g_wd, grads[4][e])):
            errors[name] = max(errors.get(name, 0.0), rel_l2(ref, got.float().cpu()))

    # ---- tokens: output, d_x, d_router_weights rows --------------------------------------------------------------
    tokens = sorted({(i * (T - 1)) // max(1, n_tokens - 1) for i in range(n_tokens)}) if n_tokens > 1 else [0]
    topk0 = case.topk.cpu()
    needed = {}                                    # owner rank -> sorted local expert ids the sampled tokens use
    for t in tokens:
        for ge in topk0[t].tolist():
            needed.setdefault(ge // e_loc, set()).add(ge % e_loc)
    expert_weights = {}
    for owner, local in sorted(needed.items()):
        wts = local_wts if owner == 0 else rank_weights(owner)
        for le in sorted(local):
            expert_weights[owner * e_loc + le] = tuple(wts[i][le].cpu() for i in (3, 4, 5))
        del wts
    del local_wts
    wsg, wsu, wsd = (case.weights[i].cpu() for i in (0, 1, 2))
    ref_out, ref_dx, ref_drw = [], [], []
    for t in tokens:
        xs = case.x[t].float().cpu()[None]
        d_out = case.dy[t].float().cpu()[None]
        rw_t = case.rw[t].cpu()
        gate_s, up_s, hidden_s, y_s = O._ffn_fwd(xs, wsg, wsu, wsd, None, O._bf16)
        dxs = O._ffn_bwd(xs, gate_s, up_s, hidden_s, d_out, wsg, wsu, wsd, None, O._bf16)[0]
        acc, dacc, drw = y_s.clone(), dxs.clone(), torch.zeros(K)
        for k, ge in enumerate(topk0[t].tolist()):
            wg, wu, wd = expert_weights[ge]
            dye = O._bf16(d_out * rw_t[k])
            if mxfp8:
                y, dxe, _, _, _, d_router = O._ffn_mxfp8(xs, dye, wg, wu, wd, None)
                drw[k] = (d_router[0] / rw_t[k]) if rw_t[k] > 0 else 0.0
            else:
                gate, up, hidden, y = O._ffn_fwd(xs, wg, wu, wd, None, O._bf16)
                dxe = O._ffn_bwd(xs, gate, up, hidden, dye, wg, wu, wd, None, O._bf16)[0]
                drw[k] = (d_out * y).sum()
            acc += rw_t[k] * y
            dacc += dxe
        ref_out.append(O._bf16(acc))
        ref_dx.append(O._bf16(dacc))
        ref_drw.append(drw)
    idx = torch.tensor(tokens, device=dev)
    errors["output"] = rel_l2(torch.cat(ref_out), out[idx].float().cpu())
    errors["d_x"] = rel_l2(torch.cat(ref_dx), grads[0][idx].float().cpu())
    errors["d_router_weights"] = rel_l2(torch.stack(ref_drw), grads[1][idx].float().cpu())

    worst = max(errors.values())
    return {"schedule_exact": schedule_exact, "rel_l2_max": worst, "rel_l2": errors, "tolerance": tol,
            "ok": bool(schedule_exact and worst <= tol), "tokens_checked": len(tokens),
            "experts_checked": len(expert_rows), "expert_rows": [int(v["x"].shape[0]) for v in expert_rows.values()],
            "oracle": "cpu oracle quantizing at the same points" if mxfp8 else "cpu oracle with bf16 rounding points",
            "seconds": round(time.time() - t_start, 1)}


# ------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------
def bind_near_gpu(index: int):
    """Restricts the calling thread to the host cores of the NUMA node the GPU hangs off.  Used around the allocation
    of the pinned staging buffers of the end-to-end loop, so that their pages are node-local to the GPU that reads and
    writes them (the caller restores the previous mask afterwards).  MOK_BENCH_NO_NUMA=1 skips it."""
    if os.environ.get("MOK_BENCH_NO_NUMA") == "1":
        return {"numa_node": None, "bound": False}
    try:
        import torch
        p = torch.cuda.get_device_properties(index)
        bdf = f"{p.pci_domain_id:04x}:{p.pci_bus_id:02x}:{p.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return {"numa_node": node, "bound": False}
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            cpus = set()
            for part in f.read().strip().split(","):
                a, _, b = part.partition("-")
                cpus.update(range(int(a), int(b or a) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return {"numa_node": node, "bound": False}
        os.sched_setaffinity(0, allowed)
        return {"numa_node": node, "bound": True, "cpus": len(allowed)}
    except (OSError, ValueError, AttributeError):
        return {"numa_node": None, "bound": False}


def run_gpu_arm(args, w):
    import torch
    import torch.distributed as dist
    import mok
    F = mok.functional

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} needs {args.gpus} ranks (torchrun), found WORLD_SIZE={world}")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29555")
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)

    T, H, E, I, K = w["T"], w["H"], w["E"], w["I"], w["K"]
    if E % world != 0:
        raise SystemExit(f"{E} experts do not shard over {world} ranks")
    e_loc = E // world
    base_cfg = F.MoKConfig() if w["cap_mult"] is None else F.MoKConfig(schedule_capacity_multiplier=w["cap_mult"])
    capacity = T * K * max(2, math.ceil(world * base_cfg.schedule_capacity_multiplier))
    minibatch = args.minibatch or base_cfg.minibatch_size
    # headline: one window covers the expected rows (routes + per-expert padding) so backward never replays gate / up
    expected = T * K + e_loc * 256
    one_window = min(capacity, -(-int(expected * 1.06) // minibatch) * minibatch)
    mb = args.macrobatch or w["macrobatch"] or one_window
    mb = min(-(-mb // minibatch) * minibatch, -(-capacity // minibatch) * minibatch)

    def config_for(macrobatch):
        return F.MoKConfig(minibatch_size=minibatch, macrobatch_size=macrobatch,
                           schedule_capacity_multiplier=base_cfg.schedule_capacity_multiplier)

    router = router_parameters(w, dev)
    x, dy, topk, rw = make_activations(w, rank, dev, router)
    weights = make_weights(w, e_loc, rank, dev)
    ws = F.get_workspace(config_for(mb), dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
    case = types.SimpleNamespace(w=w, dev=dev, world=world, rank=rank, e_loc=e_loc, capacity=capacity, router=router,
                                 x=x, dy=dy, topk=topk, rw=rw, weights=weights)
    peaks = measured_peaks()
    sampler = ClockSampler(local)   # started before the warm-up so that it is already reporting in the timed region
    sampler.start()

    def timed(fn, steps):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn(steps)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)  # noqa: E731
    all_cores = os.sched_getaffinity(0)
    host = bind_near_gpu(local)
    host_in = tuple(pin(t) for t in (x, dy, topk, rw))
    host_out = [(pin(x), pin(x), pin(rw)) for _ in range(2)]
    host_metric = [torch.empty(3, dtype=torch.float32, pin_memory=True) for _ in range(2)]
    os.sched_setaffinity(0, all_cores)
    dev_in = [tuple(torch.empty_like(t) for t in (x, dy, topk, rw)) for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h_full = sum(t.numel() * t.element_size() for t in host_out[0])
    d2h = d2h_full if args.e2e_full_output else host_metric[0].numel() * host_metric[0].element_size()

    def measure(mxfp8: bool, primary: bool):
        """Times the step in one precision; returns the figures of its part of the line."""
        nonlocal weights
        dtype = "mxfp8" if mxfp8 else "bf16"
        config = config_for(mb)
        qg = None
        dropped_bf16 = False
        if mxfp8:   # routed weights are quantized once, outside the timed region, as a trainer caches them
            qg = mok.ops.mxfp8_quantize(weights[3], True, True)
            qu = mok.ops.mxfp8_quantize(weights[4], True, True)
            qd = mok.ops.mxfp8_quantize(weights[5], True, True)
            fwd_w = weights[:3] + ((qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1]))
            bwd_w = weights[:3] + (qg, qu, (qd[2], qd[3]))
            if 3.0 * e_loc * I * H * 2 > 12e9:   # the bf16 copies are not needed meanwhile; they are redrawn from the seed
                dropped_bf16 = True
                weights = weights[:3] + (None, None, None)
                case.weights = weights
                torch.cuda.empty_cache()
        else:
            fwd_w = bwd_w = weights

        def step(x_, dy_, topk_, rw_, cfg=config):
            sched = F.build_schedule(ws, cfg, topk_, num_local_experts=e_loc)
            out, ctx = F.forward(cfg, ws, sched, x_, rw_, *fwd_w)
            grads = F.backward(cfg, ws, sched, ctx, dy_, x_, rw_, *bwd_w)
            return sched, out, grads

        def plain_steps(steps, cfg=config):
            for _ in range(steps):
                step(x, dy, topk, rw, cfg)

        for _ in range(args.warmup):
            plain_steps(1)
        torch.cuda.synchronize()
        mok.ops.check_status(dev)
        launches0 = mok.ops.lib().mok_launch_count()
        t_begin = time.time()
        ms_step = timed(plain_steps, args.steps)
        t_end = time.time()
        launches = (mok.ops.lib().mok_launch_count() - launches0) // args.steps
        clocks = sampler.window(t_begin, t_end)
        mok.ops.check_status(dev)

        # End to end: every step takes its inputs (x, d_output, routes, router weights) from pinned host memory and
        # returns its result to pinned host memory: by default the norms of output, d_x and d_router_weights (what a
        # training loop reads back is a metric; the tensors stay on the device for the next layer), with
        # --e2e-full-output the three tensors in full.  The copies run on two copy streams with two input and two output
        # slots, the way a prefetching data loader feeds a training loop: step i + 1's inputs travel while step i
        # computes, step i's results while step i + 1 computes.  All of it lies between the timing events.
        def e2e_steps(steps):
            main = torch.cuda.current_stream()
            begin = torch.cuda.Event()
            begin.record(main)
            copy_in.wait_event(begin)
            copy_out.wait_event(begin)
            ready = [torch.cuda.Event() for _ in range(steps)]
            consumed = [torch.cuda.Event() for _ in range(steps)]
            stored = [torch.cuda.Event() for _ in range(steps)]

            def prefetch(i):
                with torch.cuda.stream(copy_in):
                    if i >= 2:
                        copy_in.wait_event(consumed[i - 2])      # the step that used this slot has read it
                    for d_t, h_t in zip(dev_in[i % 2], host_in):
                        d_t.copy_(h_t, non_blocking=True)
                    ready[i].record(copy_in)

            prefetch(0)
            for i in range(steps):
                if i + 1 < steps:
                    prefetch(i + 1)
                main.wait_event(ready[i])
                _, out, grads = step(*dev_in[i % 2])
                if not args.e2e_full_output:   # the step's result as a metric: norms of output, d_x and d_router_weights
                    results = (torch.stack([torch.linalg.vector_norm(t, dtype=torch.float32) for t in (out, grads[0], grads[1])]),)
                    targets = (host_metric[i % 2],)
                else:
                    results, targets = (out, grads[0], grads[1]), host_out[i % 2]
                consumed[i].record(main)
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(consumed[i])
                    for h_t, d_t in zip(targets, results):
                        h_t.copy_(d_t, non_blocking=True)
                        d_t.record_stream(copy_out)
                    stored[i].record(copy_out)
            main.wait_event(stored[steps - 1])

        e2e_steps(1)
        ms_e2e = timed(e2e_steps, max(2, args.steps))
        mok.ops.check_status(dev)

        tokens = T * world
        fl = flops_per_token(w) * T            # per rank
        tflops = fl / (ms_step * 1e-3) / 1e12
        res = {"ms_per_step": ms_step, "tokens_per_s": tokens / (ms_step * 1e-3), "tflops_per_gpu": tflops,
               "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
               "gpu_launches": int(launches), "clocks": clocks}
        if mxfp8:   # no measured fp8 figure exists on this pool; the dense fp8 rate of the part is twice its bf16 rate
            res["frac_of_2x_bf16_burst"] = tflops / (2.0 * peaks["burst"])
            res["frac_of_2x_bf16_sustained"] = tflops / (2.0 * peaks["sustained"])
        else:
            res["frac_of_bf16_peak_burst"] = tflops / peaks["burst"]
            res["frac_of_bf16_peak_sustained"] = tflops / peaks["sustained"]

        if primary:
            # where one step spends its time: CUDA events between the three public calls (one extra, untimed step)
            marks = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            torch.cuda.synchronize()
            marks[0].record()
            sched_p = F.build_schedule(ws, config, topk, num_local_experts=e_loc)
            marks[1].record()
            out_p, ctx_p = F.forward(config, ws, sched_p, x, rw, *fwd_w)
            marks[2].record()
            grads_p = F.backward(config, ws, sched_p, ctx_p, dy, x, rw, *bwd_w)
            marks[3].record()
            torch.cuda.synchronize()
            res["phases"] = {"build_schedule_ms": marks[0].elapsed_time(marks[1]), "forward_ms": marks[1].elapsed_time(marks[2]),
                             "backward_ms": marks[2].elapsed_time(marks[3])}
            del sched_p, out_p, ctx_p, grads_p

            # the step with the reference's default ring: several windows, backward replays gate / up of windows >= 1
            ring_mb = min(REFERENCE_DEFAULT_MACROBATCH // minibatch * minibatch, mb)
            if ring_mb < mb and not args.no_ring:
                ring_cfg = config_for(ring_mb)
                torch.cuda.empty_cache()
                plain_steps(2, ring_cfg)
                ms_ring = timed(lambda n: plain_steps(n, ring_cfg), max(2, min(3, args.steps)))
                mok.ops.check_status(dev)
                res["ring"] = {"macrobatch_size": ring_mb, "windows_in_use": -(-int(expected) // ring_mb),
                               "ms_per_step": ms_ring, "tokens_per_s": tokens / (ms_ring * 1e-3)}
                torch.cuda.empty_cache()

        tracing = primary and os.environ.get("MOK_TRACE") == "1"
        if tracing:   # drop what the earlier steps recorded, keep the timeline of exactly one step
            mok.ops.lib().mok_trace_dump(os.devnull.encode())
        sched, out, grads = step(x, dy, topk, rw)
        torch.cuda.synchronize()
        if tracing:
            trace_dir = os.environ.get("MOK_TRACE_DIR", ROOT)   # where the phase timelines go (one file per rank)
            os.makedirs(trace_dir, exist_ok=True)
            mok.ops.lib().mok_trace_dump(os.path.join(trace_dir, f"trace_{dtype}_ep{world}_rank{rank}.txt").encode())
        mok.ops.check_status(dev)

        if not args.no_parity:
            if rank == 0:
                res["parity"] = sampled_parity(case, mxfp8, sched, out, grads, n_tokens=2 if mxfp8 else 4)
            dist.barrier()
        valid_rows = torch.tensor([float((sched.peer_rank >= 0).sum().item())], device=dev, dtype=torch.float64)
        all_rows = [torch.zeros_like(valid_rows) for _ in range(world)]
        dist.all_gather(all_rows, valid_rows)
        res["hot_rank_share_of_routes"] = max(v.item() for v in all_rows) / max(1.0, sum(v.item() for v in all_rows))
        del out, grads
        torch.cuda.empty_cache()
        if mxfp8:
            forms, rows_done = time_gemm_forms_mxfp8(dev, w, e_loc, sched, qg, mb)
        else:
            forms, rows_done = time_gemm_forms(dev, w, e_loc, sched, weights, mb)
        res["forms"], res["rows"] = forms, rows_done
        if primary:
            res["comm"] = time_comm_kernels(dev, w, ws, sched, mb, world, config.fwd_num_comm_sms * 8)
        del fwd_w, bwd_w, qg
        if mxfp8:
            del qu, qd
        torch.cuda.empty_cache()
        if dropped_bf16:
            weights = make_weights(w, e_loc, rank, dev)
            case.weights = weights
        return res

    primary_mx = args.dtype == "mxfp8"
    main_res = measure(primary_mx, True)
    other_res = None
    if not args.single:
        torch.cuda.empty_cache()
        other_res = measure(not primary_mx, False)
    sampler.stop()

    # the copies of the end-to-end loop alone (all ranks at once): what the host side delivers without any compute
    def copies_only(steps):
        for i in range(steps):
            with torch.cuda.stream(copy_in):
                for d_t, h_t in zip(dev_in[i % 2], host_in):
                    d_t.copy_(h_t, non_blocking=True)
            with torch.cuda.stream(copy_out):
                for h_t, d_t in zip(host_out[i % 2], (x, dy, rw)):
                    h_t.copy_(d_t, non_blocking=True)
        torch.cuda.current_stream().wait_stream(copy_in)
        torch.cuda.current_stream().wait_stream(copy_out)
    copies_only(1)
    ms_copies = timed(copies_only, 3)

    if rank == 0:
        tokens = T * world
        forms = main_res["forms"]
        dominant = forms["fwd_gate"]
        peak_tc = peaks["burst"] * (2.0 if primary_mx else 1.0)
        peak_src = ("2 x " if primary_mx else "") + peaks["source"] + " bf16 burst"
        rows_done = main_res["rows"]
        # DRAM bytes of one forward-form launch, scaled by rows from an ncu capture of a 16384-row launch with 1024 rows
        # per expert (56.3 KB per schedule row); only quoted while the rows per expert stay near that case
        rows_per_expert = rows_done / max(1, e_loc)
        traffic = int(56.3e3 * rows_done) if (not primary_mx and H == 7168 and I == 2048 and 512 <= rows_per_expert <= 2048) else None
        roofline = {"bound": "tensor",
                    "kernel": ("mxfp8_gemm_kernel" if primary_mx else "grouped_gemm_kernel") + " (forward gate form)",
                    "achieved": dominant["tflops"], "peak": peak_tc, "unit": "TFLOP/s", "frac": dominant["tflops"] / peak_tc,
                    "traffic": traffic,
                    "traffic_source": ("ncu dram bytes of a 16384-row launch of this kernel, scaled by rows" if traffic else None),
                    "peak_source": peak_src, "rows": rows_done, "forms": forms}
        comm = main_res.get("comm", {})
        if world > 1:
            # NVLink: payload that must cross the links per step (dispatch x, combine y, dispatch d_y, combine d_x of the
            # rows whose source is another rank) against the measured peer-copy bandwidth per direction
            nv_bytes = 4.0 * rows_done * H * 2 * (world - 1) / world
            nv_ms = nv_bytes / (NVLINK_PEER_COPY_GBS * 1e9) * 1e3
            roofline["nvlink"] = {"bytes_per_step_per_direction": nv_bytes, "peak_gbs": NVLINK_PEER_COPY_GBS,
                                  "time_at_peak_ms": nv_ms, "share_of_step": nv_ms / main_res["ms_per_step"],
                                  "dispatch_kernel_gbs": comm.get("dispatch_full_grid", {}).get("nvlink_gbs"),
                                  "combine_kernel_gbs": comm.get("combine_full_grid", {}).get("nvlink_gbs")}
            tc_ms = flops_per_token(w) * T / (peak_tc * 1e12) * 1e3
            if nv_ms > tc_ms:   # the links, not the tensor cores, bound this shape: report against them
                roofline.update({"bound": "nvlink", "kernel": "dispatch_kernel (pull over NVLink)",
                                 "achieved": comm.get("dispatch_full_grid", {}).get("nvlink_gbs"), "peak": NVLINK_PEER_COPY_GBS,
                                 "unit": "GB/s", "peak_source": "measured peer copy per direction",
                                 "frac": (comm.get("dispatch_full_grid", {}).get("nvlink_gbs") or 0.0) / NVLINK_PEER_COPY_GBS,
                                 "step_frac_of_nvlink_roof": nv_ms / main_res["ms_per_step"]})
        e2e = dict(main_res["e2e"])
        e2e["copies_alone_ms_per_step"] = ms_copies
        e2e["copies_alone_h2d_gbs_per_rank"] = h2d / (ms_copies * 1e-3) / 1e9
        e2e["copies_alone_d2h_gbs_per_rank"] = d2h_full / (ms_copies * 1e-3) / 1e9
        e2e["result_read_back"] = ("output, d_x, d_router_weights in full" if args.e2e_full_output else
                                   "fp32 norms of output, d_x and d_router_weights (a metric, as a training step reads back)")
        e2e["host"] = host
        line = {
            "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": tokens / (main_res["ms_per_step"] * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": w["label"].replace("bf16", args.dtype), "tokens_per_rank": T, "hidden": H, "experts": E,
                       "intermediate": I, "topk": K, "shared_expert": True, "parallelism": f"ep{world}", "macrobatch_size": mb,
                       "minibatch_size": minibatch, "schedule_capacity": capacity,
                       "schedule_capacity_multiplier": base_cfg.schedule_capacity_multiplier,
                       "hot_rank_share_of_routes": main_res["hot_rank_share_of_routes"],
                       "l2_policy": "inputs_larger_than_L2"},
            "tflops_per_gpu": main_res["tflops_per_gpu"],
            "roofline": roofline, "e2e": e2e, "gpu_launches": main_res["gpu_launches"], "clocks": main_res["clocks"],
            "comm": comm, "phases": main_res.get("phases"),
        }
        for key in ("frac_of_bf16_peak_burst", "frac_of_bf16_peak_sustained", "frac_of_2x_bf16_burst", "frac_of_2x_bf16_sustained",
                    "parity", "ring"):
            if key in main_res:
                line[key] = main_res[key]
        if other_res is not None:
            line["bf16" if primary_mx else "mxfp8"] = {k: v for k, v in other_res.items() if k != "hot_rank_share_of_routes"}
        if not args.no_cpu:
            ct, ce = cpu_sample_size(w)
            tps, sec, cores = cpu_sample(w, ct, ce, 1, 0)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": cpu_sample_text(w, ct, ce) + ", one pass"}
        print(json.dumps(line), flush=True)
    dist.barrier()
    F.clear_workspace_cache()
    dist.destroy_process_group()
    if rank == 0:
        bad = [name for name, res in (("primary", main_res), ("secondary", other_res))
               if res is not None and "parity" in res and not res["parity"]["ok"]]
        if bad:
            sys.stderr.write(f"bench: the sampled parity check failed for the {', '.join(bad)} precision\n")
            sys.exit(4)


def run_gemm_only(args, w):
    """Small stand-alone case of the dominant kernel for profiling: `--gemm-only ROWS` schedule rows spread evenly
    over `--gemm-experts` experts of the workload's H and I (a few hundred MB: larger than L2, quick to capture)."""
    import torch
    import mok  # noqa: F401
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    e, rows = args.gemm_experts, args.gemm_only
    per = rows // e // 256 * 256
    rows = per * e
    H, I = w["H"], w["I"]
    sched = types.SimpleNamespace(
        peer_rank=torch.zeros(rows, dtype=torch.int32, device=dev),
        num_tokens=torch.tensor([rows], dtype=torch.int32, device=dev),
        tokens_per_expert=torch.full((e,), per, dtype=torch.int32, device=dev))
    g = torch.Generator(device=dev).manual_seed(0)
    wt = lambda *s: torch.randn(*s, generator=g, device=dev, dtype=torch.bfloat16).mul_(w["std"])  # noqa: E731
    weights = (None, None, None, wt(e, I, H), None, wt(e, H, I))
    if args.dtype == "mxfp8":
        qg = mok.ops.mxfp8_quantize(weights[3], True, False)
        forms, rows_done = time_gemm_forms_mxfp8(dev, w, e, sched, qg, rows)
        # the quantizer on a [4 * rows, H] activation-sized matrix (bf16 in, e4m3 + scales out in both layouts)
        act = torch.randn(4 * rows, H, generator=g, device=dev, dtype=torch.bfloat16)
        for both in (False, True):
            mok.ops.mxfp8_quantize(act, True, both)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
            torch.cuda.synchronize()
            ev[0].record()
            for _ in range(5):
                mok.ops.mxfp8_quantize(act, True, both)
            ev[1].record()
            torch.cuda.synchronize()
            ms = ev[0].elapsed_time(ev[1]) / 5
            nbytes = act.numel() * (2 + (2 if both else 1) * (1 + 1 / 32))
            forms["quantize_" + ("both_layouts" if both else "normal")] = {"ms": ms, "hbm_gbs": nbytes / (ms * 1e-3) / 1e9}
    else:
        forms, rows_done = time_gemm_forms(dev, w, e, sched, weights, rows)
    peaks = measured_peaks()
    print(json.dumps({"mode": "gemm-only", "rows": rows_done, "experts": e, "hidden": H, "intermediate": I, "forms": forms,
                      "peak_burst_tflops": peaks["burst"], "peak_source": peaks["source"]}), flush=True)


def run_router_only(args, w):
    """`--router`: the device router (forward and backward) on the workload's tokens, hidden size, expert count and
    top-k, next to the PyTorch expression it replaces (fp32 matmul, topk, softmax and their autograd) on the same GPU."""
    import torch
    import mok
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    T, H, E, K = w["T"], w["H"], w["E"], w["K"]
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(T, H, generator=g, device=dev, dtype=torch.bfloat16)
    wr = torch.randn(E, H, generator=g, device=dev) * H ** -0.5
    d_w = torch.randn(T, K, generator=g, device=dev)

    def timed(fn, reps=10):
        for _ in range(3):
            fn()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(reps):
            fn()
        ev[1].record()
        torch.cuda.synchronize()
        return ev[0].elapsed_time(ev[1]) / reps

    routes, weights, _ = mok.ops.router_fwd(x, wr, None, K)
    fwd_ms = timed(lambda: mok.ops.router_fwd(x, wr, None, K))
    bwd_ms = timed(lambda: mok.ops.router_bwd(x, wr, routes, weights, d_w, False))
    mok.ops.check_status(dev)

    def torch_fwd():
        vals, idx = torch.topk(x.float() @ wr.t(), K, dim=-1)
        return idx, torch.softmax(vals, dim=-1)

    xg, wg = x.detach().clone().requires_grad_(True), wr.detach().clone().requires_grad_(True)

    def torch_fwd_bwd():
        vals, _ = torch.topk(xg.float() @ wg.t(), K, dim=-1)
        torch.softmax(vals, dim=-1).backward(d_w)
        xg.grad = wg.grad = None

    t_fwd = timed(torch_fwd)
    t_both = timed(torch_fwd_bwd)
    idx, _ = torch_fwd()
    agree = (idx.sort(dim=1).values == routes.long().sort(dim=1).values).all(dim=1).float().mean().item()
    fl = 2.0 * T * H * E
    print(json.dumps({
        "mode": "router", "tokens": T, "hidden": H, "experts": E, "topk": K,
        "forward_ms": fwd_ms, "backward_ms": bwd_ms,
        # two bf16 terms of the fp32 matrix in the forward product; two products in the backward
        "forward_tflops": 2 * fl / (fwd_ms * 1e-3) / 1e12, "backward_tflops": 2 * fl / (bwd_ms * 1e-3) / 1e12,
        "x_bytes_over_forward_gbs": x.numel() * 2 / (fwd_ms * 1e-3) / 1e9,
        "torch_forward_ms": t_fwd, "torch_forward_backward_ms": t_both,
        "tokens_with_the_same_expert_set_as_torch_fp32": agree}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--router", action="store_true", help="time the device router on the workload's shapes")
    ap.add_argument("--gemm-only", type=int, default=0, help="profile helper: time only the GEMM forms on this many rows")
    ap.add_argument("--gemm-experts", type=int, default=16)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--macrobatch", type=int, default=0, help="rows of the routed activation ring (default: one window)")
    ap.add_argument("--minibatch", type=int, default=0, help="minibatch_size of the layer configuration (default 4096)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline sample")
    ap.add_argument("--no-parity", action="store_true", help="skip the sampled parity check against the CPU oracle")
    ap.add_argument("--no-ring", action="store_true", help="skip the extra timing at the reference's default macrobatch")
    ap.add_argument("--single", action="store_true", help="time only the precision named by --dtype")
    ap.add_argument("--e2e-full-output", action="store_true",
                    help="end-to-end loop copies output, d_x and d_router_weights to the host in full instead of their norms")
    ap.add_argument("--dtype", default="bf16", choices=("bf16", "mxfp8"))
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    if args.gemm_only:
        run_gemm_only(args, w)
    elif args.router:
        run_router_only(args, w)
    elif args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_gpu_arm(args, w)


if __name__ == "__main__":
    main()
