"""Benchmark of the expert-parallel MoE layer, forward + backward (tokens/s).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload c2|c1|c0|tiny]

One step = build_schedule + forward + backward of one MoE layer over one batch of synthetic tokens through
`mok.functional`.  The default workload is the DeepSeek-V3-shaped layer (32768 tokens per rank, hidden 7168,
256 routed experts of intermediate 2048 sharded over the N ranks, top-8, one shared expert).  Rank 0 prints one
JSON line.  Under torchrun (N > 1) every rank runs one GPU; times are the maximum over ranks.

`--impl reference` times the CPU restatement of the reference math (oracle/) on the host cores, on a bounded
sample of the same layer shape; that leg never touches the GPU library.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

WORKLOADS = {
    # name: tokens/rank, hidden, experts (global), intermediate, topk, weight std, bias std
    "c2": dict(T=32768, H=7168, E=256, I=2048, K=8, std=0.006, bias=0.0, label="deepseek-v3-shaped bf16"),
    # the benchmark's row shapes on a few GB of device memory: the case profiler captures of the bandwidth kernels use
    "c2s": dict(T=4096, H=7168, E=16, I=2048, K=8, std=0.006, bias=0.0, label="deepseek-v3-shaped bf16, 16 experts"),
    "c1": dict(T=16384, H=2048, E=128, I=768, K=8, std=0.02, bias=0.5, label="qwen3-moe-shaped bf16"),
    "c0": dict(T=2048, H=512, E=8, I=1024, K=2, std=0.02, bias=0.0, label="cpu-plumbing shape"),
    "tiny": dict(T=512, H=256, E=8, I=256, K=2, std=0.02, bias=0.0, label="tiny"),
}


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

    def stop(self, t_begin: float = 0.0, t_end: float = float("inf")):
        """Summarises the samples that arrived inside [t_begin, t_end] (wall clock); all of them by default."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        time.sleep(0.05)
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


# ------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference math, timed on the host cores
# ------------------------------------------------------------------------------------------------------------
def cpu_sample(w, tokens: int, experts: int, steps: int, warmup: int):
    """Times fwd+bwd of a bounded sample: `tokens` tokens, `experts` experts, same H / I / K as the workload."""
    import torch
    from oracle import moe_oracle as O
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


def run_reference_arm(args, w):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    tokens, experts = cpu_sample_size(w)
    tps, sec, cores = cpu_sample(w, tokens, experts, max(1, args.steps), min(args.warmup, 1))
    sample = f"{tokens} tokens, {experts} experts, H={w['H']} I={w['I']} top-{min(w['K'], experts)}, fp32 math with bf16 rounding points"
    line = {
        "impl": "reference", "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": tps, "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": w["label"], "tokens_per_rank": w["T"], "hidden": w["H"], "experts": w["E"],
                   "intermediate": w["I"], "topk": w["K"], "shared_expert": True},
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------------------
def make_gpu_inputs(w, e_loc: int, rank: int, dev):
    """Seeded synthetic layer: x, dy ~ N(0,1); weights ~ N(0, std); logits = x W_r (+ bias ~ N(0, bias));
    top-k routing with softmax over the selected logits (renormalised weights)."""
    import torch
    g = torch.Generator(device=dev).manual_seed(0 + rank)
    gw = torch.Generator(device=dev).manual_seed(12345)          # router and bias are shared by all ranks
    T, H, E, I, K = w["T"], w["H"], w["E"], w["I"], w["K"]
    bf = dict(device=dev, dtype=torch.bfloat16)
    x = torch.randn(T, H, generator=g, **bf)
    dy = torch.randn(T, H, generator=g, **bf)
    w_r = torch.randn(H, E, generator=gw, device=dev) * w["std"]
    logits = x.float() @ w_r
    if w["bias"] > 0:
        logits += torch.randn(E, generator=gw, device=dev) * w["bias"]
    vals, topk = torch.topk(logits, K, dim=1)
    rw = torch.softmax(vals, dim=-1).contiguous()

    def wt(*shape):
        return torch.randn(*shape, generator=g, **bf).mul_(w["std"])
    weights = (wt(I, H), wt(I, H), wt(H, I), wt(e_loc, I, H), wt(e_loc, I, H), wt(e_loc, H, I))
    return x, dy, topk.contiguous(), rw, weights


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
    for name, fn in (("fwd_gate", fwd), ("dgrad_down", dgrad), ("wgrad_gate", wgrad)):
        for _ in range(2):
            nat.check(fn(), name)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        reps = 5
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(reps):
            fn()
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1]) / reps
        out[name] = {"ms": ms, "tflops": 2.0 * rows_done * H * I / (ms * 1e-3) / 1e12}
    nat.check_status(dev)
    return out, rows_done


def time_gemm_forms_mxfp8(dev, w, e_loc, sched, qg, qd, rows_buf):
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
    for name, fn in (("fwd_gate", fwd), ("wgrad_gate", wgrad)):
        for _ in range(2):
            nat.check(fn(), name)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        reps = 5
        torch.cuda.synchronize()
        ev[0].record()
        for _ in range(reps):
            fn()
        ev[1].record()
        torch.cuda.synchronize()
        ms = ev[0].elapsed_time(ev[1]) / reps
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
    e_loc = E // world
    capacity_factor = max(2, -(-world // 2))
    capacity = T * K * capacity_factor
    # one window covers the expected rows (routes + per-expert padding) so backward never replays gate/up
    expected = T * K + e_loc * 256
    mb = min(capacity, -(-int(expected * 1.06) // 4096) * 4096)
    if args.macrobatch:
        mb = args.macrobatch
    config = F.MoKConfig(minibatch_size=4096 if mb % 4096 == 0 else 256, macrobatch_size=mb)
    x, dy, topk, rw, weights = make_gpu_inputs(w, e_loc, rank, dev)
    ws = F.get_workspace(config, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)

    mxfp8 = args.dtype == "mxfp8"
    if mxfp8:   # routed weights are quantized once, outside the timed region, as a trainer caches them
        qg = mok.ops.mxfp8_quantize(weights[3], True, True)
        qu = mok.ops.mxfp8_quantize(weights[4], True, True)
        qd = mok.ops.mxfp8_quantize(weights[5], True, True)
        fwd_w = weights[:3] + ((qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1]))
        bwd_w = weights[:3] + (qg, qu, (qd[2], qd[3]))
        weights = weights[:3] + (None, None, None)       # the bf16 copies are not needed any more
        torch.cuda.empty_cache()
    else:
        fwd_w = bwd_w = weights

    def step(x_, dy_, topk_, rw_):
        sched = F.build_schedule(ws, config, topk_, num_local_experts=e_loc)
        out, ctx = F.forward(config, ws, sched, x_, rw_, *fwd_w)
        grads = F.backward(config, ws, sched, ctx, dy_, x_, rw_, *bwd_w)
        return sched, out, grads

    def timed(fn, steps):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    sampler = ClockSampler(local)   # started before the warm-up so that it is already reporting in the timed region
    sampler.start()
    for _ in range(args.warmup):
        out = step(x, dy, topk, rw)
        del out
    torch.cuda.synchronize()
    mok.ops.check_status(dev)
    launches0 = mok.ops.lib().mok_launch_count()
    t_begin = time.time()
    ms_step = timed(lambda: step(x, dy, topk, rw), args.steps)
    t_end = time.time()
    launches = (mok.ops.lib().mok_launch_count() - launches0) // args.steps
    clocks = sampler.stop(t_begin, t_end)
    mok.ops.check_status(dev)

    # End to end: every step takes its inputs (x, d_output, routes, router weights) from pinned host memory and returns
    # output, d_x and d_router_weights to pinned host memory.  The copies run on two copy streams with two input and two
    # output slots, the way a prefetching data loader feeds a training loop: step i + 1's inputs travel while step i
    # computes, step i's results while step i + 1 computes.  All of it lies between the two timing events.
    pin = lambda t: torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)  # noqa: E731
    host_in = tuple(pin(t) for t in (x, dy, topk, rw))
    dev_in = [tuple(torch.empty_like(t) for t in (x, dy, topk, rw)) for _ in range(2)]
    host_out = [(pin(x), pin(x), pin(rw)) for _ in range(2)]
    copy_in, copy_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)

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
            consumed[i].record(main)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(consumed[i])
                for h_t, d_t in zip(host_out[i % 2], (out, grads[0], grads[1])):
                    h_t.copy_(d_t, non_blocking=True)
                    d_t.record_stream(copy_out)
                stored[i].record(copy_out)
        main.wait_event(stored[steps - 1])

    def timed_e2e(steps):
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_steps(steps)
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / steps

    e2e_steps(1)
    ms_e2e = timed_e2e(max(2, args.steps))
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out[0])

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
    phases = {"build_schedule_ms": marks[0].elapsed_time(marks[1]), "forward_ms": marks[1].elapsed_time(marks[2]),
              "backward_ms": marks[2].elapsed_time(marks[3])}
    del sched_p, out_p, ctx_p, grads_p

    tracing = os.environ.get("MOK_TRACE") == "1"
    if tracing:   # drop what the earlier steps recorded, keep the timeline of exactly one step
        mok.ops.lib().mok_trace_dump(os.devnull.encode())
    sched, out, grads = step(x, dy, topk, rw)
    if tracing:
        trace_dir = os.environ.get("MOK_TRACE_DIR", ROOT)   # where the phase timelines go (one file per rank)
        os.makedirs(trace_dir, exist_ok=True)
        mok.ops.lib().mok_trace_dump(os.path.join(trace_dir, f"trace_{args.dtype}_ep{world}_rank{rank}.txt").encode())
    del out, grads
    if mxfp8:
        forms, rows_done = time_gemm_forms_mxfp8(dev, w, e_loc, sched, qg, qd, mb)
    else:
        forms, rows_done = time_gemm_forms(dev, w, e_loc, sched, weights, mb)
    comm = time_comm_kernels(dev, w, ws, sched, mb, world, config.fwd_num_comm_sms * 8)
    if rank == 0:
        peaks = measured_peaks()
        tokens = T * world
        fl = flops_per_token(w) * T            # per rank
        dominant = forms["fwd_gate"]
        # MXFP8: no measured fp8 figure exists on this pool; the dense fp8 rate of the part is twice its bf16 rate
        peak_tc = peaks["burst"] * (2.0 if mxfp8 else 1.0)
        peak_src = ("2 x " if mxfp8 else "") + peaks["source"] + " bf16 burst"
        # DRAM bytes of one forward-form launch: ncu measured 56.3 KB per schedule row on a 16384-row capture with
        # 1024 rows per expert (profiles/); scaled by rows, valid while the rows per expert stay near that
        rows_per_expert = rows_done / max(1, e_loc)
        traffic = int(56.3e3 * rows_done) if (not mxfp8 and 512 <= rows_per_expert <= 2048) else None
        line = {
            "metric": "moe_layer_fwd_bwd_tokens_per_s", "value": tokens / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": args.dtype, "data": "synthetic",
            "config": {"workload": w["label"].replace("bf16", args.dtype), "tokens_per_rank": T, "hidden": H, "experts": E, "intermediate": I, "topk": K,
                       "shared_expert": True, "parallelism": f"ep{world}", "macrobatch_size": mb,
                       "schedule_capacity": capacity, "l2_policy": "inputs_larger_than_L2"},
            "tflops_per_gpu": fl / (ms_step * 1e-3) / 1e12,
            "frac_of_bf16_peak_sustained": fl / (ms_step * 1e-3) / 1e12 / peaks["sustained"],
            "roofline": {"bound": "tensor",
                         "kernel": ("mxfp8_gemm_kernel" if mxfp8 else "grouped_gemm_kernel") + " (forward gate form)",
                         "achieved": dominant["tflops"], "peak": peak_tc, "unit": "TFLOP/s", "frac": dominant["tflops"] / peak_tc,
                         "traffic": traffic, "peak_source": peak_src, "rows": rows_done, "forms": forms},
            "e2e": {"value": tokens / (ms_e2e * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches), "clocks": clocks, "comm": comm, "phases": phases,
        }
        if world == 1 and not args.no_cpu:
            ct, ce = cpu_sample_size(w)
            tps, sec, cores = cpu_sample(w, ct, ce, 1, 0)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"{ct} tokens, {ce} experts, H={H} I={I} top-{min(K, ce)}, one pass of the CPU oracle"}
        print(json.dumps(line), flush=True)
    F.clear_workspace_cache()
    dist.destroy_process_group()


def run_gemm_only(args, w):
    """Small stand-alone case of the dominant kernel for profiling: `--gemm-only ROWS` schedule rows spread evenly
    over `--gemm-experts` experts of the workload's H and I (a few hundred MB: larger than L2, quick to capture)."""
    import types
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
        forms, rows_done = time_gemm_forms_mxfp8(dev, w, e, sched, qg, None, rows)
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
    ap.add_argument("--macrobatch", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true")
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
