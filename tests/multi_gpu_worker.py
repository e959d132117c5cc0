"""One EP rank of the multi-GPU parity check (spawned by tests/test_gpu_multi.py, or run under torchrun).

Every rank draws the inputs of ALL ranks on the CPU (seeded), runs the CPU oracle for the whole EP group, runs its
own share on its GPU through `mok.functional`, and compares: schedule bit-exact, outputs and gradients inside the
bf16 tolerance (max |diff| <= 0.5, sum|diff|/sum|ref| <= 0.01, rel-L2 <= 1e-2), and a second run bitwise equal.
"""
from __future__ import annotations

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "mixture-of-kittens_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

FIELDS = ("d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
          "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")

CASES = (
    # E, H, I, K, T, config kwargs, swiglu limit
    (8, 256, 256, 2, 512, {}, None),
    (16, 512, 256, 4, 1024, dict(minibatch_size=256, macrobatch_size=2048), 2.0),   # several windows + clamp
)


def check_group(group, dev, cases, seed: int, tag: str) -> None:
    """Schedule, BF16 and MXFP8 layer parity and run-twice equality of this process's rank inside `group`."""
    import numpy as np
    import torch
    import torch.distributed as dist
    import mok
    from oracle import moe_oracle as O
    F = mok.functional
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    for E, H, I, K, T, cfg, limit in cases:
        e_loc = E // world
        config = F.MoKConfig(**cfg)
        inputs = [O.make_rank_inputs(r, E, e_loc, K, T, H, I, seed=seed) for r in range(world)]
        ref = O.moe_layer_oracle(inputs, swiglu_limit=limit)[rank]
        mine = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in vars(inputs[rank]).items()}
        ws = F.get_workspace(config, group, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
        assert ws.group_name == group.group_name and ws.ep_rank == rank and ws.ep_size == world
        assert len(ws.x_buffer_ptrs) == len(ws.combine_buffer_ptrs) == len(ws.barrier_buffer_ptrs) == world
        weights = (mine["w_shared_gate"], mine["w_shared_up"], mine["w_shared_down"],
                   mine["w_routed_gate"], mine["w_routed_up"], mine["w_routed_down"])

        def once():
            sched = F.build_schedule(ws, config, mine["topk_experts"], num_local_experts=e_loc)
            out, ctx = F.forward(config, ws, sched, mine["x"], mine["router_weights"], *weights, swiglu_limit=limit)
            grads = F.backward(config, ws, sched, ctx, mine["d_output"], mine["x"], mine["router_weights"], *weights,
                               swiglu_limit=limit)
            torch.cuda.synchronize()
            mok.ops.check_status(dev)
            return sched, out, grads

        sched, out, grads = once()
        topk_all = np.stack([i.topk_experts.to(torch.int32).numpy() for i in inputs])
        pr, pt, nt, tpe = O.schedule_oracle(topk_all, e_loc, ws.schedule_capacity, rank)
        assert np.array_equal(sched.peer_rank.cpu().numpy(), pr), "peer_rank"
        assert np.array_equal(sched.peer_token_idx.cpu().numpy(), pt), "peer_token_idx"
        assert int(sched.num_tokens.item()) == int(nt[0]) and np.array_equal(sched.tokens_per_expert.cpu().numpy(), tpe)
        for name, got in (("output", out),) + tuple(zip(FIELDS, grads)):
            mx, l1, l2, cos = O.error_stats(getattr(ref, name).float(), got.float().cpu())
            assert mx <= 0.5 and l1 <= 0.01 and l2 <= 0.01 and cos >= 0.9999, (tag, rank, name, mx, l1, l2, cos)
        _, out2, grads2 = once()
        assert torch.equal(out, out2), "output not bitwise reproducible"
        for name, a, b in zip(FIELDS, grads, grads2):
            assert torch.equal(a, b), f"{name} not bitwise reproducible"
        # de-duplicated dispatch (a token crosses NVLink once per destination rank and is fanned out locally) against
        # row-by-row pulls, each forced in turn: the rows are copies either way, so everything downstream is bitwise equal
        variants = {}
        for flag in ("1", "0"):
            os.environ["MOK_DEDUP"] = flag
            try:
                variants[flag] = once()
            finally:
                del os.environ["MOK_DEDUP"]
        staged, plain = variants["1"], variants["0"]
        assert plain[0].row_source is None and staged[0].row_source is not None
        assert int(staged[0].num_unique.item()) <= int((staged[0].peer_rank >= 0).sum().item())
        for other in (staged, plain):
            assert torch.equal(out, other[1]), "output differs between de-duplicated and row-by-row dispatch"
            for name, a, b in zip(FIELDS, grads, other[2]):
                assert torch.equal(a, b), f"{name} differs between de-duplicated and row-by-row dispatch"

        # the same layer in MXFP8 against the oracle that quantizes at the same points (rel-L2 <= 3e-2)
        emu = O.moe_layer_oracle(inputs, swiglu_limit=limit, mxfp8=True)[rank]
        qg = mok.ops.mxfp8_quantize(mine["w_routed_gate"], True, True)
        qu = mok.ops.mxfp8_quantize(mine["w_routed_up"], True, True)
        qd = mok.ops.mxfp8_quantize(mine["w_routed_down"], True, True)
        sched = F.build_schedule(ws, config, mine["topk_experts"], num_local_experts=e_loc)
        out8, ctx8 = F.forward(config, ws, sched, mine["x"], mine["router_weights"], *weights[:3], (qg[0], qg[1]),
                               (qu[0], qu[1]), (qd[0], qd[1]), swiglu_limit=limit)
        grads8 = F.backward(config, ws, sched, ctx8, mine["d_output"], mine["x"], mine["router_weights"], *weights[:3],
                            qg, qu, (qd[2], qd[3]), swiglu_limit=limit)
        torch.cuda.synchronize()
        mok.ops.check_status(dev)
        for name, got in (("output", out8),) + tuple(zip(FIELDS, grads8)):
            _, _, l2, _ = O.error_stats(getattr(emu, name).float(), got.float().cpu())
            assert l2 <= 3e-2, (tag, rank, "mxfp8", name, l2)
        F.clear_workspace_cache()


def check_barrier_counters(dev) -> None:
    """After two barriers on a fresh workspace the local target and the local counter both read 2 * ep_size: every rank
    added one to every counter per call (reference tests/test_misc.py:1730-1771)."""
    import torch
    import torch.distributed as dist
    import mok
    F = mok.functional
    F.clear_workspace_cache()
    ws = F.get_workspace(F.MoKConfig(minibatch_size=256, macrobatch_size=512), dist.group.WORLD, device=dev,
                         num_local_tokens=512, hidden_size=256, topk=1)
    assert int(ws.barrier_buffer.item()) == 0 and int(ws.barrier_target.item()) == 0
    for _ in range(2):
        mok.ops.barrier_all(ws.barrier_buffer, ws.barrier_buffer_ptrs, ws.barrier_buffer_multicast_ptr, ws.barrier_target)
        torch.cuda.synchronize()
    dist.barrier()
    assert int(ws.barrier_buffer.item()) == 2 * ws.ep_size and int(ws.barrier_target.item()) == 2 * ws.ep_size
    mok.ops.check_status(dev)
    F.clear_workspace_cache()


def run(rank: int, world: int, port: int) -> None:
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    # every rank computes the CPU oracle of the whole group: share the host cores instead of oversubscribing them
    # (eight processes with a full-size thread pool each spent a quarter of an hour here; one thread needs seconds)
    torch.set_num_threads(max(1, len(os.sched_getaffinity(0)) // world))
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        check_barrier_counters(dev)
        check_group(dist.group.WORLD, dev, CASES, 1234, f"EP={world}")
        dist.barrier()
        if world >= 4:
            # two EP groups of half the world, each with its own workspaces, routes and data: nothing may go through
            # the world group (reference tests/test_misc.py:648-707)
            half = world // 2
            groups = [dist.new_group(ranks=list(range(s, s + half))) for s in (0, half)]
            mine = groups[rank // half]
            check_group(mine, dev, CASES[:1], 1234 + 100 * (rank // half), f"EP={half} inside a world of {world}")
            dist.barrier()
            for g in groups:
                dist.destroy_process_group(g)
        if rank == 0:
            print(f"multi-gpu parity ok at EP={world}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    run(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("MASTER_PORT", "29541")))
