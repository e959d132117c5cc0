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


def run(rank: int, world: int, port: int) -> None:
    import numpy as np
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import mok
    from oracle import moe_oracle as O
    F = mok.functional
    try:
        for E, H, I, K, T, cfg, limit in CASES:
            e_loc = E // world
            config = F.MoKConfig(**cfg)
            inputs = [O.make_rank_inputs(r, E, e_loc, K, T, H, I) for r in range(world)]
            ref = O.moe_layer_oracle(inputs, swiglu_limit=limit)[rank]
            mine = {k: (v.to(dev) if torch.is_tensor(v) else v) for k, v in vars(inputs[rank]).items()}
            ws = F.get_workspace(config, dist.group.WORLD, device=dev, num_local_tokens=T, hidden_size=H, topk=K)
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
                assert mx <= 0.5 and l1 <= 0.01 and l2 <= 0.01 and cos >= 0.9999, (rank, name, mx, l1, l2, cos)
            _, out2, grads2 = once()
            assert torch.equal(out, out2), "output not bitwise reproducible"
            for name, a, b in zip(FIELDS, grads, grads2):
                assert torch.equal(a, b), f"{name} not bitwise reproducible"

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
                assert l2 <= 3e-2, (rank, "mxfp8", name, l2)
            F.clear_workspace_cache()
        dist.barrier()
        if rank == 0:
            print(f"multi-gpu parity ok at EP={world}", flush=True)
    finally:
        dist.destroy_process_group()


if __name__ == "__main__":
    run(int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ.get("MASTER_PORT", "29541")))
