"""Generates the golden fixtures in this directory from the reference project's own PyTorch helpers.

Run once in a container where the reference checkout is present:

    python tests/golden/make_golden.py /path/to/reference

It loads `<reference>/tests/utils.py` by path (that file needs only torch), runs it on CPU under
gloo at world_size 1 and 2 and stores the OUTPUTS as small `.npz` files.  Inputs are not stored:
they are re-drawn from the same seeds by `oracle.moe_oracle.make_rank_inputs`, and a checksum of
every input tensor is stored so a drift of the random generator would be noticed.

gloo refuses `all_gather_into_tensor(out[ws, ws], in[ws])`; the wrapper below flattens the output
view, which does not change the values.
"""
from __future__ import annotations

import importlib.util
import math
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, E, H, I, K, T) — tiny layer shapes; the arithmetic does not depend on size.
LAYER_CASES = (
    ("tiny", 4, 64, 96, 2, 128),
    ("small", 8, 128, 64, 3, 256),
)
SCHEDULE_CASES = (  # (name, E, K, T)
    ("sched_a", 8, 2, 512),
    ("sched_b", 16, 3, 768),     # routes not a multiple of 1024
    ("sched_c", 4, 1, 2048),
)


def _load_ref(ref_root):
    spec = importlib.util.spec_from_file_location("ref_utils", os.path.join(ref_root, "tests", "utils.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _u16(t):
    return t.contiguous().view(torch.uint16).numpy() if t.dtype == torch.bfloat16 else t.contiguous().numpy()


def _checksum(t):
    return float(t.double().abs().sum())


def _worker(rank, ws, ref_root, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=ws)
    U = _load_ref(ref_root)
    orig = dist.all_gather_into_tensor

    def flat_all_gather(out, inp, group=None, async_op=False):
        return orig(out.view(-1), inp.reshape(-1), group=group, async_op=async_op)
    dist.all_gather_into_tensor = flat_all_gather
    dev = torch.device("cpu")

    for name, E, H, I, K, T in LAYER_CASES:
        for limit in (None, 4.0):
            inp = U.generate_inputs(rank, dev, E, E // ws, K, T, H, I)
            out = U.run_reference_bf16(*inp, swiglu_limit=limit)
            fwd = U.run_forward_reference_bf16(inp[0], inp[1], *inp[3:9], swiglu_limit=limit)
            tag = f"layer_{name}_ws{ws}_r{rank}_{'clamp' if limit else 'plain'}"
            names = ("output", "d_x", "d_router_weights", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
                     "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down")
            blob = {n: _u16(t.detach()) for n, t in zip(names, out)}
            blob["combine_buffer"] = _u16(fwd[0])
            blob["y_shared"] = _u16(fwd[4])
            blob["fwd_epilogue"] = _u16(U.run_fwd_epilogue_reference(fwd[4], fwd[0], inp[2]))
            blob["input_checksums"] = np.array([_checksum(t) for t in inp], dtype=np.float64)
            blob["shape"] = np.array([E, H, I, K, T, ws, rank], dtype=np.int64)
            blob["limit"] = np.array([limit if limit else -1.0])
            np.savez_compressed(os.path.join(HERE, tag + ".npz"), **blob)

    for name, E, K, T in SCHEDULE_CASES:
        topk = U.generate_topk_experts(rank, dev, E, K, T).to(torch.int32)
        topk_all = U.run_all_gather_top_experts_reference(topk)
        cap = T * K * max(2, math.ceil(ws * 1.5))
        s = U.run_schedule_reference(topk_all, E // ws, cap, rank)
        np.savez_compressed(os.path.join(HERE, f"{name}_ws{ws}_r{rank}.npz"),
                            topk_all=topk_all.numpy(), peer_rank=s[0].numpy(), peer_token_idx=s[1].numpy(),
                            num_tokens=s[2].numpy(), tokens_per_expert=s[3].numpy(),
                            meta=np.array([E // ws, cap, rank], dtype=np.int64))
    # hand-built exact-capacity case of the reference tests: route = token % ws, one local expert
    T, K = 512, 1
    pattern = torch.arange(T, dtype=torch.int32).remainder(ws)
    topk_all = pattern.view(1, T, K).expand(ws, -1, -1).contiguous()
    s = U.run_schedule_reference(topk_all, 1, T * K, rank)
    np.savez_compressed(os.path.join(HERE, f"sched_exact_ws{ws}_r{rank}.npz"),
                        topk_all=topk_all.numpy(), peer_rank=s[0].numpy(), peer_token_idx=s[1].numpy(),
                        num_tokens=s[2].numpy(), tokens_per_expert=s[3].numpy(),
                        meta=np.array([1, T * K, rank], dtype=np.int64))

    if rank == 0 and ws == 1:
        g = torch.Generator().manual_seed(1234)
        for tag, shape in (("q2d", (256, 384)), ("q3d", (2, 128, 256))):
            x = torch.randn(shape, generator=g, dtype=torch.bfloat16)
            q = U.run_mxfp8_quantize_reference(x, True, True)
            np.savez_compressed(os.path.join(HERE, f"mxfp8_{tag}.npz"), x=_u16(x),
                                x_fp8=q[0].view(torch.uint8).numpy(), x_sc=q[1].numpy(),
                                x_fp8_t=q[2].view(torch.uint8).numpy(), x_sc_t=q[3].numpy())
        # SwiGLU and epilogue helpers on random data
        a = torch.randn(64, 96, generator=g, dtype=torch.bfloat16) * 3
        b = torch.randn(64, 96, generator=g, dtype=torch.bfloat16) * 3
        np.savez_compressed(os.path.join(HERE, "swiglu.npz"), gate=_u16(a), up=_u16(b),
                            plain=_u16(U.run_swiglu_reference(a, b)), clamp=_u16(U.run_swiglu_reference(a, b, 4.0)))
        ys = torch.randn(128, 64, generator=g, dtype=torch.bfloat16)
        cb = torch.randn(128 * 3, 64, generator=g, dtype=torch.bfloat16)
        w = torch.softmax(torch.randn(128, 3, generator=g), dim=-1)
        np.savez_compressed(os.path.join(HERE, "epilogues.npz"), y_shared=_u16(ys), combine=_u16(cb), w=w.numpy(),
                            fwd=_u16(U.run_fwd_epilogue_reference(ys, cb, w)),
                            bwd=_u16(U.run_bwd_epilogue_reference(ys, cb)))
    dist.barrier()
    dist.destroy_process_group()


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of the reference project>")
    ref_root = sys.argv[1]
    for i, ws in enumerate((1, 2)):
        mp.spawn(_worker, args=(ws, ref_root, 29610 + i), nprocs=ws, join=True)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
