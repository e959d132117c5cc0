"""CPU checks of bench.py: the reference arm (the CPU restatement timed on the host cores) prints one well-formed JSON
line, the FLOP formula is the reference's, and the GPU arm refuses to run without a GPU instead of falling back."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, capture_output=True, text=True,
                          timeout=300)


def test_reference_arm_prints_one_json_line():
    r = _run("--impl", "reference", "--workload", "tiny", "--steps", "1", "--warmup", "0")
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    line = json.loads(lines[0])
    assert line["impl"] == "reference" and line["metric"] == "moe_layer_fwd_bwd_tokens_per_s" and line["unit"] == "tokens/s"
    assert line["higher_is_better"] is True and line["n_gpus"] == 1 and line["steps"] == 1 and line["value"] > 0
    # the arm says what it timed: a bounded sample, with the sample's own token and expert counts
    assert line["config"]["workload"].startswith("tiny: bounded CPU sample")
    assert line["config"]["tokens_per_rank"] * line["ms_per_step"] > 0 and line["config"]["host_threads"] == line["cpu_baseline"]["cores"]
    base = line["cpu_baseline"]
    assert base["kind"] == "port" and base["cores"] >= 1 and base["value"] == line["value"] and base["sample"]
    assert line["e2e"] == {"value": line["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    assert line["gpu_launches"] == 0


def test_reference_arm_runs_on_rank_zero_only():
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "tiny", "--gpus", "2",
                        "--steps", "1", "--warmup", "0"], cwd=ROOT, capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0 and not [l for l in r.stdout.splitlines() if l.startswith("{")]


def test_flop_formula_counts_routed_and_shared_experts():
    sys.path.insert(0, ROOT)
    import bench
    w = bench.WORKLOADS["c2"]
    # 3 GEMMs forward + 6 backward, 2*H*I FLOP each, for the K routed experts and the shared one (reference README formula)
    assert bench.flops_per_token(w) == 18 * (8 + 1) * 7168 * 2048
    assert w["T"] == 32768 and w["E"] == 256


def test_gpu_arm_fails_loudly_without_a_gpu():
    import torch
    if torch.cuda.is_available():
        return
    r = _run("--workload", "tiny", "--steps", "1", "--warmup", "1", "--no-cpu")
    assert r.returncode != 0
    assert not [l for l in r.stdout.splitlines() if l.startswith("{")]


def test_sampled_parity_checker_agrees_with_the_whole_layer_oracle():
    """bench.py's sampled check (a few tokens, one or two experts, rank 0's schedule) fed with the results of the
    whole-layer oracle for a two-rank case must report agreement; fed with a corrupted row it must not.  This pins
    the checker's own gathering logic (rows of an expert from every source rank, other ranks' experts redrawn from
    their seeds) on the CPU, in both precisions."""
    import types
    import numpy as np
    import torch
    sys.path.insert(0, ROOT)
    import bench
    from oracle import moe_oracle as O
    w = bench.WORKLOADS["tiny"]
    dev, world = torch.device("cpu"), 2
    e_loc = w["E"] // world
    capacity = w["T"] * w["K"] * 2
    router = bench.router_parameters(w, dev)
    acts = [bench.make_activations(w, r, dev, router) for r in range(world)]
    wts = [bench.make_weights(w, e_loc, r, dev) for r in range(world)]
    ranks = [O.RankInputs(a[0], a[2], a[3], *wt, a[1]) for a, wt in zip(acts, wts)]
    topk_all = np.stack([a[2].to(torch.int32).numpy() for a in acts])
    pr, pt, nt, tpe = O.schedule_oracle(topk_all, e_loc, capacity, 0)
    sched = types.SimpleNamespace(peer_rank=torch.from_numpy(pr), peer_token_idx=torch.from_numpy(pt),
                                  num_tokens=torch.from_numpy(nt), tokens_per_expert=torch.from_numpy(tpe))
    case = types.SimpleNamespace(w=w, dev=dev, world=world, rank=0, e_loc=e_loc, capacity=capacity, router=router,
                                 x=acts[0][0], dy=acts[0][1], topk=acts[0][2], rw=acts[0][3], weights=wts[0])
    for mxfp8 in (False, True):
        ref = O.moe_layer_oracle(ranks, mxfp8=mxfp8)[0]
        grads = [ref.d_x, ref.d_router_weights, ref.d_w_routed_gate, ref.d_w_routed_up, ref.d_w_routed_down]
        good = bench.sampled_parity(case, mxfp8, sched, ref.output, grads, n_tokens=3)
        assert good["schedule_exact"] and good["ok"] and good["rel_l2_max"] < 2e-3, good
        assert good["tokens_checked"] == 3 and good["experts_checked"] == 2 and min(good["expert_rows"]) > 0
        broken = ref.output.clone()
        broken[0] += 1.0
        bad = bench.sampled_parity(case, mxfp8, sched, broken, grads, n_tokens=3)
        assert not bad["ok"] and bad["rel_l2"]["output"] > good["tolerance"]
    shifted = types.SimpleNamespace(**{**vars(sched), "peer_token_idx": sched.peer_token_idx.roll(1)})
    assert not bench.sampled_parity(case, False, shifted, ref.output, grads, n_tokens=1)["schedule_exact"]
