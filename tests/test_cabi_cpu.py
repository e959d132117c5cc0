"""CPU-only checks: the C-ABI library loads and exports every symbol the header declares, rejects bad arguments
before touching a GPU, the Python layer mirrors the reference interface, and the expert-parallel partition logic
holds across two gloo ranks."""
import inspect
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from mok import _native as nat
    header = open(os.path.join(ROOT, "include", "mok_b200.h")).read()
    declared = sorted(set(re.findall(r"\b(mok_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) >= 14
    L = nat.lib()
    for name in declared:
        assert hasattr(L, name), f"{name} is declared in include/mok_b200.h but not exported"
    assert L.mok_version() >= 100


def test_entry_points_reject_bad_arguments_without_a_gpu():
    from mok import _native as nat
    L = nat.lib()
    assert L.mok_schedule(None, 1, 512, 1, 1, 512, 0, None, None, None, None, None, None, None) == -1
    assert L.mok_mxfp8_quantize(None, 1, 128, 128, None, None, None, None, None) == -1
    assert L.mok_fwd_epilogue(None, None, None, None, 512, 256, 1, None, None) == -1
    assert L.mok_bwd_epilogue(None, None, None, 512, 256, 1, None, None) == -1
    assert L.mok_barrier_all(None, None, 2, None, None, 0, None) == -1
    assert L.mok_schedule_dedup(None, 2, 512, 2, 4, 2048, 0, None, None, None, None, None, None, None, None, 1024, None, None) == -1
    assert L.mok_schedule_dedup_scratch_bytes(8, 32768, 8, 1048576) == 4 * (8 * 262144 + 1048576 + 4096)
    assert L.mok_stage_unique_rows(None, 2, 0, None, None, None, None, 0, 256, 512, 256, None, 0, 0, None, None) == -1
    assert L.mok_dispatch_rows_staged(None, None, 2, 0, None, None, None, None, None, 0, 0, 256, 2, 512, 256, None, None, 0, None,
                                      None) == -1
    assert L.mok_grouped_gemm_bf16(None, None, None, None, None, 1, 256, 256, 64, 0, None, None) == -1
    args = nat.LayerArgs()
    assert L.mok_moe_forward_bf16(nat.ctypes.byref(args), None) == -1
    assert L.mok_moe_backward_bf16(nat.ctypes.byref(args), None) == -1
    assert L.mok_schedule_scratch_bytes(8, 32768, 8, 32) == 4 * (8 * 256 * 32 + 32 * 8 + 32)


def test_layer_args_struct_matches_header_field_order():
    from mok import _native as nat
    header = open(os.path.join(ROOT, "include", "mok_b200.h")).read()
    body = header[header.index("typedef struct mok_layer_args {"):header.index("} mok_layer_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S).replace("typedef struct mok_layer_args {", "")
    names = []
    for stmt in body.split(";"):
        stmt = stmt.strip()
        if not stmt:
            continue
        for part in stmt.split(","):
            m = re.search(r"([A-Za-z_][A-Za-z0-9_]*)\s*$", part.strip())
            if m:
                names.append(m.group(1))
    assert names == [f[0] for f in nat.LayerArgs._fields_]


def test_python_surface_mirrors_the_reference_interface():
    import mok
    F = mok.functional
    cfg = F.MoKConfig()
    assert (cfg.fwd_num_comm_sms, cfg.bwd_num_comm_sms, cfg.minibatch_size, cfg.macrobatch_size,
            cfg.schedule_capacity_multiplier, cfg.all_gather_top_experts_chunk_bytes) == (40, 28, 4096, 131072, 0.5, 2048)
    for name in ("validate_workspace_args", "create_workspace", "get_workspace", "clear_workspace_cache", "build_schedule",
                 "validate_inputs", "forward", "recompute_forward_context", "backward", "MoKSchedule", "MoKForwardContext",
                 "MoKWorkspace"):
        assert hasattr(F, name)
    assert list(inspect.signature(F.forward).parameters) == [
        "config", "workspace", "schedule", "x", "router_weights", "shared_gate_weights", "shared_up_weights",
        "shared_down_weights", "routed_gate_weights", "routed_up_weights", "routed_down_weights", "swiglu_limit"]
    assert list(inspect.signature(F.backward).parameters)[:7] == [
        "config", "workspace", "schedule", "forward_context", "grad_output", "x", "router_weights"]
    ops = {"all_gather_top_experts": ("all_gather_top_experts_buffer",), "barrier_all": ("barrier_buffer", "target"),
           "schedule": (), "mxfp8_quantize": (), "fwd_epilogue": (), "bwd_epilogue": (),
           "dispatch_mlp_swiglu_combine_fwd_bf16": ("combine_buffer",), "recompute_forward_context_bf16": (),
           "dispatch_mlp_swiglu_combine_bwd_bf16": ("d_x_routed_buffer", "d_router_weight_buffer", "x_routed", "gate_routed",
                                                    "up_routed", "hidden_routed"),
           "dispatch_mlp_swiglu_combine_fwd_mxfp8": ("combine_buffer",), "recompute_forward_context_mxfp8": (),
           "dispatch_mlp_swiglu_combine_bwd_mxfp8": None}
    for name, mutated in ops.items():
        schema = getattr(torch.ops.mok, name).default._schema
        if mutated is not None:
            got = tuple(a.name for a in schema.arguments if a.alias_info is not None and a.alias_info.is_write)
            assert got == mutated, (name, got)


def test_fake_impls_give_the_documented_shapes():
    from torch._subclasses.fake_tensor import FakeTensorMode
    import mok  # noqa: F401
    with FakeTensorMode():
        topk_all = torch.empty(2, 512, 4, dtype=torch.int32)
        pr, pt, nt, tpe = torch.ops.mok.schedule(topk_all, 8, 4096, 1)
        assert pr.shape == (4096,) and pt.shape == (4096,) and nt.shape == (1,) and tpe.shape == (8,)
        x = torch.empty(3, 256, 384, dtype=torch.bfloat16)
        q, sc, qt, sct = torch.ops.mok.mxfp8_quantize(x, True, True)
        assert q.shape == (3, 256, 384) and sc.shape == (6, 3, 32, 16) and qt.shape == (3, 384, 256) and sct.shape == (9, 2, 32, 16)
        assert q.dtype == torch.float8_e4m3fn and sc.dtype == torch.uint8
        rs, up, ut, ub, nu = torch.ops.mok.schedule_dedup(topk_all, pr, pt, nt, 8, 1)
        assert rs.shape == (4096,) and up.shape == ut.shape == (1024,) and ub.shape == (17,) and nu.shape == (1,)


def _gloo_rank(rank, world, port, out):
    import torch.distributed as dist
    from oracle import moe_oracle as O
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    T, K, E = 512, 3, 8
    g = torch.Generator().manual_seed(77 + rank)
    mine = torch.topk(torch.randn(T, E, generator=g), K, dim=1).indices.to(torch.int32)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine)
    topk_all = torch.stack(gathered).numpy()
    pr, pt, nt, tpe = O.schedule_oracle(topk_all, E // world, T * K * 2, rank)
    valid = pr >= 0
    # every row names a route whose expert lives on this rank
    assert ((topk_all.reshape(world, -1)[pr[valid], pt[valid]] // (E // world)) == rank).all()
    assert int(nt[0]) == int(tpe.sum()) and (tpe % 256 == 0).all()
    counts = torch.tensor([int(valid.sum())])
    dist.all_reduce(counts)
    if rank == 0:
        out.put(int(counts.item()) == world * T * K)    # the ranks' schedules partition all routes
    dist.destroy_process_group()


def test_schedules_of_two_gloo_ranks_partition_all_routes():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, 29655, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert q.get(timeout=5) is True


def test_functional_argument_checks_on_cpu():
    import mok
    F = mok.functional
    with pytest.raises(ValueError, match="schedule_capacity_multiplier"):
        F.validate_workspace_args(F.MoKConfig(schedule_capacity_multiplier=0.0), None, device=torch.device("cpu"),
                                  num_local_tokens=512, hidden_size=256, topk=1)
    with pytest.raises(RuntimeError, match="torch.distributed must be initialized"):
        F.validate_workspace_args(F.MoKConfig(), None, device=torch.device("cpu"), num_local_tokens=512, hidden_size=256, topk=1)
    with pytest.raises(TypeError):
        F.build_schedule(object(), F.MoKConfig(), torch.zeros(1), num_local_experts=1)
    with pytest.raises(TypeError):
        F.validate_inputs(object(), None, None, torch.zeros(1))
    assert np.array_equal(mok.ops.SUPPORTED_EP_SIZES, (1, 2, 4, 8))


def test_header_is_plain_c():
    """The boundary is a C ABI: the header must compile as C99 (no C++ or torch types in any signature)."""
    import shutil
    import subprocess
    if shutil.which("gcc") is None:
        pytest.skip("no C compiler")
    header = os.path.join(ROOT, "include", "mok_b200.h")
    r = subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-Werror", "-fsyntax-only", "-x", "c", header],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
