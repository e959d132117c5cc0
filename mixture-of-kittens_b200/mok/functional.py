"""Orchestration layer of the MoE kernel library: configuration, symmetric workspaces, schedules, and the
forward / recompute / backward call sequences.

The public names, signatures, defaults, argument checks and return orders follow the reference
`mok/functional.py` (citations below are lines of that file) so existing callers work unchanged.  What differs:
EP sizes 1, 2, 4, 8 are accepted; peers are reached through per-rank addresses only (no multicast object is
required — when the symmetric-memory backend offers none, the two `*_multicast_ptr` fields hold the local
address); kernels report problems through `mok.ops.check_status()` instead of trapping.
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist

from . import ops as _ops
from .ops import (
    all_gather_top_experts,
    barrier_all,
    bwd_epilogue,
    dispatch_mlp_swiglu_combine_bwd_bf16,
    dispatch_mlp_swiglu_combine_bwd_mxfp8,
    dispatch_mlp_swiglu_combine_fwd_bf16,
    dispatch_mlp_swiglu_combine_fwd_mxfp8,
    fwd_epilogue,
    recompute_forward_context_bf16,
    recompute_forward_context_mxfp8,
    schedule,
    schedule_dedup,
)

SUPPORTED_EP_SIZES = _ops.SUPPORTED_EP_SIZES


@dataclass(frozen=True, slots=True)
class MoKConfig:                       # reference :24-31
    fwd_num_comm_sms: int = 40
    bwd_num_comm_sms: int = 28
    minibatch_size: int = 4096
    macrobatch_size: int = 131072
    schedule_capacity_multiplier: float = 0.5
    all_gather_top_experts_chunk_bytes: int = 2048


@dataclass(frozen=True, slots=True)
class MoKSchedule:                     # reference :34-39
    peer_rank: torch.Tensor          # (schedule_capacity,) int32, -1 on padding rows
    peer_token_idx: torch.Tensor     # (schedule_capacity,) int32, token * topk + k on the source rank
    num_tokens: torch.Tensor         # (1,) int32, padded total (stays on the device)
    tokens_per_expert: torch.Tensor  # (num_local_experts,) int32, each padded to 256
    # De-duplicated dispatch (not in the reference, whose dispatch pulls a token once per route): built for EP > 1 when
    # a token has two or more routes per rank on average (see `_dedup_wanted`).  Every (source rank, token) this rank
    # serves is numbered in the order of its first row.
    row_source: torch.Tensor | None = None      # (schedule_capacity,) int32 number of the row's token, -1 on padding rows
    unique_peer: torch.Tensor | None = None     # (U,) int32 source rank of staged token u
    unique_token: torch.Tensor | None = None    # (U,) int32 its token index on that rank
    unique_before: torch.Tensor | None = None   # (schedule_capacity / 256 + 1,) int32 tokens first used below row 256 * i
    num_unique: torch.Tensor | None = None      # (1,) int32


@dataclass(frozen=True, slots=True)
class MoKForwardContext:               # reference :42-50
    x_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    gate_shared: torch.Tensor
    gate_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    up_shared: torch.Tensor
    up_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]
    hidden_shared: torch.Tensor
    hidden_routed: torch.Tensor | tuple[torch.Tensor, torch.Tensor]


@dataclass(slots=True)
class MoKWorkspace:                    # reference :53-88 (same fields, same order; one more at the end)
    group_name: str
    ep_rank: int
    ep_size: int
    device: torch.device
    num_local_tokens: int
    hidden_size: int
    topk: int
    schedule_capacity: int
    x_buffer: torch.Tensor                            # (T, H) bfloat16
    x_buffer_handle: Any
    x_buffer_ptrs: list[int]
    combine_buffer: torch.Tensor                      # (T * topk, H) bfloat16
    combine_buffer_handle: Any
    combine_buffer_ptrs: list[int]
    d_y_buffer: torch.Tensor                          # (T, H) bfloat16
    d_y_buffer_handle: Any
    d_y_buffer_ptrs: list[int]
    d_x_routed_buffer: torch.Tensor                   # (T * topk, H) bfloat16
    d_x_routed_buffer_handle: Any
    d_x_routed_buffer_ptrs: list[int]
    router_weight_buffer: torch.Tensor                # (T, topk) float32
    router_weight_buffer_handle: Any
    router_weight_buffer_ptrs: list[int]
    d_router_weight_buffer: torch.Tensor              # (T, topk) float32
    d_router_weight_buffer_handle: Any
    d_router_weight_buffer_ptrs: list[int]
    all_gather_top_experts_buffer: torch.Tensor       # (ep_size, T, topk) int32
    all_gather_top_experts_buffer_handle: Any
    all_gather_top_experts_buffer_multicast_ptr: int
    barrier_buffer: torch.Tensor                      # (1,) int32
    barrier_buffer_handle: Any
    barrier_buffer_ptrs: list[int]
    barrier_buffer_multicast_ptr: int
    barrier_target: torch.Tensor                      # (1,) int32
    # every rank's address of the route gather buffer (unicast all-gather; the reference reaches peers through the
    # multicast address alone and has no such field)
    all_gather_top_experts_buffer_ptrs: list[int] = field(default_factory=list)


_WORKSPACE_CACHE: dict[tuple[str, int, int, int, int, int], MoKWorkspace] = {}


def _capacity_factor(config: MoKConfig, ep_size: int) -> int:
    return max(2, math.ceil(ep_size * config.schedule_capacity_multiplier))


def validate_workspace_args(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device, num_local_tokens: int,
                            hidden_size: int, topk: int) -> None:
    """Checks the arguments used to create or look up a workspace (reference :94-159)."""
    mult = config.schedule_capacity_multiplier
    if type(mult) not in (int, float) or not math.isfinite(mult) or mult <= 0:
        raise ValueError("schedule_capacity_multiplier must be a positive finite number")
    if not dist.is_initialized():
        raise RuntimeError("torch.distributed must be initialized")
    if not isinstance(group, dist.ProcessGroup):
        raise TypeError("group must be a torch.distributed.ProcessGroup")
    if not isinstance(device, torch.device):
        raise TypeError("device must be a torch.device")
    if device.type != "cuda":
        raise ValueError("device must be a CUDA device")
    index = device.index if device.index is not None else torch.cuda.current_device()
    if index != torch.cuda.current_device():
        raise ValueError("MoK workspace device must be the current CUDA device")
    if torch.cuda.get_device_capability(index) not in ((10, 0), (10, 3)):
        raise NotImplementedError("MoK currently requires an SM100 or SM103 GPU")
    if type(num_local_tokens) is not int or num_local_tokens < 512:
        raise ValueError("num_local_tokens must be an integer at least 512")
    if num_local_tokens % 256 != 0:
        raise ValueError("num_local_tokens must be divisible by 256")
    if type(hidden_size) is not int or hidden_size <= 0:
        raise ValueError("hidden_size must be a positive integer")
    if hidden_size % 256 != 0:
        raise ValueError("hidden_size must be divisible by 256")
    if type(topk) is not int or not 0 < topk <= 255:
        raise ValueError("topk must be an integer in [1, 255]")
    group_name = group.group_name
    if not isinstance(group_name, str) or not group_name:
        raise RuntimeError("process group must have a nonempty group_name")
    ep_rank = dist.get_rank(group=group)
    ep_size = dist.get_world_size(group=group)
    if ep_size not in SUPPORTED_EP_SIZES:
        raise ValueError(f"MoK EP size must be one of {', '.join(map(str, SUPPORTED_EP_SIZES))}")
    if not 0 <= ep_rank < ep_size:
        raise RuntimeError("current process is not a member of the EP process group")


def create_workspace(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device, num_local_tokens: int,
                     hidden_size: int, topk: int) -> MoKWorkspace:
    """Allocates a caller-owned workspace: eight buffers every EP rank can address (reference :162-276)."""
    validate_workspace_args(config, group, device=device, num_local_tokens=num_local_tokens, hidden_size=hidden_size, topk=topk)
    index = device.index if device.index is not None else torch.cuda.current_device()
    device = torch.device("cuda", index)
    group_name = group.group_name
    ep_rank = dist.get_rank(group=group)
    ep_size = dist.get_world_size(group=group)

    local_shape = torch.tensor([num_local_tokens, hidden_size, topk], dtype=torch.int64, device=device)
    gathered = torch.empty(ep_size * 3, dtype=torch.int64, device=device)
    dist.all_gather_into_tensor(gathered, local_shape, group=group)
    if not torch.all(gathered.view(ep_size, 3) == local_shape).item():   # one-time set-up, a host sync is fine here
        raise ValueError("MoK requires identical token, hidden, and top-k shapes on every EP rank")

    symm_mem = None
    if ep_size > 1:
        import warnings
        import torch.distributed._symmetric_memory as symm_mem
        enable = getattr(symm_mem, "enable_symm_mem_for_group", None)   # newer PyTorch enables groups on first use
        if enable is not None:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore", FutureWarning)
                enable(group_name)
    schedule_capacity = num_local_tokens * topk * _capacity_factor(config, ep_size)

    def allocate(*shape: int, dtype: torch.dtype, zero: bool = False):
        if ep_size == 1:
            buffer = (torch.zeros if zero else torch.empty)(*shape, dtype=dtype, device=device)
            return buffer, None, [int(buffer.data_ptr())]
        buffer = symm_mem.empty(*shape, dtype=dtype, device=device)
        if zero:
            buffer.zero_()
        handle = symm_mem.rendezvous(buffer, group_name)
        return buffer, handle, [int(handle.buffer_ptrs[peer]) for peer in range(ep_size)]

    def multicast_or_local(buffer: torch.Tensor, handle: Any) -> int:
        mc = 0 if handle is None else int(getattr(handle, "multicast_ptr", 0) or 0)
        return mc if mc > 0 else int(buffer.data_ptr())

    x_buffer, x_handle, x_ptrs = allocate(num_local_tokens, hidden_size, dtype=torch.bfloat16)
    combine_buffer, combine_handle, combine_ptrs = allocate(num_local_tokens * topk, hidden_size, dtype=torch.bfloat16)
    d_y_buffer, d_y_handle, d_y_ptrs = allocate(num_local_tokens, hidden_size, dtype=torch.bfloat16)
    d_x_routed_buffer, d_x_routed_handle, d_x_routed_ptrs = allocate(num_local_tokens * topk, hidden_size, dtype=torch.bfloat16)
    rw_buffer, rw_handle, rw_ptrs = allocate(num_local_tokens, topk, dtype=torch.float32)
    drw_buffer, drw_handle, drw_ptrs = allocate(num_local_tokens, topk, dtype=torch.float32)
    ag_buffer, ag_handle, ag_ptrs = allocate(ep_size, num_local_tokens, topk, dtype=torch.int32)
    barrier_buffer, barrier_handle, barrier_ptrs = allocate(1, dtype=torch.int32, zero=True)
    barrier_target = torch.zeros(1, dtype=torch.int32, device=device)
    _ops.register_all_gather_peers(ag_buffer, ag_ptrs)   # for callers of the five-argument op; dies with the buffer

    dist.barrier(group=group, async_op=True, device_ids=[index]).block_current_stream()

    return MoKWorkspace(
        group_name=group_name, ep_rank=ep_rank, ep_size=ep_size, device=device,
        num_local_tokens=num_local_tokens, hidden_size=hidden_size, topk=topk, schedule_capacity=schedule_capacity,
        x_buffer=x_buffer, x_buffer_handle=x_handle, x_buffer_ptrs=x_ptrs,
        combine_buffer=combine_buffer, combine_buffer_handle=combine_handle, combine_buffer_ptrs=combine_ptrs,
        d_y_buffer=d_y_buffer, d_y_buffer_handle=d_y_handle, d_y_buffer_ptrs=d_y_ptrs,
        d_x_routed_buffer=d_x_routed_buffer, d_x_routed_buffer_handle=d_x_routed_handle, d_x_routed_buffer_ptrs=d_x_routed_ptrs,
        router_weight_buffer=rw_buffer, router_weight_buffer_handle=rw_handle, router_weight_buffer_ptrs=rw_ptrs,
        d_router_weight_buffer=drw_buffer, d_router_weight_buffer_handle=drw_handle, d_router_weight_buffer_ptrs=drw_ptrs,
        all_gather_top_experts_buffer=ag_buffer, all_gather_top_experts_buffer_handle=ag_handle,
        all_gather_top_experts_buffer_multicast_ptr=multicast_or_local(ag_buffer, ag_handle),
        barrier_buffer=barrier_buffer, barrier_buffer_handle=barrier_handle, barrier_buffer_ptrs=barrier_ptrs,
        barrier_buffer_multicast_ptr=multicast_or_local(barrier_buffer, barrier_handle),
        barrier_target=barrier_target, all_gather_top_experts_buffer_ptrs=ag_ptrs,
    )


def get_workspace(config: MoKConfig, group: dist.ProcessGroup, *, device: torch.device, num_local_tokens: int,
                  hidden_size: int, topk: int) -> MoKWorkspace:
    """Returns the cached workspace for these sizes, creating it on first use (reference :279-330)."""
    validate_workspace_args(config, group, device=device, num_local_tokens=num_local_tokens, hidden_size=hidden_size, topk=topk)
    index = device.index if device.index is not None else torch.cuda.current_device()
    key = (group.group_name, index, num_local_tokens, hidden_size, topk,
           _capacity_factor(config, dist.get_world_size(group=group)))
    workspace = _WORKSPACE_CACHE.get(key)
    if workspace is None:
        workspace = create_workspace(config, group, device=torch.device("cuda", index), num_local_tokens=num_local_tokens,
                                     hidden_size=hidden_size, topk=topk)
        _WORKSPACE_CACHE[key] = workspace
    return workspace


def _stage(buffer: torch.Tensor, value: torch.Tensor) -> None:
    """Copies an input into its symmetric buffer unless the caller already produced it there (pass the workspace
    buffer itself as the argument to skip the copy; the reference marks these copies as removable, :509,:709-711)."""
    if value is not buffer:
        buffer.copy_(value)


def _barrier(workspace: MoKWorkspace) -> None:
    barrier_all(workspace.barrier_buffer, workspace.barrier_buffer_ptrs, workspace.barrier_buffer_multicast_ptr,
                workspace.barrier_target)


def clear_workspace_cache() -> None:
    """Drops the cached workspaces after every participating rank has reached this point (reference :333-346)."""
    for workspace in _WORKSPACE_CACHE.values():
        _barrier(workspace)
        torch.cuda.synchronize(workspace.device)
        _ops.unregister_all_gather_peers(workspace.all_gather_top_experts_buffer)
    _WORKSPACE_CACHE.clear()


def _dedup_wanted(workspace: MoKWorkspace) -> bool:
    """Whether dispatch stages every token once per destination rank and fans it out locally (`schedule_dedup`) or
    pulls row by row as the reference does.  Staging saves NVLink bytes and costs one more local pass over the rows; it
    is switched on when a token has on average at least two routes per destination rank (topk >= 2 * ep_size: half or
    more of the pulls disappear).  Measured on the DeepSeek-V3-shaped layer: EP 2 / top-8 79.8 ms against 81.0 ms
    row by row; EP 8 / top-8 (one route per rank on average, a third of the pulls saved) 85.7 - 88.0 ms against 84.3 ms.
    MOK_DEDUP=1 / MOK_DEDUP=0 force it on / off."""
    if workspace.ep_size == 1:
        return False
    forced = os.environ.get("MOK_DEDUP")
    if forced in ("0", "1"):
        return forced == "1"
    return workspace.topk >= 2 * workspace.ep_size


def build_schedule(workspace: MoKWorkspace, config: MoKConfig, top_experts: torch.Tensor, *, num_local_experts: int) -> MoKSchedule:
    """All-gathers the routing choices and builds this rank's padded expert schedule (reference :349-425).

    Inputs:  top_experts int64 [num_local_tokens, topk]
    Outputs: MoKSchedule (all tensors stay on the device; nothing is read back)
    """
    if not isinstance(workspace, MoKWorkspace):
        raise TypeError("workspace must be a MoKWorkspace")
    if not isinstance(config, MoKConfig):
        raise TypeError("config must be a MoKConfig")
    sm_total = torch.cuda.get_device_properties(workspace.device).multi_processor_count
    for name in ("fwd_num_comm_sms", "bwd_num_comm_sms"):
        value = getattr(config, name)
        if type(value) is not int or value <= 0:
            raise ValueError(f"{name} must be a positive integer")
        if value % 2 != 0:
            raise ValueError(f"{name} must be even")
    if config.fwd_num_comm_sms >= sm_total or config.bwd_num_comm_sms >= sm_total:
        raise ValueError("communication-SM counts must leave at least one compute SM")
    if type(config.minibatch_size) is not int or config.minibatch_size <= 0 or config.minibatch_size % 256 != 0:
        raise ValueError("minibatch_size must be positive and divisible by 256")
    if (type(config.macrobatch_size) is not int or config.macrobatch_size <= 0
            or config.macrobatch_size % config.minibatch_size != 0):
        raise ValueError("macrobatch_size must be a positive multiple of minibatch_size")
    chunk = config.all_gather_top_experts_chunk_bytes
    if type(chunk) is not int or chunk <= 0 or chunk % 16 != 0:
        raise ValueError("all_gather_top_experts_chunk_bytes must be a positive multiple of 16")
    if (workspace.num_local_tokens * workspace.topk * 4) % chunk != 0:
        raise ValueError("all_gather_top_experts_chunk_bytes must divide one rank's route-buffer bytes")
    if not top_experts.is_cuda or top_experts.device != workspace.device:
        raise ValueError("top_experts must be on the workspace CUDA device")
    if top_experts.dtype not in (torch.int64, torch.int32):   # int32 (what the device router writes) skips a conversion
        raise TypeError("top_experts must have dtype torch.int64 (or torch.int32)")
    if not top_experts.is_contiguous():
        raise ValueError("top_experts must be contiguous")
    if tuple(top_experts.shape) != (workspace.num_local_tokens, workspace.topk):
        raise ValueError("top_experts must have shape (num_local_tokens, topk)")
    if type(num_local_experts) is not int or num_local_experts <= 0:
        raise ValueError("num_local_experts must be a positive integer")

    routes = top_experts if top_experts.dtype == torch.int32 else top_experts.to(torch.int32)
    all_gather_top_experts(routes, workspace.all_gather_top_experts_buffer,
                           workspace.all_gather_top_experts_buffer_multicast_ptr, workspace.ep_rank, chunk,
                           workspace.all_gather_top_experts_buffer_ptrs or None)
    _barrier(workspace)
    peer_rank, peer_token_idx, num_tokens, tokens_per_expert = schedule(
        workspace.all_gather_top_experts_buffer, num_local_experts, workspace.schedule_capacity, workspace.ep_rank)
    if not _dedup_wanted(workspace):
        return MoKSchedule(peer_rank=peer_rank, peer_token_idx=peer_token_idx, num_tokens=num_tokens,
                           tokens_per_expert=tokens_per_expert)
    row_source, unique_peer, unique_token, unique_before, num_unique = schedule_dedup(
        workspace.all_gather_top_experts_buffer, peer_rank, peer_token_idx, num_tokens, num_local_experts, workspace.ep_rank)
    return MoKSchedule(peer_rank=peer_rank, peer_token_idx=peer_token_idx, num_tokens=num_tokens,
                       tokens_per_expert=tokens_per_expert, row_source=row_source, unique_peer=unique_peer,
                       unique_token=unique_token, unique_before=unique_before, num_unique=num_unique)


def validate_inputs(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, x: torch.Tensor,
                    router_weights: torch.Tensor | None = None, grad_output: torch.Tensor | None = None) -> None:
    """Checks runtime inputs against the workspace and schedule (reference :428-467)."""
    if not isinstance(config, MoKConfig):
        raise TypeError("config must be a MoKConfig")
    if not isinstance(workspace, MoKWorkspace):
        raise TypeError("workspace must be a MoKWorkspace")
    if not isinstance(schedule, MoKSchedule):
        raise TypeError("schedule must be a MoKSchedule")
    act_shape = (workspace.num_local_tokens, workspace.hidden_size)
    checks = [("x", x, torch.bfloat16, act_shape)]
    if grad_output is not None:
        checks.append(("grad_output", grad_output, torch.bfloat16, act_shape))
    if router_weights is not None:
        checks.append(("router_weights", router_weights, torch.float32, (workspace.num_local_tokens, workspace.topk)))
    for name, tensor, dtype, shape in checks:
        if not tensor.is_cuda or tensor.device != workspace.device or tensor.dtype != dtype or not tensor.is_contiguous():
            raise ValueError(f"{name} must be contiguous {dtype} on the workspace CUDA device")
        if tuple(tensor.shape) != shape:
            raise ValueError(f"{name} shape does not match the workspace")
    if schedule.peer_rank.numel() != workspace.schedule_capacity:
        raise ValueError("schedule capacity does not match the workspace")


def forward(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, x: torch.Tensor, router_weights: torch.Tensor,
            shared_gate_weights: torch.Tensor, shared_up_weights: torch.Tensor, shared_down_weights: torch.Tensor,
            routed_gate_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
            routed_up_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
            routed_down_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
            swiglu_limit: float | None = None) -> tuple[torch.Tensor, MoKForwardContext]:
    """MoE forward (reference :470-568).  Returns (output bf16 [T, H], forward context for backward)."""
    validate_inputs(config, workspace, schedule, x, router_weights)
    _stage(workspace.x_buffer, x)
    _stage(workspace.router_weight_buffer, router_weights)
    _barrier(workspace)   # every peer's x is in place before anyone pulls

    sched = (schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert)
    tail = (workspace.topk, swiglu_limit, config.fwd_num_comm_sms, config.macrobatch_size, config.minibatch_size,
            schedule.row_source, schedule.unique_peer, schedule.unique_token, schedule.unique_before)
    if isinstance(routed_gate_weights, tuple):
        g_fp8, g_sc = routed_gate_weights
        u_fp8, u_sc = routed_up_weights
        d_fp8, d_sc = routed_down_weights
        (x_t, x_t_sc, gate_shared, gate_q, gate_sc, up_shared, up_q, up_sc, hidden_shared, hid_t, hid_t_sc,
         y_shared, _y_routed) = dispatch_mlp_swiglu_combine_fwd_mxfp8(
            workspace.x_buffer, workspace.x_buffer_ptrs, workspace.combine_buffer, workspace.combine_buffer_ptrs,
            shared_gate_weights, g_fp8, g_sc, shared_up_weights, u_fp8, u_sc, shared_down_weights, d_fp8, d_sc, *sched, *tail)
        context = MoKForwardContext(x_routed=(x_t, x_t_sc), gate_shared=gate_shared, gate_routed=(gate_q, gate_sc),
                                    up_shared=up_shared, up_routed=(up_q, up_sc), hidden_shared=hidden_shared,
                                    hidden_routed=(hid_t, hid_t_sc))
    else:
        (x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared, hidden_routed, y_shared,
         _y_routed) = dispatch_mlp_swiglu_combine_fwd_bf16(
            workspace.x_buffer, workspace.x_buffer_ptrs, workspace.combine_buffer, workspace.combine_buffer_ptrs,
            shared_gate_weights, routed_gate_weights, shared_up_weights, routed_up_weights,
            shared_down_weights, routed_down_weights, *sched, *tail)
        context = MoKForwardContext(x_routed=x_routed, gate_shared=gate_shared, gate_routed=gate_routed, up_shared=up_shared,
                                    up_routed=up_routed, hidden_shared=hidden_shared, hidden_routed=hidden_routed)

    _barrier(workspace)   # every peer's pushes into this rank's combine buffer have landed
    output = fwd_epilogue(y_shared, workspace.combine_buffer, workspace.router_weight_buffer)
    return output, context


def recompute_forward_context(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, x: torch.Tensor,
                              shared_gate_weights: torch.Tensor, shared_up_weights: torch.Tensor,
                              routed_gate_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
                              routed_up_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
                              swiglu_limit: float | None = None) -> MoKForwardContext:
    """Recomputes the activations backward needs, for manual activation checkpointing (reference :571-649)."""
    validate_inputs(config, workspace, schedule, x)
    if isinstance(routed_gate_weights, tuple) != isinstance(routed_up_weights, tuple):
        raise TypeError("routed gate and up weights must use the same precision representation")
    if isinstance(routed_gate_weights, tuple) and (len(routed_gate_weights) != 2 or len(routed_up_weights) != 2):
        raise ValueError("MXFP8 routed gate and up weights must be data/scale pairs")
    _stage(workspace.x_buffer, x)
    _barrier(workspace)

    sched = (schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert)
    tail = (workspace.topk, swiglu_limit, config.fwd_num_comm_sms, config.macrobatch_size, config.minibatch_size,
            schedule.row_source, schedule.unique_peer, schedule.unique_token, schedule.unique_before)
    if isinstance(routed_gate_weights, tuple):
        g_fp8, g_sc = routed_gate_weights
        u_fp8, u_sc = routed_up_weights
        (x_t, x_t_sc, gate_shared, gate_q, gate_sc, up_shared, up_q, up_sc, hidden_shared, hid_t,
         hid_t_sc) = recompute_forward_context_mxfp8(workspace.x_buffer, workspace.x_buffer_ptrs, shared_gate_weights, g_fp8, g_sc,
                                                     shared_up_weights, u_fp8, u_sc, *sched, *tail)
        x_routed, gate_routed, up_routed, hidden_routed = (x_t, x_t_sc), (gate_q, gate_sc), (up_q, up_sc), (hid_t, hid_t_sc)
    else:
        (x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared,
         hidden_routed) = recompute_forward_context_bf16(workspace.x_buffer, workspace.x_buffer_ptrs, shared_gate_weights,
                                                         routed_gate_weights, shared_up_weights, routed_up_weights, *sched, *tail)
    _barrier(workspace)
    return MoKForwardContext(x_routed=x_routed, gate_shared=gate_shared, gate_routed=gate_routed, up_shared=up_shared,
                             up_routed=up_routed, hidden_shared=hidden_shared, hidden_routed=hidden_routed)


def backward(config: MoKConfig, workspace: MoKWorkspace, schedule: MoKSchedule, forward_context: MoKForwardContext,
             grad_output: torch.Tensor, x: torch.Tensor, router_weights: torch.Tensor,
             shared_gate_weights: torch.Tensor, shared_up_weights: torch.Tensor, shared_down_weights: torch.Tensor,
             routed_gate_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor],
             routed_up_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor],
             routed_down_weights: torch.Tensor | tuple[torch.Tensor, torch.Tensor],
             swiglu_limit: float | None = None, *, router_grad_view: bool = False) -> tuple[torch.Tensor, ...]:
    """MoE backward (reference :652-780).

    Returns (d_x, d_router_weights, d_routed_gate_weights, d_routed_up_weights, d_routed_down_weights,
             d_shared_gate_weights, d_shared_up_weights, d_shared_down_weights).

    The peers write this rank's router-weight gradients into `workspace.d_router_weight_buffer`.  By default a copy
    is returned, as the reference does (:778, which marks the copy as removable); with `router_grad_view=True` the
    buffer itself is returned and stays valid until the next `backward` on this workspace overwrites it.
    """
    validate_inputs(config, workspace, schedule, x, router_weights, grad_output)
    if not isinstance(forward_context, MoKForwardContext):
        raise TypeError("forward_context must be a MoKForwardContext")
    _stage(workspace.d_y_buffer, grad_output)
    _stage(workspace.x_buffer, x)
    _stage(workspace.router_weight_buffer, router_weights)
    _barrier(workspace)

    bufs = (workspace.d_y_buffer, workspace.d_y_buffer_ptrs, workspace.d_x_routed_buffer, workspace.d_x_routed_buffer_ptrs,
            workspace.router_weight_buffer, workspace.router_weight_buffer_ptrs,
            workspace.d_router_weight_buffer, workspace.d_router_weight_buffer_ptrs)
    sched = (schedule.peer_rank, schedule.peer_token_idx, schedule.num_tokens, schedule.tokens_per_expert)
    tail = (workspace.topk, swiglu_limit, config.bwd_num_comm_sms, config.macrobatch_size, config.minibatch_size,
            schedule.row_source, schedule.unique_peer, schedule.unique_token, schedule.unique_before)
    ctx = forward_context
    if isinstance(routed_gate_weights, tuple):
        g_fp8, g_sc, g_t_fp8, g_t_sc = routed_gate_weights
        u_fp8, u_sc, u_t_fp8, u_t_sc = routed_up_weights
        d_t_fp8, d_t_sc = routed_down_weights
        out = dispatch_mlp_swiglu_combine_bwd_mxfp8(
            *bufs, shared_gate_weights, g_t_fp8, g_t_sc, shared_up_weights, u_t_fp8, u_t_sc, shared_down_weights, d_t_fp8, d_t_sc,
            *ctx.x_routed, ctx.gate_shared, *ctx.gate_routed, ctx.up_shared, *ctx.up_routed, ctx.hidden_shared, *ctx.hidden_routed,
            workspace.x_buffer, workspace.x_buffer_ptrs, g_fp8, g_sc, u_fp8, u_sc, *sched, *tail)
        d_x_shared = out[0]
        d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down, d_w_routed_down = out[12:18]
    else:
        out = dispatch_mlp_swiglu_combine_bwd_bf16(
            *bufs, shared_gate_weights, routed_gate_weights, shared_up_weights, routed_up_weights,
            shared_down_weights, routed_down_weights,
            ctx.x_routed, ctx.gate_shared, ctx.gate_routed, ctx.up_shared, ctx.up_routed, ctx.hidden_shared, ctx.hidden_routed,
            workspace.x_buffer, workspace.x_buffer_ptrs, *sched, *tail)
        d_x_shared = out[0]
        d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down, d_w_routed_down = out[9:15]

    _barrier(workspace)
    d_x = bwd_epilogue(d_x_shared, workspace.d_x_routed_buffer)
    d_router_weights = workspace.d_router_weight_buffer if router_grad_view else workspace.d_router_weight_buffer.clone()
    return (d_x, d_router_weights, d_w_routed_gate, d_w_routed_up, d_w_routed_down,
            d_w_shared_gate, d_w_shared_up, d_w_shared_down)
