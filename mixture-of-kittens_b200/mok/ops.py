"""`torch.ops.mok.*`: the twelve custom ops of the MoE layer, backed by libmok_b200.so (sm_100a CUDA).

Names, argument order, mutation sets and return shapes follow the reference op surface (mok/ops.py of the
reference project) so callers and `torch.compile` graphs carry over unchanged.  Differences:
  * EP sizes 1, 2, 4 and 8 are accepted (the reference accepts 1, 4, 8, 16, 32, 64; one 8-GPU node is the
    domain here, and EP = 2 is new);
  * the ops allocate their outputs and pass raw device pointers to the C ABI on the current CUDA stream;
  * device-side problems are reported through a status word (see `check_status`) instead of a trap.
"""
from __future__ import annotations

import torch

from . import _native
from ._native import LayerArgs, check, check_status, lib, ptr, ptr_array, status_word, stream_ptr  # noqa: F401

SUPPORTED_EP_SIZES = (1, 2, 4, 8)

# all_gather_top_experts keeps the reference signature (a multicast address, no pointer list) and takes the peers'
# buffer addresses as an optional last argument; `mok.functional` passes the list its workspace carries.  Callers that
# use the five-argument form register the list of their symmetric buffer here instead.  An entry lives exactly as long
# as the buffer it was registered for: it is dropped when that tensor is freed, so a later allocation at the same
# address can never inherit it.
_ALL_GATHER_PEERS: dict[int, list[int]] = {}


def register_all_gather_peers(buffer: torch.Tensor, peer_ptrs: list[int]) -> None:
    import weakref
    key = int(buffer.data_ptr())
    _ALL_GATHER_PEERS[key] = [int(p) for p in peer_ptrs]
    weakref.finalize(buffer, _ALL_GATHER_PEERS.pop, key, None)


def unregister_all_gather_peers(buffer: torch.Tensor) -> None:
    _ALL_GATHER_PEERS.pop(int(buffer.data_ptr()), None)


# ------------------------------------------------------------------------------------------------------------
# validation helpers
# ------------------------------------------------------------------------------------------------------------
def _require(cond: bool, message: str, exc: type[Exception] = ValueError) -> None:
    if not cond:
        raise exc(message)


def _check_ptr_list(name: str, pointers, ep_size: int | None = None) -> int:
    _require(isinstance(pointers, list) and all(type(p) is int and p > 0 for p in pointers),
             f"{name} must be a list of positive integers", TypeError)
    if ep_size is None:
        _require(len(pointers) in SUPPORTED_EP_SIZES, f"{name} length must be one of {SUPPORTED_EP_SIZES}")
    else:
        _require(len(pointers) == ep_size, f"{name} length must match x_ptrs")
    return len(pointers)


def _check_layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size) -> None:
    _require(type(topk) is int and 0 < topk <= 255, "topk must be an integer in [1, 255]")
    _require(swiglu_limit is None or (type(swiglu_limit) in (int, float) and swiglu_limit >= 0),
             "swiglu_limit must be None or a non-negative number")
    _require(type(num_comm_sms) is int and num_comm_sms > 0 and num_comm_sms % 2 == 0,
             "num_comm_sms must be a positive even integer")
    _require(type(minibatch_size) is int and minibatch_size > 0 and minibatch_size % 256 == 0,
             "minibatch_size must be positive and divisible by 256")
    _require(type(macrobatch_size) is int and macrobatch_size > 0 and macrobatch_size % minibatch_size == 0,
             "macrobatch_size must be a positive multiple of minibatch_size")


def _check_activation_dims(x: torch.Tensor, w_shared_gate: torch.Tensor, w_routed_gate: torch.Tensor):
    _require(x.ndim == 2, "x must have shape (num_local_tokens, hidden_size)")
    num_local_tokens, hidden_size = x.shape
    _require(num_local_tokens >= 512 and num_local_tokens % 256 == 0,
             "num_local_tokens must be at least 512 and divisible by 256")
    _require(hidden_size > 0 and hidden_size % 256 == 0, "hidden_size must be positive and divisible by 256")
    _require(w_shared_gate.ndim == 2 and w_shared_gate.shape[1] == hidden_size,
             "w_shared_gate must have shape (intermediate_size, hidden_size)")
    intermediate_size = w_shared_gate.shape[0]
    _require(intermediate_size > 0 and intermediate_size % 256 == 0,
             "intermediate_size must be positive and divisible by 256")
    _require(w_routed_gate.ndim == 3 and w_routed_gate.shape[0] > 0,
             "w_routed_gate must have shape (num_local_experts, intermediate_size, hidden_size)")
    return num_local_tokens, hidden_size, intermediate_size, w_routed_gate.shape[0]


def _check_schedule(schedule_peer_rank: torch.Tensor) -> int:
    _require(schedule_peer_rank.ndim == 1 and schedule_peer_rank.numel() > 0,
             "schedule_peer_rank must be a nonempty 1D tensor")
    capacity = schedule_peer_rank.numel()
    _require(capacity % 256 == 0, "schedule_capacity must be divisible by 256")
    return capacity


def _check_shapes_devices(device: torch.device, expected) -> None:
    for name, tensor, shape in expected:
        _require(tuple(tensor.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}")
    for name, tensor, _ in expected:
        _require(tensor.device == device, f"{name} must be on {device}")


def _check_bf16_contiguous(named) -> None:
    for name, tensor in named:
        _require(tensor.dtype == torch.bfloat16 and tensor.is_contiguous(), f"{name} must be contiguous bfloat16", TypeError)


def _layer_args(*, ep_size: int, rank: int, x: torch.Tensor, intermediate: int, num_local_experts: int, topk: int,
                capacity: int, macrobatch_size: int, minibatch_size: int, num_comm_sms: int, swiglu_limit) -> LayerArgs:
    a = LayerArgs()
    a.ep_size, a.rank = ep_size, rank
    a.num_local_tokens, a.hidden = x.shape
    a.intermediate = intermediate
    a.num_local_experts = num_local_experts
    a.topk = topk
    a.schedule_capacity = capacity
    a.macrobatch_size = macrobatch_size
    a.minibatch_size = minibatch_size
    a.num_comm_sms = num_comm_sms
    a.has_swiglu_limit = 0 if swiglu_limit is None else 1
    a.swiglu_limit = 0.0 if swiglu_limit is None else float(swiglu_limit)
    a.status = status_word(x.device).data_ptr()
    a.x_local = x.data_ptr()
    return a


def _local_rank(x: torch.Tensor, x_ptrs: list[int]) -> int:
    """Index of this rank in the pointer list (informational; 0 when the local view has another address)."""
    try:
        return x_ptrs.index(int(x.data_ptr()))
    except ValueError:
        return 0


def _keep(args: LayerArgs, **arrays):
    """Stores ctypes pointer arrays on the struct (keeps them alive) and sets the matching fields."""
    holder = []
    for field, values in arrays.items():
        arr = ptr_array(values)
        holder.append(arr)
        setattr(args, field, _native.ctypes.cast(arr, _native.c_void_p))
    args._keepalive = holder
    return args


def _set_ptrs(args: LayerArgs, **tensors) -> None:
    for field, tensor in tensors.items():
        setattr(args, field, None if tensor is None else tensor.data_ptr())


def _new_fp8(like: torch.Tensor, rows: int, cols: int):
    """An e4m3 [rows, cols] buffer and its e8m0 scale tiles [rows/128, cols/128, 32, 16]."""
    return (like.new_empty((rows, cols), dtype=torch.float8_e4m3fn),
            like.new_empty((rows // 128, cols // 128, 32, 16), dtype=torch.uint8))


def _check_fp8_pair(name: str, data: torch.Tensor, scales: torch.Tensor, shape, device) -> None:
    rows = 1
    for s in shape[:-1]:
        rows *= s
    _require(tuple(data.shape) == tuple(shape), f"{name} must have shape {tuple(shape)}")
    _require(tuple(scales.shape) == (rows // 128, shape[-1] // 128, 32, 16),
             f"{name}_sc must have shape {(rows // 128, shape[-1] // 128, 32, 16)}")
    _require(data.device == device and scales.device == device, f"{name} and its scales must be on {device}")
    _require(data.dtype == torch.float8_e4m3fn and scales.dtype == torch.uint8 and data.is_contiguous() and scales.is_contiguous(),
             f"{name} must be contiguous float8_e4m3fn with contiguous uint8 scales", TypeError)


_check_fp8_weight = _check_fp8_pair


# ------------------------------------------------------------------------------------------------------------
# schedule-side ops
# ------------------------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::all_gather_top_experts", mutates_args=("all_gather_top_experts_buffer",))
def all_gather_top_experts(
    top_experts: torch.Tensor,
    all_gather_top_experts_buffer: torch.Tensor,
    all_gather_top_experts_buffer_multicast_ptr: int,
    rank: int,
    chunk_bytes: int,
    peer_buffer_ptrs: list[int] | None = None,
) -> None:
    """Writes this rank's routes into slot `rank` of every EP rank's gather buffer.

    Inputs:
        top_experts:                                 int32 [num_local_tokens, topk]
        all_gather_top_experts_buffer:               int32 [ep_size, num_local_tokens, topk]
        all_gather_top_experts_buffer_multicast_ptr: int (kept for interface compatibility; not dereferenced)
        rank:                                        int
        chunk_bytes:                                 int (kept for interface compatibility; validated only)
        peer_buffer_ptrs:                            list[int] [ep_size] or None: every rank's address of the gather
                                                     buffer (not in the reference signature; None looks the list up
                                                     among those given to `register_all_gather_peers`)
    """
    _require(top_experts.is_cuda and top_experts.dtype == torch.int32 and top_experts.is_contiguous() and top_experts.ndim == 2,
             "top_experts must be contiguous CUDA int32 [num_local_tokens, topk]")
    buf = all_gather_top_experts_buffer
    _require(buf.is_cuda, "all_gather_top_experts_buffer must be a CUDA tensor")
    _require(buf.dtype == torch.int32, "all_gather_top_experts_buffer must have dtype torch.int32", TypeError)
    _require(buf.is_contiguous(), "all_gather_top_experts_buffer must be contiguous")
    _require(buf.ndim == 3, "all_gather_top_experts_buffer must have shape (ep_size, num_local_tokens, topk)")
    _require(all(s > 0 for s in top_experts.shape), "top_experts dimensions must be positive")
    _require(all(s > 0 for s in buf.shape), "all_gather_top_experts_buffer dimensions must be positive")
    ep_size = buf.shape[0]
    _require(ep_size in SUPPORTED_EP_SIZES, f"all_gather_top_experts_buffer ep_size must be one of {SUPPORTED_EP_SIZES}")
    _require(buf.device == top_experts.device and tuple(buf.shape[1:]) == tuple(top_experts.shape),
             "all_gather_top_experts_buffer must match top_experts shape and device")
    _require(type(all_gather_top_experts_buffer_multicast_ptr) is int and all_gather_top_experts_buffer_multicast_ptr > 0,
             "all_gather_top_experts_buffer_multicast_ptr must be a positive integer", TypeError)
    _require(type(rank) is int and 0 <= rank < ep_size, "rank must be an integer in [0, ep_size)")
    _require(type(chunk_bytes) is int and chunk_bytes > 0, "chunk_bytes must be a positive integer")
    _require(chunk_bytes % 16 == 0, "chunk_bytes must be divisible by 16")
    _require((top_experts.numel() * 4) % chunk_bytes == 0, "chunk_bytes must divide one rank's route-buffer bytes")

    if ep_size == 1:
        buf[0].copy_(top_experts)
        return
    peers = peer_buffer_ptrs if peer_buffer_ptrs is not None else _ALL_GATHER_PEERS.get(int(buf.data_ptr()))
    if peers is not None:
        _require(isinstance(peers, list) and all(type(p) is int and p > 0 for p in peers),
                 "peer_buffer_ptrs must be a list of positive integers", TypeError)
    if peers is None or len(peers) != ep_size:
        raise RuntimeError("all_gather_top_experts_buffer is not a registered symmetric buffer "
                           "(create it with mok.functional.create_workspace or call ops.register_all_gather_peers)")
    check(lib().mok_all_gather_top_experts(ptr(top_experts), top_experts.numel(), ptr_array(peers), ep_size, rank,
                                           stream_ptr(buf.device)), "all_gather_top_experts")


@torch.library.custom_op("mok::barrier_all", mutates_args=("barrier_buffer", "target"))
def barrier_all(
    barrier_buffer: torch.Tensor,
    barrier_buffer_ptrs: list[int],
    barrier_buffer_multicast_ptr: int,
    target: torch.Tensor,
) -> None:
    """Device-side barrier over the EP ranks (stream ordered, no host wait).

    Inputs:
        barrier_buffer:               int32 [1]
        barrier_buffer_ptrs:          list[int] [ep_size]
        barrier_buffer_multicast_ptr: int (kept for interface compatibility; not dereferenced)
        target:                       int32 [1]
    """
    _require(barrier_buffer.is_cuda, "barrier_buffer must be a CUDA tensor")
    _require(barrier_buffer.dtype == torch.int32, "barrier_buffer must have dtype torch.int32", TypeError)
    _require(barrier_buffer.is_contiguous(), "barrier_buffer must be contiguous")
    _require(tuple(barrier_buffer.shape) == (1,), "barrier_buffer must have shape (1,)")
    _require(isinstance(barrier_buffer_ptrs, list) and all(type(p) is int and p > 0 for p in barrier_buffer_ptrs),
             "barrier_buffer_ptrs must be a list of positive integers", TypeError)
    ep_size = len(barrier_buffer_ptrs)
    _require(ep_size in SUPPORTED_EP_SIZES, f"barrier_buffer_ptrs length must be one of {SUPPORTED_EP_SIZES}")
    _require(type(barrier_buffer_multicast_ptr) is int and barrier_buffer_multicast_ptr > 0,
             "barrier_buffer_multicast_ptr must be a positive integer", TypeError)
    _require(target.is_cuda and target.device == barrier_buffer.device and target.dtype == torch.int32
             and target.is_contiguous() and tuple(target.shape) == (1,),
             "target must be contiguous int32 [1] on the barrier CUDA device")
    if ep_size == 1:
        return
    check(lib().mok_barrier_all(ptr(barrier_buffer), ptr_array(barrier_buffer_ptrs), ep_size, ptr(target),
                                ptr(status_word(barrier_buffer.device)), 0, stream_ptr(barrier_buffer.device)), "barrier_all")


@torch.library.custom_op("mok::schedule", mutates_args=())
def schedule(
    topk_all: torch.Tensor,
    num_local_experts: int,
    schedule_capacity: int,
    rank: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Builds this rank's padded per-expert receive schedule on the device.

    Inputs:
        topk_all:          int32 [ep_size, num_local_tokens, topk]
    Outputs:
        schedule_peer_rank [cap], schedule_peer_token_idx [cap], num_tokens [1], tokens_per_expert [E_loc] (int32)
    """
    _require(topk_all.ndim == 3, "topk_all must have shape (ep_size, num_local_tokens, topk)")
    ep_size, num_local_tokens, topk = topk_all.shape
    _require(ep_size in SUPPORTED_EP_SIZES, f"topk_all ep_size must be one of {SUPPORTED_EP_SIZES}")
    _require(num_local_tokens >= 512 and num_local_tokens % 256 == 0,
             "topk_all num_local_tokens must be at least 512 and divisible by 256")
    _require(0 < topk <= 255, "topk_all topk must be in [1, 255]")
    _require(type(num_local_experts) is int and num_local_experts > 0, "num_local_experts must be a positive integer")
    _require(type(schedule_capacity) is int and schedule_capacity > 0 and schedule_capacity % 256 == 0,
             "schedule_capacity must be positive and divisible by 256")
    _require(schedule_capacity >= num_local_tokens * topk, "schedule_capacity must hold at least one rank's routed tokens")
    _require(type(rank) is int and 0 <= rank < ep_size, "rank must be an integer in [0, ep_size)")
    _require(topk_all.is_cuda and topk_all.dtype == torch.int32 and topk_all.is_contiguous(),
             "topk_all must be a contiguous CUDA int32 tensor")

    opts = dict(dtype=torch.int32, device=topk_all.device)
    peer_rank = torch.empty(schedule_capacity, **opts)
    peer_token = torch.empty(schedule_capacity, **opts)
    num_tokens = torch.empty(1, **opts)
    per_expert = torch.empty(num_local_experts, **opts)
    scratch = torch.empty(lib().mok_schedule_scratch_bytes(ep_size, num_local_tokens, topk, num_local_experts) // 4, **opts)
    check(lib().mok_schedule(ptr(topk_all), ep_size, num_local_tokens, topk, num_local_experts, schedule_capacity, rank,
                             ptr(peer_rank), ptr(peer_token), ptr(num_tokens), ptr(per_expert), ptr(scratch),
                             ptr(status_word(topk_all.device)), stream_ptr(topk_all.device)), "schedule")
    return peer_rank, peer_token, num_tokens, per_expert


def _attach_dedup(args: LayerArgs, x: torch.Tensor, capacity: int, which: tuple[str, ...], need_x: bool, row_source, unique_peer,
                  unique_token, unique_before):
    """Sets the de-duplicated-dispatch fields of the layer arguments (all four index tensors or none) and allocates the
    staging buffers the call needs: one [staged_rows, H] bf16 buffer per staged input (`which`: "x", "d_y"; the x buffer
    of a backward call only when later macrobatches are replayed)."""
    given = [t is not None for t in (row_source, unique_peer, unique_token, unique_before)]
    if not any(given) or args.ep_size == 1:
        return None
    _require(all(given), "the four dedup_* tensors must be given together")
    for name, t in (("dedup_row_source", row_source), ("dedup_unique_peer", unique_peer), ("dedup_unique_token", unique_token),
                    ("dedup_unique_before", unique_before)):
        _require(t.device == x.device and t.dtype == torch.int32 and t.is_contiguous() and t.ndim == 1,
                 f"{name} must be a contiguous 1D int32 tensor on {x.device}")
    _require(row_source.numel() == capacity, "dedup_row_source must have schedule_capacity entries")
    _require(unique_before.numel() == capacity // 256 + 1, "dedup_unique_before must have schedule_capacity / 256 + 1 entries")
    _require(unique_peer.numel() == unique_token.numel() and unique_peer.numel() > 0,
             "dedup_unique_peer and dedup_unique_token must have the same, positive length")
    staged_rows = unique_peer.numel()
    _set_ptrs(args, row_source=row_source, unique_peer=unique_peer, unique_token=unique_token, unique_before=unique_before)
    args.staged_rows = staged_rows
    buffers = []
    if "x" in which and need_x:
        buffers.append(x.new_empty((staged_rows, x.shape[1])))
        args.staged_x = buffers[-1].data_ptr()
    if "d_y" in which:
        buffers.append(x.new_empty((staged_rows, x.shape[1])))
        args.staged_d_y = buffers[-1].data_ptr()
    return buffers


@torch.library.custom_op("mok::schedule_dedup", mutates_args=())
def schedule_dedup(
    topk_all: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    num_local_experts: int,
    rank: int,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Extends a schedule for de-duplicated dispatch: every (source rank, token) this rank serves is numbered in the
    order of its first schedule row, so that dispatch can pull each token once and fan it out locally.  Not among the
    reference ops (its dispatch pulls one row per route).

    Inputs:  topk_all int32 [ep_size, num_local_tokens, topk] and the outputs of `schedule`
    Outputs: row_source [cap] (number of the row's token, -1 on padding rows), unique_peer [U], unique_token [U]
             (source rank and token index of staged token u; U = min(cap, ep_size * num_local_tokens)),
             unique_before [cap / 256 + 1] (staged tokens first used below row 256 * i), num_unique [1]  (all int32)
    """
    _require(topk_all.ndim == 3 and topk_all.is_cuda and topk_all.dtype == torch.int32 and topk_all.is_contiguous(),
             "topk_all must be a contiguous CUDA int32 tensor of shape (ep_size, num_local_tokens, topk)")
    ep_size, num_local_tokens, topk = topk_all.shape
    _require(ep_size in SUPPORTED_EP_SIZES, f"topk_all ep_size must be one of {SUPPORTED_EP_SIZES}")
    cap = _check_schedule(schedule_peer_rank)
    for name, t, shape in (("schedule_peer_rank", schedule_peer_rank, (cap,)), ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
                           ("num_tokens", num_tokens, (1,))):
        _require(t.device == topk_all.device and t.dtype == torch.int32 and t.is_contiguous() and tuple(t.shape) == shape,
                 f"{name} must be contiguous int32 {shape} on {topk_all.device}")
    _require(type(num_local_experts) is int and num_local_experts > 0, "num_local_experts must be a positive integer")
    _require(type(rank) is int and 0 <= rank < ep_size, "rank must be an integer in [0, ep_size)")
    opts = dict(dtype=torch.int32, device=topk_all.device)
    max_unique = min(cap, ep_size * num_local_tokens)
    row_source = torch.empty(cap, **opts)
    unique_peer = torch.empty(max_unique, **opts)
    unique_token = torch.empty(max_unique, **opts)
    unique_before = torch.empty(cap // 256 + 1, **opts)
    num_unique = torch.empty(1, **opts)
    scratch = torch.empty(lib().mok_schedule_dedup_scratch_bytes(ep_size, num_local_tokens, topk, cap) // 4, **opts)
    check(lib().mok_schedule_dedup(ptr(topk_all), ep_size, num_local_tokens, topk, num_local_experts, cap, rank,
                                   ptr(schedule_peer_rank), ptr(schedule_peer_token_idx), ptr(num_tokens), ptr(row_source),
                                   ptr(unique_peer), ptr(unique_token), ptr(unique_before), ptr(num_unique), max_unique,
                                   ptr(scratch), stream_ptr(topk_all.device)), "schedule_dedup")
    return row_source, unique_peer, unique_token, unique_before, num_unique


@torch.library.custom_op(
    "mok::mxfp8_quantize", mutates_args=(),
    schema="(Tensor x_bf16, bool return_normal, bool return_transposed) -> (Tensor?, Tensor?, Tensor?, Tensor?)",
)
def mxfp8_quantize(x_bf16: torch.Tensor, return_normal: bool, return_transposed: bool):
    """bf16 [M, N] or [E, M, N] -> (x_fp8, x_sc, x_fp8_t, x_sc_t): e4m3 data with e8m0 scales per 32 elements
    along the row, for the matrix and/or its transpose; scales in the [rows/128, cols/128, 32, 16] layout."""
    _require(x_bf16.ndim in (2, 3), "x_bf16 must have shape (M, N) or (E, M, N)")
    _require(all(s > 0 for s in x_bf16.shape), "x_bf16 dimensions must be positive")
    _require(x_bf16.shape[-2] % 128 == 0 and x_bf16.shape[-1] % 128 == 0, "x_bf16 M and N dimensions must be divisible by 128")
    _require(type(return_normal) is bool and type(return_transposed) is bool,
             "return_normal and return_transposed must be booleans", TypeError)
    _require(return_normal or return_transposed, "at least one quantized layout must be requested")
    _require(x_bf16.is_cuda and x_bf16.dtype == torch.bfloat16 and x_bf16.is_contiguous(),
             "x_bf16 must be a contiguous CUDA bfloat16 tensor")
    experts = x_bf16.shape[0] if x_bf16.ndim == 3 else 1
    rows, cols = x_bf16.shape[-2:]
    t_shape = (experts, cols, rows) if x_bf16.ndim == 3 else (cols, rows)
    q = x_bf16.new_empty(x_bf16.shape, dtype=torch.float8_e4m3fn) if return_normal else None
    sc = x_bf16.new_empty((experts * rows // 128, cols // 128, 32, 16), dtype=torch.uint8) if return_normal else None
    qt = x_bf16.new_empty(t_shape, dtype=torch.float8_e4m3fn) if return_transposed else None
    sct = x_bf16.new_empty((experts * cols // 128, rows // 128, 32, 16), dtype=torch.uint8) if return_transposed else None
    check(lib().mok_mxfp8_quantize(ptr(x_bf16), experts, rows, cols, ptr(q), ptr(sc), ptr(qt), ptr(sct), stream_ptr(x_bf16.device)),
          "mxfp8_quantize")
    return q, sc, qt, sct


# ------------------------------------------------------------------------------------------------------------
# BF16 layer ops
# ------------------------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::dispatch_mlp_swiglu_combine_fwd_bf16", mutates_args=("combine_buffer",))
def dispatch_mlp_swiglu_combine_fwd_bf16(
    x: torch.Tensor,
    x_ptrs: list[int],
    combine_buffer: torch.Tensor,
    combine_buffer_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_shared_down: torch.Tensor,
    w_routed_down: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
    dedup_row_source: torch.Tensor | None = None,
    dedup_unique_peer: torch.Tensor | None = None,
    dedup_unique_token: torch.Tensor | None = None,
    dedup_unique_before: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor]:
    """BF16 forward: dispatch, routed + shared SwiGLU FFN, combine into the owners' slot buffers.

    Outputs: x_routed [MB,H], gate_shared [T,I], gate_routed [MB,I], up_shared, up_routed, hidden_shared,
             hidden_routed, y_shared [T,H], y_routed [MB,H]  (all bfloat16)
    """
    T, H, I, E = _check_activation_dims(x, w_shared_gate, w_routed_gate)
    _check_layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _check_ptr_list("x_ptrs", x_ptrs)
    _check_ptr_list("combine_buffer_ptrs", combine_buffer_ptrs, ep_size)
    cap = _check_schedule(schedule_peer_rank)
    _check_shapes_devices(x.device, (
        ("combine_buffer", combine_buffer, (T * topk, H)),
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_routed_gate", w_routed_gate, (E, I, H)),
        ("w_shared_up", w_shared_up, (I, H)), ("w_routed_up", w_routed_up, (E, I, H)),
        ("w_shared_down", w_shared_down, (H, I)), ("w_routed_down", w_routed_down, (E, H, I)),
        ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
        ("num_tokens", num_tokens, (1,)), ("tokens_per_expert", tokens_per_expert, (E,)),
    ))
    _require(schedule_peer_rank.device == x.device, f"schedule_peer_rank must be on {x.device}")
    _check_bf16_contiguous((("x", x), ("w_shared_gate", w_shared_gate), ("w_routed_gate", w_routed_gate),
                            ("w_shared_up", w_shared_up), ("w_routed_up", w_routed_up),
                            ("w_shared_down", w_shared_down), ("w_routed_down", w_routed_down)))

    new = lambda r, c: x.new_empty((r, c))  # noqa: E731
    x_routed, y_routed = new(macrobatch_size, H), new(macrobatch_size, H)
    gate_shared, up_shared, hidden_shared = new(T, I), new(T, I), new(T, I)
    gate_routed, up_routed, hidden_routed = new(macrobatch_size, I), new(macrobatch_size, I), new(macrobatch_size, I)
    y_shared = torch.empty_like(x)

    a = _layer_args(ep_size=ep_size, rank=_local_rank(x, x_ptrs), x=x, intermediate=I, num_local_experts=E, topk=topk,
                    capacity=cap, macrobatch_size=macrobatch_size, minibatch_size=minibatch_size,
                    num_comm_sms=num_comm_sms, swiglu_limit=swiglu_limit)
    _keep(a, x_ptrs=x_ptrs, combine_ptrs=combine_buffer_ptrs)
    a.peer_rank, a.peer_token_idx = schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr()
    a.num_tokens, a.tokens_per_expert = num_tokens.data_ptr(), tokens_per_expert.data_ptr()
    a.w_shared_gate, a.w_shared_up, a.w_shared_down = w_shared_gate.data_ptr(), w_shared_up.data_ptr(), w_shared_down.data_ptr()
    a.w_routed_gate, a.w_routed_up, a.w_routed_down = w_routed_gate.data_ptr(), w_routed_up.data_ptr(), w_routed_down.data_ptr()
    a.x_routed, a.y_routed, a.y_shared = x_routed.data_ptr(), y_routed.data_ptr(), y_shared.data_ptr()
    a.gate_shared, a.up_shared, a.hidden_shared = gate_shared.data_ptr(), up_shared.data_ptr(), hidden_shared.data_ptr()
    a.gate_routed, a.up_routed, a.hidden_routed = gate_routed.data_ptr(), up_routed.data_ptr(), hidden_routed.data_ptr()
    _staging = _attach_dedup(a, x, cap, ('x',), True, dedup_row_source, dedup_unique_peer, dedup_unique_token,
                             dedup_unique_before)  # noqa: F841  (keeps the staging buffers alive until the launch is queued)
    check(lib().mok_moe_forward_bf16(_native.ctypes.byref(a), stream_ptr(x.device)), "dispatch_mlp_swiglu_combine_fwd_bf16")
    return (x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared, hidden_routed, y_shared, y_routed)


@torch.library.custom_op("mok::recompute_forward_context_bf16", mutates_args=())
def recompute_forward_context_bf16(
    x: torch.Tensor,
    x_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
    dedup_row_source: torch.Tensor | None = None,
    dedup_unique_peer: torch.Tensor | None = None,
    dedup_unique_token: torch.Tensor | None = None,
    dedup_unique_before: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Rebuilds the saved forward context (first macrobatch) without the down projection and combine.

    Outputs: x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared, hidden_routed
    """
    T, H, I, E = _check_activation_dims(x, w_shared_gate, w_routed_gate)
    _check_layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _check_ptr_list("x_ptrs", x_ptrs)
    cap = _check_schedule(schedule_peer_rank)
    _check_shapes_devices(x.device, (
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_routed_gate", w_routed_gate, (E, I, H)),
        ("w_shared_up", w_shared_up, (I, H)), ("w_routed_up", w_routed_up, (E, I, H)),
        ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
        ("num_tokens", num_tokens, (1,)), ("tokens_per_expert", tokens_per_expert, (E,)),
    ))
    _require(schedule_peer_rank.device == x.device, f"schedule_peer_rank must be on {x.device}")
    _check_bf16_contiguous((("x", x), ("w_shared_gate", w_shared_gate), ("w_routed_gate", w_routed_gate),
                            ("w_shared_up", w_shared_up), ("w_routed_up", w_routed_up)))

    new = lambda r, c: x.new_empty((r, c))  # noqa: E731
    x_routed = new(macrobatch_size, H)
    gate_shared, up_shared, hidden_shared = new(T, I), new(T, I), new(T, I)
    gate_routed, up_routed, hidden_routed = new(macrobatch_size, I), new(macrobatch_size, I), new(macrobatch_size, I)
    a = _layer_args(ep_size=ep_size, rank=_local_rank(x, x_ptrs), x=x, intermediate=I, num_local_experts=E, topk=topk,
                    capacity=cap, macrobatch_size=macrobatch_size, minibatch_size=minibatch_size,
                    num_comm_sms=num_comm_sms, swiglu_limit=swiglu_limit)
    _keep(a, x_ptrs=x_ptrs)
    a.peer_rank, a.peer_token_idx = schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr()
    a.num_tokens, a.tokens_per_expert = num_tokens.data_ptr(), tokens_per_expert.data_ptr()
    a.w_shared_gate, a.w_shared_up = w_shared_gate.data_ptr(), w_shared_up.data_ptr()
    a.w_routed_gate, a.w_routed_up = w_routed_gate.data_ptr(), w_routed_up.data_ptr()
    a.x_routed = x_routed.data_ptr()
    a.gate_shared, a.up_shared, a.hidden_shared = gate_shared.data_ptr(), up_shared.data_ptr(), hidden_shared.data_ptr()
    a.gate_routed, a.up_routed, a.hidden_routed = gate_routed.data_ptr(), up_routed.data_ptr(), hidden_routed.data_ptr()
    _staging = _attach_dedup(a, x, cap, ('x',), True, dedup_row_source, dedup_unique_peer, dedup_unique_token,
                             dedup_unique_before)  # noqa: F841  (keeps the staging buffers alive until the launch is queued)
    check(lib().mok_moe_recompute_bf16(_native.ctypes.byref(a), stream_ptr(x.device)), "recompute_forward_context_bf16")
    return (x_routed, gate_shared, gate_routed, up_shared, up_routed, hidden_shared, hidden_routed)


@torch.library.custom_op(
    "mok::dispatch_mlp_swiglu_combine_bwd_bf16",
    mutates_args=("d_x_routed_buffer", "d_router_weight_buffer", "x_routed", "gate_routed", "up_routed", "hidden_routed"),
)
def dispatch_mlp_swiglu_combine_bwd_bf16(
    d_y_buffer: torch.Tensor,
    d_y_buffer_ptrs: list[int],
    d_x_routed_buffer: torch.Tensor,
    d_x_routed_buffer_ptrs: list[int],
    router_weight_buffer: torch.Tensor,
    router_weight_buffer_ptrs: list[int],
    d_router_weight_buffer: torch.Tensor,
    d_router_weight_buffer_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_shared_down: torch.Tensor,
    w_routed_down: torch.Tensor,
    x_routed: torch.Tensor,
    gate_shared: torch.Tensor,
    gate_routed: torch.Tensor,
    up_shared: torch.Tensor,
    up_routed: torch.Tensor,
    hidden_shared: torch.Tensor,
    hidden_routed: torch.Tensor,
    x: torch.Tensor,
    x_ptrs: list[int],
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
    dedup_row_source: torch.Tensor | None = None,
    dedup_unique_peer: torch.Tensor | None = None,
    dedup_unique_token: torch.Tensor | None = None,
    dedup_unique_before: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """BF16 backward of the layer.

    Outputs: d_x_shared [T,H], d_x_routed [MB,H], d_gate_shared [T,I], d_gate_routed [MB,I], d_up_shared,
             d_up_routed, d_hidden_shared, d_hidden_routed, d_y_routed [MB,H], d_w_shared_gate [I,H],
             d_w_routed_gate [E,I,H], d_w_shared_up, d_w_routed_up, d_w_shared_down [H,I], d_w_routed_down [E,H,I]
    The routed input gradients and router-weight gradients land in the owners' symmetric buffers.
    """
    T, H, I, E = _check_activation_dims(x, w_shared_gate, w_routed_gate)
    _check_layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _check_ptr_list("x_ptrs", x_ptrs)
    for name, pointers in (("d_y_buffer_ptrs", d_y_buffer_ptrs), ("d_x_routed_buffer_ptrs", d_x_routed_buffer_ptrs),
                           ("router_weight_buffer_ptrs", router_weight_buffer_ptrs),
                           ("d_router_weight_buffer_ptrs", d_router_weight_buffer_ptrs)):
        _check_ptr_list(name, pointers, ep_size)
    cap = _check_schedule(schedule_peer_rank)
    MB = macrobatch_size
    _check_shapes_devices(x.device, (
        ("d_y_buffer", d_y_buffer, (T, H)), ("d_x_routed_buffer", d_x_routed_buffer, (T * topk, H)),
        ("router_weight_buffer", router_weight_buffer, (T, topk)), ("d_router_weight_buffer", d_router_weight_buffer, (T, topk)),
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_routed_gate", w_routed_gate, (E, I, H)),
        ("w_shared_up", w_shared_up, (I, H)), ("w_routed_up", w_routed_up, (E, I, H)),
        ("w_shared_down", w_shared_down, (H, I)), ("w_routed_down", w_routed_down, (E, H, I)),
        ("x_routed", x_routed, (MB, H)), ("gate_shared", gate_shared, (T, I)), ("gate_routed", gate_routed, (MB, I)),
        ("up_shared", up_shared, (T, I)), ("up_routed", up_routed, (MB, I)),
        ("hidden_shared", hidden_shared, (T, I)), ("hidden_routed", hidden_routed, (MB, I)),
        ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
        ("num_tokens", num_tokens, (1,)), ("tokens_per_expert", tokens_per_expert, (E,)),
    ))
    _require(schedule_peer_rank.device == x.device, f"schedule_peer_rank must be on {x.device}")
    _check_bf16_contiguous((("x", x), ("d_y_buffer", d_y_buffer), ("x_routed", x_routed), ("gate_shared", gate_shared),
                            ("gate_routed", gate_routed), ("up_shared", up_shared), ("up_routed", up_routed),
                            ("hidden_shared", hidden_shared), ("hidden_routed", hidden_routed),
                            ("w_shared_gate", w_shared_gate), ("w_routed_gate", w_routed_gate),
                            ("w_shared_up", w_shared_up), ("w_routed_up", w_routed_up),
                            ("w_shared_down", w_shared_down), ("w_routed_down", w_routed_down)))

    new = lambda *shape: x.new_empty(shape)  # noqa: E731
    d_x_shared, d_x_routed, d_y_routed = new(T, H), new(MB, H), new(MB, H)
    d_gate_shared, d_up_shared, d_hidden_shared = new(T, I), new(T, I), new(T, I)
    d_gate_routed, d_up_routed, d_hidden_routed = new(MB, I), new(MB, I), new(MB, I)
    d_w_shared_gate, d_w_shared_up, d_w_shared_down = new(I, H), new(I, H), new(H, I)
    d_w_routed_gate, d_w_routed_up, d_w_routed_down = new(E, I, H), new(E, I, H), new(E, H, I)
    row_scratch = torch.empty(2 * MB + E, dtype=torch.float32, device=x.device)

    a = _layer_args(ep_size=ep_size, rank=_local_rank(x, x_ptrs), x=x, intermediate=I, num_local_experts=E, topk=topk,
                    capacity=cap, macrobatch_size=MB, minibatch_size=minibatch_size, num_comm_sms=num_comm_sms,
                    swiglu_limit=swiglu_limit)
    _keep(a, x_ptrs=x_ptrs, d_y_ptrs=d_y_buffer_ptrs, d_x_routed_ptrs=d_x_routed_buffer_ptrs,
          router_weight_ptrs=router_weight_buffer_ptrs, d_router_weight_ptrs=d_router_weight_buffer_ptrs)
    a.peer_rank, a.peer_token_idx = schedule_peer_rank.data_ptr(), schedule_peer_token_idx.data_ptr()
    a.num_tokens, a.tokens_per_expert = num_tokens.data_ptr(), tokens_per_expert.data_ptr()
    a.w_shared_gate, a.w_shared_up, a.w_shared_down = w_shared_gate.data_ptr(), w_shared_up.data_ptr(), w_shared_down.data_ptr()
    a.w_routed_gate, a.w_routed_up, a.w_routed_down = w_routed_gate.data_ptr(), w_routed_up.data_ptr(), w_routed_down.data_ptr()
    a.x_routed = x_routed.data_ptr()
    a.gate_shared, a.up_shared, a.hidden_shared = gate_shared.data_ptr(), up_shared.data_ptr(), hidden_shared.data_ptr()
    a.gate_routed, a.up_routed, a.hidden_routed = gate_routed.data_ptr(), up_routed.data_ptr(), hidden_routed.data_ptr()
    a.d_x_shared, a.d_x_routed, a.d_y_routed = d_x_shared.data_ptr(), d_x_routed.data_ptr(), d_y_routed.data_ptr()
    a.d_gate_shared, a.d_up_shared, a.d_hidden_shared = d_gate_shared.data_ptr(), d_up_shared.data_ptr(), d_hidden_shared.data_ptr()
    a.d_gate_routed, a.d_up_routed, a.d_hidden_routed = d_gate_routed.data_ptr(), d_up_routed.data_ptr(), d_hidden_routed.data_ptr()
    a.d_w_shared_gate, a.d_w_shared_up, a.d_w_shared_down = d_w_shared_gate.data_ptr(), d_w_shared_up.data_ptr(), d_w_shared_down.data_ptr()
    a.d_w_routed_gate, a.d_w_routed_up, a.d_w_routed_down = d_w_routed_gate.data_ptr(), d_w_routed_up.data_ptr(), d_w_routed_down.data_ptr()
    a.row_scratch = row_scratch.data_ptr()
    a.d_y_local = d_y_buffer.data_ptr()
    _staging = _attach_dedup(a, x, cap, ('x', 'd_y'), macrobatch_size < cap, dedup_row_source, dedup_unique_peer, dedup_unique_token,
                             dedup_unique_before)  # noqa: F841  (keeps the staging buffers alive until the launch is queued)
    check(lib().mok_moe_backward_bf16(_native.ctypes.byref(a), stream_ptr(x.device)), "dispatch_mlp_swiglu_combine_bwd_bf16")
    return (d_x_shared, d_x_routed, d_gate_shared, d_gate_routed, d_up_shared, d_up_routed, d_hidden_shared, d_hidden_routed,
            d_y_routed, d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down, d_w_routed_down)


# ------------------------------------------------------------------------------------------------------------
# epilogues
# ------------------------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::fwd_epilogue", mutates_args=())
def fwd_epilogue(y_shared: torch.Tensor, combine_buffer: torch.Tensor, topk_weights: torch.Tensor) -> torch.Tensor:
    """output[t] = bf16(y_shared[t] + sum_k topk_weights[t, k] * combine_buffer[t*topk + k]), k ascending, fp32 sum.
    If the device status word of this GPU holds an error bit (see `check_status`) the output is all NaN."""
    _require(y_shared.ndim == 2, "y_shared must have shape (num_local_tokens, hidden_size)")
    T, H = y_shared.shape
    _require(T >= 512 and T % 256 == 0, "num_local_tokens must be at least 512 and divisible by 256")
    _require(H > 0 and H % 256 == 0, "hidden_size must be positive and divisible by 256")
    _require(topk_weights.device == y_shared.device and combine_buffer.device == y_shared.device,
             "all tensors must be on the same CUDA device")
    _require(topk_weights.ndim == 2 and topk_weights.shape[0] == T, "topk_weights must have shape (num_local_tokens, topk)")
    topk = topk_weights.shape[1]
    _require(0 < topk <= 255, "topk must be in [1, 255]")
    _require(tuple(combine_buffer.shape) == (T * topk, H), "combine_buffer must have shape (num_local_tokens * topk, hidden_size)")
    _require(y_shared.is_cuda and y_shared.dtype == torch.bfloat16 and combine_buffer.dtype == torch.bfloat16
             and topk_weights.dtype == torch.float32 and y_shared.is_contiguous() and combine_buffer.is_contiguous()
             and topk_weights.is_contiguous(), "fwd_epilogue needs contiguous CUDA bfloat16 activations and float32 weights")
    out = torch.empty_like(y_shared)
    check(lib().mok_fwd_epilogue(ptr(y_shared), ptr(combine_buffer), ptr(topk_weights), ptr(out), T, H, topk,
                                 ptr(status_word(y_shared.device)), stream_ptr(y_shared.device)), "fwd_epilogue")
    return out


@torch.library.custom_op("mok::bwd_epilogue", mutates_args=())
def bwd_epilogue(d_x_shared: torch.Tensor, d_x_routed_buffer: torch.Tensor) -> torch.Tensor:
    """d_x[t] = bf16(d_x_shared[t] + sum_k d_x_routed_buffer[t*topk + k]), k ascending, fp32 sum.
    If the device status word of this GPU holds an error bit (see `check_status`) the output is all NaN."""
    _require(d_x_shared.ndim == 2, "d_x_shared must have shape (num_local_tokens, hidden_size)")
    T, H = d_x_shared.shape
    _require(T >= 512 and T % 256 == 0, "num_local_tokens must be at least 512 and divisible by 256")
    _require(H > 0 and H % 256 == 0, "hidden_size must be positive and divisible by 256")
    _require(d_x_routed_buffer.device == d_x_shared.device, "d_x_routed_buffer must be on the same CUDA device")
    _require(d_x_routed_buffer.ndim == 2 and d_x_routed_buffer.shape[1] == H and d_x_routed_buffer.shape[0] % T == 0
             and 0 < d_x_routed_buffer.shape[0] <= T * 255,
             "d_x_routed_buffer must have shape (num_local_tokens * topk, hidden_size)")
    _require(d_x_shared.is_cuda and d_x_shared.dtype == torch.bfloat16 and d_x_routed_buffer.dtype == torch.bfloat16
             and d_x_shared.is_contiguous() and d_x_routed_buffer.is_contiguous(),
             "bwd_epilogue needs contiguous CUDA bfloat16 tensors")
    out = torch.empty_like(d_x_shared)
    check(lib().mok_bwd_epilogue(ptr(d_x_shared), ptr(d_x_routed_buffer), ptr(out), T, H, d_x_routed_buffer.shape[0] // T,
                                 ptr(status_word(d_x_shared.device)), stream_ptr(d_x_shared.device)), "bwd_epilogue")
    return out


# ------------------------------------------------------------------------------------------------------------
# MXFP8 layer ops
# ------------------------------------------------------------------------------------------------------------
@torch.library.custom_op("mok::dispatch_mlp_swiglu_combine_fwd_mxfp8", mutates_args=("combine_buffer",))
def dispatch_mlp_swiglu_combine_fwd_mxfp8(
    x: torch.Tensor,
    x_ptrs: list[int],
    combine_buffer: torch.Tensor,
    combine_buffer_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_routed_gate_sc: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_routed_up_sc: torch.Tensor,
    w_shared_down: torch.Tensor,
    w_routed_down: torch.Tensor,
    w_routed_down_sc: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
    dedup_row_source: torch.Tensor | None = None,
    dedup_unique_peer: torch.Tensor | None = None,
    dedup_unique_token: torch.Tensor | None = None,
    dedup_unique_before: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """MXFP8 forward (routed experts in e4m3 with e8m0 block scales, shared expert in bf16).

    Outputs: x_fp8_t_routed [H,MB], x_sc_t_routed, gate_shared, gate_fp8_routed [MB,I], gate_sc_routed, up_shared,
             up_fp8_routed, up_sc_routed, hidden_shared, hidden_fp8_t_routed [I,MB], hidden_sc_t_routed, y_shared, y_routed
    """
    T, H, I, E = _check_activation_dims(x, w_shared_gate, w_routed_gate)
    _check_layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _check_ptr_list("x_ptrs", x_ptrs)
    _check_ptr_list("combine_buffer_ptrs", combine_buffer_ptrs, ep_size)
    cap = _check_schedule(schedule_peer_rank)
    MB = macrobatch_size
    _check_shapes_devices(x.device, (
        ("combine_buffer", combine_buffer, (T * topk, H)),
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_shared_up", w_shared_up, (I, H)), ("w_shared_down", w_shared_down, (H, I)),
        ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
        ("num_tokens", num_tokens, (1,)), ("tokens_per_expert", tokens_per_expert, (E,)),
    ))
    _check_fp8_weight("w_routed_gate", w_routed_gate, w_routed_gate_sc, (E, I, H), x.device)
    _check_fp8_weight("w_routed_up", w_routed_up, w_routed_up_sc, (E, I, H), x.device)
    _check_fp8_weight("w_routed_down", w_routed_down, w_routed_down_sc, (E, H, I), x.device)
    _check_bf16_contiguous((("x", x), ("w_shared_gate", w_shared_gate), ("w_shared_up", w_shared_up),
                            ("w_shared_down", w_shared_down)))

    new = lambda *shape: x.new_empty(shape)  # noqa: E731
    x_t, x_t_sc = _new_fp8(x, H, MB)
    gate_q, gate_sc = _new_fp8(x, MB, I)
    up_q, up_sc = _new_fp8(x, MB, I)
    hid_t, hid_t_sc = _new_fp8(x, I, MB)
    gate_shared, up_shared, hidden_shared, y_shared, y_routed = new(T, I), new(T, I), new(T, I), new(T, H), new(MB, H)
    scratch = dict(x_routed=new(MB, H), gate_routed=new(MB, I), up_routed=new(MB, I), hidden_routed=new(MB, I))
    x_q, x_sc = _new_fp8(x, MB, H)
    hid_q, hid_sc = _new_fp8(x, MB, I)

    a = _layer_args(ep_size=ep_size, rank=_local_rank(x, x_ptrs), x=x, intermediate=I, num_local_experts=E, topk=topk,
                    capacity=cap, macrobatch_size=MB, minibatch_size=minibatch_size, num_comm_sms=num_comm_sms,
                    swiglu_limit=swiglu_limit)
    _keep(a, x_ptrs=x_ptrs, combine_ptrs=combine_buffer_ptrs)
    _set_ptrs(a, peer_rank=schedule_peer_rank, peer_token_idx=schedule_peer_token_idx, num_tokens=num_tokens,
              tokens_per_expert=tokens_per_expert, w_shared_gate=w_shared_gate, w_shared_up=w_shared_up,
              w_shared_down=w_shared_down, w_gate_fp8=w_routed_gate, w_gate_sc=w_routed_gate_sc, w_up_fp8=w_routed_up,
              w_up_sc=w_routed_up_sc, w_down_fp8=w_routed_down, w_down_sc=w_routed_down_sc,
              gate_shared=gate_shared, up_shared=up_shared, hidden_shared=hidden_shared, y_shared=y_shared, y_routed=y_routed,
              x_fp8=x_q, x_sc=x_sc, x_fp8_t=x_t, x_sc_t=x_t_sc, gate_fp8=gate_q, gate_sc=gate_sc, up_fp8=up_q, up_sc=up_sc,
              hidden_fp8=hid_q, hidden_sc=hid_sc, hidden_fp8_t=hid_t, hidden_sc_t=hid_t_sc, **scratch)
    _staging = _attach_dedup(a, x, cap, ('x',), True, dedup_row_source, dedup_unique_peer, dedup_unique_token,
                             dedup_unique_before)  # noqa: F841  (keeps the staging buffers alive until the launch is queued)
    check(lib().mok_moe_forward_mxfp8(_native.ctypes.byref(a), stream_ptr(x.device)), "dispatch_mlp_swiglu_combine_fwd_mxfp8")
    return (x_t, x_t_sc, gate_shared, gate_q, gate_sc, up_shared, up_q, up_sc, hidden_shared, hid_t, hid_t_sc, y_shared, y_routed)


@torch.library.custom_op("mok::recompute_forward_context_mxfp8", mutates_args=())
def recompute_forward_context_mxfp8(
    x: torch.Tensor,
    x_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate: torch.Tensor,
    w_routed_gate_sc: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_routed_up_sc: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
    dedup_row_source: torch.Tensor | None = None,
    dedup_unique_peer: torch.Tensor | None = None,
    dedup_unique_token: torch.Tensor | None = None,
    dedup_unique_before: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor]:
    """MXFP8 context recomputation (first macrobatch): dispatch, quantize, gate / up GEMMs, SwiGLU, quantize.

    Outputs: x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed, gate_sc_routed, up_shared, up_fp8_routed,
             up_sc_routed, hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed
    """
    T, H, I, E = _check_activation_dims(x, w_shared_gate, w_routed_gate)
    _check_layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _check_ptr_list("x_ptrs", x_ptrs)
    cap = _check_schedule(schedule_peer_rank)
    MB = macrobatch_size
    _check_shapes_devices(x.device, (
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_shared_up", w_shared_up, (I, H)),
        ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
        ("num_tokens", num_tokens, (1,)), ("tokens_per_expert", tokens_per_expert, (E,)),
    ))
    _check_fp8_weight("w_routed_gate", w_routed_gate, w_routed_gate_sc, (E, I, H), x.device)
    _check_fp8_weight("w_routed_up", w_routed_up, w_routed_up_sc, (E, I, H), x.device)
    _check_bf16_contiguous((("x", x), ("w_shared_gate", w_shared_gate), ("w_shared_up", w_shared_up)))

    new = lambda *shape: x.new_empty(shape)  # noqa: E731
    x_t, x_t_sc = _new_fp8(x, H, MB)
    gate_q, gate_sc = _new_fp8(x, MB, I)
    up_q, up_sc = _new_fp8(x, MB, I)
    hid_t, hid_t_sc = _new_fp8(x, I, MB)
    gate_shared, up_shared, hidden_shared = new(T, I), new(T, I), new(T, I)
    scratch = dict(x_routed=new(MB, H), gate_routed=new(MB, I), up_routed=new(MB, I), hidden_routed=new(MB, I))
    x_q, x_sc = _new_fp8(x, MB, H)
    hid_q, hid_sc = _new_fp8(x, MB, I)
    a = _layer_args(ep_size=ep_size, rank=_local_rank(x, x_ptrs), x=x, intermediate=I, num_local_experts=E, topk=topk,
                    capacity=cap, macrobatch_size=MB, minibatch_size=minibatch_size, num_comm_sms=num_comm_sms,
                    swiglu_limit=swiglu_limit)
    _keep(a, x_ptrs=x_ptrs)
    _set_ptrs(a, peer_rank=schedule_peer_rank, peer_token_idx=schedule_peer_token_idx, num_tokens=num_tokens,
              tokens_per_expert=tokens_per_expert, w_shared_gate=w_shared_gate, w_shared_up=w_shared_up,
              w_gate_fp8=w_routed_gate, w_gate_sc=w_routed_gate_sc, w_up_fp8=w_routed_up, w_up_sc=w_routed_up_sc,
              gate_shared=gate_shared, up_shared=up_shared, hidden_shared=hidden_shared,
              x_fp8=x_q, x_sc=x_sc, x_fp8_t=x_t, x_sc_t=x_t_sc, gate_fp8=gate_q, gate_sc=gate_sc, up_fp8=up_q, up_sc=up_sc,
              hidden_fp8=hid_q, hidden_sc=hid_sc, hidden_fp8_t=hid_t, hidden_sc_t=hid_t_sc, **scratch)
    _staging = _attach_dedup(a, x, cap, ('x',), True, dedup_row_source, dedup_unique_peer, dedup_unique_token,
                             dedup_unique_before)  # noqa: F841  (keeps the staging buffers alive until the launch is queued)
    check(lib().mok_moe_recompute_mxfp8(_native.ctypes.byref(a), stream_ptr(x.device)), "recompute_forward_context_mxfp8")
    return (x_t, x_t_sc, gate_shared, gate_q, gate_sc, up_shared, up_q, up_sc, hidden_shared, hid_t, hid_t_sc)


@torch.library.custom_op(
    "mok::dispatch_mlp_swiglu_combine_bwd_mxfp8",
    mutates_args=("d_x_routed_buffer", "d_router_weight_buffer", "x_fp8_t_routed", "x_sc_t_routed", "gate_fp8_routed",
                  "gate_sc_routed", "up_fp8_routed", "up_sc_routed", "hidden_fp8_t_routed", "hidden_sc_t_routed"),
)
def dispatch_mlp_swiglu_combine_bwd_mxfp8(
    d_y_buffer: torch.Tensor,
    d_y_buffer_ptrs: list[int],
    d_x_routed_buffer: torch.Tensor,
    d_x_routed_buffer_ptrs: list[int],
    router_weight_buffer: torch.Tensor,
    router_weight_buffer_ptrs: list[int],
    d_router_weight_buffer: torch.Tensor,
    d_router_weight_buffer_ptrs: list[int],
    w_shared_gate: torch.Tensor,
    w_routed_gate_T: torch.Tensor,
    w_routed_gate_T_sc: torch.Tensor,
    w_shared_up: torch.Tensor,
    w_routed_up_T: torch.Tensor,
    w_routed_up_T_sc: torch.Tensor,
    w_shared_down: torch.Tensor,
    w_routed_down_T: torch.Tensor,
    w_routed_down_T_sc: torch.Tensor,
    x_fp8_t_routed: torch.Tensor,
    x_sc_t_routed: torch.Tensor,
    gate_shared: torch.Tensor,
    gate_fp8_routed: torch.Tensor,
    gate_sc_routed: torch.Tensor,
    up_shared: torch.Tensor,
    up_fp8_routed: torch.Tensor,
    up_sc_routed: torch.Tensor,
    hidden_shared: torch.Tensor,
    hidden_fp8_t_routed: torch.Tensor,
    hidden_sc_t_routed: torch.Tensor,
    x: torch.Tensor,
    x_ptrs: list[int],
    w_routed_gate: torch.Tensor,
    w_routed_gate_sc: torch.Tensor,
    w_routed_up: torch.Tensor,
    w_routed_up_sc: torch.Tensor,
    schedule_peer_rank: torch.Tensor,
    schedule_peer_token_idx: torch.Tensor,
    num_tokens: torch.Tensor,
    tokens_per_expert: torch.Tensor,
    topk: int,
    swiglu_limit: float | None,
    num_comm_sms: int,
    macrobatch_size: int,
    minibatch_size: int,
    dedup_row_source: torch.Tensor | None = None,
    dedup_unique_peer: torch.Tensor | None = None,
    dedup_unique_token: torch.Tensor | None = None,
    dedup_unique_before: torch.Tensor | None = None,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor,
           torch.Tensor, torch.Tensor]:
    """MXFP8 backward of the layer.

    Outputs: d_x_shared [T,H], d_x_routed [MB,H], d_gate_shared, d_gate_fp8_routed [MB,I], d_gate_sc_routed, d_up_shared,
             d_up_fp8_routed, d_up_sc_routed, d_hidden_shared, d_hidden_routed [MB,I] bf16, d_y_fp8_routed [MB,H],
             d_y_sc_routed, d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down, d_w_routed_down
    """
    T, H, I, E = _check_activation_dims(x, w_shared_gate, w_routed_gate)
    _check_layer_scalars(topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size)
    ep_size = _check_ptr_list("x_ptrs", x_ptrs)
    for name, pointers in (("d_y_buffer_ptrs", d_y_buffer_ptrs), ("d_x_routed_buffer_ptrs", d_x_routed_buffer_ptrs),
                           ("router_weight_buffer_ptrs", router_weight_buffer_ptrs),
                           ("d_router_weight_buffer_ptrs", d_router_weight_buffer_ptrs)):
        _check_ptr_list(name, pointers, ep_size)
    cap = _check_schedule(schedule_peer_rank)
    MB = macrobatch_size
    dev = x.device
    _check_shapes_devices(dev, (
        ("d_y_buffer", d_y_buffer, (T, H)), ("d_x_routed_buffer", d_x_routed_buffer, (T * topk, H)),
        ("router_weight_buffer", router_weight_buffer, (T, topk)), ("d_router_weight_buffer", d_router_weight_buffer, (T, topk)),
        ("w_shared_gate", w_shared_gate, (I, H)), ("w_shared_up", w_shared_up, (I, H)), ("w_shared_down", w_shared_down, (H, I)),
        ("gate_shared", gate_shared, (T, I)), ("up_shared", up_shared, (T, I)), ("hidden_shared", hidden_shared, (T, I)),
        ("schedule_peer_token_idx", schedule_peer_token_idx, (cap,)),
        ("num_tokens", num_tokens, (1,)), ("tokens_per_expert", tokens_per_expert, (E,)),
    ))
    _check_fp8_weight("w_routed_gate", w_routed_gate, w_routed_gate_sc, (E, I, H), dev)
    _check_fp8_weight("w_routed_up", w_routed_up, w_routed_up_sc, (E, I, H), dev)
    _check_fp8_weight("w_routed_gate_T", w_routed_gate_T, w_routed_gate_T_sc, (E, H, I), dev)
    _check_fp8_weight("w_routed_up_T", w_routed_up_T, w_routed_up_T_sc, (E, H, I), dev)
    _check_fp8_weight("w_routed_down_T", w_routed_down_T, w_routed_down_T_sc, (E, I, H), dev)
    _check_fp8_pair("x_fp8_t_routed", x_fp8_t_routed, x_sc_t_routed, (H, MB), dev)
    _check_fp8_pair("gate_fp8_routed", gate_fp8_routed, gate_sc_routed, (MB, I), dev)
    _check_fp8_pair("up_fp8_routed", up_fp8_routed, up_sc_routed, (MB, I), dev)
    _check_fp8_pair("hidden_fp8_t_routed", hidden_fp8_t_routed, hidden_sc_t_routed, (I, MB), dev)
    _check_bf16_contiguous((("x", x), ("d_y_buffer", d_y_buffer), ("gate_shared", gate_shared), ("up_shared", up_shared),
                            ("hidden_shared", hidden_shared), ("w_shared_gate", w_shared_gate), ("w_shared_up", w_shared_up),
                            ("w_shared_down", w_shared_down)))

    new = lambda *shape: x.new_empty(shape)  # noqa: E731
    d_x_shared, d_x_routed, d_hidden_routed = new(T, H), new(MB, H), new(MB, I)
    d_gate_shared, d_up_shared, d_hidden_shared = new(T, I), new(T, I), new(T, I)
    d_gate_q, d_gate_sc = _new_fp8(x, MB, I)
    d_up_q, d_up_sc = _new_fp8(x, MB, I)
    d_y_q, d_y_sc = _new_fp8(x, MB, H)
    d_w_shared_gate, d_w_shared_up, d_w_shared_down = new(I, H), new(I, H), new(H, I)
    d_w_routed_gate, d_w_routed_up, d_w_routed_down = new(E, I, H), new(E, I, H), new(E, H, I)
    scratch = dict(x_routed=new(MB, H), gate_routed=new(MB, I), up_routed=new(MB, I), hidden_routed=new(MB, I),
                   d_y_routed=new(MB, H), d_gate_routed=new(MB, I), d_up_routed=new(MB, I))
    x_q, x_sc = _new_fp8(x, MB, H)
    hid_q, hid_sc = _new_fp8(x, MB, I)
    d_y_t, d_y_t_sc = _new_fp8(x, H, MB)
    d_gate_t, d_gate_t_sc = _new_fp8(x, I, MB)
    d_up_t, d_up_t_sc = _new_fp8(x, I, MB)
    row_scratch = torch.empty(2 * MB + E + MB * (I // 128), dtype=torch.float32, device=dev)

    a = _layer_args(ep_size=ep_size, rank=_local_rank(x, x_ptrs), x=x, intermediate=I, num_local_experts=E, topk=topk,
                    capacity=cap, macrobatch_size=MB, minibatch_size=minibatch_size, num_comm_sms=num_comm_sms,
                    swiglu_limit=swiglu_limit)
    _keep(a, x_ptrs=x_ptrs, d_y_ptrs=d_y_buffer_ptrs, d_x_routed_ptrs=d_x_routed_buffer_ptrs,
          router_weight_ptrs=router_weight_buffer_ptrs, d_router_weight_ptrs=d_router_weight_buffer_ptrs)
    _set_ptrs(a, peer_rank=schedule_peer_rank, peer_token_idx=schedule_peer_token_idx, num_tokens=num_tokens,
              tokens_per_expert=tokens_per_expert, d_y_local=d_y_buffer,
              w_shared_gate=w_shared_gate, w_shared_up=w_shared_up, w_shared_down=w_shared_down,
              w_gate_fp8=w_routed_gate, w_gate_sc=w_routed_gate_sc, w_up_fp8=w_routed_up, w_up_sc=w_routed_up_sc,
              w_gate_t_fp8=w_routed_gate_T, w_gate_t_sc=w_routed_gate_T_sc, w_up_t_fp8=w_routed_up_T, w_up_t_sc=w_routed_up_T_sc,
              w_down_t_fp8=w_routed_down_T, w_down_t_sc=w_routed_down_T_sc,
              gate_shared=gate_shared, up_shared=up_shared, hidden_shared=hidden_shared,
              x_fp8=x_q, x_sc=x_sc, x_fp8_t=x_fp8_t_routed, x_sc_t=x_sc_t_routed, gate_fp8=gate_fp8_routed, gate_sc=gate_sc_routed,
              up_fp8=up_fp8_routed, up_sc=up_sc_routed, hidden_fp8=hid_q, hidden_sc=hid_sc,
              hidden_fp8_t=hidden_fp8_t_routed, hidden_sc_t=hidden_sc_t_routed,
              d_x_shared=d_x_shared, d_x_routed=d_x_routed, d_hidden_routed=d_hidden_routed,
              d_gate_shared=d_gate_shared, d_up_shared=d_up_shared, d_hidden_shared=d_hidden_shared,
              d_y_fp8=d_y_q, d_y_sc=d_y_sc, d_y_fp8_t=d_y_t, d_y_sc_t=d_y_t_sc,
              d_gate_fp8=d_gate_q, d_gate_sc=d_gate_sc, d_up_fp8=d_up_q, d_up_sc=d_up_sc,
              d_gate_fp8_t=d_gate_t, d_gate_sc_t=d_gate_t_sc, d_up_fp8_t=d_up_t, d_up_sc_t=d_up_t_sc,
              d_w_shared_gate=d_w_shared_gate, d_w_shared_up=d_w_shared_up, d_w_shared_down=d_w_shared_down,
              d_w_routed_gate=d_w_routed_gate, d_w_routed_up=d_w_routed_up, d_w_routed_down=d_w_routed_down,
              row_scratch=row_scratch, **scratch)
    _staging = _attach_dedup(a, x, cap, ('x', 'd_y'), macrobatch_size < cap, dedup_row_source, dedup_unique_peer, dedup_unique_token,
                             dedup_unique_before)  # noqa: F841  (keeps the staging buffers alive until the launch is queued)
    check(lib().mok_moe_backward_mxfp8(_native.ctypes.byref(a), stream_ptr(dev)), "dispatch_mlp_swiglu_combine_bwd_mxfp8")
    return (d_x_shared, d_x_routed, d_gate_shared, d_gate_q, d_gate_sc, d_up_shared, d_up_q, d_up_sc, d_hidden_shared,
            d_hidden_routed, d_y_q, d_y_sc, d_w_shared_gate, d_w_routed_gate, d_w_shared_up, d_w_routed_up, d_w_shared_down,
            d_w_routed_down)


# ------------------------------------------------------------------------------------------------------------
# router (no counterpart among the reference's ops: there the routes and router weights are inputs)
# ------------------------------------------------------------------------------------------------------------
def _router_terms(w_router: torch.Tensor, padded: int):
    """[E, H] router weight -> bf16 (hi, lo) terms padded with zero rows to `padded` experts; lo is None for bf16 input
    (hi + lo carries an fp32 weight to about 16 mantissa bits)."""
    w32 = w_router.float()
    hi = w32.to(torch.bfloat16)
    lo = (w32 - hi.float()).to(torch.bfloat16) if w_router.dtype == torch.float32 else None
    pad = padded - w_router.shape[0]
    if pad:
        hi = torch.nn.functional.pad(hi, (0, 0, 0, pad))
        lo = torch.nn.functional.pad(lo, (0, 0, 0, pad)) if lo is not None else None
    return hi.contiguous(), (lo.contiguous() if lo is not None else None)


def _check_router(x: torch.Tensor, w_router: torch.Tensor, bias: torch.Tensor | None, topk: int):
    _require(x.ndim == 2, "x must have shape (num_local_tokens, hidden_size)")
    T, H = x.shape
    _require(T > 0 and T % 256 == 0, "num_local_tokens must be positive and divisible by 256")
    _require(H > 0 and H % 256 == 0, "hidden_size must be positive and divisible by 256")
    _require(w_router.ndim == 2 and w_router.shape[1] == H, "w_router must have shape (num_experts, hidden_size)")
    E = w_router.shape[0]
    _require(0 < E <= 1024, "num_experts must be in [1, 1024]")
    _require(type(topk) is int and 0 < topk <= min(E, 32), "topk must be an integer in [1, min(num_experts, 32)]")
    _require(x.is_cuda and w_router.device == x.device, "x and w_router must be on the same CUDA device")
    _require(x.dtype == torch.bfloat16 and x.is_contiguous(), "x must be contiguous bfloat16", TypeError)
    _require(w_router.dtype in (torch.float32, torch.bfloat16) and w_router.is_contiguous(),
             "w_router must be contiguous float32 or bfloat16", TypeError)
    if bias is not None:
        _require(tuple(bias.shape) == (E,) and bias.device == x.device, "bias must have shape (num_experts,) on the device of x")
        _require(bias.dtype == torch.float32 and bias.is_contiguous(), "bias must be contiguous float32", TypeError)
    return T, H, E, -(-E // 256) * 256


@torch.library.custom_op("mok::router_fwd", mutates_args=())
def router_fwd(x: torch.Tensor, w_router: torch.Tensor, bias: torch.Tensor | None, topk: int
               ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """logits = x @ w_router.T (+ bias) in fp32, top-k (descending, ties to the lower index), softmax over the selected
    logits.

    Inputs:  x bf16 [T, H]; w_router f32 | bf16 [E, H]; bias f32 [E] | None; topk int
    Outputs: top_experts int32 [T, topk]; router_weights f32 [T, topk]; logits f32 [T, E] (without the bias)
    """
    T, H, E, padded = _check_router(x, w_router, bias, topk)
    hi, lo = _router_terms(w_router, padded)
    logits = torch.empty((T, padded), dtype=torch.float32, device=x.device)
    routes = torch.empty((T, topk), dtype=torch.int32, device=x.device)
    weights = torch.empty((T, topk), dtype=torch.float32, device=x.device)
    check(lib().mok_router_forward(ptr(x), ptr(hi), ptr(lo), ptr(bias), T, H, E, padded, topk, ptr(logits), ptr(routes),
                                   ptr(weights), ptr(status_word(x.device)), stream_ptr(x.device)), "router_fwd")
    return routes, weights, (logits if padded == E else logits[:, :E].contiguous())


@torch.library.custom_op("mok::router_bwd", mutates_args=())
def router_bwd(x: torch.Tensor, w_router: torch.Tensor, top_experts: torch.Tensor, router_weights: torch.Tensor,
               d_router_weights: torch.Tensor, has_bias: bool) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradient of router_fwd's weights with respect to x, w_router and the bias.

    Inputs:  x bf16 [T, H]; w_router [E, H]; top_experts int32 [T, topk]; router_weights, d_router_weights f32 [T, topk]
    Outputs: d_x bf16 [T, H]; d_w_router f32 [E, H]; d_bias f32 [E] (zeros when has_bias is False)
    """
    _require(top_experts.ndim == 2, "top_experts must have shape (num_local_tokens, topk)")
    topk = top_experts.shape[1]
    T, H, E, padded = _check_router(x, w_router, None, topk)
    for name, t, dt in (("top_experts", top_experts, torch.int32), ("router_weights", router_weights, torch.float32),
                        ("d_router_weights", d_router_weights, torch.float32)):
        _require(tuple(t.shape) == (T, topk) and t.device == x.device, f"{name} must have shape (num_local_tokens, topk) on the device of x")
        _require(t.dtype == dt and t.is_contiguous(), f"{name} must be contiguous {dt}", TypeError)
    hi, _ = _router_terms(w_router, padded)
    d_logits = torch.empty((T, padded), dtype=torch.bfloat16, device=x.device)
    d_x = torch.empty_like(x)
    d_w = torch.empty((padded, H), dtype=torch.float32, device=x.device)
    d_bias = torch.zeros((E,), dtype=torch.float32, device=x.device)
    check(lib().mok_router_backward(ptr(x), ptr(hi), ptr(top_experts), ptr(router_weights), ptr(d_router_weights), T, H, E, padded,
                                    topk, ptr(d_logits), ptr(d_x), ptr(d_w), ptr(d_bias) if has_bias else ptr(None),
                                    ptr(status_word(x.device)), stream_ptr(x.device)), "router_bwd")
    return d_x, d_w[:E].contiguous() if padded != E else d_w, d_bias
