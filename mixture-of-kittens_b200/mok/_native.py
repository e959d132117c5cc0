"""ctypes binding of libmok_b200.so (the C ABI declared in include/mok_b200.h).

The library is the only compute backend: if it is missing or a call fails, the error is raised — there is no
fallback path.  Build it with `python mixture-of-kittens_b200/build.py`.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int32, c_int64, c_uint32, c_uint64, c_void_p, c_char_p, POINTER

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "libmok_b200.so")
_lib = None

MOK_OK = 0
_ERRORS = {-1: "invalid argument", -2: "unsupported configuration", -3: "CUDA error", -4: "size beyond the library's limits"}
STATUS_BITS = {
    1: "schedule overflow: padded routes exceed schedule_capacity (raise schedule_capacity_multiplier)",
    2: "cross-GPU barrier wait ran out",
    4: "a GEMM pipeline wait ran out",
    8: "a schedule row named a peer or token outside the buffers",
}
MAX_EP = 8


class LayerArgs(ctypes.Structure):
    """Mirror of `mok_layer_args` (include/mok_b200.h)."""
    _fields_ = (
        [(n, c_int) for n in ("ep_size", "rank", "num_local_tokens", "hidden", "intermediate", "num_local_experts", "topk",
                              "schedule_capacity", "macrobatch_size", "minibatch_size", "num_comm_sms", "has_swiglu_limit")]
        + [("swiglu_limit", c_float), ("reserved0", c_int)]
        + [(n, c_void_p) for n in (
            "peer_rank", "peer_token_idx", "num_tokens", "tokens_per_expert",
            "x_local", "d_y_local", "x_ptrs", "combine_ptrs", "d_y_ptrs", "d_x_routed_ptrs", "router_weight_ptrs", "d_router_weight_ptrs",
            "w_shared_gate", "w_shared_up", "w_shared_down", "w_routed_gate", "w_routed_up", "w_routed_down",
            "x_routed", "gate_shared", "up_shared", "hidden_shared", "gate_routed", "up_routed", "hidden_routed",
            "y_shared", "y_routed",
            "d_x_shared", "d_x_routed", "d_gate_shared", "d_up_shared", "d_hidden_shared",
            "d_gate_routed", "d_up_routed", "d_hidden_routed", "d_y_routed",
            "d_w_shared_gate", "d_w_shared_up", "d_w_shared_down", "d_w_routed_gate", "d_w_routed_up", "d_w_routed_down",
            "row_scratch", "status",
            "w_gate_fp8", "w_gate_sc", "w_up_fp8", "w_up_sc", "w_down_fp8", "w_down_sc",
            "w_gate_t_fp8", "w_gate_t_sc", "w_up_t_fp8", "w_up_t_sc", "w_down_t_fp8", "w_down_t_sc",
            "x_fp8", "x_sc", "x_fp8_t", "x_sc_t", "gate_fp8", "gate_sc", "up_fp8", "up_sc",
            "hidden_fp8", "hidden_sc", "hidden_fp8_t", "hidden_sc_t", "d_y_fp8", "d_y_sc", "d_y_fp8_t", "d_y_sc_t",
            "d_gate_fp8", "d_gate_sc", "d_up_fp8", "d_up_sc", "d_gate_fp8_t", "d_gate_sc_t", "d_up_fp8_t", "d_up_sc_t",
            "row_source", "unique_peer", "unique_token", "unique_before", "staged_x", "staged_d_y")]
        + [("staged_rows", c_int), ("reserved1", c_int)]
    )


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(f"{_LIB_PATH} is missing: build it with `python mixture-of-kittens_b200/build.py`; "
                              "there is no fallback implementation")
        L = ctypes.CDLL(_LIB_PATH)
        L.mok_version.restype = c_int
        L.mok_last_error.restype = c_char_p
        L.mok_launch_count.restype = ctypes.c_longlong
        L.mok_schedule_scratch_bytes.restype = c_int64
        L.mok_schedule_scratch_bytes.argtypes = [c_int, c_int, c_int, c_int]
        L.mok_schedule.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_void_p]
        L.mok_schedule_static.argtypes = [c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p,
                                          c_void_p, c_void_p, c_void_p]
        L.mok_schedule_static.restype = c_int
        L.mok_schedule_dedup_scratch_bytes.restype = c_int64
        L.mok_schedule_dedup_scratch_bytes.argtypes = [c_int, c_int, c_int, c_int]
        L.mok_schedule_dedup.argtypes = [c_void_p] + [c_int] * 6 + [c_void_p] * 8 + [c_int, c_void_p, c_void_p]
        L.mok_schedule_dedup.restype = c_int
        L.mok_stage_unique_rows.argtypes = [POINTER(c_uint64), c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                            c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p]
        L.mok_stage_unique_rows.restype = c_int
        L.mok_dispatch_rows_staged.argtypes = [POINTER(c_uint64), POINTER(c_uint64), c_int, c_int, c_void_p, c_void_p, c_void_p,
                                               c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p,
                                               c_int, c_void_p, c_void_p]
        L.mok_dispatch_rows_staged.restype = c_int
        L.mok_all_gather_top_experts.argtypes = [c_void_p, c_int64, POINTER(c_uint64), c_int, c_int, c_void_p]
        L.mok_barrier_all.argtypes = [c_void_p, POINTER(c_uint64), c_int, c_void_p, c_void_p, c_int, c_void_p]
        L.mok_fwd_epilogue.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]
        L.mok_bwd_epilogue.argtypes = [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]
        L.mok_mxfp8_quantize.argtypes = [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]
        for name in ("mok_moe_forward_bf16", "mok_moe_recompute_bf16", "mok_moe_backward_bf16",
                     "mok_moe_forward_mxfp8", "mok_moe_recompute_mxfp8", "mok_moe_backward_mxfp8"):
            getattr(L, name).argtypes = [POINTER(LayerArgs), c_void_p]
            getattr(L, name).restype = c_int
        L.mok_grouped_gemm_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                            c_int, c_void_p, c_void_p]
        L.mok_grouped_wgrad_bf16.argtypes = [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                             c_void_p, c_void_p]
        L.mok_trace_dump.argtypes = [c_char_p]
        L.mok_trace_dump.restype = c_int
        L.mok_dispatch_rows.argtypes = [POINTER(c_uint64), POINTER(c_uint64), c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                        c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        L.mok_combine_rows.argtypes = [POINTER(c_uint64), POINTER(c_uint64), c_int, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                       c_int, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]
        L.mok_dispatch_rows.restype = c_int
        L.mok_combine_rows.restype = c_int
        L.mok_grouped_gemm_mxfp8.argtypes = [c_void_p] * 7 + [c_int] * 4 + [c_void_p, c_void_p]
        L.mok_grouped_wgrad_mxfp8.argtypes = [c_void_p] * 7 + [c_int] * 4 + [c_void_p, c_void_p]
        L.mok_grouped_gemm_mxfp8.restype = c_int
        L.mok_grouped_wgrad_mxfp8.restype = c_int
        L.mok_router_forward.argtypes = [c_void_p] * 4 + [c_int64] + [c_int] * 4 + [c_void_p] * 5
        L.mok_router_backward.argtypes = [c_void_p] * 5 + [c_int64] + [c_int] * 4 + [c_void_p] * 6
        L.mok_router_forward.restype = c_int
        L.mok_router_backward.restype = c_int
        for name in ("mok_schedule", "mok_all_gather_top_experts", "mok_barrier_all", "mok_fwd_epilogue", "mok_bwd_epilogue",
                     "mok_mxfp8_quantize", "mok_moe_forward_bf16", "mok_moe_recompute_bf16", "mok_moe_backward_bf16",
                     "mok_grouped_gemm_bf16", "mok_grouped_wgrad_bf16"):
            getattr(L, name).restype = c_int
        _lib = L
    return _lib


def check(rc: int, what: str) -> None:
    if rc == MOK_OK:
        return
    detail = lib().mok_last_error().decode() if rc == -3 else ""
    if rc == -2:
        raise NotImplementedError(f"{what}: {_ERRORS[rc]}")
    raise RuntimeError(f"{what} failed: {_ERRORS.get(rc, rc)} {detail}".strip())


def stream_ptr(device: torch.device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def ptr_array(values) -> ctypes.Array:
    return (c_uint64 * len(values))(*[int(v) for v in values])


_STATUS: dict[int, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """uint32-sized device word the kernels OR their error bits into (one per device)."""
    index = device.index if device.index is not None else torch.cuda.current_device()
    word = _STATUS.get(index)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", index))
        _STATUS[index] = word
    return word


def check_status(device: torch.device | None = None, *, reset: bool = True) -> None:
    """Reads the device status word (this synchronises) and raises if a kernel reported a problem."""
    devices = list(_STATUS) if device is None else [device.index if device.index is not None else torch.cuda.current_device()]
    for index in devices:
        word = _STATUS.get(index)
        if word is None:
            continue
        bits = int(word.item())
        if bits:
            if reset:
                word.zero_()
            raise RuntimeError("MoK device status: " + "; ".join(msg for bit, msg in STATUS_BITS.items() if bits & bit))
