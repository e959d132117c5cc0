"""Shape/dtype functions ("fake" implementations) of the `mok::*` ops, so FakeTensor tracing and
`torch.compile(fullgraph=True)` see the same outputs the CUDA ops allocate (reference: mok/_fake_impls.py)."""
import torch

from . import ops as _ops  # noqa: F401  (the ops must be defined before their fakes are registered)

_FP8 = torch.float8_e4m3fn
_U8 = torch.uint8


def _sc(t, rows, cols):
    return t.new_empty((rows // 128, cols // 128, 32, 16), dtype=_U8)


@torch.library.register_fake("mok::all_gather_top_experts")
def _(top_experts, all_gather_top_experts_buffer, all_gather_top_experts_buffer_multicast_ptr, rank, chunk_bytes,
      peer_buffer_ptrs=None):
    return None


@torch.library.register_fake("mok::barrier_all")
def _(barrier_buffer, barrier_buffer_ptrs, barrier_buffer_multicast_ptr, target):
    return None


@torch.library.register_fake("mok::schedule")
def _(topk_all, num_local_experts, schedule_capacity, rank):
    i32 = dict(dtype=torch.int32)
    return (topk_all.new_empty((schedule_capacity,), **i32), topk_all.new_empty((schedule_capacity,), **i32),
            topk_all.new_empty((1,), **i32), topk_all.new_empty((num_local_experts,), **i32))


@torch.library.register_fake("mok::schedule_dedup")
def _(topk_all, schedule_peer_rank, schedule_peer_token_idx, num_tokens, num_local_experts, rank):
    i32 = dict(dtype=torch.int32)
    cap = schedule_peer_rank.shape[0]
    unique = min(cap, topk_all.shape[0] * topk_all.shape[1])
    return (topk_all.new_empty((cap,), **i32), topk_all.new_empty((unique,), **i32), topk_all.new_empty((unique,), **i32),
            topk_all.new_empty((cap // 256 + 1,), **i32), topk_all.new_empty((1,), **i32))


@torch.library.register_fake("mok::mxfp8_quantize")
def _(x_bf16, return_normal, return_transposed):
    e = x_bf16.shape[0] if x_bf16.ndim == 3 else 1
    rows, cols = x_bf16.shape[-2], x_bf16.shape[-1]
    t_shape = (e, cols, rows) if x_bf16.ndim == 3 else (cols, rows)
    return (x_bf16.new_empty(x_bf16.shape, dtype=_FP8) if return_normal else None,
            _sc(x_bf16, e * rows, cols) if return_normal else None,
            x_bf16.new_empty(t_shape, dtype=_FP8) if return_transposed else None,
            _sc(x_bf16, e * cols, rows) if return_transposed else None)


def _fwd_mxfp8_context(x, w_shared_gate, macrobatch_size):
    t, h = x.shape
    i = w_shared_gate.shape[0]
    mb = macrobatch_size
    return (x.new_empty((h, mb), dtype=_FP8), _sc(x, h, mb),
            x.new_empty((t, i)), x.new_empty((mb, i), dtype=_FP8), _sc(x, mb, i),
            x.new_empty((t, i)), x.new_empty((mb, i), dtype=_FP8), _sc(x, mb, i),
            x.new_empty((t, i)), x.new_empty((i, mb), dtype=_FP8), _sc(x, i, mb))


def _fwd_bf16_context(x, w_shared_gate, macrobatch_size):
    t, h = x.shape
    i = w_shared_gate.shape[0]
    mb = macrobatch_size
    return (x.new_empty((mb, h)), x.new_empty((t, i)), x.new_empty((mb, i)), x.new_empty((t, i)), x.new_empty((mb, i)),
            x.new_empty((t, i)), x.new_empty((mb, i)))


@torch.library.register_fake("mok::dispatch_mlp_swiglu_combine_fwd_mxfp8")
def _(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up,
      w_routed_up, w_routed_up_sc, w_shared_down, w_routed_down, w_routed_down_sc, schedule_peer_rank,
      schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size,
      minibatch_size, dedup_row_source=None, dedup_unique_peer=None,
      dedup_unique_token=None, dedup_unique_before=None):
    return _fwd_mxfp8_context(x, w_shared_gate, macrobatch_size) + (x.new_empty(x.shape), x.new_empty((macrobatch_size, x.shape[1])))


@torch.library.register_fake("mok::dispatch_mlp_swiglu_combine_fwd_bf16")
def _(x, x_ptrs, combine_buffer, combine_buffer_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up,
      w_shared_down, w_routed_down, schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk,
      swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, dedup_row_source=None, dedup_unique_peer=None,
      dedup_unique_token=None, dedup_unique_before=None):
    return _fwd_bf16_context(x, w_shared_gate, macrobatch_size) + (x.new_empty(x.shape), x.new_empty((macrobatch_size, x.shape[1])))


@torch.library.register_fake("mok::recompute_forward_context_mxfp8")
def _(x, x_ptrs, w_shared_gate, w_routed_gate, w_routed_gate_sc, w_shared_up, w_routed_up, w_routed_up_sc,
      schedule_peer_rank, schedule_peer_token_idx, num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms,
      macrobatch_size, minibatch_size, dedup_row_source=None, dedup_unique_peer=None,
      dedup_unique_token=None, dedup_unique_before=None):
    return _fwd_mxfp8_context(x, w_shared_gate, macrobatch_size)


@torch.library.register_fake("mok::recompute_forward_context_bf16")
def _(x, x_ptrs, w_shared_gate, w_routed_gate, w_shared_up, w_routed_up, schedule_peer_rank, schedule_peer_token_idx,
      num_tokens, tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, dedup_row_source=None, dedup_unique_peer=None,
      dedup_unique_token=None, dedup_unique_before=None):
    return _fwd_bf16_context(x, w_shared_gate, macrobatch_size)


def _wgrads(d, e, i, h):
    return (d.new_empty((i, h)), d.new_empty((e, i, h)), d.new_empty((i, h)), d.new_empty((e, i, h)),
            d.new_empty((h, i)), d.new_empty((e, h, i)))


@torch.library.register_fake("mok::dispatch_mlp_swiglu_combine_bwd_mxfp8")
def _(d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
      router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs, w_shared_gate, w_routed_gate_T,
      w_routed_gate_T_sc, w_shared_up, w_routed_up_T, w_routed_up_T_sc, w_shared_down, w_routed_down_T,
      w_routed_down_T_sc, x_fp8_t_routed, x_sc_t_routed, gate_shared, gate_fp8_routed, gate_sc_routed, up_shared,
      up_fp8_routed, up_sc_routed, hidden_shared, hidden_fp8_t_routed, hidden_sc_t_routed, x, x_ptrs, w_routed_gate,
      w_routed_gate_sc, w_routed_up, w_routed_up_sc, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
      tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, dedup_row_source=None, dedup_unique_peer=None,
      dedup_unique_token=None, dedup_unique_before=None):
    d = d_y_buffer
    t, h = d.shape
    i = w_shared_gate.shape[0]
    e = w_routed_gate.shape[0]
    mb = macrobatch_size
    return (d.new_empty((t, h)), d.new_empty((mb, h)),
            d.new_empty((t, i)), d.new_empty((mb, i), dtype=_FP8), _sc(d, mb, i),
            d.new_empty((t, i)), d.new_empty((mb, i), dtype=_FP8), _sc(d, mb, i),
            d.new_empty((t, i)), d.new_empty((mb, i)), d.new_empty((mb, h), dtype=_FP8), _sc(d, mb, h)) + _wgrads(d, e, i, h)


@torch.library.register_fake("mok::dispatch_mlp_swiglu_combine_bwd_bf16")
def _(d_y_buffer, d_y_buffer_ptrs, d_x_routed_buffer, d_x_routed_buffer_ptrs, router_weight_buffer,
      router_weight_buffer_ptrs, d_router_weight_buffer, d_router_weight_buffer_ptrs, w_shared_gate, w_routed_gate,
      w_shared_up, w_routed_up, w_shared_down, w_routed_down, x_routed, gate_shared, gate_routed, up_shared, up_routed,
      hidden_shared, hidden_routed, x, x_ptrs, schedule_peer_rank, schedule_peer_token_idx, num_tokens,
      tokens_per_expert, topk, swiglu_limit, num_comm_sms, macrobatch_size, minibatch_size, dedup_row_source=None, dedup_unique_peer=None,
      dedup_unique_token=None, dedup_unique_before=None):
    d = d_y_buffer
    t, h = d.shape
    i = w_shared_gate.shape[0]
    e = w_routed_gate.shape[0]
    mb = macrobatch_size
    return (d.new_empty((t, h)), d.new_empty((mb, h)), d.new_empty((t, i)), d.new_empty((mb, i)), d.new_empty((t, i)),
            d.new_empty((mb, i)), d.new_empty((t, i)), d.new_empty((mb, i)), d.new_empty((mb, h))) + _wgrads(d, e, i, h)


@torch.library.register_fake("mok::fwd_epilogue")
def _(y_shared, combine_buffer, topk_weights):
    return torch.empty_like(y_shared)


@torch.library.register_fake("mok::bwd_epilogue")
def _(d_x_shared, d_x_routed_buffer):
    return torch.empty_like(d_x_shared)


@torch.library.register_fake("mok::router_fwd")
def _(x, w_router, bias, topk):
    T, E = x.shape[0], w_router.shape[0]
    return (x.new_empty((T, topk), dtype=torch.int32), x.new_empty((T, topk), dtype=torch.float32),
            x.new_empty((T, E), dtype=torch.float32))


@torch.library.register_fake("mok::router_bwd")
def _(x, w_router, top_experts, router_weights, d_router_weights, has_bias):
    E, H = w_router.shape
    return (torch.empty_like(x), x.new_empty((E, H), dtype=torch.float32), x.new_empty((E,), dtype=torch.float32))
