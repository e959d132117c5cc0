"""Autograd and `nn.Module` front ends over `mok.functional` (what a trainer calls).

The reference leaves this wrapper to the user (its README shows the calls by hand); it is provided here so that a
layer can be dropped into a model: `moe_layer(...)` is a differentiable function of x, the router weights and the
expert weights, `MoKMoE` a module with its own top-k softmax router.  With `recompute=True` only the layer inputs are
kept between forward and backward and the activations are rebuilt by `recompute_forward_context` (manual activation
checkpointing, reference README "recompute" section).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import functional as F
from . import ops


def quantize_routed_weights(w_routed_gate: torch.Tensor, w_routed_up: torch.Tensor, w_routed_down: torch.Tensor):
    """MXFP8 copies of the routed expert weights, each as (e4m3, scales, e4m3 of the transpose, its scales): what the
    MXFP8 forward and backward consume.  A trainer computes them once per optimizer step (or once, for inference) and
    passes them to `moe_layer(..., quantized_weights=...)`; `MoKMoE` caches them until a weight changes."""
    return tuple(ops.mxfp8_quantize(w, True, True) for w in (w_routed_gate, w_routed_up, w_routed_down))


class _MoKLayerFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, router_weights, w_shared_gate, w_shared_up, w_shared_down, w_routed_gate, w_routed_up, w_routed_down,
                config, workspace, schedule, swiglu_limit, recompute, mxfp8, quantized):
        weights = (w_shared_gate, w_shared_up, w_shared_down, w_routed_gate, w_routed_up, w_routed_down)
        if mxfp8:
            qg, qu, qd = quantized if quantized is not None else quantize_routed_weights(w_routed_gate, w_routed_up, w_routed_down)
            fwd_routed = ((qg[0], qg[1]), (qu[0], qu[1]), (qd[0], qd[1]))
            ctx.bwd_routed = (qg, qu, (qd[2], qd[3]))
        else:
            fwd_routed = weights[3:]
            ctx.bwd_routed = weights[3:]
        out, fwd_ctx = F.forward(config, workspace, schedule, x, router_weights, *weights[:3], *fwd_routed, swiglu_limit=swiglu_limit)
        ctx.save_for_backward(x, router_weights, *weights[:3])
        ctx.fwd_routed = fwd_routed
        ctx.fwd_ctx = None if recompute else fwd_ctx
        ctx.args = (config, workspace, schedule, swiglu_limit)
        return out

    @staticmethod
    def backward(ctx, d_out):
        x, router_weights, wsg, wsu, wsd = ctx.saved_tensors
        config, workspace, schedule, swiglu_limit = ctx.args
        fwd_ctx = ctx.fwd_ctx
        if fwd_ctx is None:
            fwd_ctx = F.recompute_forward_context(config, workspace, schedule, x, wsg, wsu, ctx.fwd_routed[0], ctx.fwd_routed[1],
                                                  swiglu_limit=swiglu_limit)
        (d_x, d_rw, d_wrg, d_wru, d_wrd, d_wsg, d_wsu, d_wsd) = F.backward(
            config, workspace, schedule, fwd_ctx, d_out.contiguous(), x, router_weights, wsg, wsu, wsd, *ctx.bwd_routed,
            swiglu_limit=swiglu_limit)
        return d_x, d_rw, d_wsg, d_wsu, d_wsd, d_wrg, d_wru, d_wrd, None, None, None, None, None, None, None


class _RouterFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_router, bias, topk):
        routes, weights, _logits = ops.router_fwd(x, w_router, bias, topk)
        ctx.save_for_backward(x, w_router, routes, weights)
        ctx.has_bias = bias is not None
        ctx.mark_non_differentiable(routes)
        return routes, weights

    @staticmethod
    def backward(ctx, _d_routes, d_weights):
        x, w_router, routes, weights = ctx.saved_tensors
        d_x, d_w, d_bias = ops.router_bwd(x, w_router, routes, weights, d_weights.contiguous(), ctx.has_bias)
        return d_x, d_w.to(w_router.dtype), (d_bias if ctx.has_bias else None), None


def route(x: torch.Tensor, w_router: torch.Tensor, bias: torch.Tensor | None = None, *, topk: int
          ) -> tuple[torch.Tensor, torch.Tensor]:
    """Differentiable softmax top-k router on the device: logits = x @ w_router.T (+ bias) in fp32, the topk largest
    per token, weights = softmax over the selected logits.  Returns (top_experts int32 [T, topk], router_weights fp32
    [T, topk]); gradients flow from router_weights to x, w_router ([E, H], fp32 or bf16) and bias."""
    return _RouterFunction.apply(x, w_router, bias, topk)


def moe_layer(x: torch.Tensor, top_experts: torch.Tensor, router_weights: torch.Tensor,
              w_shared_gate: torch.Tensor, w_shared_up: torch.Tensor, w_shared_down: torch.Tensor,
              w_routed_gate: torch.Tensor, w_routed_up: torch.Tensor, w_routed_down: torch.Tensor, *,
              group: dist.ProcessGroup | None = None, config: F.MoKConfig | None = None, swiglu_limit: float | None = None,
              recompute: bool = False, mxfp8: bool = False, quantized_weights=None) -> torch.Tensor:
    """Differentiable MoE layer: output [T, H] bf16 from x [T, H] bf16, top_experts int64 or int32 [T, K], router_weights fp32
    [T, K] and the bf16 expert weights of this rank.  Gradients flow to x, router_weights and all six weights.
    With `mxfp8=True` the routed weights are quantized inside unless `quantized_weights` (from
    `quantize_routed_weights`) is given."""
    config = config or F.MoKConfig()
    group = group or dist.group.WORLD
    workspace = F.get_workspace(config, group, device=x.device, num_local_tokens=x.shape[0], hidden_size=x.shape[1],
                                topk=top_experts.shape[1])
    schedule = F.build_schedule(workspace, config, top_experts, num_local_experts=w_routed_gate.shape[0])
    return _MoKLayerFunction.apply(x, router_weights, w_shared_gate, w_shared_up, w_shared_down, w_routed_gate, w_routed_up,
                                   w_routed_down, config, workspace, schedule, swiglu_limit, recompute, mxfp8, quantized_weights)


class MoKMoE(torch.nn.Module):
    """Expert-parallel MoE layer with a softmax top-k router (weights renormalised over the selected experts), one
    shared expert and `num_experts / ep_size` routed experts on this rank."""

    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, topk: int, *,
                 group: dist.ProcessGroup | None = None, config: F.MoKConfig | None = None, swiglu_limit: float | None = None,
                 recompute: bool = False, mxfp8: bool = False, device=None, init_std: float = 0.02,
                 cache_quantized: bool = True):
        super().__init__()
        self.group = group or dist.group.WORLD
        ep = dist.get_world_size(self.group)
        if num_experts % ep != 0:
            raise ValueError("num_experts must be divisible by the EP size")
        self.topk, self.num_experts = topk, num_experts
        self.config = config or F.MoKConfig()
        self.swiglu_limit, self.recompute, self.mxfp8 = swiglu_limit, recompute, mxfp8
        self._quantized = None
        self.cache_quantized = cache_quantized
        e_loc = num_experts // ep

        def param(*shape, dtype=torch.bfloat16):
            return torch.nn.Parameter(torch.randn(*shape, device=device, dtype=torch.float32).mul_(init_std).to(dtype))
        self.router = param(num_experts, hidden_size, dtype=torch.float32)
        self.w_shared_gate, self.w_shared_up = param(intermediate_size, hidden_size), param(intermediate_size, hidden_size)
        self.w_shared_down = param(hidden_size, intermediate_size)
        self.w_routed_gate, self.w_routed_up = param(e_loc, intermediate_size, hidden_size), param(e_loc, intermediate_size, hidden_size)
        self.w_routed_down = param(e_loc, hidden_size, intermediate_size)

    def invalidate_quantized(self) -> None:
        """Drops the cached MXFP8 copies of the routed weights; the next forward quantizes again.  Call it after any
        weight update the version counters cannot see: writes through `param.data` (fused or foreach optimizers that
        hold flat buffers, ZeRO-style shards, `param.data.copy_`)."""
        self._quantized = None

    def _quantized_weights(self):
        """MXFP8 copies of the routed weights, rebuilt only after one of them changed (optimizer step, load_state_dict).
        The change is detected through the parameters' version counters, which in-place updates of the Parameter bump
        and writes through `.data` do not: after those call `invalidate_quantized()`, or construct the module with
        `cache_quantized=False` to quantize in every forward."""
        params = (self.w_routed_gate, self.w_routed_up, self.w_routed_down)
        key = tuple((p.data_ptr(), p._version) for p in params)
        if not self.cache_quantized or self._quantized is None or self._quantized[0] != key:
            with torch.no_grad():
                self._quantized = (key, quantize_routed_weights(*params))
        return self._quantized[1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        experts, weights = route(x, self.router, topk=self.topk)
        return moe_layer(x, experts, weights, self.w_shared_gate, self.w_shared_up, self.w_shared_down,
                         self.w_routed_gate, self.w_routed_up, self.w_routed_down, group=self.group, config=self.config,
                         swiglu_limit=self.swiglu_limit, recompute=self.recompute, mxfp8=self.mxfp8,
                         quantized_weights=self._quantized_weights() if self.mxfp8 else None)
