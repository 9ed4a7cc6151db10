"""`torch.library` custom ops around the layer's kernels, so that `torch.compile(fullgraph=True)` can trace
`MoE.forward`: Dynamo treats each op as opaque instead of trying to look into the ctypes calls.

The reference registers every kernel as a custom op for the same reason (sonicmoe/functional/forward.py,
backward.py).  Here the granularity is coarser -- router top-k, routing metadata, routed experts forward,
routed experts backward -- because nothing between those kernels needs to be visible to the compiler.
The eager path does not go through these ops; `moe_TC_softmax_topk_layer` switches to them only while
compiling.
"""

from __future__ import annotations

import torch
from torch import Tensor

from . import Route, _RoutedExperts, _TopkSoftmax, _route_metadata

NS = "sonicmoe_b200"


class _Ctx:
    """Stand-in for the autograd context when a Function's forward/backward is called directly."""

    def __init__(self):
        self.saved_tensors = ()

    def save_for_backward(self, *tensors):
        self.saved_tensors = tensors

    def mark_non_differentiable(self, *a):
        pass


# ---- top-k + softmax ----------------------------------------------------------------------------------
@torch.library.custom_op(f"{NS}::topk_softmax", mutates_args=(), device_types="cuda")
def topk_softmax_op(logits: Tensor, K: int) -> tuple[Tensor, Tensor]:
    return _TopkSoftmax.forward(_Ctx(), logits, K)


@topk_softmax_op.register_fake
def _(logits, K):
    T = logits.shape[0]
    return logits.new_empty((T, K), dtype=torch.float32), logits.new_empty((T, K), dtype=torch.int32)


@torch.library.custom_op(f"{NS}::topk_softmax_backward", mutates_args=(), device_types="cuda")
def topk_softmax_backward_op(dscores: Tensor, scores: Tensor, indices: Tensor, E: int, bf16_logits: bool) -> Tensor:
    ctx = _Ctx()
    ctx.saved_tensors = (scores, indices)
    ctx.E = E
    ctx.logits_dtype = torch.bfloat16 if bf16_logits else torch.float32
    return _TopkSoftmax.backward(ctx, dscores, None)[0]


@topk_softmax_backward_op.register_fake
def _(dscores, scores, indices, E, bf16_logits):
    return scores.new_empty((scores.shape[0], E), dtype=torch.bfloat16 if bf16_logits else torch.float32)


def _topk_setup(ctx, inputs, output):
    logits, _K = inputs
    scores, indices = output
    ctx.save_for_backward(scores, indices)
    ctx.E = logits.shape[1]
    ctx.bf16 = logits.dtype == torch.bfloat16


def _topk_backward(ctx, dscores, _dindices):
    scores, indices = ctx.saved_tensors
    return topk_softmax_backward_op(dscores.contiguous(), scores, indices, ctx.E, ctx.bf16), None


topk_softmax_op.register_autograd(_topk_backward, setup_context=_topk_setup)


# ---- routing metadata ---------------------------------------------------------------------------------
@torch.library.custom_op(f"{NS}::route_metadata", mutates_args=(), device_types="cuda")
def route_metadata_op(expert_idx: Tensor, E: int, K: int) -> tuple[Tensor, Tensor, Tensor, Tensor, Tensor]:
    r = _route_metadata(expert_idx, None, E, K)
    # the three index vectors are rows of one buffer: hand out independent tensors
    return (r.expert_frequency, r.expert_frequency_offset, r.x_gather_idx.clone(), r.s_scatter_idx.clone(),
            r.s_reverse_scatter_idx.clone())


@route_metadata_op.register_fake
def _(expert_idx, E, K):
    n = expert_idx.numel()
    i32 = dict(dtype=torch.int32)
    return (expert_idx.new_empty((E,), **i32), expert_idx.new_empty((E + 1,), **i32),
            expert_idx.new_empty((n,), **i32), expert_idx.new_empty((n,), **i32), expert_idx.new_empty((n,), **i32))


# ---- routed experts -----------------------------------------------------------------------------------
def _route(freq, off, gather, scatter, reverse, K):
    return Route(freq, off, gather, scatter, reverse, None, K)


@torch.library.custom_op(f"{NS}::routed_experts", mutates_args=(), device_types="cuda")
def routed_experts_op(x: Tensor, w1e: Tensor, w2e: Tensor, scores: Tensor, off: Tensor, gather: Tensor,
                      scatter: Tensor, reverse: Tensor, K: int, inference: bool) -> tuple[Tensor, Tensor]:
    ctx = _Ctx()
    route = _route(None, off, gather, scatter, reverse, K)
    o = _RoutedExperts.forward(ctx, x, w1e.permute(1, 2, 0), w2e.permute(1, 2, 0), scores, route, x.shape[0],
                               inference)
    z = ctx.saved_tensors[3] if ctx.saved_tensors else x.new_empty((0,))
    return o, z


@routed_experts_op.register_fake
def _(x, w1e, w2e, scores, off, gather, scatter, reverse, K, inference):
    z = x.new_empty((0,)) if inference else x.new_empty((gather.numel(), w1e.shape[1]))
    return torch.empty_like(x), z


@torch.library.custom_op(f"{NS}::routed_experts_backward", mutates_args=(), device_types="cuda")
def routed_experts_backward_op(dout: Tensor, x: Tensor, w1e: Tensor, w2e: Tensor, z: Tensor, scores: Tensor,
                               off: Tensor, gather: Tensor, scatter: Tensor, reverse: Tensor,
                               K: int) -> tuple[Tensor, Tensor, Tensor, Tensor]:
    ctx = _Ctx()
    ctx.saved_tensors = (x, w1e, w2e, z, scores)
    ctx.route = _route(None, off, gather, scatter, reverse, K)
    E, two_i, H = w1e.shape
    ctx.dims = (x.shape[0], H, two_i // 2, E, gather.numel())
    dx, dw1, dw2, ds = _RoutedExperts.backward(ctx, dout)[:4]
    return dx, dw1.permute(2, 0, 1), dw2.permute(2, 0, 1), ds  # back to (E, out, in) storage order


@routed_experts_backward_op.register_fake
def _(dout, x, w1e, w2e, z, scores, off, gather, scatter, reverse, K):
    return torch.empty_like(x), torch.empty_like(w1e), torch.empty_like(w2e), torch.empty_like(scores)


def _experts_setup(ctx, inputs, output):
    x, w1e, w2e, scores, off, gather, scatter, reverse, K, inference = inputs
    _o, z = output
    ctx.save_for_backward(x, w1e, w2e, z, scores, off, gather, scatter, reverse)
    ctx.K = K


def _experts_backward(ctx, dout, _dz):
    x, w1e, w2e, z, scores, off, gather, scatter, reverse = ctx.saved_tensors
    dx, dw1, dw2, ds = routed_experts_backward_op(dout.contiguous(), x, w1e, w2e, z, scores, off, gather, scatter,
                                                  reverse, ctx.K)
    return dx, dw1, dw2, ds, None, None, None, None, None, None


routed_experts_op.register_autograd(_experts_backward, setup_context=_experts_setup)


def layer_with_custom_ops(x, router_logits, w1, w2, K, E, inference):
    """The body of `moe_TC_softmax_topk_layer` after the router linear, expressed with the custom ops."""
    scores, indices = topk_softmax_op(router_logits.contiguous(), K)
    freq, off, gather, scatter, reverse = route_metadata_op(indices.reshape(-1), E, K)
    w1e = w1.permute(2, 0, 1).contiguous()
    w2e = w2.permute(2, 0, 1).contiguous()
    o, _z = routed_experts_op(x.contiguous(), w1e, w2e, scores.reshape(-1), off, gather, scatter, reverse, K,
                              inference)
    return o, freq
