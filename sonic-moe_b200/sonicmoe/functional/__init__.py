"""Functional / autograd layer of the MoE hot path, backed by libsonicmoe_b200.so.

Public entry points keep the reference's names and argument conventions
(sonicmoe/functional/__init__.py:423-562):

* ``moe_TC_softmax_topk_layer``  – router linear, top-k + softmax, routed experts (token-choice top-k);
* ``moe_general_routing_inputs`` – routed experts for caller-supplied (score, token, expert) pairs with a
  variable number of experts per token (token rounding uses this);
* ``TC_topk_router_metadata`` / ``general_routing_router_metadata`` – the grouped-row index vectors;
* ``forward_token_choice_rounding`` – the token-rounding router.

Everything runs on the tensors' CUDA device on the *current* stream; the ``stream_id`` arguments are
accepted for call compatibility and ignored (the reference requires them to equal the current stream).
What is saved for backward follows the reference's recompute policy: x, z (pre-activation), scores and
the index vectors are kept; gathered inputs, y1 and y2 are not.
"""

from __future__ import annotations

import os
from contextlib import contextmanager
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import _lib
from .._lib import check, lib, ptr, stream_ptr
from ..count_cumsum import count_cumsum
from ..enums import ActivationType, is_glu
from .token_rounding import forward_token_choice_rounding

__all__ = [
    "count_cumsum",
    "enable_quack_gemm",
    "is_using_quack_gemm",
    "moe_TC_softmax_topk_layer",
    "moe_general_routing_inputs",
    "TC_topk_router_metadata",
    "general_routing_router_metadata",
    "forward_token_choice_rounding",
    "topk_softmax",
    "set_fused_combine",
    "set_fused_router",
    "layer_router_logits",
]


# ------------------------------------------------------------------------------------------------
# toggles
# ------------------------------------------------------------------------------------------------
@contextmanager
def enable_quack_gemm(enable: bool = True):
    """Accepted for source compatibility with the reference (sonicmoe/functional/utils.py:12-25).

    The reference switches to its QuACK GEMMs here; this build has a single GEMM implementation, so the
    context manager changes nothing.
    """
    yield


def is_using_quack_gemm() -> bool:
    return False


# Down-projection epilogue: False = write y2 (TK,H) and reduce it with a deterministic gather-sum;
# True = scatter-reduce into an fp32 (T,H) accumulator from inside the GEMM epilogue (atomic adds).
_FUSED_COMBINE = os.getenv("SONICMOE_FUSED_COMBINE", "0") == "1"


def set_fused_combine(enable: bool) -> bool:
    """Select the fused scatter-reduce epilogue for the down projection; returns the previous setting."""
    global _FUSED_COMBINE
    prev, _FUSED_COMBINE = _FUSED_COMBINE, bool(enable)
    return prev


# ------------------------------------------------------------------------------------------------
# routing metadata
# ------------------------------------------------------------------------------------------------
@dataclass
class Route:
    """Index vectors of one routing decision (all int32, on the activations' device)."""

    expert_frequency: torch.Tensor         # (E,)   rows per expert
    expert_frequency_offset: torch.Tensor  # (E+1,) first grouped row of each expert
    x_gather_idx: torch.Tensor             # (TK,)  token of each grouped row
    s_scatter_idx: torch.Tensor            # (TK,)  flat (token, k) slot of each grouped row
    s_reverse_scatter_idx: torch.Tensor    # (TK,)  grouped row of each flat slot
    token_offset: torch.Tensor | None      # (T+1,) first flat slot of each token; None = fixed K per token
    K: int                                 # experts per token when token_offset is None
    # called in the backward pass with dx as soon as it exists (before the weight-gradient GEMMs are launched): an
    # expert-parallel caller starts sending dx back to the tokens' ranks while those GEMMs run
    on_dx: object = None
    # shared by the chunks of one batch whose rows reach the same experts in several calls (`WeightGradSum`)
    wgrad_sum: object = None


class WeightGradSum:
    """One pair of weight-gradient buffers for ``chunks`` calls of the routed experts on the same weights.

    The first backward pass to run stores its dW1 / dW2, every later one adds to them inside the weight-gradient
    GEMMs' epilogue (`smoe_*_weight_grad_accumulate`), and only the last returns gradients to autograd (the others
    return None).  The result is what autograd's own accumulation of per-chunk bf16 gradients gives (bit for bit
    with two chunks), without a full set of gradient tensors per chunk and the read-add-write pass that adds them.
    Every chunk's backward pass has to run (all chunk outputs feed the loss)."""

    def __init__(self, chunks: int):
        self.remaining = chunks
        self.dw1 = self.dw2 = None

    def buffers(self, w1e, w2e):
        """(dw1, dw2, accumulate?) for the chunk whose backward pass runs now."""
        first = self.dw1 is None
        if first:
            self.dw1, self.dw2 = torch.empty_like(w1e), torch.empty_like(w2e)
        return self.dw1, self.dw2, not first

    def finish_chunk(self):
        """The gradients if this was the last chunk, else (None, None)."""
        self.remaining -= 1
        if self.remaining > 0:
            return None, None
        dw1, dw2 = self.dw1, self.dw2
        self.dw1 = self.dw2 = None
        return dw1, dw2


def _one_row_per_token(route: "Route", T: int) -> bool:
    """Every token has exactly one routed row (top-1 routing, or the rows an expert-parallel rank received): the
    combine and the dX reduction are permutations, which the GEMM epilogues write directly."""
    return route.token_offset is None and route.K == 1 and route.x_gather_idx.numel() == T


def _route_metadata(expert_idx: torch.Tensor, token_idx: torch.Tensor | None, E: int, K: int) -> Route:
    dev = expert_idx.device
    _lib.require_cuda(expert_idx, "expert indices")
    n = expert_idx.numel()
    expert_idx = expert_idx.contiguous()
    if expert_idx.dtype != torch.int32:
        expert_idx = expert_idx.to(torch.int32)
    if token_idx is not None:
        token_idx = token_idx.contiguous()
        if token_idx.dtype != torch.int32:
            token_idx = token_idx.to(torch.int32)
    with torch.cuda.device(dev):
        freq = torch.empty(E, dtype=torch.int32, device=dev)
        off = torch.empty(E + 1, dtype=torch.int32, device=dev)
        idx3 = torch.empty(3, n, dtype=torch.int32, device=dev)
        ws = _lib.device_state(dev).route_workspace(E)
        rc = lib.smoe_route_metadata(
            expert_idx.data_ptr(), ptr(token_idx), n, E, max(K, 1), freq.data_ptr(), off.data_ptr(),
            idx3[0].data_ptr(), idx3[1].data_ptr(), idx3[2].data_ptr(), ws.data_ptr(), stream_ptr(dev),
        )
        check(rc, "route_metadata")
    return Route(freq, off, idx3[2], idx3[0], idx3[1], None, K)


def TC_topk_router_metadata(topk_router_indices: torch.Tensor, expert_frequency_offset: torch.Tensor, K: int):
    """Index vectors for token-choice top-k routing (reference: sonicmoe/functional/__init__.py:19-46).

    ``expert_frequency_offset`` is the inclusive cumsum the reference passes in; only its length (E) is
    used, the offsets are recomputed together with the sort.  Rows of one expert are ordered by flat slot
    (a stable sort; the reference's argsort leaves that order unspecified).
    Returns (expert_frequency_offset with leading 0, x_gather_idx, s_scatter_idx, s_reverse_scatter_idx,
    num_activated_expert_per_token_offset).
    """
    E = expert_frequency_offset.numel()
    r = _route_metadata(topk_router_indices.reshape(-1), None, E, K)
    T = topk_router_indices.shape[0]
    tok_off = torch.arange(0, T * K + 1, K, dtype=torch.int32, device=topk_router_indices.device)
    return r.expert_frequency_offset, r.x_gather_idx, r.s_scatter_idx, r.s_reverse_scatter_idx, tok_off


def _sorted_offsets(sorted_idx: torch.Tensor, T: int) -> torch.Tensor:
    dev = sorted_idx.device
    with torch.cuda.device(dev):
        out = torch.empty(T + 1, dtype=torch.int32, device=dev)
        check(lib.smoe_sorted_offsets(sorted_idx.data_ptr(), sorted_idx.numel(), T, out.data_ptr(), stream_ptr(dev)),
              "sorted_offsets")
    return out


def general_routing_router_metadata(
    router_scores_selected: torch.Tensor, sorted_selected_T: torch.Tensor, selected_E: torch.Tensor, T: int, E: int
):
    """Index vectors for caller-supplied pairs sorted by token (reference: functional/__init__.py:49-82).

    Returns (expert_frequency, expert_frequency_offset, x_gather_idx, s_scatter_idx, s_reverse_scatter_idx,
    num_activated_expert_per_token_offset).
    """
    tok = sorted_selected_T.contiguous().to(torch.int32)
    r = _route_metadata(selected_E, tok, E, 0)
    tok_off = _sorted_offsets(tok, T)
    return (r.expert_frequency, r.expert_frequency_offset, r.x_gather_idx, r.s_scatter_idx,
            r.s_reverse_scatter_idx, tok_off)


# ------------------------------------------------------------------------------------------------
# top-k + softmax
# ------------------------------------------------------------------------------------------------
class _TopkSoftmax(torch.autograd.Function):
    """scores (T,K) fp32 = softmax over the K largest logits of each row; indices (T,K) int32.

    Largest first; equal logits are ordered by lower expert id.  Reference:
    TC_Softmax_Topk_Router_Function (sonicmoe/functional/__init__.py:85-111).
    """

    @staticmethod
    def forward(ctx, router_logits: torch.Tensor, K: int):
        _lib.require_cuda(router_logits, "router_logits")
        if router_logits.dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"router logits must be fp32 or bf16, got {router_logits.dtype}")
        logits = router_logits.contiguous()
        T, E = logits.shape
        dev = logits.device
        with torch.cuda.device(dev):
            scores = torch.empty(T, K, dtype=torch.float32, device=dev)
            indices = torch.empty(T, K, dtype=torch.int32, device=dev)
            check(lib.smoe_topk_softmax(logits.data_ptr(), _lib.dtype_code(logits.dtype), scores.data_ptr(),
                                        indices.data_ptr(), T, E, K, stream_ptr(dev)), "topk_softmax")
        ctx.save_for_backward(scores, indices)
        ctx.E = E
        ctx.logits_dtype = logits.dtype
        ctx.mark_non_differentiable(indices)
        return scores, indices

    @staticmethod
    def backward(ctx, dscores: torch.Tensor, _unused):
        scores, indices = ctx.saved_tensors
        T, K = scores.shape
        dev = scores.device
        dscores = dscores.contiguous().float()
        with torch.cuda.device(dev):
            dlogits = torch.empty(T, ctx.E, dtype=ctx.logits_dtype, device=dev)
            check(lib.smoe_softmax_topk_backward(dlogits.data_ptr(), _lib.dtype_code(ctx.logits_dtype),
                                                 dscores.data_ptr(), scores.data_ptr(), indices.data_ptr(),
                                                 T, ctx.E, K, stream_ptr(dev)), "softmax_topk_backward")
        return dlogits, None


def topk_softmax(router_logits: torch.Tensor, K: int) -> tuple[torch.Tensor, torch.Tensor]:
    return _TopkSoftmax.apply(router_logits, K)


# ------------------------------------------------------------------------------------------------
# fused routing front end
# ------------------------------------------------------------------------------------------------
_FUSED_ROUTER = os.getenv("SONICMOE_FUSED_ROUTER", "1") != "0"


def set_fused_router(enable: bool) -> bool:
    """Use the one-pass router kernel where it applies (default) or always the separate router linear + top-k;
    returns the previous setting."""
    global _FUSED_ROUTER
    prev, _FUSED_ROUTER = _FUSED_ROUTER, bool(enable)
    return prev


def fused_router_applies(x: torch.Tensor, router_w: torch.Tensor, K: int) -> bool:
    return (_FUSED_ROUTER and x.is_cuda and x.dtype == torch.bfloat16 and router_w.dtype == torch.bfloat16
            and not torch.compiler.is_compiling()
            and bool(lib.smoe_router_forward_supported(x.shape[1], router_w.shape[0], K)))


@torch.no_grad()
def layer_router_logits(x: torch.Tensor, router_w: torch.Tensor, K: int) -> torch.Tensor:
    """The router logits exactly as `moe_TC_softmax_topk_layer` computes them for these inputs (the fused kernel's
    where it applies, the router linear's otherwise) -- what a check of the routing decision must be run on."""
    if fused_router_applies(x, router_w, K):
        return _FusedRouter.apply(x, router_w, K)[0]
    return F.linear(x if x.dtype == router_w.dtype else x.to(router_w.dtype), router_w)


class _FusedRouter(torch.autograd.Function):
    """(logits (T,E) bf16, scores (T,K) fp32, indices (T,K) int32, expert_frequency (E) int32, prob_colsum (E) fp32)
    from one pass over x: router GEMM, top-K + softmax over the winners, token counts and the column sums of the
    full softmax, in one kernel.  Routing is decided on the bf16 logits this returns.  Backward: one kernel turns
    the gradients of logits, scores and prob_colsum into dlogits; the two router GEMMs stay library calls, as the
    forward one does in the reference (sonicmoe/functional/__init__.py:438-446, sonicmoe/moe.py:251-274)."""

    @staticmethod
    def forward(ctx, x, router_w, K: int):
        x = x.contiguous()
        router_w = router_w.contiguous()
        T, H = x.shape
        E = router_w.shape[0]
        dev = x.device
        st = _lib.device_state(dev)
        with torch.cuda.device(dev):
            logits = torch.empty(T, E, dtype=torch.bfloat16, device=dev)
            scores = torch.empty(T, K, dtype=torch.float32, device=dev)
            indices = torch.empty(T, K, dtype=torch.int32, device=dev)
            freq = torch.empty(E, dtype=torch.int32, device=dev)
            colsum = torch.empty(E, dtype=torch.float32, device=dev)
            ws = st.router_workspace(E)
            check(lib.smoe_router_forward(x.data_ptr(), router_w.data_ptr(), logits.data_ptr(), scores.data_ptr(),
                                          indices.data_ptr(), freq.data_ptr(), colsum.data_ptr(), ws.data_ptr(),
                                          T, H, E, K, st.status.data_ptr(), stream_ptr(dev)), "router_forward")
        ctx.save_for_backward(x, router_w, logits, scores, indices)
        ctx.mark_non_differentiable(indices, freq)
        ctx.set_materialize_grads(False)
        return logits, scores, indices, freq, colsum

    @staticmethod
    def backward(ctx, g_logits, g_scores, _gi, _gf, g_colsum):
        x, router_w, logits, scores, indices = ctx.saved_tensors
        if g_logits is None and g_scores is None and g_colsum is None:
            return None, None, None
        T, E = logits.shape
        K = scores.shape[1]
        dev = x.device
        if g_logits is not None:
            g_logits = g_logits.contiguous().to(torch.bfloat16)
        if g_scores is not None:
            g_scores = g_scores.contiguous().float()
        if g_colsum is not None:
            g_colsum = g_colsum.contiguous().float()
        with torch.cuda.device(dev):
            dlogits = torch.empty_like(logits)
            check(lib.smoe_router_backward(dlogits.data_ptr(), logits.data_ptr(), ptr(g_scores), scores.data_ptr(),
                                           indices.data_ptr(), ptr(g_colsum), ptr(g_logits), T, E, K,
                                           stream_ptr(dev)), "router_backward")
        dx = dlogits @ router_w if ctx.needs_input_grad[0] else None
        dw = dlogits.t() @ x if ctx.needs_input_grad[1] else None
        return dx, dw, None


# ------------------------------------------------------------------------------------------------
# routed experts
# ------------------------------------------------------------------------------------------------
def _expert_major(w: torch.Tensor) -> torch.Tensor:
    """(out, in, E) view as passed by MoE.forward -> contiguous (E, out, in) storage (no copy if it is one)."""
    return w.permute(2, 0, 1).contiguous()


_ACT_CODE = {ActivationType.SWIGLU: 0, ActivationType.GEGLU: 1, ActivationType.REGLU: 2, ActivationType.RELU_SQ: 3,
             ActivationType.RELU: 4, ActivationType.GELU: 5, ActivationType.SILU: 6}


def _check_experts_args(x, w1, w2, b1, b2, activation_type):
    if (b1 is None) != (b2 is None):
        raise AssertionError("b1 and b2 has to be None or not None at the same time!")
    if isinstance(activation_type, str):
        activation_type = ActivationType(activation_type)
    if activation_type not in _ACT_CODE:
        raise ValueError(f"unknown activation {activation_type}")
    _lib.require_cuda(x, "x")
    if x.dtype != torch.bfloat16 or w1.dtype != torch.bfloat16 or w2.dtype != torch.bfloat16:
        raise TypeError("the sm_100a kernels take bf16 activations and weights "
                        f"(got x {x.dtype}, w1 {w1.dtype}, w2 {w2.dtype})")
    H = x.shape[1]
    n1 = w1.shape[0]
    gated = is_glu(activation_type)
    if w1.shape[1] != H or w2.shape[0] != H or w2.shape[1] * (2 if gated else 1) != n1 or w1.shape[2] != w2.shape[2]:
        raise ValueError(f"inconsistent shapes: x {tuple(x.shape)}, w1 {tuple(w1.shape)}, w2 {tuple(w2.shape)}")
    if H % 64 != 0 or w2.shape[1] % 64 != 0:
        raise ValueError("hidden size and intermediate size must be multiples of 64")
    if (b1 is not None or activation_type != ActivationType.SWIGLU) and n1 % 128 != 0:
        raise ValueError("with a bias or a non-SwiGLU activation the up projection needs a multiple of 128 output rows")
    if b1 is not None and (b1.dtype != x.dtype or b2.dtype != x.dtype):
        raise TypeError("biases must have the activations' dtype")
    return activation_type


def _experts(x, w1, b1, w2, b2, scores_flat, route, T, inference, activation_type):
    """Routed experts: the tuned bias-free SwiGLU kernels, or the general ones for a bias / another activation."""
    if b1 is None and activation_type == ActivationType.SWIGLU:
        return _RoutedExperts.apply(x, w1, w2, scores_flat, route, T, inference)
    return _RoutedExpertsGeneral.apply(x, w1, b1, w2, b2, scores_flat, route, T, inference,
                                       _ACT_CODE[activation_type])


class _RoutedExperts(torch.autograd.Function):
    """o[t] = sum over the pairs (t, e) routed to token t of score * W2[e] swiglu(W1[e] x[t]).

    Forward: gather-fused up projection with the SwiGLU epilogue (z, y1), down projection, combine.
    Backward: dH GEMM with the fused dSwiGLU / ds / y1*s epilogue, the two weight-gradient GEMMs over the
    ragged token dimension, the dX GEMM and its reduction over each token's rows.
    Reference: _UpProjection + _DownProjection (sonicmoe/functional/__init__.py:114-420).
    """

    @staticmethod
    def forward(ctx, x, w1, w2, scores_flat, route: Route, T: int, inference: bool):
        dev = x.device
        x = x.contiguous()
        w1e = _expert_major(w1)  # (E, 2I, H)
        w2e = _expert_major(w2)  # (E, H, I)
        E, two_i, H = w1e.shape
        I = two_i // 2
        TK = route.x_gather_idx.numel()
        scores_flat = scores_flat.contiguous()
        st = _lib.device_state(dev)
        need_grad = not inference
        with torch.cuda.device(dev):
            stream = stream_ptr(dev)
            z = torch.empty(TK, two_i, dtype=x.dtype, device=dev) if need_grad else None
            y1 = torch.empty(TK, I, dtype=x.dtype, device=dev)
            check(lib.smoe_up_projection_forward(
                x.data_ptr(), w1e.data_ptr(), ptr(z), y1.data_ptr(), route.expert_frequency_offset.data_ptr(),
                route.x_gather_idx.data_ptr(), T, H, I, E, TK, st.status.data_ptr(), stream), "up_projection_forward")
            o = torch.empty(T, H, dtype=x.dtype, device=dev)
            if _one_row_per_token(route, T):
                check(lib.smoe_down_projection_forward_rows(
                    y1.data_ptr(), w2e.data_ptr(), o.data_ptr(), scores_flat.data_ptr(),
                    int(scores_flat.dtype == torch.bfloat16), route.expert_frequency_offset.data_ptr(),
                    route.x_gather_idx.data_ptr(), route.s_scatter_idx.data_ptr(), H, I, E, TK,
                    st.status.data_ptr(), stream), "down_projection_forward_rows")
            elif _FUSED_COMBINE:
                o_acc = torch.zeros(T, H, dtype=torch.float32, device=dev)
                check(lib.smoe_down_projection_forward_scatter(
                    y1.data_ptr(), w2e.data_ptr(), o_acc.data_ptr(), scores_flat.data_ptr(),
                    int(scores_flat.dtype == torch.bfloat16), route.expert_frequency_offset.data_ptr(),
                    route.x_gather_idx.data_ptr(), route.s_scatter_idx.data_ptr(), T, H, I, E, TK,
                    st.status.data_ptr(), stream), "down_projection_forward_scatter")
                check(lib.smoe_cast_f32_to_bf16(o_acc.data_ptr(), o.data_ptr(), T * H, stream), "cast")
            else:
                y2 = torch.empty(TK, H, dtype=x.dtype, device=dev)
                check(lib.smoe_down_projection_forward(
                    y1.data_ptr(), w2e.data_ptr(), y2.data_ptr(), route.expert_frequency_offset.data_ptr(),
                    H, I, E, TK, st.status.data_ptr(), stream), "down_projection_forward")
                check(lib.smoe_gather_sum(
                    y2.data_ptr(), o.data_ptr(), scores_flat.data_ptr(), _lib.dtype_code(scores_flat.dtype),
                    route.s_reverse_scatter_idx.data_ptr(), ptr(route.token_offset), T, H, max(route.K, 1), stream),
                    "gather_sum")
        if need_grad:
            ctx.save_for_backward(x, w1e, w2e, z, scores_flat)
            ctx.route = route
            ctx.dims = (T, H, I, E, TK)
            ctx.w_shapes = (w1.shape, w2.shape)
        return o

    @staticmethod
    def backward(ctx, dout):
        x, w1e, w2e, z, scores_flat = ctx.saved_tensors
        route: Route = ctx.route
        T, H, I, E, TK = ctx.dims
        dev = x.device
        dout = dout.contiguous()
        if dout.dtype != x.dtype:
            dout = dout.to(x.dtype)
        st = _lib.device_state(dev)
        off = route.expert_frequency_offset.data_ptr()
        gat = route.x_gather_idx.data_ptr()
        with torch.cuda.device(dev):
            stream = stream_ptr(dev)
            dz = torch.empty(TK, 2 * I, dtype=x.dtype, device=dev)
            y1s = torch.empty(TK, I, dtype=x.dtype, device=dev)
            ncols = lib.smoe_ds_partial_columns(I)
            ds_partial = torch.empty(ncols, TK, dtype=torch.float32, device=dev)
            check(lib.smoe_down_projection_backward_act(
                dout.data_ptr(), w2e.data_ptr(), z.data_ptr(), scores_flat.data_ptr(),
                int(scores_flat.dtype == torch.bfloat16), dz.data_ptr(), y1s.data_ptr(), ds_partial.data_ptr(),
                off, gat, route.s_scatter_idx.data_ptr(), T, H, I, E, TK, st.status.data_ptr(), stream),
                "down_projection_backward_act")
            ds = torch.empty_like(scores_flat)
            check(lib.smoe_ds_reduce(ds_partial.data_ptr(), route.s_scatter_idx.data_ptr(), ds.data_ptr(),
                                     _lib.dtype_code(ds.dtype), TK, ncols, stream), "ds_reduce")
            # dX first: nothing else depends on the weight gradients, and a caller that has to send dx somewhere
            # (expert parallelism) can do so while the two weight-gradient GEMMs run
            dx = torch.empty(T, H, dtype=x.dtype, device=dev)
            if _one_row_per_token(route, T):
                check(lib.smoe_up_projection_backward_dx_rows(
                    dz.data_ptr(), w1e.data_ptr(), dx.data_ptr(), off, gat, H, I, E, TK, st.status.data_ptr(), stream),
                    "up_projection_backward_dx_rows")
            else:
                dx_expanded = torch.empty(TK, H, dtype=x.dtype, device=dev)
                check(lib.smoe_up_projection_backward_dx(
                    dz.data_ptr(), w1e.data_ptr(), dx_expanded.data_ptr(), off, H, I, E, TK, st.status.data_ptr(),
                    stream), "up_projection_backward_dx")
                check(lib.smoe_gather_sum(
                    dx_expanded.data_ptr(), dx.data_ptr(), None, _lib.SMOE_F32,
                    route.s_reverse_scatter_idx.data_ptr(), ptr(route.token_offset), T, H, max(route.K, 1), stream),
                    "gather_sum")
                del dx_expanded
            if route.on_dx is not None:
                route.on_dx(dx)
            shared = route.wgrad_sum
            if shared is None:
                dw1, dw2, add = torch.empty_like(w1e), torch.empty_like(w2e), False
            else:
                dw1, dw2, add = shared.buffers(w1e, w2e)
            down = lib.smoe_down_projection_weight_grad_accumulate if add else lib.smoe_down_projection_weight_grad
            check(down(dout.data_ptr(), y1s.data_ptr(), dw2.data_ptr(), off, gat, T, H, I, E, TK,
                       st.status.data_ptr(), stream), "down_projection_weight_grad")
            del y1s, ds_partial
            up = lib.smoe_up_projection_weight_grad_accumulate if add else lib.smoe_up_projection_weight_grad
            check(up(x.data_ptr(), dz.data_ptr(), dw1.data_ptr(), off, gat, T, H, I, E, TK, st.status.data_ptr(),
                     stream), "up_projection_weight_grad")
            if shared is not None:
                dw1, dw2 = shared.finish_chunk()
                if dw1 is None:
                    return dx, None, None, ds, None, None, None
        # gradients in the layout of the (out, in, E) views the caller passed
        return dx, dw1.permute(1, 2, 0), dw2.permute(1, 2, 0), ds, None, None, None


class _RoutedExpertsGeneral(torch.autograd.Function):
    """`_RoutedExperts` with optional expert biases and any activation of ``ActivationType``.

    o[t] = sum score * (W2[e] act(W1[e] x[t] + b1[e]) + b2[e]).  Gradients also for b1, b2; the score gradient
    gains the term <dout[t], b2[e]>.  Reference: sonicmoe/functional/__init__.py:114-420 with b1/b2 and
    activation_type, bias kernels sonicmoe/functional/backward.py:36-168.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2, scores_flat, route: Route, T: int, inference: bool, act: int):
        dev = x.device
        x = x.contiguous()
        w1e = _expert_major(w1)  # (E, N1, H)
        w2e = _expert_major(w2)  # (E, H, I)
        E, n1, H = w1e.shape
        I = w2e.shape[2]
        TK = route.x_gather_idx.numel()
        scores_flat = scores_flat.contiguous()
        b1c = None if b1 is None else b1.contiguous()
        b2c = None if b2 is None else b2.contiguous()
        st = _lib.device_state(dev)
        off = route.expert_frequency_offset.data_ptr()
        with torch.cuda.device(dev):
            stream = stream_ptr(dev)
            z = torch.empty(TK, n1, dtype=x.dtype, device=dev) if not inference else None
            y1 = torch.empty(TK, I, dtype=x.dtype, device=dev)
            check(lib.smoe_up_projection_forward_act(
                x.data_ptr(), w1e.data_ptr(), ptr(b1c), ptr(z), y1.data_ptr(), off, route.x_gather_idx.data_ptr(),
                T, H, n1, E, TK, act, st.status.data_ptr(), stream), "up_projection_forward_act")
            y2 = torch.empty(TK, H, dtype=x.dtype, device=dev)
            check(lib.smoe_down_projection_forward_bias(
                y1.data_ptr(), w2e.data_ptr(), ptr(b2c), y2.data_ptr(), off, H, I, E, TK, st.status.data_ptr(),
                stream), "down_projection_forward_bias")
            o = torch.empty(T, H, dtype=x.dtype, device=dev)
            check(lib.smoe_gather_sum(
                y2.data_ptr(), o.data_ptr(), scores_flat.data_ptr(), _lib.dtype_code(scores_flat.dtype),
                route.s_reverse_scatter_idx.data_ptr(), ptr(route.token_offset), T, H, max(route.K, 1), stream),
                "gather_sum")
        if not inference:
            ctx.save_for_backward(x, w1e, w2e, z, scores_flat, b2c)
            ctx.route = route
            ctx.dims = (T, H, I, E, TK, n1)
            ctx.act = act
            ctx.has_bias = b1 is not None
        return o

    @staticmethod
    def backward(ctx, dout):
        x, w1e, w2e, z, scores_flat, b2c = ctx.saved_tensors
        route: Route = ctx.route
        T, H, I, E, TK, n1 = ctx.dims
        dev = x.device
        dout = dout.contiguous().to(x.dtype)
        st = _lib.device_state(dev)
        off = route.expert_frequency_offset.data_ptr()
        gat = route.x_gather_idx.data_ptr()
        sct = route.s_scatter_idx.data_ptr()
        sc_bf16 = int(scores_flat.dtype == torch.bfloat16)
        with torch.cuda.device(dev):
            stream = stream_ptr(dev)
            dz = torch.empty(TK, n1, dtype=x.dtype, device=dev)
            y1s = torch.empty(TK, I, dtype=x.dtype, device=dev)
            ncols = lib.smoe_ds_partial_columns(I)
            ds_partial = torch.empty(ncols, TK, dtype=torch.float32, device=dev)
            check(lib.smoe_down_projection_backward_dact(
                dout.data_ptr(), w2e.data_ptr(), z.data_ptr(), scores_flat.data_ptr(), sc_bf16, dz.data_ptr(),
                y1s.data_ptr(), ds_partial.data_ptr(), off, gat, sct, T, H, I, E, TK, ctx.act, st.status.data_ptr(),
                stream), "down_projection_backward_dact")
            ds = torch.empty_like(scores_flat)
            check(lib.smoe_ds_reduce(ds_partial.data_ptr(), sct, ds.data_ptr(), _lib.dtype_code(ds.dtype), TK, ncols,
                                     stream), "ds_reduce")
            db1 = db2 = None
            if ctx.has_bias:
                check(lib.smoe_ds_add_bias_term(dout.data_ptr(), b2c.data_ptr(), off, gat, sct, ds.data_ptr(),
                                                _lib.dtype_code(ds.dtype), E, H, TK, stream), "ds_add_bias_term")
                db2 = torch.empty(E, H, dtype=x.dtype, device=dev)
                check(lib.smoe_expert_column_sum(dout.data_ptr(), H, gat, scores_flat.data_ptr(),
                                                 _lib.dtype_code(scores_flat.dtype), sct, off, db2.data_ptr(), E, H,
                                                 stream), "expert_column_sum")
                db1 = torch.empty(E, n1, dtype=x.dtype, device=dev)
                check(lib.smoe_expert_column_sum(dz.data_ptr(), n1, None, None, 0, None, off, db1.data_ptr(), E, n1,
                                                 stream), "expert_column_sum")
            dw2 = torch.empty_like(w2e)
            check(lib.smoe_down_projection_weight_grad(
                dout.data_ptr(), y1s.data_ptr(), dw2.data_ptr(), off, gat, T, H, I, E, TK, st.status.data_ptr(),
                stream), "down_projection_weight_grad")
            # the two kernels below take the up projection's output rows as 2 * (their I argument)
            half = n1 // 2
            dw1 = torch.empty_like(w1e)
            check(lib.smoe_up_projection_weight_grad(
                x.data_ptr(), dz.data_ptr(), dw1.data_ptr(), off, gat, T, H, half, E, TK, st.status.data_ptr(),
                stream), "up_projection_weight_grad")
            dx_expanded = torch.empty(TK, H, dtype=x.dtype, device=dev)
            check(lib.smoe_up_projection_backward_dx(
                dz.data_ptr(), w1e.data_ptr(), dx_expanded.data_ptr(), off, H, half, E, TK, st.status.data_ptr(),
                stream), "up_projection_backward_dx")
            dx = torch.empty(T, H, dtype=x.dtype, device=dev)
            check(lib.smoe_gather_sum(
                dx_expanded.data_ptr(), dx.data_ptr(), None, _lib.SMOE_F32, route.s_reverse_scatter_idx.data_ptr(),
                ptr(route.token_offset), T, H, max(route.K, 1), stream), "gather_sum")
        return dx, dw1.permute(1, 2, 0), db1, dw2.permute(1, 2, 0), db2, ds, None, None, None, None


def moe_TC_softmax_topk_layer(
    x: torch.Tensor,
    router_w: torch.Tensor,
    w1: torch.Tensor,
    b1: torch.Tensor | None,
    w2: torch.Tensor,
    b2: torch.Tensor | None,
    K: int,
    stream_id: int = 0,
    activation_type: ActivationType | str = ActivationType.SWIGLU,
    is_inference_mode_enabled: bool = False,
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Token-choice top-K MoE layer: returns (o (T,H), router_logits (T,E), expert_frequency (E,) int32).

    x (T,H) bf16; router_w (E,H); w1 (2I,H,E) and w2 (H,I,E) are the ``permute(1,2,0)`` views of the
    (E,2I,H) / (E,H,I) parameters, gate/up rows of w1 interleaved.
    Reference: sonicmoe/functional/__init__.py:423-490.
    """
    o, router_logits, freq, _ = moe_TC_softmax_topk_layer_with_router_stats(
        x, router_w, w1, b1, w2, b2, K, stream_id, activation_type, is_inference_mode_enabled)
    return o, router_logits, freq


def moe_TC_softmax_topk_layer_with_router_stats(x, router_w, w1, b1, w2, b2, K, stream_id=0,
                                                activation_type=ActivationType.SWIGLU,
                                                is_inference_mode_enabled=False):
    """`moe_TC_softmax_topk_layer` plus a fourth result: the column sums (E,) fp32 of softmax(router_logits) when the
    fused routing kernel produced them (what the load-balancing loss needs), else None."""
    activation_type = _check_experts_args(x, w1, w2, b1, b2, activation_type)
    E = router_w.size(0)
    T = x.size(0)
    inference = is_inference_mode_enabled or not torch.is_grad_enabled()
    if fused_router_applies(x, router_w, K):
        router_logits, scores, indices, _freq, colsum = _FusedRouter.apply(x, router_w, K)
    else:
        colsum = None
        # a router kept in fp32 (an extension over the reference) computes its logits in fp32
        router_logits = F.linear(x if x.dtype == router_w.dtype else x.to(router_w.dtype), router_w)
        if torch.compiler.is_compiling() and b1 is None and activation_type == ActivationType.SWIGLU:
            # opaque custom ops instead of autograd functions with ctypes calls inside (torch.compile, fullgraph)
            from .compiled_ops import layer_with_custom_ops

            o, freq = layer_with_custom_ops(x, router_logits, w1, w2, K, E, inference)
            return o, router_logits, freq, None
        scores, indices = topk_softmax(router_logits, K)
    route = _route_metadata(indices.reshape(-1), None, E, K)
    o = _experts(x, w1, b1, w2, b2, scores.reshape(-1), route, T, inference, activation_type)
    return o, router_logits, route.expert_frequency, colsum


def moe_general_routing_inputs(
    x: torch.Tensor,
    router_scores: torch.Tensor,
    token_indices: torch.Tensor,
    expert_indices: torch.Tensor,
    w1: torch.Tensor,
    b1: torch.Tensor | None,
    w2: torch.Tensor,
    b2: torch.Tensor | None,
    E: int,
    stream_id: int = 0,
    activation_type: ActivationType | str = ActivationType.SWIGLU,
    is_inference_mode_enabled: bool = False,
) -> tuple[torch.Tensor, torch.Tensor]:
    """Routed experts for an arbitrary list of (score, token, expert) pairs; ``token_indices`` ascending.

    Returns (o (T,H), expert_frequency (E,) int32).  Gradients flow to x, w1, w2 and router_scores.
    Reference: sonicmoe/functional/__init__.py:497-562.
    """
    activation_type = _check_experts_args(x, w1, w2, b1, b2, activation_type)
    T = x.size(0)
    E = w2.size(-1)
    tok = token_indices.contiguous().to(torch.int32)
    route = _route_metadata(expert_indices, tok, E, 0)
    route.token_offset = _sorted_offsets(tok, T)
    inference = is_inference_mode_enabled or not torch.is_grad_enabled()
    o = _experts(x, w1, b1, w2, b2, router_scores, route, T, inference, activation_type)
    return o, route.expert_frequency
