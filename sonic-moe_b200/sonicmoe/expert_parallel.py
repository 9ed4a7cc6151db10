"""Expert parallelism for the MoE layer: experts sharded over the ranks of one process group, token rows
exchanged with an all-to-all each way (NCCL over NVLink on GPUs).

The reference has no distributed code; this module extends its layer so that the result equals the
single-device layer applied to every rank's tokens with all E experts.  Rank r owns experts
[r*E/W, (r+1)*E/W); the router is replicated.  Per forward pass:

  1. route locally over the global experts (top-k + softmax, counting sort by expert = by destination rank);
  2. exchange per-expert row counts (all-to-all of E int32) and read the split sizes on the host;
  3. dispatch: gather the routed rows of x in grouped order, all-to-all them together with their scores;
  4. run the local experts on the received rows (the same gather-fused grouped GEMMs; every received row
     is a "token" with exactly one expert, its output already multiplied by its score);
  5. return the rows with the reverse all-to-all and sum each token's K rows.

Backward is the mirror image through autograd: every step is an autograd function whose backward is the
adjoint step (row gather <-> row sum, all-to-all <-> reverse all-to-all); score gradients come out of the
local experts' backward and travel back with the reverse all-to-all.

Device work goes through an ``ops`` object; the default runs the library's CUDA kernels and refuses CPU
tensors.  Tests inject a CPU implementation to exercise the multi-rank logic with the gloo backend.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .enums import ActivationType, is_glu
from .moe import Experts


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all along dim 0; the backward pass is the same exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        x = x.contiguous()
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x, out_splits, in_splits, group=group)
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        back = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(back, g, ctx.in_splits, ctx.out_splits, group=ctx.group)
        return back, None, None, None


class CudaOps:
    """The device operations of the expert-parallel layer on the library's CUDA kernels."""

    def topk_softmax(self, logits, K):
        from . import functional as fn

        return fn.topk_softmax(logits, K)

    def route_metadata(self, expert_idx, E, K):
        from . import functional as fn

        return fn._route_metadata(expert_idx, None, E, K)

    def gather_rows(self, x, route):
        return _GatherRows.apply(x, route)

    def sum_rows(self, rows, route, T):
        return _SumRows.apply(rows, route, T)

    def local_experts(self, x_rows, w1, w2, scores, local_expert, num_local_experts, inference):
        """rows -> score * expert(row); w1 (E_l,2I,H), w2 (E_l,H,I); one expert per row."""
        from . import functional as fn

        R = x_rows.shape[0]
        rows = torch.arange(R, dtype=torch.int32, device=x_rows.device)
        route = fn._route_metadata(local_expert, rows, num_local_experts, 0)
        route.K = 1  # every received row is its own token with a single routed pair
        return fn._RoutedExperts.apply(x_rows, w1.permute(1, 2, 0), w2.permute(1, 2, 0), scores, route, R, inference)


class Fp8CudaOps(CudaOps):
    """As CudaOps, with the local experts' forward and activation-gradient GEMMs in FP8 (E4M3, block scales;
    ``scale_format`` "fp32", "ue8m0" or None for the FP8 module's default)."""

    def __init__(self, scale_format: str | None = None):
        self.scale_format = scale_format

    def local_experts(self, x_rows, w1, w2, scores, local_expert, num_local_experts, inference):
        from . import functional as fn
        from .functional.fp8 import _RoutedExpertsFp8

        R = x_rows.shape[0]
        rows = torch.arange(R, dtype=torch.int32, device=x_rows.device)
        route = fn._route_metadata(local_expert, rows, num_local_experts, 0)
        route.K = 1
        return _RoutedExpertsFp8.apply(x_rows, w1.permute(1, 2, 0), w2.permute(1, 2, 0), scores, route, R, inference,
                                       self.scale_format)


class _GatherRows(torch.autograd.Function):
    """out[r] = x[x_gather_idx[r]] (grouped order); backward: dx[t] = sum of the K rows routed from token t."""

    @staticmethod
    def forward(ctx, x, route):
        from . import _lib

        _lib.require_cuda(x, "x")
        x = x.contiguous()
        T, H = x.shape
        n = route.x_gather_idx.numel()
        dev = x.device
        with torch.cuda.device(dev):
            out = torch.empty(n, H, dtype=x.dtype, device=dev)
            _lib.check(_lib.lib.smoe_gather_sum(x.data_ptr(), out.data_ptr(), None, 0, route.x_gather_idx.data_ptr(),
                                                None, n, H, 1, _lib.stream_ptr(dev)), "gather_sum")
        ctx.route, ctx.T = route, T
        return out

    @staticmethod
    def backward(ctx, g):
        return _sum_rows(g.contiguous(), ctx.route, ctx.T), None


class _SumRows(torch.autograd.Function):
    """out[t] = sum_k rows[s_reverse_scatter_idx[t*K+k]]; backward: drows[r] = dout[x_gather_idx[r]]."""

    @staticmethod
    def forward(ctx, rows, route, T):
        ctx.route = route
        return _sum_rows(rows.contiguous(), route, T)

    @staticmethod
    def backward(ctx, g):
        return _GatherRows.apply(g, ctx.route), None, None


def _sum_rows(rows, route, T):
    from . import _lib

    _lib.require_cuda(rows, "rows")
    H = rows.shape[1]
    dev = rows.device
    with torch.cuda.device(dev):
        out = torch.empty(T, H, dtype=rows.dtype, device=dev)
        _lib.check(_lib.lib.smoe_gather_sum(rows.data_ptr(), out.data_ptr(), None, 0,
                                            route.s_reverse_scatter_idx.data_ptr(), _lib.ptr(route.token_offset),
                                            T, H, max(route.K, 1), _lib.stream_ptr(dev)), "gather_sum")
    return out


def dispatch_plan(expert_frequency: torch.Tensor, world_size: int, group) -> tuple[torch.Tensor, list[int], list[int]]:
    """Exchange per-expert row counts.

    expert_frequency (E,) int32: rows this rank routes to every global expert.  Returns
    (recv_counts (W, E_l): rows arriving from each source rank for each local expert,
     send_splits[dst], recv_splits[src]) -- the split sizes of the row all-to-all, read on the host.
    """
    E = expert_frequency.numel()
    e_local = E // world_size
    recv_counts = torch.empty_like(expert_frequency)
    dist.all_to_all_single(recv_counts, expert_frequency.contiguous(), group=group)
    both = torch.stack([expert_frequency.view(world_size, e_local).sum(1),
                        recv_counts.view(world_size, e_local).sum(1)]).cpu()
    return recv_counts.view(world_size, e_local), both[0].tolist(), both[1].tolist()


def received_row_experts(recv_counts: torch.Tensor) -> torch.Tensor:
    """Local expert id of every received row: rows arrive source by source, expert by expert within a source."""
    W, e_local = recv_counts.shape
    ids = torch.arange(e_local, dtype=torch.int32, device=recv_counts.device).repeat(W)
    return torch.repeat_interleave(ids, recv_counts.reshape(-1).long())


def moe_ep_softmax_topk_layer(x, router_w, w1_local, w2_local, K, num_experts, group=None, ops=None,
                              is_inference_mode_enabled=False, logit_bias=None):
    """Expert-parallel token-choice top-K layer.

    x (T_local,H); router_w (E,H) replicated; w1_local (E/W,2I,H), w2_local (E/W,H,I): this rank's experts.
    ``logit_bias`` (E,), optional, is added to the router logits before the top-k (load-skew experiments).
    Returns (o (T_local,H), router_logits (T_local,E), expert_frequency (E,) of this rank's tokens).
    """
    ops = ops or CudaOps()
    W = dist.get_world_size(group)
    if num_experts % W != 0:
        raise ValueError(f"{num_experts} experts do not divide over {W} ranks")
    e_local = num_experts // W
    if w1_local.shape[0] != e_local or w2_local.shape[0] != e_local:
        raise ValueError("w1_local / w2_local must hold exactly this rank's experts")
    T = x.shape[0]
    inference = is_inference_mode_enabled or not torch.is_grad_enabled()

    router_logits = F.linear(x if x.dtype == router_w.dtype else x.to(router_w.dtype), router_w)
    if logit_bias is not None:
        router_logits = router_logits + logit_bias.to(router_logits.dtype)
    scores, indices = ops.topk_softmax(router_logits, K)
    route = ops.route_metadata(indices.reshape(-1), num_experts, K)

    recv_counts, send_splits, recv_splits = dispatch_plan(route.expert_frequency, W, group)
    x_send = ops.gather_rows(x, route)
    s_send = scores.reshape(-1)[route.s_scatter_idx.long()]
    x_recv = _AllToAllRows.apply(x_send, send_splits, recv_splits, group)
    s_recv = _AllToAllRows.apply(s_send, send_splits, recv_splits, group)

    local_expert = received_row_experts(recv_counts)
    o_recv = ops.local_experts(x_recv, w1_local, w2_local, s_recv, local_expert, e_local, inference)

    y_back = _AllToAllRows.apply(o_recv, recv_splits, send_splits, group)
    o = ops.sum_rows(y_back, route, T)
    return o, router_logits, route.expert_frequency


class ExpertParallelMoE(nn.Module):
    """`MoE` with its experts sharded over a process group (same constructor plus ``process_group``).

    Parameters: ``router.weight (E,H)`` replicated, ``c_fc.weight (E/W,2I,H)``, ``c_proj.weight (E/W,H,I)``.
    ``load_full_state_dict`` shards a checkpoint of the single-device module.
    """

    def __init__(self, num_experts, num_experts_per_tok, hidden_size, intermediate_size,
                 activation_function=ActivationType.SWIGLU, add_bias=False, std=0.02, process_group=None):
        super().__init__()
        if add_bias or activation_function != ActivationType.SWIGLU:
            raise NotImplementedError("expert parallelism is implemented for bias-free SwiGLU experts")
        self.group = process_group
        self.world_size = dist.get_world_size(process_group)
        self.rank = dist.get_rank(process_group)
        if num_experts % self.world_size != 0:
            raise ValueError(f"{num_experts} experts do not divide over {self.world_size} ranks")
        self.num_experts = num_experts
        self.num_local_experts = num_experts // self.world_size
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation_function = activation_function
        self.router = nn.Linear(hidden_size, num_experts, bias=False)
        up = 2 * intermediate_size if is_glu(activation_function) else intermediate_size
        self.c_fc = Experts(self.num_local_experts, hidden_size, up, add_bias=False, std=std)
        self.c_proj = Experts(self.num_local_experts, intermediate_size, hidden_size, add_bias=False, std=std)
        self.ops = None  # CudaOps unless a test injects another implementation

    @torch.no_grad()
    def load_full_state_dict(self, state: dict) -> None:
        lo = self.rank * self.num_local_experts
        hi = lo + self.num_local_experts
        self.router.weight.copy_(state["router.weight"])
        self.c_fc.weight.copy_(state["c_fc.weight"][lo:hi])
        self.c_proj.weight.copy_(state["c_proj.weight"][lo:hi])

    def forward(self, hidden_states, is_inference_mode: bool = False):
        shape = hidden_states.shape
        x = hidden_states.view(-1, self.hidden_size)
        o, logits, freq = moe_ep_softmax_topk_layer(
            x, self.router.weight, self.c_fc.weight, self.c_proj.weight, self.top_k, self.num_experts,
            group=self.group, ops=self.ops, is_inference_mode_enabled=is_inference_mode or not self.training)
        probs = F.softmax(logits, dim=-1, dtype=torch.float32)
        aux = self.num_experts * (F.normalize(probs.sum(0), p=1, dim=0) * F.normalize(freq.float(), p=1, dim=0)).sum()
        return o.view(shape), aux
