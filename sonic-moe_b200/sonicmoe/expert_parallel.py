"""Expert parallelism for the MoE layer: experts sharded over the ranks of one process group, token rows
exchanged with an all-to-all each way (NCCL over NVLink on GPUs).

The reference has no distributed code; this module extends its layer so that the result equals the
single-device layer applied to every rank's tokens with all E experts.  Rank r owns experts
[r*E/W, (r+1)*E/W); the router is replicated.

A token row crosses the link ONCE PER DESTINATION RANK, not once per routed (token, expert) pair: with K
experts per token spread over W ranks a token reaches at most min(K, W) ranks (K=8 over 8 ranks: 5.2 on
average, over 2 ranks: 2), and the expert rank adds up the token's local experts before anything travels
back.  Per forward pass:

  1. route locally over the global experts (top-k + softmax);
  2. plan: for every destination rank the ascending list of tokens with at least one expert there, and the
     (token, expert, score) pairs in the same order; exchange the two counts per rank pair and read the split
     sizes on the host (the one host synchronisation of the layer; the backward pass has none);
  3. dispatch: the listed rows of x go to their destination ranks -- over peer memory by default: one kernel
     gathers each row and stores it straight into the destination's exchange buffer (sonicmoe/peer.py); or an
     NCCL / gloo all-to-all of the gathered rows; the pairs' scores and (row within the sender's segment, local
     expert) indices follow by all-to-all (a few bytes per pair);
  4. run the local experts on the received tokens as a layer with caller-supplied pairs and a variable number
     of experts per token (the general-routing form of the same gather-fused grouped GEMMs): one output row per
     received token, already weighted by the scores and summed over that token's local experts;
  5. return those rows (copy-engine copies into the source ranks' buffers, or the reverse all-to-all) and add up
     each token's rows (one per destination rank).

Backward is the mirror image through autograd: every step is an autograd function whose backward is the
adjoint step (row gather <-> row sum, all-to-all <-> reverse all-to-all); score gradients come out of the
local experts' backward and travel back with the reverse all-to-all.

Device work goes through an ``ops`` object; the default runs the library's CUDA kernels and refuses CPU
tensors.  Tests inject a CPU implementation to exercise the multi-rank logic with the gloo backend.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .enums import ActivationType, is_glu
from .moe import Experts


# Exchange timing (benchmarks): while a list is installed here every all-to-all on a CUDA tensor appends a
# (start, end) pair of CUDA events recorded on the current stream around it.
_exchange_events: list | None = None


def record_exchanges(enable: bool) -> list | None:
    """Start (True) or stop (False) recording CUDA events around every all-to-all; returns the list that was
    being filled (pairs of events; read them after a synchronize)."""
    global _exchange_events
    prev, _exchange_events = _exchange_events, ([] if enable else None)
    try:
        from . import peer

        peer.exchange_events = _exchange_events
    except ImportError:  # no library on this machine: only the collective transport exists
        pass
    return prev


def _timed_exchange(fn, on_cuda: bool):
    """Run fn(); while recording is on, between two CUDA events on the current stream."""
    if _exchange_events is None or not on_cuda:
        return fn()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    out = fn()
    e1.record()
    _exchange_events.append((e0, e1))
    return out


def _exchange(out, x, out_splits, in_splits, group):
    _timed_exchange(lambda: dist.all_to_all_single(out, x, out_splits, in_splits, group=group), x.is_cuda)


class _AllToAllRows(torch.autograd.Function):
    """Variable-split all-to-all along dim 0; the backward pass is the same exchange with the splits swapped."""

    @staticmethod
    def forward(ctx, x, in_splits, out_splits, group):
        x = x.contiguous()
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        _exchange(out, x, out_splits, in_splits, group)
        ctx.in_splits, ctx.out_splits, ctx.group = in_splits, out_splits, group
        return out

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        back = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        _exchange(back, g, ctx.in_splits, ctx.out_splits, ctx.group)
        return back, None, None, None


@dataclass
class RowList:
    """A gather list with its inverse: ``rows[i]`` is the source row of entry i; the entries of source row t are
    ``rev[offset[t] : offset[t+1]]``.  (The field names the row kernels expect.)"""

    x_gather_idx: torch.Tensor           # (n,) int32 source row of every entry
    s_reverse_scatter_idx: torch.Tensor  # (n,) int32 entries grouped by source row
    token_offset: torch.Tensor           # (T+1,) int32
    K: int = 0


@dataclass
class DispatchPlan:
    rows: RowList                 # entries = (destination rank, token), destination-major, tokens ascending
    pair_slot: torch.Tensor       # (P,) int64 flat (token, k) slot of every pair, ordered by (destination, token)
    pair_row: torch.Tensor        # (P,) int32 position of the pair's token inside its destination's segment
    pair_expert: torch.Tensor     # (P,) int32 expert id local to the destination rank
    send_rows: list[int]          # rows sent to / received from every rank
    recv_rows: list[int]
    send_pairs: list[int]
    recv_pairs: list[int]
    # where segments land when ranks write into each other's buffers (peer transport); rows
    dispatch_offset: list[int]    # [d]: first row, in rank d's receive buffer, of the segment this rank sends to d
    return_offset: list[int]      # [s]: first row, in rank s's entry list, of the segment rank s sent here
    token_capacity: int           # most tokens any rank holds: a rank receives at most world_size * this many rows


def _chunk_routing(indices: torch.Tensor, e_local: int, world_size: int):
    """Device-side part of one chunk's plan that does not need the split sizes."""
    T, K = indices.shape
    dev = indices.device
    idx = indices.long()
    dest = idx // e_local                                                   # (T, K)
    to_rank = torch.zeros(T, world_size, dtype=torch.bool, device=dev).scatter_(1, dest, True)
    by_rank = to_rank.t().contiguous()                                      # (W, T)
    row_counts = by_rank.sum(1)
    pair_counts = torch.bincount(dest.reshape(-1), minlength=world_size)
    counts = torch.cat([row_counts, pair_counts, row_counts.new_tensor([T])]).to(torch.int32)
    return idx, dest, to_rank, by_rank, counts


def plan_dispatch(indices: torch.Tensor, num_experts: int, world_size: int, group,
                  bounds: list[int] | None = None) -> list[DispatchPlan]:
    """indices (T, K): global expert of every (token, k) slot.  One plan per chunk of tokens
    [bounds[c], bounds[c+1]) (default: one chunk, all tokens); all chunks share ONE exchange of counts and one
    device->host read (the split sizes)."""
    T, K = indices.shape
    dev = indices.device
    W = world_size
    e_local = num_experts // W
    bounds = bounds or [0, T]
    chunks = len(bounds) - 1
    parts = [_chunk_routing(indices[bounds[c]:bounds[c + 1]], e_local, W) for c in range(chunks)]
    # every rank learns every rank's counts (and token count): rows[s][d], pairs[s][d] from rank s to rank d
    width = chunks * (2 * W + 1)
    mine = torch.cat([p[4] for p in parts])
    everyone = torch.empty(W * width, dtype=torch.int32, device=dev)
    dist.all_gather_into_tensor(everyone, mine, group=group)
    host = everyone.view(W, chunks, 2 * W + 1).cpu().tolist()               # the layer's one host synchronisation
    me = dist.get_rank(group)
    plans = []
    for c, (idx, dest, to_rank, by_rank, _) in enumerate(parts):
        Tc = bounds[c + 1] - bounds[c]
        rows_sd = [host[s][c][:W] for s in range(W)]
        pairs_sd = [host[s][c][W:2 * W] for s in range(W)]
        send_rows, send_pairs = rows_sd[me], pairs_sd[me]
        recv_rows = [rows_sd[s][me] for s in range(W)]
        recv_pairs = [pairs_sd[s][me] for s in range(W)]
        dispatch_offset = [sum(rows_sd[s][d] for s in range(me)) for d in range(W)]
        return_offset = [sum(rows_sd[s][d] for d in range(me)) for s in range(W)]
        token_capacity = max(host[s][c][2 * W] for s in range(W))
        n = sum(send_rows)

        # entries: positions of the set bits of by_rank in row-major order = destination-major, tokens ascending
        flat = by_rank.reshape(-1)
        entry = torch.argsort((~flat).to(torch.uint8), stable=True)[:n]
        entry_token = (entry % max(Tc, 1)).to(torch.int32)
        rev = torch.argsort(entry_token, stable=True).to(torch.int32)
        per_token = to_rank.sum(1)
        offset = torch.zeros(Tc + 1, dtype=torch.int32, device=dev)
        offset[1:] = per_token.cumsum(0)
        rows = RowList(entry_token, rev, offset)

        # pairs ordered by (destination, token): the order in which the destination lists them by received row
        flat_dest = dest.reshape(-1)
        token_of_slot = torch.arange(Tc, device=dev).repeat_interleave(K)
        pair_slot = torch.argsort(flat_dest * max(Tc, 1) + token_of_slot, stable=True)
        rank_in_segment = by_rank.long().cumsum(1) - 1                      # (W, Tc) position of token t in segment d
        pair_row = rank_in_segment[flat_dest[pair_slot], token_of_slot[pair_slot]].to(torch.int32)
        pair_expert = (idx.reshape(-1)[pair_slot] % e_local).to(torch.int32)
        plans.append(DispatchPlan(rows, pair_slot, pair_row, pair_expert, send_rows, recv_rows, send_pairs,
                                  recv_pairs, dispatch_offset, return_offset, token_capacity))
    return plans


def received_pair_tokens(pair_row: torch.Tensor, recv_rows: list[int], recv_pairs: list[int]) -> torch.Tensor:
    """Row of the receive buffer every received pair refers to: its row inside the sender's segment plus the first
    row of that segment.  Segments arrive source by source, so the result ascends."""
    dev = pair_row.device
    base = torch.tensor([0] + recv_rows[:-1], dtype=torch.int64, device=dev).cumsum(0)
    src = torch.repeat_interleave(torch.arange(len(recv_pairs), device=dev),
                                  torch.tensor(recv_pairs, dtype=torch.int64, device=dev),
                                  output_size=sum(recv_pairs))
    return (pair_row.long() + base[src]).to(torch.int32)


class CudaOps:
    """The device operations of the expert-parallel layer on the library's CUDA kernels."""

    # the chunks of one batch add their weight gradients into one pair of buffers inside the GEMM epilogues
    shares_weight_grads = True

    def topk_softmax(self, logits, K):
        from . import functional as fn

        return fn.topk_softmax(logits, K)

    def gather_rows(self, x, rows: RowList):
        return _GatherRows.apply(x, rows)

    def sum_rows(self, entries, rows: RowList, T):
        return _SumRows.apply(entries, rows, T)

    def _route(self, tokens, experts, num_local_experts, R):
        from . import functional as fn

        route = fn._route_metadata(experts, tokens, num_local_experts, 0)
        route.token_offset = fn._sorted_offsets(tokens, R)
        return route

    def local_layer(self, x_rows, w1, w2, scores, tokens, experts, num_local_experts, inference, on_dx=None,
                    wgrad_sum=None):
        """out[r] = sum over the pairs (r, e) of score * expert_e(x_rows[r]); w1 (E_l,2I,H), w2 (E_l,H,I);
        ``tokens`` ascending.  ``on_dx``: called in the backward pass with the gradient of x_rows as soon as it
        exists, before the weight-gradient GEMMs are launched.  ``wgrad_sum``: the `functional.WeightGradSum` the
        chunks of one batch share."""
        from . import functional as fn

        R = x_rows.shape[0]
        route = self._route(tokens, experts, num_local_experts, R)
        route.on_dx, route.wgrad_sum = on_dx, wgrad_sum
        return fn._RoutedExperts.apply(x_rows, w1.permute(1, 2, 0), w2.permute(1, 2, 0), scores, route, R, inference)


class Fp8CudaOps(CudaOps):
    """As CudaOps, with the local experts' forward and activation-gradient GEMMs in FP8 (E4M3, block scales;
    ``scale_format`` "fp32", "ue8m0" or None for the FP8 module's default)."""

    def __init__(self, scale_format: str | None = None):
        self.scale_format = scale_format

    def local_layer(self, x_rows, w1, w2, scores, tokens, experts, num_local_experts, inference, on_dx=None,
                    wgrad_sum=None):
        from .functional.fp8 import _RoutedExpertsFp8

        R = x_rows.shape[0]
        route = self._route(tokens, experts, num_local_experts, R)
        route.on_dx, route.wgrad_sum = on_dx, wgrad_sum
        return _RoutedExpertsFp8.apply(x_rows, w1.permute(1, 2, 0), w2.permute(1, 2, 0), scores, route, R, inference,
                                       self.scale_format)


class _GatherRows(torch.autograd.Function):
    """out[i] = x[rows.x_gather_idx[i]]; backward: dx[t] = sum of the entries gathered from row t."""

    @staticmethod
    def forward(ctx, x, rows):
        from . import _lib

        _lib.require_cuda(x, "x")
        x = x.contiguous()
        T, H = x.shape
        n = rows.x_gather_idx.numel()
        dev = x.device
        with torch.cuda.device(dev):
            out = torch.empty(n, H, dtype=x.dtype, device=dev)
            _lib.check(_lib.lib.smoe_gather_sum(x.data_ptr(), out.data_ptr(), None, 0, rows.x_gather_idx.data_ptr(),
                                                None, n, H, 1, _lib.stream_ptr(dev)), "gather_sum")
        ctx.rows, ctx.T = rows, T
        return out

    @staticmethod
    def backward(ctx, g):
        return _sum_rows(g.contiguous(), ctx.rows, ctx.T), None


class _SumRows(torch.autograd.Function):
    """out[t] = sum of the entries of row t; backward: dentries[i] = dout[rows.x_gather_idx[i]]."""

    @staticmethod
    def forward(ctx, entries, rows, T):
        ctx.rows = rows
        return _sum_rows(entries.contiguous(), rows, T)

    @staticmethod
    def backward(ctx, g):
        return _GatherRows.apply(g, ctx.rows), None, None


def _sum_rows(entries, rows, T):
    from . import _lib

    _lib.require_cuda(entries, "rows")
    H = entries.shape[1]
    dev = entries.device
    with torch.cuda.device(dev):
        out = torch.empty(T, H, dtype=entries.dtype, device=dev)
        _lib.check(_lib.lib.smoe_gather_sum(entries.data_ptr(), out.data_ptr(), None, 0,
                                            rows.s_reverse_scatter_idx.data_ptr(), _lib.ptr(rows.token_offset),
                                            T, H, max(rows.K, 1), _lib.stream_ptr(dev)), "gather_sum")
    return out


# A transport moves token rows between the ranks in two steps each way, so that a caller can keep several chunks of
# tokens in flight:  h = dispatch_start(x, plan, keep, tag); x_recv = dispatch_wait(h)  and
# h = combine_start(rows, plan, tag); o = combine_finish(h, plan, T).  `micro_batches` is how many chunks it
# wants the layer to cut the tokens into (1 = no pipelining).


class CollectiveTransport:
    """Token rows by `all_to_all_single` of the process group's backend (NCCL on GPUs, gloo in the CPU tests)."""

    micro_batches = 1

    def __init__(self, group, ops, micro_batches: int = 1):
        self.group, self.ops, self.micro_batches = group, ops, micro_batches

    def dispatch_start(self, x, plan, keep, tag):
        return _AllToAllRows.apply(self.ops.gather_rows(x, plan.rows), plan.send_rows, plan.recv_rows, self.group)

    def dispatch_wait(self, handle):
        return handle

    def combine_start(self, rows, plan, tag):
        return _AllToAllRows.apply(rows, plan.recv_rows, plan.send_rows, self.group)

    def combine_finish(self, handle, plan, T):
        return self.ops.sum_rows(handle, plan.rows, T)


class _Lease:
    """Gives a slot of the peer transport's receive buffer back when the autograd graph that reads it goes away."""

    def __init__(self, transport, slot):
        self.transport, self.slot = transport, slot

    def __del__(self):
        self.transport.release_slot(self.slot)


class _EarlyReturn:
    """Sends the gradient of the dispatched rows back to the tokens' ranks as soon as the local experts' backward
    pass has produced it: copy-engine copies and the barrier on the transport's copy stream, while the compute
    stream goes on with the two weight-gradient GEMMs, which nothing downstream waits for.  `start` is what the
    local layer calls (`on_dx`); `_PeerDispatch.backward` then only waits for the event."""

    def __init__(self, transport, plan, tag):
        self.transport, self.plan, self.tag = transport, plan, tag
        self.dx = self.landed = self.view = None

    def start(self, dx):
        tr, plan = self.transport, self.plan
        self.dx = dx
        self.landed, self.view = tr.send_async(dx, plan.recv_rows, plan.return_offset, sum(plan.send_rows),
                                               ("return_bwd", self.tag), plan.token_capacity)


class _PeerDispatch(torch.autograd.Function):
    """x (T,H) -> the rows this rank's experts need, written by their owners straight into this rank's exchange
    buffer (gather fused with the send); backward: the row gradients go back and each token's are added up."""

    @staticmethod
    def forward(ctx, x, plan, transport, keep, slot, tag, early):
        if keep:
            ctx.lease = _Lease(transport, slot)
        ctx.plan, ctx.transport, ctx.T, ctx.tag, ctx.early = plan, transport, x.shape[0], tag, early
        return _timed_exchange(lambda: transport.dispatch_rows(x, plan, ("dispatch_fwd", slot, tag)), True)

    @staticmethod
    def backward(ctx, g):
        early = ctx.early
        if early is not None and early.landed is not None:
            # the rows left while the weight-gradient GEMMs ran (every rank takes this branch or none does: whether
            # the local layer called the hook does not depend on the data)
            if g.data_ptr() != early.dx.data_ptr():
                raise RuntimeError("the gradient handed to the dispatch is not the tensor the local layer announced")
            ctx.transport.compute_wait(early.landed)
            back = early.view
            early.dx = None
        else:
            back = _timed_exchange(lambda: ctx.transport.return_rows(g, ctx.plan, ("return_bwd", ctx.tag)), True)
        ctx.lease = None
        return _sum_rows(back, ctx.plan.rows, ctx.T), None, None, None, None, None, None


class _PeerCombine(torch.autograd.Function):
    """The expert ranks' per-token partial sums back to the tokens' ranks and added up there; backward: the output
    gradient's rows dispatched to the expert ranks (the same fused gather + send)."""

    @staticmethod
    def forward(ctx, rows, plan, transport, T, tag):
        ctx.plan, ctx.transport, ctx.tag = plan, transport, tag
        back = _timed_exchange(lambda: transport.return_rows(rows, plan, ("return_fwd", tag)), True)
        return _sum_rows(back, plan.rows, T)

    @staticmethod
    def backward(ctx, g):
        return (_timed_exchange(lambda: ctx.transport.dispatch_rows(g, ctx.plan, ("dispatch_bwd", ctx.tag)), True),
                None, None, None, None)


class PeerMemoryTransport:
    """Token rows through buffers the ranks map from each other (sonicmoe/peer.py): the library's own kernels and
    copy-engine copies over NVLink instead of an NCCL all-to-all.  Every exchange runs in order on the caller's
    stream, except the return of the row gradients in the backward pass, which travels on a copy stream while the
    weight-gradient GEMMs run (`_EarlyReturn`).  bf16 CUDA rows, one node."""

    micro_batches = 1

    def __init__(self, group, device, depth: int = 2):
        from .peer import AsyncPeerTransport

        self.impl = AsyncPeerTransport(group, device, depth)

    def dispatch_start(self, x, plan, keep, tag):
        if tag == 0:
            self._slot = self.impl.take_slot(keep)
        early = _EarlyReturn(self.impl, plan, tag) if keep else None
        return _PeerDispatch.apply(x, plan, self.impl, keep and tag == 0, self._slot, tag, early), early

    def dispatch_wait(self, handle):
        return handle[0]

    def dx_hook(self, handle):
        return None if handle[1] is None else handle[1].start

    def combine_start(self, rows, plan, tag):
        return (rows, tag)

    def combine_finish(self, handle, plan, T):
        rows, tag = handle
        return _PeerCombine.apply(rows, plan, self.impl, T, tag)

    def close(self):
        self.impl.close()


class _Flight:
    """What the autograd nodes of one chunk's exchange share: the events that say when its rows have landed."""

    def __init__(self):
        self.landed = None       # forward: the rows are in this rank's buffer (recorded on the copy stream)
        self.grad_ready = None   # backward: the gradient rows to send have been produced (compute stream)
        self.grad_landed = None  # backward: the gradient rows are in this rank's buffer (copy stream)
        self.early_dx = None     # backward: the gradient tensor whose return the local layer's hook already started
        self.early_landed = self.early_view = None


class _DispatchStart(torch.autograd.Function):
    """Gather the chunk's rows (compute stream), then send them to their destination ranks with copy-engine copies
    on the copy stream.  Returns this rank's receive buffer, valid once `_AfterLanding` has made the compute stream
    wait.  Backward: the gradient rows computed here go back the same way and each token's are added up."""

    @staticmethod
    def forward(ctx, x, plan, transport, flight, keep, slot, tag):
        if keep:
            ctx.lease = _Lease(transport, slot)
        ctx.plan, ctx.transport, ctx.flight, ctx.T, ctx.tag = plan, transport, flight, x.shape[0], tag
        send = _gather_rows_plain(x, plan.rows)
        flight.landed, view = transport.send_async(send, plan.send_rows, plan.dispatch_offset, sum(plan.recv_rows),
                                                   ("dispatch_fwd", slot, tag), plan.token_capacity)
        return view

    @staticmethod
    def backward(ctx, g):
        tr, plan, flight = ctx.transport, ctx.plan, ctx.flight
        if flight.early_landed is not None:
            # sent from the local layer's hook, while this chunk's weight-gradient GEMMs ran
            if g.data_ptr() != flight.early_dx.data_ptr():
                raise RuntimeError("the gradient handed to the dispatch is not the tensor the local layer announced")
            landed, back = flight.early_landed, flight.early_view
            flight.early_dx = None
        else:
            landed, back = tr.send_async(g, plan.recv_rows, plan.return_offset, sum(plan.send_rows),
                                         ("return_bwd", ctx.tag), plan.token_capacity, after=flight.grad_ready)
        tr.compute_wait(landed)
        ctx.lease = None
        return _sum_rows(back, plan.rows, ctx.T), None, None, None, None, None, None


class _AfterLanding(torch.autograd.Function):
    """Forward: the compute stream waits until the chunk's rows have landed.  Backward: marks, on the compute
    stream, the moment the gradient of those rows exists -- the copy stream may send it from then on, while the
    compute stream goes on with other chunks."""

    @staticmethod
    def forward(ctx, rows, transport, flight):
        ctx.transport, ctx.flight = transport, flight
        transport.compute_wait(flight.landed)
        return rows.view_as(rows)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        ctx.flight.grad_ready = ctx.transport.mark_compute()
        return g, None, None


class _CombineStart(torch.autograd.Function):
    """Send the rows computed here for other ranks' tokens back to them (copy stream).  Backward: hands out the
    output-gradient rows that `_CombineFinish.backward` had the token ranks send here."""

    @staticmethod
    def forward(ctx, rows, plan, transport, flight, tag):
        ctx.plan, ctx.transport, ctx.flight, ctx.tag = plan, transport, flight, tag
        rows = rows.contiguous()
        flight.landed, view = transport.send_async(rows, plan.recv_rows, plan.return_offset, sum(plan.send_rows),
                                                   ("return_fwd", tag), plan.token_capacity,
                                                   after=transport.mark_compute())
        return view

    @staticmethod
    def backward(ctx, _unused):
        ctx.transport.compute_wait(ctx.flight.grad_landed)
        return ctx.flight.grad_view, None, None, None, None


class _CombineFinish(torch.autograd.Function):
    """Wait for the returned rows and add up each token's.  Backward: gather the output gradient's rows and send
    them to the expert ranks (asynchronously: the next chunk's backward GEMMs run meanwhile)."""

    @staticmethod
    def forward(ctx, entries, plan, transport, flight, T, tag):
        ctx.plan, ctx.transport, ctx.flight, ctx.tag = plan, transport, flight, tag
        ctx.shape = entries.shape
        transport.compute_wait(flight.landed)
        return _sum_rows(entries, plan.rows, T)

    @staticmethod
    def backward(ctx, g):
        tr, plan, flight = ctx.transport, ctx.plan, ctx.flight
        send = _gather_rows_plain(g.contiguous(), plan.rows)
        flight.grad_landed, flight.grad_view = tr.send_async(send, plan.send_rows, plan.dispatch_offset,
                                                             sum(plan.recv_rows), ("dispatch_bwd", ctx.tag),
                                                             plan.token_capacity)
        # the gradient of `entries` is not a tensor anybody reads: _CombineStart.backward returns the received rows
        return g.new_zeros(1).expand(ctx.shape), None, None, None, None, None


def _gather_rows_plain(x, rows):
    from . import _lib

    x = x.contiguous()
    n, H = rows.x_gather_idx.numel(), x.shape[1]
    dev = x.device
    with torch.cuda.device(dev):
        out = torch.empty(n, H, dtype=x.dtype, device=dev)
        _lib.check(_lib.lib.smoe_gather_sum(x.data_ptr(), out.data_ptr(), None, 0, rows.x_gather_idx.data_ptr(), None,
                                            n, H, 1, _lib.stream_ptr(dev)), "gather_sum")
    return out


class PipelinedPeerTransport:
    """Peer-memory transport whose copies run on a second, high-priority stream through the copy engines, so that
    the exchange of one chunk of tokens overlaps the grouped GEMMs of another (the GEMMs are persistent kernels that
    occupy every multiprocessor: only copy engines can move data beside them).  The layer cuts its tokens into
    `micro_batches` chunks; per pass only the first chunk's dispatch and the last chunk's return are exposed."""

    def __init__(self, group, device, micro_batches: int = 2, depth: int = 2):
        from .peer import AsyncPeerTransport

        self.impl = AsyncPeerTransport(group, device, depth)
        self.micro_batches = micro_batches

    def dispatch_start(self, x, plan, keep, tag):
        if tag == 0:
            self._slot = self.impl.take_slot(keep)
        flight = _Flight()
        view = _DispatchStart.apply(x, plan, self.impl, flight, keep and tag == 0, self._slot, tag)
        return view, flight, (plan, tag) if keep else None

    def dispatch_wait(self, handle):
        view, flight, _ = handle
        return _AfterLanding.apply(view, self.impl, flight)

    def dx_hook(self, handle):
        _, flight, going_back = handle
        if going_back is None:
            return None
        plan, tag = going_back

        def start(dx):
            flight.early_dx = dx
            flight.early_landed, flight.early_view = self.impl.send_async(
                dx, plan.recv_rows, plan.return_offset, sum(plan.send_rows), ("return_bwd", tag), plan.token_capacity)

        return start

    def combine_start(self, rows, plan, tag):
        flight = _Flight()
        return _CombineStart.apply(rows, plan, self.impl, flight, tag), flight, tag

    def combine_finish(self, handle, plan, T):
        entries, flight, tag = handle
        return _CombineFinish.apply(entries, plan, self.impl, flight, T, tag)

    def close(self):
        self.impl.close()


_default_transports: dict = {}


def default_transport(group, x, ops):
    """For bf16 CUDA rows on more than one rank: peer memory, one exchange at a time on the caller's stream
    (SONICMOE_EP_TRANSPORT=peer_pipelined: peer memory with the tokens cut into two chunks whose exchanges overlap
    the other chunk's GEMMs; =nccl: the collective).  The collective otherwise.  One peer transport per (process
    group, device, kind) is kept for functional callers."""
    import os

    W = dist.get_world_size(group)
    kind = os.environ.get("SONICMOE_EP_TRANSPORT", "peer")
    if not (x.is_cuda and x.dtype == torch.bfloat16 and W > 1 and kind in ("peer", "peer_pipelined")):
        return CollectiveTransport(group, ops)
    key = (id(group) if group is not None else None, x.device.index, kind)
    if key not in _default_transports:
        from .peer import PeerMemoryUnavailable

        try:
            _default_transports[key] = (PipelinedPeerTransport(group, x.device) if kind == "peer_pipelined" else
                                        PeerMemoryTransport(group, x.device))
        except PeerMemoryUnavailable as exc:  # raised on every rank together: all of them take the collective
            import warnings

            warnings.warn(f"expert-parallel rows go through all_to_all_single: {exc}")
            _default_transports[key] = CollectiveTransport(group, ops)
    return _default_transports[key]


def close_default_transports() -> None:
    """Collective: release the peer-memory buffers of the default transports (before destroying the process group)."""
    for t in _default_transports.values():
        if hasattr(t, "close"):
            t.close()
    _default_transports.clear()


def moe_ep_softmax_topk_layer(x, router_w, w1_local, w2_local, K, num_experts, group=None, ops=None,
                              is_inference_mode_enabled=False, logit_bias=None, transport=None):
    """Expert-parallel token-choice top-K layer.

    x (T_local,H); router_w (E,H) replicated; w1_local (E/W,2I,H), w2_local (E/W,H,I): this rank's experts.
    ``logit_bias`` (E,), optional, is added to the router logits before the top-k (load-skew experiments).
    Returns (o (T_local,H), router_logits (T_local,E), expert_frequency (E,) of this rank's tokens).

    The tokens are cut into ``transport.micro_batches`` chunks (every rank the same number; a rank with few tokens
    gets short or empty chunks).  Order of work: all chunks' dispatches start; then chunk by chunk the local
    experts run as soon as that chunk's rows have landed and its results start travelling back; finally every
    chunk's returned rows are added up.  With a transport that copies asynchronously the exchange of one chunk
    overlaps the GEMMs of another, in the backward pass as well (autograd runs the mirror image of this order).
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
    transport = transport or default_transport(group, x, ops)
    M = max(1, int(transport.micro_batches))
    bounds = [T * c // M for c in range(M + 1)]
    with torch.no_grad():
        plans = plan_dispatch(indices, num_experts, W, group, bounds)
        expert_frequency = torch.bincount(indices.reshape(-1).long(), minlength=num_experts).to(torch.int32)

    flights = [transport.dispatch_start(x[bounds[c]:bounds[c + 1]], plans[c], not inference, c) for c in range(M)]
    routed = []
    for c, plan in enumerate(plans):
        s_send = scores[bounds[c]:bounds[c + 1]].reshape(-1)[plan.pair_slot]
        s_recv = _AllToAllRows.apply(s_send, plan.send_pairs, plan.recv_pairs, group)
        with torch.no_grad():
            meta = _AllToAllRows.apply(torch.stack([plan.pair_row, plan.pair_expert], dim=1), plan.send_pairs,
                                       plan.recv_pairs, group)
            tokens = received_pair_tokens(meta[:, 0], plan.recv_rows, plan.recv_pairs)
            experts = meta[:, 1].contiguous()
        routed.append((s_recv, tokens, experts))
    returning = []
    extra = {}
    if M > 1 and not inference and getattr(ops, "shares_weight_grads", False):
        from .functional import WeightGradSum

        extra["wgrad_sum"] = WeightGradSum(M)
    for c, plan in enumerate(plans):
        x_recv = transport.dispatch_wait(flights[c])
        s_recv, tokens, experts = routed[c]
        hook = transport.dx_hook(flights[c]) if hasattr(transport, "dx_hook") else None
        if hook is not None:
            extra["on_dx"] = hook
        o_recv = ops.local_layer(x_recv, w1_local, w2_local, s_recv, tokens, experts, e_local, inference, **extra)
        returning.append(transport.combine_start(o_recv, plan, c))
    outs = [transport.combine_finish(returning[c], plans[c], bounds[c + 1] - bounds[c]) for c in range(M)]
    o = outs[0] if M == 1 else torch.cat(outs)
    return o, router_logits, expert_frequency


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
        self.transport = None  # default_transport() unless set (a module with its own PeerMemoryTransport)

    @torch.no_grad()
    def load_full_state_dict(self, state: dict) -> None:
        lo = self.rank * self.num_local_experts
        hi = lo + self.num_local_experts
        self.router.weight.copy_(state["router.weight"])
        self.c_fc.weight.copy_(state["c_fc.weight"][lo:hi])
        self.c_proj.weight.copy_(state["c_proj.weight"][lo:hi])

    def forward(self, hidden_states, is_inference_mode: bool = False, logit_bias=None):
        shape = hidden_states.shape
        x = hidden_states.view(-1, self.hidden_size)
        o, logits, freq = moe_ep_softmax_topk_layer(
            x, self.router.weight, self.c_fc.weight, self.c_proj.weight, self.top_k, self.num_experts,
            group=self.group, ops=self.ops, is_inference_mode_enabled=is_inference_mode or not self.training,
            logit_bias=logit_bias, transport=self.transport)
        probs = F.softmax(logits, dim=-1, dtype=torch.float32)
        aux = self.num_experts * (F.normalize(probs.sum(0), p=1, dim=0) * F.normalize(freq.float(), p=1, dim=0)).sum()
        return o.view(shape), aux
