"""Token-rounding router: top-K token choice, then every expert's token count is rounded to a multiple
of the GEMM tile (128 rows) by dropping its lowest-score top-K tokens or admitting its highest-score
non-top-K tokens.

Behaviour follows ``forward_token_choice_rounding`` of the reference benchmark
(benchmarks/moe-token-rounding.py:139-191), including the dtypes in which it does its arithmetic
(probabilities, renormalisation and the "-1" shift happen in the activation dtype).  The reference
leaves ties to ``topk`` / ``argsort``, whose order is unspecified; here every tie is resolved towards
the lower index (lower expert id in the top-K, lower token id in the per-expert ranking), and the pairs of
one token are listed by ascending expert.

The differentiable part (softmax, renormalisation of the K winners) is PyTorch; the top-K and the whole
selection (the reference's two full sorts) run in the library's CUDA kernels: a radix select per expert
instead of a sort.  Its outputs feed ``moe_general_routing_inputs``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

from .. import _lib
from .._lib import check, lib, stream_ptr

TILE_M = 128  # the reference hard-codes 128 whatever Mtile it is given (benchmarks/moe-token-rounding.py:143)

_MODE = {"down": 0, "up": 1, "nr": 2}  # SMOE_ROUND_DOWN / _UP / _NEAREST


def rounded_counts(expert_freq: torch.Tensor, routing: str, tile: int = TILE_M) -> torch.Tensor:
    """Per-expert target count: 'up' = ceil, 'down' = floor, 'nr' = nearest (ties to even) multiple of tile."""
    if routing == "down":
        return (expert_freq // tile * tile).to(torch.int32)
    if routing == "up":
        return (torch.ceil(expert_freq / tile) * tile).to(torch.int32)
    if routing == "nr":
        return torch.round(expert_freq / tile).to(torch.int32) * tile
    raise NotImplementedError(f"unknown routing mode {routing!r}")


@torch.no_grad()
def topk_indices(probs: torch.Tensor, K: int) -> torch.Tensor:
    """(T,K) int32 columns of the K largest entries per row, largest first, lower column first among equals."""
    _lib.require_cuda(probs, "router scores")
    if probs.dtype not in (torch.float32, torch.bfloat16):
        raise TypeError(f"token rounding takes fp32 or bf16 activations, got {probs.dtype}")
    probs = probs.contiguous()
    T, E = probs.shape
    dev = probs.device
    with torch.cuda.device(dev):
        unused = torch.empty(T, K, dtype=torch.float32, device=dev)
        idx = torch.empty(T, K, dtype=torch.int32, device=dev)
        check(lib.smoe_topk_softmax(probs.data_ptr(), _lib.dtype_code(probs.dtype), unused.data_ptr(), idx.data_ptr(),
                                    T, E, K, stream_ptr(dev)), "topk_softmax")
    return idx


@torch.no_grad()
def select_pairs(scores: torch.Tensor, topk_idx: torch.Tensor, routing: str, tile: int = TILE_M):
    """scores (T,E): probabilities with the top-K entries renormalised; topk_idx (T,K) int32.

    Returns (tokens (n,) int32 ascending, experts (n,) int32 ascending within a token, expert_count (E,) int32).
    Reads the number of pairs back from the device (one synchronisation, as the reference's boolean-mask
    indexing does).
    """
    if routing not in _MODE:
        raise NotImplementedError(f"unknown routing mode {routing!r}")
    _lib.require_cuda(scores, "router scores")
    scores = scores.contiguous()
    topk_idx = topk_idx.contiguous()
    T, E = scores.shape
    K = topk_idx.shape[1]
    dev = scores.device
    extra = {"down": 0, "up": tile - 1, "nr": tile // 2}[routing]
    capacity = min(T * E, T * K + E * extra)
    with torch.cuda.device(dev):
        ws = torch.empty(lib.smoe_token_rounding_workspace_bytes(T, E), dtype=torch.uint8, device=dev)
        count = torch.empty(E, dtype=torch.int32, device=dev)
        tokens = torch.empty(capacity, dtype=torch.int32, device=dev)
        experts = torch.empty(capacity, dtype=torch.int32, device=dev)
        n = torch.empty(1, dtype=torch.int32, device=dev)
        check(lib.smoe_token_rounding_select(scores.data_ptr(), _lib.dtype_code(scores.dtype), topk_idx.data_ptr(),
                                             T, E, K, tile, _MODE[routing], count.data_ptr(), tokens.data_ptr(),
                                             experts.data_ptr(), n.data_ptr(), capacity, ws.data_ptr(),
                                             stream_ptr(dev)), "token_rounding_select")
    n = int(n.item())
    if n > capacity:
        raise _lib.SonicMoEError(f"token rounding kept {n} pairs, more than the {capacity} it was given room for")
    return tokens[:n], experts[:n], count


def forward_token_choice_rounding(x: torch.Tensor, router_w: torch.Tensor, E: int, K: int, Mtile: int = TILE_M,
                                  routing: str = "nr"):
    """Returns (router_scores (TK',), token_indices (TK',) ascending, expert_indices (TK',)).

    The scores stay differentiable w.r.t. x and router_w: softmax, then the top-K entries divided by their
    sum, as in the reference; the selection itself carries no gradient.
    """
    _lib.require_cuda(x, "x")
    logits = F.linear(x, router_w)
    probs = F.softmax(logits, dim=-1, dtype=torch.float32).to(x.dtype)
    topk_idx = topk_indices(probs.detach(), K)
    idx64 = topk_idx.long()
    topk_val = probs.gather(-1, idx64)
    topk_val = topk_val / topk_val.sum(dim=-1, keepdim=True)
    scores = probs.scatter(-1, idx64, topk_val)
    tokens, experts, _ = select_pairs(scores.detach(), topk_idx, routing)
    return scores[tokens.long(), experts.long()].contiguous(), tokens, experts
