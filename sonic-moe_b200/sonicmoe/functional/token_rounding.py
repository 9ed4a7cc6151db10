"""Token-rounding router: top-K token choice, then every expert's token count is rounded to a multiple
of the GEMM tile (128 rows) by dropping its lowest-score top-K tokens or admitting its highest-score
non-top-K tokens.

Behaviour follows ``forward_token_choice_rounding`` of the reference benchmark
(benchmarks/moe-token-rounding.py:139-191), including the dtypes in which it does its arithmetic
(probabilities, renormalisation and the "-1" shift happen in the activation dtype).  The reference
leaves ties to ``topk`` / ``argsort``, whose order is unspecified; here every tie is resolved towards
the lower index (lower expert id in the top-K, lower token id in the per-expert ranking).

This stage is routing policy expressed with PyTorch device ops; its outputs feed
``moe_general_routing_inputs``.
"""

from __future__ import annotations

import torch
import torch.nn.functional as F

TILE_M = 128  # the reference hard-codes 128 whatever Mtile it is given (benchmarks/moe-token-rounding.py:143)


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
def _select(scores: torch.Tensor, topk_idx: torch.Tensor, routing: str):
    """scores (T,E): probabilities with the top-K entries renormalised -> (tokens, experts) of the kept pairs."""
    T, E = scores.shape
    freq = torch.bincount(topk_idx.reshape(-1), minlength=E).to(torch.int32)
    target = rounded_counts(freq, routing)

    # ranking value: top-K entries keep their renormalised score, every other entry is shifted below them
    ranking = scores - 1
    ranking.scatter_(1, topk_idx, scores.gather(1, topk_idx))
    per_expert = ranking.sort(dim=0, descending=True, stable=True).indices  # (T,E): tokens of each expert, best first

    keep = torch.arange(T, device=scores.device, dtype=torch.int32)[:, None] < target[None, :]
    tokens = per_expert[keep]                                   # expert-major inside each rank row
    experts = torch.arange(E, device=scores.device, dtype=torch.int32)[None, :].expand(T, -1)[keep]
    # pairs sorted by token, then by the (rank, expert) order they were selected in
    by_token = tokens.sort(stable=True)
    return by_token.values.to(torch.int32), experts[by_token.indices].to(torch.int32)


def forward_token_choice_rounding(x: torch.Tensor, router_w: torch.Tensor, E: int, K: int, Mtile: int = TILE_M,
                                  routing: str = "nr"):
    """Returns (router_scores (TK',), token_indices (TK',) ascending, expert_indices (TK',)).

    The scores stay differentiable w.r.t. x and router_w: softmax, then the top-K entries divided by their
    sum, as in the reference; the selection itself carries no gradient.
    """
    logits = F.linear(x, router_w)
    probs = F.softmax(logits, dim=-1, dtype=torch.float32).to(x.dtype)
    # top-K per token: value descending, lower expert id first among equals
    topk_idx = probs.detach().sort(dim=-1, descending=True, stable=True).indices[:, :K]
    topk_val = probs.gather(-1, topk_idx)
    topk_val = topk_val / topk_val.sum(dim=-1, keepdim=True)
    scores = probs.scatter(-1, topk_idx, topk_val)
    tokens, experts = _select(scores.detach(), topk_idx, routing)
    return scores[tokens.long(), experts.long()].contiguous(), tokens, experts
