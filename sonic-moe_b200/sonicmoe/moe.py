"""``MoE`` module: router + per-expert up / down projections with top-K token-choice routing.

Constructor arguments, parameter names and shapes, the interleaved gate/up layout of ``c_fc.weight`` and
the ``forward`` signature follow the reference module (sonicmoe/moe.py:58-257), so state dicts are
interchangeable:

    router.weight (E, H)   c_fc.weight (E, 2I, H) [gate_j = row 2j, up_j = row 2j+1]   c_proj.weight (E, H, I)
"""

from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F

from .enums import ActivationType, KernelBackendMoE, is_glu
from .functional import moe_TC_softmax_topk_layer, moe_TC_softmax_topk_layer_with_router_stats


def _glu_halves(z: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    return z[..., 0::2], z[..., 1::2]  # gate, up


def _activation(kind: ActivationType, z: torch.Tensor) -> torch.Tensor:
    """Plain PyTorch definition of every activation the layer accepts (reference: sonicmoe/moe.py:24-55)."""
    if kind == ActivationType.SWIGLU:
        g, u = _glu_halves(z)
        return u * F.silu(g)
    if kind == ActivationType.GEGLU:
        g, u = _glu_halves(z)
        return (F.gelu(g.float()) * u).to(g.dtype)
    if kind == ActivationType.REGLU:
        g, u = _glu_halves(z)
        return (F.relu(g) * u).to(g.dtype)
    if kind == ActivationType.GELU:
        return F.gelu(z.float()).to(z.dtype)
    if kind == ActivationType.RELU:
        return F.relu(z)
    if kind == ActivationType.SILU:
        return F.silu(z)
    if kind == ActivationType.RELU_SQ:
        return F.relu(z) ** 2
    raise ValueError(f"unknown activation {kind}")


class Experts(nn.Module):
    """E independent linear maps stored as one (E, out_features, in_features) parameter."""

    def __init__(self, num_experts: int, in_features: int, out_features: int, add_bias: bool = True,
                 std: float | None = None) -> None:
        super().__init__()
        self.weight = nn.Parameter(torch.empty(num_experts, out_features, in_features))
        self.bias = nn.Parameter(torch.empty(num_experts, out_features)) if add_bias else None
        self.std = std
        self.num_experts = num_experts
        self.in_features = in_features
        self.out_features = out_features
        self.reset_parameters()

    def torch_forward(self, grouped: torch.Tensor, expert_frequency: torch.Tensor) -> list[torch.Tensor]:
        """Apply expert e to its slice of the expert-sorted rows; returns the per-expert outputs."""
        parts = grouped.split(expert_frequency.tolist(), dim=0)
        return [
            F.linear(parts[e], self.weight[e], None if self.bias is None else self.bias[e])
            for e in range(self.num_experts)
        ]

    def extra_repr(self) -> str:
        return f"num_experts={self.num_experts}, in_features={self.in_features}, out_features={self.out_features}"

    @torch.no_grad()
    def reset_parameters(self) -> None:
        nn.init.normal_(self.weight, mean=0, std=self.std)
        if self.bias is not None:
            self.bias.zero_()


class MoE(nn.Module):
    def __init__(
        self,
        num_experts: int,
        num_experts_per_tok: int,
        hidden_size: int,
        intermediate_size: int,
        activation_function: ActivationType,
        add_bias: bool,
        std: float,
    ) -> None:
        super().__init__()
        self.num_experts = num_experts
        self.top_k = num_experts_per_tok
        self.hidden_size = hidden_size
        self.intermediate_size = intermediate_size
        self.activation_function = activation_function

        self.router = nn.Linear(in_features=hidden_size, out_features=num_experts, bias=False)
        up_features = 2 * intermediate_size if is_glu(activation_function) else intermediate_size
        self.c_fc = Experts(num_experts, hidden_size, up_features, add_bias=add_bias, std=std)
        self.c_proj = Experts(num_experts, intermediate_size, hidden_size, add_bias=add_bias, std=std)

        # The reference records the construction-time stream here; kernels of this build always run on
        # the current stream, the attribute is kept for code that reads it.
        self.stream_id = torch.cuda.current_stream().cuda_stream if torch.cuda.is_available() else 0

    def forward(
        self,
        hidden_states: torch.Tensor,
        kernel_backend_moe: KernelBackendMoE = KernelBackendMoE.sonicmoe,
        is_inference_mode: bool = False,
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """Returns (output with the input's shape, switch-style load-balancing loss)."""
        original_shape = hidden_states.shape
        hidden_states = hidden_states.view(-1, self.hidden_size)

        prob_colsum = None
        if kernel_backend_moe == KernelBackendMoE.sonicmoe:
            out, router_logits, expert_frequency, prob_colsum = moe_TC_softmax_topk_layer_with_router_stats(
                hidden_states,
                self.router.weight,
                self.c_fc.weight.permute(1, 2, 0),
                self.c_fc.bias,
                self.c_proj.weight.permute(1, 2, 0),
                self.c_proj.bias,
                self.top_k,
                self.stream_id,
                self.activation_function,
                is_inference_mode or not self.training,
            )
        elif kernel_backend_moe == KernelBackendMoE.torch:
            out, router_logits, expert_frequency = self._torch_forward(hidden_states)
        else:
            raise ValueError(f"kernel backend {kernel_backend_moe} is not provided by this build")

        out = out.view(original_shape)
        if prob_colsum is not None:
            # the fused routing kernel already summed softmax(router_logits) over the tokens
            share = F.normalize(expert_frequency.float(), p=1, dim=0)
            aux_loss = self.num_experts * (F.normalize(prob_colsum, p=1, dim=0) * share).sum()
        else:
            aux_loss = self._compute_switch_loss(
                logits=router_logits,
                probs=F.softmax(router_logits, dim=-1, dtype=torch.float32),
                expert_frequency=expert_frequency,
            )
        return out, aux_loss

    def _compute_switch_loss(self, logits: torch.Tensor, probs: torch.Tensor,
                             expert_frequency: torch.Tensor) -> torch.Tensor:
        """E * <normalised mean router probability, normalised token share> (reference: sonicmoe/moe.py:261-274).

        Expert frequencies are per rank: nothing is reduced across data-parallel workers.
        """
        probs = probs.view(-1, probs.size(-1))
        share = F.normalize(expert_frequency.float(), p=1, dim=0)
        mean_prob = F.normalize(probs.sum(0), p=1, dim=0)
        return logits.size(-1) * (mean_prob * share).sum()

    # ---- plain PyTorch definition of the layer (KernelBackendMoE.torch) ------------------------------
    def _torch_forward(self, x: torch.Tensor):
        """Eager definition of the layer; selected explicitly, never used as a fallback.

        Reference: sonicmoe/moe.py:276-363 (top-k on the logits, softmax over the K winners in fp32,
        per-expert linear maps on expert-sorted rows, fp32 index_add back to token order).
        """
        T = x.size(0)
        router_logits = self.router(x)
        if self.top_k == 1:
            top_logits, selected = router_logits.max(dim=-1, keepdim=True)
        else:
            top_logits, selected = router_logits.topk(self.top_k, dim=-1)
        gates = F.softmax(top_logits.float(), dim=-1).type_as(x)

        flat = selected.flatten()
        with torch.no_grad():
            order = flat.sort().indices
        expert_frequency = flat.bincount(minlength=self.num_experts).to(torch.int32)
        token_of_row = order // self.top_k

        grouped = x[token_of_row]
        hidden = self.c_fc.torch_forward(grouped, expert_frequency)
        hidden = torch.cat([_activation(self.activation_function, h) for h in hidden], dim=0)
        hidden = torch.cat(self.c_proj.torch_forward(hidden, expert_frequency), dim=0)
        hidden = hidden * gates.flatten()[order].unsqueeze(-1)
        out = torch.zeros((T, self.hidden_size), dtype=torch.float32, device=x.device).index_add(
            0, token_of_row, hidden.float())
        return out, router_logits, expert_frequency
