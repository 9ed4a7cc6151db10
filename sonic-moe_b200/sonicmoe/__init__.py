"""B200-native SonicMoE layer: the reference's Python surface over libsonicmoe_b200.so.

Exports match the reference package (sonicmoe/__init__.py:5-8).
"""

from .count_cumsum import count_cumsum
from .enums import ActivationType, KernelBackendMoE
from .functional import enable_quack_gemm, moe_general_routing_inputs, moe_TC_softmax_topk_layer
from .moe import MoE
from ._lib import SonicMoEError, check_status

__all__ = [
    "ActivationType",
    "KernelBackendMoE",
    "MoE",
    "count_cumsum",
    "enable_quack_gemm",
    "moe_TC_softmax_topk_layer",
    "moe_general_routing_inputs",
    # beyond the reference's exports: the status check of the bounded-wait GEMM kernels
    "SonicMoEError",
    "check_status",
]
