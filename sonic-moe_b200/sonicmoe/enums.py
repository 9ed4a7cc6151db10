"""Backend and activation selectors of the MoE layer.

Names and string values follow the reference (sonicmoe/enums.py:12-30) so that configuration files
and checkpoints written for it keep working.
"""

from enum import Enum

LIBRARY_NAME = "sonicmoe"


class KernelBackendMoE(Enum):
    scattermoe = "scattermoe"  # third-party backend of the reference; not provided here
    torch = "torch"            # plain PyTorch ops, the layer's slow definition
    sonicmoe = "sonicmoe"      # sm_100a kernels of libsonicmoe_b200.so


class ActivationType(Enum):
    SWIGLU = "swiglu"
    GEGLU = "geglu"
    REGLU = "reglu"
    RELU_SQ = "relu_sq"
    RELU = "relu"
    GELU = "gelu"
    SILU = "silu"


_GLU = frozenset({ActivationType.SWIGLU, ActivationType.GEGLU, ActivationType.REGLU})


def is_glu(activation_type: ActivationType) -> bool:
    """Gated activations take 2*I pre-activations per token (gate = even column, up = odd column)."""
    return activation_type in _GLU
