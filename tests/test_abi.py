"""The C-ABI library loads without a GPU and exports exactly what include/sonicmoe_b200.h declares."""

import ctypes
import os
import re

from conftest import ROOT


def _declared():
    text = open(os.path.join(ROOT, "include", "sonicmoe_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(smoe_\w+)\s*\(", text)))


def test_header_symbols_are_exported(built_library):
    lib = ctypes.CDLL(built_library)
    names = _declared()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_header(built_library):
    from sonicmoe import _lib

    assert sorted(_lib.SIGNATURES) == _declared()
    assert _lib.lib.smoe_abi_version() >= 1


def test_queries_and_argument_checks_without_gpu(built_library):
    """Entry points validate sizes before touching the device, so these calls are safe on a CPU-only box."""
    from sonicmoe import _lib

    lib = _lib.lib
    assert lib.smoe_ds_partial_columns(1024) == 8   # one row of partials per 128 accumulator columns
    assert lib.smoe_ds_partial_columns(64) == 2
    assert lib.smoe_route_metadata_workspace_bytes(128) >= 128 * 4
    # hidden size not a multiple of 64 -> shape error, nothing launched
    assert lib.smoe_up_projection_forward(None, None, None, None, None, None, 16, 100, 64, 8, 32, None, None) == -1
    assert lib.smoe_down_projection_forward(None, None, None, None, 128, 100, 8, 32, None, None) == -1
    # more experts than the kernels' tile table holds
    assert lib.smoe_up_projection_backward_dx(None, None, None, None, 128, 64, 5000, 32, None, None) == -1
    assert lib.smoe_topk_softmax(None, 0, None, None, 4, 8, 9, None) == -1      # K > E
    assert lib.smoe_topk_softmax(None, 7, None, None, 4, 8, 2, None) == -6      # unknown dtype
    assert lib.smoe_gather_sum(None, None, None, 0, None, None, 4, 12, 2, None) == -1  # H % 8
    # expert-parallel kernel: segment table checked on the host before anything is launched
    assert lib.smoe_gather_sum_to_peers(None, None, 0, None, None, 8, 64, 1, None, None, 0, 0, None) == -1
    assert lib.smoe_gather_sum_to_peers(None, None, 0, None, None, 8, 64, 1, None, None, 17, 0, None) == -1
    assert lib.smoe_router_forward_supported(4096, 128, 8) == 1
    assert lib.smoe_router_forward_supported(4096, 8, 2) == 0 and lib.smoe_router_forward_supported(4096, 128, 17) == 0
    # empty problems are no-ops
    assert lib.smoe_topk_softmax(None, 0, None, None, 0, 8, 2, None) == 0
    assert lib.smoe_up_projection_forward(None, None, None, None, None, None, 16, 128, 64, 8, 0, None, None) == 0
