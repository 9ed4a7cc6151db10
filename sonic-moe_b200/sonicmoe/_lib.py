"""ctypes binding of libsonicmoe_b200.so (declared in include/sonicmoe_b200.h).

The library is the only compute path of the `sonicmoe` backend: if it cannot be loaded the import
fails loudly, there is no eager / CPU substitute.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_longlong, c_size_t, c_uint, c_void_p

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libsonicmoe_b200.so")

SMOE_F32, SMOE_BF16, SMOE_I32, SMOE_I64 = 0, 1, 2, 3

_ERRORS = {
    -1: "unsupported or inconsistent sizes",
    -2: "a pointer or pitch is not 16-byte aligned",
    -3: "no usable CUDA driver / device",
    -4: "the driver rejected a TMA descriptor",
    -5: "kernel launch failed",
    -6: "unknown dtype code",
    -7: "workspace missing or too small",
    -8: "size exceeds the built-in scratch of the allocation-free entry point",
}

P, I, LL = c_void_p, c_int, c_longlong

# name -> (restype, argtypes); must list every function the header declares.
SIGNATURES: dict[str, tuple] = {
    "smoe_abi_version": (I, []),
    "smoe_topk_softmax": (I, [P, I, P, P, I, I, I, P]),
    "smoe_softmax_topk_backward": (I, [P, I, P, P, P, I, I, I, P]),
    "smoe_count_cumsum_workspace_bytes": (c_size_t, [I]),
    "smoe_count_cumsum": (I, [P, I, LL, I, P, P, P, P]),
    "smoe_count_cumsum_noalloc_max_experts": (I, []),
    "smoe_count_cumsum_noalloc": (I, [P, I, LL, I, P, P, P]),
    "smoe_route_metadata_workspace_bytes": (c_size_t, [I]),
    "smoe_route_metadata": (I, [P, P, LL, I, I, P, P, P, P, P, P, P]),
    "smoe_sorted_offsets": (I, [P, LL, I, P, P]),
    "smoe_token_rounding_workspace_bytes": (c_size_t, [I, I]),
    "smoe_token_rounding_select": (I, [P, I, P, I, I, I, I, I, P, P, P, P, I, P, P]),
    "smoe_gather_sum": (I, [P, P, P, I, P, P, I, I, I, P]),
    "smoe_cast_f32_to_bf16": (I, [P, P, LL, P]),
    "smoe_ds_reduce": (I, [P, P, P, I, I, I, P]),
    "smoe_up_projection_forward": (I, [P, P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_down_projection_forward": (I, [P, P, P, P, I, I, I, I, P, P]),
    "smoe_down_projection_forward_rows": (I, [P, P, P, P, I, P, P, P, I, I, I, I, P, P]),
    "smoe_up_projection_backward_dx_rows": (I, [P, P, P, P, P, I, I, I, I, P, P]),
    "smoe_mxfp8_down_projection_forward_rows": (I, [P, P, P, P, P, P, I, P, P, P, I, I, I, I, P, P]),
    "smoe_mxfp8_up_projection_backward_dx_rows": (I, [P, P, P, P, P, P, P, I, I, I, I, P, P]),
    "smoe_down_projection_forward_scatter": (I, [P, P, P, P, I, P, P, P, I, I, I, I, I, P, P]),
    "smoe_down_projection_backward_act": (I, [P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_ds_partial_columns": (I, [I]),
    "smoe_up_projection_backward_dx": (I, [P, P, P, P, I, I, I, I, P, P]),
    "smoe_down_projection_weight_grad": (I, [P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_up_projection_weight_grad": (I, [P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_down_projection_weight_grad_accumulate": (I, [P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_up_projection_weight_grad_accumulate": (I, [P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_up_projection_forward_act": (I, [P, P, P, P, P, P, P, I, I, I, I, I, I, P, P]),
    "smoe_down_projection_forward_bias": (I, [P, P, P, P, P, I, I, I, I, P, P]),
    "smoe_down_projection_backward_dact": (I, [P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, P, P]),
    "smoe_expert_column_sum": (I, [P, LL, P, P, I, P, P, P, I, I, P]),
    "smoe_ds_add_bias_term": (I, [P, P, P, P, P, P, I, I, I, I, P]),
    "smoe_fp8_quantize_rows": (I, [P, P, P, LL, I, P]),
    "smoe_fp8_quantize_blocks": (I, [P, P, P, I, I, I, P]),
    "smoe_fp8_up_projection_forward": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_fp8_down_projection_forward": (I, [P, P, P, P, P, P, I, I, I, I, P, P]),
    "smoe_fp8_down_projection_backward_act": (I, [P, P, P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_fp8_up_projection_backward_dx": (I, [P, P, P, P, P, P, I, I, I, I, P, P]),
    "smoe_mxfp8_scale_row_bytes": (I, [I]),
    "smoe_mxfp8_quantize_rows": (I, [P, P, P, LL, I, P]),
    "smoe_mxfp8_quantize_blocks": (I, [P, P, P, I, I, I, P]),
    "smoe_mxfp8_up_projection_forward": (I, [P, P, P, P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_mxfp8_up_projection_forward_q": (I, [P, P, P, P, P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_mxfp8_down_projection_forward": (I, [P, P, P, P, P, P, I, I, I, I, P, P]),
    "smoe_mxfp8_down_projection_backward_act": (I, [P, P, P, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_mxfp8_down_projection_backward_act_q": (I, [P, P, P, P, P, P, I, P, P, P, P, P, P, P, P, I, I, I, I, I, P, P]),
    "smoe_mxfp8_up_projection_backward_dx": (I, [P, P, P, P, P, P, I, I, I, I, P, P]),
    "smoe_router_forward_supported": (I, [I, I, I]),
    "smoe_router_forward_workspace_bytes": (c_size_t, [I]),
    "smoe_router_forward": (I, [P, P, P, P, P, P, P, P, I, I, I, I, P, P]),
    "smoe_router_backward": (I, [P, P, P, P, P, P, P, I, I, I, P]),
    "smoe_peer_alloc": (I, [c_size_t, P]),
    "smoe_peer_free": (I, [P]),
    "smoe_peer_export": (I, [P, P]),
    "smoe_peer_open": (I, [P, P]),
    "smoe_peer_close": (I, [P]),
    "smoe_peer_copy": (I, [P, P, c_size_t, P]),
    "smoe_stream_write_value": (I, [P, c_uint, P]),
    "smoe_stream_wait_values": (I, [P, I, c_uint, P]),
    "smoe_gather_sum_to_peers": (I, [P, P, I, P, P, I, I, I, P, P, I, I, P]),
}


class SonicMoEError(RuntimeError):
    pass


def _load() -> ctypes.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python sonic-moe_b200/build.py` "
            "(needs nvcc; the sonicmoe backend has no fallback without it)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the build is stale
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


# kernels one successful entry-point call launches (1 unless listed)
_KERNELS_PER_CALL = {"route_metadata": 3, "count_cumsum": 2, "router_forward": 2}
_launches = 0


def check(rc: int, what: str) -> None:
    global _launches
    if rc != 0:
        raise SonicMoEError(f"{what} failed: {_ERRORS.get(rc, 'error')} (code {rc})")
    _launches += _KERNELS_PER_CALL.get(what, 1)


def launch_count() -> int:
    """Kernels of this library launched so far by this process through the Python layer."""
    return _launches


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr(device: torch.device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def dtype_code(dt: torch.dtype) -> int:
    try:
        return {torch.float32: SMOE_F32, torch.bfloat16: SMOE_BF16, torch.int32: SMOE_I32, torch.int64: SMOE_I64}[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise SonicMoEError(
            f"{name} lives on {t.device}: the sonicmoe backend runs sm_100a CUDA kernels only and has no CPU path"
        )


class _DeviceState:
    """Per-device scratch owned by the Python side: the GEMM status word and the routing workspace."""

    def __init__(self, device: torch.device) -> None:
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.route_ws = torch.empty(0, dtype=torch.int32, device=device)
        self.router_ws = torch.empty(0, dtype=torch.uint8, device=device)

    def route_workspace(self, E: int) -> torch.Tensor:
        need = lib.smoe_route_metadata_workspace_bytes(E) // 4
        if self.route_ws.numel() < need:
            self.route_ws = torch.empty(need, dtype=torch.int32, device=self.status.device)
        return self.route_ws


    def router_workspace(self, E: int) -> torch.Tensor:
        need = lib.smoe_router_forward_workspace_bytes(E)
        if self.router_ws.numel() < need:
            self.router_ws = torch.empty(need, dtype=torch.uint8, device=self.status.device)
        return self.router_ws


_states: dict[int, _DeviceState] = {}


def device_state(device: torch.device) -> _DeviceState:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _states.get(idx)
    if st is None:
        st = _states[idx] = _DeviceState(torch.device("cuda", idx))
    return st


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if a GEMM kernel abandoned one of its bounded waits since the last check."""
    devs = [device_state(device)] if device is not None else list(_states.values())
    for st in devs:
        code = int(st.status.item())
        if code != 0:
            st.status.zero_()
            raise SonicMoEError(f"grouped GEMM kernel gave up waiting (status {code}); results are invalid")
