"""FP8 (E4M3) expert path: activations quantised per row and 128 columns, weights per 128 x 128 block.
Forward and activation-gradient GEMMs run in FP8 on the tensor cores; the weight-gradient GEMMs, the router
and every saved tensor stay in bf16.

Two scale formats:

* ``"fp32"``  -- scale = amax / 448 in fp32, applied in software between 128-deep k-blocks
  (`smoe_fp8_*` entry points);
* ``"ue8m0"`` -- scale = the smallest power of two >= amax / 448, stored as one exponent byte and applied
  by the tensor cores' own block scaling (`smoe_mxfp8_*` entry points).  Same relative precision (E4M3
  keeps 3 mantissa bits whatever the scale; at most one binade of range is given up), no software promotion.

The reference has no FP8 path; the functions mirror the bf16 ones of ``sonicmoe.functional``.
"""

from __future__ import annotations

import os

import torch
import torch.nn.functional as F

from .. import _lib
from .._lib import check, lib, ptr, stream_ptr
from ..enums import ActivationType

BLOCK = 128
SCALE_FORMATS = ("fp32", "ue8m0")
_default_scale_format = os.environ.get("SONICMOE_FP8_SCALES", "fp32")


def set_scale_format(fmt: str) -> None:
    """Scale format used when a call does not name one ("fp32" or "ue8m0"; env SONICMOE_FP8_SCALES)."""
    global _default_scale_format
    _check_format(fmt)
    _default_scale_format = fmt


def _check_format(fmt: str) -> str:
    if fmt not in SCALE_FORMATS:
        raise ValueError(f"unknown FP8 scale format {fmt!r}: expected one of {SCALE_FORMATS}")
    return fmt


def refuse_unsupported(b1, b2, activation_type) -> None:
    """The FP8 experts are bias-free SwiGLU only; anything else is refused instead of silently dropping the
    biases or misreading the up projection's width."""
    if isinstance(activation_type, str):
        activation_type = ActivationType(activation_type)
    if b1 is not None or b2 is not None or activation_type != ActivationType.SWIGLU:
        raise NotImplementedError("the FP8 expert path is implemented for bias-free SwiGLU experts")


def _entry(name: str, fmt: str):
    """The library function ``name`` of the family that takes this scale format."""
    return getattr(lib, ("smoe_fp8_" if fmt == "fp32" else "smoe_mxfp8_") + name)


def quantize_rows(x: torch.Tensor, scale_format: str = "fp32") -> tuple[torch.Tensor, torch.Tensor]:
    """x (rows, cols) bf16 -> (q (rows, cols) uint8 holding E4M3, scales).

    fp32: scale (rows, cols/128) fp32.  ue8m0: (rows, 4*ceil(cols/512)) uint8, byte b of a row = exponent + 127 of
    block b (rows padded to whole 32-bit words with 127 = 2^0).
    """
    _lib.require_cuda(x, "x")
    _check_format(scale_format)
    x = x.contiguous()
    rows, cols = x.shape
    dev = x.device
    with torch.cuda.device(dev):
        q = torch.empty(rows, cols, dtype=torch.uint8, device=dev)
        if scale_format == "fp32":
            s = torch.empty(rows, cols // BLOCK, dtype=torch.float32, device=dev)
        else:
            s = torch.empty(rows, lib.smoe_mxfp8_scale_row_bytes(cols), dtype=torch.uint8, device=dev)
        check(_entry("quantize_rows", scale_format)(x.data_ptr(), q.data_ptr(), s.data_ptr(), rows, cols,
                                                    stream_ptr(dev)), "fp8_quantize_rows")
    return q, s


def quantize_blocks(w: torch.Tensor, scale_format: str = "fp32") -> tuple[torch.Tensor, torch.Tensor]:
    """w (E, rows, cols) bf16 -> (q uint8, scale (E, ceil(rows/128), cols/128) fp32, or uint8 exponent bytes)."""
    _lib.require_cuda(w, "w")
    _check_format(scale_format)
    w = w.contiguous()
    E, rows, cols = w.shape
    dev = w.device
    with torch.cuda.device(dev):
        q = torch.empty(E, rows, cols, dtype=torch.uint8, device=dev)
        s = torch.empty(E, (rows + BLOCK - 1) // BLOCK, cols // BLOCK,
                        dtype=torch.float32 if scale_format == "fp32" else torch.uint8, device=dev)
        check(_entry("quantize_blocks", scale_format)(w.data_ptr(), q.data_ptr(), s.data_ptr(), E, rows, cols,
                                                      stream_ptr(dev)), "fp8_quantize_blocks")
    return q, s


def dequantize(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 values of a quantised (rows, cols) or (E, rows, cols) tensor, for either scale format (tests, debugging)."""
    v = q.view(torch.float8_e4m3fn).float()
    s = scale.float() if scale.dtype == torch.float32 else torch.exp2(scale.float() - 127.0)
    nblk = v.shape[-1] // BLOCK
    s = s[..., :nblk].repeat_interleave(BLOCK, dim=-1)
    if v.dim() == 3:
        s = s.repeat_interleave(BLOCK, dim=-2)[:, : v.shape[1]]
    return v * s


class _RoutedExpertsFp8(torch.autograd.Function):
    """FP8 counterpart of ``_RoutedExperts``: same inputs, outputs and saved tensors (x, z, scores, indices)."""

    @staticmethod
    def forward(ctx, x, w1, w2, scores_flat, route, T: int, inference: bool, fmt: str = None):
        from . import _expert_major

        from . import _one_row_per_token

        fmt = _check_format(fmt or _default_scale_format)
        rows_form = fmt == "ue8m0" and _one_row_per_token(route, T)  # epilogues write o / dx rows directly
        dev = x.device
        x = x.contiguous()
        w1e = _expert_major(w1)
        w2e = _expert_major(w2)
        E, two_i, H = w1e.shape
        I = two_i // 2
        TK = route.x_gather_idx.numel()
        scores_flat = scores_flat.contiguous()
        st = _lib.device_state(dev)
        off = route.expert_frequency_offset.data_ptr()
        xq, xs = quantize_rows(x, fmt)
        w1q, w1s = quantize_blocks(w1e, fmt)
        w2q, w2s = quantize_blocks(w2e, fmt)
        with torch.cuda.device(dev):
            stream = stream_ptr(dev)
            z = torch.empty(TK, two_i, dtype=x.dtype, device=dev) if not inference else None
            if fmt == "ue8m0":  # the up projection's epilogue writes y1 quantised: no bf16 y1, no pass over it
                y1q = torch.empty(TK, I, dtype=torch.uint8, device=dev)
                ld = lib.smoe_mxfp8_scale_row_bytes(I)
                if (I // BLOCK) % 4 == 0:
                    y1s = torch.empty(TK, ld, dtype=torch.uint8, device=dev)
                else:  # the kernel does not write the padding bytes of a scale row
                    y1s = torch.full((TK, ld), 127, dtype=torch.uint8, device=dev)
                check(lib.smoe_mxfp8_up_projection_forward_q(
                    xq.data_ptr(), xs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), ptr(z), y1q.data_ptr(), y1s.data_ptr(),
                    off, route.x_gather_idx.data_ptr(), T, H, I, E, TK, st.status.data_ptr(), stream),
                    "mxfp8_up_projection_forward_q")
            else:
                y1 = torch.empty(TK, I, dtype=x.dtype, device=dev)
                check(_entry("up_projection_forward", fmt)(
                    xq.data_ptr(), xs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), ptr(z), y1.data_ptr(), off,
                    route.x_gather_idx.data_ptr(), T, H, I, E, TK, st.status.data_ptr(), stream),
                    "fp8_up_projection_forward")
                y1q, y1s = quantize_rows(y1, fmt)
            o = torch.empty(T, H, dtype=x.dtype, device=dev)
            if rows_form:
                check(lib.smoe_mxfp8_down_projection_forward_rows(
                    y1q.data_ptr(), y1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), o.data_ptr(),
                    scores_flat.data_ptr(), int(scores_flat.dtype == torch.bfloat16), off,
                    route.x_gather_idx.data_ptr(), route.s_scatter_idx.data_ptr(), H, I, E, TK,
                    st.status.data_ptr(), stream), "mxfp8_down_projection_forward_rows")
            else:
                y2 = torch.empty(TK, H, dtype=x.dtype, device=dev)
                check(_entry("down_projection_forward", fmt)(
                    y1q.data_ptr(), y1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), y2.data_ptr(), off, H, I, E, TK,
                    st.status.data_ptr(), stream), "fp8_down_projection_forward")
                check(lib.smoe_gather_sum(
                    y2.data_ptr(), o.data_ptr(), scores_flat.data_ptr(), _lib.dtype_code(scores_flat.dtype),
                    route.s_reverse_scatter_idx.data_ptr(), ptr(route.token_offset), T, H, max(route.K, 1), stream),
                    "gather_sum")
        if not inference:
            # the quantised weights are kept for the backward pass (1 byte per weight) instead of being rebuilt
            ctx.save_for_backward(x, w1e, w2e, z, scores_flat, w1q, w1s, w2q, w2s)
            ctx.route = route
            ctx.dims = (T, H, I, E, TK)
            ctx.fmt = fmt
            ctx.rows_form = rows_form
        return o

    @staticmethod
    def backward(ctx, dout):
        x, w1e, w2e, z, scores_flat, w1q, w1s, w2q, w2s = ctx.saved_tensors
        route = ctx.route
        T, H, I, E, TK = ctx.dims
        fmt = ctx.fmt
        dev = x.device
        dout = dout.contiguous().to(x.dtype)
        st = _lib.device_state(dev)
        off = route.expert_frequency_offset.data_ptr()
        gat = route.x_gather_idx.data_ptr()
        doutq, douts = quantize_rows(dout, fmt)
        with torch.cuda.device(dev):
            stream = stream_ptr(dev)
            dz = torch.empty(TK, 2 * I, dtype=x.dtype, device=dev)
            y1s = torch.empty(TK, I, dtype=x.dtype, device=dev)
            ncols = lib.smoe_ds_partial_columns(I)
            ds_partial = torch.empty(ncols, TK, dtype=torch.float32, device=dev)
            fused_dz = fmt == "ue8m0"  # the dH epilogue also writes dz quantised (no separate pass over dz)
            if fused_dz:
                ld = lib.smoe_mxfp8_scale_row_bytes(2 * I)
                dzq = torch.empty(TK, 2 * I, dtype=torch.uint8, device=dev)
                if (2 * I // BLOCK) % 4 == 0:
                    dzs = torch.empty(TK, ld, dtype=torch.uint8, device=dev)
                else:  # the kernel does not write the padding bytes of a scale row
                    dzs = torch.full((TK, ld), 127, dtype=torch.uint8, device=dev)
                check(lib.smoe_mxfp8_down_projection_backward_act_q(
                    doutq.data_ptr(), douts.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), z.data_ptr(),
                    scores_flat.data_ptr(), int(scores_flat.dtype == torch.bfloat16), dz.data_ptr(), y1s.data_ptr(),
                    ds_partial.data_ptr(), dzq.data_ptr(), dzs.data_ptr(), off, gat, route.s_scatter_idx.data_ptr(),
                    T, H, I, E, TK, st.status.data_ptr(), stream), "mxfp8_down_projection_backward_act_q")
            else:
                check(_entry("down_projection_backward_act", fmt)(
                    doutq.data_ptr(), douts.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), z.data_ptr(),
                    scores_flat.data_ptr(), int(scores_flat.dtype == torch.bfloat16), dz.data_ptr(), y1s.data_ptr(),
                    ds_partial.data_ptr(), off, gat, route.s_scatter_idx.data_ptr(), T, H, I, E, TK,
                    st.status.data_ptr(), stream), "fp8_down_projection_backward_act")
            ds = torch.empty_like(scores_flat)
            check(lib.smoe_ds_reduce(ds_partial.data_ptr(), route.s_scatter_idx.data_ptr(), ds.data_ptr(),
                                     _lib.dtype_code(ds.dtype), TK, ncols, stream), "ds_reduce")
            # dX before the weight gradients (bf16 GEMMs): nothing downstream waits for those, and an expert-parallel
            # caller sends dx back to the tokens' ranks while they run (route.on_dx)
            if not fused_dz:
                dzq, dzs = quantize_rows(dz, fmt)
            dx = torch.empty(T, H, dtype=x.dtype, device=dev)
            if ctx.rows_form:
                check(lib.smoe_mxfp8_up_projection_backward_dx_rows(
                    dzq.data_ptr(), dzs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), dx.data_ptr(), off, gat, H, I, E,
                    TK, st.status.data_ptr(), stream), "mxfp8_up_projection_backward_dx_rows")
            else:
                dx_expanded = torch.empty(TK, H, dtype=x.dtype, device=dev)
                check(_entry("up_projection_backward_dx", fmt)(
                    dzq.data_ptr(), dzs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), dx_expanded.data_ptr(), off, H, I,
                    E, TK, st.status.data_ptr(), stream), "fp8_up_projection_backward_dx")
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
            up = lib.smoe_up_projection_weight_grad_accumulate if add else lib.smoe_up_projection_weight_grad
            check(up(x.data_ptr(), dz.data_ptr(), dw1.data_ptr(), off, gat, T, H, I, E, TK, st.status.data_ptr(),
                     stream), "up_projection_weight_grad")
            if shared is not None:
                dw1, dw2 = shared.finish_chunk()
                if dw1 is None:
                    return dx, None, None, ds, None, None, None, None
        return dx, dw1.permute(1, 2, 0), dw2.permute(1, 2, 0), ds, None, None, None, None


def moe_fp8_softmax_topk_layer(x, router_w, w1, b1, w2, b2, K, stream_id=0,
                               activation_type: ActivationType | str = ActivationType.SWIGLU,
                               is_inference_mode_enabled: bool = False, scale_format: str | None = None):
    """``moe_TC_softmax_topk_layer`` with the expert GEMMs of forward and activation gradients in FP8
    (``scale_format``: "fp32", "ue8m0" or None for the module default)."""
    from . import _check_experts_args, _route_metadata, topk_softmax

    refuse_unsupported(b1, b2, activation_type)
    activation_type = _check_experts_args(x, w1, w2, b1, b2, activation_type)
    H = x.shape[1]
    if H % BLOCK != 0 or (w1.shape[0] // 2) % BLOCK != 0:
        raise ValueError("the FP8 path needs hidden and intermediate sizes that are multiples of 128")
    E = router_w.size(0)
    T = x.size(0)
    router_logits = F.linear(x if x.dtype == router_w.dtype else x.to(router_w.dtype), router_w)
    scores, indices = topk_softmax(router_logits, K)
    route = _route_metadata(indices.reshape(-1), None, E, K)
    inference = is_inference_mode_enabled or not torch.is_grad_enabled()
    o = _RoutedExpertsFp8.apply(x, w1, w2, scores.reshape(-1), route, T, inference, scale_format)
    return o, router_logits, route.expert_frequency
