"""CPU simulation of the FP8 (E4M3, block-scaled) expert path.  TEST INFRASTRUCTURE ONLY.

The reference has no FP8 path, so there is nothing to restate: this file applies, in plain PyTorch on the
CPU, the same quantisation points as the device path (activations per row and 128 columns, weights per
128 x 128 block, scale = amax / 448 -- or, with ``pow2=True``, the smallest power of two not below it, the form
the tensor cores' own block scaling takes -- round-to-nearest E4M3) around the fp32 expert math of
``oracle.moe_oracle``.  Tests use it to separate the error of the number format (this simulation vs the fp32
oracle) from the error of the kernels (device vs this simulation).
"""

from __future__ import annotations

import torch

from . import moe_oracle as orc

FP8_MAX = 448.0


def block_scale(amax: torch.Tensor, pow2: bool) -> torch.Tensor:
    """amax / 448 (1 for an all-zero block); pow2: rounded up to a power of two, at least 2^-127."""
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    if pow2:
        m, e = torch.frexp(scale)            # scale = m 2^e, m in [0.5, 1)
        e = torch.where(m == 0.5, e - 1, e).clamp(min=-127)
        scale = torch.where(amax > 0, torch.ldexp(torch.ones_like(scale), e), torch.ones_like(scale))
    return scale


def _fake_quant(x: torch.Tensor, amax: torch.Tensor, pow2: bool = False) -> torch.Tensor:
    scale = block_scale(amax, pow2)
    q = (x / scale).to(torch.float8_e4m3fn).float()
    return q * scale


def quant_rows(x: torch.Tensor, pow2: bool = False) -> torch.Tensor:
    """Quantise-dequantise with one scale per row and 128 consecutive columns."""
    rows, cols = x.shape
    v = x.float().view(rows, cols // 128, 128)
    return _fake_quant(v, v.abs().amax(-1, keepdim=True), pow2).view(rows, cols)


def quant_blocks(w: torch.Tensor, pow2: bool = False) -> torch.Tensor:
    """Quantise-dequantise with one scale per 128 x 128 block of each expert's matrix."""
    E, rows, cols = w.shape
    rb = (rows + 127) // 128
    pad = torch.zeros(E, rb * 128, cols)
    pad[:, :rows] = w.float()
    v = pad.view(E, rb, 128, cols // 128, 128)
    out = _fake_quant(v, v.abs().amax(dim=(2, 4), keepdim=True), pow2).view(E, rb * 128, cols)
    return out[:, :rows]


def bf16(x: torch.Tensor) -> torch.Tensor:
    return x.bfloat16().float()


def experts_forward_backward(x, w1, w2, scores_flat, route: orc.Route, dout, pow2: bool = False):
    """Forward and backward of the routed experts with the device path's rounding points:
    fp8 operands for the forward and activation-gradient GEMMs, bf16 z / y1 / y2 / dz / y1s, bf16 weight-gradient
    GEMMs.  x, w1, w2, dout hold bf16-representable fp32 values."""
    T, H = x.shape
    E = w1.shape[0]
    off = route.expert_frequency_offset.tolist()
    g = route.x_gather_idx.long()
    xq, w1q, w2q = quant_rows(x, pow2), quant_blocks(w1, pow2), quant_blocks(w2, pow2)
    TK = g.numel()
    z = torch.empty(TK, w1.shape[1])
    for e in range(E):
        z[off[e]:off[e + 1]] = xq[g[off[e]:off[e + 1]]] @ w1q[e].T
    y1 = bf16(orc.swiglu(z))
    zb = bf16(z)
    y1q = quant_rows(y1, pow2)
    y2 = torch.empty(TK, H)
    for e in range(E):
        y2[off[e]:off[e + 1]] = y1q[off[e]:off[e + 1]] @ w2q[e].T
    y2 = bf16(y2)
    s = scores_flat.reshape(-1)[route.s_scatter_idx.long()]
    o = torch.zeros(T, H).index_add(0, g, y2 * s[:, None])
    # backward
    dq = quant_rows(dout, pow2)
    dy1 = torch.empty(TK, w2.shape[2])
    for e in range(E):
        dy1[off[e]:off[e + 1]] = dq[g[off[e]:off[e + 1]]] @ w2q[e]
    gate, up = zb[:, 0::2], zb[:, 1::2]
    sig = torch.sigmoid(gate)
    y1r = gate * sig * up
    ds_rows = (dy1 * y1r).sum(-1)
    dz = bf16(torch.stack([dy1 * up * sig * (1 + gate * (1 - sig)) * s[:, None], dy1 * gate * sig * s[:, None]],
                          dim=-1).reshape(TK, -1))
    y1s = bf16(y1r * s[:, None])
    dzq = quant_rows(dz, pow2)
    dw1 = torch.zeros_like(w1)
    dw2 = torch.zeros_like(w2)
    dx_exp = torch.empty(TK, H)
    for e in range(E):
        a, b = off[e], off[e + 1]
        dw2[e] = dout[g[a:b]].T @ y1s[a:b]
        dw1[e] = dz[a:b].T @ x[g[a:b]]
        dx_exp[a:b] = dzq[a:b] @ w1q[e]
    dx = torch.zeros(T, H).index_add(0, g, bf16(dx_exp))
    ds = torch.empty_like(ds_rows)
    ds[route.s_scatter_idx.long()] = ds_rows
    return dict(o=o, dx=dx, dw1=dw1, dw2=dw2, ds=ds)
