"""Expert histogram and inclusive prefix sum (reference: sonicmoe/count_cumsum/__init__.py:17-29)."""

from __future__ import annotations

import torch

from .. import _lib


@torch.no_grad()
def count_cumsum(x: torch.Tensor, E: int, do_cumsum: bool = True):
    """count[e] = number of entries of the 1-D int32/int64 tensor ``x`` equal to e, for e in [0, E).

    Returns ``count`` (int32) or ``(count, cumsum)`` with ``cumsum`` the inclusive prefix sum (int32, no
    leading zero), like the reference.  Runs on the tensor's CUDA device, on the current stream.
    """
    if x.dim() != 1:
        raise ValueError("x should be 1-dimensional")
    if x.dtype not in (torch.int32, torch.int64):
        raise TypeError("x should be int32 or int64")
    _lib.require_cuda(x, "x")
    x = x.contiguous()
    dev = x.device
    with torch.cuda.device(dev):
        count = torch.empty(E, dtype=torch.int32, device=dev)
        cumsum = torch.empty(E, dtype=torch.int32, device=dev) if do_cumsum else None
        # bins beyond 4096 are counted with global atomics and need no scratch
        ws = _lib.device_state(dev).route_workspace(E) if E <= 4096 else None
        rc = _lib.lib.smoe_count_cumsum(
            x.data_ptr(), _lib.dtype_code(x.dtype), x.numel(), E, count.data_ptr(), _lib.ptr(cumsum),
            _lib.ptr(ws), _lib.stream_ptr(dev),
        )
        _lib.check(rc, "count_cumsum")
    return (count, cumsum) if do_cumsum else count
