"""Peer-memory transport of the expert-parallel layer (one node, NVLink / NVSwitch).

Every rank owns a few exchange buffers that the other ranks map through CUDA IPC (`smoe_peer_*` in the library).
Token rows then move with the library's own kernels and copy-engine copies instead of an NCCL all-to-all:

* dispatch: `smoe_gather_sum_to_peers` gathers the routed rows and stores each one directly into its destination
  rank's buffer (the gather and the send are one kernel, no staging copy);
* combine: the rows an expert rank computed for another rank's tokens are contiguous per source rank, so they go
  back with one copy-engine copy per peer (`smoe_peer_copy`), and the source adds up each token's rows.

After the writes of an exchange every rank joins a one-element all-reduce on the same stream (NCCL, a few
microseconds): when it completes on a rank, every peer's writes into that rank's buffer have completed.  The same
barriers order buffer reuse: a buffer is written again only after another exchange's barrier, which its owner joins
only after the kernels that read the buffer.  The buffer that receives the dispatched rows of the forward pass also
holds them for the backward pass (they are the layer's saved activation), so it rotates over `depth` slots: that
many forward passes may be in flight before their backward passes.

Exchanges that run on the copy stream beside the GEMMs (`AsyncPeerTransport.send_async`) end with arrival flags
instead of that barrier: after a destination's segment the sender copies its exchange counter into the destination's
flag word, and whoever reads the rows makes its stream wait (a stream memory operation, no kernel) until all W
words have reached the exchange's number.  A reader therefore waits for every sender of every exchange, and buffer
reuse stays ordered without a global barrier.  Per buffer, written in exchange X of step n and again in step n + 1:
a sender produces the rows of the second write only after its compute stream has consumed a later exchange Y from
the buffer's owner, and the owner started Y after the kernels that read the buffer on its own compute stream --
return_fwd (read by the forward pass's final sum; Y = the next step's dispatch), dispatch_bwd (read by dH and dW2;
Y = the next step's forward return), return_bwd (read by the backward pass's final sum; Y = the next step's dispatch
of the output gradient).  The buffer of the forward dispatch is read as late as dW1, after the dx return has already
left, which is why it alternates between `depth` >= 2 slots (Y = any exchange of the step in between).

Requirements: one process per GPU on one node, every rank able to map every other rank's memory (peer access),
bf16 rows whose length is a multiple of 8.
"""

from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from . import _lib
from ._lib import check, lib, stream_ptr


class _DeviceMemory:
    """A raw device allocation presented to torch through the CUDA array interface."""

    def __init__(self, ptr: int, nbytes: int):
        self.ptr, self.nbytes = ptr, nbytes
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerMemoryUnavailable(RuntimeError):
    """Some rank could not allocate, export or map an exchange buffer (raised on every rank of the group)."""


class PeerBuffer:
    """`nbytes` of device memory on this rank, and where every rank's buffer of the same name is mapped here.

    Construction is collective, and so is its failure: every rank reports whether its part worked, and if any
    rank's did not, all of them undo theirs and raise `PeerMemoryUnavailable` together (no rank is left waiting in a
    collective for one that gave up)."""

    def __init__(self, nbytes: int, group, device: torch.device):
        self.group, self.device, self.nbytes = group, device, nbytes
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.own_ptr, self.ptrs, self.bytes = None, [], None
        with torch.cuda.device(device):
            own = ctypes.c_void_p()
            handle = (ctypes.c_ubyte * 64)()
            mine_ok = lib.smoe_peer_alloc(nbytes, ctypes.byref(own)) == 0
            if mine_ok:
                self.own_ptr = own.value
                mine_ok = lib.smoe_peer_export(self.own_ptr, handle) == 0
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle) if mine_ok else None, group=group)
            opened = []
            if mine_ok and all(h is not None for h in handles):
                for r, h in enumerate(handles):
                    if r == self.rank:
                        self.ptrs.append(self.own_ptr)
                        continue
                    p = ctypes.c_void_p()
                    raw = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                    if lib.smoe_peer_open(raw, ctypes.byref(p)) != 0:
                        mine_ok = False
                        break
                    opened.append(p.value)
                    self.ptrs.append(p.value)
            else:
                mine_ok = False
            all_ok = torch.tensor([1 if mine_ok else 0], dtype=torch.int32, device=device)
            dist.all_reduce(all_ok, op=dist.ReduceOp.MIN, group=group)
            if all_ok.item() == 0:
                for p in opened:
                    lib.smoe_peer_close(p)
                dist.barrier(group=group)
                if self.own_ptr is not None:
                    lib.smoe_peer_free(self.own_ptr)
                self.own_ptr, self.ptrs = None, []
                raise PeerMemoryUnavailable("an exchange buffer could not be allocated, exported or mapped on some rank "
                                            "(CUDA IPC / peer access between the GPUs of this node)")
            self.bytes = torch.as_tensor(_DeviceMemory(self.own_ptr, nbytes), device=device)

    def rows(self, n: int, H: int, dtype: torch.dtype) -> torch.Tensor:
        """The first n rows of this rank's buffer as an (n, H) tensor."""
        item = torch.empty(0, dtype=dtype).element_size()
        return self.bytes[: n * H * item].view(dtype).view(n, H)

    def close(self) -> None:
        """Collective: unmap the peers' buffers, then (after everybody has) free this rank's."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for r, p in enumerate(self.ptrs):
                if r != self.rank:
                    lib.smoe_peer_close(p)
            self.ptrs = []
            dist.barrier(group=self.group)
            self.bytes = None
            lib.smoe_peer_free(self.own_ptr)
            self.own_ptr = None


class PeerTransport:
    """dispatch / combine of token rows over peer memory.  `plan` is an `expert_parallel.DispatchPlan`."""

    def __init__(self, group, device: torch.device, depth: int = 2):
        self.group, self.device, self.depth = group, device, depth
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > lib_max_peers():
            raise ValueError(f"the peer transport handles at most {lib_max_peers()} ranks")
        self.buffers: dict[tuple, PeerBuffer] = {}
        self.flag = torch.zeros(1, dtype=torch.float32, device=device)
        self.slot = 0
        self.leased = [False] * depth
        # find out now, together, whether the ranks can map each other's memory at all
        PeerBuffer(1 << 16, group, device).close()

    # -- plumbing ------------------------------------------------------------------------------------------
    def _buffer(self, key: tuple, nbytes: int) -> PeerBuffer:
        """Every rank asks for the same (key, nbytes) in the same order, so (re)allocation is collective."""
        buf = self.buffers.get(key)
        if buf is None or buf.nbytes < nbytes:
            if buf is not None:
                buf.close()
            buf = self.buffers[key] = PeerBuffer(nbytes, self.group, self.device)
        return buf

    def _barrier(self) -> None:
        dist.all_reduce(self.flag, group=self.group)

    def close(self) -> None:
        for buf in self.buffers.values():
            buf.close()
        self.buffers = {}

    # -- the two exchanges ---------------------------------------------------------------------------------
    def dispatch_rows(self, x: torch.Tensor, plan, key: tuple) -> torch.Tensor:
        """Rows plan.rows.x_gather_idx of x, delivered to their destination ranks; returns the rows this rank
        received (source by source), a view of the exchange buffer `key`."""
        _lib.require_cuda(x, "rows")
        if x.dtype != torch.bfloat16 or x.shape[1] % 8 != 0:
            raise TypeError("the peer transport moves bf16 rows whose length is a multiple of 8")
        x = x.contiguous()
        H = x.shape[1]
        W = self.world
        buf = self._buffer(key, W * plan.token_capacity * H * 2)
        n = plan.rows.x_gather_idx.numel()
        seg_ptr = (ctypes.c_void_p * W)(*[buf.ptrs[d] + plan.dispatch_offset[d] * H * 2 for d in range(W)])
        starts = [0]
        for d in range(W):
            starts.append(starts[-1] + plan.send_rows[d])
        seg_start = (ctypes.c_int * (W + 1))(*starts)
        # start with the right-hand neighbour's segment (wrapping round to this rank's own last): at any moment the
        # ranks then write to different destinations
        first = starts[(self.rank + 1) % W] if n > 0 else 0
        if first >= n:
            first = 0
        with torch.cuda.device(self.device):
            check(lib.smoe_gather_sum_to_peers(x.data_ptr(), None, 0, plan.rows.x_gather_idx.data_ptr(), None, n, H, 1,
                                               seg_ptr, seg_start, W, first, stream_ptr(self.device)),
                  "gather_sum_to_peers")
            self._barrier()
        return buf.rows(sum(plan.recv_rows), H, x.dtype)

    def return_rows(self, rows: torch.Tensor, plan, key: tuple) -> torch.Tensor:
        """The inverse exchange: segment s of `rows` (what rank s dispatched here) goes back to rank s; returns this
        rank's entries in dispatch order (destination-major), a view of the exchange buffer `key`."""
        _lib.require_cuda(rows, "rows")
        rows = rows.contiguous()
        H = rows.shape[1]
        W = self.world
        item = rows.element_size()
        buf = self._buffer(key, W * plan.token_capacity * H * item)
        with torch.cuda.device(self.device):
            stream = stream_ptr(self.device)
            starts = [0]
            for s in range(W):
                starts.append(starts[-1] + plan.recv_rows[s])
            for k in range(1, W + 1):  # right-hand neighbour first, this rank's own segment last (see dispatch_rows)
                s = (self.rank + k) % W
                check(lib.smoe_peer_copy(buf.ptrs[s] + plan.return_offset[s] * H * item,
                                         rows.data_ptr() + starts[s] * H * item, plan.recv_rows[s] * H * item, stream),
                      "peer_copy")
            self._barrier()
        return buf.rows(sum(plan.send_rows), H, rows.dtype)

    # -- slots of the buffer that keeps the forward pass's received rows for the backward pass --------------------
    def take_slot(self, keep: bool) -> int:
        slot = self.slot
        if self.leased[slot]:
            raise RuntimeError(f"{self.depth} forward passes of the expert-parallel layer are already waiting for their "
                               "backward pass: construct PeerTransport with a larger depth")
        self.leased[slot] = keep
        self.slot = (slot + 1) % self.depth
        return slot

    def release_slot(self, slot: int) -> None:
        self.leased[slot] = False


# Exchange timing (benchmarks): while a list is installed here, send_async appends (start, end) CUDA event pairs
# recorded on the copy stream around each exchange (copies + barrier).
exchange_events: list | None = None


class _Arrived:
    """Exchange number `seq` of a transport: its rows are here once every sender's flag word has reached `seq`."""

    def __init__(self, seq: int):
        self.seq = seq


class AsyncPeerTransport(PeerTransport):
    """The peer transport with its copies on a second, high-priority stream: `send_async` returns at once with a
    token; whoever reads the received rows hands it to `compute_wait` first.  Segments travel with copy-engine
    copies only (no kernel), so they run beside kernels that occupy every multiprocessor, and arrival is signalled
    by flag words that the streams write and wait for themselves.  Where the driver offers no stream memory
    operations, each exchange ends with a one-element all-reduce on a process group of its own instead (so that it
    never queues behind the layer's small all-to-alls)."""

    def __init__(self, group, device: torch.device, depth: int = 2):
        super().__init__(group, device, depth)
        ranks = dist.get_process_group_ranks(group) if group is not None else list(range(dist.get_world_size()))
        self.barrier_group = dist.new_group(ranks=ranks, backend="nccl")
        with torch.cuda.device(device):
            self.comm = torch.cuda.Stream(device=device, priority=-1)
        # Arrival flags: word p of `flags` on this rank = number of the last exchange whose rows from rank p have
        # landed here.  Written by the senders' copy engines, waited for by this rank's streams: no kernel on either
        # side.  Without stream memory operations (or SONICMOE_EP_BARRIER=nccl) every exchange ends with an
        # all-reduce barrier on the copy stream instead.
        self.seq = 0
        self.counter = torch.zeros(1, dtype=torch.int32, device=device)
        self.flags = None
        ok = os.environ.get("SONICMOE_EP_BARRIER", "flags") == "flags" and self._stream_values_work()
        verdict = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
        dist.all_reduce(verdict, op=dist.ReduceOp.MIN, group=group)
        if verdict.item() == 1:
            self.flags = PeerBuffer(1 << 16, group, device)

    def _stream_values_work(self) -> bool:
        with torch.cuda.device(self.device):
            stream = self.comm.cuda_stream
            ok = (lib.smoe_stream_write_value(self.counter.data_ptr(), 0, stream) == 0 and
                  lib.smoe_stream_wait_values(self.counter.data_ptr(), 1, 0, stream) == 0)
            self.comm.synchronize()
        return ok

    def close(self) -> None:
        if self.flags is not None:
            self.flags.close()
            self.flags = None
        super().close()

    def mark_compute(self) -> torch.cuda.Event:
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        return ev

    def compute_wait(self, landed) -> None:
        """The current stream waits for what `send_async` returned: the rows of that exchange are in this rank's
        buffer afterwards."""
        if isinstance(landed, _Arrived):
            with torch.cuda.device(self.device):
                check(lib.smoe_stream_wait_values(self.flags.own_ptr, self.world, landed.seq, stream_ptr(self.device)),
                      "stream_wait_values")
        else:
            torch.cuda.current_stream(self.device).wait_event(landed)

    def send_async(self, src: torch.Tensor, seg_rows: list[int], dst_offsets: list[int], n_recv: int, key: tuple,
                   token_capacity: int, after: torch.cuda.Event | None = None):
        """Segment d of `src` (seg_rows[d] consecutive rows) goes to row dst_offsets[d] of rank d's buffer `key`, once
        `after` (default: everything issued so far on the current stream) has happened.  Returns (what to hand to
        `compute_wait` before reading, this rank's first n_recv rows of the buffer).  Every rank calls this the same
        number of times in the same order (the exchanges are numbered)."""
        _lib.require_cuda(src, "rows")
        src = src.contiguous()
        H = src.shape[1]
        item = src.element_size()
        W = self.world
        buf = self._buffer(key, W * token_capacity * H * item)
        if after is None:
            after = self.mark_compute()
        with torch.cuda.device(self.device), torch.cuda.stream(self.comm):
            self.comm.wait_event(after)
            timing = exchange_events is not None
            if timing:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(self.comm)
            stream = self.comm.cuda_stream
            starts = [0]
            for d in range(W):
                starts.append(starts[-1] + seg_rows[d])
            if self.flags is not None:
                self.seq = (self.seq + 1) & 0xFFFFFFFF
                check(lib.smoe_stream_write_value(self.counter.data_ptr(), self.seq, stream), "stream_write_value")
            for k in range(1, W + 1):  # right-hand neighbour first: no two ranks copy to the same destination at once
                d = (self.rank + k) % W
                check(lib.smoe_peer_copy(buf.ptrs[d] + dst_offsets[d] * H * item, src.data_ptr() + starts[d] * H * item,
                                         seg_rows[d] * H * item, stream), "peer_copy")
                if self.flags is not None:  # the segment has landed: tell its receiver
                    check(lib.smoe_peer_copy(self.flags.ptrs[d] + 4 * self.rank, self.counter.data_ptr(), 4, stream),
                          "peer_copy")
            if self.flags is not None:
                done = _Arrived(self.seq)
            else:
                dist.all_reduce(self.flag, group=self.barrier_group)
                done = torch.cuda.Event()
                done.record(self.comm)
            if timing:
                e1.record(self.comm)
                exchange_events.append((e0, e1))
        src.record_stream(self.comm)
        return done, buf.rows(n_recv, H, src.dtype)


def lib_max_peers() -> int:
    return 16  # SMOE_MAX_PEERS
