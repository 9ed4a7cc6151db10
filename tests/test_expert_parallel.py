"""Expert parallelism: the multi-rank host logic on CPU (gloo, world_size 2, device ops supplied by the oracle),
and the CUDA ops on GPU (one rank everywhere; two NCCL ranks when two GPUs are present)."""

import os
import socket
import tempfile

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, ROOT
from oracle import moe_oracle as orc

E, K, H, I = 8, 2, 64, 64
TOKENS = (40, 56, 24, 48, 32, 8, 64, 16)  # tokens per rank (ragged on purpose)


class OracleOps:
    """CPU stand-ins for the device operations, written with differentiable torch ops (test only)."""

    def topk_softmax(self, logits, K):
        idx = torch.sort(logits.float(), dim=-1, descending=True, stable=True).indices[:, :K]
        return torch.softmax(logits.float().gather(-1, idx), dim=-1), idx.to(torch.int32)

    def gather_rows(self, x, rows):
        return x[rows.x_gather_idx.long()]

    def sum_rows(self, entries, rows, T):
        # through the inverse list, as the device kernel does, so that a wrong inverse fails here too
        off = rows.token_offset.tolist()
        rev = rows.s_reverse_scatter_idx.long()
        out = [entries[rev[off[t]:off[t + 1]]].sum(0) for t in range(T)]
        return torch.stack(out) if out else entries.new_zeros(0, entries.shape[1])

    def local_layer(self, x_rows, w1, w2, scores, tokens, experts, num_local_experts, inference):
        assert (tokens[1:] >= tokens[:-1]).all()
        # a function of the rows, the scores and the weights even when no row arrived (as the device layer's autograd node is): every rank
        # then takes part in the backward exchanges
        out = x_rows * 0.0 + 0.0 * (w1.sum() + w2.sum() + scores.sum())
        for e in range(num_local_experts):
            pos = (experts == e).nonzero().squeeze(-1)
            if pos.numel():
                rows = tokens[pos].long()
                out = out.index_add(0, rows, (orc.swiglu(x_rows[rows] @ w1[e].T) @ w2[e].T) * scores[pos, None])
        return out


def _emu_dispatch(x, plan, group=None):
    """What sonicmoe/peer.py's dispatch does, on CPU: every rank writes its segment for rank d at row
    plan.dispatch_offset[d] of rank d's buffer (the writes travel through all_gather_object here)."""
    W, me = dist.get_world_size(group), dist.get_rank(group)
    segs = x[plan.rows.x_gather_idx.long()].split(plan.send_rows)
    out = [None] * W
    dist.all_gather_object(out, [(plan.dispatch_offset[d], segs[d]) for d in range(W)], group=group)
    buf = torch.full((sum(plan.recv_rows), x.shape[1]), float("nan"), dtype=x.dtype)
    for s in range(W):
        off, rows = out[s][me]
        assert rows.shape[0] == plan.recv_rows[s]
        buf[off:off + rows.shape[0]] = rows
    assert not buf.isnan().any()
    return buf


def _emu_return(rows, plan, group=None):
    W, me = dist.get_world_size(group), dist.get_rank(group)
    segs = rows.split(plan.recv_rows)
    out = [None] * W
    dist.all_gather_object(out, [(plan.return_offset[s], segs[s]) for s in range(W)], group=group)
    buf = torch.full((sum(plan.send_rows), rows.shape[1]), float("nan"), dtype=rows.dtype)
    for d in range(W):
        off, r = out[d][me]
        assert r.shape[0] == plan.send_rows[d]
        buf[off:off + r.shape[0]] = r
    assert not buf.isnan().any()
    return buf


def _emu_sum(entries, plan, T):
    return torch.zeros(T, entries.shape[1], dtype=entries.dtype).index_add(0, plan.rows.x_gather_idx.long(), entries)


class _EmuDispatch(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, plan):
        ctx.plan, ctx.T = plan, x.shape[0]
        return _emu_dispatch(x, plan)

    @staticmethod
    def backward(ctx, g):
        return _emu_sum(_emu_return(g, ctx.plan), ctx.plan, ctx.T), None


class _EmuCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, rows, plan, T):
        ctx.plan = plan
        return _emu_sum(_emu_return(rows, plan), plan, T)

    @staticmethod
    def backward(ctx, g):
        return _emu_dispatch(g, ctx.plan), None, None


class EmulatedPeerTransport:
    """The peer-memory transport's addressing (segment offsets inside the other ranks' buffers) without GPUs, with
    the layer's tokens cut into `micro_batches` chunks as the pipelined transport asks for."""

    def __init__(self, micro_batches=1):
        self.micro_batches = micro_batches

    def dispatch_start(self, x, plan, keep, tag):
        return _EmuDispatch.apply(x, plan)

    def dispatch_wait(self, handle):
        return handle

    def combine_start(self, rows, plan, tag):
        return rows

    def combine_finish(self, handle, plan, T):
        return _EmuCombine.apply(handle, plan, T)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(world, dtype):
    full = orc.make_inputs(1, H, I, E, K, seed=0, dtype=dtype, w_std=0.1)
    per_rank = [orc.make_inputs(TOKENS[r], H, I, E, K, seed=100 + r, dtype=dtype) for r in range(world)]
    return full, per_rank


def _logit_bias(E_):
    """The skew of the load-imbalance benchmark at test size: 2 * log(1 / rank) with a seeded permutation of ranks."""
    g = torch.Generator().manual_seed(5)
    return 2.0 * torch.log(1.0 / (torch.randperm(E_, generator=g) + 1).float())


def _worker(rank, world, port, backend, outdir, use_cuda, use_bias=False, emulate_peer=False):
    import sys

    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    if use_cuda:
        torch.cuda.set_device(rank)
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        from sonicmoe.expert_parallel import ExpertParallelMoE

        dtype = torch.bfloat16 if use_cuda else torch.float32
        dev = torch.device("cuda", rank) if use_cuda else torch.device("cpu")
        full, per_rank = _inputs(world, dtype)
        m = ExpertParallelMoE(E, K, H, I).to(dev, dtype)
        m.load_full_state_dict({"router.weight": full["router_w"], "c_fc.weight": full["w1"],
                                "c_proj.weight": full["w2"]})
        if not use_cuda:
            m.ops = OracleOps()
            if emulate_peer:
                m.transport = EmulatedPeerTransport(micro_batches=emulate_peer)
        x = per_rank[rank]["x"].to(dev).requires_grad_(True)
        o, aux = m(x, logit_bias=_logit_bias(E).to(dev) if use_bias else None)
        grads = torch.autograd.grad(o, [x, m.router.weight, m.c_fc.weight, m.c_proj.weight],
                                    per_rank[rank]["dout"].to(dev))
        if use_cuda:
            from sonicmoe import _lib

            torch.cuda.synchronize()
            _lib.check_status()
        torch.save({"o": o.detach().float().cpu(), "aux": aux.detach().float().cpu(),
                    "grads": [g.float().cpu() for g in grads]}, os.path.join(outdir, f"rank{rank}.pt"))
        dist.barrier()
        if use_cuda:
            from sonicmoe.expert_parallel import close_default_transports

            close_default_transports()
    finally:
        dist.destroy_process_group()


def _run_and_check(world, backend, use_cuda, tol, use_bias=False, emulate_peer=False):
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_worker, args=(world, _free_port(), backend, outdir, use_cuda, use_bias, emulate_peer), nprocs=world,
                 join=True)
        res = [torch.load(os.path.join(outdir, f"rank{r}.pt")) for r in range(world)]
    dtype = torch.bfloat16 if use_cuda else torch.float32
    full, per_rank = _inputs(world, dtype)
    f32 = {k: v.float() for k, v in full.items()}
    x_all = torch.cat([p["x"].float() for p in per_rank])
    dout_all = torch.cat([p["dout"].float() for p in per_rank])
    logits = None
    if use_cuda:  # route the oracle on the logits the device computed (bf16 linear, bf16 bias add)
        logits = torch.cat([torch.nn.functional.linear(p["x"].cuda(), full["router_w"].cuda()) for p in per_rank])
        if use_bias:
            logits = logits + _logit_bias(E).cuda().to(logits.dtype)
        logits = logits.float().cpu()
    elif use_bias:
        logits = x_all @ f32["router_w"].T + _logit_bias(E)
    ref = orc.moe_layer(x_all, f32["router_w"], f32["w1"], f32["w2"], K, dout=dout_all, logits=logits)

    def rel(a, b):
        return ((a - b).norm() / (b.norm() + 1e-30)).item()

    e_local = E // world
    start = 0
    drouter = torch.zeros_like(f32["router_w"])
    for r in range(world):
        n = TOKENS[r]
        assert rel(res[r]["o"], ref["o"][start:start + n]) < tol
        assert rel(res[r]["grads"][0], ref["dx"][start:start + n]) < tol
        # every rank holds the full-batch gradient of its own experts
        assert rel(res[r]["grads"][2], ref["dw1"][r * e_local:(r + 1) * e_local]) < tol
        assert rel(res[r]["grads"][3], ref["dw2"][r * e_local:(r + 1) * e_local]) < tol
        drouter += res[r]["grads"][1]
        start += n
    assert rel(drouter, ref["drouter_w"]) < max(tol, 2e-2 if use_cuda else tol)


@pytest.mark.parametrize("world", [2, 4])
def test_expert_parallel_host_logic_gloo(built_library, world):
    _run_and_check(world, "gloo", use_cuda=False, tol=1e-5)


def test_received_pair_tokens():
    from sonicmoe.expert_parallel import received_pair_tokens

    # two sources: 3 rows / 4 pairs from rank 0, 2 rows / 2 pairs from rank 1
    rows = received_pair_tokens(torch.tensor([0, 0, 1, 2, 0, 1], dtype=torch.int32), [3, 2], [4, 2])
    assert rows.tolist() == [0, 0, 1, 2, 3, 4]
    assert received_pair_tokens(torch.zeros(0, dtype=torch.int32), [0, 0], [0, 0]).numel() == 0


def _idle_rank_worker(rank, world, port, outdir):
    """Every token of every rank picks experts of rank 0 only: rank 1 receives no rows and still has to take part
    in every exchange and return zero gradients for its experts."""
    import sys

    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from sonicmoe.expert_parallel import moe_ep_softmax_topk_layer

        full, per_rank = _inputs(world, torch.float32)
        e_local = E // world
        bias = torch.zeros(E)
        bias[:e_local] = 100.0
        x = per_rank[rank]["x"].clone().requires_grad_(True)
        w1 = full["w1"][rank * e_local:(rank + 1) * e_local].clone().requires_grad_(True)
        w2 = full["w2"][rank * e_local:(rank + 1) * e_local].clone().requires_grad_(True)
        o, logits, freq = moe_ep_softmax_topk_layer(x, full["router_w"], w1, w2, K, E, ops=OracleOps(), logit_bias=bias)
        grads = torch.autograd.grad(o, [x, w1, w2], per_rank[rank]["dout"])
        torch.save({"o": o.detach(), "logits": logits.detach(), "grads": grads}, os.path.join(outdir, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_expert_parallel_rank_without_rows_gloo(built_library):
    world = 2
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_idle_rank_worker, args=(world, _free_port(), outdir), nprocs=world, join=True)
        res = [torch.load(os.path.join(outdir, f"rank{r}.pt")) for r in range(world)]
    full, per_rank = _inputs(world, torch.float32)
    x_all = torch.cat([p["x"] for p in per_rank])
    dout_all = torch.cat([p["dout"] for p in per_rank])
    logits = torch.cat([r["logits"] for r in res])
    ref = orc.moe_layer(x_all, full["router_w"], full["w1"], full["w2"], K, dout=dout_all, logits=logits)
    assert ref["expert_frequency"][E // world:].sum() == 0
    n0 = TOKENS[0]
    e_local = E // world
    for r, sl in ((0, slice(0, n0)), (1, slice(n0, n0 + TOKENS[1]))):
        assert (res[r]["o"] - ref["o"][sl]).norm() <= 1e-5 * ref["o"][sl].norm()
        assert (res[r]["grads"][0] - ref["dx"][sl]).norm() <= 1e-5 * ref["dx"][sl].norm()
    assert (res[0]["grads"][1] - ref["dw1"][:e_local]).norm() <= 1e-5 * ref["dw1"][:e_local].norm()
    assert (res[1]["grads"][1] == 0).all() and (res[1]["grads"][2] == 0).all()


@pytest.mark.parametrize("world,micro_batches", [(2, 1), (4, 1), (2, 2), (4, 3), (8, 2)])
def test_peer_transport_addressing_gloo(built_library, world, micro_batches):
    """Segments written at the plan's offsets into the other ranks' buffers reproduce the all-to-all's result, also
    with the tokens cut into chunks that are exchanged and computed one after the other."""
    _run_and_check(world, "gloo", use_cuda=False, tol=1e-5, emulate_peer=micro_batches)


def test_expert_parallel_logit_bias_gloo(built_library):
    _run_and_check(2, "gloo", use_cuda=False, tol=1e-5, use_bias=True)


@pytest.mark.gpu
@pytest.mark.parametrize("use_bias", [False, True])
def test_expert_parallel_single_rank_cuda(built_library, use_bias):
    _run_and_check(1, "nccl", use_cuda=True, tol=1e-2, use_bias=use_bias)


def _fp8_worker(rank, world, port, outdir, fmt):
    """The expert-parallel layer with the FP8 device ops beside the single-device FP8 layer on the same inputs."""
    import sys

    for p in (ROOT, PKG):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world)
    try:
        from sonicmoe import _lib
        from sonicmoe.expert_parallel import Fp8CudaOps, moe_ep_softmax_topk_layer
        from sonicmoe.functional.fp8 import moe_fp8_softmax_topk_layer

        T_, H_, I_, E_, K_ = 600, 256, 128, 8, 2
        inp = orc.make_inputs(T_, H_, I_, E_, K_, seed=21, dtype=torch.bfloat16)
        dev = torch.device("cuda", rank)
        leaves = {k: inp[k].to(dev).requires_grad_(True) for k in ("x", "router_w", "w1", "w2")}
        o, logits, freq = moe_ep_softmax_topk_layer(leaves["x"], leaves["router_w"], leaves["w1"], leaves["w2"], K_, E_,
                                                    ops=Fp8CudaOps(fmt))
        grads = torch.autograd.grad(o, list(leaves.values()), inp["dout"].to(dev))
        o2, _, freq2 = moe_fp8_softmax_topk_layer(leaves["x"], leaves["router_w"], leaves["w1"].permute(1, 2, 0), None,
                                                  leaves["w2"].permute(1, 2, 0), None, K_, scale_format=fmt)
        grads2 = torch.autograd.grad(o2, list(leaves.values()), inp["dout"].to(dev))
        torch.cuda.synchronize()
        _lib.check_status()
        torch.save({"ep": [o.detach().float().cpu()] + [g.float().cpu() for g in grads],
                    "single": [o2.detach().float().cpu()] + [g.float().cpu() for g in grads2],
                    "freq": (freq.cpu(), freq2.cpu()), "logits": logits.detach().float().cpu()},
                   os.path.join(outdir, "rank0.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("fmt", ["fp32", "ue8m0"])
def test_expert_parallel_fp8_ops_single_rank_cuda(built_library, fmt):
    """`Fp8CudaOps` (what the FP8 expert-parallel benchmark runs): equal to the single-device FP8 layer on the same
    inputs, and as close to the fp32 oracle as that layer is (E4M3 x E4M3 products: see test_fp8_gpu.py)."""
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_fp8_worker, args=(1, _free_port(), outdir, fmt), nprocs=1, join=True)
        res = torch.load(os.path.join(outdir, "rank0.pt"))
    assert torch.equal(res["freq"][0], res["freq"][1])
    inp = {k: v.float() for k, v in orc.make_inputs(600, 256, 128, 8, 2, seed=21, dtype=torch.bfloat16).items()}
    ref = orc.moe_layer(inp["x"], inp["router_w"], inp["w1"], inp["w2"], 2, dout=inp["dout"], logits=res["logits"])
    want = [ref["o"], ref["dx"], ref["drouter_w"], ref["dw1"], ref["dw2"]]
    for got_ep, got_single, w in zip(res["ep"], res["single"], want):
        assert (got_ep - got_single).norm() <= 2e-2 * got_single.norm()
        assert (got_ep - w).norm() <= 9e-2 * w.norm()


@pytest.mark.gpu
@pytest.mark.parametrize("transport", ["peer", "peer_pipelined", "nccl"])
def test_expert_parallel_two_ranks_cuda(built_library, transport, monkeypatch):
    """Two ranks on two GPUs: rows over peer memory -- one exchange at a time with the library's gather-and-store
    kernel ("peer", the default), or pipelined over two chunks of tokens with copy-engine copies on a second stream
    ("peer_pipelined") -- into buffers mapped through CUDA IPC, and over the NCCL all-to-all."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    monkeypatch.setenv("SONICMOE_EP_TRANSPORT", transport)
    monkeypatch.setenv("NCCL_NVLS_ENABLE", "0")
    _run_and_check(2, "nccl", use_cuda=True, tol=1e-2)
