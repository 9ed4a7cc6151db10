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
TOKENS = (40, 56, 24, 48)  # tokens per rank (ragged on purpose)


class OracleOps:
    """CPU stand-ins for the device operations, written with differentiable torch ops (test only)."""

    def topk_softmax(self, logits, K):
        idx = torch.sort(logits.float(), dim=-1, descending=True, stable=True).indices[:, :K]
        return torch.softmax(logits.float().gather(-1, idx), dim=-1), idx.to(torch.int32)

    def route_metadata(self, expert_idx, E, K):
        r = orc.route_metadata(expert_idx, E, expert_idx.numel() // K, K=K)
        r.K = K
        return r

    def gather_rows(self, x, route):
        return x[route.x_gather_idx.long()]

    def sum_rows(self, rows, route, T):
        return rows[route.s_reverse_scatter_idx.long()].view(T, route.K, -1).sum(1)

    def local_experts(self, x_rows, w1, w2, scores, local_expert, num_local_experts, inference):
        out = torch.zeros_like(x_rows)
        for e in range(num_local_experts):
            pos = (local_expert == e).nonzero().squeeze(-1)
            if pos.numel():
                out = out.index_add(0, pos, (orc.swiglu(x_rows[pos] @ w1[e].T) @ w2[e].T) * scores[pos, None])
        return out


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(world, dtype):
    full = orc.make_inputs(1, H, I, E, K, seed=0, dtype=dtype, w_std=0.1)
    per_rank = [orc.make_inputs(TOKENS[r], H, I, E, K, seed=100 + r, dtype=dtype) for r in range(world)]
    return full, per_rank


def _worker(rank, world, port, backend, outdir, use_cuda):
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
        x = per_rank[rank]["x"].to(dev).requires_grad_(True)
        o, aux = m(x)
        grads = torch.autograd.grad(o, [x, m.router.weight, m.c_fc.weight, m.c_proj.weight],
                                    per_rank[rank]["dout"].to(dev))
        if use_cuda:
            from sonicmoe import _lib

            torch.cuda.synchronize()
            _lib.check_status()
        torch.save({"o": o.detach().float().cpu(), "aux": aux.detach().float().cpu(),
                    "grads": [g.float().cpu() for g in grads]}, os.path.join(outdir, f"rank{rank}.pt"))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _run_and_check(world, backend, use_cuda, tol):
    with tempfile.TemporaryDirectory() as outdir:
        mp.spawn(_worker, args=(world, _free_port(), backend, outdir, use_cuda), nprocs=world, join=True)
        res = [torch.load(os.path.join(outdir, f"rank{r}.pt")) for r in range(world)]
    dtype = torch.bfloat16 if use_cuda else torch.float32
    full, per_rank = _inputs(world, dtype)
    f32 = {k: v.float() for k, v in full.items()}
    x_all = torch.cat([p["x"].float() for p in per_rank])
    dout_all = torch.cat([p["dout"].float() for p in per_rank])
    logits = None
    if use_cuda:  # route the oracle on the logits the device computed (bf16 linear)
        logits = torch.cat([torch.nn.functional.linear(p["x"].cuda(), full["router_w"].cuda()).float().cpu()
                            for p in per_rank])
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


def test_dispatch_plan_helpers():
    from sonicmoe.expert_parallel import received_row_experts

    counts = torch.tensor([[2, 0, 1], [0, 3, 1]], dtype=torch.int32)  # (W=2, E_l=3)
    assert received_row_experts(counts).tolist() == [0, 0, 2, 1, 1, 1, 2]
    assert received_row_experts(torch.zeros(2, 3, dtype=torch.int32)).numel() == 0


@pytest.mark.gpu
def test_expert_parallel_single_rank_cuda(built_library):
    _run_and_check(1, "nccl", use_cuda=True, tol=1e-2)


@pytest.mark.gpu
def test_expert_parallel_two_ranks_cuda(built_library):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    _run_and_check(2, "nccl", use_cuda=True, tol=1e-2)
