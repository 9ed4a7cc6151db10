"""The CPU oracle against the fixtures produced by the reference's own code (tests/golden/make_golden.py)."""

import numpy as np
import pytest
import torch

from conftest import golden
from oracle import moe_oracle as orc

LAYER = ["layer_small", "layer_ties", "layer_k1"]


def _inputs(meta):
    T, H, I, E, K, seed, is_bf16 = [int(v) for v in meta]
    inp = orc.make_inputs(T, H, I, E, K, seed=seed, dtype=torch.bfloat16 if is_bf16 else torch.float32)
    return (T, H, I, E, K), {k: v.float() for k, v in inp.items()}


def _close(a, b, tol=2e-5):
    a = torch.as_tensor(np.asarray(a)).double()
    b = torch.as_tensor(np.asarray(b)).double()
    err = (a - b).norm() / (b.norm() + 1e-30)
    assert err < tol, f"relative Frobenius error {err:.3e}"


@pytest.mark.parametrize("name", LAYER)
def test_layer_forward_backward_matches_reference(name):
    g = golden(name)
    (T, H, I, E, K), inp = _inputs(g["meta"])
    r = orc.moe_layer(inp["x"], inp["router_w"], inp["w1"], inp["w2"], K, dout=inp["dout"])
    _close(r["logits"], g["logits"])
    assert torch.equal(r["expert_frequency"], torch.from_numpy(g["expert_frequency"]))
    _close(r["o"], g["o"])
    _close(r["aux_loss"], g["aux_loss"])
    _close(r["dx"], g["dx"])
    _close(r["drouter_w"], g["drouter_w"])
    _close(r["dw1"], g["dw1"])
    _close(r["dw2"], g["dw2"])


def test_layer_config1_summaries():
    """The CPU-runnable benchmark configuration (T2048 H768 I256 E8 K2, fp32): norm, sum and a strided sample of every tensor."""
    g = golden("layer_cfg1")
    (T, H, I, E, K), inp = _inputs(g["meta"])
    r = orc.moe_layer(inp["x"], inp["router_w"], inp["w1"], inp["w2"], K, dout=inp["dout"])
    assert torch.equal(r["expert_frequency"], torch.from_numpy(g["expert_frequency"]))
    for key in ("o", "dx", "drouter_w", "dw1", "dw2", "logits"):
        flat = r[key].reshape(-1).double()
        step = max(1, flat.numel() // 64)
        got = np.concatenate([[flat.norm().item(), flat.sum().item()], flat[::step][:64].numpy()])
        ref = g[key]
        assert abs(got[0] - ref[0]) <= 2e-5 * abs(ref[0]), key
        assert abs(got[1] - ref[1]) <= 2e-4 * abs(ref[0]), key
        _close(got[2:], ref[2:], tol=1e-4)
    _close(r["aux_loss"], g["aux_loss"])


def test_topk_tie_rule():
    logits = torch.tensor([[1.0, 3.0, 3.0, 0.5, 3.0, -0.0, 0.0, 2.0]])
    s, idx = orc.topk_softmax(logits, 4)
    assert idx.tolist() == [[1, 2, 4, 7]]
    assert abs(s.sum().item() - 1) < 1e-6
    s, idx = orc.topk_softmax(torch.tensor([[0.0, -0.0, -1.0, -0.0]]), 3)
    assert idx.tolist() == [[0, 1, 3]]


@pytest.mark.parametrize("n,E", [(0, 8), (1, 4), (1000, 8), (4099, 72), (70000, 256)])
def test_count_cumsum_and_route_metadata(n, E):
    g = torch.Generator().manual_seed(n + E)
    idx = torch.randint(0, E, (n,), generator=g, dtype=torch.int32)
    c, cs = orc.count_cumsum(idx, E)
    assert c.dtype == torch.int32 and cs.dtype == torch.int32
    assert c.sum().item() == n and (cs[-1].item() == n)
    K = 1
    r = orc.route_metadata(idx, E, n, K=K)
    assert r.expert_frequency_offset[0] == 0 and r.expert_frequency_offset[-1] == n
    sorted_e = idx[r.s_scatter_idx.long()]
    assert torch.equal(sorted_e, sorted_e.sort().values)
    assert torch.equal(r.s_reverse_scatter_idx[r.s_scatter_idx.long()].long(), torch.arange(n))
    # stable: slots of one expert ascend
    for e in range(min(E, 8)):
        a, b = r.expert_frequency_offset[e].item(), r.expert_frequency_offset[e + 1].item()
        seg = r.s_scatter_idx[a:b]
        assert torch.equal(seg, seg.sort().values)


@pytest.mark.parametrize("name", ["rounding_nr", "rounding_up", "rounding_down"])
def test_token_rounding_matches_reference(name):
    g = golden(name)
    T, H, I, E, K, seed = [int(v) for v in g["meta"]]
    routing = str(g["routing"])
    inp = orc.make_inputs(T, H, I, E, K, seed=seed, dtype=torch.float32)
    logits = inp["x"] @ inp["router_w"].T
    scores, tokens, experts, _ = orc.token_rounding_route(logits, K, routing, torch.float32)
    # the reference orders the pairs of one token arbitrarily: compare as sorted (token, expert) lists
    def canon(tok, exp, sc):
        key = tok.long() * E + exp.long()
        o = key.argsort()
        return key[o], sc[o]
    k_ref, s_ref = canon(torch.from_numpy(g["tokens"]), torch.from_numpy(g["experts"]), torch.from_numpy(g["scores"]))
    k_got, s_got = canon(tokens, experts, scores)
    assert torch.equal(k_got, k_ref)
    _close(s_got, s_ref, tol=1e-6)
    counts = torch.bincount(experts.long(), minlength=E)
    assert (counts % 128 == 0).all()
    assert torch.equal(tokens, tokens.sort().values)
    r = orc.general_routing_layer(inp["x"], inp["w1"], inp["w2"], scores, tokens, experts)
    _close(r["o"], g["o"])


def test_general_routing_gradients_match_autograd():
    """The hand-derived backward of the oracle against autograd on an independent per-expert formulation."""
    T, H, I, E, K = 48, 32, 16, 4, 2
    inp = orc.make_inputs(T, H, I, E, K, seed=7, x_std=1.0, w_std=0.2)
    g = torch.Generator().manual_seed(3)
    n = 100
    tokens = torch.randint(0, T, (n,), generator=g).sort().values.int()
    experts = torch.randint(0, E, (n,), generator=g).int()
    scores = torch.rand(n, generator=g)
    x = inp["x"].clone().requires_grad_(True)
    w1 = inp["w1"].clone().requires_grad_(True)
    w2 = inp["w2"].clone().requires_grad_(True)
    sc = scores.clone().requires_grad_(True)
    o = torch.zeros(T, H)
    for e in range(E):
        pos = experts == e
        t_idx = tokens[pos].long()
        h = x[t_idx] @ w1[e].T
        h = torch.nn.functional.silu(h[:, ::2]) * h[:, 1::2]
        o = o.index_add(0, t_idx, (h @ w2[e].T) * sc[pos, None])
    grads = torch.autograd.grad(o, [x, w1, w2, sc], inp["dout"])
    r = orc.general_routing_layer(inp["x"], inp["w1"], inp["w2"], scores, tokens, experts, dout=inp["dout"])
    _close(r["o"], o.detach(), tol=1e-5)
    for got, ref in zip((r["dx"], r["dw1"], r["dw2"], r["ds"]), grads):
        _close(got, ref, tol=1e-5)
