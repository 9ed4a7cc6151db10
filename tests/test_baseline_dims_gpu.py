"""Parity at the dimensions of the benchmark configurations (full H / I / E / K, fewer tokens).

Every kernel of the layer is called through the C ABI in the order the layer calls them, each one fed by the
previous one's device output, and the whole chain is compared with the CPU oracle's fp32 chain:
`z, y1, o, dz, y1s, ds, dx, dW1, dW2` by relative Frobenius error <= 1e-2 (the bound stated for the bf16 layer),
routing (top-k indices, expert counts, offsets, the three index vectors) bit-exact on the logits the device
computed.  Shapes follow the reference's own test matrix (tests/moe_test.py:25-56) at the benchmark sizes:

* config 2: H 4096, I 1024, E 128, K 8 -- 64-k-block main loops, N = 2048 / 4096 dual-tile schedules;
* config 3: H 4096, I 1024, E 256, K 8 with token rounding to multiples of 128 ("nr"), caller-supplied pairs;
* config 5: H 2048, I 768, E 64, K 4 with the Zipf logit bias -- I = 768 is where dW2 falls back to single tiles
  and where a 512-wide unit would be half empty;
* the expert-parallel FP8 layer's per-rank shape (H 7168, I 2048, 32 local experts) for the bf16 kernels.

Weights are drawn on the GPU (seeded) and copied to the host for the oracle, so a 128-expert layer costs
seconds, not minutes, to set up.
"""

import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-2


def rel(a, b):
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


def draw(T, H, I, E, seed):
    """bf16 layer inputs as in the benchmark: weights N(0, 0.02), x and the upstream gradient N(0, 1)."""
    g = torch.Generator(device="cuda").manual_seed(seed)

    def rn(*shape, std):
        return (torch.randn(*shape, generator=g, device="cuda") * std).bfloat16()

    return dict(router_w=rn(E, H, std=0.02), w1=rn(E, 2 * I, H, std=0.02), w2=rn(E, H, I, std=0.02),
                x=rn(T, H, std=1.0), dout=rn(T, H, std=1.0))


def device_chain(_lib, inp, scores_flat, route, T, H, I, E, fixed_k):
    """The layer's kernels in order through the C ABI; returns every intermediate (device tensors)."""
    lib = _lib.lib
    dev = torch.device("cuda", 0)
    st = _lib.device_state(dev).status
    stream = torch.cuda.current_stream().cuda_stream
    TK = route.x_gather_idx.numel()
    off, gat, sct, rev = (route.expert_frequency_offset.data_ptr(), route.x_gather_idx.data_ptr(),
                          route.s_scatter_idx.data_ptr(), route.s_reverse_scatter_idx.data_ptr())
    tok_off = None if route.token_offset is None else route.token_offset.data_ptr()
    x, w1, w2, dout = inp["x"], inp["w1"], inp["w2"], inp["dout"]
    nan = float("nan")

    def full(*shape, dtype=torch.bfloat16):
        return torch.full(shape, nan, dtype=dtype, device=dev)

    out = {}
    z, y1 = full(TK, 2 * I), full(TK, I)
    assert lib.smoe_up_projection_forward(x.data_ptr(), w1.data_ptr(), z.data_ptr(), y1.data_ptr(), off, gat,
                                          T, H, I, E, TK, st.data_ptr(), stream) == 0
    y2 = full(TK, H)
    assert lib.smoe_down_projection_forward(y1.data_ptr(), w2.data_ptr(), y2.data_ptr(), off, H, I, E, TK,
                                            st.data_ptr(), stream) == 0
    o = full(T, H)
    assert lib.smoe_gather_sum(y2.data_ptr(), o.data_ptr(), scores_flat.data_ptr(), _lib.dtype_code(scores_flat.dtype),
                               rev, tok_off, T, H, fixed_k, stream) == 0
    dz, y1s = full(TK, 2 * I), full(TK, I)
    ncols = lib.smoe_ds_partial_columns(I)
    dsp = full(ncols, TK, dtype=torch.float32)
    assert lib.smoe_down_projection_backward_act(
        dout.data_ptr(), w2.data_ptr(), z.data_ptr(), scores_flat.data_ptr(),
        int(scores_flat.dtype == torch.bfloat16), dz.data_ptr(), y1s.data_ptr(), dsp.data_ptr(), off, gat, sct,
        T, H, I, E, TK, st.data_ptr(), stream) == 0
    ds = full(TK, dtype=torch.float32)
    assert lib.smoe_ds_reduce(dsp.data_ptr(), sct, ds.data_ptr(), _lib.SMOE_F32, TK, ncols, stream) == 0
    dw2 = full(E, H, I)
    assert lib.smoe_down_projection_weight_grad(dout.data_ptr(), y1s.data_ptr(), dw2.data_ptr(), off, gat,
                                                T, H, I, E, TK, st.data_ptr(), stream) == 0
    dw1 = full(E, 2 * I, H)
    assert lib.smoe_up_projection_weight_grad(x.data_ptr(), dz.data_ptr(), dw1.data_ptr(), off, gat,
                                              T, H, I, E, TK, st.data_ptr(), stream) == 0
    dxe = full(TK, H)
    assert lib.smoe_up_projection_backward_dx(dz.data_ptr(), w1.data_ptr(), dxe.data_ptr(), off, H, I, E, TK,
                                              st.data_ptr(), stream) == 0
    dx = full(T, H)
    assert lib.smoe_gather_sum(dxe.data_ptr(), dx.data_ptr(), None, 0, rev, tok_off, T, H, fixed_k, stream) == 0
    torch.cuda.synchronize()
    assert st.item() == 0
    out.update(z=z, y1=y1, y2=y2, o=o, dz=dz, y1s=y1s, ds=ds, dw1=dw1, dw2=dw2, dx_exp=dxe, dx=dx)
    return out


def compare_chain(got, inp, scores_cpu, route_cpu):
    f32 = {k: v.float().cpu() for k, v in inp.items()}
    fwd = orc.experts_forward(f32["x"], f32["w1"], f32["w2"], scores_cpu.float(), route_cpu)
    bwd = orc.experts_backward(f32["x"], f32["w1"], f32["w2"], scores_cpu.float(), route_cpu, fwd, f32["dout"])
    want = dict(z=fwd["z"], y1=fwd["y1"], y2=fwd["y2"], o=fwd["o"], dz=bwd["dz"], y1s=bwd["y1s"], ds=bwd["ds"],
                dw1=bwd["dw1"], dw2=bwd["dw2"], dx_exp=bwd["dx_exp"], dx=bwd["dx"])
    errs = {k: rel(got[k], want[k]) for k in want}
    assert all(e < TOL for e in errs.values()), errs
    return errs


def check_route(route_dev, route_cpu):
    for name in ("expert_frequency", "expert_frequency_offset", "x_gather_idx", "s_scatter_idx",
                 "s_reverse_scatter_idx"):
        assert torch.equal(getattr(route_dev, name).cpu(), getattr(route_cpu, name)), name


TOPK_CASES = [
    # T, H, I, E, K, zipf bias
    pytest.param(2048, 4096, 1024, 128, 8, False, id="config2_T2048_H4096_I1024_E128_K8"),
    pytest.param(4096, 2048, 768, 64, 4, True, id="config5_T4096_H2048_I768_E64_K4_zipf"),
    pytest.param(1024, 7168, 2048, 32, 8, False, id="config4_rank_shape_T1024_H7168_I2048_E32_K8"),
]


@pytest.mark.parametrize("T,H,I,E,K,zipf", TOPK_CASES)
def test_topk_layer_chain_at_benchmark_dimensions(built_library, T, H, I, E, K, zipf):
    from sonicmoe import _lib, functional as fn

    inp = draw(T, H, I, E, seed=H + E)
    logits = torch.nn.functional.linear(inp["x"], inp["router_w"])
    if zipf:
        g = torch.Generator().manual_seed(E)
        ranks = torch.randperm(E, generator=g) + 1
        # a quarter of the benchmark's 2*log(1/rank): skewed (hot experts several times the mean) without every
        # token choosing the same K experts
        logits = logits + (0.5 * torch.log(1.0 / ranks.float())).to(logits.dtype).cuda()
    scores, idx = fn.topk_softmax(logits, K)
    route = fn._route_metadata(idx.reshape(-1), None, E, K)
    s_ref, i_ref = orc.topk_softmax(logits.float().cpu(), K)
    assert torch.equal(idx.cpu(), i_ref)
    assert rel(scores, s_ref) < 1e-5
    r_ref = orc.route_metadata(i_ref, E, T, K=K)
    check_route(route, r_ref)
    if zipf:
        load = r_ref.expert_frequency.float()
        assert load.max() / load.mean() > 3.0
    got = device_chain(_lib, inp, scores.reshape(-1).contiguous(), route, T, H, I, E, K)
    compare_chain(got, inp, s_ref, r_ref)


def test_token_rounding_chain_at_benchmark_dimensions(built_library):
    """Config 3: E 256, K 8, every expert's count rounded to the nearest multiple of 128, pairs through the
    general-routing metadata (variable number of experts per token, bf16 scores)."""
    from sonicmoe import _lib, functional as fn

    T, H, I, E, K = 2048, 4096, 1024, 256, 8
    inp = draw(T, H, I, E, seed=3)
    scores, tokens, experts = fn.forward_token_choice_rounding(inp["x"], inp["router_w"], E, K, 128, "nr")
    logits = torch.nn.functional.linear(inp["x"], inp["router_w"])
    s_ref, t_ref, e_ref, _ = orc.token_rounding_route(logits.float().cpu(), K, "nr", torch.bfloat16)
    assert torch.equal(tokens.cpu(), t_ref) and torch.equal(experts.cpu(), e_ref)
    assert torch.equal(scores.cpu(), s_ref)
    route = fn._route_metadata(experts, tokens, E, 0)
    route.token_offset = fn._sorted_offsets(tokens, T)
    r_ref = orc.route_metadata(e_ref, E, T, token_idx=t_ref)
    check_route(route, r_ref)
    assert torch.equal(route.token_offset.cpu(), r_ref.token_offset)
    assert (r_ref.expert_frequency % 128 == 0).all()
    got = device_chain(_lib, inp, scores.contiguous(), route, T, H, I, E, 0)
    compare_chain(got, inp, s_ref, r_ref)


def test_empty_batch_returns_zero_gradients(built_library):
    """T = 0: every entry point accepts it; the module returns an empty output and zero weight gradients."""
    import sonicmoe
    from sonicmoe import _lib
    from sonicmoe.enums import ActivationType

    E, K, H, I = 8, 2, 256, 128
    m = sonicmoe.MoE(E, K, H, I, ActivationType.SWIGLU, False, 0.02).cuda().to(torch.bfloat16)
    x = torch.zeros(0, H, dtype=torch.bfloat16, device="cuda", requires_grad=True)
    for p in m.parameters():
        p.grad = torch.full_like(p, float("nan"))
        p.grad = None
    o, _aux = m(x)
    assert o.shape == (0, H)
    o.backward(torch.zeros_like(o))
    torch.cuda.synchronize()
    _lib.check_status()
    assert x.grad.shape == (0, H)
    assert (m.c_fc.weight.grad == 0).all() and (m.c_proj.weight.grad == 0).all()
    lib = _lib.lib
    st = _lib.device_state(torch.device("cuda", 0)).status.data_ptr()
    off = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
    d = torch.empty(16, dtype=torch.bfloat16, device="cuda").data_ptr()
    assert lib.smoe_up_projection_forward(d, d, d, d, off.data_ptr(), d, 0, H, I, E, 0, st, None) == 0
    assert lib.smoe_down_projection_backward_act(d, d, d, d, 0, d, d, d, off.data_ptr(), d, d, 0, H, I, E, 0, st,
                                                 None) == 0
    assert lib.smoe_up_projection_forward(d, d, d, d, off.data_ptr(), d, 0, H, I, E, 5, st, None) != 0  # rows, no tokens
