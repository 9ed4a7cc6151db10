"""Whole-layer parity on the GPU: the `sonicmoe.MoE` module and the functional entry points against the
CPU oracle and against the golden fixtures produced by the reference.

Tolerance: relative Frobenius error <= 1e-2 for every bf16 output and gradient (the bound stated for the
bf16 layer); routing (indices, expert frequencies) bit-exact on the same logits.
"""

import pytest
import torch

from conftest import golden
from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-2


def rel(a, b):
    a = a.detach().float().cpu()
    b = torch.as_tensor(b).detach().float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


def _module(T, H, I, E, K, seed, **kw):
    import sonicmoe
    from sonicmoe.enums import ActivationType

    inp = orc.make_inputs(T, H, I, E, K, seed=seed, dtype=torch.bfloat16, **kw)
    m = sonicmoe.MoE(E, K, H, I, ActivationType.SWIGLU, False, 0.02).cuda().to(torch.bfloat16)
    with torch.no_grad():
        m.router.weight.copy_(inp["router_w"])
        m.c_fc.weight.copy_(inp["w1"])
        m.c_proj.weight.copy_(inp["w2"])
    return m, inp


# reference test matrix shapes (tests/moe_test.py:25-38) scaled to sizes the CPU oracle finishes in seconds,
# plus ragged / tiny / single-expert-per-token cases
LAYER_SHAPES = [
    (512, 256, 128, 16, 4),
    (1024, 768, 256, 8, 2),
    (777, 768, 320, 32, 8),
    (640, 1536, 256, 64, 16),
    (64, 128, 64, 4, 1),
    (2048, 768, 256, 128, 8),
    (30, 256, 64, 256, 8),   # far fewer tokens than experts: most experts are empty
]


@pytest.mark.parametrize("T,H,I,E,K", LAYER_SHAPES)
@pytest.mark.parametrize("fused_combine", [False, True])
def test_module_forward_backward_vs_oracle(built_library, T, H, I, E, K, fused_combine):
    from sonicmoe import _lib, functional

    m, inp = _module(T, H, I, E, K, seed=T + E)
    prev = functional.set_fused_combine(fused_combine)
    try:
        x = inp["x"].cuda().requires_grad_(True)
        o, aux = m(x.view(1, T, H))
        assert o.shape == (1, T, H) and o.dtype == torch.bfloat16
        grads = torch.autograd.grad(o, [x, m.router.weight, m.c_fc.weight, m.c_proj.weight],
                                    inp["dout"].cuda().view(1, T, H))
    finally:
        functional.set_fused_combine(prev)
    torch.cuda.synchronize()
    _lib.check_status()

    logits = functional.layer_router_logits(x.detach(), m.router.weight.detach(), K)
    f32 = {k: v.float() for k, v in inp.items()}
    ref = orc.moe_layer(f32["x"], f32["router_w"], f32["w1"], f32["w2"], K, dout=f32["dout"],
                        logits=logits.float().cpu())
    # routing on the same logits tensor is bit-exact
    scores, idx = functional.topk_softmax(logits, K)
    assert torch.equal(idx.cpu(), ref["indices"])
    assert rel(o.view(T, H), ref["o"]) < TOL
    assert rel(aux, ref["aux_loss"]) < 1e-3
    # dx = expert path + router path; the router path is torch autograd on bf16 logits
    assert rel(grads[0], ref["dx"]) < TOL
    assert rel(grads[1], ref["drouter_w"]) < 2e-2  # dlogits are rounded to bf16 before the router GEMM
    assert rel(grads[2], ref["dw1"]) < TOL
    assert rel(grads[3], ref["dw2"]) < TOL
    assert grads[2].shape == m.c_fc.weight.shape and grads[3].shape == m.c_proj.weight.shape


@pytest.mark.parametrize("name", ["layer_small", "layer_ties", "layer_k1"])
def test_functional_layer_vs_reference_golden(built_library, name):
    """The device path against outputs of the reference's own eager layer (fp32 router, bf16 experts)."""
    from sonicmoe import _lib
    from sonicmoe.functional import moe_TC_softmax_topk_layer

    g = golden(name)
    T, H, I, E, K, seed, _ = [int(v) for v in g["meta"]]
    inp = orc.make_inputs(T, H, I, E, K, seed=seed, dtype=torch.bfloat16)
    x = inp["x"].cuda().requires_grad_(True)
    rw = inp["router_w"].float().cuda().requires_grad_(True)  # fp32 router: same logits as the reference run
    w1 = inp["w1"].cuda().requires_grad_(True)
    w2 = inp["w2"].cuda().requires_grad_(True)
    o, logits, freq = moe_TC_softmax_topk_layer(x, rw, w1.permute(1, 2, 0), None, w2.permute(1, 2, 0), None, K)
    grads = torch.autograd.grad(o, [x, rw, w1, w2], inp["dout"].cuda())
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(freq.cpu(), torch.from_numpy(g["expert_frequency"]))
    assert rel(logits, g["logits"]) < 1e-5
    assert rel(o, g["o"]) < TOL
    for got, key in zip(grads, ("dx", "drouter_w", "dw1", "dw2")):
        assert rel(got, g[key]) < TOL, key


def test_inference_mode_matches_training_forward(built_library):
    m, inp = _module(512, 256, 128, 16, 4, seed=3)
    x = inp["x"].cuda()
    o_train, _ = m(x)
    m.eval()
    with torch.no_grad():
        o_eval, _ = m(x)
    o_flag, _ = m.train()(x, is_inference_mode=True)
    assert torch.equal(o_train, o_eval) and torch.equal(o_train, o_flag)


@pytest.mark.parametrize("routing", ["nr", "up", "down"])
@pytest.mark.parametrize("T,H,I,E,K", [(1024, 256, 128, 8, 2), (2048, 512, 128, 16, 4)])
def test_token_rounding_layer_vs_oracle(built_library, routing, T, H, I, E, K):
    """Token-rounding router + general-routing layer: selections bit-exact, outputs and gradients in tolerance."""
    from sonicmoe import _lib
    from sonicmoe.functional import forward_token_choice_rounding, moe_general_routing_inputs

    inp = orc.make_inputs(T, H, I, E, K, seed=T + E + len(routing), dtype=torch.bfloat16)
    x = inp["x"].cuda().requires_grad_(True)
    w1 = inp["w1"].cuda().requires_grad_(True)
    w2 = inp["w2"].cuda().requires_grad_(True)
    scores, tokens, experts = forward_token_choice_rounding(x.detach(), inp["router_w"].cuda(), E, K, 128, routing)
    logits = torch.nn.functional.linear(x.detach(), inp["router_w"].cuda())
    s_ref, t_ref, e_ref, _ = orc.token_rounding_route(logits.cpu(), K, routing, torch.bfloat16)
    assert torch.equal(tokens.cpu(), t_ref) and torch.equal(experts.cpu(), e_ref)
    assert torch.equal(scores.cpu(), s_ref)
    counts = torch.bincount(experts.long(), minlength=E)
    assert (counts % 128 == 0).all()

    sc = scores.detach().clone().requires_grad_(True)
    o, freq = moe_general_routing_inputs(x, sc, tokens, experts, w1.permute(1, 2, 0), None, w2.permute(1, 2, 0),
                                         None, E, 0, __import__("sonicmoe").ActivationType.SWIGLU)
    grads = torch.autograd.grad(o, [x, w1, w2, sc], inp["dout"].cuda())
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(freq.cpu(), counts.cpu().int())
    f32 = {k: v.float() for k, v in inp.items()}
    ref = orc.general_routing_layer(f32["x"], f32["w1"], f32["w2"], s_ref.float(), t_ref, e_ref, dout=f32["dout"])
    assert rel(o, ref["o"]) < TOL
    assert rel(grads[0], ref["dx"]) < TOL
    assert rel(grads[1], ref["dw1"]) < TOL
    assert rel(grads[2], ref["dw2"]) < TOL
    assert grads[3].dtype == torch.bfloat16 and rel(grads[3], ref["ds"]) < TOL


def test_general_routing_with_empty_tokens_and_experts(built_library):
    from sonicmoe import ActivationType, _lib
    from sonicmoe.functional import moe_general_routing_inputs

    T, H, I, E = 200, 128, 64, 8
    inp = orc.make_inputs(T, H, I, E, 2, seed=5, dtype=torch.bfloat16, w_std=0.05)
    g = torch.Generator().manual_seed(1)
    n = 300
    tokens = torch.randint(0, T // 2, (n,), generator=g).sort().values.int()  # upper half of the tokens unused
    experts = torch.randint(0, E - 2, (n,), generator=g).int()                # two experts unused
    scores = torch.rand(n, generator=g)
    x = inp["x"].cuda().requires_grad_(True)
    w1 = inp["w1"].cuda().requires_grad_(True)
    w2 = inp["w2"].cuda().requires_grad_(True)
    sc = scores.cuda().requires_grad_(True)
    o, freq = moe_general_routing_inputs(x, sc, tokens.cuda(), experts.cuda(), w1.permute(1, 2, 0), None,
                                         w2.permute(1, 2, 0), None, E, 0, ActivationType.SWIGLU)
    grads = torch.autograd.grad(o, [x, w1, w2, sc], inp["dout"].cuda())
    torch.cuda.synchronize()
    _lib.check_status()
    f32 = {k: v.float() for k, v in inp.items()}
    ref = orc.general_routing_layer(f32["x"], f32["w1"], f32["w2"], scores, tokens, experts, dout=f32["dout"])
    assert (o[T // 2:] == 0).all() and (grads[0][T // 2:] == 0).all()
    assert (grads[1][E - 2:] == 0).all() and (grads[2][E - 2:] == 0).all()
    assert rel(o, ref["o"]) < TOL and rel(grads[0], ref["dx"]) < TOL
    assert rel(grads[1], ref["dw1"]) < TOL and rel(grads[2], ref["dw2"]) < TOL
    assert grads[3].dtype == torch.float32 and rel(grads[3], ref["ds"]) < 1e-2


def test_linearity_at_full_hidden_size(built_library):
    """Size-independent property at the benchmark's H and I: with the routing fixed, the layer output is linear in
    the routing scores, o(a*s1 + b*s2) = a*o(s1) + b*o(s2), and doubling dout doubles every gradient."""
    from sonicmoe import ActivationType, _lib
    from sonicmoe.functional import moe_general_routing_inputs

    T, H, I, E, K = 4096, 4096, 1024, 16, 2
    inp = orc.make_inputs(T, H, I, E, K, seed=1, dtype=torch.bfloat16)
    g = torch.Generator().manual_seed(2)
    experts = torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(T)]).reshape(-1).int().cuda()
    tokens = torch.arange(T).repeat_interleave(K).int().cuda()
    s1 = torch.rand(T * K, generator=g).cuda()
    s2 = torch.rand(T * K, generator=g).cuda()
    x = inp["x"].cuda()
    w1 = inp["w1"].cuda().permute(1, 2, 0)
    w2 = inp["w2"].cuda().permute(1, 2, 0)

    def run(s):
        with torch.no_grad():
            return moe_general_routing_inputs(x, s, tokens, experts, w1, None, w2, None, E, 0,
                                              ActivationType.SWIGLU)[0].float()

    o1, o2, o12 = run(s1), run(s2), run(0.5 * s1 + 2.0 * s2)
    assert ((o12 - (0.5 * o1 + 2.0 * o2)).norm() / o12.norm()).item() < TOL
    torch.cuda.synchronize()
    _lib.check_status()


def test_torch_compile_fullgraph_matches_eager(built_library):
    """`torch.compile(fullgraph=True)` of the module (the reference compiles it in its tests and benchmarks,
    tests/moe_test.py:80-81): same output and gradients as the eager module."""
    from sonicmoe import _lib

    T, H, I, E, K = 512, 256, 128, 16, 4
    m, inp = _module(T, H, I, E, K, seed=9)
    x = inp["x"].cuda().requires_grad_(True)
    dout = inp["dout"].cuda()
    o_ref, aux_ref = m(x)
    g_ref = torch.autograd.grad(o_ref, [x, m.router.weight, m.c_fc.weight, m.c_proj.weight], dout)
    compiled = torch.compile(m, fullgraph=True)
    o, aux = compiled(x)
    g = torch.autograd.grad(o, [x, m.router.weight, m.c_fc.weight, m.c_proj.weight], dout)
    torch.cuda.synchronize()
    _lib.check_status()
    assert torch.equal(o, o_ref)
    assert rel(aux, aux_ref) < 1e-5
    for a, b in zip(g, g_ref):
        assert a.shape == b.shape and rel(a, b) < 1e-3


@pytest.mark.parametrize("act,bias", [("swiglu", True), ("geglu", False), ("reglu", True), ("gelu", True),
                                      ("relu", False), ("silu", True), ("relu_sq", False)])
def test_bias_and_activations_vs_oracle(built_library, act, bias):
    """Every activation of the layer, with and without expert biases (the reference test matrix has
    add_bias, tests/moe_test.py:25-56; activations are a benchmark flag, benchmarks/moe-cute.py:62-94)."""
    import sonicmoe
    from sonicmoe import _lib
    from sonicmoe.enums import ActivationType, is_glu

    T, H, I, E, K = 700, 256, 128, 8, 2
    kind = ActivationType(act)
    n1 = 2 * I if is_glu(kind) else I
    g = torch.Generator().manual_seed(len(act) + bias)
    m = sonicmoe.MoE(E, K, H, I, kind, bias, 0.05).cuda().to(torch.bfloat16)
    with torch.no_grad():
        m.router.weight.copy_(torch.randn(E, H, generator=g) * 0.05)
        if bias:
            m.c_fc.bias.copy_(torch.randn(E, n1, generator=g) * 0.1)
            m.c_proj.bias.copy_(torch.randn(E, H, generator=g) * 0.1)
    x = torch.randn(T, H, generator=g).bfloat16().cuda().requires_grad_(True)
    dout = torch.randn(T, H, generator=g).bfloat16().cuda()
    o, _aux = m(x)
    params = [m.c_fc.weight, m.c_proj.weight] + ([m.c_fc.bias, m.c_proj.bias] if bias else [])
    grads = torch.autograd.grad(o, [x] + params, dout)
    torch.cuda.synchronize()
    _lib.check_status()

    from sonicmoe.functional import layer_router_logits

    logits = layer_router_logits(x.detach(), m.router.weight.detach(), K).float().cpu()
    scores, idx = orc.topk_softmax(logits, K)
    route = orc.route_metadata(idx, E, T, K=K)
    f = lambda t: None if t is None else t.detach().float().cpu()
    ref = orc.experts_autograd(f(x), f(m.c_fc.weight), f(m.c_fc.bias), f(m.c_proj.weight), f(m.c_proj.bias),
                               scores.reshape(-1), route, act, f(dout))
    dlogits = orc.softmax_topk_backward(scores, idx, ref["ds"].reshape(T, K), E)
    dx_ref = ref["dx"] + dlogits @ f(m.router.weight)
    assert rel(o, ref["o"]) < TOL
    assert rel(grads[0], dx_ref) < TOL
    assert rel(grads[1], ref["dw1"]) < TOL
    assert rel(grads[2], ref["dw2"]) < TOL
    if bias:
        assert rel(grads[3], ref["db1"]) < TOL
        assert rel(grads[4], ref["db2"]) < TOL


def test_second_device_in_one_process(built_library):
    """Kernel attributes (dynamic shared memory) and the SM count are cached per device, not per process: a layer on
    cuda:1 of a process that already ran one on cuda:0 launches and gives the same result."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from sonicmoe import _lib

    T, H, I, E, K = 512, 256, 128, 16, 4
    outs = []
    for d in (0, 1):
        m, inp = _module(T, H, I, E, K, seed=3)
        m = m.to(f"cuda:{d}")
        x = inp["x"].to(f"cuda:{d}").requires_grad_(True)
        o, _ = m(x)
        o.backward(inp["dout"].to(f"cuda:{d}"))
        torch.cuda.synchronize(d)
        _lib.check_status(torch.device("cuda", d))
        outs.append((o.detach().cpu(), x.grad.cpu(), m.c_fc.weight.grad.cpu()))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


@pytest.mark.parametrize("kind", ["bf16", "fp8"])
def test_chunks_share_weight_gradient_buffers(built_library, kind):
    """A batch processed as three chunks that share a `WeightGradSum`: the last chunk's backward pass hands autograd
    the sum of the chunks' weight gradients (accumulated in the GEMM epilogues), the others hand it nothing; the
    parameters' gradients match the whole batch's within bf16 accumulation error, and the two-chunk case equals
    autograd's own accumulation of per-chunk gradients bit for bit.  The `on_dx` hook sees each chunk's dx before
    the chunk's weight gradients are launched.  Same contract for the FP8 local experts."""
    from sonicmoe import _lib, functional as fn
    from sonicmoe.functional.fp8 import _RoutedExpertsFp8

    T, H, I, E, K = 1536, 512, 256, 8, 2
    g = torch.Generator(device="cuda").manual_seed(11)

    def rn(*shape, std):
        return (torch.randn(*shape, generator=g, device="cuda") * std).bfloat16()

    x0, dout = rn(T, H, std=1.0), rn(T, H, std=1.0)
    w1, w2 = rn(E, 2 * I, H, std=0.05).requires_grad_(True), rn(E, H, I, std=0.05).requires_grad_(True)
    logits = rn(T, E, std=1.0)
    scores, idx = fn.topk_softmax(logits, K)

    def run(bounds, share):
        w1.grad = w2.grad = None
        x = x0.clone().requires_grad_(True)
        shared = fn.WeightGradSum(len(bounds) - 1) if share else None
        outs, announced = [], []
        for a, b in zip(bounds[:-1], bounds[1:]):
            route = fn._route_metadata(idx[a:b].reshape(-1), None, E, K)
            route.wgrad_sum = shared
            route.on_dx = lambda dx, a=a, b=b: announced.append((a, b, dx.clone()))
            args = (x[a:b], w1.permute(1, 2, 0), w2.permute(1, 2, 0), scores[a:b].reshape(-1), route, b - a, False)
            outs.append(_RoutedExpertsFp8.apply(*args, "ue8m0") if kind == "fp8" else fn._RoutedExperts.apply(*args))
        torch.cat(outs).backward(dout)
        torch.cuda.synchronize()
        _lib.check_status()
        assert len(announced) == len(bounds) - 1
        for a, b, dx in announced:
            assert torch.equal(dx, x.grad[a:b])
        return w1.grad.clone(), w2.grad.clone()

    whole = run([0, T], False)
    tol = 1e-2  # FP8 too: activations are quantised row by row, so cutting the batch changes no quantised value
    for bounds in ([0, 700, T], [0, 100, 100, T]):  # uneven chunks; an empty one
        separate, shared = run(bounds, False), run(bounds, True)
        for a, b, c in zip(shared, separate, whole):
            assert rel(a, c) < tol and rel(b, c) < tol
            if len(bounds) == 3:
                assert torch.equal(a, b)
