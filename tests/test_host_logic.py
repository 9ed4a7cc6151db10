"""Host-side logic that needs no GPU: module surface, state-dict layout, eager backend vs oracle, errors."""

import numpy as np
import pytest
import torch

from oracle import moe_oracle as orc


def _module(E=8, K=2, H=128, I=64, seed=0):
    import sonicmoe
    from sonicmoe.enums import ActivationType

    inp = orc.make_inputs(96, H, I, E, K, seed=seed)
    m = sonicmoe.MoE(E, K, H, I, ActivationType.SWIGLU, False, 0.02)
    with torch.no_grad():
        m.router.weight.copy_(inp["router_w"])
        m.c_fc.weight.copy_(inp["w1"])
        m.c_proj.weight.copy_(inp["w2"])
    return m, inp


def test_public_surface(built_library):
    import sonicmoe
    from sonicmoe import KernelBackendMoE, MoE, count_cumsum, enable_quack_gemm, moe_TC_softmax_topk_layer  # noqa: F401
    from sonicmoe.enums import ActivationType, is_glu
    from sonicmoe.functional import count_cumsum as cc2, moe_general_routing_inputs  # noqa: F401

    assert KernelBackendMoE("sonicmoe") is KernelBackendMoE.sonicmoe
    assert ActivationType("swiglu") is ActivationType.SWIGLU
    assert is_glu(ActivationType.GEGLU) and not is_glu(ActivationType.RELU_SQ)
    with enable_quack_gemm(True):
        pass


def test_state_dict_layout(built_library):
    m, _ = _module()
    sd = m.state_dict()
    assert set(sd) == {"router.weight", "c_fc.weight", "c_proj.weight"}
    assert sd["router.weight"].shape == (8, 128)
    assert sd["c_fc.weight"].shape == (8, 128, 128)   # (E, 2I, H)
    assert sd["c_proj.weight"].shape == (8, 128, 64)  # (E, H, I)
    import sonicmoe
    from sonicmoe.enums import ActivationType

    mb = sonicmoe.MoE(4, 2, 64, 64, ActivationType.GELU, True, 0.02)
    assert mb.c_fc.weight.shape == (4, 64, 64) and mb.c_fc.bias.shape == (4, 64) and mb.c_proj.bias.shape == (4, 64)


def test_eager_backend_matches_oracle(built_library):
    from sonicmoe import KernelBackendMoE

    m, inp = _module()
    x = inp["x"].clone().requires_grad_(True)
    o, aux = m(x.view(2, 48, 128), kernel_backend_moe=KernelBackendMoE.torch)
    assert o.shape == (2, 48, 128)
    grads = torch.autograd.grad(o, [x, m.router.weight, m.c_fc.weight, m.c_proj.weight], inp["dout"].view(2, 48, 128))
    ref = orc.moe_layer(inp["x"], inp["router_w"], inp["w1"], inp["w2"], 2, dout=inp["dout"])
    for got, want in zip((o.reshape(96, 128), aux, *grads),
                         (ref["o"], ref["aux_loss"], ref["dx"], ref["drouter_w"], ref["dw1"], ref["dw2"])):
        assert (got.detach() - want).norm() <= 2e-5 * want.norm()


def test_cuda_backend_refuses_cpu_and_unsupported_inputs(built_library):
    from sonicmoe import _lib
    from sonicmoe.functional import moe_TC_softmax_topk_layer

    m, inp = _module()
    with pytest.raises(_lib.SonicMoEError):
        m(inp["x"])  # CPU tensor: no fallback
    w1 = m.c_fc.weight.permute(1, 2, 0)
    w2 = m.c_proj.weight.permute(1, 2, 0)
    with pytest.raises(AssertionError):
        moe_TC_softmax_topk_layer(inp["x"], m.router.weight, w1, torch.zeros(8, 128), w2, None, 2)
    with pytest.raises(ValueError):
        moe_TC_softmax_topk_layer(inp["x"], m.router.weight, w1, None, w2, None, 2, 0, "not-an-activation")
    with pytest.raises(_lib.SonicMoEError):  # a supported activation still has no CPU path
        moe_TC_softmax_topk_layer(inp["x"], m.router.weight, w1, None, w2, None, 2, 0, "gelu")
    with pytest.raises(ValueError):
        m(inp["x"], kernel_backend_moe=__import__("sonicmoe").KernelBackendMoE.scattermoe)


def test_rounded_counts():
    from sonicmoe.functional.token_rounding import rounded_counts

    f = torch.tensor([0, 1, 63, 64, 65, 127, 128, 191, 192, 193, 320, 448])
    assert rounded_counts(f, "down").tolist() == [0, 0, 0, 0, 0, 0, 128, 128, 128, 128, 256, 384]
    assert rounded_counts(f, "up").tolist() == [0, 128, 128, 128, 128, 128, 128, 256, 256, 256, 384, 512]
    # nearest, exact halves go to the even multiple (64 -> 0, 192 -> 256, 320 -> 256, 448 -> 512)
    assert rounded_counts(f, "nr").tolist() == [0, 0, 0, 0, 128, 128, 128, 128, 256, 256, 256, 512]
    assert torch.equal(rounded_counts(f, "nr"), orc.rounded_counts(f, "nr"))


def test_token_rounding_router_has_no_cpu_path():
    """The selection runs in the library's CUDA kernels only: CPU tensors are refused, unknown modes too."""
    from sonicmoe import _lib
    from sonicmoe.functional.token_rounding import forward_token_choice_rounding, select_pairs

    inp = orc.make_inputs(512, 64, 64, 8, 2, seed=11, dtype=torch.float32)
    with pytest.raises(_lib.SonicMoEError):
        forward_token_choice_rounding(inp["x"], inp["router_w"], 8, 2, 128, "nr")
    with pytest.raises(NotImplementedError):
        select_pairs(torch.zeros(4, 8), torch.zeros(4, 2, dtype=torch.int32), "sideways")


@pytest.mark.parametrize("name", ["state_dict_swiglu", "state_dict_gelu_bias"])
def test_reference_state_dict_loads_and_reproduces_reference_output(built_library, name):
    """Checkpoint interchange: the state dict of a module the reference constructed and initialised loads with
    strict=True into this build's `MoE`, and the eager backend then reproduces the reference's output, aux loss and
    every gradient (fixtures: tests/golden/make_golden.py, reference sonicmoe/moe.py:58-68, 186-204)."""
    import sonicmoe
    from conftest import golden
    from sonicmoe import KernelBackendMoE
    from sonicmoe.enums import ActivationType

    g = golden(name)
    T, H, I, E, K, _seed, add_bias = [int(v) for v in g["meta"]]
    state = {k[len("param."):]: torch.from_numpy(g[k]) for k in g.files if k.startswith("param.")}
    m = sonicmoe.MoE(E, K, H, I, ActivationType(str(g["activation"])), bool(add_bias), 0.02)
    missing = m.load_state_dict(state, strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    x = torch.from_numpy(g["x"]).requires_grad_(True)
    o, aux = m(x, kernel_backend_moe=KernelBackendMoE.torch)
    names = [n for n, _ in m.named_parameters()]
    grads = torch.autograd.grad(o, [x] + list(m.parameters()), torch.from_numpy(g["dout"]))

    def close(a, b):
        b = torch.from_numpy(np.asarray(b))
        assert (a.detach() - b).norm() <= 2e-5 * b.norm() + 1e-12

    close(o, g["o"])
    close(aux, g["aux_loss"])
    close(grads[0], g["dx"])
    for n, got in zip(names, grads[1:]):
        close(got, g[f"grad.{n}"])


def test_fp8_layer_refuses_biases_and_other_activations(built_library):
    """The FP8 experts are bias-free SwiGLU: other configurations are refused, not silently mis-computed."""
    from sonicmoe.functional.fp8 import moe_fp8_softmax_topk_layer

    m, inp = _module()
    w1 = m.c_fc.weight.permute(1, 2, 0)
    w2 = m.c_proj.weight.permute(1, 2, 0)
    b1, b2 = torch.zeros(8, 128), torch.zeros(8, 128)
    with pytest.raises(NotImplementedError):
        moe_fp8_softmax_topk_layer(inp["x"], m.router.weight, w1, b1, w2, b2, 2)
    with pytest.raises(NotImplementedError):
        moe_fp8_softmax_topk_layer(inp["x"], m.router.weight, w1, None, w2, None, 2, 0, "geglu")


def test_weight_grad_sum_bookkeeping():
    """`WeightGradSum`: the first chunk gets fresh buffers and stores, later chunks get the same buffers and add, only
    the last chunk hands the gradients on, and the object is empty again afterwards."""
    import torch

    from sonicmoe.functional import WeightGradSum

    w1, w2 = torch.zeros(2, 4, 3), torch.zeros(2, 3, 2)
    shared = WeightGradSum(3)
    d1, d2, add = shared.buffers(w1, w2)
    assert not add and d1.shape == w1.shape and d2.shape == w2.shape
    assert shared.finish_chunk() == (None, None)
    e1, e2, add = shared.buffers(w1, w2)
    assert add and e1 is d1 and e2 is d2
    assert shared.finish_chunk() == (None, None)
    f1, f2, add = shared.buffers(w1, w2)
    assert add and f1 is d1
    out1, out2 = shared.finish_chunk()
    assert out1 is d1 and out2 is d2
    assert shared.dw1 is None and shared.dw2 is None and shared.remaining == 0
