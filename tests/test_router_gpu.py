"""The fused routing front end (router GEMM + top-K + softmax + token counts + softmax column sums in one kernel)
and its backward kernel, through the C ABI.

The routing decision is checked bit for bit on the logits the kernel itself writes (bf16): indices must equal a stable
descending sort of that output, counts must equal a bincount of the indices.  Floating-point outputs: logits against
the fp32 product within bf16 rounding, scores 1e-5, column sums 1e-4 (they use the fast exponential), gradients 1e-2.
Reference: sonicmoe/functional/__init__.py:438-446 (router linear + top-k), sonicmoe/moe.py:251-274 (aux loss)."""

import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

SHAPES = [
    # T, H, E, K
    (1000, 512, 64, 4),      # ragged last tile
    (4096, 4096, 128, 8),    # the benchmark layer's router
    (300, 768, 256, 8),      # widest accumulator, 4 stages
    (129, 256, 32, 2),       # one row in the second tile
    (512, 1024, 128, 16),    # the 16-entry winner list
    (20000, 2048, 64, 4),    # more tiles than SMs: several tiles per CTA, both accumulators in flight
]


def rel(a, b):
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


def _run(T, H, E, K, seed=0):
    from sonicmoe import _lib

    lib = _lib.lib
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cuda").manual_seed(seed + T)
    x = torch.randn(T, H, generator=g, device=dev).bfloat16()
    w = (torch.randn(E, H, generator=g, device=dev) * 0.05).bfloat16()
    nan = float("nan")
    logits = torch.full((T, E), nan, dtype=torch.bfloat16, device=dev)
    scores = torch.full((T, K), nan, dtype=torch.float32, device=dev)
    indices = torch.full((T, K), -1, dtype=torch.int32, device=dev)
    count = torch.full((E,), -1, dtype=torch.int32, device=dev)
    colsum = torch.full((E,), nan, dtype=torch.float32, device=dev)
    ws = torch.empty(lib.smoe_router_forward_workspace_bytes(E), dtype=torch.uint8, device=dev)
    st = _lib.device_state(dev).status
    assert lib.smoe_router_forward_supported(H, E, K) == 1
    assert lib.smoe_router_forward(x.data_ptr(), w.data_ptr(), logits.data_ptr(), scores.data_ptr(), indices.data_ptr(),
                                   count.data_ptr(), colsum.data_ptr(), ws.data_ptr(), T, H, E, K, st.data_ptr(),
                                   torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert st.item() == 0
    return x, w, logits, scores, indices, count, colsum


@pytest.mark.parametrize("T,H,E,K", SHAPES)
def test_router_forward(built_library, T, H, E, K):
    x, w, logits, scores, indices, count, colsum = _run(T, H, E, K)
    exact = x.float() @ w.float().T
    assert rel(logits, exact) < 4e-3                      # one bf16 rounding of an fp32-accumulated product
    lib_logits = torch.nn.functional.linear(x, w)         # the library GEMM rounds the same sums: equal up to last-bit flips
    assert (logits.float() - lib_logits.float()).abs().max() <= 2.0 ** -7 * exact.abs().max()
    s_ref, i_ref = orc.topk_softmax(logits.float().cpu(), K)
    assert torch.equal(indices.cpu(), i_ref)
    assert rel(scores, s_ref) < 1e-5
    assert torch.equal(count.cpu(), torch.bincount(i_ref.reshape(-1).long(), minlength=E).int())
    assert count.sum().item() == T * K
    p = torch.softmax(logits.float(), dim=-1).sum(0)
    assert rel(colsum, p) < 1e-4
    # bit-reproducible
    again = _run(T, H, E, K)
    for a, b in zip((logits, scores, indices, count, colsum), again[2:]):
        assert torch.equal(a, b)


def test_router_forward_ties_and_signed_zeros(built_library):
    """Rows full of equal logits: the winners are the lowest columns, in order."""
    from sonicmoe import _lib

    lib = _lib.lib
    T, H, E, K = 256, 128, 64, 8
    dev = torch.device("cuda", 0)
    x = torch.zeros(T, H, dtype=torch.bfloat16, device=dev)
    x[:, 0] = 1.0
    w = torch.zeros(E, H, dtype=torch.bfloat16, device=dev)
    w[1::2, 0] = -0.0          # -0.0 and +0.0 logits are equal
    w[40:44, 0] = 3.0          # four clear winners
    logits = torch.empty(T, E, dtype=torch.bfloat16, device=dev)
    scores = torch.empty(T, K, dtype=torch.float32, device=dev)
    indices = torch.empty(T, K, dtype=torch.int32, device=dev)
    count = torch.empty(E, dtype=torch.int32, device=dev)
    colsum = torch.empty(E, dtype=torch.float32, device=dev)
    ws = torch.empty(lib.smoe_router_forward_workspace_bytes(E), dtype=torch.uint8, device=dev)
    assert lib.smoe_router_forward(x.data_ptr(), w.data_ptr(), logits.data_ptr(), scores.data_ptr(), indices.data_ptr(),
                                   count.data_ptr(), colsum.data_ptr(), ws.data_ptr(), T, H, E, K, None,
                                   torch.cuda.current_stream().cuda_stream) == 0
    assert indices[0].tolist() == [40, 41, 42, 43, 0, 1, 2, 3]
    assert (indices == indices[0]).all()


@pytest.mark.parametrize("T,E,K", [(777, 64, 4), (2048, 128, 8), (100, 256, 16), (513, 32, 1)])
@pytest.mark.parametrize("parts", ["all", "scores", "colsum", "logits"])
def test_router_backward(built_library, T, E, K, parts):
    """dlogits against autograd on an fp32 restatement: softmax over the K winners, column sums of the full softmax,
    plus a direct gradient on the logits."""
    from sonicmoe import _lib

    lib = _lib.lib
    dev = torch.device("cuda", 0)
    g = torch.Generator(device="cuda").manual_seed(T + E)
    logits = torch.randn(T, E, generator=g, device=dev).bfloat16()
    g_scores = torch.randn(T, K, generator=g, device=dev)
    g_colsum = torch.randn(E, generator=g, device=dev)
    g_logits = (torch.randn(T, E, generator=g, device=dev) * 0.1).bfloat16()
    use_s, use_c, use_l = (parts in ("all", "scores")), (parts in ("all", "colsum")), (parts in ("all", "logits"))

    lf = logits.float().requires_grad_(True)
    order = torch.sort(lf.detach(), dim=-1, descending=True, stable=True).indices[:, :K]
    scores = torch.softmax(lf.gather(-1, order), dim=-1)
    loss = lf.sum() * 0.0
    if use_s:
        loss = loss + (scores * g_scores).sum()
    if use_c:
        loss = loss + (torch.softmax(lf, dim=-1).sum(0) * g_colsum).sum()
    if use_l:
        loss = loss + (lf * g_logits.float()).sum()
    (want,) = torch.autograd.grad(loss, lf)

    out = torch.full((T, E), float("nan"), dtype=torch.bfloat16, device=dev)
    idx = order.int().contiguous()
    sc = scores.detach().contiguous()
    assert lib.smoe_router_backward(out.data_ptr(), logits.data_ptr(), g_scores.data_ptr() if use_s else None,
                                    sc.data_ptr(), idx.data_ptr(), g_colsum.data_ptr() if use_c else None,
                                    g_logits.data_ptr() if use_l else None, T, E, K,
                                    torch.cuda.current_stream().cuda_stream) == 0
    assert rel(out, want) < 1e-2
    if parts == "scores":   # only the K winners' columns are non-zero
        assert (out != 0).sum(1).max().item() <= K


def test_layer_with_fused_router_matches_separate_router(built_library):
    """The layer with the one-pass router against the layer with router linear + top-k kernel: same aux loss and
    gradients within tolerance (logits can differ in the last bf16 bit, which may move a near-tie)."""
    import sonicmoe
    from sonicmoe import functional
    from sonicmoe.enums import ActivationType

    T, H, I, E, K = 1024, 512, 256, 64, 4
    inp = orc.make_inputs(T, H, I, E, K, seed=9, dtype=torch.bfloat16)
    m = sonicmoe.MoE(E, K, H, I, ActivationType.SWIGLU, False, 0.02).cuda().to(torch.bfloat16)
    with torch.no_grad():
        m.router.weight.copy_(inp["router_w"])
        m.c_fc.weight.copy_(inp["w1"])
        m.c_proj.weight.copy_(inp["w2"])
    res = {}
    for fused in (True, False):
        prev = functional.set_fused_router(fused)
        try:
            x = inp["x"].cuda().requires_grad_(True)
            o, aux = m(x)
            # the aux loss takes part in the backward pass: its gradient reaches the router through the column sums
            grads = torch.autograd.grad([o, aux], [x, m.router.weight, m.c_fc.weight], [inp["dout"].cuda(),
                                                                                       torch.tensor(3.0, device="cuda")])
            res[fused] = (o, aux, *grads)
        finally:
            functional.set_fused_router(prev)
    assert rel(res[True][1], res[False][1]) < 1e-4
    for a, b in zip(res[True], res[False]):
        assert rel(a, b) < 2e-2
