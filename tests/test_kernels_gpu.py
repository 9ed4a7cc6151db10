"""Parity of every CUDA entry point (called through the C-ABI library) against the CPU oracle.

Integer / index outputs must be bit-exact; floating-point outputs are compared by relative Frobenius
error: 1e-2 for bf16 tensors (the bound stated for this layer), 1e-5 for fp32 routing quantities.
"""

import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

BF16_TOL = 1e-2
F32_TOL = 1e-5


@pytest.fixture(scope="module")
def smoe(built_library):
    assert torch.cuda.is_available()
    import sonicmoe  # noqa: F401
    from sonicmoe import _lib, functional

    yield _lib, functional
    torch.cuda.synchronize()
    _lib.check_status()


def rel(a, b):
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


# ---------------------------------------------------------------------------------------------------
# router
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("T,E,K", [(1, 8, 2), (1000, 8, 2), (4096, 128, 8), (333, 256, 8), (257, 72, 4), (64, 24, 1),
                                   (100, 1920, 16), (40, 4096, 16), (17, 5000, 3), (50, 64, 33)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_topk_softmax_bit_exact_indices(smoe, T, E, K, dtype):
    _, fn = smoe
    g = torch.Generator().manual_seed(T * 131 + E)
    logits = torch.randn(T, E, generator=g).to(dtype)  # bf16 rounding produces plenty of ties
    if T > 2:
        logits[1, :] = 0.5  # a fully tied row
        logits[2, ::2] = -0.0
        logits[2, 1::2] = 0.0
    scores, idx = fn.topk_softmax(logits.cuda(), K)
    s_ref, i_ref = orc.topk_softmax(logits, K)
    assert torch.equal(idx.cpu(), i_ref)
    assert rel(scores, s_ref) < F32_TOL
    assert torch.allclose(scores.sum(-1).cpu(), torch.ones(T), atol=1e-5)


@pytest.mark.parametrize("T,E,K", [(500, 8, 2), (1024, 128, 8), (77, 72, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_softmax_topk_backward(smoe, T, E, K, dtype):
    _, fn = smoe
    g = torch.Generator().manual_seed(5)
    logits = torch.randn(T, E, generator=g).to(dtype)
    dscores = torch.randn(T, K, generator=g)
    lg = logits.cuda().requires_grad_(True)
    scores, idx = fn.topk_softmax(lg, K)
    (dl,) = torch.autograd.grad(scores, lg, dscores.cuda())
    s_ref, i_ref = orc.topk_softmax(logits, K)
    dl_ref = orc.softmax_topk_backward(s_ref, i_ref, dscores, E)
    assert dl.dtype == dtype and dl.shape == (T, E)
    assert rel(dl, dl_ref) < (F32_TOL if dtype == torch.float32 else BF16_TOL)
    assert ((dl.cpu() != 0).sum(-1) <= K).all()


def _count_sizes():
    sizes = [0, 1, 2, 3, 5, 31, 32, 33, 1000, 1023, 1025, 4099, 16384 + 7, 65536 + 3, 2097152]
    g = torch.Generator().manual_seed(0)
    sizes += torch.randint(2900, 3100, (6,), generator=g).tolist()
    return sizes


@pytest.mark.parametrize("E", [4, 8, 72, 256, 1920, 2048, 4096, 16384, 50000])
@pytest.mark.parametrize("dtype", [torch.int32, torch.int64])
def test_count_cumsum_exact(smoe, E, dtype):
    import sonicmoe

    for n in _count_sizes():
        g = torch.Generator().manual_seed(n + E)
        x = torch.randint(0, E, (n,), generator=g, dtype=dtype)
        count, cumsum = sonicmoe.count_cumsum(x.cuda(), E, do_cumsum=True)
        c_ref, cs_ref = orc.count_cumsum(x, E)
        assert count.dtype == torch.int32 and cumsum.dtype == torch.int32
        assert torch.equal(count.cpu(), c_ref), (n, E)
        assert torch.equal(cumsum.cpu(), cs_ref), (n, E)
        only = sonicmoe.count_cumsum(x.cuda(), E, do_cumsum=False)
        assert torch.equal(only.cpu(), c_ref)


@pytest.mark.parametrize("T,E,K", [(1, 4, 1), (7, 8, 2), (1000, 8, 2), (4096, 128, 8), (2048, 256, 8), (300, 4096, 4),
                                   (32768, 128, 8)])
def test_route_metadata_fixed_k_bit_exact(smoe, T, E, K):
    _, fn = smoe
    g = torch.Generator().manual_seed(T + E)
    logits = torch.randn(T, E, generator=g)
    if E >= 8:
        logits[:, 3] -= 100.0  # an expert nobody picks
        logits[:, 1] += 1.0    # a hot expert
    _, idx = orc.topk_softmax(logits, K)
    ref = orc.route_metadata(idx, E, T, K=K)
    off, gather, scatter, reverse, tok_off = fn.TC_topk_router_metadata(
        idx.cuda(), torch.empty(E, dtype=torch.int32, device="cuda"), K)
    assert torch.equal(off.cpu(), ref.expert_frequency_offset)
    assert torch.equal(scatter.cpu(), ref.s_scatter_idx)
    assert torch.equal(reverse.cpu(), ref.s_reverse_scatter_idx)
    assert torch.equal(gather.cpu(), ref.x_gather_idx)
    assert torch.equal(tok_off.cpu(), ref.token_offset)


@pytest.mark.parametrize("T,E,n", [(50, 8, 0), (50, 8, 1), (640, 4, 1024), (5000, 256, 40000), (70001, 64, 150000)])
def test_route_metadata_general_bit_exact(smoe, T, E, n):
    _, fn = smoe
    g = torch.Generator().manual_seed(n + 1)
    tokens = torch.randint(0, T, (n,), generator=g).sort().values.int()
    experts = torch.randint(0, E, (n,), generator=g).int()
    ref = orc.route_metadata(experts, E, T, token_idx=tokens)
    freq, off, gather, scatter, reverse, tok_off = fn.general_routing_router_metadata(
        torch.empty(n, device="cuda"), tokens.cuda(), experts.cuda(), T, E)
    assert torch.equal(freq.cpu(), ref.expert_frequency)
    assert torch.equal(off.cpu(), ref.expert_frequency_offset)
    assert torch.equal(scatter.cpu(), ref.s_scatter_idx)
    assert torch.equal(reverse.cpu(), ref.s_reverse_scatter_idx)
    assert torch.equal(gather.cpu(), ref.x_gather_idx)
    assert torch.equal(tok_off.cpu(), ref.token_offset)


# ---------------------------------------------------------------------------------------------------
# token rounding
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("routing", ["nr", "up", "down"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,K", [(1024, 8, 2), (2048, 16, 4), (1000, 24, 3), (4096, 256, 8), (130, 300, 2), (64, 4, 1)])
def test_token_rounding_selection_bit_exact(smoe, T, E, K, dtype, routing):
    """Kept (token, expert) pairs, their order, the scores and the rounded counts against the oracle's full sorts.
    bf16 scores tie massively after the "-1" shift, so the lower-token-first rule is exercised on every expert;
    T = 1000 and 130 are not multiples of 32 or of the tile (counts are capped at T)."""
    _lib, fn = smoe
    from sonicmoe.functional.token_rounding import select_pairs, topk_indices

    g = torch.Generator().manual_seed(T * 3 + E + K)
    logits = torch.randn(T, E, generator=g) * 2.0
    s_ref, t_ref, e_ref, score_matrix = orc.token_rounding_route(logits, K, routing, dtype)
    probs = torch.softmax(logits.float(), dim=-1).to(dtype)
    topk = topk_indices(probs.cuda(), K)
    assert torch.equal(topk.cpu().long(), probs.sort(dim=-1, descending=True, stable=True).indices[:, :K])
    tokens, experts, count = select_pairs(score_matrix.cuda(), topk, routing)
    assert torch.equal(tokens.cpu(), t_ref) and torch.equal(experts.cpu(), e_ref)
    freq = torch.bincount(topk.cpu().long().reshape(-1), minlength=E)
    want = orc.rounded_counts(freq, routing).clamp(max=T)
    assert torch.equal(count.cpu(), want.int())
    assert torch.equal(torch.bincount(e_ref.long(), minlength=E).int(), want.int())
    assert torch.equal(score_matrix[tokens.cpu().long(), experts.cpu().long()], s_ref)


def test_token_rounding_selection_all_ties(smoe):
    """Every score equal: the top-K goes to the lowest expert ids and every cut keeps the lowest token ids."""
    _lib, fn = smoe
    from sonicmoe.functional.token_rounding import select_pairs, topk_indices

    T, E, K = 700, 8, 2
    logits = torch.zeros(T, E)
    for routing in ("nr", "up", "down"):
        s_ref, t_ref, e_ref, score_matrix = orc.token_rounding_route(logits, K, routing, torch.bfloat16)
        topk = topk_indices(torch.softmax(logits, -1).bfloat16().cuda(), K)
        tokens, experts, count = select_pairs(score_matrix.cuda(), topk, routing)
        assert torch.equal(tokens.cpu(), t_ref) and torch.equal(experts.cpu(), e_ref)


# ---------------------------------------------------------------------------------------------------
# grouped GEMMs and reductions, one entry point at a time
# ---------------------------------------------------------------------------------------------------
SHAPES = [
    # T, H, I, E, K, skewed routing
    (1024, 512, 256, 8, 2, False),
    (1000, 768, 320, 8, 2, True),    # ragged tiles, N tails, an empty and a hot expert
    (300, 128, 64, 16, 4, True),     # experts far smaller than one tile
    (2048, 1024, 512, 32, 8, False),
    (1024, 512, 960, 4, 2, True),    # dual-tile units with a partly filled second tile (2I = 1920, I = 960)
]


def _problem(T, H, I, E, K, skew, seed=0):
    inp = orc.make_inputs(T, H, I, E, K, seed=seed, dtype=torch.bfloat16, w_std=0.05)
    g = torch.Generator().manual_seed(seed + 99)
    logits = torch.randn(T, E, generator=g)
    if skew:
        logits[:, 0] += 2.0
        logits[:, E - 1] -= 100.0
    scores, idx = orc.topk_softmax(logits, K)
    route = orc.route_metadata(idx, E, T, K=K)
    f32 = {k: v.float() for k, v in inp.items()}
    fwd = orc.experts_forward(f32["x"], f32["w1"], f32["w2"], scores, route)
    return inp, f32, scores, route, fwd


def _dev(route):
    return {k: getattr(route, k).cuda() for k in ("expert_frequency_offset", "x_gather_idx", "s_scatter_idx",
                                                  "s_reverse_scatter_idx", "token_offset")}


@pytest.mark.parametrize("shape", SHAPES)
def test_forward_kernels(smoe, shape):
    _lib, _ = smoe
    lib = _lib.lib
    T, H, I, E, K, skew = shape
    inp, f32, scores, route, fwd = _problem(*shape)
    d = _dev(route)
    TK = T * K
    st = _lib.device_state(torch.device("cuda", 0)).status
    stream = torch.cuda.current_stream().cuda_stream
    x, w1, w2 = inp["x"].cuda(), inp["w1"].cuda(), inp["w2"].cuda()
    nan = float("nan")
    z = torch.full((TK, 2 * I), nan, dtype=torch.bfloat16, device="cuda")
    y1 = torch.full((TK, I), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_up_projection_forward(x.data_ptr(), w1.data_ptr(), z.data_ptr(), y1.data_ptr(),
                                          d["expert_frequency_offset"].data_ptr(), d["x_gather_idx"].data_ptr(),
                                          T, H, I, E, TK, st.data_ptr(), stream) == 0
    assert rel(z, fwd["z"]) < BF16_TOL and rel(y1, fwd["y1"]) < BF16_TOL
    # inference variant: z is not written
    y1b = torch.full((TK, I), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_up_projection_forward(x.data_ptr(), w1.data_ptr(), None, y1b.data_ptr(),
                                          d["expert_frequency_offset"].data_ptr(), d["x_gather_idx"].data_ptr(),
                                          T, H, I, E, TK, st.data_ptr(), stream) == 0
    assert torch.equal(y1b, y1)

    y1_in = fwd["y1"].bfloat16().cuda()
    y2_ref = torch.empty(TK, H)
    off = route.expert_frequency_offset.tolist()
    for e in range(E):
        y2_ref[off[e]:off[e + 1]] = y1_in[off[e]:off[e + 1]].float().cpu() @ f32["w2"][e].T
    y2 = torch.full((TK, H), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_down_projection_forward(y1_in.data_ptr(), w2.data_ptr(), y2.data_ptr(),
                                            d["expert_frequency_offset"].data_ptr(), H, I, E, TK, st.data_ptr(),
                                            stream) == 0
    assert rel(y2, y2_ref) < BF16_TOL

    # combine: deterministic gather-sum, and the fused scatter-reduce epilogue
    sc = scores.reshape(-1).cuda()
    o_ref = torch.zeros(T, H).index_add(0, route.x_gather_idx.long(),
                                        y2.float().cpu() * sc.cpu()[route.s_scatter_idx.long()][:, None])
    o = torch.full((T, H), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_gather_sum(y2.data_ptr(), o.data_ptr(), sc.data_ptr(), _lib.SMOE_F32,
                               d["s_reverse_scatter_idx"].data_ptr(), None, T, H, K, stream) == 0
    assert rel(o, o_ref) < BF16_TOL
    o2 = torch.full((T, H), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_gather_sum(y2.data_ptr(), o2.data_ptr(), sc.data_ptr(), _lib.SMOE_F32,
                               d["s_reverse_scatter_idx"].data_ptr(), d["token_offset"].data_ptr(), T, H, 0,
                               stream) == 0
    assert torch.equal(o2, o)
    o_acc = torch.zeros(T, H, dtype=torch.float32, device="cuda")
    assert lib.smoe_down_projection_forward_scatter(
        y1_in.data_ptr(), w2.data_ptr(), o_acc.data_ptr(), sc.data_ptr(), 0, d["expert_frequency_offset"].data_ptr(),
        d["x_gather_idx"].data_ptr(), d["s_scatter_idx"].data_ptr(), T, H, I, E, TK, st.data_ptr(), stream) == 0
    o3 = torch.empty(T, H, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_cast_f32_to_bf16(o_acc.data_ptr(), o3.data_ptr(), T * H, stream) == 0
    assert rel(o3, fwd["o"] if False else o_ref) < BF16_TOL
    torch.cuda.synchronize()
    assert st.item() == 0


@pytest.mark.parametrize("shape", SHAPES)
def test_backward_kernels(smoe, shape):
    _lib, _ = smoe
    lib = _lib.lib
    T, H, I, E, K, skew = shape
    inp, f32, scores, route, fwd = _problem(*shape)
    d = _dev(route)
    TK = T * K
    st = _lib.device_state(torch.device("cuda", 0)).status
    stream = torch.cuda.current_stream().cuda_stream
    x, w1, w2, dout = inp["x"].cuda(), inp["w1"].cuda(), inp["w2"].cuda(), inp["dout"].cuda()
    # the device path saves z in bf16; give the oracle the same rounded z
    zb = fwd["z"].bfloat16()
    fwd_b = dict(fwd, z=zb.float(), y1=orc.swiglu(zb.float()))
    ref = orc.experts_backward(f32["x"], f32["w1"], f32["w2"], scores, route, fwd_b, f32["dout"])
    nan = float("nan")
    sc = scores.reshape(-1).cuda()
    off_p, gat_p, sct_p = (d["expert_frequency_offset"].data_ptr(), d["x_gather_idx"].data_ptr(),
                           d["s_scatter_idx"].data_ptr())

    dz = torch.full((TK, 2 * I), nan, dtype=torch.bfloat16, device="cuda")
    y1s = torch.full((TK, I), nan, dtype=torch.bfloat16, device="cuda")
    ncols = lib.smoe_ds_partial_columns(I)
    dsp = torch.full((ncols, TK), nan, dtype=torch.float32, device="cuda")
    zdev = zb.cuda()
    assert lib.smoe_down_projection_backward_act(
        dout.data_ptr(), w2.data_ptr(), zdev.data_ptr(), sc.data_ptr(), 0, dz.data_ptr(), y1s.data_ptr(),
        dsp.data_ptr(), off_p, gat_p, sct_p, T, H, I, E, TK, st.data_ptr(), stream) == 0
    assert rel(dz, ref["dz"]) < BF16_TOL and rel(y1s, ref["y1s"]) < BF16_TOL
    for dt, tol in ((torch.float32, 1e-4), (torch.bfloat16, BF16_TOL)):
        ds = torch.full((TK,), nan, dtype=dt, device="cuda")
        assert lib.smoe_ds_reduce(dsp.data_ptr(), sct_p, ds.data_ptr(), _lib.dtype_code(dt), TK, ncols, stream) == 0
        assert rel(ds, ref["ds"]) < tol

    dz_in = ref["dz"].bfloat16().cuda()
    y1s_in = ref["y1s"].bfloat16().cuda()
    offl = route.expert_frequency_offset.tolist()
    g = route.x_gather_idx.long()
    dw2_ref = torch.zeros(E, H, I)
    dw1_ref = torch.zeros(E, 2 * I, H)
    dx_ref = torch.empty(TK, H)
    for e in range(E):
        a, b = offl[e], offl[e + 1]
        dw2_ref[e] = f32["dout"][g[a:b]].T @ y1s_in[a:b].float().cpu()
        dw1_ref[e] = dz_in[a:b].float().cpu().T @ f32["x"][g[a:b]]
        dx_ref[a:b] = dz_in[a:b].float().cpu() @ f32["w1"][e]
    dw2 = torch.full((E, H, I), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_down_projection_weight_grad(dout.data_ptr(), y1s_in.data_ptr(), dw2.data_ptr(), off_p, gat_p,
                                                T, H, I, E, TK, st.data_ptr(), stream) == 0
    assert rel(dw2, dw2_ref) < BF16_TOL
    dw1 = torch.full((E, 2 * I, H), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_up_projection_weight_grad(x.data_ptr(), dz_in.data_ptr(), dw1.data_ptr(), off_p, gat_p,
                                              T, H, I, E, TK, st.data_ptr(), stream) == 0
    assert rel(dw1, dw1_ref) < BF16_TOL
    if skew:  # the expert nobody picked gets exact zeros
        assert (dw1[E - 1] == 0).all() and (dw2[E - 1] == 0).all()
    dxe = torch.full((TK, H), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_up_projection_backward_dx(dz_in.data_ptr(), w1.data_ptr(), dxe.data_ptr(), off_p, H, I, E, TK,
                                              st.data_ptr(), stream) == 0
    assert rel(dxe, dx_ref) < BF16_TOL
    dx = torch.full((T, H), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_gather_sum(dxe.data_ptr(), dx.data_ptr(), None, 0, d["s_reverse_scatter_idx"].data_ptr(), None,
                               T, H, K, stream) == 0
    assert rel(dx, torch.zeros(T, H).index_add(0, g, dxe.float().cpu())) < BF16_TOL
    torch.cuda.synchronize()
    assert st.item() == 0


@pytest.mark.parametrize("shape", SHAPES)
def test_weight_grad_accumulate_adds_to_buffer(smoe, shape):
    """The accumulating forms add each chunk's bf16-rounded gradient to what the buffer holds (fp32 add, rounded to
    bf16): bit-identical to `buffer + plain call`, the sum autograd forms for a weight used by two chunks.  Experts
    without rows and TK = 0 leave the buffer as it was."""
    _lib, _ = smoe
    lib = _lib.lib
    T, H, I, E, K, skew = shape
    inp, f32, scores, route, fwd = _problem(*shape)
    d = _dev(route)
    TK = T * K
    st = _lib.device_state(torch.device("cuda", 0)).status
    stream = torch.cuda.current_stream().cuda_stream
    x, dout = inp["x"].cuda(), inp["dout"].cuda()
    g = torch.Generator(device="cuda").manual_seed(5)
    dz = (torch.randn(TK, 2 * I, generator=g, device="cuda") * 0.1).bfloat16()
    y1s = (torch.randn(TK, I, generator=g, device="cuda") * 0.1).bfloat16()
    off_p, gat_p = d["expert_frequency_offset"].data_ptr(), d["x_gather_idx"].data_ptr()
    for name, a, b, shape_w in (("down", dout, y1s, (E, H, I)), ("up", x, dz, (E, 2 * I, H))):
        plain = getattr(lib, f"smoe_{name}_projection_weight_grad")
        accum = getattr(lib, f"smoe_{name}_projection_weight_grad_accumulate")
        one = torch.full(shape_w, float("nan"), dtype=torch.bfloat16, device="cuda")
        assert plain(a.data_ptr(), b.data_ptr(), one.data_ptr(), off_p, gat_p, T, H, I, E, TK, st.data_ptr(),
                     stream) == 0
        base = (torch.randn(shape_w, generator=g, device="cuda") * one.float().std()).bfloat16()
        buf = base.clone()
        assert accum(a.data_ptr(), b.data_ptr(), buf.data_ptr(), off_p, gat_p, T, H, I, E, TK, st.data_ptr(),
                     stream) == 0
        assert torch.equal(buf, (base.float() + one.float()).bfloat16()), name
        if skew:
            assert torch.equal(buf[E - 1], base[E - 1])
        zero_off = torch.zeros(E + 1, dtype=torch.int32, device="cuda")
        assert accum(a.data_ptr(), b.data_ptr(), buf.data_ptr(), zero_off.data_ptr(), gat_p, T, H, I, E, 0,
                     st.data_ptr(), stream) == 0
        assert torch.equal(buf, (base.float() + one.float()).bfloat16())
    torch.cuda.synchronize()
    assert st.item() == 0


def test_kernels_are_deterministic(smoe):
    """No atomics on the default path: two runs give identical bits."""
    _lib, _ = smoe
    lib = _lib.lib
    T, H, I, E, K = 1000, 768, 320, 8, 2
    inp, f32, scores, route, fwd = _problem(T, H, I, E, K, True)
    d = _dev(route)
    st = _lib.device_state(torch.device("cuda", 0)).status
    stream = torch.cuda.current_stream().cuda_stream
    x, w1 = inp["x"].cuda(), inp["w1"].cuda()
    outs = []
    for _ in range(2):
        z = torch.empty(T * K, 2 * I, dtype=torch.bfloat16, device="cuda")
        y1 = torch.empty(T * K, I, dtype=torch.bfloat16, device="cuda")
        lib.smoe_up_projection_forward(x.data_ptr(), w1.data_ptr(), z.data_ptr(), y1.data_ptr(),
                                       d["expert_frequency_offset"].data_ptr(), d["x_gather_idx"].data_ptr(),
                                       T, H, I, E, T * K, st.data_ptr(), stream)
        outs.append((z, y1))
    assert torch.equal(outs[0][0], outs[1][0]) and torch.equal(outs[0][1], outs[1][1])



@pytest.mark.parametrize("shape", [(1000, 512, 256, 8, 1, True), (2048, 1024, 512, 16, 1, False)])
def test_one_row_per_token_forms(smoe, shape):
    """K = 1: the row-writing epilogues (no y2 / dx_expanded buffer, no gather-and-sum pass) give bit for bit what the
    store + gather_sum pairs give, in bf16 and with FP8 (ue8m0) operands."""
    _lib, _ = smoe
    from sonicmoe.functional import fp8

    lib = _lib.lib
    T, H, I, E, K, skew = shape
    inp, f32, scores, route, fwd = _problem(*shape)
    d = _dev(route)
    TK = T
    st = _lib.device_state(torch.device("cuda", 0)).status
    stream = torch.cuda.current_stream().cuda_stream
    w1, w2 = inp["w1"].cuda(), inp["w2"].cuda()
    off, gat, sct, rev = (d["expert_frequency_offset"].data_ptr(), d["x_gather_idx"].data_ptr(),
                          d["s_scatter_idx"].data_ptr(), d["s_reverse_scatter_idx"].data_ptr())
    nan = float("nan")
    g = torch.Generator().manual_seed(3)
    y1 = torch.randn(TK, I, generator=g).bfloat16().cuda()
    dz = (torch.randn(TK, 2 * I, generator=g) * 0.1).bfloat16().cuda()
    for sc in (scores.reshape(-1).cuda(), scores.reshape(-1).bfloat16().cuda()):
        bf = int(sc.dtype == torch.bfloat16)
        y2 = torch.empty(TK, H, dtype=torch.bfloat16, device="cuda")
        o_two = torch.full((T, H), nan, dtype=torch.bfloat16, device="cuda")
        assert lib.smoe_down_projection_forward(y1.data_ptr(), w2.data_ptr(), y2.data_ptr(), off, H, I, E, TK,
                                                st.data_ptr(), stream) == 0
        assert lib.smoe_gather_sum(y2.data_ptr(), o_two.data_ptr(), sc.data_ptr(), _lib.dtype_code(sc.dtype), rev, None,
                                   T, H, 1, stream) == 0
        o_one = torch.full((T, H), nan, dtype=torch.bfloat16, device="cuda")
        assert lib.smoe_down_projection_forward_rows(y1.data_ptr(), w2.data_ptr(), o_one.data_ptr(), sc.data_ptr(), bf,
                                                     off, gat, sct, H, I, E, TK, st.data_ptr(), stream) == 0
        assert torch.equal(o_one, o_two)
    dxe = torch.empty(TK, H, dtype=torch.bfloat16, device="cuda")
    dx_two = torch.full((T, H), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_up_projection_backward_dx(dz.data_ptr(), w1.data_ptr(), dxe.data_ptr(), off, H, I, E, TK,
                                              st.data_ptr(), stream) == 0
    assert lib.smoe_gather_sum(dxe.data_ptr(), dx_two.data_ptr(), None, _lib.SMOE_F32, rev, None, T, H, 1, stream) == 0
    dx_one = torch.full((T, H), nan, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_up_projection_backward_dx_rows(dz.data_ptr(), w1.data_ptr(), dx_one.data_ptr(), off, gat, H, I, E,
                                                   TK, st.data_ptr(), stream) == 0
    assert torch.equal(dx_one, dx_two)

    # FP8 operands (H, I multiples of 128)
    if H % 128 == 0 and I % 128 == 0:
        y1q, y1s = fp8.quantize_rows(y1, "ue8m0")
        w2q, w2s = fp8.quantize_blocks(w2, "ue8m0")
        w1q, w1s = fp8.quantize_blocks(w1, "ue8m0")
        dzq, dzs = fp8.quantize_rows(dz, "ue8m0")
        sc = scores.reshape(-1).cuda()
        assert lib.smoe_mxfp8_down_projection_forward(y1q.data_ptr(), y1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(),
                                                      y2.data_ptr(), off, H, I, E, TK, st.data_ptr(), stream) == 0
        assert lib.smoe_gather_sum(y2.data_ptr(), o_two.data_ptr(), sc.data_ptr(), _lib.SMOE_F32, rev, None, T, H, 1,
                                   stream) == 0
        o_one.fill_(nan)
        assert lib.smoe_mxfp8_down_projection_forward_rows(
            y1q.data_ptr(), y1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), o_one.data_ptr(), sc.data_ptr(), 0, off, gat,
            sct, H, I, E, TK, st.data_ptr(), stream) == 0
        assert torch.equal(o_one, o_two)
        assert lib.smoe_mxfp8_up_projection_backward_dx(dzq.data_ptr(), dzs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(),
                                                        dxe.data_ptr(), off, H, I, E, TK, st.data_ptr(), stream) == 0
        assert lib.smoe_gather_sum(dxe.data_ptr(), dx_two.data_ptr(), None, _lib.SMOE_F32, rev, None, T, H, 1,
                                   stream) == 0
        dx_one.fill_(nan)
        assert lib.smoe_mxfp8_up_projection_backward_dx_rows(
            dzq.data_ptr(), dzs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), dx_one.data_ptr(), off, gat, H, I, E, TK,
            st.data_ptr(), stream) == 0
        assert torch.equal(dx_one, dx_two)
    torch.cuda.synchronize()
    assert st.item() == 0


_DUAL_SNIPPET = """
import sys, torch
sys.path.insert(0, {root!r}); sys.path.insert(0, {pkg!r})
from oracle import moe_oracle as orc
from sonicmoe import MoE, _lib
from sonicmoe.enums import ActivationType
T, H, I, E, K = 2048, 1024, 512, 8, 2
inp = orc.make_inputs(T, H, I, E, K, seed=5, dtype=torch.bfloat16, w_std=0.05)
moe = MoE(E, K, H, I, ActivationType.SWIGLU, False, 0.02).cuda().bfloat16()
with torch.no_grad():
    moe.router.weight.copy_(inp["router_w"]); moe.c_fc.weight.copy_(inp["w1"]); moe.c_proj.weight.copy_(inp["w2"])
x = inp["x"].cuda().requires_grad_(True)
o, _ = moe(x)
o.backward(inp["dout"].cuda())
torch.cuda.synchronize(); _lib.check_status()
torch.save({{"o": o.detach().cpu(), "dx": x.grad.cpu(), "dw1": moe.c_fc.weight.grad.cpu(),
            "dw2": moe.c_proj.weight.grad.cpu()}}, {out!r})
"""


def test_dual_tiles_match_single_tiles(smoe, tmp_path):
    """The two-tiles-per-gathered-stage kernels accumulate every tile in the same order as the single-tile kernels:
    layer outputs and all gradients must be bit-identical with SMOE_DUAL=1 (default) and SMOE_DUAL=0."""
    import os
    import subprocess
    import sys

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    pkg = os.path.join(root, "sonic-moe_b200")
    results = {}
    for dual in ("1", "0"):
        out = str(tmp_path / f"dual{dual}.pt")
        env = dict(os.environ, SMOE_DUAL=dual)
        subprocess.run([sys.executable, "-c", _DUAL_SNIPPET.format(root=root, pkg=pkg, out=out)], check=True, env=env,
                       timeout=300)
        results[dual] = torch.load(out)
    for name in ("o", "dx", "dw1", "dw2"):
        assert torch.equal(results["1"][name], results["0"][name]), name


@pytest.mark.parametrize("H", [256, 4096])
def test_gather_sum_to_segments(smoe, H):
    """The expert-parallel dispatch / return kernel on one GPU: the "other ranks' buffers" are separate local
    allocations (a peer mapping is just another device pointer to the kernel).  Plain row moves must be bit-exact,
    weighted per-token sums equal to smoe_gather_sum's."""
    import ctypes

    _lib, _ = smoe
    lib = _lib.lib
    g = torch.Generator().manual_seed(H)
    T_src, n = 700, 1500
    src = torch.randn(T_src, H, generator=g).bfloat16().cuda()
    idx = torch.randint(0, T_src, (n,), generator=g).int().cuda()
    starts = [0, 400, 400, 1100, n]           # four segments, one of them empty
    bufs = [torch.full((starts[s + 1] - starts[s] + 3, H), float("nan"), dtype=torch.bfloat16, device="cuda")
            for s in range(4)]
    seg_ptr = (ctypes.c_void_p * 4)(*[b.data_ptr() for b in bufs])
    seg_start = (ctypes.c_int * 5)(*starts)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.smoe_gather_sum_to_peers(src.data_ptr(), None, 0, idx.data_ptr(), None, n, H, 1, seg_ptr, seg_start, 4, 777,
                                        stream) == 0
    want = src[idx.long()]
    for s in range(4):
        rows = starts[s + 1] - starts[s]
        assert torch.equal(bufs[s][:rows], want[starts[s]:starts[s + 1]])
        assert bufs[s][rows:].isnan().all()     # nothing written past a segment's end

    # variable number of source rows per output row, weighted: against smoe_gather_sum on one buffer
    T_out = 300
    counts = torch.randint(0, 5, (T_out,), generator=g)
    off = torch.zeros(T_out + 1, dtype=torch.int32)
    off[1:] = counts.cumsum(0)
    m = int(off[-1])
    rev = torch.randint(0, T_src, (m,), generator=g).int().cuda()
    w = torch.rand(m, generator=g).cuda()
    off = off.cuda()
    ref = torch.empty(T_out, H, dtype=torch.bfloat16, device="cuda")
    assert lib.smoe_gather_sum(src.data_ptr(), ref.data_ptr(), w.data_ptr(), _lib.SMOE_F32, rev.data_ptr(),
                               off.data_ptr(), T_out, H, 0, stream) == 0
    starts = [0, 120, T_out]
    outs = [torch.empty(starts[s + 1] - starts[s], H, dtype=torch.bfloat16, device="cuda") for s in range(2)]
    seg_ptr = (ctypes.c_void_p * 2)(*[b.data_ptr() for b in outs])
    seg_start = (ctypes.c_int * 3)(*starts)
    assert lib.smoe_gather_sum_to_peers(src.data_ptr(), w.data_ptr(), _lib.SMOE_F32, rev.data_ptr(), off.data_ptr(),
                                        T_out, H, 0, seg_ptr, seg_start, 2, 0, stream) == 0
    assert torch.equal(torch.cat(outs), ref)
    # argument checks: segment table must cover [0, T], pointers 16-byte aligned
    bad = (ctypes.c_int * 3)(0, 120, T_out - 1)
    assert lib.smoe_gather_sum_to_peers(src.data_ptr(), None, 0, rev.data_ptr(), off.data_ptr(), T_out, H, 0, seg_ptr,
                                        bad, 2, 0, stream) == -1


def test_peer_buffer_alloc_export_copy(smoe):
    """Exchange-buffer plumbing that one process can exercise: allocate, export a handle, copy through the copy
    engine, free.  (Mapping a handle needs a second process: tests/test_expert_parallel.py on two GPUs.)"""
    import ctypes

    _lib, _ = smoe
    lib = _lib.lib
    p = ctypes.c_void_p()
    assert lib.smoe_peer_alloc(1 << 20, ctypes.byref(p)) == 0 and p.value
    handle = (ctypes.c_ubyte * 64)()
    assert lib.smoe_peer_export(p.value, handle) == 0 and any(handle)
    src = torch.arange(1 << 18, dtype=torch.int32, device="cuda")
    assert lib.smoe_peer_copy(p.value, src.data_ptr(), 1 << 20, torch.cuda.current_stream().cuda_stream) == 0
    back = torch.empty_like(src)
    assert lib.smoe_peer_copy(back.data_ptr(), p.value, 1 << 20, torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(back, src)
    assert lib.smoe_peer_free(p.value) == 0
    assert lib.smoe_peer_alloc(0, ctypes.byref(p)) == -1


def test_stream_flag_write_then_wait(smoe):
    """The arrival flags of the peer transport on one GPU: a stream writes a counter, a second stream waits until
    the flag words have reached a value that is already (or about to be) there, then copies them out.  (Only waits
    that will be satisfied are issued.)"""
    _lib, _ = smoe
    lib = _lib.lib
    flags = torch.zeros(4, dtype=torch.int32, device="cuda")
    counter = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    producer, consumer = torch.cuda.Stream(), torch.cuda.Stream()
    for seq in (1, 2, 7):
        assert lib.smoe_stream_write_value(counter.data_ptr(), seq, producer.cuda_stream) == 0
        for w in range(4):  # the sender's copy engine delivers its counter to each receiver word
            assert lib.smoe_peer_copy(flags.data_ptr() + 4 * w, counter.data_ptr(), 4, producer.cuda_stream) == 0
        assert lib.smoe_stream_wait_values(flags.data_ptr(), 4, seq, consumer.cuda_stream) == 0
        with torch.cuda.stream(consumer):
            seen = flags.clone()
        consumer.synchronize()
        assert (seen >= seq).all()
    assert lib.smoe_stream_wait_values(flags.data_ptr(), 0, 99, consumer.cuda_stream) == 0
    assert lib.smoe_stream_write_value(None, 1, consumer.cuda_stream) != 0
    torch.cuda.synchronize()
