"""FP8 (E4M3, 1x128 / 128x128 block scales) path in both scale formats -- fp32 amax/448 scales applied in software
and power-of-two UE8M0 scales applied by the tensor cores: quantisation kernels, each FP8 GEMM against the exact
dequantised fp32 product, and the whole layer against a CPU simulation and the fp32 oracle on the bf16 master
weights."""

import json
import os

import pytest
import torch

from oracle import moe_oracle as orc

pytestmark = pytest.mark.gpu

FP8_TOL = 3e-2


def rel(a, b):
    a = a.detach().float().cpu()
    b = b.detach().float().cpu()
    return ((a - b).norm() / (b.norm() + 1e-30)).item()


def dequant_rows(q, s):
    return q.view(torch.float8_e4m3fn).float() * s.repeat_interleave(128, dim=-1)


def dequant_blocks(q, s):
    E, rows, cols = q.shape
    full = s.repeat_interleave(128, dim=1)[:, :rows].repeat_interleave(128, dim=2)
    return q.view(torch.float8_e4m3fn).float() * full


@pytest.mark.parametrize("rows,cols", [(1, 128), (1000, 256), (4096, 1024)])
def test_quantize_rows(built_library, rows, cols):
    from sonicmoe.functional import fp8

    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, cols, generator=g) * torch.rand(rows, 1, generator=g) * 3).bfloat16()
    x[0, :128] = 0  # an all-zero block keeps scale 1
    q, s = fp8.quantize_rows(x.cuda())
    amax = x.float().view(rows, cols // 128, 128).abs().amax(-1)
    s_ref = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    assert torch.equal(s.cpu(), s_ref)
    assert rel(dequant_rows(q, s), x) < 0.04          # e4m3 has 3 mantissa bits
    assert dequant_rows(q, s).abs().max().item() <= x.float().abs().max().item() * 1.0001


@pytest.mark.parametrize("E,rows,cols", [(2, 128, 128), (3, 320, 256), (4, 512, 1024)])
def test_quantize_blocks(built_library, E, rows, cols):
    from sonicmoe.functional import fp8

    g = torch.Generator().manual_seed(rows + E)
    w = (torch.randn(E, rows, cols, generator=g) * 0.02).bfloat16()
    q, s = fp8.quantize_blocks(w.cuda())
    rb, cb = (rows + 127) // 128, cols // 128
    pad = torch.zeros(E, rb * 128, cols)
    pad[:, :rows] = w.float()
    amax = pad.view(E, rb, 128, cb, 128).abs().amax(dim=(2, 4))
    assert torch.equal(s.cpu(), torch.where(amax > 0, amax / 448.0, torch.ones_like(amax)))
    assert rel(dequant_blocks(q, s), w) < 0.04


@pytest.mark.parametrize("rows,cols", [(1, 128), (1000, 256), (4096, 1024), (333, 640)])
def test_quantize_rows_pow2(built_library, rows, cols):
    from oracle import fp8_sim
    from sonicmoe.functional import fp8

    g = torch.Generator().manual_seed(rows)
    x = (torch.randn(rows, cols, generator=g) * torch.rand(rows, 1, generator=g) * 3).bfloat16()
    x[0, :128] = 0                      # an all-zero block keeps scale 2^0
    if rows > 2:
        x[1, :128] = 0
        x[1, 5] = 448.0                 # amax / 448 exactly a power of two
        x[2, :128] = 2.0 ** -130        # scale clamps at 2^-127
    q, s = fp8.quantize_rows(x.cuda(), "ue8m0")
    nblk = cols // 128
    assert s.dtype == torch.uint8 and s.shape == (rows, 4 * ((nblk + 3) // 4))
    amax = x.float().view(rows, nblk, 128).abs().amax(-1)
    want = fp8_sim.block_scale(amax, pow2=True)
    assert torch.equal(torch.exp2(s.cpu()[:, :nblk].float() - 127.0), want)
    assert (s.cpu()[:, nblk:] == 127).all()
    # bit-exact with the simulation's quantise-dequantise
    assert torch.equal(fp8.dequantize(q, s).cpu(), fp8_sim.quant_rows(x.float(), pow2=True))


@pytest.mark.parametrize("E,rows,cols", [(2, 128, 128), (3, 320, 256), (4, 512, 1024)])
def test_quantize_blocks_pow2(built_library, E, rows, cols):
    from oracle import fp8_sim
    from sonicmoe.functional import fp8

    g = torch.Generator().manual_seed(rows + E)
    w = (torch.randn(E, rows, cols, generator=g) * 0.02).bfloat16()
    q, s = fp8.quantize_blocks(w.cuda(), "ue8m0")
    assert s.dtype == torch.uint8 and s.shape == (E, (rows + 127) // 128, cols // 128)
    assert torch.equal(fp8.dequantize(q, s).cpu(), fp8_sim.quant_blocks(w.float(), pow2=True))


SHAPES = [(512, 256, 128, 4, 2, False), (1000, 512, 256, 8, 2, True), (300, 128, 128, 16, 4, True),
          (2048, 1024, 640, 8, 4, False),   # 8 and 5 k-blocks (two scale words per row, a partial group)
          # one rank of the expert-parallel FP8 benchmark: H 7168, I 2048, 32 local experts, one row per received token
          (2048, 7168, 2048, 32, 1, False)]


def draw_inputs(T, H, I, E, K, seed, w_std):
    """Small layers: the oracle's seeded CPU inputs.  Large ones are drawn on the GPU (a billion weights take the CPU
    generator most of a minute) and copied to the host."""
    if E * I * H < 1 << 26:
        return orc.make_inputs(T, H, I, E, K, seed=seed, dtype=torch.bfloat16, w_std=w_std)
    g = torch.Generator(device="cuda").manual_seed(seed)

    def rn(*shape, std):
        return (torch.randn(*shape, generator=g, device="cuda") * std).bfloat16().cpu()

    return dict(router_w=rn(E, H, std=w_std), w1=rn(E, 2 * I, H, std=w_std), w2=rn(E, H, I, std=w_std),
                x=rn(T, H, std=1.0), dout=rn(T, H, std=1.0))


@pytest.mark.parametrize("fmt", ["fp32", "ue8m0"])
@pytest.mark.parametrize("shape", SHAPES)
def test_fp8_gemms_match_dequantised_products(built_library, shape, fmt):
    """Each FP8 GEMM computes exactly sum_kb (A_q . B_q)_kb * sa * sb in fp32: compare with that product."""
    from sonicmoe import _lib
    from sonicmoe.functional import fp8

    lib = _lib.lib
    T, H, I, E, K, skew = shape
    inp = draw_inputs(T, H, I, E, K, seed=T, w_std=0.05)
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(T, E, generator=g)
    if skew:
        logits[:, 0] += 2.0
        logits[:, E - 1] -= 100.0
    scores, idx = orc.topk_softmax(logits, K)
    route = orc.route_metadata(idx, E, T, K=K)
    off = route.expert_frequency_offset.tolist()
    gat = route.x_gather_idx.long()
    TK = T * K
    dev = torch.device("cuda", 0)
    st = _lib.device_state(dev).status
    stream = torch.cuda.current_stream().cuda_stream
    d_off, d_gat, d_sct = (route.expert_frequency_offset.cuda(), route.x_gather_idx.cuda(), route.s_scatter_idx.cuda())

    x, w1, w2, dout = inp["x"].cuda(), inp["w1"].cuda(), inp["w2"].cuda(), inp["dout"].cuda()
    xq, xs = fp8.quantize_rows(x, fmt)
    w1q, w1s = fp8.quantize_blocks(w1, fmt)
    w2q, w2s = fp8.quantize_blocks(w2, fmt)
    xd, w1d, w2d = fp8.dequantize(xq, xs).cpu(), fp8.dequantize(w1q, w1s).cpu(), fp8.dequantize(w2q, w2s).cpu()

    # up projection
    nan = float("nan")
    z = torch.full((TK, 2 * I), nan, dtype=torch.bfloat16, device=dev)
    y1 = torch.full((TK, I), nan, dtype=torch.bfloat16, device=dev)
    assert fp8._entry("up_projection_forward", fmt)(xq.data_ptr(), xs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(),
                                              z.data_ptr(), y1.data_ptr(), d_off.data_ptr(), d_gat.data_ptr(),
                                              T, H, I, E, TK, st.data_ptr(), stream) == 0
    z_ref = torch.empty(TK, 2 * I)
    for e in range(E):
        z_ref[off[e]:off[e + 1]] = xd[gat[off[e]:off[e + 1]]] @ w1d[e].T
    assert rel(z, z_ref) < 1e-2 and rel(y1, orc.swiglu(z_ref)) < 1e-2

    if fmt == "ue8m0":
        # the variant whose epilogue quantises y1: same z, and bytes + scales identical to the row quantiser applied
        # to the bf16 y1 of the plain variant
        z2 = torch.full((TK, 2 * I), nan, dtype=torch.bfloat16, device=dev)
        ld = lib.smoe_mxfp8_scale_row_bytes(I)
        y1q_f = torch.zeros(TK, I, dtype=torch.uint8, device=dev)
        y1s_f = torch.full((TK, ld), 127, dtype=torch.uint8, device=dev)
        assert lib.smoe_mxfp8_up_projection_forward_q(
            xq.data_ptr(), xs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), z2.data_ptr(), y1q_f.data_ptr(),
            y1s_f.data_ptr(), d_off.data_ptr(), d_gat.data_ptr(), T, H, I, E, TK, st.data_ptr(), stream) == 0
        assert torch.equal(z2, z)
        y1q_r, y1s_r = fp8.quantize_rows(y1, "ue8m0")
        assert torch.equal(y1q_f, y1q_r) and torch.equal(y1s_f, y1s_r)

    # down projection
    y1b = orc.swiglu(z_ref).bfloat16().cuda()
    y1q, y1s = fp8.quantize_rows(y1b, fmt)
    y1d = fp8.dequantize(y1q, y1s).cpu()
    y2 = torch.full((TK, H), nan, dtype=torch.bfloat16, device=dev)
    assert fp8._entry("down_projection_forward", fmt)(y1q.data_ptr(), y1s.data_ptr(), w2q.data_ptr(), w2s.data_ptr(),
                                                y2.data_ptr(), d_off.data_ptr(), H, I, E, TK, st.data_ptr(),
                                                stream) == 0
    y2_ref = torch.empty(TK, H)
    for e in range(E):
        y2_ref[off[e]:off[e + 1]] = y1d[off[e]:off[e + 1]] @ w2d[e].T
    assert rel(y2, y2_ref) < 1e-2

    # dH with the dSwiGLU epilogue
    dq, dsc = fp8.quantize_rows(dout, fmt)
    dd = fp8.dequantize(dq, dsc).cpu()
    zb = z_ref.bfloat16()
    dz = torch.full((TK, 2 * I), nan, dtype=torch.bfloat16, device=dev)
    ys = torch.full((TK, I), nan, dtype=torch.bfloat16, device=dev)
    ncols = lib.smoe_ds_partial_columns(I)
    dsp = torch.zeros(ncols, TK, dtype=torch.float32, device=dev)
    sc = scores.reshape(-1).cuda()
    zdev = zb.cuda()
    assert fp8._entry("down_projection_backward_act", fmt)(
        dq.data_ptr(), dsc.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), zdev.data_ptr(), sc.data_ptr(), 0,
        dz.data_ptr(), ys.data_ptr(), dsp.data_ptr(), d_off.data_ptr(), d_gat.data_ptr(), d_sct.data_ptr(),
        T, H, I, E, TK, st.data_ptr(), stream) == 0
    if fmt == "ue8m0":
        # the variant whose epilogue also quantises dz: same dz / y1s / ds, and bytes + scales identical to the row
        # quantiser applied to the bf16 dz
        dz2 = torch.full((TK, 2 * I), nan, dtype=torch.bfloat16, device=dev)
        ys2 = torch.full((TK, I), nan, dtype=torch.bfloat16, device=dev)
        dsp2 = torch.zeros(ncols, TK, dtype=torch.float32, device=dev)
        ld = lib.smoe_mxfp8_scale_row_bytes(2 * I)
        dzq_f = torch.zeros(TK, 2 * I, dtype=torch.uint8, device=dev)
        dzs_f = torch.full((TK, ld), 127, dtype=torch.uint8, device=dev)
        assert lib.smoe_mxfp8_down_projection_backward_act_q(
            dq.data_ptr(), dsc.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), zdev.data_ptr(), sc.data_ptr(), 0,
            dz2.data_ptr(), ys2.data_ptr(), dsp2.data_ptr(), dzq_f.data_ptr(), dzs_f.data_ptr(), d_off.data_ptr(),
            d_gat.data_ptr(), d_sct.data_ptr(), T, H, I, E, TK, st.data_ptr(), stream) == 0
        assert torch.equal(dz2, dz) and torch.equal(ys2, ys) and torch.equal(dsp2, dsp)
        dzq_r, dzs_r = fp8.quantize_rows(dz, "ue8m0")
        assert torch.equal(dzq_f, dzq_r) and torch.equal(dzs_f, dzs_r)
    dy1 = torch.empty(TK, I)
    for e in range(E):
        dy1[off[e]:off[e + 1]] = dd[gat[off[e]:off[e + 1]]] @ w2d[e]
    s = scores.reshape(-1)[route.s_scatter_idx.long()][:, None]
    zf = zb.float()
    gate, up = zf[:, 0::2], zf[:, 1::2]
    sig = torch.sigmoid(gate)
    y1r = gate * sig * up
    dz_ref = torch.stack([dy1 * up * sig * (1 + gate * (1 - sig)) * s, dy1 * gate * sig * s], dim=-1).reshape(TK, 2 * I)
    assert rel(dz, dz_ref) < 1e-2 and rel(ys, y1r * s) < 1e-2
    assert rel(dsp.sum(0), (dy1 * y1r).sum(-1)) < 1e-3

    # dX
    dzb = dz_ref.bfloat16().cuda()
    dzq, dzs = fp8.quantize_rows(dzb, fmt)
    dzd = fp8.dequantize(dzq, dzs).cpu()
    dxe = torch.full((TK, H), nan, dtype=torch.bfloat16, device=dev)
    assert fp8._entry("up_projection_backward_dx", fmt)(dzq.data_ptr(), dzs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(),
                                                  dxe.data_ptr(), d_off.data_ptr(), H, I, E, TK, st.data_ptr(),
                                                  stream) == 0
    dx_ref = torch.empty(TK, H)
    for e in range(E):
        dx_ref[off[e]:off[e + 1]] = dzd[off[e]:off[e + 1]] @ w1d[e]
    assert rel(dxe, dx_ref) < 1e-2
    torch.cuda.synchronize()
    assert st.item() == 0


LAYER_CASES = [(512, 256, 128, 16, 4, "fp32"), (512, 256, 128, 16, 4, "ue8m0"), (1024, 512, 256, 8, 2, "fp32"),
               (1024, 512, 256, 8, 2, "ue8m0"), (777, 1024, 384, 32, 8, "fp32"), (777, 1024, 384, 32, 8, "ue8m0"),
               # the expert-parallel FP8 benchmark's per-rank dimensions (H 7168, I 2048, 32 experts, K 8)
               (512, 7168, 2048, 32, 8, "ue8m0")]


@pytest.mark.parametrize("T,H,I,E,K,fmt", LAYER_CASES)
def test_fp8_layer(built_library, T, H, I, E, K, fmt):
    """Whole FP8 layer.

    Kernel numerics: against a CPU simulation with the same quantisation points (oracle/fp8_sim.py), <= 2e-2
    (a last-bit difference in an intermediate can flip its E4M3 rounding, a 6-12 % change of that element, so
    two correct implementations of the chained layer differ by about 1 %; each single FP8 GEMM is checked to 1e-2
    against its exact dequantised product in test_fp8_gemms_match_dequantised_products).
    Number format: against the fp32 oracle on the bf16 master weights.  Rounding both operands of a product to
    E4M3 (3 mantissa bits, relative rms error ~2.6 % each) leaves ~3.6 % relative error in every GEMM output
    whatever the reduction length, ~5-7 % after two chained GEMMs, so the 3e-2 stated for this path cannot be
    met by any E4M3 x E4M3 implementation on Gaussian data; the test requires the device path to be no further
    from fp32 than the simulation is (within 10 %) and below 9e-2 in absolute terms.
    """
    from oracle import fp8_sim
    from sonicmoe import _lib
    from sonicmoe.functional import topk_softmax
    from sonicmoe.functional.fp8 import moe_fp8_softmax_topk_layer

    inp = draw_inputs(T, H, I, E, K, seed=T + E, w_std=0.02)
    x = inp["x"].cuda().requires_grad_(True)
    rw = inp["router_w"].cuda().requires_grad_(True)
    w1 = inp["w1"].cuda().requires_grad_(True)
    w2 = inp["w2"].cuda().requires_grad_(True)
    o, logits, freq = moe_fp8_softmax_topk_layer(x, rw, w1.permute(1, 2, 0), None, w2.permute(1, 2, 0), None, K,
                                                 scale_format=fmt)
    scores_dev, idx = topk_softmax(logits.detach(), K)
    # gradient of the expert path only (scores detached) so that it can be compared term by term
    grads = torch.autograd.grad(o, [x, w1, w2], inp["dout"].cuda())
    torch.cuda.synchronize()
    _lib.check_status()
    f32 = {k: v.float() for k, v in inp.items()}
    ref = orc.moe_layer(f32["x"], f32["router_w"], f32["w1"], f32["w2"], K, dout=f32["dout"],
                        logits=logits.detach().float().cpu())
    assert torch.equal(idx.cpu(), ref["indices"])
    assert torch.equal(freq.cpu(), ref["expert_frequency"])
    sim = fp8_sim.experts_forward_backward(f32["x"], f32["w1"], f32["w2"], ref["scores"], ref["route"], f32["dout"],
                                           pow2=fmt == "ue8m0")
    dlogits = orc.softmax_topk_backward(ref["scores"], ref["indices"], sim["ds"].reshape(T, K), E)
    sim_dx = sim["dx"] + dlogits @ f32["router_w"]
    ref_pairs = {"o": (o, sim["o"], ref["o"]), "dx": (grads[0], sim_dx, ref["dx"]),
                 "dw1": (grads[1], sim["dw1"], ref["dw1"]), "dw2": (grads[2], sim["dw2"], ref["dw2"])}
    report = {}
    for name, (dev_t, sim_t, f32_t) in ref_pairs.items():
        kernel_err = rel(dev_t, sim_t)
        format_err = rel(sim_t, f32_t)
        total_err = rel(dev_t, f32_t)
        report[name] = {"device_vs_fp32": total_err, "simulation_vs_fp32": format_err, "device_vs_simulation": kernel_err}
        assert kernel_err < 2e-2, (name, kernel_err)
        assert total_err < 9e-2 and total_err < 1.1 * format_err + 1e-2, (name, total_err, format_err)
    path = os.environ.get("SMOE_FP8_ERROR_REPORT")   # a file to which the measured errors of every case are appended
    if path:
        with open(path, "a") as f:
            f.write(json.dumps({"T": T, "H": H, "I": I, "E": E, "K": K, "scales": fmt, **report}) + "\n")
