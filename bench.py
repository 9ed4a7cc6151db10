"""Benchmark of the MoE-layer hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload: benchmark configuration 2 — T=32768 tokens, H=4096, I=1024, E=128 experts, top-K=8, SwiGLU, bf16,
token-choice softmax top-k routing; weights iid N(0, 0.02), x and upstream gradient iid N(0, 1), seeded,
synthetic.  One step = one forward + backward of the layer through `sonicmoe.MoE` (all gradients: x,
router, up and down projections).  FLOP model of the reference benchmark: 18 * T*K * I * H per step
(benchmarks/moe-cute.py:231-234, 297-300); router GEMM, softmax and combine are timed but not counted.

With N > 1 the same layer runs expert-parallel: every rank keeps its own T tokens and E/N of the experts, token
rows travel to the experts' ranks and back with an NCCL all-to-all each way (weak scaling; `value` is the sum over
ranks).  Before timing, the N > 1 run checks itself: output and gradients of a small slice of every rank's tokens
against the CPU oracle on the gathered slice (errors in the JSON line).

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU oracle (a port of the reference's
torch-eager layer) on the host cores on a bounded sample of the same workload.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "sonic-moe_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

CFG = dict(T=32768, H=4096, I=1024, E=128, K=8)
CPU_SAMPLE_TOKENS = 512  # tokens of the same layer shape the CPU baseline processes per step
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def flops_per_step(T, H, I, K):
    return 18.0 * T * K * I * H


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS if k in p} | {"source": "measured"}
    return dict(FALLBACK_PEAKS, source="fallback")


# --------------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples nvidia-smi while the timed region runs (read-only queries)."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.rows: list[list[str]] = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._pump, daemon=True)
        self.thread.start()

    def _pump(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 7:
                self.rows.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# --------------------------------------------------------------------------------------------------
# the CPU arm (oracle port of the reference's torch-eager layer)
# --------------------------------------------------------------------------------------------------
def cpu_sample_inputs(cfg, tokens, device_for_rng):
    """fp32 weights of the full layer and `tokens` tokens, values as in the GPU arm (N(0,.02) / N(0,1))."""
    H, I, E = cfg["H"], cfg["I"], cfg["E"]
    g = torch.Generator(device=device_for_rng).manual_seed(0)

    def rn(*shape, std):
        t = torch.randn(*shape, generator=g, device=device_for_rng, dtype=torch.float32) * std
        return t.bfloat16().float().cpu()

    return dict(router_w=rn(E, H, std=0.02), w1=rn(E, 2 * I, H, std=0.02), w2=rn(E, H, I, std=0.02),
                x=rn(tokens, H, std=1.0), dout=rn(tokens, H, std=1.0))


def cpu_step(inp, K):
    from oracle import moe_oracle as orc

    t0 = time.perf_counter()
    orc.moe_layer(inp["x"], inp["router_w"], inp["w1"], inp["w2"], K, dout=inp["dout"])
    return time.perf_counter() - t0


def time_config1_cpu(reps=3):
    """The reference's own CPU-runnable case (T2048 H768 I256 E8 K2, fp32, seed 0), whole layer forward+backward."""
    from oracle import moe_oracle as orc

    c1 = dict(T=2048, H=768, I=256, E=8, K=2)
    inp = orc.make_inputs(c1["T"], c1["H"], c1["I"], c1["E"], c1["K"], seed=0, dtype=torch.float32)
    cpu_step(inp, c1["K"])
    dt = min(cpu_step(inp, c1["K"]) for _ in range(reps))
    return {"config": c1, "ms_per_step": dt * 1e3,
            "tflops": flops_per_step(c1["T"], c1["H"], c1["I"], c1["K"]) / dt / 1e12}


def run_reference_arm(args, rank, world):
    """The CPU arm: the oracle port of the reference's torch-eager layer (sonicmoe/moe.py:276-363) on all host
    threads.  Every step processes CPU_SAMPLE_TOKENS tokens of the benchmark layer (full H, I, E, K): a bounded
    sample, stated in `config.tokens_per_step` -- the rate, not the step time, is what compares with the GPU arm."""
    if rank != 0:
        return
    cfg = CFG
    torch.set_num_threads(os.cpu_count() or 1)
    rng_dev = "cuda" if torch.cuda.is_available() else "cpu"
    inp = cpu_sample_inputs(cfg, CPU_SAMPLE_TOKENS, rng_dev)
    for _ in range(args.warmup):
        cpu_step(inp, cfg["K"])
    times = [cpu_step(inp, cfg["K"]) for _ in range(args.steps)]
    dt = sum(times) / len(times)
    fl = flops_per_step(CPU_SAMPLE_TOKENS, cfg["H"], cfg["I"], cfg["K"])
    value = fl / dt / 1e12
    sample = (f"{CPU_SAMPLE_TOKENS} tokens per step of the same layer (H{cfg['H']} I{cfg['I']} E{cfg['E']} "
              f"K{cfg['K']}), fp32, forward+backward with all gradients")
    config = dict(workload_config(args.gpus), T=CPU_SAMPLE_TOKENS, tokens_per_step=CPU_SAMPLE_TOKENS,
                  full_workload_tokens=cfg["T"], l2_policy="n/a (host)")
    line = {
        "impl": "reference", "metric": "moe_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "tokens_per_s": CPU_SAMPLE_TOKENS / dt,
        "config": config,
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "config1_cpu": time_config1_cpu(),
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    par = "single" if n_gpus == 1 else f"ep{n_gpus}"
    return {"workload": "moe_layer_fwd_bwd_top8_of_128_T32768_H4096_I1024_swiglu_bf16", **CFG,
            "routing": "softmax_topk", "parallelism": par,
            "tokens": "T per GPU",
            "l2_policy": "inputs larger than L2 (weights 3 GiB, activations > 1 GiB per step)"}


# --------------------------------------------------------------------------------------------------
# the GPU arm
# --------------------------------------------------------------------------------------------------
def build_layer(cfg, dev):
    import sonicmoe
    from sonicmoe.enums import ActivationType

    torch.manual_seed(0)
    torch.cuda.manual_seed(0)
    with torch.device(dev):
        moe = sonicmoe.MoE(cfg["E"], cfg["K"], cfg["H"], cfg["I"], ActivationType.SWIGLU, False, 0.02)
        torch.nn.init.normal_(moe.router.weight, 0.0, 0.02)
    return moe.to(torch.bfloat16)


def zero_grads(moe, x):
    x.grad = None
    for p in moe.parameters():
        p.grad = None


def time_kernels(moe, x, dout, cfg, peaks, reps=5):
    """CUDA-event time of each grouped GEMM launched alone on the benchmark's tensors (inputs far larger than
    L2), and of the two gather-sum reductions; returns per-kernel figures and the dominant GEMM."""
    from sonicmoe import _lib, functional as fn

    lib = _lib.lib
    dev = x.device
    T, H, I, E, K = (cfg[k] for k in "THIEK")
    TK = T * K
    st = _lib.device_state(dev).status.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    with torch.no_grad():
        logits = torch.nn.functional.linear(x, moe.router.weight).contiguous()
        scores, idx = fn.topk_softmax(logits, K)
        route = fn._route_metadata(idx.reshape(-1), None, E, K)
    off, gat, sct, rev = (route.expert_frequency_offset.data_ptr(), route.x_gather_idx.data_ptr(),
                          route.s_scatter_idx.data_ptr(), route.s_reverse_scatter_idx.data_ptr())
    bf = dict(dtype=torch.bfloat16, device=dev)
    w1, w2 = moe.c_fc.weight.detach(), moe.c_proj.weight.detach()
    z = torch.empty(TK, 2 * I, **bf); y1 = torch.empty(TK, I, **bf); y2 = torch.empty(TK, H, **bf)
    dz = torch.empty(TK, 2 * I, **bf); y1s = torch.empty(TK, I, **bf); o = torch.empty(T, H, **bf)
    dw1 = torch.empty_like(w1); dw2 = torch.empty_like(w2)
    ncols = lib.smoe_ds_partial_columns(I)
    dsp = torch.empty(ncols, TK, dtype=torch.float32, device=dev)
    sc = scores.reshape(-1)
    unit = 2.0 * TK * I * H  # flops of one TK x I x H contraction
    ops = {
        "up_projection_forward": (2 * unit, lambda: lib.smoe_up_projection_forward(
            x.data_ptr(), w1.data_ptr(), z.data_ptr(), y1.data_ptr(), off, gat, T, H, I, E, TK, st, stream)),
        "down_projection_forward": (unit, lambda: lib.smoe_down_projection_forward(
            y1.data_ptr(), w2.data_ptr(), y2.data_ptr(), off, H, I, E, TK, st, stream)),
        "down_projection_backward_act": (unit, lambda: lib.smoe_down_projection_backward_act(
            dout.data_ptr(), w2.data_ptr(), z.data_ptr(), sc.data_ptr(), 0, dz.data_ptr(), y1s.data_ptr(),
            dsp.data_ptr(), off, gat, sct, T, H, I, E, TK, st, stream)),
        "down_projection_weight_grad": (unit, lambda: lib.smoe_down_projection_weight_grad(
            dout.data_ptr(), y1s.data_ptr(), dw2.data_ptr(), off, gat, T, H, I, E, TK, st, stream)),
        "up_projection_weight_grad": (2 * unit, lambda: lib.smoe_up_projection_weight_grad(
            x.data_ptr(), dz.data_ptr(), dw1.data_ptr(), off, gat, T, H, I, E, TK, st, stream)),
        "up_projection_backward_dx": (2 * unit, lambda: lib.smoe_up_projection_backward_dx(
            dz.data_ptr(), w1.data_ptr(), y2.data_ptr(), off, H, I, E, TK, st, stream)),
    }
    gather_bytes = TK * H * 2 + T * H * 2 + TK * 8
    hbm_ops = {
        "gather_sum_weighted": (gather_bytes, lambda: lib.smoe_gather_sum(
            y2.data_ptr(), o.data_ptr(), sc.data_ptr(), _lib.SMOE_F32, rev, None, T, H, K, stream)),
        "gather_sum_plain": (gather_bytes, lambda: lib.smoe_gather_sum(
            y2.data_ptr(), o.data_ptr(), None, 0, rev, None, T, H, K, stream)),
    }
    # routing kernels (HBM / latency bound): the fused front end, the counting sort, the router backward kernel
    rw = moe.router.weight.detach()
    if lib.smoe_router_forward_supported(H, E, K):
        r_logits = torch.empty(T, E, **bf)
        r_scores = torch.empty(T, K, dtype=torch.float32, device=dev)
        r_idx = torch.empty(T, K, dtype=torch.int32, device=dev)
        r_cnt = torch.empty(E, dtype=torch.int32, device=dev)
        r_col = torch.empty(E, dtype=torch.float32, device=dev)
        r_ws = _lib.device_state(dev).router_workspace(E)
        hbm_ops["router_forward_fused"] = (T * H * 2 + E * H * 2 + T * E * 2 + T * K * 8, lambda: lib.smoe_router_forward(
            x.data_ptr(), rw.data_ptr(), r_logits.data_ptr(), r_scores.data_ptr(), r_idx.data_ptr(), r_cnt.data_ptr(),
            r_col.data_ptr(), r_ws.data_ptr(), T, H, E, K, st, stream))
        g_sc = torch.randn(T, K, device=dev)
        d_logits = torch.empty(T, E, **bf)
        hbm_ops["router_backward"] = (2 * T * E * 2 + T * K * 12, lambda: lib.smoe_router_backward(
            d_logits.data_ptr(), logits.data_ptr(), g_sc.data_ptr(), sc.data_ptr(), idx.data_ptr(), None, None, T, E, K,
            stream))
    m_ws = _lib.device_state(dev).route_workspace(E)
    m_out = torch.empty(3, TK, dtype=torch.int32, device=dev)
    m_cnt = torch.empty(E, dtype=torch.int32, device=dev)
    m_off = torch.empty(E + 1, dtype=torch.int32, device=dev)
    idx_flat = idx.reshape(-1).contiguous()
    hbm_ops["route_metadata"] = (TK * 4 + 3 * TK * 4, lambda: lib.smoe_route_metadata(
        idx_flat.data_ptr(), None, TK, E, K, m_cnt.data_ptr(), m_off.data_ptr(), m_out[0].data_ptr(),
        m_out[1].data_ptr(), m_out[2].data_ptr(), m_ws.data_ptr(), stream))
    # the expert-parallel dispatch kernel (row gather whose output goes to per-rank segments) with four local buffers
    # standing in for four ranks': every token to 3.6 of 4 ranks on average, as top-8 over 4 x 32 experts gives
    import ctypes

    W_seg = 4
    g_seg = torch.Generator(device=dev).manual_seed(7)
    member = torch.rand(T, W_seg, generator=g_seg, device=dev) < 0.9
    seg_rows = [torch.nonzero(member[:, d]).flatten().int() for d in range(W_seg)]
    seg_idx = torch.cat(seg_rows).contiguous()
    n_seg = seg_idx.numel()
    seg_bufs = [torch.empty(max(r.numel(), 1), H, **bf) for r in seg_rows]
    seg_start = [0]
    for r in seg_rows:
        seg_start.append(seg_start[-1] + r.numel())
    seg_ptr_c = (ctypes.c_void_p * W_seg)(*[b.data_ptr() for b in seg_bufs])
    seg_start_c = (ctypes.c_int * (W_seg + 1))(*seg_start)
    # algorithmic bytes: every source row read once, every routed row written once (the kernel walks the segments one
    # after the other, so a source larger than L2 is in fact read once per segment)
    hbm_ops["dispatch_gather_to_segments"] = (T * H * 2 + n_seg * H * 2 + n_seg * 4, lambda: lib.smoe_gather_sum_to_peers(
        x.data_ptr(), None, 0, seg_idx.data_ptr(), None, n_seg, H, 1, seg_ptr_c, seg_start_c, W_seg, seg_start[1],
        stream))
    out = {}

    def timed(fn_):
        fn_()  # warm
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            rc = fn_()
            assert rc == 0, rc
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    for name, (fl, f) in ops.items():
        ms = timed(f)
        tf = fl / (ms * 1e-3) / 1e12
        out[name] = {"ms": round(ms, 4), "tflops": round(tf, 1), "frac_of_bf16_peak": round(tf / peaks["bf16_tflops"], 3)}
    for name, (by, f) in hbm_ops.items():
        ms = timed(f)
        gbs = by / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 4), "gbs": round(gbs, 1), "frac_of_hbm_peak": round(gbs / peaks["hbm_gbs"], 3)}
    _lib.check_status(dev)
    dominant = max(ops, key=lambda n: out[n]["ms"])
    return out, dominant, ops[dominant][0]


# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu capture summarised under profiles/
# (None until a capture exists for the kernel).
NCU_TRAFFIC_BYTES = {  # profiles/grouped_gemm_router_gather_T8192_E32_ncu_full.txt, scaled x4 to T=32768, E=128
    "up_projection_forward": 6.53e9,
    "down_projection_forward": 3.59e9,
    "down_projection_backward_act": 6.29e9,
    "down_projection_weight_grad": 2.74e9,
    "up_projection_weight_grad": 4.60e9,
    "up_projection_backward_dx": 5.37e9,
}


def profile_step(args, local_rank):
    """Where one steady-state step's time goes: every kernel's device time inside the step (CUPTI through
    torch.profiler), their sum, and the part of the step during which no kernel ran (launch gaps / host stalls).
    Prints one JSON object; not a benchmark number (profiling slows the host side down)."""
    from torch.profiler import ProfilerActivity, profile

    cfg = CFG
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    T, H = cfg["T"], cfg["H"]
    moe = build_layer(cfg, dev)
    g = torch.Generator(device=dev).manual_seed(1234)
    x = torch.randn(T, H, generator=g, device=dev).bfloat16().requires_grad_(True)
    dout = torch.randn(T, H, generator=g, device=dev).bfloat16()

    def step():
        zero_grads(moe, x)
        o, _aux = moe(x)
        o.backward(dout)

    for _ in range(5):
        step()
    torch.cuda.synchronize()
    n = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        e0.record()
        for _ in range(n):
            step()
        e1.record()
        torch.cuda.synchronize()
    step_ms = e0.elapsed_time(e1) / n
    spans = []
    per_kernel = {}
    for ev in prof.events():
        if ev.device_type.name != "CUDA":
            continue
        dur_us = ev.time_range.end - ev.time_range.start
        if dur_us <= 0:
            continue
        spans.append((ev.time_range.start, ev.time_range.end))
        name = ev.name.split("<")[0].split("(")[0][-60:]
        k = per_kernel.setdefault(name, [0, 0.0])
        k[0] += 1
        k[1] += dur_us
    spans.sort()
    busy = 0.0
    cur_s, cur_e = spans[0]
    for s_, e_ in spans[1:]:
        if s_ <= cur_e:
            cur_e = max(cur_e, e_)
        else:
            busy += cur_e - cur_s
            cur_s, cur_e = s_, e_
    busy += cur_e - cur_s
    kernels = sorted(((v[1] / n / 1e3, v[0] // n, k) for k, v in per_kernel.items()), reverse=True)
    print(json.dumps({
        "step_ms_cuda_events": step_ms, "kernel_busy_ms_per_step": busy / n / 1e3,
        "idle_ms_per_step": step_ms - busy / n / 1e3,
        "kernel_ms_sum_per_step": sum(k[0] for k in kernels), "launches_per_step": sum(k[1] for k in kernels),
        "kernels": [{"ms_per_step": round(ms, 4), "launches_per_step": cnt, "name": name} for ms, cnt, name in kernels],
    }), flush=True)


def run_gpu_arm(args, rank, world, local_rank):
    from sonicmoe import _lib

    cfg = CFG
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    distributed = world > 1
    if distributed:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    T, H, I, E, K = (cfg[k] for k in "THIEK")

    moe = build_layer(cfg, dev)
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    x_host = torch.randn(T, H, generator=g, device=dev).bfloat16().cpu().pin_memory()
    dout_host = torch.randn(T, H, generator=g, device=dev).bfloat16().cpu().pin_memory()
    x = x_host.to(dev, non_blocking=True).requires_grad_(True)
    dout = dout_host.to(dev, non_blocking=True)
    o_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    dx_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()

    def step_resident():
        zero_grads(moe, x)
        o, _aux = moe(x)
        o.backward(dout)

    def zero_param_grads():
        for p in moe.parameters():
            p.grad = None

    steps_e2e = host_pipeline(dev, x_host, dout_host, o_host, dx_host, zero_param_grads, lambda xs: moe(xs)[0])

    def barrier():
        torch.cuda.synchronize()
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_region(fn, steps):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if distributed:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item()

    for _ in range(max(args.warmup, 3)):
        step_resident()
    _lib.check_status(dev)

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = _lib.launch_count()
    total_ms = timed_region(step_resident, args.steps)
    launches = _lib.launch_count() - launches_before
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status(dev)

    def step_forward():  # training-mode forward alone (saves what backward needs), as the reference's benchmark times it
        o, _aux = moe(x)
        del o

    step_forward()
    fwd_ms = timed_region(step_forward, args.steps) / args.steps

    steps_e2e(2)
    e2e_ms = timed_region(lambda: steps_e2e(args.steps), 1)
    _lib.check_status(dev)

    ms_per_step = total_ms / args.steps
    fl = flops_per_step(T, H, I, K)
    value = world * fl / (ms_per_step * 1e-3) / 1e12
    e2e_value = world * fl / (e2e_ms / args.steps * 1e-3) / 1e12

    if rank != 0:
        if distributed:
            dist.barrier()
            dist.destroy_process_group()
        return

    kernels, dominant, dom_flops = time_kernels(moe, x.detach(), dout, cfg, peaks)
    achieved = kernels[dominant]["tflops"]
    roofline = {"bound": "tensor", "kernel": dominant, "achieved": achieved, "peak": peaks["bf16_tflops"],
                "unit": "TFLOP/s", "frac": round(achieved / peaks["bf16_tflops"], 3),
                "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "flops_per_launch": dom_flops,
                "traffic": NCU_TRAFFIC_BYTES.get(dominant),
                "layer_frac_of_sustained_peak": round(value / world / peaks["bf16_tflops_sustained"], 3)}

    cpu_baseline = None
    if world == 1:
        torch.set_num_threads(os.cpu_count() or 1)
        inp = cpu_sample_inputs(cfg, CPU_SAMPLE_TOKENS, dev)
        cpu_step(inp, K)  # warm
        dt = min(cpu_step(inp, K) for _ in range(2))
        cpu_baseline = {
            "value": flops_per_step(CPU_SAMPLE_TOKENS, H, I, K) / dt / 1e12, "unit": "TFLOP/s",
            "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{CPU_SAMPLE_TOKENS} tokens of the same layer shape, fp32 oracle forward+backward, "
                      f"{dt * 1e3:.0f} ms"}

    line = {
        "metric": "moe_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "tokens_per_s": world * T / (ms_per_step * 1e-3),
        "tflops_per_gpu": value / world,
        "forward_ms": fwd_ms, "backward_ms": ms_per_step - fwd_ms,
        "forward_tflops_per_gpu": fl / 3.0 / (fwd_ms * 1e-3) / 1e12,
        "config": workload_config(world),
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "ms_per_step": e2e_ms / args.steps,
                "h2d_bytes_per_step": 2 * T * H * 2, "d2h_bytes_per_step": 2 * T * H * 2,
                "api": "sonicmoe.MoE.forward + backward; every step copies x and dout from pinned host memory and o and dx "
                       "back to it; copies on side streams, double-buffered, overlapping the neighbouring steps' compute"},
        "gpu_launches": launches,
        "roofline": roofline,
        "kernels": kernels,
        "cpu_baseline": cpu_baseline,
    }
    print(json.dumps(line), flush=True)
    if distributed:
        dist.barrier()
        dist.destroy_process_group()


EP_CFG = dict(T=65536, H=2048, I=768, E=64, K=4)  # benchmark configuration 5: tokens per GPU, Zipf-skewed routing
EP_FP8_CFG = dict(T=16384, H=7168, I=2048, E=256, K=8)  # benchmark configuration 4: tokens per GPU, FP8 experts
ROUNDING_CFG = dict(T=16384, H=4096, I=1024, E=256, K=8)  # benchmark configuration 3: token rounding to multiples of 128


def run_rounding_arm(args, local_rank):
    """Token-rounding routing (benchmark configuration 3): T=16384, H=4096, I=1024, E=256, K=8; after top-K every expert's
    token count is rounded to the nearest multiple of 128.  As in the reference's benchmark
    (benchmarks/moe-token-rounding.py:355-455) the timed region is the routed layer forward + backward on
    precomputed routing; the router's own time is reported beside it.  FLOPs use the realised pair count."""
    from sonicmoe import _lib
    from sonicmoe.enums import ActivationType
    from sonicmoe.functional import forward_token_choice_rounding, moe_general_routing_inputs

    cfg = ROUNDING_CFG
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    T, H, I, E, K = (cfg[k] for k in "THIEK")
    g = torch.Generator(device=dev).manual_seed(0)
    router_w = (torch.randn(E, H, generator=g, device=dev) * 0.02).bfloat16()
    w1 = (torch.randn(E, 2 * I, H, generator=g, device=dev) * 0.02).bfloat16().requires_grad_(True)
    w2 = (torch.randn(E, H, I, generator=g, device=dev) * 0.02).bfloat16().requires_grad_(True)
    x = torch.randn(T, H, generator=g, device=dev).bfloat16().requires_grad_(True)
    dout = torch.randn(T, H, generator=g, device=dev).bfloat16()

    def route():
        with torch.no_grad():
            return forward_token_choice_rounding(x.detach(), router_w, E, K, 128, "nr")

    scores, tokens, experts = route()
    scores = scores.detach().requires_grad_(True)
    params = [x, scores, w1, w2]

    def step():
        for p_ in params:
            p_.grad = None
        o, _freq = moe_general_routing_inputs(x, scores, tokens, experts, w1.permute(1, 2, 0), None,
                                              w2.permute(1, 2, 0), None, E, 0, ActivationType.SWIGLU)
        o.backward(dout)

    def timed(fn, n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    for _ in range(max(args.warmup, 3)):
        step()
    ms = timed(step, args.steps)
    route_ms = timed(route, 3)
    _lib.check_status(dev)
    pairs = tokens.numel()
    counts = torch.bincount(experts.long(), minlength=E)
    value = 18.0 * pairs * I * H / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "moe_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "tokens_per_s": T / (ms * 1e-3),
        "config": {"workload": "moe_layer_fwd_bwd_token_rounding_nr128_T16384_H4096_I1024_E256_K8", **cfg,
                   "routing": "token choice top-K, per-expert count rounded to the nearest multiple of 128"},
        "routed_pairs": pairs, "pairs_vs_topk": pairs / (T * K), "router_ms": route_ms,
        "all_counts_multiple_of_128": bool((counts % 128 == 0).all().item()),
    }), flush=True)


EP_WORKLOADS = {
    # name: (config, fp8 experts, Zipf logit bias, workload label)
    "topk": (CFG, False, False, "moe_layer_fwd_bwd_top8_of_128_T32768_H4096_I1024_swiglu_bf16"),
    "ep_zipf": (EP_CFG, False, True, "moe_layer_fwd_bwd_expert_parallel_zipf_T65536_per_gpu_H2048_I768_E64_K4"),
    "ep_fp8": (EP_FP8_CFG, True, False, "moe_layer_fwd_bwd_expert_parallel_fp8_T16384_per_gpu_H7168_I2048_E256_K8"),
}
EP_PARITY_TOKENS = 2048          # tokens of the gathered batch the in-run parity check uses (all ranks together)
EP_PARITY_MAX_WEIGHT_BYTES = 16e9  # fp32 copy of all experts the CPU oracle may hold


def expert_weights(e, H, I, dev):
    """Expert e's weights, the same on whichever rank draws them (seeded by the expert's global id)."""
    g = torch.Generator(device=dev).manual_seed(1000 + e)
    w1 = (torch.randn(2 * I, H, generator=g, device=dev) * 0.02).bfloat16()
    w2 = (torch.randn(H, I, generator=g, device=dev) * 0.02).bfloat16()
    return w1, w2


def ep_parity_check(layer, x, dout, router_w, w1, w2, logit_bias, cfg, rank, world, dev):
    """Expert-parallel forward + backward on a slice of every rank's tokens against the CPU oracle applied to the
    gathered slice with all E experts (rank 0 draws the other ranks' experts from their seeds).  Returns the relative
    Frobenius errors (rank 0) -- the run's own evidence that the exchanged result equals the single-device layer."""
    import torch.distributed as dist

    T, H, I, E, K = (cfg[k] for k in "THIEK")
    e_local = E // world
    n = max(128, EP_PARITY_TOKENS // world)
    xs = x[:n].detach().clone().requires_grad_(True)
    ds = dout[:n]
    for p_ in (router_w, w1, w2):
        p_.grad = None
    o, logits = layer(xs)
    o.backward(ds)
    torch.cuda.synchronize()

    def gathered(t):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        return torch.cat(parts).float().cpu()

    x_all, d_all, o_all, dx_all, lg_all = (gathered(t) for t in (xs.detach(), ds, o.detach(), xs.grad, logits.detach()))
    drouter = router_w.grad.detach().float().clone()
    dist.all_reduce(drouter)
    out = None
    if rank == 0:
        from oracle import moe_oracle as orc

        w1_all = torch.empty(E, 2 * I, H)
        w2_all = torch.empty(E, H, I)
        for e in range(E):
            a, b = expert_weights(e, H, I, dev)
            w1_all[e], w2_all[e] = a.float().cpu(), b.float().cpu()
        ref = orc.moe_layer(x_all, router_w.detach().float().cpu(), w1_all, w2_all, K, dout=d_all, logits=lg_all)

        def rel(a, b):
            return ((a.float().cpu() - b).norm() / (b.norm() + 1e-30)).item()

        out = {"tokens": n * world, "o": rel(o_all, ref["o"]), "dx": rel(dx_all, ref["dx"]),
               "dw1_rank0": rel(w1.grad, ref["dw1"][:e_local]), "dw2_rank0": rel(w2.grad, ref["dw2"][:e_local]),
               "drouter": rel(drouter, ref["drouter_w"]), "tolerance": 1e-2, "against": "CPU oracle, fp32"}
        out["ok"] = all(v < out["tolerance"] for k_, v in out.items() if k_ in ("o", "dx", "dw1_rank0", "dw2_rank0",
                                                                                 "drouter"))
    for p_ in (router_w, w1, w2):
        p_.grad = None
    dist.barrier()
    return out


def host_pipeline(dev, x_host, dout_host, o_host, dx_host, zero_grads, forward):
    """End-to-end steps: every step's x and dout come from pinned host memory and its o and dx go back to pinned host
    memory.  Returns steps(n), which runs n such steps; a timed region around it contains every copy.

    The copies run on two side streams with double-buffered device inputs, so the host->device copies of step i+1
    and the device->host copies of step i-1 overlap the compute of step i (what a prefetching input pipeline does).
    Within a step the forward pass waits for x only and the backward pass for dout, and o leaves while the backward
    pass runs, so the pipeline fills with one copy of x and drains with one copy of dx."""
    T, H = x_host.shape
    copy_in, copy_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    x_buf = [torch.empty(T, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    dout_buf = [torch.empty(T, H, dtype=torch.bfloat16, device=dev) for _ in range(2)]
    x_ready = [torch.cuda.Event() for _ in range(2)]
    dout_ready = [torch.cuda.Event() for _ in range(2)]
    buf_free = [torch.cuda.Event() for _ in range(2)]

    def enqueue_inputs(i):
        b = i % 2
        with torch.cuda.stream(copy_in):
            copy_in.wait_event(buf_free[b])  # the step that last used this buffer pair has finished with it
            x_buf[b].copy_(x_host, non_blocking=True)
            x_ready[b].record(copy_in)
            dout_buf[b].copy_(dout_host, non_blocking=True)
            dout_ready[b].record(copy_in)

    def steps(n):
        cur = torch.cuda.current_stream(dev)
        enqueue_inputs(0)
        for i in range(n):
            b = i % 2
            if i + 1 < n:
                enqueue_inputs(i + 1)
            cur.wait_event(x_ready[b])
            xs = x_buf[b].detach().requires_grad_(True)
            zero_grads()
            o = forward(xs)
            fwd_done = torch.cuda.Event()
            fwd_done.record(cur)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(fwd_done)
                o_host.copy_(o.detach(), non_blocking=True)
            o.record_stream(copy_out)
            cur.wait_event(dout_ready[b])
            o.backward(dout_buf[b])
            buf_free[b].record(cur)
            done = torch.cuda.Event()
            done.record(cur)
            with torch.cuda.stream(copy_out):
                copy_out.wait_event(done)
                dx_host.copy_(xs.grad, non_blocking=True)
            xs.grad.record_stream(copy_out)
        cur.wait_stream(copy_out)

    return steps


def run_ep_arm(args, rank, world, local_rank, workload):
    """Expert-parallel layer, experts sharded over the ranks, dispatch/combine by NCCL all-to-all.
    Default workload with --gpus N > 1: the benchmark layer itself (T=32768 tokens per GPU, E=128 experts, 128/N per
    rank).  `--workload ep_zipf` (benchmark configuration 5): T=65536 tokens per GPU, H=2048, I=768, E=64, K=4, router
    logits biased by 2*log(1/rank_e) with a seeded permutation of expert ranks.  `--workload ep_fp8` (benchmark
    configuration 4): T=16384 per GPU, H=7168, I=2048, E=256, K=8, expert GEMMs of forward and activation gradients in
    FP8 E4M3 with 1x128 / 128x128 block scales (weight gradients bf16)."""
    import torch.distributed as dist

    from sonicmoe import _lib, expert_parallel as ep

    cfg, fp8, zipf, label = EP_WORKLOADS[workload]
    ops = ep.Fp8CudaOps(args.fp8_scales) if fp8 else None
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", device_id=dev)
    peaks = load_peaks()
    T, H, I, E, K = (cfg[k] for k in "THIEK")
    e_local = E // world
    g = torch.Generator(device=dev).manual_seed(0)
    router_w = (torch.randn(E, H, generator=g, device=dev) * 0.02).bfloat16().requires_grad_(True)
    ranks = torch.randperm(E, generator=g, device=dev) + 1
    logit_bias = 2.0 * torch.log(1.0 / ranks.float()) if zipf else None
    mine = [expert_weights(rank * e_local + e, H, I, dev) for e in range(e_local)]
    w1 = torch.stack([m[0] for m in mine]).requires_grad_(True)
    w2 = torch.stack([m[1] for m in mine]).requires_grad_(True)
    del mine
    g = torch.Generator(device=dev).manual_seed(1 + rank)
    x_host = torch.randn(T, H, generator=g, device=dev).bfloat16().cpu().pin_memory()
    dout_host = torch.randn(T, H, generator=g, device=dev).bfloat16().cpu().pin_memory()
    x = x_host.to(dev).requires_grad_(True)
    dout = dout_host.to(dev)
    o_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    dx_host = torch.empty(T, H, dtype=torch.bfloat16).pin_memory()
    params = [router_w, w1, w2]
    stats = {}

    def layer(xs):
        o, logits, freq = ep.moe_ep_softmax_topk_layer(xs, router_w, w1, w2, K, E, logit_bias=logit_bias, ops=ops)
        stats["freq"] = freq
        return o, logits

    parity = None
    if E * 3.0 * I * H * 4 <= EP_PARITY_MAX_WEIGHT_BYTES:
        parity = ep_parity_check(layer, x, dout, router_w, w1, w2, logit_bias, cfg, rank, world, dev)
    elif rank == 0:
        parity = {"skipped": "an fp32 copy of all experts for the CPU oracle exceeds the host-memory bound of this "
                             "check; the same path is compared with the oracle in tests/test_expert_parallel.py"}

    def step():
        x.grad = None
        for p_ in params:
            p_.grad = None
        o, _ = layer(x)
        o.backward(dout)

    def zero_param_grads():
        for p_ in params:
            p_.grad = None

    steps_e2e = host_pipeline(dev, x_host, dout_host, o_host, dx_host, zero_param_grads, lambda xs: layer(xs)[0])

    def barrier():
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return ms.item() / n

    for _ in range(max(args.warmup, 3)):
        step()
    _lib.check_status(dev)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    launches_before = _lib.launch_count()
    ms_per_step = timed(step, args.steps)
    launches = _lib.launch_count() - launches_before
    clocks = sampler.stop() if rank == 0 else None
    _lib.check_status(dev)

    # time spent inside the all-to-alls (CUDA events around each one, on the compute stream), max over ranks
    ep.record_exchanges(True)
    step()
    torch.cuda.synchronize()
    events = ep.record_exchanges(False)
    a2a = torch.tensor([sum(a.elapsed_time(b) for a, b in events)], device=dev)
    dist.all_reduce(a2a, op=dist.ReduceOp.MAX)

    steps_e2e(2)
    e2e_ms = timed(lambda: steps_e2e(args.steps), 1) / args.steps
    _lib.check_status(dev)

    # The four row exchanges of a step alone (no GEMMs between them, ranks aligned by a barrier): what the transfers
    # cost at the link, apart from the waiting for slower ranks that the per-exchange times of a real step include.
    exchange_alone = None
    transport = ep.default_transport(None, x, ops or ep.CudaOps()) if world > 1 else None
    if transport is not None and hasattr(transport, "impl"):
        with torch.no_grad():
            logits_ = torch.nn.functional.linear(x.detach(), router_w.detach())
            if logit_bias is not None:
                logits_ = logits_ + logit_bias.to(logits_.dtype)
            _, idx_ = (ops or ep.CudaOps()).topk_softmax(logits_, K)
            plan = ep.plan_dispatch(idx_, E, world, None)[0]
            impl = transport.impl

            def exchanges():
                rows = impl.dispatch_rows(x.detach(), plan, ("bench_dispatch",))
                impl.return_rows(rows, plan, ("bench_return",))
                rows = impl.dispatch_rows(dout, plan, ("bench_dispatch",))
                impl.return_rows(rows, plan, ("bench_return",))

            exchanges()
            alone_ms = timed(exchanges, args.steps)
        out_rows = sum(r for d, r in enumerate(plan.send_rows) if d != rank)   # dispatches
        back_rows = sum(r for s_, r in enumerate(plan.recv_rows) if s_ != rank)  # returns
        sent_t = torch.tensor([2.0 * (out_rows + back_rows) * H * 2], device=dev)
        dist.all_reduce(sent_t, op=dist.ReduceOp.MAX)
        exchange_alone = {"ms_per_step": alone_ms, "share_of_step": alone_ms / ms_per_step,
                          "bytes_to_other_ranks_per_step": sent_t.item(),
                          "gbs_per_direction": sent_t.item() / (alone_ms * 1e-3) / 1e9,
                          "note": "dispatch x, return, dispatch dout, return, back to back with their barriers; "
                                  "GB/s = bytes one rank sends to other ranks in the four exchanges / that time "
                                  "(measured peer copy in one direction: 770 GB/s)"}

    freq = stats["freq"].float()
    dist.all_reduce(freq)  # rows per expert over all ranks
    kernels = dominant = None
    if rank == 0 and not fp8:
        # the local problem of one rank: all routed rows of T tokens over E/N experts
        kcfg = dict(cfg, E=e_local, K=min(K, e_local))
        moe_local = build_layer(kcfg, dev)
        kernels, dominant, dom_flops = time_kernels(moe_local, x.detach(), dout, kcfg, peaks)
        del moe_local
    if rank == 0:
        total_rows = freq.sum().item()
        fl = 18.0 * total_rows * I * H
        value = fl / (ms_per_step * 1e-3) / 1e12
        per_rank_rows = freq.view(world, e_local).sum(1)
        line = {
            "metric": "moe_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp8_e4m3 (weight gradients bf16)" if fp8 else "bf16", "data": "synthetic",
            "tokens_per_s": world * T / (ms_per_step * 1e-3), "tflops_per_gpu": value / world,
            "config": {"workload": label, **cfg, "tokens": "T per GPU", "parallelism": f"ep{world}",
                       "collective": ("token rows once per destination rank over peer memory (own gather-and-store "
                                      "kernel + copy-engine copies; a one-element NCCL all-reduce as the barrier on "
                                      "the compute stream, stream-written arrival flags on the copy stream); "
                                      "scores and indices by NCCL all_to_all_single"
                                      if world > 1 and os.environ.get("SONICMOE_EP_TRANSPORT", "peer").startswith("peer") else
                                      "NCCL all_to_all_single (token rows once per destination rank, scores, indices)"),
                       "routing": "softmax_topk" + (" + per-expert logit bias 2*log(1/rank)" if zipf else ""),
                       "l2_policy": "inputs larger than L2"},
            **({"fp8_scale_format": args.fp8_scales} if fp8 else {}),
            "clocks": clocks,
            "e2e": {"value": fl / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": 2 * T * H * 2, "d2h_bytes_per_step": 2 * T * H * 2,
                    "api": "moe_ep_softmax_topk_layer forward + backward; every step copies x and dout from pinned host "
                           "memory and o and dx back to it (per rank); copies on side streams, double-buffered, "
                           "overlapping the neighbouring steps' compute"},
            "gpu_launches": launches,
            "all_to_all_ms_per_step": a2a.item(), "all_to_all_share": a2a.item() / ms_per_step,
            "all_to_all_note": "sum of the exchanges' durations on the streams they run on (CUDA events, max over ranks); "
                               "with the peer transport the backward return of the row gradients runs on the copy stream "
                               "beside the weight-gradient GEMMs, so part of this time is not exposed",
            "exchanges_alone": exchange_alone,
            "expert_load_max_over_mean": (freq.max() / freq.mean()).item(),
            "rank_load_max_over_mean": (per_rank_rows.max() / per_rank_rows.mean()).item(),
            "ep_parity": parity,
            "comm_nranks_ok": dist.get_world_size() == world,
        }
        if kernels is not None:
            achieved = kernels[dominant]["tflops"]
            line["roofline"] = {"bound": "tensor", "kernel": dominant, "achieved": achieved,
                                "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                "frac": round(achieved / peaks["bf16_tflops"], 3),
                                "peak_source": f"{peaks['source']} cuBLAS bf16 burst", "flops_per_launch": dom_flops,
                                "traffic": None,
                                "note": "rank 0's local problem: the routed rows of T tokens over E/N experts"}
            line["kernels"] = kernels
        line["cpu_baseline"] = None  # N = 1 only
        print(json.dumps(line), flush=True)
    dist.barrier()
    ep.close_default_transports()
    dist.destroy_process_group()



def run_fp8_arm(args, local_rank):
    """The benchmark layer (the default workload's shapes) with the expert GEMMs of forward and activation gradients in
    FP8 E4M3 (1x128 / 128x128 block scales, `--fp8-scales`), weight gradients in bf16: a side workload, not the
    headline line (whose dtype is bf16).  `--kernels-only` times each FP8 GEMM alone on `--tokens` / `--experts`
    (the command the ncu captures of these kernels use)."""
    from sonicmoe import _lib
    from sonicmoe.functional import _route_metadata, fp8, topk_softmax

    fmt = args.fp8_scales
    cfg = dict(CFG, T=args.tokens, E=args.experts) if args.kernels_only else dict(CFG)
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    T, H, I, E, K = (cfg[k] for k in "THIEK")
    TK = T * K
    g = torch.Generator(device=dev).manual_seed(0)
    router_w = (torch.randn(E, H, generator=g, device=dev) * 0.02).bfloat16().requires_grad_(True)
    w1 = (torch.randn(E, 2 * I, H, generator=g, device=dev) * 0.02).bfloat16().requires_grad_(True)
    w2 = (torch.randn(E, H, I, generator=g, device=dev) * 0.02).bfloat16().requires_grad_(True)
    x = torch.randn(T, H, generator=g, device=dev).bfloat16().requires_grad_(True)
    dout = torch.randn(T, H, generator=g, device=dev).bfloat16()

    def timed(fn, n):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    if args.kernels_only:
        lib = _lib.lib
        with torch.no_grad():
            scores, idx = topk_softmax(torch.randn(T, E, generator=g, device=dev), K)
            route = _route_metadata(idx.reshape(-1), None, E, K)
            off, gat, sct = (route.expert_frequency_offset.data_ptr(), route.x_gather_idx.data_ptr(),
                             route.s_scatter_idx.data_ptr())
            st = _lib.device_state(dev).status.data_ptr()
            stream = torch.cuda.current_stream().cuda_stream
            xq, xs = fp8.quantize_rows(x.detach(), fmt)
            w1q, w1s = fp8.quantize_blocks(w1.detach(), fmt)
            w2q, w2s = fp8.quantize_blocks(w2.detach(), fmt)
            z = torch.randn(TK, 2 * I, device=dev).bfloat16()
            y1 = torch.randn(TK, I, device=dev).bfloat16()
            y2 = torch.empty(TK, H, dtype=torch.bfloat16, device=dev)
            dz = torch.empty_like(z)
            y1s = torch.empty_like(y1)
            y1q, y1sc = fp8.quantize_rows(y1, fmt)
            zq, zs = fp8.quantize_rows(z, fmt)
            dq, dqs = fp8.quantize_rows(dout, fmt)
            dsp = torch.empty(lib.smoe_ds_partial_columns(I), TK, dtype=torch.float32, device=dev)
            sc = scores.reshape(-1).contiguous()
            unit = 2.0 * TK * I * H
            calls = {
                "quantize_rows(x)": (0.0, lambda: fp8.quantize_rows(x.detach(), fmt)),
                "quantize_blocks(w1)": (0.0, lambda: fp8.quantize_blocks(w1.detach(), fmt)),
                "up_projection_forward": (2 * unit, lambda: fp8._entry("up_projection_forward", fmt)(
                    xq.data_ptr(), xs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), z.data_ptr(), y1.data_ptr(), off, gat,
                    T, H, I, E, TK, st, stream)),
                "down_projection_forward": (unit, lambda: fp8._entry("down_projection_forward", fmt)(
                    y1q.data_ptr(), y1sc.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), y2.data_ptr(), off, H, I, E, TK, st,
                    stream)),
                "down_projection_backward_act": (unit, lambda: fp8._entry("down_projection_backward_act", fmt)(
                    dq.data_ptr(), dqs.data_ptr(), w2q.data_ptr(), w2s.data_ptr(), z.data_ptr(), sc.data_ptr(), 0,
                    dz.data_ptr(), y1s.data_ptr(), dsp.data_ptr(), off, gat, sct, T, H, I, E, TK, st, stream)),
                "up_projection_backward_dx": (2 * unit, lambda: fp8._entry("up_projection_backward_dx", fmt)(
                    zq.data_ptr(), zs.data_ptr(), w1q.data_ptr(), w1s.data_ptr(), y2.data_ptr(), off, H, I, E, TK, st,
                    stream)),
            }
            kernels = {}
            for name, (flops, fn) in calls.items():
                ms = timed(fn, args.reps)
                kernels[name] = {"ms": ms, **({"tflops": flops / ms / 1e9} if flops else {})}
        _lib.check_status(dev)
        print(json.dumps({"config": {**cfg, "fp8_scale_format": fmt}, "kernels": kernels}), flush=True)
        return

    params = [x, router_w, w1, w2]

    def step():
        for p_ in params:
            p_.grad = None
        o, _logits, _freq = fp8.moe_fp8_softmax_topk_layer(x, router_w, w1.permute(1, 2, 0), None, w2.permute(1, 2, 0),
                                                           None, K, scale_format=fmt)
        o.backward(dout)

    for _ in range(max(args.warmup, 3)):
        step()
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(step, args.steps)
    clocks = sampler.stop()
    _lib.check_status(dev)
    value = 18.0 * TK * I * H / (ms * 1e-3) / 1e12
    print(json.dumps({
        "metric": "moe_fwd_bwd_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8_e4m3 (weight gradients bf16)", "data": "synthetic",
        "tokens_per_s": T / (ms * 1e-3), "fp8_scale_format": fmt, "clocks": clocks,
        "config": {"workload": "moe_layer_fwd_bwd_fp8_T32768_H4096_I1024_E128_K8", **cfg},
    }), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    # profiling aid: time (or let ncu capture) each kernel alone on a reduced token / expert count
    ap.add_argument("--kernels-only", action="store_true")
    # profiling aid: per-kernel device time and idle time inside a steady-state step (torch.profiler)
    ap.add_argument("--profile-step", action="store_true")
    ap.add_argument("--tokens", type=int, default=CFG["T"])
    ap.add_argument("--experts", type=int, default=CFG["E"])
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--workload", default="topk", choices=["topk", "ep_zipf", "ep_fp8", "token_rounding", "fp8"])
    # ep_fp8: "fp32" = amax/448 scales applied in software, "ue8m0" = rounded up to a power of two, applied by the tensor cores
    ap.add_argument("--fp8-scales", default="ue8m0", choices=["fp32", "ue8m0"])
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference_arm(args, rank, world)
        return
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the layer has no CPU path (use --impl reference for the CPU arm)")
    if args.profile_step:
        profile_step(args, local_rank)
        return
    if args.workload == "token_rounding":
        run_rounding_arm(args, local_rank)
        return
    if args.workload == "fp8":
        run_fp8_arm(args, local_rank)
        return
    if args.workload in ("ep_zipf", "ep_fp8") or (args.workload == "topk" and world > 1 and not args.kernels_only):
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        os.environ.setdefault("RANK", "0")
        os.environ.setdefault("WORLD_SIZE", "1")
        run_ep_arm(args, rank, world, local_rank, args.workload)
        return
    if args.kernels_only:
        cfg = dict(CFG, T=args.tokens, E=args.experts)
        dev = torch.device("cuda", local_rank)
        torch.cuda.set_device(dev)
        moe = build_layer(cfg, dev)
        g = torch.Generator(device=dev).manual_seed(1)
        x = torch.randn(cfg["T"], cfg["H"], generator=g, device=dev).bfloat16()
        dout = torch.randn(cfg["T"], cfg["H"], generator=g, device=dev).bfloat16()
        kernels, dominant, _ = time_kernels(moe, x, dout, cfg, load_peaks(), reps=args.reps)
        print(json.dumps({"config": cfg, "kernels": kernels, "dominant": dominant}), flush=True)
        return
    run_gpu_arm(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
