"""Generate the golden fixtures in this directory by running the REFERENCE's own code on CPU.

Needs a checkout of the reference project, named by $SONICMOE_REFERENCE; it is not needed to run the tests, only to
regenerate the fixtures:

    SONICMOE_REFERENCE=<path to the sonic-moe checkout> python tests/golden/make_golden.py

What runs:
  * sonicmoe/moe.py `MoE(...)(x, kernel_backend_moe=KernelBackendMoE.torch)` forward + autograd backward,
    loaded file-by-file (the package import needs CUDA-only dependencies); its two sibling imports are
    stubbed: `count_cumsum` by bincount/cumsum (the module's own fallback, moe.py:308-309) and
    `moe_TC_softmax_topk_layer` by None (unused by the torch backend);
  * `forward_token_choice_rounding` and `ref_moe_token_rounding` from benchmarks/moe-token-rounding.py,
    extracted from the file's source (the script itself imports CUDA-only packages at the top).
  * `MoE(...).state_dict()` of modules the reference initialised itself (its own `reset_parameters`), stored
    with an input and the reference's eager output and gradients: the checkpoint-interchange fixtures
    (`state_dict_*.npz`).
Inputs come from oracle.moe_oracle.make_inputs (seeded), so the tests can rebuild them.

`python tests/golden/make_golden.py state_dict` regenerates only the fixtures whose name starts with that prefix.
"""

from __future__ import annotations

import ast
import importlib.util
import os
import sys
import types

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.environ.get("SONICMOE_REFERENCE")
if not REF or not os.path.isdir(REF):
    raise SystemExit("set SONICMOE_REFERENCE to the path of the reference checkout")
sys.path.insert(0, ROOT)
sys.dont_write_bytecode = True

from oracle.moe_oracle import make_inputs  # noqa: E402

# (name, T, H, I, E, K, seed, dtype used to round the inputs)
LAYER_CASES = [
    ("layer_small", 96, 128, 64, 8, 2, 0, torch.bfloat16),
    ("layer_ties", 160, 64, 64, 16, 4, 1, torch.bfloat16),
    ("layer_k1", 64, 64, 64, 4, 1, 2, torch.bfloat16),
    ("layer_cfg1", 2048, 768, 256, 8, 2, 0, torch.float32),   # BASELINE config 1; only summaries are stored
]
# (name, T, H, I, E, K, seed, activation, add_bias): modules initialised by the reference, parameters stored
STATE_DICT_CASES = [
    ("state_dict_swiglu", 48, 64, 64, 4, 2, 7, "swiglu", False),
    ("state_dict_gelu_bias", 48, 64, 128, 4, 2, 8, "gelu", True),
]
ROUNDING_CASES = [
    ("rounding_nr", 512, 64, 64, 8, 2, 3, "nr"),
    ("rounding_up", 512, 64, 64, 8, 2, 4, "up"),
    ("rounding_down", 640, 64, 64, 4, 2, 5, "down"),
]


def load_reference_moe():
    def count_cumsum(x, E, do_cumsum=True):
        c = x.bincount(minlength=E).to(torch.int32)
        return (c, c.cumsum(-1).to(torch.int32)) if do_cumsum else c

    pkg = types.ModuleType("sonicmoe")
    pkg.__path__ = [os.path.join(REF, "sonicmoe")]
    sys.modules["sonicmoe"] = pkg
    cc = types.ModuleType("sonicmoe.count_cumsum")
    cc.count_cumsum = count_cumsum
    sys.modules["sonicmoe.count_cumsum"] = cc
    fn = types.ModuleType("sonicmoe.functional")
    fn.moe_TC_softmax_topk_layer = None
    sys.modules["sonicmoe.functional"] = fn
    for name in ("enums", "moe"):
        spec = importlib.util.spec_from_file_location(f"sonicmoe.{name}", os.path.join(REF, "sonicmoe", f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[f"sonicmoe.{name}"] = mod
        spec.loader.exec_module(mod)
    # MoE.__init__ records the current CUDA stream (moe.py:206)
    torch.cuda.current_stream = lambda *a, **k: types.SimpleNamespace(cuda_stream=0)
    return sys.modules["sonicmoe.moe"], sys.modules["sonicmoe.enums"], count_cumsum


def load_reference_rounding(count_cumsum):
    path = os.path.join(REF, "benchmarks", "moe-token-rounding.py")
    tree = ast.parse(open(path).read())
    wanted = {"forward_token_choice_rounding", "ref_moe_token_rounding"}
    ns = {"torch": torch, "F": F, "count_cumsum": count_cumsum}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in wanted:
            node.decorator_list = []  # drop the cuda autocast decorator
            code = compile(ast.Module(body=[node], type_ignores=[]), path, "exec")
            exec(code, ns)
    return ns["forward_token_choice_rounding"], ns["ref_moe_token_rounding"]


def run_layer(moe_mod, enums, T, H, I, E, K, seed, dtype):
    inp = make_inputs(T, H, I, E, K, seed=seed, dtype=dtype)
    inp = {k: v.float() for k, v in inp.items()}
    m = moe_mod.MoE(E, K, H, I, enums.ActivationType.SWIGLU, False, 0.02)
    with torch.no_grad():
        m.router.weight.copy_(inp["router_w"])
        m.c_fc.weight.copy_(inp["w1"])
        m.c_proj.weight.copy_(inp["w2"])
    x = inp["x"].clone().requires_grad_(True)
    o, aux = m(x, kernel_backend_moe=enums.KernelBackendMoE.torch)
    grads = torch.autograd.grad(o, [x, m.router.weight, m.c_fc.weight, m.c_proj.weight], inp["dout"])
    logits = m.router(x.detach())
    freq = logits.topk(K, dim=-1).indices.flatten().bincount(minlength=E) if K > 1 else \
        logits.max(dim=-1).indices.bincount(minlength=E)
    return dict(o=o.detach(), aux_loss=aux.detach(), dx=grads[0], drouter_w=grads[1], dw1=grads[2], dw2=grads[3],
                logits=logits.detach(), expert_frequency=freq.to(torch.int32))


def run_state_dict(moe_mod, enums, T, H, I, E, K, seed, act, add_bias):
    """A module the reference constructs and initialises itself; biases (zero after its reset) get seeded noise so
    that they matter.  Everything a loader needs is stored: the state dict, x, dout, o, aux and all gradients."""
    torch.manual_seed(seed)
    m = moe_mod.MoE(E, K, H, I, enums.ActivationType(act), add_bias, 0.02)
    if add_bias:
        with torch.no_grad():
            m.c_fc.bias.normal_(0, 0.05)
            m.c_proj.bias.normal_(0, 0.05)
    with torch.no_grad():  # values a bf16 module can hold exactly, so that a bf16 GPU run sees the same numbers
        for p in m.parameters():
            p.copy_(p.bfloat16().float())
    x = torch.randn(T, H).bfloat16().float().requires_grad_(True)
    dout = torch.randn(T, H).bfloat16().float()
    o, aux = m(x, kernel_backend_moe=enums.KernelBackendMoE.torch)
    names = [n for n, _ in m.named_parameters()]
    grads = torch.autograd.grad(o, [x] + list(m.parameters()), dout)
    out = {f"param.{k}": v.detach().numpy() for k, v in m.state_dict().items()}
    out.update({f"grad.{n}": g.numpy() for n, g in zip(names, grads[1:])})
    out.update(x=x.detach().numpy(), dout=dout.numpy(), o=o.detach().numpy(), aux_loss=aux.detach().numpy(),
               dx=grads[0].numpy())
    return out


def summarise(t: torch.Tensor, n=64):
    """A large tensor is stored as (norm, sum, strided sample) instead of in full."""
    flat = t.reshape(-1).double()
    step = max(1, flat.numel() // n)
    return np.concatenate([[flat.norm().item(), flat.sum().item()], flat[::step][:n].numpy()])


def main():
    torch.manual_seed(0)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    moe_mod, enums, count_cumsum = load_reference_moe()
    prefix = sys.argv[1] if len(sys.argv) > 1 else ""
    for name, T, H, I, E, K, seed, act, add_bias in STATE_DICT_CASES:
        if not name.startswith(prefix):
            continue
        arrays = run_state_dict(moe_mod, enums, T, H, I, E, K, seed, act, add_bias)
        meta = np.array([T, H, I, E, K, seed, int(add_bias)], dtype=np.int64)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), meta=meta, activation=np.array(act), **arrays)
        print(name, sorted(k for k in arrays if k.startswith("param.")))
    for name, T, H, I, E, K, seed, dtype in LAYER_CASES:
        if not name.startswith(prefix):
            continue
        r = run_layer(moe_mod, enums, T, H, I, E, K, seed, dtype)
        meta = np.array([T, H, I, E, K, seed, 1 if dtype == torch.bfloat16 else 0], dtype=np.int64)
        if T * H > 100_000:
            arrays = {k: summarise(v) for k, v in r.items() if k not in ("expert_frequency", "aux_loss")}
            arrays["expert_frequency"] = r["expert_frequency"].numpy()
            arrays["aux_loss"] = r["aux_loss"].numpy()
            arrays["summary_only"] = np.array(1)
        else:
            arrays = {k: v.numpy() for k, v in r.items()}
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), meta=meta, **arrays)
        print(name, {k: v.shape for k, v in arrays.items()})

    route_fn, ref_layer = load_reference_rounding(count_cumsum)
    for name, T, H, I, E, K, seed, routing in ROUNDING_CASES:
        if not name.startswith(prefix):
            continue
        inp = make_inputs(T, H, I, E, K, seed=seed, dtype=torch.float32)
        scores, tokens, experts = route_fn(inp["x"], inp["router_w"], E, K, 128, routing)
        o = ref_layer(inp["x"], scores, tokens, experts, inp["w1"], None, inp["w2"], None, E)
        meta = np.array([T, H, I, E, K, seed], dtype=np.int64)
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), meta=meta, routing=np.array(routing),
                            scores=scores.numpy(), tokens=tokens.numpy(), experts=experts.numpy(), o=o.numpy())
        print(name, scores.shape, "pairs", "counts", torch.bincount(experts.long(), minlength=E).tolist())


if __name__ == "__main__":
    main()
