"""Shared helpers of the parity tests: build a backend from an oracle layer, load fixtures,
error metrics with the tolerances of the parity contract."""
import os

import torch
from safetensors import safe_open
from safetensors.torch import load_file

from oracle import ek_oracle as O
from oracle import configs as OC

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# bf16 outputs: max relative error 2e-2 (relative to the largest reference magnitude) and
# mean absolute error 1e-3, as the parity contract states.
MAX_REL = 2e-2
MEAN_ABS = 1e-3


def output_errors(got: torch.Tensor, ref: torch.Tensor):
    g, r = got.float().cpu(), ref.float().cpu()
    d = (g - r).abs()
    scale = r.abs().max().clamp_min(1e-6)
    return (d.max() / scale).item(), d.mean().item()


def record(what: str, **numbers):
    """One line per parity case with the measured figures (shown by `pytest -rP` / `-s`); appended to
    the file named by EK_PARITY_REPORT when that is set, so that a GPU run leaves the margins to
    the tolerances on record."""
    line = "PARITY " + what + ": " + ", ".join(
        f"{k}={v:.3e}" if isinstance(v, float) else f"{k}={v}" for k, v in numbers.items())
    print(line)
    path = os.environ.get("EK_PARITY_REPORT")
    if path:
        with open(path, "a") as f:
            f.write(line + "\n")


def assert_outputs_close(got, ref, what=""):
    max_rel, mean_abs = output_errors(got, ref)
    assert max_rel <= MAX_REL and mean_abs <= MEAN_ABS, f"{what}: max-rel {max_rel:.3e}, mean-abs {mean_abs:.3e}"


def quant_code(q: str) -> int:
    return {"bf16": 0, "fp8": 1, "int8": 2}[q]


def backend_config(cfg: O.MoEConfig, max_tokens: int, n_experts=None, **kw):
    import ek_b200
    return ek_b200.BackendConfig(
        hidden=cfg.hidden, intermediate=cfg.intermediate, n_experts=n_experts or cfg.n_experts,
        top_k=cfg.top_k, scoring=cfg.scoring, n_group=cfg.n_group, topk_group=cfg.topk_group,
        norm_topk_prob=cfg.norm_topk_prob, routed_scaling=cfg.routed_scaling,
        n_shared_experts=cfg.n_shared, bf16_combine=cfg.bf16_combine, quant=quant_code(cfg.quant),
        max_tokens=max_tokens, max_layers=kw.pop("max_layers", 2), model_name=kw.pop("model_name", "model"), **kw)


def register_layer(be, layer_idx: int, layer: dict, device=None):
    """Registers router, experts and shared expert of an oracle layer with the names the
    weight server uses."""
    from ek_b200.backend import expert_tensors

    def mv(t):
        return t if device is None or t is None else t.to(device)

    be.register_router(layer_idx, mv(layer["wg"]), mv(layer["bias"]))
    for e, w in enumerate(layer["experts"]):
        be.register_expert(be.expert_id(layer_idx, e),
                           expert_tensors(layer_idx, e, mv(w.up), mv(w.gate), mv(w.down), mv(w.up_s), mv(w.gate_s),
                                          mv(w.down_s)))
    if layer.get("shared") is not None:
        w = layer["shared"]
        be.register_expert(be.shared_id(layer_idx),
                           expert_tensors(layer_idx, None, mv(w.up), mv(w.gate), mv(w.down), mv(w.up_s),
                                          mv(w.gate_s), mv(w.down_s), shared=True))


def load_golden(name: str):
    path = os.path.join(GOLDEN, name + ".safetensors")
    t = load_file(path)
    with safe_open(path, "pt") as f:
        meta = f.metadata()
    return t, meta


def golden_experts(t, layer: int, n: int):
    pre = f"model.layers.{layer}.mlp.experts."
    return [O.ExpertWeights(t[f"{pre}{e}.up_proj.weight"], t[f"{pre}{e}.gate_proj.weight"],
                            t[f"{pre}{e}.down_proj.weight"]) for e in range(n)]


def golden_shared(t, layer: int):
    pre = f"model.layers.{layer}.mlp.shared_experts."
    return O.ExpertWeights(t[pre + "up_proj.weight"], t[pre + "gate_proj.weight"], t[pre + "down_proj.weight"])


def build_host_shim(tmpdir) -> str:
    """Compiles tests/host_shim/worker_threads.cpp (the C++ mirror of the worker driving the C ABI)
    against the in-tree library; returns the binary's path."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lib_dir = os.path.join(root, "expert-kit_b200", "lib")
    out = os.path.join(str(tmpdir), "worker_threads")
    cmd = ["g++", "-std=c++17", "-O2", "-Wall", "-Werror", "-I", os.path.join(root, "include"),
           os.path.join(root, "tests", "host_shim", "worker_threads.cpp"), "-o", out,
           "-L", lib_dir, "-lek_b200", "-Wl,-rpath," + lib_dir, "-pthread"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return out
