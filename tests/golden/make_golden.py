"""Generate golden input/output vectors by running the REFERENCE's own Python
modules on CPU.  Run once in a container that has the reference checkout:

    python tests/golden/make_golden.py /path/to/reference

It imports `expertkit_torch/models/qwen3_moe.py` and
`expertkit_torch/models/deepseek_v3/model.py` unmodified, builds their
intercepted MoE blocks with seeded random weights at small sizes and records

  * the local path (`normal_forward` / `moe` + shared expert), and
  * the remote path (`ek_forward` / `ek_moe`) with the gRPC client replaced by
    an in-process stand-in that evaluates the named experts one by one, which
    pins the expert-id string format and the [T,k,H] -> weighted-sum step.

The DeepSeek-V3 router is a third-party class; with the installed
`transformers` its top-k step lives in `DeepseekV3MoE.route_tokens_to_experts`,
which is what the script calls (the reference pins an older release whose
router returned the pair directly; the arithmetic is the same).

The fixtures are written next to this file as `*.safetensors`; the tests read
only those files.
"""
import os
import sys

import torch
from safetensors.torch import save_file

HERE = os.path.dirname(os.path.abspath(__file__))


def _seed_module(mod: torch.nn.Module, seed: int, std: float):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in mod.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * std)


class StubClient:
    """Stands in for ExpertKitClient.forward_expert(expert_ids, hidden_state):
    evaluates the experts named by the id strings and returns [T,k,H]."""

    def __init__(self, experts, prefix):
        self.experts = experts
        self.prefix = prefix
        self.seen_ids = []

    def forward_expert(self, expert_ids, hidden_state):
        T = hidden_state.shape[0]
        k = len(expert_ids[0])
        out = torch.zeros(T, k, hidden_state.shape[1], dtype=hidden_state.dtype)
        for t, ids in enumerate(expert_ids):
            for s, name in enumerate(ids):
                self.seen_ids.append(name)
                model, rest = name.split("/l")
                layer, e = rest.split("-e")
                assert model == self.prefix
                out[t, s] = self.experts[int(e)](hidden_state[t:t + 1])[0]
        return out


def golden_qwen3(ref_root: str):
    sys.path.insert(0, os.path.join(ref_root, "ek-integration", "expertkit_torch"))
    from expertkit_torch.models import qwen3_moe as ref
    from transformers.models.qwen3_moe import modeling_qwen3_moe as hf
    from transformers.models.qwen3_moe.configuration_qwen3_moe import Qwen3MoeConfig

    H, I, E, k, T = 128, 64, 8, 2, 24
    cfg = Qwen3MoeConfig(hidden_size=H, moe_intermediate_size=I, num_experts=E,
                         num_experts_per_tok=k, norm_topk_prob=True, num_hidden_layers=2)
    ref.intercept_moe(enable_ek=False, ek_model_name="qwen3")
    block = hf.Qwen3MoeSparseMoeBlock(cfg)
    _seed_module(block, 2001, 0.05)
    block = block.to(torch.bfloat16)
    g = torch.Generator().manual_seed(2002)
    x = torch.randn(1, T, H, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        y_local, logits = block(x)
        # remote path with the in-process stand-in client
        hs = x.view(-1, H)
        p = torch.nn.functional.softmax(block.gate(hs), dim=1, dtype=torch.float)
        rw, sel = torch.topk(p, k, dim=-1)
        rw = rw / rw.sum(dim=-1, keepdim=True)
        rw = rw.to(hs.dtype)
        stub = StubClient(block.experts, "qwen3")
        block.client = stub
        y_remote = block.ek_forward(hidden_states=hs, routing_weights=rw, selected_experts=sel,
                                    batch_size=1, sequence_length=T, hidden_dim=H)
    t = {
        "x": x.view(T, H).contiguous(),
        "gate.weight": block.gate.weight.detach().contiguous(),
        "router_logits": logits.contiguous(),
        "selected_experts": sel.to(torch.int32).contiguous(),
        "routing_weights": rw.contiguous(),
        "y_local": y_local.view(T, H).contiguous(),
        "y_remote": y_remote.view(T, H).contiguous(),
    }
    for e in range(E):
        m = block.experts[e]
        t[f"model.layers.0.mlp.experts.{e}.gate_proj.weight"] = m.gate_proj.weight.detach().contiguous()
        t[f"model.layers.0.mlp.experts.{e}.up_proj.weight"] = m.up_proj.weight.detach().contiguous()
        t[f"model.layers.0.mlp.experts.{e}.down_proj.weight"] = m.down_proj.weight.detach().contiguous()
    meta = {"hidden": str(H), "intermediate": str(I), "n_experts": str(E), "top_k": str(k),
            "first_id": stub.seen_ids[0], "layer": str(block.layer_id)}
    save_file(t, os.path.join(HERE, "qwen3_tiny.safetensors"), metadata=meta)
    print("qwen3_tiny:", {k_: tuple(v.shape) for k_, v in t.items() if not k_.startswith("model.")}, meta)


def golden_dsv3(ref_root: str):
    from expertkit_torch.models.deepseek_v3 import model as ref
    from transformers.models.deepseek_v3 import modeling_deepseek_v3 as hf
    from transformers.models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3Config

    H, I, E, k, T = 128, 64, 16, 4, 24
    cfg = DeepseekV3Config(hidden_size=H, moe_intermediate_size=I, n_routed_experts=E,
                           num_experts_per_tok=k, n_group=4, topk_group=2, n_shared_experts=1,
                           norm_topk_prob=True, routed_scaling_factor=2.5,
                           num_hidden_layers=4, intermediate_size=4 * I)
    hf_moe_cls = hf.DeepseekV3MoE           # third-party block, kept for its routing step
    ref.intercept_moe(None, "dsv3")          # local mode: experts evaluated in-process
    block = hf.DeepseekV3MoE(cfg)
    _seed_module(block, 3001, 0.05)
    block = block.to(torch.bfloat16)
    router_helper = hf_moe_cls(cfg)
    router_helper.gate = block.gate
    g = torch.Generator().manual_seed(3002)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    with torch.no_grad():
        logits = block.gate(x)
        ids, w = router_helper.route_tokens_to_experts(logits)
        routed_local = block.moe(x, ids, w)
        shared = block.shared_experts(x)
        y_local = routed_local + shared
        stub = StubClient(block.experts, "dsv3")
        block.client = stub
        routed_remote = block.ek_moe(x, ids, w)
        y_remote = routed_remote + shared
    t = {
        "x": x.contiguous(),
        "gate.weight": block.gate.weight.detach().contiguous(),
        "gate.e_score_correction_bias": block.gate.e_score_correction_bias.detach().float().contiguous(),
        "router_logits": logits.contiguous(),
        "topk_indices": ids.to(torch.int32).contiguous(),
        "topk_weights": w.contiguous(),
        "routed_local": routed_local.contiguous(),
        "routed_remote": routed_remote.contiguous(),
        "shared_out": shared.contiguous(),
        "y_local": y_local.contiguous(),
        "y_remote": y_remote.contiguous(),
    }
    for e in range(E):
        m = block.experts[e]
        t[f"model.layers.3.mlp.experts.{e}.gate_proj.weight"] = m.gate_proj.weight.detach().contiguous()
        t[f"model.layers.3.mlp.experts.{e}.up_proj.weight"] = m.up_proj.weight.detach().contiguous()
        t[f"model.layers.3.mlp.experts.{e}.down_proj.weight"] = m.down_proj.weight.detach().contiguous()
    s = block.shared_experts
    t["model.layers.3.mlp.shared_experts.gate_proj.weight"] = s.gate_proj.weight.detach().contiguous()
    t["model.layers.3.mlp.shared_experts.up_proj.weight"] = s.up_proj.weight.detach().contiguous()
    t["model.layers.3.mlp.shared_experts.down_proj.weight"] = s.down_proj.weight.detach().contiguous()
    meta = {"hidden": str(H), "intermediate": str(I), "n_experts": str(E), "top_k": str(k),
            "n_group": "4", "topk_group": "2", "routed_scaling": "2.5",
            "first_id": stub.seen_ids[0], "layer": str(block.layer_id)}
    save_file(t, os.path.join(HERE, "dsv3_tiny.safetensors"), metadata=meta)
    print("dsv3_tiny:", {k_: tuple(v.shape) for k_, v in t.items() if not k_.startswith("model.")}, meta)


if __name__ == "__main__":
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("EK_REFERENCE_ROOT", "")
    if not root or not os.path.isdir(root):
        raise SystemExit("usage: make_golden.py <reference checkout>")
    torch.manual_seed(0)
    torch.set_num_threads(1)
    golden_qwen3(root)
    golden_dsv3(root)
