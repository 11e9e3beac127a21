"""Modules with the call shapes of the reference's vLLM integration, served by the local backend.

The reference offers two modes (expertkit_vllm/plugin.py:12-43):

* expert mode swaps vLLM's `FusedMoE` for `GrpcExpert`
  (expertkit_vllm/experts/grpc_expert.py:11-210): `forward(hidden_states, router_logits)` picks
  top-k experts from the router logits vLLM computed, fetches the `[T, k, H]` expert outputs over
  gRPC and sums them with the routing weights;
* moe mode swaps `DeepseekV2MoE` for `ExpertKitMoE`
  (expertkit_vllm/models/deepseek_v2.py:17-228): `forward(hidden_states)` owns the gate, routes,
  fetches the expert outputs and sums them.

`B200GrpcExpert` and `B200ExpertKitMoE` keep those signatures; routing, bucketing, the grouped
expert FFNs and the weighted combine run as this library's kernels on device buffers.  Two things
the reference leaves unfinished are done here, as vLLM's own layers do them: the routing weights
are scores (softmax, or sigmoid with the correction bias and group-limited selection,
renormalised) rather than raw top-k logits (grpc_expert.py:120-121), and the shared expert's output
is added to the routed one (deepseek_v2.py:228 drops it).  Neither module imports vLLM.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import _lib as L
from .backend import Backend, EKError


def _layer_from_prefix(prefix: str, pos: int) -> int:
    """"model.layers.12.mlp.experts" -> 12 (grpc_expert.py:85-92, pos -3);
    "model.layers.12.mlp" -> 12 (deepseek_v2.py:42-46, pos -2); 0 when the prefix has another form."""
    try:
        return int(prefix.split(".")[pos])
    except (IndexError, ValueError):
        return 0


class B200GrpcExpert(torch.nn.Module):
    """Stand-in for vLLM's `FusedMoE` with `GrpcExpert`'s constructor and
    `forward(hidden_states, router_logits) -> [T, H]`.

    The backend must hold the routed experts of the layer named by `prefix` and be configured with
    the same routing rule as the arguments describe (checked here).  As in vLLM, the result is the
    ROUTED output only: the shared expert and the routed scaling factor stay with the caller
    (`DeepseekV2MoE`), so configure the backend with `routed_scaling = 1.0` for this mode."""

    def __init__(self, num_experts: int, top_k: int, hidden_size: int, intermediate_size: int, prefix: str = "", *,
                 backend: Backend, renormalize: bool = True, use_grouped_topk: bool = False,
                 num_expert_group: Optional[int] = None, topk_group: Optional[int] = None,
                 scoring_func: str = "softmax", e_score_correction_bias: Optional[torch.Tensor] = None,
                 activation: str = "silu", **_unused):
        super().__init__()
        c = backend.cfg
        want = dict(n_experts=num_experts, top_k=top_k, hidden=hidden_size, intermediate=intermediate_size,
                    scoring=L.EK_SCORE_SIGMOID if scoring_func == "sigmoid" else L.EK_SCORE_SOFTMAX,
                    n_group=(num_expert_group or 1) if use_grouped_topk else 1,
                    topk_group=(topk_group or 1) if use_grouped_topk else 1)
        for k, v in want.items():
            if getattr(c, k) != v:
                raise EKError(3, f"backend was created with {k}={getattr(c, k)}, the layer asks for {v}")
        if bool(c.norm_topk_prob) != bool(renormalize):
            raise EKError(3, "backend and layer disagree on renormalising the routing weights")
        if scoring_func not in ("softmax", "sigmoid") or activation != "silu":
            raise EKError(20, "only softmax / sigmoid scoring with SiLU experts is supported")
        self.backend = backend
        self.num_experts, self.top_k, self.hidden_size, self.prefix = num_experts, top_k, hidden_size, prefix
        self.layer_idx = _layer_from_prefix(prefix, -3)
        self.e_score_correction_bias = e_score_correction_bias

    def forward(self, hidden_states: torch.Tensor, router_logits: torch.Tensor) -> torch.Tensor:
        if not hidden_states.is_cuda:
            raise RuntimeError("B200GrpcExpert runs on CUDA tensors only")
        T, H = hidden_states.shape
        be = self.backend
        be.use_torch_stream()
        x = hidden_states.to(torch.bfloat16).contiguous()
        try:
            art = be.route_from_logits_device(router_logits, self.e_score_correction_bias)
            out = be.moe_forward(self.layer_idx, x, art["ids"])            # [T, k, H], the ForwardResp payload
            y = be.combine(out, art["weights"], None)
        except EKError as e:
            raise RuntimeError(f"expert forward failed: {e}") from e      # the gRPC client raises RuntimeError too
        return y.view(T, H).to(hidden_states.dtype)


class B200ExpertKitMoE(torch.nn.Module):
    """Stand-in for `DeepseekV2MoE` with `ExpertKitMoE`'s constructor shape
    (`config`, `quant_config`, `prefix`) and `forward(hidden_states) -> [T, H]`.

    `config` needs the fields the reference reads (deepseek_v2.py:35-90): `hidden_size`,
    `n_routed_experts`, `num_experts_per_tok`, `norm_topk_prob`, `n_shared_experts`,
    `routed_scaling_factor`.  The gate weight, the correction bias, the experts and the shared
    expert of the layer live in the backend (registered from the weight server's bundles), so the
    module itself holds no parameters.  One fused call: router, group-limited top-k, bucketing,
    expert FFNs, weighted combine with the scaling factor, plus the shared expert."""

    def __init__(self, config, quant_config=None, prefix: str = "", *, backend: Backend):
        super().__init__()
        c = backend.cfg
        checks = (("hidden_size", c.hidden), ("n_routed_experts", c.n_experts), ("num_experts_per_tok", c.top_k))
        for name, have in checks:
            if getattr(config, name) != have:
                raise EKError(3, f"config.{name}={getattr(config, name)} but the backend was created with {have}")
        if bool(getattr(config, "norm_topk_prob", True)) != bool(c.norm_topk_prob):
            raise EKError(3, "config.norm_topk_prob disagrees with the backend")
        if (getattr(config, "n_shared_experts", None) or 0) != c.n_shared_experts:
            raise EKError(3, "config.n_shared_experts disagrees with the backend")
        if abs(float(getattr(config, "routed_scaling_factor", 1.0)) - c.routed_scaling) > 1e-6:
            raise EKError(3, "config.routed_scaling_factor disagrees with the backend")
        self.backend = backend
        self.layer_idx = _layer_from_prefix(prefix, -2)
        self.hidden_size = config.hidden_size
        self.n_routed_experts = config.n_routed_experts
        self.num_experts_per_tok = config.num_experts_per_tok
        self.norm_topk_prob = bool(c.norm_topk_prob)
        self.n_shared_experts = getattr(config, "n_shared_experts", None)
        self.routed_scaling_factor = c.routed_scaling
        self.debug_mode = os.getenv("EXPERTKIT_DEBUG_MODE", "0") == "1"

    def forward(self, hidden_states: torch.Tensor) -> torch.Tensor:
        if not hidden_states.is_cuda:
            raise RuntimeError("B200ExpertKitMoE runs on CUDA tensors only")
        T, H = hidden_states.shape
        x = hidden_states.reshape(-1, H).to(torch.bfloat16).contiguous()
        y = torch.empty_like(x)
        self.backend.use_torch_stream()
        try:
            self.backend.moe_forward_fused_async(self.layer_idx, x, y)
        except EKError as e:
            raise RuntimeError(f"expert forward failed: {e}") from e
        return y.view(T, H).to(hidden_states.dtype)

    def check(self):
        """Device-side errors of the asynchronous forward surface here; call once per model forward."""
        self.backend.sync()


def register(backend_for_layer, mode: Optional[str] = None):
    """The reference's plugin hook (expertkit_vllm/plugin.py:12-43) for this backend: when
    EXPERTKIT_ENABLE=1, replaces vLLM's `FusedMoE` (EXPERTKIT_MODE=expert_mode, the default) or
    `DeepseekV2MoE` (moe_mode) with factories that build the modules above around
    `backend_for_layer(prefix) -> Backend`.  Imports vLLM lazily; does nothing unless enabled."""
    if os.getenv("EXPERTKIT_ENABLE") != "1":
        return False
    mode = mode or os.getenv("EXPERTKIT_MODE", "expert_mode")
    if mode == "expert_mode":
        import vllm.model_executor.layers.fused_moe.layer as fused_moe

        def make_expert(num_experts, top_k, hidden_size, intermediate_size, prefix="", *a, **kw):
            kw.pop("backend", None)
            return B200GrpcExpert(num_experts, top_k, hidden_size, intermediate_size, prefix,
                                  backend=backend_for_layer(prefix), **kw)
        fused_moe.FusedMoE = make_expert
    elif mode == "moe_mode":
        import vllm.model_executor.models.deepseek_v2 as ds_v2

        def make_moe(config, quant_config=None, prefix="", **kw):
            return B200ExpertKitMoE(config, quant_config, prefix, backend=backend_for_layer(prefix))
        ds_v2.DeepseekV2MoE = make_moe
    else:
        raise ValueError(f"unknown EXPERTKIT_MODE: {mode}")
    return True
