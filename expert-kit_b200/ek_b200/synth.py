"""Seeded synthetic MoE layers, generated on the device.

Checkpoints are not available offline, so benchmarks and full-size self-checks use layers of the
published shapes with random weights: router and expert matrices ~N(0, 0.02), fp8 payloads by
per-128x128-block absmax quantisation (scale_inv = max|w| / 448) under the tensor names the weight
server emits (ek-db/src/safetensor/transformer.rs:249-280).

Every tensor depends only on (seed, layer, expert): any single expert can be generated again later
-- on another rank, or to hand its bytes to a checker -- without generating the ones before it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Iterable, Optional

import torch

from .backend import Backend, BackendConfig, expert_tensors

FP8_MAX = 448.0


@dataclass
class LayerShape:
    """Shape and routing rule of one benchmark layer."""
    name: str
    hidden: int
    intermediate: int
    n_experts: int
    top_k: int
    scoring: int            # 0 softmax, 1 sigmoid
    n_group: int = 1
    topk_group: int = 1
    routed_scaling: float = 1.0
    n_shared: int = 0
    bf16_combine: bool = False
    quant: int = 0          # 0 bf16, 1 fp8 block, 2 int8 block
    zipf_s: float = 0.0     # > 0: router logits carry a Zipf(s) expert-popularity offset

    def backend_config(self, max_tokens: int, device: int, ep_rank: int = 0, ep_size: int = 1,
                       max_layers: int = 1, n_experts: Optional[int] = None) -> BackendConfig:
        return BackendConfig(hidden=self.hidden, intermediate=self.intermediate,
                             n_experts=n_experts or self.n_experts, top_k=self.top_k, scoring=self.scoring,
                             n_group=self.n_group, topk_group=self.topk_group, norm_topk_prob=True,
                             routed_scaling=self.routed_scaling, n_shared_experts=self.n_shared,
                             bf16_combine=self.bf16_combine, quant=self.quant, max_tokens=max_tokens,
                             max_layers=max_layers, device=device, ep_rank=ep_rank, ep_size=ep_size,
                             model_name=self.name)


# DeepSeek-V3 MoE layer, W8A16: fp8 e4m3 weights with 128x128 fp32 block scales
DSV3 = LayerShape("dsv3", 7168, 2048, 256, 8, scoring=1, n_group=8, topk_group=4, routed_scaling=2.5,
                  n_shared=1, bf16_combine=False, quant=1)
# Qwen3-30B-A3B MoE layer, bf16 weights, Zipf(1.1)-skewed expert load
QWEN3 = LayerShape("qwen3", 2048, 768, 128, 8, scoring=0, n_shared=0, bf16_combine=True, quant=0, zipf_s=1.1)

ZIPF_MU = 0.05   # mean of the activations along the popularity direction


def _gen(dev: torch.device, *key: int) -> torch.Generator:
    seed = 0x9E3779B97F4A7C15
    for k in key:
        seed = (seed ^ (int(k) + 0x632BE59BD9B4E019)) * 0xD6E8FEB86659FD93 % (1 << 63)
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    return g


def quantize_fp8_block(w: torch.Tensor):
    r, c = w.shape
    b = w.view(r // 128, 128, c // 128, 128)
    amax = b.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    s = (amax / FP8_MAX).float()
    q = (b / s[:, None, :, None]).to(torch.float8_e4m3fn).view(r, c)
    return q.contiguous(), s.contiguous()


def quantize_int8_block(w: torch.Tensor):
    r, c = w.shape
    b = w.view(r // 128, 128, c // 128, 128)
    amax = b.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    s = (amax / 127.0).float()
    q = torch.round(b / s[:, None, :, None]).clamp(-127, 127).to(torch.int8).view(r, c)
    return q.contiguous(), s.contiguous()


def make_router(shape: LayerShape, dev: torch.device, seed: int, layer: int, n_experts: Optional[int] = None):
    """(router weight [E,H] bf16, popularity direction [H] or None).  With `zipf_s` the weight
    carries a rank-dependent offset log(rank^-s) along a fixed +-1 direction u; inputs made by
    `make_tokens` have a small mean along u, so expert load follows a Zipf law while the router
    stays a bias-free linear map."""
    E = n_experts or shape.n_experts
    g = _gen(dev, seed, layer, 1 << 20)
    wg = torch.randn(E, shape.hidden, generator=g, device=dev) * 0.02
    u = None
    if shape.zipf_s > 0:
        u = torch.randint(0, 2, (shape.hidden,), generator=g, device=dev).float() * 2 - 1
        rank = torch.randperm(E, generator=g, device=dev).float() + 1.0
        off = -shape.zipf_s * torch.log(rank)
        wg = wg + off[:, None] * u[None, :] / (ZIPF_MU * shape.hidden)
    return wg.to(torch.bfloat16), u


def make_tokens(shape: LayerShape, dev: torch.device, seed: int, T: int, u: Optional[torch.Tensor] = None):
    g = _gen(dev, seed, T, 1 << 21)
    x = torch.randn(T, shape.hidden, generator=g, device=dev)
    if u is not None:
        x = x + ZIPF_MU * u[None, :]
    return x.to(torch.bfloat16)


def make_expert(shape: LayerShape, dev: torch.device, seed: int, layer: int, expert: int) -> Dict[str, torch.Tensor]:
    """One expert's tensors under the weight server's names; `expert` = -1 is the shared expert
    (intermediate = n_shared * intermediate)."""
    H = shape.hidden
    I = shape.intermediate * (shape.n_shared if expert < 0 else 1)
    g = _gen(dev, seed, layer, expert + 1)
    mats = [torch.randn(s, generator=g, device=dev) * 0.02 for s in ((I, H), (I, H), (H, I))]   # up, gate, down
    if shape.quant == 0:
        up, gate, down = (m.to(torch.bfloat16) for m in mats)
        return expert_tensors(layer, None if expert < 0 else expert, up, gate, down, shared=expert < 0)
    qf = quantize_fp8_block if shape.quant == 1 else quantize_int8_block
    (up, us), (gate, gs), (down, ds) = (qf(m) for m in mats)
    return expert_tensors(layer, None if expert < 0 else expert, up, gate, down, us, gs, ds, shared=expert < 0)


def build_backend(shape: LayerShape, max_tokens: int, seed: int, dev: Optional[torch.device] = None,
                  ep_rank: int = 0, ep_size: int = 1, n_layers: int = 1, n_experts: Optional[int] = None,
                  experts: Optional[Iterable[int]] = None):
    """A backend holding `n_layers` synthetic layers: the router (same on every rank), the shared
    expert and the routed experts this rank owns (or the explicit list `experts`).
    Returns (backend, {layer: popularity direction})."""
    dev = dev or torch.device("cuda", torch.cuda.current_device())
    E = n_experts or shape.n_experts
    be = Backend(shape.backend_config(max_tokens, dev.index, ep_rank, ep_size, n_layers, E))
    el = E // ep_size
    mine = list(experts) if experts is not None else list(range(ep_rank * el, (ep_rank + 1) * el))
    dirs = {}
    for layer in range(n_layers):
        wg, u = make_router(shape, dev, seed, layer, E)
        dirs[layer] = u
        be.register_router(layer, wg, torch.zeros(E, device=dev) if shape.scoring == 1 else None)
        for e in mine:
            be.register_expert(be.expert_id(layer, e), make_expert(shape, dev, seed, layer, e))
        if shape.n_shared > 0:
            be.register_expert(be.shared_id(layer), make_expert(shape, dev, seed, layer, -1))
    return be, dirs
