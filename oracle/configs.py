"""Seeded synthetic layers and inputs for the benchmark configurations.
TEST INFRASTRUCTURE ONLY (see ek_oracle.py).

Real checkpoints are not available offline, so every configuration is
reproduced by shape, dtype and value distribution from a fixed seed:
weights ~N(0, 0.02), activations ~N(0, 1), fp8 payloads obtained by
per-128x128-block absmax quantisation (scale_inv = max|w| / 448), stored under
the tensor names the weight server emits
(ek-db/src/safetensor/transformer.rs:249-280).
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch

from .ek_oracle import MoEConfig, ExpertWeights, SCORE_SIGMOID, SCORE_SOFTMAX

FP8_MAX = 448.0
BLOCK = 128


def config(cfg_id: int) -> MoEConfig:
    if cfg_id == 1:   # tiny DeepSeek-V3 structure, bf16
        return MoEConfig(hidden=1024, intermediate=256, n_experts=16, top_k=4,
                         scoring=SCORE_SIGMOID, n_group=1, topk_group=1,
                         norm_topk_prob=True, routed_scaling=1.0, n_shared=1,
                         bf16_combine=False, quant="bf16")
    if cfg_id == 2:   # Qwen3-30B-A3B shape, bf16
        return MoEConfig(hidden=2048, intermediate=768, n_experts=128, top_k=8,
                         scoring=SCORE_SOFTMAX, norm_topk_prob=True, n_shared=0,
                         bf16_combine=True, quant="bf16")
    if cfg_id == 3:   # DeepSeek-V3 shape, fp8 block-scaled weights
        return MoEConfig(hidden=7168, intermediate=2048, n_experts=256, top_k=8,
                         scoring=SCORE_SIGMOID, n_group=8, topk_group=4,
                         norm_topk_prob=True, routed_scaling=2.5, n_shared=1,
                         bf16_combine=False, quant="fp8")
    raise ValueError(cfg_id)


def seed_for(cfg_id: int, case: int) -> int:
    return 1000 * cfg_id + case


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(seed)
    return g


def quantize_fp8_block(w: torch.Tensor):
    """Per 128x128 block absmax quantisation to e4m3 with an fp32 inverse scale."""
    rows, cols = w.shape
    m, n = rows // BLOCK, cols // BLOCK
    blocks = w.reshape(m, BLOCK, n, BLOCK).permute(0, 2, 1, 3)
    amax = blocks.abs().amax(dim=(2, 3)).clamp_min(1e-12)
    scale_inv = (amax / FP8_MAX).to(torch.float32)
    q = (blocks / scale_inv[:, :, None, None]).to(torch.float8_e4m3fn)
    q = q.permute(0, 2, 1, 3).reshape(rows, cols).contiguous()
    return q, scale_inv.contiguous()


def quantize_int8_block(w: torch.Tensor):
    rows, cols = w.shape
    m, n = rows // BLOCK, cols // BLOCK
    blocks = w.reshape(m, BLOCK, n, BLOCK).permute(0, 2, 1, 3)
    amax = blocks.abs().amax(dim=(2, 3)).clamp_min(1e-12)
    scale = (amax / 127.0).to(torch.float32)
    q = torch.round(blocks / scale[:, :, None, None]).clamp(-127, 127).to(torch.int8)
    q = q.permute(0, 2, 1, 3).reshape(rows, cols).contiguous()
    return q, scale.contiguous()


def make_expert(hidden: int, inter: int, quant: str, g: torch.Generator,
                std: float = 0.02) -> ExpertWeights:
    up = torch.randn(inter, hidden, generator=g) * std
    gate = torch.randn(inter, hidden, generator=g) * std
    down = torch.randn(hidden, inter, generator=g) * std
    if quant == "bf16":
        return ExpertWeights(up.to(torch.bfloat16), gate.to(torch.bfloat16),
                             down.to(torch.bfloat16))
    qf = quantize_fp8_block if quant == "fp8" else quantize_int8_block
    uq, us = qf(up)
    gq, gs = qf(gate)
    dq, ds = qf(down)
    return ExpertWeights(uq, gq, dq, us, gs, ds)


def make_layer(cfg: MoEConfig, seed: int, n_experts: Optional[int] = None,
               zipf_s: float = 0.0):
    """Router weight (bf16 ~N(0,0.02)), zero correction bias, experts and the
    optional shared expert.  With `zipf_s` > 0 the router gets a rank-dependent
    logit offset log(rank^-s) along a fixed +-1 direction `u`; inputs made by
    `make_inputs(..., mean_dir=u)` carry a small mean along `u`, so that expert
    load follows a Zipf law while the router stays a bias-free linear map."""
    g = _gen(seed)
    E = n_experts or cfg.n_experts
    wg = torch.randn(E, cfg.hidden, generator=g) * 0.02
    u = None
    if zipf_s > 0:
        u = (torch.randint(0, 2, (cfg.hidden,), generator=g).float() * 2 - 1)
        rank = torch.randperm(E, generator=g).float() + 1.0
        off = -zipf_s * torch.log(rank)
        wg = wg + off[:, None] * u[None, :] / (ZIPF_MU * cfg.hidden)
    wg = wg.to(torch.bfloat16)
    bias = torch.zeros(E, dtype=torch.float32)
    experts: List[ExpertWeights] = [make_expert(cfg.hidden, cfg.intermediate, cfg.quant, g)
                                    for _ in range(E)]
    shared = None
    if cfg.n_shared > 0:
        shared = make_expert(cfg.hidden, cfg.intermediate * cfg.n_shared, cfg.quant, g)
    return dict(wg=wg, bias=bias, experts=experts, shared=shared, mean_dir=u)


ZIPF_MU = 0.05


def make_inputs(cfg: MoEConfig, T: int, seed: int, mean_dir: Optional[torch.Tensor] = None):
    g = _gen(seed + 7919)
    x = torch.randn(T, cfg.hidden, generator=g)
    if mean_dir is not None:
        x = x + ZIPF_MU * mean_dir[None, :]
    return x.to(torch.bfloat16)


def zipf_ids(T: int, k: int, E: int, s: float, g: torch.Generator,
             cover_all: bool = False, rot: int = 0) -> torch.Tensor:
    """Direct synthetic assignments (controller-level entry point): every token
    draws k distinct experts without replacement from a Zipf(s) law over a
    rotated expert ranking.  With `cover_all`, experts left empty are appended
    to the first tokens' last slots where that keeps a token's experts distinct
    (the continuous-batching configuration demands every expert >= 1 token)."""
    p = torch.arange(1, E + 1, dtype=torch.float64) ** (-s)
    p = p / p.sum()
    order = torch.roll(torch.arange(E), rot)
    ids = torch.multinomial(p.float().expand(T, E), k, replacement=False, generator=g)
    ids = order[ids]
    if cover_all and T * k >= E:
        present = torch.zeros(E, dtype=torch.bool)
        present[ids.reshape(-1)] = True
        missing = [e for e in range(E) if not present[e]]
        t = 0
        cnt = torch.bincount(ids.reshape(-1), minlength=E)
        for e in missing:
            placed = False
            while not placed and t < T * k:
                tok, slot = divmod(t, k)
                old = int(ids[tok, slot])
                if cnt[old] > 1 and e not in ids[tok].tolist():
                    cnt[old] -= 1
                    ids[tok, slot] = e
                    cnt[e] += 1
                    placed = True
                t += 1
    return ids.to(torch.int32)


def algorithmic_bytes(cfg: MoEConfig, T: int, active_experts: int) -> int:
    """Bytes one pass must move at minimum: weights (+ block scales) of every
    expert that received a token and of the shared expert, the router weight,
    activations in and results out."""
    bw = 2 if cfg.quant == "bf16" else 1
    H, I = cfg.hidden, cfg.intermediate
    sc = 0 if cfg.quant == "bf16" else 12 * math.ceil(I / 128) * math.ceil(H / 128)
    per = 3 * H * I * bw + sc
    per_shared = (3 * H * I * cfg.n_shared * bw
                  + (0 if cfg.quant == "bf16" else 12 * math.ceil(I * cfg.n_shared / 128) * math.ceil(H / 128)))
    return active_experts * per + (per_shared if cfg.n_shared else 0) + 2 * H * cfg.n_experts + 4 * T * H


def algorithmic_flops(cfg: MoEConfig, T: int) -> int:
    H, I = cfg.hidden, cfg.intermediate
    return 2 * T * H * cfg.n_experts + 6 * H * I * T * cfg.top_k + 6 * H * I * cfg.n_shared * T
