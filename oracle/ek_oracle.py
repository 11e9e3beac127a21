"""CPU oracle for the Expert Kit MoE expert-layer path.  TEST INFRASTRUCTURE ONLY.

This module restates, on CPU with the same ATen operators the reference issues
through `tch`/PyTorch, the arithmetic of the one path the CUDA backend replaces.
Nothing in the shipped package may import it: only `tests/`, the smoke check and
the CPU-baseline leg of the benchmark do, and only as the checker.

PARITY STATUS: partially pinned.  The reference's own known-answer files
(`ek-computation/resources/qwen3-l0e1.*.safetensors`,
`ek-computation/resources/w8a16active-l0q_a_proj.safetensors`,
`ek-db/resources/ds-tiny/*`) are Git-LFS pointers without data, so none of them
can be checked.  What IS pinned: the softmax routing, per-expert FFN and
weighted combine are checked against outputs of the reference's own Python
module `expertkit_torch/models/qwen3_moe.py` (its local `normal_forward` path)
and the DeepSeek-V3 expert loop / shared expert against
`expertkit_torch/models/deepseek_v3/model.py` (`moe`, `forward`), both executed
in the build container by `tests/golden/make_golden.py`; the fixtures it wrote
are committed under `tests/golden/`.  The sigmoid group-limited router lives in
the third-party `transformers` package (pinned 4.51.3 by the reference,
`uv.lock:2603`); it is restated here from its published behaviour and compared
with the installed `transformers` as a second opinion only.  The Rust worker
(`ek-computation/src/ffn/expert_torch.rs`) cannot be built (no Rust toolchain):
its FFN values are unpinned beyond the Python cross-check.

Each function cites the reference file:line it follows.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

SCORE_SOFTMAX = 0
SCORE_SIGMOID = 1


@dataclass
class MoEConfig:
    """Compute-relevant configuration of one MoE layer (reference: `inference.*`
    in ek-base/src/config.rs:26-31 plus the HF model config read by
    expertkit_torch/models/*)."""
    hidden: int
    intermediate: int
    n_experts: int
    top_k: int
    scoring: int = SCORE_SOFTMAX
    n_group: int = 1
    topk_group: int = 1
    norm_topk_prob: bool = True
    routed_scaling: float = 1.0
    n_shared: int = 0
    # 0: fp32 routing weights in the combine (DeepSeek-V3); 1: bf16 (Qwen3)
    bf16_combine: bool = False
    quant: str = "bf16"          # "bf16" | "fp8" | "int8"


# ----------------------------------------------------------------------------
# canonical top-k: descending score, ties -> lower index
# ----------------------------------------------------------------------------
def canonical_topk(scores: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """`torch.topk` leaves the order of equal values (and, with sorted=False,
    of everything) implementation-defined; parity is defined on the canonical
    order "descending score, ties broken towards the lower index"."""
    vals, idx = torch.sort(scores, dim=-1, descending=True, stable=True)
    return vals[..., :k].contiguous(), idx[..., :k].contiguous()


# ----------------------------------------------------------------------------
# routing
# ----------------------------------------------------------------------------
def router_logits_softmax(x: torch.Tensor, wg: torch.Tensor) -> torch.Tensor:
    """expertkit_torch/models/qwen3_moe.py:161 -- `self.gate(hidden_states)`,
    an `nn.Linear` without bias evaluated in the activation dtype (bf16)."""
    return F.linear(x, wg.to(x.dtype))


def route_softmax(logits: torch.Tensor, k: int, norm: bool,
                  out_dtype=torch.bfloat16) -> Tuple[torch.Tensor, torch.Tensor]:
    """expertkit_torch/models/qwen3_moe.py:162-169: fp32 softmax over experts,
    top-k, optional renormalisation, cast to the activation dtype."""
    p = F.softmax(logits, dim=1, dtype=torch.float)
    w, ids = canonical_topk(p, k)
    if norm:
        w = w / w.sum(dim=-1, keepdim=True)
    return ids.to(torch.int32), w.to(out_dtype)


def router_logits_sigmoid(x: torch.Tensor, wg: torch.Tensor) -> torch.Tensor:
    """Call site expertkit_torch/models/deepseek_v3/model.py:56,142; the router
    (third-party `transformers` DeepseekV3TopkRouter) upcasts activations and
    weight to fp32 before the linear."""
    return F.linear(x.to(torch.float32), wg.to(torch.float32))


def route_sigmoid_grouped(logits: torch.Tensor, bias: Optional[torch.Tensor], k: int,
                          n_group: int, topk_group: int, norm: bool,
                          scaling: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Group-limited sigmoid routing as used through model.py:142.

    s = sigmoid(logits); c = s + bias; a group's score is the sum of its two
    largest c; the best `topk_group` groups stay, all other c become 0.0; the
    k largest remaining c are selected; the routing weight is the UNBIASED s of
    the selected experts, renormalised with a 1e-20 guard and multiplied by the
    routed scaling factor.  Weights stay fp32."""
    T, E = logits.shape
    s = torch.sigmoid(logits.to(torch.float32))
    c = s if bias is None else s + bias.to(torch.float32)
    if n_group > 1:
        per = E // n_group
        g = c.view(T, n_group, per)
        top2, _ = canonical_topk(g, 2)
        gscore = top2.sum(dim=-1)
        _, gidx = canonical_topk(gscore, topk_group)
        gmask = torch.zeros_like(gscore)
        gmask.scatter_(1, gidx, 1.0)
        emask = gmask.unsqueeze(-1).expand(T, n_group, per).reshape(T, E)
        c = c.masked_fill(~emask.bool(), 0.0)
    _, ids = canonical_topk(c, k)
    w = s.gather(1, ids)
    if norm:
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    w = w * scaling
    return ids.to(torch.int32), w


def route(cfg: MoEConfig, x: torch.Tensor, wg: torch.Tensor,
          bias: Optional[torch.Tensor] = None):
    """Returns (logits, ids int32 [T,k], weights [T,k])."""
    if cfg.scoring == SCORE_SOFTMAX:
        logits = router_logits_softmax(x, wg)
        ids, w = route_softmax(logits, cfg.top_k, cfg.norm_topk_prob,
                               torch.bfloat16 if cfg.bf16_combine else torch.float32)
    else:
        logits = router_logits_sigmoid(x, wg)
        ids, w = route_sigmoid_grouped(logits, bias, cfg.top_k, cfg.n_group,
                                       cfg.topk_group, cfg.norm_topk_prob,
                                       cfg.routed_scaling)
    return logits, ids, w


# ----------------------------------------------------------------------------
# bucketing / permutation
# ----------------------------------------------------------------------------
def bucket(ids: torch.Tensor, n_experts: int):
    """ek-computation/src/controller/executor.rs:283-299 (`break_down_to_egress`)
    walks tokens in ascending order and appends (token, slot) to the list of the
    named expert, so rows of one expert are in ascending token order
    (`assemble_seq_tensors`, executor.rs:112-133 gathers them in that order).
    Equivalent to a stable counting sort of the flattened [T*k] assignments by
    expert index.  Returns counts[E], offsets[E+1], perm[T*k] with
    perm[offsets[e]+r] = flat index (token*k+slot) of the r-th row of expert e."""
    flat = ids.reshape(-1).to(torch.int64)
    counts = torch.bincount(flat, minlength=n_experts).to(torch.int32)
    offsets = torch.zeros(n_experts + 1, dtype=torch.int32)
    offsets[1:] = torch.cumsum(counts, 0)
    perm = torch.sort(flat, stable=True)[1].to(torch.int32)
    return counts, offsets, perm


# ----------------------------------------------------------------------------
# block dequantisation
# ----------------------------------------------------------------------------
def w8a16_activate(wq: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    """ek-computation/src/ffn/expert_torch.rs:24-53: view the [m*B, n*B] payload
    as m x n blocks of B x B, upcast to fp32, multiply each block by its fp32
    scale, round to bf16, restore the shape."""
    m, n = scale.shape
    rows, cols = wq.shape
    assert rows == m * block and cols == n * block
    blocks = (wq.reshape(m, block, n, block).permute(0, 2, 1, 3)
              .reshape(m, n, block * block).to(torch.float32))
    out = (blocks * scale.reshape(m, n, 1).to(torch.float32)).to(torch.bfloat16)
    return out.reshape(m, n, block, block).permute(0, 2, 1, 3).reshape(rows, cols)


# ----------------------------------------------------------------------------
# expert FFN
# ----------------------------------------------------------------------------
def expert_ffn(x: torch.Tensor, up_w: torch.Tensor, gate_w: torch.Tensor,
               down_w: torch.Tensor) -> torch.Tensor:
    """ek-computation/src/ffn/expert_torch.rs:61-85: weights cast to bf16 once,
    then `up = x @ W1^T; gate = x @ W3^T; hidden = up * silu(gate);
    out = hidden @ W2^T`, every tensor bf16 (w1 = up, w3 = gate, w2 = down)."""
    w1 = up_w.to(torch.bfloat16)
    w2 = down_w.to(torch.bfloat16)
    w3 = gate_w.to(torch.bfloat16)
    x = x.to(torch.bfloat16)
    up = x.matmul(w1.transpose(0, 1))
    gate = x.matmul(w3.transpose(0, 1))
    hidden = up * F.silu(gate)
    return hidden.matmul(w2.transpose(0, 1))


@dataclass
class ExpertWeights:
    """One expert as delivered by the weight server
    (ek-db/src/safetensor/transformer.rs:249-296): `{gate,up,down}_proj.weight`
    plus `*_scale_inv` when quantised."""
    up: torch.Tensor
    gate: torch.Tensor
    down: torch.Tensor
    up_s: Optional[torch.Tensor] = None
    gate_s: Optional[torch.Tensor] = None
    down_s: Optional[torch.Tensor] = None

    def bf16(self):
        """What `load_module` holds after its one-time cast; for quantised
        payloads the cast is preceded by `w8a16_activate`."""
        if self.up_s is None:
            return (self.up.to(torch.bfloat16), self.gate.to(torch.bfloat16),
                    self.down.to(torch.bfloat16))
        return (w8a16_activate(self.up, self.up_s), w8a16_activate(self.gate, self.gate_s),
                w8a16_activate(self.down, self.down_s))


def moe_expert_outputs(x: torch.Tensor, ids: torch.Tensor, experts) -> torch.Tensor:
    """Controller semantics, ek-computation/src/controller/executor.rs:141-251:
    for every distinct expert gather its rows (ascending token order), run the
    expert, scatter row r back to result[token][slot]; stack to [T,k,H] in the
    request's slot order.  `experts[e]` is an ExpertWeights or a callable."""
    T, k = ids.shape
    H = x.shape[1]
    out = torch.zeros(T, k, H, dtype=torch.bfloat16)
    E = len(experts)
    counts, offsets, perm = bucket(ids, E)
    for e in range(E):
        n = int(counts[e])
        if n == 0:
            continue
        flat = perm[int(offsets[e]):int(offsets[e]) + n].to(torch.int64)
        tok = flat // k
        slot = flat % k
        xe = x[tok]
        ex = experts[e]
        if callable(ex):
            ye = ex(xe)
        else:
            up, gate, down = ex.bf16()
            ye = expert_ffn(xe, up, gate, down)
        out[tok, slot] = ye.to(torch.bfloat16)
    return out


# ----------------------------------------------------------------------------
# combine
# ----------------------------------------------------------------------------
def combine(outputs: torch.Tensor, w: torch.Tensor, bf16_combine: bool) -> torch.Tensor:
    """DeepSeek-V3 (expertkit_torch/models/deepseek_v3/model.py:96-104): fp32
    routing weights broadcast-multiplied with the bf16 [T,k,H] outputs (type
    promotion to fp32), `torch.sum(dim=1)`, cast to bf16.  Qwen3
    (expertkit_torch/models/qwen3_moe.py:102-104): weights already bf16, so the
    product and the sum are bf16 tensors."""
    if bf16_combine:
        ww = w.to(torch.bfloat16).unsqueeze(-1)
        return torch.sum(ww * outputs.to(torch.bfloat16), dim=1)
    ww = w.to(torch.float32).unsqueeze(-1)
    return torch.sum(ww * outputs.to(torch.bfloat16), dim=1).to(torch.bfloat16)


def moe_layer(cfg: MoEConfig, x: torch.Tensor, wg: torch.Tensor, bias, experts,
              shared: Optional[ExpertWeights] = None):
    """The whole layer as the reference splits it between frontend, controller
    and worker: route (frontend) -> per-expert FFN (controller + worker) ->
    weighted combine (frontend) -> + shared expert (model.py:152).
    Returns dict with every intermediate the parity tests compare."""
    logits, ids, w = route(cfg, x, wg, bias)
    counts, offsets, perm = bucket(ids, cfg.n_experts)
    outs = moe_expert_outputs(x, ids, experts)
    y = combine(outs, w, cfg.bf16_combine)
    if shared is not None:
        up, gate, down = shared.bf16()
        y = y + expert_ffn(x, up, gate, down)
    return dict(logits=logits, ids=ids, weights=w, counts=counts, offsets=offsets,
                perm=perm, expert_out=outs, y=y)
