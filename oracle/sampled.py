"""Full-size layers against the oracle without evaluating every expert on the CPU.
TEST INFRASTRUCTURE ONLY (see ek_oracle.py).

A DeepSeek-V3-shape layer has 257 experts of 44 MB each; the CPU restatement needs seconds per
expert.  Routing, counts, offsets and the permutation need no expert weights, so they are
checked for ALL tokens; the layer output is checked on a handful of tokens, for which only the
experts those tokens use (at most top_k per token, plus the shared expert) are evaluated with
`ek_oracle.expert_ffn` in the reference's operator order
(expertkit_torch/models/deepseek_v3/model.py:90-106,139-153;
ek-computation/src/ffn/expert_torch.rs:61-85).
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch

from . import ek_oracle as O


def expert_from_named(t: Dict[str, torch.Tensor]) -> O.ExpertWeights:
    """Picks gate/up/down (+ scales) out of a bundle by the reference's suffix rule
    (ek-computation/src/ffn/meta.rs:57-75)."""
    def pick(suffix):
        for k, v in t.items():
            if k.endswith(suffix):
                return v.cpu()
        return None
    return O.ExpertWeights(pick("up_proj.weight"), pick("gate_proj.weight"), pick("down_proj.weight"),
                           pick("up_proj.weight_scale_inv"), pick("gate_proj.weight_scale_inv"),
                           pick("down_proj.weight_scale_inv"))


def logits_noise(cfg: O.MoEConfig, ref_logits: torch.Tensor) -> torch.Tensor:
    """How far two correct evaluations of the router's linear layer may lie apart, per element:
    one bf16 last place for the softmax router (its linear layer runs in bf16, so two fp32
    summation orders can round to neighbouring bf16 values), 1e-5 absolute for the fp32 sums of
    the sigmoid router (H terms of magnitude ~1e-2 added in another order)."""
    a = ref_logits.float().abs()
    if cfg.scoring == O.SCORE_SOFTMAX:
        return torch.maximum(a, torch.tensor(2.0 ** -126)) * 2.0 ** -7
    return torch.full_like(a, 1e-5)


def check_routing(cfg: O.MoEConfig, x: torch.Tensor, wg: torch.Tensor, bias: Optional[torch.Tensor],
                  got: Dict[str, torch.Tensor]) -> Dict:
    """`got`: ids [T,k], weights [T,k] and, when available, logits [T,E], counts, offsets, perm as the
    CUDA path produced them (host tensors).  Three statements:
      * given ITS logits, the CUDA routing equals the oracle's bit for bit (all tokens);
      * counts / offsets / perm equal the oracle's stable counting sort of those ids (all tokens);
      * against the oracle's own logits, the tokens whose ids differ are counted, and each of them
        must be a near-tie: its logits agree with the oracle's within `logits_noise`, and the
        experts (or groups) that changed places are ones the oracle itself scores that close."""
    ref_logits, ref_ids, ref_w = O.route(cfg, x, wg, bias)
    E, k = cfg.n_experts, cfg.top_k
    out = dict(tokens=int(x.shape[0]))
    ids = got["ids"].to(torch.int32)
    differ = (ids != ref_ids).any(1)
    out["ids_differ"] = int(differ.sum())
    out["ids_equal"] = out["ids_differ"] == 0
    if got.get("logits") is not None:
        lg = got["logits"].float()
        if cfg.scoring == O.SCORE_SOFTMAX:
            ids2, w2 = O.route_softmax(lg.to(torch.bfloat16), k, cfg.norm_topk_prob,
                                       torch.bfloat16 if cfg.bf16_combine else torch.float32)
        else:
            ids2, w2 = O.route_sigmoid_grouped(lg, bias, k, cfg.n_group, cfg.topk_group, cfg.norm_topk_prob,
                                               cfg.routed_scaling)
        out["exact_given_logits"] = bool(torch.equal(ids, ids2))
        noise = logits_noise(cfg, ref_logits)
        dl = (lg - ref_logits.float()).abs()
        out["logits_max_noise_units"] = float((dl / noise).max())
        # every differing token must come with logits that agree within that noise ...
        out["differ_unexplained"] = int((differ & ((dl / noise).amax(1) > 2.0)).sum()) if differ.any() else 0
        # ... and must be a swap between experts (or, with group-limited routing, groups) that the
        # oracle itself scores closer together than twice the noise
        bad = 0
        if differ.any():
            if cfg.scoring == O.SCORE_SOFTMAX:
                choice, cn = ref_logits.float(), noise
            else:   # selection runs on sigmoid(l) + bias; d sigmoid / dl <= 1/4
                choice = torch.sigmoid(ref_logits.float()) + (0 if bias is None else bias.float())
                cn = noise * 0.25
            for t in differ.nonzero().flatten().tolist():
                a, b = ids[t].tolist(), ref_ids[t].tolist()
                only_got, only_ref = sorted(set(a) - set(b)), sorted(set(b) - set(a))
                if not only_got:        # same set, two neighbours in another order
                    pairs = [(a[i], b[i]) for i in range(k) if a[i] != b[i]]
                elif cfg.n_group > 1 and len(only_got) > 1:
                    continue            # a near-tie between two groups swaps several experts at once
                else:
                    pairs = list(zip(only_got, only_ref))
                    if len(pairs) > 1:
                        bad += 1
                        continue
                for ea, eb in pairs:
                    if abs(float(choice[t, ea] - choice[t, eb])) > 4.0 * float(max(cn[t, ea], cn[t, eb])):
                        bad += 1
                        break
        out["differ_not_a_tie_swap"] = bad
    if got.get("counts") is not None:
        c, o, p = O.bucket(ids, E)
        out["bucket_exact"] = bool(torch.equal(got["counts"], c) and torch.equal(got["offsets"], o)
                                   and torch.equal(got["perm"], p))
    same = ~differ
    if same.any() and got.get("weights") is not None:
        rel = ((got["weights"].float() - ref_w.float()).abs() / ref_w.float().abs().clamp_min(1e-12))[same]
        out["weights_max_rel"] = float(rel.max())
    out["_ref"] = dict(ids=ref_ids, weights=ref_w, same=same)
    return out


def check_outputs_sampled(cfg: O.MoEConfig, x: torch.Tensor, y: torch.Tensor, routing: Dict,
                          fetch_expert: Callable[[int], O.ExpertWeights], n_tokens: int = 4) -> Dict:
    """Evaluates the oracle on `n_tokens` tokens spread over the batch (among those routed
    identically) and compares with rows of the CUDA result `y`.  `fetch_expert(e)` returns expert
    e's weights as delivered to the backend; e = -1 is the shared expert."""
    ref = routing["_ref"]
    cand = ref["same"].nonzero().flatten()
    if cand.numel() == 0:
        return dict(tokens_checked=0)
    pick = cand[torch.linspace(0, cand.numel() - 1, min(n_tokens, cand.numel())).round().long()].unique()
    xs = x[pick]
    ids = ref["ids"][pick]
    cache: Dict[int, object] = {}

    def run(e):
        if e not in cache:
            up, gate, down = fetch_expert(e).bf16()
            cache[e] = lambda rows, up=up, gate=gate, down=down: O.expert_ffn(rows, up, gate, down)
        return cache[e]

    experts = [None] * cfg.n_experts
    for e in ids.unique().tolist():
        experts[e] = run(e)
    outs = O.moe_expert_outputs(xs, ids, experts)
    yr = O.combine(outs, ref["weights"][pick], cfg.bf16_combine)
    if cfg.n_shared > 0:
        yr = yr + run(-1)(xs)
    g, r = y[pick].float().cpu(), yr.float()
    d = (g - r).abs()
    return dict(tokens_checked=int(pick.numel()), experts_evaluated=len(cache),
                max_rel=float(d.max() / r.abs().max().clamp_min(1e-6)), mean_abs=float(d.mean()),
                mean_ref=float(r.abs().mean()), tokens=pick.tolist())
