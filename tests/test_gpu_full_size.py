"""The benchmarked configuration itself against the oracle: the DeepSeek-V3-shape layer with all
256 routed experts (8 groups, top-4 groups, top-8, x2.5), fp8 block-scaled weights, shared expert.

The layer is generated on the device from a seed (11.3 GB of weights: too large to build on the
CPU in a test).  Routing artefacts -- expert ids, routing weights, per-expert counts, offsets and
the permutation -- need no expert weights and are checked against the oracle for ALL tokens; the
layer output is checked on a sample of tokens for which only the experts those tokens use are
copied back and evaluated with the oracle's FFN (oracle/sampled.py).
"""
import pytest
import torch

import helpers as Hh
from oracle import ek_oracle as O
from oracle import sampled as S

pytestmark = pytest.mark.gpu

SEED = 4300


@pytest.fixture(scope="module")
def dsv3_full():
    from ek_b200 import synth
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    be, _ = synth.build_backend(synth.DSV3, 4096, SEED, dev)
    wg, _ = synth.make_router(synth.DSV3, dev, SEED, 0)
    cfg = O.MoEConfig(hidden=7168, intermediate=2048, n_experts=256, top_k=8, scoring=O.SCORE_SIGMOID, n_group=8,
                      topk_group=4, norm_topk_prob=True, routed_scaling=2.5, n_shared=1, bf16_combine=False, quant="fp8")

    def fetch(e):
        return S.expert_from_named(synth.make_expert(synth.DSV3, dev, SEED, 0, e))

    yield cfg, be, wg.cpu(), fetch, dev
    be.close()


@pytest.mark.parametrize("T,n_sample", [(1, 1), (32, 6), (256, 6), (1024, 5), (4096, 5)])
def test_cfg3_full_layer_256_experts(dsv3_full, T, n_sample):
    from ek_b200 import synth
    cfg, be, wg, fetch, dev = dsv3_full
    x = synth.make_tokens(synth.DSV3, dev, SEED, T)
    y, art = be.moe_forward_fused(0, x, debug=True)
    xc = x.cpu()
    r = S.check_routing(cfg, xc, wg, torch.zeros(cfg.n_experts), art)
    Hh.record(f"cfg3 E=256 T={T} routing", **{k: v for k, v in r.items() if k != "_ref"})
    assert r["exact_given_logits"], "routing is not the canonical top-k of the kernel's own logits"
    assert r["bucket_exact"], "counts / offsets / permutation differ from the stable counting sort"
    assert r["logits_max_noise_units"] <= 2.0
    assert r["differ_unexplained"] == 0 and r["differ_not_a_tie_swap"] == 0
    assert r["ids_differ"] <= max(0, T // 500), f"{r['ids_differ']} tokens routed differently"
    assert r["weights_max_rel"] <= 5e-6
    counts = be.expert_counts(0)
    assert torch.equal(counts, art["counts"]) and int(counts.sum()) == T * cfg.top_k
    o = S.check_outputs_sampled(cfg, xc, y.cpu(), r, fetch, n_sample)
    Hh.record(f"cfg3 E=256 T={T} outputs", **o)
    assert o["tokens_checked"] >= min(n_sample, T) - 1
    assert o["max_rel"] <= Hh.MAX_REL
    # outputs of a few units: one bf16 rounding of |v| ~ 2 already moves a value by 4e-3, so the
    # mean-abs bound is taken relative to mean|ref| (1e-2), as in test_gpu_parity.py
    assert o["mean_abs"] <= Hh.MEAN_ABS * max(1.0, o["mean_ref"] / 0.1)


def test_cfg3_full_layer_controller_level_reply(dsv3_full):
    """The [T,k,H] reply of the controller-level call at full expert count: rows of sampled
    (token, slot) pairs against the oracle's FFN of the named expert."""
    from ek_b200 import synth
    cfg, be, wg, fetch, dev = dsv3_full
    T = 96
    x = synth.make_tokens(synth.DSV3, dev, SEED + 1, T)
    g = torch.Generator().manual_seed(3)
    ids = torch.stack([torch.randperm(cfg.n_experts, generator=g)[:cfg.top_k] for _ in range(T)]).to(torch.int32)
    out = be.moe_forward(0, x, ids).cpu()
    xc = x.cpu()
    worst = (0.0, 0.0, 0.0)
    for t, s in ((0, 0), (41, 3), (95, 7)):
        up, gate, down = fetch(int(ids[t, s])).bf16()
        ref = O.expert_ffn(xc[t:t + 1], up, gate, down)
        mr, ma = Hh.output_errors(out[t, s:s + 1], ref)
        worst = max(worst, (mr, ma, ref.float().abs().mean().item()))
        assert mr <= Hh.MAX_REL and ma <= Hh.MEAN_ABS * max(1.0, ref.float().abs().mean().item() / 0.1)
    Hh.record("cfg3 E=256 [T,k,H] sampled rows", max_rel=worst[0], mean_abs=worst[1], mean_ref=worst[2])
    counts = be.expert_counts(0)
    assert torch.equal(counts, torch.bincount(ids.reshape(-1).long(), minlength=cfg.n_experts).to(torch.int32))
