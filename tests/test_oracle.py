"""CPU tests of the oracle itself: it must reproduce the golden vectors recorded from the
reference's own Python modules, and its integer parts must satisfy their defining properties."""
import numpy as np
import torch

from oracle import ek_oracle as O
from oracle import configs as OC
from helpers import load_golden, golden_experts, golden_shared


def test_qwen3_golden_reproduced_exactly():
    t, meta = load_golden("qwen3_tiny")
    H, I, E, k = (int(meta[x]) for x in ("hidden", "intermediate", "n_experts", "top_k"))
    L = int(meta["layer"])
    cfg = O.MoEConfig(H, I, E, k, scoring=O.SCORE_SOFTMAX, bf16_combine=True)
    r = O.moe_layer(cfg, t["x"], t["gate.weight"], None, golden_experts(t, L, E))
    assert torch.equal(r["logits"], t["router_logits"])
    assert torch.equal(r["ids"], t["selected_experts"])
    assert torch.equal(r["weights"], t["routing_weights"])
    assert torch.equal(r["y"], t["y_remote"])      # ek_forward: [T,k,H] reply, weighted sum
    assert torch.equal(r["y"], t["y_local"])       # normal_forward: per-expert index_add_
    assert meta["first_id"] == f"qwen3/l{L}-e{int(t['selected_experts'][0, 0])}"


def test_dsv3_golden_reproduced():
    t, meta = load_golden("dsv3_tiny")
    H, I, E, k = (int(meta[x]) for x in ("hidden", "intermediate", "n_experts", "top_k"))
    L = int(meta["layer"])
    cfg = O.MoEConfig(H, I, E, k, scoring=O.SCORE_SIGMOID, n_group=int(meta["n_group"]),
                      topk_group=int(meta["topk_group"]), routed_scaling=float(meta["routed_scaling"]), n_shared=1)
    r = O.moe_layer(cfg, t["x"], t["gate.weight"], t["gate.e_score_correction_bias"], golden_experts(t, L, E),
                    golden_shared(t, L))
    assert torch.equal(r["logits"], t["router_logits"])
    # the third-party router leaves the slot order unspecified: compare as sets per token
    assert torch.equal(torch.sort(r["ids"], 1)[0], torch.sort(t["topk_indices"], 1)[0])
    o1, o2 = torch.sort(r["ids"], 1)[1], torch.sort(t["topk_indices"], 1)[1]
    # weights by expert: equal up to the summation order of the renormalisation (<= 2 ulp fp32)
    torch.testing.assert_close(r["weights"].gather(1, o1), t["topk_weights"].gather(1, o2), rtol=3e-7, atol=0)
    assert torch.equal(r["y"], t["y_remote"])
    assert torch.equal(r["y"], t["y_local"])


def test_bucket_is_stable_counting_sort():
    g = torch.Generator().manual_seed(5)
    for T, k, E in ((1, 1, 4), (7, 3, 5), (64, 4, 16), (300, 8, 128)):
        ids = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)]).to(torch.int32)
        counts, offsets, perm = O.bucket(ids, E)
        flat = ids.reshape(-1)
        assert int(counts.sum()) == T * k and int(offsets[-1]) == T * k
        assert sorted(perm.tolist()) == list(range(T * k))
        for e in range(E):
            rows = perm[int(offsets[e]):int(offsets[e + 1])]
            assert (flat[rows.long()] == e).all()
            assert (rows[1:] > rows[:-1]).all()       # ascending token order inside an expert


def _bf16_rne_bits(f32: np.ndarray) -> np.ndarray:
    u = f32.view(np.uint32).astype(np.uint64)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype(np.uint16)


def test_w8a16_dequant_matches_independent_bit_level_restatement():
    g = torch.Generator().manual_seed(11)
    w = torch.randn(256, 384, generator=g) * 0.02
    q, s = OC.quantize_fp8_block(w)
    got = O.w8a16_activate(q, s)
    # independent: decode e4m3 by hand, multiply in fp32, round to nearest even
    b = q.view(torch.uint8).numpy().astype(np.int32)
    sign = np.where(b & 0x80, -1.0, 1.0)
    e = (b >> 3) & 0xF
    m = b & 7
    val = np.where(e == 0, m / 8.0 * 2.0 ** -6, (1 + m / 8.0) * 2.0 ** (e - 7.0)) * sign
    sc = np.repeat(np.repeat(s.numpy(), 128, 0), 128, 1)
    prod = (val.astype(np.float32) * sc.astype(np.float32)).astype(np.float32)
    bits = _bf16_rne_bits(prod)
    assert np.array_equal(bits, got.view(torch.int16).numpy().view(np.uint16))
    # the reference's own acceptance criterion (expert_torch.rs:207-212)
    assert abs((got.double() - torch.from_numpy(prod).double()).sum().item()) < 0.2


def test_canonical_topk_ties_go_to_lower_index():
    s = torch.tensor([[0.5, 0.7, 0.7, 0.1, 0.7]])
    v, i = O.canonical_topk(s, 3)
    assert i.tolist() == [[1, 2, 4]]


def test_sigmoid_router_matches_installed_transformers_second_opinion():
    tf = __import__("pytest").importorskip("transformers")
    from transformers.models.deepseek_v3 import modeling_deepseek_v3 as hf
    from transformers.models.deepseek_v3.configuration_deepseek_v3 import DeepseekV3Config
    cfg = DeepseekV3Config(hidden_size=64, moe_intermediate_size=32, n_routed_experts=32, num_experts_per_tok=4,
                           n_group=8, topk_group=3, n_shared_experts=1, norm_topk_prob=True,
                           routed_scaling_factor=2.5, num_hidden_layers=2, intermediate_size=64)
    moe = hf.DeepseekV3MoE(cfg)
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(50, 32, generator=g)
    bias = torch.randn(32, generator=g) * 0.1
    moe.gate.e_score_correction_bias.copy_(bias)
    with torch.no_grad():
        ids_hf, w_hf = moe.route_tokens_to_experts(logits)
    ids, w = O.route_sigmoid_grouped(logits, bias, 4, 8, 3, True, 2.5)
    assert torch.equal(torch.sort(ids, 1)[0], torch.sort(ids_hf.to(torch.int32), 1)[0])
    o1, o2 = torch.sort(ids, 1)[1], torch.sort(ids_hf, 1)[1]
    torch.testing.assert_close(w.gather(1, o1), w_hf.gather(1, o2), rtol=3e-7, atol=0)


def test_zipf_ids_cover_all_and_distinct():
    g = torch.Generator().manual_seed(9)
    ids = OC.zipf_ids(96, 8, 128, 1.2, g, cover_all=True)
    assert ids.shape == (96, 8)
    assert len(set(ids.reshape(-1).tolist())) == 128
    for row in ids.tolist():
        assert len(set(row)) == 8
