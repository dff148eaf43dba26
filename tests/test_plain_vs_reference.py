"""The plain implementation against outputs of the reference's own model code
(tests/golden/reference_logits.npz, made by tests/golden/make_golden.py), and its parts
against independent restatements."""
import math
import os

import numpy as np
import pytest
import torch

import plain_llama as plain

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_logits.npz"))


@pytest.mark.parametrize("tag,cfg,seed,std,norm_range", [("tiny_a", plain.TINY_A, 0, 0.02, None),
                                                         ("tiny_b", plain.TINY_B, 1, 0.03, (0.8, 1.2))])
def test_logits_match_the_reference(tag, cfg, seed, std, norm_range):
    w = plain.random_weights(cfg, seed, std=std, norm_range=norm_range, round_bf16=True)
    tokens = GOLDEN[f"{tag}_tokens"].tolist()
    ours = plain.logits(w, cfg, tokens)
    ref = torch.from_numpy(GOLDEN[f"{tag}_logits"])
    assert ours.shape == ref.shape
    assert float((ours - ref).abs().max()) < 2e-6
    assert [plain.greedy(r) for r in ref] == GOLDEN[f"{tag}_greedy"].tolist()
    hd = cfg["head_dim"]
    inv = plain.inv_frequencies(hd, cfg["rope_theta"], cfg["rope_scaling"])
    assert np.array_equal(inv.numpy(), GOLDEN[f"{tag}_inv_freq"])


def test_llama3_scaling_at_1b_size():
    scaling = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
               "original_max_position_embeddings": 8192}
    inv = plain.inv_frequencies(64, 500000.0, scaling)
    assert np.array_equal(inv.numpy(), GOLDEN["llama32_1b_inv_freq"])
    plain_inv = plain.inv_frequencies(64, 500000.0, None)
    assert float(inv[0]) == 1.0 and float(inv[31]) == pytest.approx(float(plain_inv[31]) / 32, rel=1e-6)
    # the library's own table builder gives the same numbers
    from llm_infer_engine_b200.parts.rope import inverse_frequencies
    assert torch.equal(inverse_frequencies(64, 500000.0, scaling), inv)


def test_parts_against_independent_restatements():
    g = torch.Generator().manual_seed(0)
    x, w = torch.randn(5, 12, generator=g), torch.rand(12, generator=g)
    ref = torch.stack([r / math.sqrt(float((r * r).mean()) + 1e-5) * w for r in x])
    assert torch.allclose(plain.rms_norm(x, w, 1e-5), ref, atol=1e-6)
    # attention: a single query over its prefix, written out
    q, k, v = torch.randn(4, 6, 8, generator=g), torch.randn(2, 6, 8, generator=g), torch.randn(2, 6, 8, generator=g)
    out = plain.causal_gqa_attention(q, k, v)
    h, t = 3, 4
    s = torch.tensor([float(q[h, t] @ k[h // 2, j]) / math.sqrt(8) for j in range(t + 1)])
    p = torch.softmax(s, 0)
    assert torch.allclose(out[h, t], sum(p[j] * v[h // 2, j] for j in range(t + 1)), atol=1e-6)
    # rotation keeps norms and is a rotation by p * inv_i of the pair (i, i + hd/2)
    inv = plain.inv_frequencies(8, 10000.0, None)
    cos, sin = plain.rotation_tables(torch.arange(6), inv)
    r = plain.rotate_half(q, cos, sin)
    assert torch.allclose(r.norm(dim=-1), q.norm(dim=-1), atol=1e-5)
    ang = 5 * float(inv[1])
    assert float(r[0, 5, 1]) == pytest.approx(float(q[0, 5, 1]) * math.cos(ang) - float(q[0, 5, 5]) * math.sin(ang), abs=1e-5)


def test_top_p_filter_is_the_reference_formula():
    """kept_by_top_p against the literal sequence of torch ops in src/sampler.py:14-22."""
    g = torch.Generator().manual_seed(1)
    for top_p in (0.0, 0.3, 0.9, 1.0):
        probs = torch.softmax(torch.randn(50, generator=g) * 2, -1)
        sorted_probs, sorted_indices = torch.sort(probs, descending=True)
        cumulative = torch.cumsum(sorted_probs, dim=-1)
        remove = cumulative > top_p
        remove[1:] = remove[:-1].clone()
        remove[0] = False
        to_remove = torch.zeros_like(probs, dtype=torch.bool)
        to_remove.scatter_(dim=-1, index=sorted_indices, src=remove)
        assert torch.equal(plain.kept_by_top_p(probs, top_p), ~to_remove)
    logits = torch.tensor([0.0, 5.0, 1.0, 5.0])
    assert plain.greedy(logits) == 1
    assert plain.sample_with_uniform(logits, 0.0, 1.0, 0.99) == 1
    assert plain.sample_with_uniform(logits, 1.0, 1.0, 0.0) == 0
    assert plain.sample_with_uniform(logits, 1.0, 1.0, 0.999999) == 3
    # distribution check of the explicit draw
    probs = torch.softmax(logits.double(), -1)
    n = 4000
    counts = torch.zeros(4)
    for i in range(n):
        counts[plain.sample_with_uniform(logits, 1.0, 1.0, (i + 0.5) / n)] += 1
    assert torch.allclose(counts / n, probs.float(), atol=2e-3)
