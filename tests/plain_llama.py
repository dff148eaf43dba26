"""Plain, slow LlamaForCausalLM in float32 torch: the oracle for every test.

Whole sequences, no cache, one function per part, and no code shared with the
package under test (it does not import it). Each function restates a formula of
Analysis196884/llm-infer-engine and cites the file:line it was read from.

Anchoring: `tests/golden/make_golden.py` ran the reference's own `Llama3`
(src/model.py) on the CPU through the Triton interpreter on two tiny random
models and stored tokens and logits; `tests/test_plain_vs_reference.py` checks
this file against those stored logits. Batches of unequal lengths, sampling with
a given uniform number and anything else the reference cannot do rest on the
formulas alone.

Weights are a dict keyed by the checkpoint (HF) tensor names of
src/loader.py:8-44; `cfg` is the config.json dict.
"""
from __future__ import annotations

import math

import torch


# ----------------------------------------------------------------------------- position encoding
def inv_frequencies(head_dim: int, theta: float, rope_scaling: dict | None) -> torch.Tensor:
    """src/rope.py:8-30. inv_i = theta^(-2i/hd); llama3 scaling rescales by wavelength."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2).float() / head_dim))
    if not rope_scaling:
        return inv
    kind = rope_scaling.get("rope_type", rope_scaling.get("type"))
    if kind in (None, "default"):
        return inv
    if kind != "llama3":
        raise ValueError(f"plain implementation knows no rope_type {kind!r}")
    factor = float(rope_scaling["factor"])
    low = float(rope_scaling["low_freq_factor"])
    high = float(rope_scaling["high_freq_factor"])
    orig = float(rope_scaling["original_max_position_embeddings"])
    low_wavelen = orig / low                                   # rope.py:19
    high_wavelen = orig / high                                 # rope.py:20
    wavelen = 2 * math.pi / inv                                # rope.py:22
    scaled = torch.where(wavelen > low_wavelen, inv / factor, inv)          # rope.py:23
    smooth = (orig / wavelen - low) / (high - low)                          # rope.py:25
    blended = (1 - smooth) * scaled / factor + smooth * scaled              # rope.py:26
    medium = (~(wavelen < high_wavelen)) & (~(wavelen > low_wavelen))       # rope.py:27
    return torch.where(medium, blended, scaled)                             # rope.py:28


def rotation_tables(positions: torch.Tensor, inv: torch.Tensor):
    """src/rope.py:33-45. angle[p, i] = p * inv_i in float32; cos and sin of it."""
    angle = torch.outer(positions.to(torch.float32), inv.to(torch.float32)).float()
    return torch.cos(angle), torch.sin(angle)


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """src/rope.py:74-91. x: [heads, T, hd]; first half pairs with second half."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1)


# ----------------------------------------------------------------------------- norm
def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """src/rms_norm.py:32-39. y = x * rsqrt(mean(x^2) + eps) * w, all float32."""
    x = x.float()
    ss = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    return x * torch.rsqrt(ss + eps) * weight.float()


# ----------------------------------------------------------------------------- mixer
def causal_gqa_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """src/flash_attn.py:42-82 (prefill) and src/flash_decode.py:73-113,182-205 (decode)
    compute the same thing: softmax(q k^T / sqrt(hd) + causal) v, query head h reading
    key/value head h // (Hq / Hkv) (flash_attn.py:92-94, flash_decode.py:53).

    q: [Hq, T, hd]; k, v: [Hkv, T, hd]; returns [Hq, T, hd].
    """
    n_heads, T, hd = q.shape
    group = n_heads // k.shape[0]
    k = k.repeat_interleave(group, dim=0)
    v = v.repeat_interleave(group, dim=0)
    scores = (q @ k.transpose(-1, -2)) / (hd ** 0.5)                        # flash_attn.py:52
    future = torch.triu(torch.ones(T, T, dtype=torch.bool), diagonal=1)     # flash_attn.py:47-49
    scores = scores.masked_fill(future, float("-inf"))
    return torch.softmax(scores, dim=-1) @ v


def attention_layer(x: torch.Tensor, w: dict, prefix: str, cfg: dict, cos, sin) -> torch.Tensor:
    """src/model.py:39-90. Projections without bias, rotate q and k, attend, project out."""
    T = x.shape[0]
    n_heads = cfg["num_attention_heads"]
    n_kv = cfg.get("num_key_value_heads", n_heads)
    hd = cfg.get("head_dim") or cfg["hidden_size"] // n_heads               # model.py:32
    q = (x @ w[prefix + "self_attn.q_proj.weight"].float().T).view(T, n_heads, hd).transpose(0, 1)
    k = (x @ w[prefix + "self_attn.k_proj.weight"].float().T).view(T, n_kv, hd).transpose(0, 1)
    v = (x @ w[prefix + "self_attn.v_proj.weight"].float().T).view(T, n_kv, hd).transpose(0, 1)
    q = rotate_half(q, cos, sin)                                            # model.py:62
    k = rotate_half(k, cos, sin)                                            # rope.py:150-171
    out = causal_gqa_attention(q, k, v)
    out = out.transpose(0, 1).reshape(T, n_heads * hd)                      # model.py:87
    return out @ w[prefix + "self_attn.o_proj.weight"].float().T            # model.py:88


# ----------------------------------------------------------------------------- feed-forward
def swiglu_mlp(x: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """src/model.py:23. w2(silu(w1 x) * w3 x); w1=gate_proj, w3=up_proj, w2=down_proj
    (src/loader.py:27-31)."""
    gate = x @ w[prefix + "mlp.gate_proj.weight"].float().T
    up = x @ w[prefix + "mlp.up_proj.weight"].float().T
    act = gate * torch.sigmoid(gate)
    return (act * up) @ w[prefix + "mlp.down_proj.weight"].float().T


# ----------------------------------------------------------------------------- block and model
def block(h: torch.Tensor, w: dict, layer: int, cfg: dict, cos, sin) -> torch.Tensor:
    """src/model.py:113-127. Pre-norm residual block."""
    p = f"model.layers.{layer}."
    eps = cfg["rms_norm_eps"]
    h = h + attention_layer(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p, cfg, cos, sin)
    h = h + swiglu_mlp(rms_norm(h, w[p + "post_attention_layernorm.weight"], eps), w, p)
    return h


def hidden_states(w: dict, cfg: dict, tokens) -> torch.Tensor:
    """src/model.py:157-177. Embedding, then the blocks in order; [T, hidden]."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    n_heads = cfg["num_attention_heads"]
    hd = cfg.get("head_dim") or cfg["hidden_size"] // n_heads
    inv = inv_frequencies(hd, float(cfg["rope_theta"]), cfg.get("rope_scaling"))
    cos, sin = rotation_tables(torch.arange(tokens.numel()), inv)
    h = w["model.embed_tokens.weight"].float()[tokens]                      # model.py:157
    for layer in range(cfg["num_hidden_layers"]):
        h = block(h, w, layer, cfg, cos, sin)
    return h


def head_weight(w: dict, cfg: dict) -> torch.Tensor:
    """src/loader.py:53-55: the embedding stands in for an absent lm_head.weight."""
    if cfg.get("tie_word_embeddings", False) or "lm_head.weight" not in w:
        return w["model.embed_tokens.weight"].float()
    return w["lm_head.weight"].float()


def logits(w: dict, cfg: dict, tokens) -> torch.Tensor:
    """src/model.py:181-183 with return_all_logits: final norm, then the head; [T, vocab]."""
    h = hidden_states(w, cfg, tokens)
    return rms_norm(h, w["model.norm.weight"], cfg["rms_norm_eps"]) @ head_weight(w, cfg).T


# ----------------------------------------------------------------------------- sampling
def greedy(logit_row: torch.Tensor) -> int:
    """src/sampler.py:29-30. argmax; the lowest index wins a tie."""
    return int(torch.argmax(logit_row.float()))


def kept_by_top_p(probs: torch.Tensor, top_p: float) -> torch.Tensor:
    """src/sampler.py:11-22. Sorted by falling probability, a token is dropped when the
    mass before it already exceeds top_p; the first is always kept. Returns a bool mask."""
    top_p = max(0.0, min(1.0, float(top_p)))
    sorted_probs, order = torch.sort(probs, descending=True, stable=True)
    cum = torch.cumsum(sorted_probs, dim=-1)
    drop_sorted = cum > top_p
    drop_sorted[1:] = drop_sorted[:-1].clone()
    drop_sorted[0] = False
    keep = torch.ones_like(probs, dtype=torch.bool)
    keep[order] = ~drop_sorted
    return keep


def sample_with_uniform(logit_row: torch.Tensor, temperature: float, top_p: float, u: float) -> int:
    """src/sampler.py:9-28 with the draw made explicit: softmax(logits / T), top-p filter,
    renormalise, then the inverse CDF over token ids at the uniform number u in [0, 1).
    (The reference draws with torch.multinomial; the distribution is the same.)"""
    if temperature <= 0:
        return greedy(logit_row)
    probs = torch.softmax(logit_row.double() / temperature, dim=-1)
    keep = kept_by_top_p(probs, top_p)
    probs = torch.where(keep, probs, torch.zeros_like(probs))
    total = probs.sum().clamp_min(1e-12)                                    # sampler.py:25
    cdf = torch.cumsum(probs, dim=-1)
    target = u * total
    idx = int(torch.searchsorted(cdf, target, right=True))
    idx = min(idx, probs.numel() - 1)
    while not bool(keep[idx]):                                              # only on rounding at the tail
        idx -= 1
    return idx


def sample_margins(logit_row: torch.Tensor, temperature: float, top_p: float, u: float):
    """How close the draw of sample_with_uniform is to going another way: (distance of u from the nearest
    edge between two kept tokens in the cumulative distribution, distance of top_p from the nearest mass at
    which a token is cut). Both are in units of probability; a float32 sampler may differ from this
    float64 one only where one of them is tiny."""
    probs = torch.softmax(logit_row.double() / temperature, dim=-1)
    keep = kept_by_top_p(probs, top_p)
    kept = torch.where(keep, probs, torch.zeros_like(probs))
    cdf = torch.cumsum(kept, dim=-1) / kept.sum().clamp_min(1e-12)
    draw_gap = float((cdf - u).abs().min())
    mass_before = torch.cumsum(torch.sort(probs, descending=True, stable=True).values, dim=-1)
    cut_gap = float((mass_before - max(0.0, min(1.0, float(top_p)))).abs().min())
    return draw_gap, cut_gap


# ----------------------------------------------------------------------------- random models
TINY_A = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2,
    "head_dim": 16, "intermediate_size": 192, "vocab_size": 256, "rope_theta": 10000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 128, "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
    "bos_token_id": 1, "eos_token_id": 2, "torch_dtype": "bfloat16",
}
TINY_B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 3, "num_key_value_heads": 1,
    "head_dim": 32, "intermediate_size": 256, "vocab_size": 384, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 64},
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False,
    "max_position_embeddings": 256, "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
    "bos_token_id": 1, "eos_token_id": [2, 3], "torch_dtype": "bfloat16",
}
TINY_C = {   # head size 64: the bfloat16 engine's tensor-core attention takes this one
    "architectures": ["LlamaForCausalLM"], "model_type": "llama",
    "num_hidden_layers": 2, "hidden_size": 160, "num_attention_heads": 6, "num_key_value_heads": 2,
    "head_dim": 64, "intermediate_size": 224, "vocab_size": 512, "rope_theta": 50000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                     "high_freq_factor": 4.0, "original_max_position_embeddings": 128},
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True,
    "max_position_embeddings": 1024, "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
    "bos_token_id": 1, "eos_token_id": 2, "torch_dtype": "bfloat16",
}


def tensor_shapes(cfg: dict) -> dict:
    """Checkpoint tensor names and shapes, src/loader.py:8-44 and src/model.py:17-19,34-37,134-137."""
    d, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    n_heads = cfg["num_attention_heads"]
    n_kv = cfg.get("num_key_value_heads", n_heads)
    hd = cfg.get("head_dim") or d // n_heads
    shapes = {"model.embed_tokens.weight": (V, d)}
    for i in range(cfg["num_hidden_layers"]):
        p = f"model.layers.{i}."
        shapes[p + "self_attn.q_proj.weight"] = (n_heads * hd, d)
        shapes[p + "self_attn.k_proj.weight"] = (n_kv * hd, d)
        shapes[p + "self_attn.v_proj.weight"] = (n_kv * hd, d)
        shapes[p + "self_attn.o_proj.weight"] = (d, n_heads * hd)
        shapes[p + "mlp.gate_proj.weight"] = (ff, d)
        shapes[p + "mlp.up_proj.weight"] = (ff, d)
        shapes[p + "mlp.down_proj.weight"] = (d, ff)
        shapes[p + "input_layernorm.weight"] = (d,)
        shapes[p + "post_attention_layernorm.weight"] = (d,)
    shapes["model.norm.weight"] = (d,)
    if not cfg.get("tie_word_embeddings", False):
        shapes["lm_head.weight"] = (V, d)
    return shapes


def random_weights(cfg: dict, seed: int, std: float = 0.02, norm_range=None, round_bf16: bool = True) -> dict:
    """Seeded random weights by checkpoint name: matrices ~N(0, std), norm weights 1 or
    ~U(norm_range). With round_bf16 every value is a bfloat16 value held in float32, so a
    bfloat16 engine and this float32 oracle see the same numbers."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm.weight") or name.endswith("layernorm.weight"):
            if norm_range is None:
                t = torch.ones(shape)
            else:
                t = torch.empty(shape).uniform_(norm_range[0], norm_range[1], generator=g)
        else:
            t = torch.randn(shape, generator=g) * std
        if round_bf16:
            t = t.to(torch.bfloat16).float()
        out[name] = t
    return out
