"""LlamaForCausalLM as a `ModelSpec`: a dense pre-norm decoder whose every layer has
grouped-query attention with rotary position encoding, a SwiGLU feed-forward and RMSNorm
(src/model.py:14-185 of the reference), under the checkpoint names of src/loader.py:8-44.
"""
from __future__ import annotations

from ..config.llama import LlamaConfig
from ..config.registry import register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

_NAMES = {"mixer": "self_attn", "feed_forward": "mlp", "mixer_norm": "input_layernorm",
          "feed_forward_norm": "post_attention_layernorm"}


def llama_spec(cfg: LlamaConfig) -> ModelSpec:
    position = PartSpec("rope", {"rot_dim": cfg.head_dim, "theta": cfg.rope_theta,
                                 "scaling": cfg.rope_scaling.to_dict() if cfg.rope_scaling else None})
    norm = PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps})
    layer = LayerSpec(
        block="pre_norm",
        mixer=PartSpec("gqa_attention", {
            "hidden": cfg.hidden_size, "n_heads": cfg.num_attention_heads, "n_kv_heads": cfg.num_key_value_heads,
            "head_dim": cfg.head_dim, "position": position, "window": 0, "scale": None}),
        feed_forward=PartSpec("swiglu", {"hidden": cfg.hidden_size, "intermediate": cfg.intermediate_size}),
        mixer_norm=norm, feed_forward_norm=norm, names=_NAMES)
    n = cfg.num_hidden_layers
    return ModelSpec(
        hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_position=cfg.max_position_embeddings,
        layers=[layer] * n, schedule=[LayerCall(i) for i in range(n)], final_norm=norm,
        tie_head=cfg.tie_word_embeddings, embedding_name="model.embed_tokens.weight",
        layer_prefix="model.layers.{i}.", final_norm_name="model.norm", head_name="lm_head.weight",
        stop_token_ids=tuple(cfg.eos_token_ids),
        ignore_unexpected=(r".*\.rotary_emb\.inv_freq$",))


register_architecture("LlamaForCausalLM", LlamaConfig, llama_spec)
