"""Typed configuration of LlamaForCausalLM, read from the architecture's own config.json keys.

The reference keeps sizes in a flat dataclass filled from flags (src/config.py:4-18) and reads
only rms_norm_eps, rope_theta, rope_scaling and max_position_embeddings from config.json
(main.py:374-382); its long-context test maps the size keys too
(tests/needle_in_haystack.py:239-252). Here every size and constant comes from config.json,
none has a default in code, and a bad or missing key is an error that names the key.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .registry import ConfigError

_MISSING = object()


def _get(cfg: dict, key: str, kind, default=_MISSING):
    value = cfg.get(key, None)
    if value is None:
        if default is _MISSING:
            raise ConfigError(f"config.json: required key {key!r} is missing")
        return default
    if kind is float and isinstance(value, (int, float)) and not isinstance(value, bool):
        return float(value)
    if kind is int and isinstance(value, int) and not isinstance(value, bool):
        return int(value)
    if kind is bool and isinstance(value, bool):
        return value
    if kind is str and isinstance(value, str):
        return value
    raise ConfigError(f"config.json: key {key!r} must be {kind.__name__}, got {value!r}")


def _positive(name: str, value):
    if value <= 0:
        raise ConfigError(f"config.json: key {name!r} must be positive, got {value!r}")
    return value


@dataclass(frozen=True)
class RopeScaling:
    """llama3 frequency scaling (src/rope.py:11-30): all four numbers are required."""
    rope_type: str
    factor: float
    low_freq_factor: float
    high_freq_factor: float
    original_max_position_embeddings: int

    @staticmethod
    def from_dict(d: Optional[dict]) -> Optional["RopeScaling"]:
        if d is None:
            return None
        if not isinstance(d, dict):
            raise ConfigError(f"config.json: 'rope_scaling' must be an object or null, got {d!r}")
        kind = d.get("rope_type", d.get("type"))
        if kind in (None, "default"):
            return None
        if kind != "llama3":
            raise ConfigError(f"config.json: rope_scaling.rope_type {kind!r} is not supported "
                              "(supported: 'default', 'llama3')")
        vals = {}
        for key in ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings"):
            if key not in d or isinstance(d[key], bool) or not isinstance(d[key], (int, float)):
                raise ConfigError(f"config.json: rope_scaling.{key} is required for rope_type 'llama3' "
                                  f"and must be a number, got {d.get(key)!r}")
            vals[key] = d[key]
        if vals["high_freq_factor"] == vals["low_freq_factor"]:
            raise ConfigError("config.json: rope_scaling.high_freq_factor must differ from low_freq_factor")
        if vals["factor"] <= 0 or vals["low_freq_factor"] <= 0 or vals["high_freq_factor"] <= 0:
            raise ConfigError("config.json: rope_scaling factors must be positive")
        return RopeScaling("llama3", float(vals["factor"]), float(vals["low_freq_factor"]),
                           float(vals["high_freq_factor"]), int(vals["original_max_position_embeddings"]))

    def to_dict(self) -> dict:
        return {"rope_type": self.rope_type, "factor": self.factor, "low_freq_factor": self.low_freq_factor,
                "high_freq_factor": self.high_freq_factor,
                "original_max_position_embeddings": self.original_max_position_embeddings}


@dataclass(frozen=True)
class LlamaConfig:
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: Optional[RopeScaling]
    max_position_embeddings: int
    tie_word_embeddings: bool
    bos_token_id: Optional[int]
    eos_token_ids: Tuple[int, ...]
    torch_dtype: str

    @staticmethod
    def from_dict(cfg: dict) -> "LlamaConfig":
        hidden = _positive("hidden_size", _get(cfg, "hidden_size", int))
        layers = _positive("num_hidden_layers", _get(cfg, "num_hidden_layers", int))
        heads = _positive("num_attention_heads", _get(cfg, "num_attention_heads", int))
        kv_heads = _positive("num_key_value_heads", _get(cfg, "num_key_value_heads", int, heads))
        if heads % kv_heads:
            raise ConfigError(f"config.json: num_attention_heads ({heads}) must be a multiple of "
                              f"num_key_value_heads ({kv_heads})")
        if "head_dim" in cfg and cfg["head_dim"] is not None:
            head_dim = _positive("head_dim", _get(cfg, "head_dim", int))
        else:
            if hidden % heads:
                raise ConfigError(f"config.json: hidden_size ({hidden}) is not a multiple of "
                                  f"num_attention_heads ({heads}) and no head_dim is given")
            head_dim = hidden // heads          # src/model.py:32
        if head_dim % 2:
            raise ConfigError(f"config.json: head_dim ({head_dim}) must be even for rotary position encoding")
        inter = _positive("intermediate_size", _get(cfg, "intermediate_size", int))
        vocab = _positive("vocab_size", _get(cfg, "vocab_size", int))
        eps = _positive("rms_norm_eps", _get(cfg, "rms_norm_eps", float))
        max_pos = _positive("max_position_embeddings", _get(cfg, "max_position_embeddings", int))

        # rope: the classic keys, or the newer single `rope_parameters` object holding both
        rope_params = cfg.get("rope_parameters")
        if "rope_theta" in cfg and cfg["rope_theta"] is not None:
            theta = _positive("rope_theta", _get(cfg, "rope_theta", float))
            scaling = RopeScaling.from_dict(cfg.get("rope_scaling"))
        elif isinstance(rope_params, dict) and "rope_theta" in rope_params:
            theta = _positive("rope_parameters.rope_theta", _get(rope_params, "rope_theta", float))
            scaling = RopeScaling.from_dict(rope_params)
        else:
            raise ConfigError("config.json: required key 'rope_theta' is missing")

        act = _get(cfg, "hidden_act", str, "silu")
        if act != "silu":
            raise ConfigError(f"config.json: hidden_act {act!r} is not supported by this architecture (silu only)")
        for key in ("attention_bias", "mlp_bias"):
            if _get(cfg, key, bool, False):
                raise ConfigError(f"config.json: {key} = true is not supported (the projections have no bias)")

        eos = cfg.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int) and not isinstance(eos, bool):
            eos_ids = (eos,)
        elif isinstance(eos, (list, tuple)) and all(isinstance(e, int) and not isinstance(e, bool) for e in eos):
            eos_ids = tuple(eos)
        else:
            raise ConfigError(f"config.json: eos_token_id must be an integer or a list of integers, got {eos!r}")
        for e in eos_ids:
            if not 0 <= e < vocab:
                raise ConfigError(f"config.json: eos_token_id {e} is outside the vocabulary (0..{vocab - 1})")
        bos = cfg.get("bos_token_id")
        if bos is not None and (isinstance(bos, bool) or not isinstance(bos, int)):
            raise ConfigError(f"config.json: bos_token_id must be an integer, got {bos!r}")

        return LlamaConfig(
            hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
            num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter, vocab_size=vocab,
            rms_norm_eps=eps, rope_theta=theta, rope_scaling=scaling, max_position_embeddings=max_pos,
            tie_word_embeddings=_get(cfg, "tie_word_embeddings", bool, False),
            bos_token_id=bos, eos_token_ids=eos_ids,
            torch_dtype=_get(cfg, "torch_dtype", str, cfg.get("dtype") or "bfloat16"),
        )

    def to_dict(self) -> dict:
        return {
            "architectures": ["LlamaForCausalLM"], "model_type": "llama",
            "hidden_size": self.hidden_size, "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads, "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim, "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size, "rms_norm_eps": self.rms_norm_eps, "rope_theta": self.rope_theta,
            "rope_scaling": self.rope_scaling.to_dict() if self.rope_scaling else None,
            "max_position_embeddings": self.max_position_embeddings,
            "tie_word_embeddings": self.tie_word_embeddings, "hidden_act": "silu",
            "attention_bias": False, "mlp_bias": False, "bos_token_id": self.bos_token_id,
            "eos_token_id": (list(self.eos_token_ids) if len(self.eos_token_ids) != 1 else self.eos_token_ids[0])
            if self.eos_token_ids else None,
            "torch_dtype": self.torch_dtype,
        }
