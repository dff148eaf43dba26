"""Makes tests/golden/reference_logits.npz by running the reference's OWN model code.

Needs a checkout of Analysis196884/llm-infer-engine (argument 1 or $LLM_INFER_ENGINE_REF);
it is imported read-only and nothing of it is copied. The reference's kernels are Triton;
on a machine without a GPU they run through Triton's interpreter (TRITON_INTERPRET=1) on
CPU tensors in float32. Two of its launchers refuse tensors that are not on a GPU
(src/rms_norm.py:43-44, src/flash_decode.py:264); the harness hands them a Tensor subclass
whose `is_cuda` says True. The reference is driven only in the ways it supports: one
sequence, a KV cache always (without one it never rotates K, src/model.py:62-75), the whole
prompt at start_pos 0 (src/model.py:145) and then one token per call.

Stored per model: the token ids, the logits at every position (prompt positions from the
prefill call with return_all_logits, the rest from one-token decode calls), the reference's
inverse frequencies (src/rope.py:8-30) and its greedy choice (src/sampler.py:29-30) per position.

    python tests/golden/make_golden.py /path/to/llm-infer-engine
"""
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
os.environ.setdefault("PYTHONDONTWRITEBYTECODE", "1")
sys.dont_write_bytecode = True

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("LLM_INFER_ENGINE_REF", "")
if not REF or not os.path.isdir(REF):
    sys.exit("usage: make_golden.py /path/to/llm-infer-engine")
sys.path.insert(0, REF)

import numpy as np
import torch

import plain_llama as plain
import src.flash_decode as ref_flash_decode
import src.model as ref_model
import src.rms_norm as ref_rms_norm
from src.config import ModelArgs
from src.kv_cache import KVCache
from src.rope import _compute_inv_freq
from src.sampler import sample as ref_sample


class _SaysCuda(torch.Tensor):
    is_cuda = property(lambda self: True)


def _as_cuda(t):
    return t.as_subclass(_SaysCuda)


_rms = ref_rms_norm.rmsnorm_triton
ref_rms_norm.rmsnorm_triton = lambda x, w, eps=1e-6: _rms(_as_cuda(x), _as_cuda(w), eps).as_subclass(torch.Tensor)
_fd = ref_flash_decode.flash_decode
ref_model.flash_decode = lambda q, k, v, mask=None: _fd(_as_cuda(q), _as_cuda(k), _as_cuda(v), mask=mask).as_subclass(torch.Tensor)

# checkpoint name -> the reference's own parameter name (inverse of src/loader.py:8-44)
_LAYER = {
    "self_attn.q_proj.weight": "attention.wq.weight", "self_attn.k_proj.weight": "attention.wk.weight",
    "self_attn.v_proj.weight": "attention.wv.weight", "self_attn.o_proj.weight": "attention.wo.weight",
    "mlp.gate_proj.weight": "feed_forward.w1.weight", "mlp.down_proj.weight": "feed_forward.w2.weight",
    "mlp.up_proj.weight": "feed_forward.w3.weight", "input_layernorm.weight": "attention_norm.weight",
    "post_attention_layernorm.weight": "ffn_norm.weight",
}


def _ref_name(name):
    if name == "model.embed_tokens.weight":
        return "tok_embeddings.weight"
    if name == "model.norm.weight":
        return "norm.weight"
    if name == "lm_head.weight":
        return "output.weight"
    _, _, idx, rest = name.split(".", 3)
    return f"layers.{idx}.{_LAYER[rest]}"


def run(tag, cfg, seed, std, norm_range, n_prompt, n_decode, out):
    w = plain.random_weights(cfg, seed, std=std, norm_range=norm_range, round_bf16=True)
    args = ModelArgs(
        dim=cfg["hidden_size"], n_layers=cfg["num_hidden_layers"], n_heads=cfg["num_attention_heads"],
        n_kv_heads=cfg["num_key_value_heads"], vocab_size=cfg["vocab_size"], hidden_dim=cfg["intermediate_size"],
        norm_eps=cfg["rms_norm_eps"], max_batch_size=1, max_seq_len=cfg["max_position_embeddings"],
        rope_theta=cfg["rope_theta"], rope_scaling=cfg["rope_scaling"], device="cpu")
    assert cfg["head_dim"] == args.dim // args.n_heads
    model = ref_model.Llama3(args).eval()
    state = {_ref_name(k): v.clone() for k, v in w.items()}
    if "output.weight" not in state:
        state["output.weight"] = state["tok_embeddings.weight"].clone()
    model.load_state_dict(state, strict=True)

    g = torch.Generator().manual_seed(1000 + seed)
    tokens = torch.randint(0, cfg["vocab_size"], (n_prompt + n_decode,), generator=g)
    cache = KVCache(args, dtype=torch.float32)
    rows = []
    with torch.no_grad():
        rows.append(model(tokens[None, :n_prompt], start_pos=0, kv_cache=cache, return_all_logits=True)[0])
        for i in range(n_decode):
            p = n_prompt + i
            rows.append(model(tokens[None, p:p + 1], start_pos=p, kv_cache=cache)[0])
    ref_logits = torch.cat(rows, dim=0).float()
    greedy = torch.stack([ref_sample(r[None, :], temperature=0.0)[0, 0] for r in ref_logits])
    ours = plain.logits(w, cfg, tokens)
    print(f"{tag}: {tuple(ref_logits.shape)} max|plain - reference| = {float((ours - ref_logits).abs().max()):.3e}"
          f" (logit scale {float(ref_logits.abs().max()):.3f})")
    out[f"{tag}_tokens"] = tokens.numpy().astype(np.int32)
    out[f"{tag}_n_prompt"] = np.int32(n_prompt)
    out[f"{tag}_logits"] = ref_logits.numpy()
    out[f"{tag}_greedy"] = greedy.numpy().astype(np.int32)
    hd = cfg["head_dim"]
    out[f"{tag}_inv_freq"] = _compute_inv_freq(hd, cfg["rope_theta"], cfg["rope_scaling"]).numpy()


def main():
    out = {}
    run("tiny_a", plain.TINY_A, seed=0, std=0.02, norm_range=None, n_prompt=17, n_decode=8, out=out)
    run("tiny_b", plain.TINY_B, seed=1, std=0.03, norm_range=(0.8, 1.2), n_prompt=70, n_decode=12, out=out)
    scaling_1b = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                  "original_max_position_embeddings": 8192}
    out["llama32_1b_inv_freq"] = _compute_inv_freq(64, 500000.0, scaling_1b).numpy()
    path = os.path.join(HERE, "reference_logits.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
