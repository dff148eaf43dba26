"""Command line in the manner of the reference's main.py: the same option names and meanings
where it has them (main.py:21-43), the same precedence command line > .env file > environment >
default (main.py:73-87), the same printed stages (main.py:243,297,457).

Differences that follow from this library's design: model sizes come from config.json (found
in --model, or in --tokenizer as the reference does, main.py:374); the size flags --dim,
--n-layers, ... are read only in random-weights mode when there is no config.json;
--quantization is not offered; --dtype chooses the bfloat16 or the true float32 path;
--prompt-ids and --prompt-ids-file run without a tokenizer; --init-std sets the spread of random
weights; stop ids come from config.json, generation_config.json and the tokenizer together.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path
from typing import List, Optional


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="Llama inference on one B200")
    p.add_argument("--env-file", type=str, default=".env", help="Path to .env file, default: .env")
    p.add_argument("--model", type=str, default=None, help="Model folder: config.json, model.safetensors, tokenizer")
    p.add_argument("--tokenizer", type=str, default=None, help="Tokenizer path (also searched for config.json)")
    p.add_argument("--weights", type=str, default=None, help="Path to safetensors weights; empty = random weights")
    p.add_argument("--prompt", type=str, default=None, help="Input prompt")
    p.add_argument("--prompt-file", type=str, default=None, help="Path to a UTF-8 text file used as input prompt")
    p.add_argument("--prompt-ids", type=str, default=None, help="Prompt as comma-separated token ids (no tokenizer)")
    p.add_argument("--prompt-ids-file", type=str, default=None,
                   help="File of token ids separated by commas or white space (no tokenizer)")
    p.add_argument("--system-prompt", type=str, default=None, help="System prompt for chat template")
    p.add_argument("--max-new-tokens", type=int, default=None, help="Maximum generated tokens")
    p.add_argument("--temperature", type=float, default=None, help="Sampling temperature (<= 0: greedy)")
    p.add_argument("--top-p", type=float, default=None, help="Nucleus sampling threshold")
    p.add_argument("--device", type=str, default=None, help="CUDA device, e.g. cuda, cuda:0 or 0")
    p.add_argument("--seed", type=int, default=None, help="Random seed (sampling and random weights)")
    p.add_argument("--init-std", type=float, default=None, help="Standard deviation of random weights, default 0.02")
    p.add_argument("--dim", type=int, default=None)
    p.add_argument("--n-layers", type=int, default=None)
    p.add_argument("--n-heads", type=int, default=None)
    p.add_argument("--n-kv-heads", type=int, default=None)
    p.add_argument("--hidden-dim", type=int, default=None)
    p.add_argument("--vocab-size", type=int, default=None)
    p.add_argument("--max-seq-len", type=int, default=None)
    p.add_argument("--max-batch", type=int, default=None, help="Sequences held at once")
    p.add_argument("--cuda-graph", type=str, default=None, choices=["on", "off"], help="CUDA Graph for decode")
    p.add_argument("--dtype", type=str, default=None, choices=["bfloat16", "float32"])
    p.add_argument("--nvtx", action="store_true", help="Mark the stages of every step with NVTX ranges")
    return p


def parse_env_file(env_file: Optional[str]) -> dict:
    """The settings of a .env file as a dict of strings. One `KEY=VALUE` a line; a leading `export`, one pair
    of quotes round the value and `#` comment lines are taken, anything else is passed over; a file that is
    not there gives no settings (the format the reference reads, main.py:46-70)."""
    try:
        text = Path(env_file).read_text(encoding="utf-8") if env_file else ""
    except OSError:
        return {}
    settings = {}
    for body in (line.strip() for line in text.splitlines()):
        if body.startswith("#"):
            continue
        if body.startswith("export "):
            body = body[7:].lstrip()
        key, eq, value = body.partition("=")
        if not eq:
            continue
        value = value.strip()
        if len(value) > 1 and value[0] in "'\"" and value[-1] == value[0]:
            value = value[1:-1]
        settings[key.strip()] = value
    return settings


# option -> (environment name, default, type). The environment names and the defaults are the reference's
# (main.py:89-121) where it has the option; an empty setting counts as not given.
OPTIONS = {
    "model": ("LLM_MODEL", None, str), "tokenizer": ("LLM_TOKENIZER", None, str), "weights": ("LLM_WEIGHTS", "", str),
    "prompt": ("LLM_PROMPT", None, str), "prompt_file": ("LLM_PROMPT_FILE", None, str),
    "prompt_ids": ("LLM_PROMPT_IDS", None, str), "prompt_ids_file": ("LLM_PROMPT_IDS_FILE", None, str),
    "system_prompt": ("LLM_SYSTEM_PROMPT", "You are a helpful assistant.", str),
    "max_new_tokens": ("LLM_MAX_NEW_TOKENS", 256, int), "temperature": ("LLM_TEMPERATURE", 0.0, float),
    "top_p": ("LLM_TOP_P", 1.0, float), "cuda_graph": ("LLM_CUDA_GRAPH", "on", str), "device": ("LLM_DEVICE", "cuda", str),
    "seed": ("LLM_SEED", None, int), "init_std": ("LLM_INIT_STD", 0.02, float), "dim": ("LLM_DIM", None, int),
    "n_layers": ("LLM_N_LAYERS", None, int), "n_heads": ("LLM_N_HEADS", None, int),
    "n_kv_heads": ("LLM_N_KV_HEADS", None, int), "hidden_dim": ("LLM_HIDDEN_DIM", None, int),
    "vocab_size": ("LLM_VOCAB_SIZE", None, int), "max_seq_len": ("LLM_MAX_SEQ_LEN", 4096, int),
    "max_batch": ("LLM_MAX_BATCH", 1, int), "dtype": ("LLM_DTYPE", "bfloat16", str),
}


def resolve(cli_value, env_key: str, env_file: dict, default, cast):
    """One option from its sources, the nearest first: command line, .env file, environment, default."""
    if cli_value is not None:
        return cli_value
    text = env_file[env_key] if env_key in env_file else os.environ.get(env_key)
    return default if text in (None, "") else cast(text)


def resolve_all(args, env_file: dict) -> dict:
    return {name: resolve(getattr(args, name), key, env_file, default, cast)
            for name, (key, default, cast) in OPTIONS.items()}


def read_ids_file(path: str) -> str:
    """Token ids from a file, separated by commas or white space, as the comma-separated text of --prompt-ids."""
    words = Path(path).expanduser().read_text(encoding="utf-8").replace(",", " ").split()
    if not words:
        raise ValueError(f"{path} holds no token ids")
    bad = [w for w in words if not w.isdigit()]
    if bad:
        raise ValueError(f"{path}: {bad[0]!r} is not a token id")
    return ",".join(words)


def device_index(text: str) -> int:
    t = str(text).strip().lower()
    if t in ("cuda", "gpu"):
        return 0
    if t.startswith("cuda:"):
        t = t[5:]
    if t.isdigit():
        return int(t)
    raise ValueError(f"--device {text!r}: this library runs on CUDA devices only (cuda, cuda:N or N)")


def config_from_flags(opts: dict) -> dict:
    """A config.json for random-weights mode when no folder provides one. Every size must be
    given: none has a default here."""
    names = {"dim": "--dim", "n_layers": "--n-layers", "n_heads": "--n-heads", "hidden_dim": "--hidden-dim",
             "vocab_size": "--vocab-size"}
    missing = [flag for key, flag in names.items() if opts[key] is None]
    if missing:
        raise ValueError("random weights without a config.json need " + ", ".join(missing))
    return {
        "architectures": ["LlamaForCausalLM"], "model_type": "llama", "hidden_size": opts["dim"],
        "num_hidden_layers": opts["n_layers"], "num_attention_heads": opts["n_heads"],
        "num_key_value_heads": opts["n_kv_heads"] or opts["n_heads"], "intermediate_size": opts["hidden_dim"],
        "vocab_size": opts["vocab_size"], "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": None,
        "max_position_embeddings": opts["max_seq_len"], "tie_word_embeddings": False,
    }


def prepare_model_folder(opts: dict, log=print) -> str:
    """Returns a folder with config.json and model.safetensors for the engine to load."""
    from ..weights import scratch_folder, write_random_model
    config_dir = next((d for d in (opts["model"], opts["tokenizer"])
                       if d and os.path.isfile(os.path.join(d, "config.json"))), None)
    if opts["weights"]:
        if not os.path.isfile(opts["weights"]):
            raise FileNotFoundError(f"weights file not found: {opts['weights']}")
        if config_dir is None:
            raise ValueError("--weights needs a config.json in --model or --tokenizer")
        folder = scratch_folder("llmie_model_")
        os.symlink(os.path.abspath(os.path.join(config_dir, "config.json")), os.path.join(folder, "config.json"))
        os.symlink(os.path.abspath(opts["weights"]), os.path.join(folder, "model.safetensors"))
        return folder
    if opts["model"] and (os.path.isfile(os.path.join(opts["model"], "model.safetensors"))
                          or os.path.isfile(os.path.join(opts["model"], "model.safetensors.index.json"))):
        return opts["model"]
    # random weights (the reference does this when --weights is empty, main.py:418-434)
    if config_dir is not None:
        with open(os.path.join(config_dir, "config.json"), encoding="utf-8") as f:
            config_json = json.load(f)
    else:
        config_json = config_from_flags(opts)
    folder = scratch_folder("llmie_random_")
    t0 = time.time()
    write_random_model(config_json, folder, seed=opts["seed"] or 0, std=opts["init_std"])
    log(f"    Random init: {time.time() - t0:.4f}s")
    return folder


class TextTokenizer:
    """transformers' tokenizer with the chat template, as the reference wraps it
    (src/tokenizer.py:3-13, main.py:169-183)."""

    def __init__(self, path: str):
        from transformers import AutoTokenizer
        self.inner = AutoTokenizer.from_pretrained(path)
        self.eos_id = self.inner.eos_token_id

    def chat_ids(self, user_prompt: str, system_prompt: str) -> List[int]:
        messages = [{"role": "system", "content": system_prompt}, {"role": "user", "content": user_prompt}]
        if getattr(self.inner, "chat_template", None):
            enc = self.inner.apply_chat_template(messages, add_generation_prompt=True, tokenize=True)
            if hasattr(enc, "keys") and "input_ids" in enc:
                enc = enc["input_ids"]
            if enc and isinstance(enc[0], list):
                enc = enc[0]
            return [int(t) for t in enc]
        return [int(t) for t in self.inner.encode(system_prompt + "\n" + user_prompt)]

    def decode(self, ids: List[int]) -> str:
        return self.inner.decode(ids, skip_special_tokens=True)


def main(argv: Optional[List[str]] = None) -> int:
    overall_start = time.time()
    parser = build_parser()
    args = parser.parse_args(argv)
    opts = resolve_all(args, parse_env_file(args.env_file))
    if args.prompt is not None and args.prompt_file is not None:
        parser.error("Use either --prompt or --prompt-file, not both.")
    if opts["prompt_file"] and not opts["prompt"]:
        path = Path(opts["prompt_file"]).expanduser()
        if not path.is_file():
            parser.error(f"Prompt file not found: {path}")
        opts["prompt"] = path.read_text(encoding="utf-8")
        if not opts["prompt"].strip():
            parser.error(f"Prompt file is empty: {path}")
    if opts["prompt_ids_file"] and not opts["prompt_ids"]:
        try:
            opts["prompt_ids"] = read_ids_file(opts["prompt_ids_file"])
        except (OSError, ValueError) as e:
            parser.error(f"--prompt-ids-file: {e}")
    if not opts["prompt"] and not opts["prompt_ids"]:
        parser.error("Missing prompt. Provide --prompt, --prompt-file, --prompt-ids or --prompt-ids-file (or LLM_PROMPT).")
    tokenizer_dir = opts["tokenizer"] or opts["model"]
    if opts["prompt"] and not opts["prompt_ids"] and not tokenizer_dir:
        parser.error("Missing tokenizer. Provide --tokenizer or --model, or give the prompt as --prompt-ids.")
    try:
        device = device_index(opts["device"])
    except ValueError as e:
        parser.error(str(e))

    print("=" * 70)
    print("INFERENCE CONFIGURATION")
    print("=" * 70)
    print(f"Device: cuda:{device}")
    print(f"CUDA Graph: {opts['cuda_graph']}")
    print(f"Dtype: {opts['dtype']}")
    if opts["prompt"]:
        shown = opts["system_prompt"]
        print(f"System Prompt: {shown[:100] + '...' if len(shown) > 100 else shown}")
        shown = opts["prompt"]
        print(f"User Prompt: {shown[:150] + '...' if len(shown) > 150 else shown}")
    print("=" * 70 + "\n")

    from .. import Engine, GenerationStats, SamplingParams, generate
    print("[2] Model loading and tokenizer init:")
    tokenizer = None
    if opts["prompt"] and not opts["prompt_ids"]:
        t0 = time.time()
        tokenizer = TextTokenizer(tokenizer_dir)
        print(f"    Tokenizer: {time.time() - t0:.4f}s")
    try:
        folder = prepare_model_folder(opts)
    except (ValueError, FileNotFoundError) as e:
        parser.error(str(e))
    t0 = time.time()
    engine = Engine(folder, dtype=opts["dtype"], device=device, max_batch=opts["max_batch"],
                    max_seq_len=opts["max_seq_len"], cuda_graph=opts["cuda_graph"] == "on", nvtx=args.nvtx)
    report = engine.model.load_report
    print(f"    Model: loaded={report['tensors']} tensors, {report['bytes'] / 1e9:.3f} GB in {time.time() - t0:.4f}s")

    if opts["prompt_ids"]:
        prompt_ids = [int(t) for t in opts["prompt_ids"].replace(" ", "").split(",") if t]
    else:
        prompt_ids = tokenizer.chat_ids(opts["prompt"], opts["system_prompt"])
    if not prompt_ids:
        parser.error("Prompt is empty after tokenization.")

    print("\n[3] Generation:")
    print(f"\n{'=' * 70}\nOUTPUT\n{'=' * 70}")
    generated: List[int] = []
    shown = {"text": ""}

    def on_tokens(_requests, tokens):
        generated.extend(tokens)
        if tokenizer is None:
            print(" ".join(str(t) for t in tokens), end=" ", flush=True)
            return
        text = tokenizer.decode(generated)
        if text and not text.endswith("�"):            # hold back half-decoded characters (main.py:265-268)
            print(text[len(shown["text"]):], end="", flush=True)
            shown["text"] = text

    stats = GenerationStats()
    sampling = SamplingParams(temperature=opts["temperature"], top_p=opts["top_p"], seed=opts["seed"] or 0)
    stop = None if tokenizer is None or tokenizer.eos_id is None else \
        sorted(set(engine.model.spec.stop_token_ids) | {tokenizer.eos_id})
    generate(engine, [prompt_ids], max_new_tokens=opts["max_new_tokens"], sampling=sampling, stop_ids=stop,
             on_tokens=on_tokens, stats=stats)
    if tokenizer is not None:
        print(tokenizer.decode(generated)[len(shown["text"]):], end="", flush=True)
    print(f"\n{'=' * 70}")
    print(f"    Prefill: {stats.prefill_seconds:.4f}s ({stats.prefill_tokens} tokens)")
    n_new = len(generated)
    decode_s = max(stats.decode_seconds, 1e-6)
    print(f"    Decode: {decode_s:.4f}s ({n_new} tokens, TPS: {stats.decode_tokens / decode_s:.2f} tokens/s)")
    print(f"\n{'=' * 70}\nTotal: {time.time() - overall_start:.4f}s\n{'=' * 70}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
