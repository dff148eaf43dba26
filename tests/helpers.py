"""Shared test helpers: tiny model folders, weights for the plain implementation, replays."""
import json
import os
import subprocess
import sys

import numpy as np
import torch

import plain_llama as plain
from llm_infer_engine_b200.weights import scratch_folder  # noqa: F401  (temporary folders deleted at exit)

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# The two tiny configurations differ in every size and option: layers, width, heads and groups
# (GQA 4/2 vs MQA 3/1), head size, feed-forward width, vocabulary (both no power of two in B),
# theta, frequency scaling, eps, tied or separate head, how weights are drawn.
TINY = {
    "a": dict(cfg=plain.TINY_A, seed=0, std=0.02, norm_range=None),
    "b": dict(cfg=plain.TINY_B, seed=1, std=0.03, norm_range=(0.8, 1.2)),
    # head size 64 (hidden != heads * head_dim), three query heads per KV head, longer sequences
    "c": dict(cfg=plain.TINY_C, seed=2, std=0.05, norm_range=(0.9, 1.1)),
}

_folders = {}


def model_folder(tag: str, dtype: str = "bfloat16", std: float = None) -> str:
    """A temporary model folder written by the library's random-weights mode."""
    from llm_infer_engine_b200 import write_random_model
    key = (tag, dtype, std)
    if key not in _folders:
        spec = TINY[tag]
        d = scratch_folder(f"llmie_tiny_{tag}_")
        write_random_model(spec["cfg"], d, seed=spec["seed"], std=std or spec["std"], norm_range=spec["norm_range"],
                           dtype=dtype)
        _folders[key] = d
    return _folders[key]


def plain_weights(folder: str) -> dict:
    """Reads the folder with the `safetensors` package (not the library's own reader)."""
    from safetensors.torch import load_file
    return {k: v.float() for k, v in load_file(os.path.join(folder, "model.safetensors")).items()}


def read_config(folder: str) -> dict:
    with open(os.path.join(folder, "config.json")) as f:
        return json.load(f)


def random_tokens(vocab: int, n: int, seed: int):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


# ------------------------------------------------------------------ replay plans (trace_run's input language)
def plan_whole(requests: dict):
    """Each request alone, all tokens in one step, logits everywhere."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def plan_tail(requests: dict, tail: int = 32):
    """Each request alone: all but the last `tail` tokens in one step, then one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}],
                      "end": []})
        for p in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[p]], "want": [0]}], "end": []})
        steps[-1]["end"] = [rid]
    return steps


def plan_batched(requests: dict, batch_size: int, prompt_frac: float = 0.5):
    """Batches of unequal lengths: prompts (a part of each request) in one step, then one token
    each while a request still has tokens; shorter requests end earlier; batch after batch."""
    steps = []
    ids = list(requests)
    for b in range(0, len(ids), batch_size):
        group = ids[b:b + batch_size]
        cut = {rid: max(1, int(len(requests[rid]) * prompt_frac)) for rid in group}
        entries = [{"id": rid, "tokens": requests[rid][:cut[rid]], "want": list(range(cut[rid]))} for rid in group]
        done = [rid for rid in group if cut[rid] == len(requests[rid])]
        steps.append({"step": len(steps), "entries": entries, "end": done})
        live = [rid for rid in group if rid not in done]
        pos = dict(cut)
        while live:
            entries = [{"id": rid, "tokens": [requests[rid][pos[rid]]], "want": [0]} for rid in live]
            for rid in live:
                pos[rid] += 1
            done = [rid for rid in live if pos[rid] == len(requests[rid])]
            steps.append({"step": len(steps), "entries": entries, "end": done})
            live = [rid for rid in live if rid not in done]
    return steps


def plan_chunked(requests: dict, chunk: int):
    """Each request alone, its tokens in steps of `chunk` tokens: every step after the first brings several
    tokens at a start position above zero (a prompt taken in pieces)."""
    steps = []
    for rid, toks in requests.items():
        for lo in range(0, len(toks), chunk):
            part = toks[lo:lo + chunk]
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": part, "want": list(range(len(part)))}],
                          "end": []})
        steps[-1]["end"] = [rid]
    return steps


def plan_mixed(requests: dict, chunk: int):
    """The first request sends its tokens in pieces of `chunk` while all the others, started together with a
    part of their prompts, go on by one token a step: steps in which one sequence brings many tokens at a
    start position above zero and the others bring one."""
    ids = list(requests)
    long_id, others = ids[0], ids[1:]
    cut = {rid: max(1, len(requests[rid]) // 2) for rid in others}
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": requests[rid][:cut[rid]], "want": list(range(cut[rid]))}
                                     for rid in others],
              "end": [rid for rid in others if cut[rid] == len(requests[rid])]}]
    pos = dict(cut)
    pos[long_id] = 0
    live = [rid for rid in ids if pos.get(rid, 0) < len(requests[rid])]
    while live:
        entries = []
        for rid in live:
            n = chunk if rid == long_id else 1
            part = requests[rid][pos[rid]:pos[rid] + n]
            entries.append({"id": rid, "tokens": part, "want": list(range(len(part)))})
            pos[rid] += len(part)
        done = [rid for rid in live if pos[rid] == len(requests[rid])]
        steps.append({"step": len(steps), "entries": entries, "end": done})
        live = [rid for rid in live if rid not in done]
    return steps


def logit_bound(dtype: str, want: torch.Tensor) -> float:
    """How far an engine's logits of one request may lie from the plain implementation's. float32 is a true
    32-bit path: rounding of sums of a few hundred terms. bfloat16 rounds every activation between kernels
    to 8 bits of mantissa, so its bound scales with the logits themselves: 1.5 % of the request's largest."""
    if dtype == "float32":
        return 2e-5 * max(1.0, float(want.abs().max()))
    return 0.015 * float(want.abs().max())


def run_plan_engine(engine, steps):
    """Drives Engine.step directly the way bin/trace_run does; returns {id: [T, V] logits}."""
    slots, got = {}, {}
    for msg in steps:
        ids = [e["id"] for e in msg["entries"]]
        for rid in ids:
            if rid not in slots:
                slots[rid] = engine.open()
        logits = engine.step([slots[r] for r in ids], [e["tokens"] for e in msg["entries"]],
                             [e["want"] for e in msg["entries"]]).float().cpu()
        row = 0
        for e in msg["entries"]:
            k = len(e["want"])
            got.setdefault(e["id"], []).append(logits[row:row + k])
            row += k
        for rid in msg["end"]:
            engine.close(slots.pop(rid))
    engine.cache.check()
    return {rid: torch.cat(parts) for rid, parts in got.items()}


def run_plan_trace_run(folder: str, dtype: str, steps, max_tokens: int, vocab: int, env=None):
    """Runs bin/trace_run as a subprocess; returns {id: [T, V] logits}."""
    out = scratch_folder("llmie_trace_")
    text = "\n".join(json.dumps(s) for s in steps) + "\n"
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype,
                           "--out", out, "--max-tokens", str(max_tokens)], input=text, capture_output=True, text=True,
                          env=env, timeout=900)
    assert proc.returncode == 0, proc.stderr[-4000:]
    dones = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert dones == [f"done {s['step']}" for s in steps], proc.stdout[-2000:]
    got = {}
    for msg in steps:
        n_want = sum(len(e["want"]) for e in msg["entries"])
        path = os.path.join(out, f"{msg['step']}.f32")
        if n_want == 0:
            assert not os.path.exists(path)
            continue
        data = torch.from_numpy(np.fromfile(path, dtype="<f4").reshape(n_want, vocab).copy())
        row = 0
        for e in msg["entries"]:
            k = len(e["want"])
            got.setdefault(e["id"], []).append(data[row:row + k])
            row += k
    return {rid: torch.cat(parts) for rid, parts in got.items()}


def max_tokens_for(steps) -> int:
    """The most tokens live requests hold at any time, each rounded up to a multiple of 64."""
    held, peak = {}, 0
    for msg in steps:
        for e in msg["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum((v + 63) // 64 * 64 for v in held.values()))
        for rid in msg["end"]:
            held.pop(rid)
    return peak
