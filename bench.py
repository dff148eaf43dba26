"""Decode and prefill throughput of the engine on one B200, Llama 3.2 1B shape, random weights.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--only all|decode|prefill] [--shape 3b|8b] [--per-kernel [--per-kernel-out FILE]]

A "step" is one decode step of the whole batch (captured forward + sampling). The default run
is the Llama 3.2 1B benchmark configuration in bfloat16 with a batch of 8, 512-token prompts and a 4096-token
context limit. It prints ONE JSON line: `value` is decoded tokens per second over K timed steps
(CUDA events, after W warm-up steps); `e2e` is the same through `generate()` with host tokens
in and out every step; `prefill` is one 2,048-token prompt; `roofline` compares the decode
step with the bytes it must read (every weight once + the live requests' cache) at the measured
HBM bandwidth; `points` gives decode at batch 1 and 64; `shapes` holds the two larger workloads
(Llama 3.2 3B shape: 16 requests of unequal prompts through `generate()`; Llama 3.1 8B shape:
a 2,048-token prefill and decode at batch 64 after 1,024-token prompts), each with the number of
layers it ran and the number the shape has. Weights (2.5 GB and more) are far larger than
L2, so every step streams them from HBM; no extra L2 flush is needed (stated in `config`).

`--impl reference` runs the unmodified reference engine on the same workload (baseline/reference_arm.py).
`--shape 3b|8b` runs only that workload at full depth (or `--layers L`). `--per-kernel` times every
kernel of the eager decode step (batch 1, 8, 64) and of the 2,048-token prefill with CUDA events and
prints one table each: time, bytes, FLOPs and the fraction of the measured peak they amount to.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tok/s at batch 1/8/64; prefill tok/s at 2,048 tokens (Llama 3.2 1B)"

_LLAMA3 = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
           "original_max_position_embeddings": 8192}
_COMMON = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "rope_theta": 500000.0,
    "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "bos_token_id": 128000, "eos_token_id": 128001, "torch_dtype": "bfloat16",
}
# the benchmark configuration: the Llama 3.2 1B shape
CONFIG_1B = dict(_COMMON, num_hidden_layers=16, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8,
                 head_dim=64, intermediate_size=8192, rope_scaling=_LLAMA3, tie_word_embeddings=True)
# the two larger shapes of the benchmark set
CONFIG_3B = dict(_COMMON, num_hidden_layers=28, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8,
                 head_dim=128, intermediate_size=8192, rope_scaling=_LLAMA3, tie_word_embeddings=True)
CONFIG_8B = dict(_COMMON, num_hidden_layers=32, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
                 head_dim=128, intermediate_size=14336, rope_scaling=dict(_LLAMA3, factor=8.0),
                 tie_word_embeddings=False)
CONTEXT = 4096
PROMPT_LEN = 512
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]), "source": "measured"}
        except (OSError, ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timed work runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.samples = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        clocks, max_clocks, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for s in self.samples:
            try:
                clocks.append(int(float(s[0])))
                max_clocks.append(int(float(s[1])))
            except ValueError:
                continue
            for name, val in zip(names, s[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        clocks.sort()
        return {"sm_mhz": clocks[len(clocks) // 2] if clocks else None,
                "sm_max_mhz": max(max_clocks) if max_clocks else None, "reasons": sorted(reasons),
                "samples": len(clocks)}


def make_model_folder(cfg: dict, n_layers: int, seed: int, tag: str) -> str:
    from llm_infer_engine_b200 import write_random_model
    from llm_infer_engine_b200.weights import scratch_folder
    cfg = dict(cfg)
    cfg["num_hidden_layers"] = n_layers
    folder = scratch_folder(f"llmie_bench_{tag}_")          # deleted at exit: these folders are gigabytes
    t0 = time.time()
    write_random_model(cfg, folder, seed=seed, std=0.02)
    print(f"[bench] wrote a random {n_layers}-layer {tag} model folder in {time.time() - t0:.1f}s", file=sys.stderr)
    return folder


def drop_folder(folder: str) -> None:
    import shutil
    shutil.rmtree(folder, ignore_errors=True)


def random_prompts(lengths, vocab: int, seed: int):
    import torch
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, vocab, (int(n),), generator=g).tolist() for n in lengths]


def time_decode(engine, batch: int, prompt_len: int, steps: int, warmup: int, seed: int):
    """Device time of `steps` decode steps of `batch` sequences after prompts of `prompt_len` tokens.
    Returns (seconds, mean context length over the timed steps, launches of this library's kernels)."""
    import torch
    from llm_infer_engine_b200.engine.engine import bucket_for
    from llm_infer_engine_b200.kernels import ops
    cache = engine.cache
    prompts = random_prompts([prompt_len] * batch, engine.vocab_size, seed)
    slots = [engine.open() for _ in range(batch)]
    try:
        logits = engine.step(slots, prompts, "last")
        sampled = torch.empty(batch, dtype=torch.int32, device=engine.device)
        ops.sample(logits, sampled)
        graph = engine.decode_graph(bucket_for(batch), prompt_len + warmup + steps + 1)
        graph.set_lanes(slots)
        graph.tokens[:batch].copy_(sampled)

        def one_step():
            for s in slots:
                cache.reserve(s, cache.lengths[s] + 1)
            out = graph.replay()
            for s in slots:
                cache.note_appended(s, cache.lengths[s] + 1, device_updated=True)
            ops.sample(out[:batch], graph.tokens)      # greedy; feeds the next step on the device

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        ctx0 = cache.lengths[slots[0]]
        launches0 = ops.LAUNCHES
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            one_step()
        end.record()
        torch.cuda.synchronize()
        seconds = start.elapsed_time(end) / 1e3
        mean_ctx = ctx0 + (steps + 1) / 2.0
        return seconds, mean_ctx, ops.LAUNCHES - launches0
    finally:
        for s in slots:
            engine.close(s)


def time_prefill(engine, n_tokens: int, warmup: int, reps: int, seed: int):
    """Median time of a one-prompt step: host token ids in, logits of the last row on the device."""
    import torch
    prompt = random_prompts([n_tokens], engine.vocab_size, seed)[0]
    times = []
    for i in range(warmup + reps):
        slot = engine.open()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([slot], [prompt], "last")
        end.record()
        torch.cuda.synchronize()
        engine.close(slot)
        if i >= warmup:
            times.append(start.elapsed_time(end) / 1e3)
    times.sort()
    return times[len(times) // 2]


def prefill_flops(cfg: dict, n_layers: int, lengths) -> float:
    """GEMM and causal-attention FLOPs of a prompt step over sequences of these lengths; the head runs on the
    last row of each."""
    d, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    hq, hkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_token = 2 * (d * (hq + 2 * hkv) * hd + hq * hd * d + 3 * d * ff)
    total = 0.0
    for T in lengths:
        total += n_layers * per_token * T + 2 * d * V
        total += n_layers * 4 * hq * hd * (T * (T + 1) / 2)      # causal QK^T and PV
    return total


def e2e_decode(engine, batch: int, steps: int, seed: int):
    """Decoded tokens per second through generate(): host prompts in, host tokens out every step."""
    from llm_infer_engine_b200 import GenerationStats, SamplingParams, generate
    prompts = random_prompts([PROMPT_LEN] * batch, engine.vocab_size, seed)
    generate(engine, prompts[:batch], max_new_tokens=8, stop_ids=[])            # warm-up: graphs, pools
    stats = GenerationStats()
    generate(engine, prompts, max_new_tokens=steps + 1, sampling=SamplingParams(), stop_ids=[], stats=stats)
    return stats.decode_tokens / stats.decode_seconds, stats


def workload_config(args, n_layers: int, pk: dict) -> dict:
    """The `config` of the JSON line: the workload and every layer size, the same for both arms."""
    c = CONFIG_1B
    return {
        "model": "Llama-3.2-1B shape", "global_batch": args.batch, "seq_len": CONTEXT, "parallelism": "single GPU",
        "layers": n_layers, "layers_full": c["num_hidden_layers"], "hidden_size": c["hidden_size"],
        "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
        "intermediate_size": c["intermediate_size"], "vocab_size": c["vocab_size"], "prompt_len": PROMPT_LEN,
        "new_tokens": args.steps, "prefill_tokens": PREFILL_TOKENS, "sampling": "greedy",
        "l2": "weights 2.5 GB per step >> 126 MB L2, no flush needed", "peaks": pk["source"],
    }


# ------------------------------------------------------------------------------------------ larger shapes
def run_3b(n_layers: int, pk: dict, new_tokens: int = 256) -> dict:
    """Llama 3.2 3B shape: 16 requests with prompt lengths uniform in [128, 2048] start together (one ragged
    prompt step), each generates `new_tokens`; through generate(), host tokens in and out."""
    import torch
    from llm_infer_engine_b200 import Engine, GenerationStats, generate
    cfg = CONFIG_3B
    folder = make_model_folder(cfg, n_layers, seed=3, tag="3b")
    g = torch.Generator().manual_seed(33)
    lens = [int(x) for x in torch.randint(128, 2049, (16,), generator=g)]
    total = sum((n + new_tokens + 64) // 64 * 64 for n in lens)
    engine = Engine(folder, dtype="bfloat16", device=0, max_batch=16, max_seq_len=CONTEXT, max_tokens=total)
    drop_folder(folder)
    prompts = random_prompts(lens, engine.vocab_size, seed=34)
    # warm-up with the same lengths: the sequences outgrow a captured step's length bucket on the way (2,048 to
    # 4,096), and capturing the next one belongs to start-up, not to the steps that are timed
    generate(engine, prompts, max_new_tokens=new_tokens, stop_ids=[])
    # three timed runs, the median of each figure: the prompt step is a single eager step of 18 thousand tokens
    # and its time scatters from run to run
    runs = []
    for _ in range(3):
        st = GenerationStats()
        generate(engine, prompts, max_new_tokens=new_tokens, stop_ids=[], stats=st)
        runs.append(st)
    print("[bench] 3B runs: prefill ms " + ", ".join(f"{r.prefill_seconds * 1e3:.1f}" for r in runs) + "; decode ms/step "
          + ", ".join(f"{r.decode_seconds / r.decode_steps * 1e3:.3f}" for r in runs), file=sys.stderr)
    stats = sorted(runs, key=lambda r: r.decode_seconds)[1]
    stats.prefill_seconds = sorted(r.prefill_seconds for r in runs)[1]
    steps = stats.decode_steps
    mean_keys = sum(lens) + 16 * (steps + 1) / 2.0                               # keys all 16 hold, mean over the steps
    step_bytes = engine.weight_bytes_per_step() + engine.kv_bytes_per_token() * mean_keys
    achieved = step_bytes / (stats.decode_seconds / steps) / 1e9
    flops = prefill_flops(cfg, n_layers, lens)
    out = {
        "model": "Llama-3.2-3B shape", "layers": n_layers, "layers_full": cfg["num_hidden_layers"],
        "requests": 16, "prompt_tokens": sum(lens), "new_tokens": new_tokens,
        "decode_tok_s": round(stats.decode_tokens / stats.decode_seconds, 1),
        "decode_ms_per_step": round(stats.decode_seconds / steps * 1e3, 4),
        "decode_gbs": round(achieved, 1), "decode_frac_hbm": round(achieved / pk["hbm_gbs"], 4),
        "prefill_tok_s": round(stats.prefill_tokens / stats.prefill_seconds, 1),
        "prefill_ms": round(stats.prefill_seconds * 1e3, 3),
        "prefill_frac_bf16": round(flops / stats.prefill_seconds / (pk["bf16_tflops"] * 1e12), 4),
        "path": "generate(): host tokens in and out every step", "timed_runs": 3,
    }
    del engine
    torch.cuda.empty_cache()
    return out


def run_8b(n_layers: int, pk: dict, steps: int, warmup: int) -> dict:
    """Llama 3.1 8B shape: one 2,048-token prefill; decode at batch 64 after 1,024-token prompts. The cache is
    sized by need (64 sequences of 1,024 + the decoded tokens), not for 64 x 8,192."""
    import torch
    from llm_infer_engine_b200 import Engine
    cfg = CONFIG_8B
    folder = make_model_folder(cfg, n_layers, seed=4, tag="8b")
    prompt_len, batch = 1024, 64
    per_seq = (prompt_len + steps + warmup + 64 + 63) // 64 * 64
    engine = Engine(folder, dtype="bfloat16", device=0, max_batch=batch, max_seq_len=8192, max_tokens=batch * per_seq)
    drop_folder(folder)
    sec, mean_ctx, _ = time_decode(engine, batch, prompt_len, steps, warmup, seed=44)
    step_bytes = engine.weight_bytes_per_step() + engine.kv_bytes_per_token() * mean_ctx * batch
    achieved = step_bytes / (sec / steps) / 1e9
    prefill_s = time_prefill(engine, PREFILL_TOKENS, warmup=3, reps=3, seed=45)
    flops = prefill_flops(cfg, n_layers, [PREFILL_TOKENS])
    out = {
        "model": "Llama-3.1-8B shape", "layers": n_layers, "layers_full": cfg["num_hidden_layers"],
        "decode_batch": batch, "prompt_len": prompt_len, "new_tokens": steps,
        "decode_tok_s": round(batch * steps / sec, 1), "decode_ms_per_step": round(sec / steps * 1e3, 4),
        "decode_gbs": round(achieved, 1), "decode_frac_hbm": round(achieved / pk["hbm_gbs"], 4),
        "prefill_tokens": PREFILL_TOKENS, "prefill_tok_s": round(PREFILL_TOKENS / prefill_s, 1),
        "prefill_ms": round(prefill_s * 1e3, 3),
        "prefill_frac_bf16": round(flops / prefill_s / (pk["bf16_tflops"] * 1e12), 4),
    }
    del engine
    torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------ per-kernel report
def kernel_table(rows, n_steps: int, pk: dict, title: str) -> str:
    """Markdown table of a KernelTimer's rows, per step: microseconds, share, bytes -> GB/s and the fraction of
    the measured copy bandwidth, FLOPs -> TFLOP/s and the fraction of the measured bf16 GEMM rate."""
    total = sum(r["us"] for r in rows) or 1.0
    lines = [f"### {title}", "",
             "| stage | kernel | launches/step | us/step | share | MB/step | GB/s | of HBM peak | GFLOP/step | TFLOP/s | "
             "of bf16 peak |", "|---|---|---|---|---|---|---|---|---|---|---|"]
    for r in sorted(rows, key=lambda r: -r["us"]):
        us = r["us"] / n_steps
        sec = us * 1e-6
        gbs = r["bytes"] / n_steps / sec / 1e9 if sec > 0 else 0.0
        tf = r["flops"] / n_steps / sec / 1e12 if sec > 0 else 0.0
        lines.append(f"| {r['stage']} | {r['kernel']} | {r['launches'] / n_steps:.0f} | {us:.1f} | "
                     f"{100 * r['us'] / total:.1f} % | {r['bytes'] / n_steps / 1e6:.2f} | {gbs:.0f} | "
                     f"{100 * gbs / pk['hbm_gbs']:.1f} % | {r['flops'] / n_steps / 1e9:.2f} | {tf:.1f} | "
                     f"{100 * tf / pk['bf16_tflops']:.1f} % |")
    lines.append(f"| | **sum** | {sum(r['launches'] for r in rows) / n_steps:.0f} | {total / n_steps:.1f} | | "
                 f"{sum(r['bytes'] for r in rows) / n_steps / 1e6:.2f} | | | "
                 f"{sum(r['flops'] for r in rows) / n_steps / 1e9:.2f} | | |")
    return "\n".join(lines) + "\n"


def run_per_kernel(args, engine, pk: dict) -> str:
    """Times every kernel of the EAGER step with CUDA events (no graph, no overlap between kernels, so the sum
    is above the captured step's time). Peaks are the measured ones."""
    import torch
    from llm_infer_engine_b200.kernels import ops, trace
    n_layers = engine.config.num_hidden_layers
    parts = [f"Per-kernel times, Llama 3.2 1B shape, {n_layers} layers, bfloat16, eager steps bracketed by CUDA events "
             f"(peaks: {pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s, {pk['source']}).\n"]
    n_steps = 8
    for batch in (1, 8, 64):
        prompts = random_prompts([PROMPT_LEN] * batch, engine.vocab_size, seed=10 + batch)
        slots = [engine.open() for _ in range(batch)]
        logits = engine.step(slots, prompts, "last")
        tokens = torch.empty(batch, dtype=torch.int32, device=engine.device)
        ops.sample(logits, tokens)
        for _ in range(3):                                  # warm-up, untimed
            logits = engine.step(slots, [[t] for t in tokens.tolist()], "last")
            ops.sample(logits, tokens)
        with trace.timing() as timer:
            for _ in range(n_steps):
                logits = engine.step(slots, [[t] for t in tokens.tolist()], "last")
                trace.push("Sample")
                ops.sample(logits, tokens)
                trace.pop()
            rows = timer.table()
        for s in slots:
            engine.close(s)
        parts.append(kernel_table(rows, n_steps, pk, f"decode, batch {batch}, context {PROMPT_LEN + 4}..{PROMPT_LEN + 4 + n_steps}"))
    prompt = random_prompts([PREFILL_TOKENS], engine.vocab_size, seed=99)[0]
    for i in range(3):
        slot = engine.open()
        engine.step([slot], [prompt], "last")
        engine.close(slot)
    with trace.timing() as timer:
        for _ in range(3):
            slot = engine.open()
            engine.step([slot], [prompt], "last")
            engine.close(slot)
        rows = timer.table()
    parts.append(kernel_table(rows, 3, pk, f"prefill, one prompt of {PREFILL_TOKENS} tokens"))
    return "\n".join(parts)


# ------------------------------------------------------------------------------------------ attention kernels alone
def attention_sweep(heads: int, kv_heads: int, head_dim: int, pk: dict) -> str:
    """The two attention kernels alone, at several batch sizes and context lengths, against the measured peaks:
    the one-token kernel by the cache bytes it has to read, the prompt kernel by its FLOPs. Every case is 16
    launches in one CUDA graph over caches that rotate through more than the L2 holds; CUDA events around two
    replays."""
    import torch
    from llm_infer_engine_b200.kernels import ops
    dev, P = "cuda", 64
    ops.set_pdl(False)                      # a launch may not start while the one before it runs: these are kernel times

    def timed(call, n=16):
        for i in range(3):
            call(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n):
                call(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) * 1e3 / (2 * n)

    lines = [f"Attention kernels alone, {heads} query / {kv_heads} KV heads of {head_dim}, bfloat16 "
             f"(peaks: {pk['hbm_gbs']:.0f} GB/s, {pk['bf16_tflops']:.0f} TFLOP/s, {pk['source']}).", "",
             "### one token a sequence (`attention_decode_mma` with rotation and cache write inside)", "",
             "| batch | context | MB of cache read | us | GB/s | of HBM peak |", "|---|---|---|---|---|---|"]
    gen = torch.Generator(device=dev).manual_seed(0)
    for batch, ctx in [(1, 512), (8, 512), (32, 512), (64, 512), (128, 512), (64, 1024), (16, 1200), (8, 3500),
                       (64, 3500)]:
        pages_per = (ctx + 16 + P - 1) // P
        nbytes = batch * ctx * kv_heads * head_dim * 2 * 2
        copies = max(2, int(300e6 // nbytes) + 1)
        ks = [torch.randn(batch * pages_per + 1, kv_heads, P, head_dim, device=dev, generator=gen).to(torch.bfloat16)
              for _ in range(copies)]
        vs = [torch.randn(batch * pages_per + 1, kv_heads, P, head_dim, device=dev, generator=gen).to(torch.bfloat16)
              for _ in range(copies)]
        table = torch.randperm(batch * pages_per, device=dev, generator=gen).to(torch.int32).view(batch, pages_per)
        qkv = torch.randn(batch, (heads + 2 * kv_heads) * head_dim, device=dev, generator=gen).to(torch.bfloat16)
        out = torch.empty(batch, heads * head_dim, dtype=torch.bfloat16, device=dev)
        rope = torch.randn(ctx + 64, head_dim // 2, 2, device=dev, generator=gen)
        slots = torch.arange(batch, device=dev, dtype=torch.int32)
        lens = torch.full((batch,), ctx, device=dev, dtype=torch.int32)
        pages = ops.attention_decode_mma_pages(batch, heads, kv_heads, ctx)
        n_runs = ((ctx + 63) // 64 + pages - 1) // pages
        counters = torch.zeros(ops.decode_counter_ints(batch, heads, kv_heads) + 64, dtype=torch.int32, device=dev)
        scratch = torch.empty(max(1, ops.decode_scratch_floats(batch, heads, head_dim, n_runs)), dtype=torch.float32,
                              device=dev)
        us = timed(lambda i: ops.attention_decode_mma_rope(
            qkv, ks[i % copies], vs[i % copies], out, rope, slots, lens, table.contiguous(), P, heads, kv_heads,
            head_dim, head_dim ** -0.5, 0, pages, n_runs, True, counters=counters, scratch=scratch))
        gbs = nbytes / us / 1e3
        lines.append(f"| {batch} | {ctx} | {nbytes / 1e6:.1f} | {us:.1f} | {gbs:.0f} | {100 * gbs / pk['hbm_gbs']:.0f} % |")
        del ks, vs
    lines += ["", "### prompts (`attention_prefill_tc`, causal, from position 0)", "",
              "| prompts | tokens each | GFLOP | us | TFLOP/s | of bf16 peak |", "|---|---|---|---|---|---|"]
    for n_seqs, T in [(8, 512), (3, 1000), (1, 2048), (1, 4096), (1, 8192), (4, 2048)]:
        pages_per = (T + P - 1) // P
        k = torch.randn(n_seqs * pages_per + 1, kv_heads, P, head_dim, device=dev, generator=gen).to(torch.bfloat16)
        v = torch.randn(n_seqs * pages_per + 1, kv_heads, P, head_dim, device=dev, generator=gen).to(torch.bfloat16)
        table = torch.arange(n_seqs * pages_per, device=dev, dtype=torch.int32).view(n_seqs, pages_per).contiguous()
        q = torch.randn(n_seqs * T, heads * head_dim, device=dev, generator=gen).to(torch.bfloat16)
        out = torch.empty_like(q)
        cu = torch.arange(0, (n_seqs + 1) * T, T, device=dev, dtype=torch.int32)
        slots = torch.arange(n_seqs, device=dev, dtype=torch.int32)
        start = torch.zeros(n_seqs, device=dev, dtype=torch.int32)
        us = timed(lambda i: ops.attention_prefill_tc(q, k, v, out, cu, slots, start, table, P, n_seqs, T, heads,
                                                      kv_heads, head_dim, head_dim ** -0.5, 0), n=8)
        ops.check_tc_status(dev)
        flops = n_seqs * 4.0 * heads * head_dim * (T * (T + 1) / 2)
        tf = flops / us / 1e6
        lines.append(f"| {n_seqs} | {T} | {flops / 1e9:.1f} | {us:.1f} | {tf:.0f} | {100 * tf / pk['bf16_tflops']:.0f} % |")
        del k, v, q, out
    ops.set_pdl(True)
    return "\n".join(lines)


# ------------------------------------------------------------------------------------------ the two arms
def run_ours(args):
    import torch
    if not torch.cuda.is_available():
        print(json.dumps({"metric": METRIC, "error": "no CUDA device"}))
        return 1
    from llm_infer_engine_b200 import Engine
    pk = peaks()
    if args.attention_sweep:
        text = attention_sweep(args.heads, args.kv_heads, args.head_dim, pk)
        print(text)
        if args.per_kernel_out:
            with open(args.per_kernel_out, "w", encoding="utf-8") as f:
                f.write(text + "\n")
        return 0
    if args.shape:                                          # one of the larger workloads alone, at full depth
        cfg = CONFIG_3B if args.shape == "3b" else CONFIG_8B
        n = args.layers or cfg["num_hidden_layers"]
        out = run_3b(n, pk) if args.shape == "3b" else run_8b(n, pk, args.steps, args.warmup)
        print(json.dumps({"metric": METRIC, "impl": "ours", "dtype": "bf16", "shape": out}))
        return 0
    full_layers = CONFIG_1B["num_hidden_layers"]
    n_layers = args.layers or full_layers
    folder = make_model_folder(CONFIG_1B, n_layers, seed=2, tag="1b")
    max_batch = max(64, args.batch)
    per_seq = PROMPT_LEN + args.steps + args.warmup + 64
    engine = Engine(folder, dtype="bfloat16", device=0, max_batch=max_batch, max_seq_len=CONTEXT,
                    max_tokens=max(max_batch * ((per_seq + 63) // 64 * 64), PREFILL_TOKENS + 64), cuda_graph=True)
    drop_folder(folder)
    if args.per_kernel:
        text = run_per_kernel(args, engine, pk)
        if args.per_kernel_out:
            with open(args.per_kernel_out, "w") as f:
                f.write(text)
        print(text, file=sys.stderr)
    sampler = ClockSampler(0)
    sampler.start()
    results = {}
    launches = 0
    batches = (args.batch, 1, 64) if args.only == "all" else ((args.batch,) if args.only == "decode" else ())
    for batch in batches:
        if batch in results:
            continue
        sec, mean_ctx, n_launch = time_decode(engine, batch, PROMPT_LEN, args.steps, args.warmup, seed=10 + batch)
        results[batch] = (sec, mean_ctx)
        if batch == args.batch:
            launches = n_launch
    prefill_s = None
    if args.only in ("all", "prefill"):
        prefill_s = time_prefill(engine, PREFILL_TOKENS, warmup=max(3, min(args.warmup, 5)),
                                 reps=5 if args.only == "all" else 2, seed=99)
    e2e_tps = None
    if args.only == "all":
        e2e_tps, stats = e2e_decode(engine, args.batch, args.steps, seed=10 + args.batch)
    sampler.stop()

    flops = prefill_flops(CONFIG_1B, n_layers, [PREFILL_TOKENS])
    out = {
        "metric": METRIC, "value": None, "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": None, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), "
        "uniform-random token ids", "impl": "ours",
        "config": workload_config(args, n_layers, pk),
        "impl_notes": {"path": "generate() / captured one-token steps", "head": "tied to the embedding"},
        "gpu_launches": int(launches),
    }
    if args.batch in results:
        sec, mean_ctx = results[args.batch]
        step_bytes = engine.weight_bytes_per_step() + engine.kv_bytes_per_token() * mean_ctx * args.batch
        achieved = step_bytes / (sec / args.steps) / 1e9
        out["value"] = round(args.batch * args.steps / sec, 1)
        out["ms_per_step"] = round(sec / args.steps * 1e3, 4)
        out["roofline"] = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                           "frac": round(achieved / pk["hbm_gbs"], 4)}
    if e2e_tps is not None:
        out["e2e"] = {"value": round(e2e_tps, 1), "unit": "tokens/s", "h2d_bytes_per_step": 4 * args.batch,
                      "d2h_bytes_per_step": 4 * args.batch}
    if prefill_s is not None:
        out["prefill"] = {"value": round(PREFILL_TOKENS / prefill_s, 1), "tokens": PREFILL_TOKENS,
                          "ms": round(prefill_s * 1e3, 3),
                          "frac": round(flops / prefill_s / (pk["bf16_tflops"] * 1e12), 4)}
    if 1 in results and 64 in results:
        out["points"] = {f"decode_b{b}": round(b * args.steps / results[b][0], 1) for b in (1, 64)}
    out["clocks"] = sampler.summary()
    if args.only == "all" and not args.layers and not args.no_shapes:
        del engine
        torch.cuda.empty_cache()
        # the larger shapes: the 3B one at full depth, the 8B one at half depth (its folder of random weights
        # would be 16 GB; both numbers are in the record)
        out["shapes"] = {"llama_3b_ragged16": run_3b(CONFIG_3B["num_hidden_layers"], pk),
                         "llama_8b_b64": run_8b(CONFIG_8B["num_hidden_layers"] // 2, pk, min(args.steps, 64), 5)}
    print(json.dumps(out))
    return 0


def run_reference(args):
    """The unmodified reference on the same workload (baseline/reference_arm.py): the same JSON keys, with
    `"impl": "reference"`. Whatever stops it is reported with its own text in an `unavailable` line."""
    sys.path.insert(0, os.path.join(ROOT, "baseline"))
    try:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device")
        import reference_arm
        n_layers = args.layers or CONFIG_1B["num_hidden_layers"]
        arm = reference_arm.ReferenceArm(CONFIG_1B, n_layers, CONTEXT)
        pk = peaks()
        arm.compile_pass(args.batch, PROMPT_LEN)
        sampler = ClockSampler(0)
        sampler.start()
        sec, mean_ctx = arm.decode(args.batch, PROMPT_LEN, args.steps, args.warmup, seed=10 + args.batch,
                                   host_io=False)
        points = {}
        prefill_s = e2e_sec = None
        if args.only == "all":
            e2e_sec, _ = arm.decode(args.batch, PROMPT_LEN, args.steps, args.warmup, seed=10 + args.batch,
                                    host_io=True)
            for b in (1, 64):
                arm.compile_pass(b, PROMPT_LEN)
                s_b, _ = arm.decode(b, PROMPT_LEN, args.steps, args.warmup, seed=10 + b, host_io=True)
                points[f"decode_b{b}"] = round(b * args.steps / s_b, 1)
            s_g, _ = arm.decode(1, PROMPT_LEN, args.steps, args.warmup, seed=11, host_io=True, graph=True)
            points["decode_b1_graph"] = round(args.steps / s_g, 1)
            prefill_s = arm.prefill(PREFILL_TOKENS, warmup=3, reps=5, seed=99)
        sampler.stop()
    except Exception as exc:                                   # noqa: BLE001 - the reason goes into the line
        text = " ".join(f"{type(exc).__name__}: {exc}".split())[:400]
        print(json.dumps({"impl": "reference", "unavailable": text}))
        return 0
    step_bytes = arm.weight_bytes_per_step() + arm.kv_bytes_per_token() * mean_ctx * args.batch
    achieved = step_bytes / (sec / args.steps) / 1e9
    out = {
        "metric": METRIC, "value": round(args.batch * args.steps / sec, 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(sec / args.steps * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: the reference's own random initialisation, uniform-random token ids",
        "impl": "reference", "config": workload_config(args, n_layers, pk),
        "impl_notes": {"path": "Llama3.forward + KVCache + sample, eager (its graph runner serves batch 1 only: "
                               "points.decode_b1_graph)", "head": "separate output matrix (its random mode)"},
        "gpu_launches": 0,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if e2e_sec is not None:
        out["e2e"] = {"value": round(args.batch * args.steps / e2e_sec, 1), "unit": "tokens/s",
                      "h2d_bytes_per_step": 8 * args.batch, "d2h_bytes_per_step": 8 * args.batch}
    if prefill_s is not None:
        flops = prefill_flops(CONFIG_1B, n_layers, [PREFILL_TOKENS])
        out["prefill"] = {"value": round(PREFILL_TOKENS / prefill_s, 1), "tokens": PREFILL_TOKENS,
                          "ms": round(prefill_s * 1e3, 3),
                          "frac": round(flops / prefill_s / (pk["bf16_tflops"] * 1e12), 4)}
    if points:
        out["points"] = points
    out["clocks"] = sampler.summary()
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--prompt-len", type=int, default=512,
                    help="tokens every sequence holds before decoding starts (the benchmark's 512; up to the context)")
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the configuration (0 = all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--only", default="all", choices=["all", "decode", "prefill"],
                    help="measure only one part (for short profiler captures); the JSON line then lacks the rest")
    ap.add_argument("--shape", default="", choices=["", "3b", "8b"],
                    help="run only the Llama 3.2 3B or Llama 3.1 8B workload, at full depth unless --layers is given")
    ap.add_argument("--no-shapes", action="store_true", help="leave the 3B and 8B workloads out of the default run")
    ap.add_argument("--per-kernel", action="store_true",
                    help="also time every kernel of the eager steps and print the tables (stderr)")
    ap.add_argument("--per-kernel-out", default="", help="write the per-kernel tables to this file as well")
    ap.add_argument("--attention-sweep", action="store_true",
                    help="time the two attention kernels alone at several batch sizes and contexts; prints a table")
    ap.add_argument("--heads", type=int, default=32, help="query heads of --attention-sweep")
    ap.add_argument("--kv-heads", type=int, default=8, help="KV heads of --attention-sweep")
    ap.add_argument("--head-dim", type=int, default=64, choices=[64, 128], help="head size of --attention-sweep")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this library runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    global PROMPT_LEN
    PROMPT_LEN = max(1, min(args.prompt_len, CONTEXT - args.steps - max(args.warmup, 3) - 8))
    if args.impl == "reference":
        return run_reference(args)
    if args.warmup < 3:
        args.warmup = 3
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
