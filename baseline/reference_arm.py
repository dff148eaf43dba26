"""The reference arm of bench.py: the unmodified reference engine on the benchmark workload.

The reference (Analysis196884/llm-infer-engine) is a folder of plain Python files (`main.py`,
`src/*.py`, Triton kernels) without packaging metadata, so its install is a copy of that folder:
`install()` copies it to `baseline/_ref/`, and this module puts that folder on `sys.path` and
imports `src.*` from it. Nothing of this repository's package, kernels or shared objects is
imported here.

What is driven, all of it the reference's own code:
  * model construction with random weights as its `main.py` does in random mode:
    `Llama3(ModelArgs(...)).to(device, dtype=torch.bfloat16)` (main.py:418-434);
  * a fresh `KVCache(args, dtype)` per run (main.py:217);
  * prefill `model(tokens[B, S], start_pos=0, kv_cache=kv)` (main.py:236-240);
  * the decode loop of main.py:257-286: `sample(logits, temperature, top_p)`, the token read on
    the host, the token written into the device input buffer, `model(input, start_pos, kv_cache)`;
  * for batch 1 also its `CUDAGraphDecodeRunner` (src/cuda_graph.py:8-70), which is batch 1 only.
Its `generate_text` itself cannot be called: it needs a tokenizer folder, prints every token and
serves one sequence, so the loop above is restated around the same calls for a batch.
"""
from __future__ import annotations

import os
import shutil
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
REF_SOURCE = os.environ.get("LLMIE_REFERENCE_SRC", "/root/reference")


def install(verbose: bool = True) -> str:
    """Copies the reference tree (main.py, llama_chat.py, src/) into baseline/_ref if it is not there yet.
    Returns the folder, or raises FileNotFoundError when there is neither a copy nor a source."""
    if os.path.isfile(os.path.join(REF_DIR, "src", "model.py")):
        return REF_DIR
    if not os.path.isfile(os.path.join(REF_SOURCE, "src", "model.py")):
        raise FileNotFoundError(f"no reference tree at {REF_DIR} and none to copy from at {REF_SOURCE}")
    os.makedirs(REF_DIR, exist_ok=True)
    for name in ("main.py", "llama_chat.py", "README.md"):
        if os.path.isfile(os.path.join(REF_SOURCE, name)):
            shutil.copy2(os.path.join(REF_SOURCE, name), os.path.join(REF_DIR, name))
    shutil.copytree(os.path.join(REF_SOURCE, "src"), os.path.join(REF_DIR, "src"), dirs_exist_ok=True,
                    ignore=shutil.ignore_patterns("__pycache__"))
    if verbose:
        print(f"[reference] copied {REF_SOURCE} to {REF_DIR}", file=sys.stderr)
    return REF_DIR


class ReferenceArm:
    def __init__(self, cfg: dict, n_layers: int, context: int, device: str = "cuda:0"):
        import torch
        ref = install(verbose=False)
        if ref not in sys.path:
            sys.path.insert(0, ref)
        from src.config import ModelArgs            # noqa: the reference's own modules
        from src.cuda_graph import CUDAGraphDecodeRunner
        from src.kv_cache import KVCache
        from src.model import Llama3
        from src.sampler import sample
        self.torch = torch
        self.ModelArgs, self.KVCache, self.Runner, self.sample = ModelArgs, KVCache, CUDAGraphDecodeRunner, sample
        self.device = device
        self.cfg = cfg
        self.context = context
        self.n_layers = n_layers
        t0 = time.time()
        torch.manual_seed(2)
        self.model = Llama3(self._args(1)).to(device, dtype=torch.bfloat16)
        self.model.eval()
        print(f"[reference] Llama3 with random weights, {n_layers} layers, in {time.time() - t0:.1f}s", file=sys.stderr)

    def _args(self, max_batch: int):
        c = self.cfg
        return self.ModelArgs(dim=c["hidden_size"], n_layers=self.n_layers, n_heads=c["num_attention_heads"],
                              n_kv_heads=c["num_key_value_heads"], vocab_size=c["vocab_size"],
                              hidden_dim=c["intermediate_size"], norm_eps=c["rms_norm_eps"], max_batch_size=max_batch,
                              max_seq_len=self.context, rope_theta=c["rope_theta"], rope_scaling=c["rope_scaling"],
                              device=self.device)

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one decode step reads: every matrix and norm of every layer, the final norm and
        the output matrix (separate from the embedding in the reference's random mode)."""
        total = 0
        for name, p in self.model.named_parameters():
            if not name.startswith("tok_embeddings"):
                total += p.numel() * p.element_size()
        return total

    def kv_bytes_per_token(self) -> int:
        c = self.cfg
        hd = c["hidden_size"] // c["num_attention_heads"]
        return 2 * self.n_layers * c["num_key_value_heads"] * hd * 2

    def _prompts(self, batch: int, length: int, seed: int):
        torch = self.torch
        g = torch.Generator().manual_seed(seed)
        rows = [torch.randint(0, self.cfg["vocab_size"], (length,), generator=g) for _ in range(batch)]
        return torch.stack(rows).to(torch.long)

    def decode(self, batch: int, prompt_len: int, steps: int, warmup: int, seed: int, host_io: bool,
               graph: bool = False):
        """Seconds for `steps` decode steps of `batch` sequences after `prompt_len`-token prompts (CUDA
        events, after `warmup` steps), greedy. With host_io every step reads the sampled tokens on the
        host and writes them into the input buffer from there, as the reference's loop does; without it
        the sampled tokens stay on the device. `graph` uses the reference's graph runner (batch 1)."""
        torch = self.torch
        args = self._args(batch)
        with torch.no_grad():
            kv = self.KVCache(args, dtype=torch.bfloat16)
            runner = self.Runner(self.model, args, kv, self.device) if graph else None
            tokens = self._prompts(batch, prompt_len, seed).to(self.device)
            logits = self.model(tokens, start_pos=0, kv_cache=kv)
            pos = prompt_len
            input_buf = torch.zeros((batch, 1), dtype=torch.long, device=self.device)
            pinned = torch.zeros((batch, 1), dtype=torch.long).pin_memory()

            def one_step(logits, pos):
                nxt = self.sample(logits, temperature=0.0, top_p=1.0)          # [batch, 1]
                if graph:
                    return runner.decode(token_id=int(nxt.item()), current_pos=pos)
                if host_io:
                    pinned.copy_(nxt.cpu())                                    # the host reads the tokens
                    input_buf.copy_(pinned, non_blocking=True)
                else:
                    input_buf.copy_(nxt)
                return self.model(input_buf, start_pos=pos, kv_cache=kv)

            for _ in range(warmup):
                logits = one_step(logits, pos)
                pos += 1
            torch.cuda.synchronize()
            ctx0 = pos
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(steps):
                logits = one_step(logits, pos)
                pos += 1
            end.record()
            torch.cuda.synchronize()
            seconds = start.elapsed_time(end) / 1e3
        del kv, runner
        torch.cuda.empty_cache()
        return seconds, ctx0 + (steps + 1) / 2.0

    def compile_pass(self, batch: int, prompt_len: int):
        """A short throw-away run, so that every Triton specialisation the timed run meets (lengths that
        are and are not multiples of 16, both split counts) is compiled before anything is timed."""
        self.decode(batch, prompt_len, steps=20, warmup=0, seed=1, host_io=False)

    def prefill(self, n_tokens: int, warmup: int, reps: int, seed: int) -> float:
        torch = self.torch
        args = self._args(1)
        times = []
        with torch.no_grad():
            kv = self.KVCache(args, dtype=torch.bfloat16)
            host_tokens = self._prompts(1, n_tokens, seed).pin_memory()
            for i in range(warmup + reps):
                torch.cuda.synchronize()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                tokens = host_tokens.to(self.device, non_blocking=True)
                self.model(tokens, start_pos=0, kv_cache=kv)
                end.record()
                torch.cuda.synchronize()
                if i >= warmup:
                    times.append(start.elapsed_time(end) / 1e3)
        times.sort()
        return times[len(times) // 2]
