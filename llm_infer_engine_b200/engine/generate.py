"""The generation loop above the step function.

Requests are taken in order, as many at a time as the cache has slots and pages for; a batch's
prompts (of unequal lengths) run in one step, then every live sequence advances one token per
step. A sequence ends at a stop token (which is kept in its output, as the reference keeps the
EOS it sampled, main.py:261,270-272), after max_new_tokens, or when the cache's per-sequence
limit is reached (main.py:274); it leaves the batch at once and its slot is given back. No
request joins a running batch: the next batch starts when the current one is finished.
Sampled token ids come back to the host once per step, as the reference's `.item()` does
(main.py:260), because the loop's decisions are made there.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

import torch

from ..kernels import ops, trace
from ..sampling.sampler import SamplingParams
from .engine import Engine, EngineError, bucket_for


@dataclass
class GenerationStats:
    prefill_tokens: int = 0
    prefill_seconds: float = 0.0
    decode_tokens: int = 0
    decode_steps: int = 0
    decode_seconds: float = 0.0
    batches: int = 0


def plan_batch(prompt_lens: Sequence[int], max_new_tokens: int, free_slots: int, free_pages: int, page_size: int,
               max_seq_len: int) -> int:
    """How many of the waiting requests (in order) start together: each needs a slot and pages for
    its prompt plus the tokens it may generate (capped by max_seq_len). At least one must fit."""
    taken, pages = 0, 0
    for plen in prompt_lens:
        if taken >= free_slots:
            break
        total = min(plen + max_new_tokens, max_seq_len)
        need = (total + page_size - 1) // page_size
        if pages + need > free_pages:
            break
        pages += need
        taken += 1
    return taken


def finished_reason(token: int, n_generated: int, length: int, stop_ids, max_new_tokens: int, max_seq_len: int):
    """Why a sequence ends after sampling `token` (None = it goes on). `length` counts the tokens
    in the cache; the sampled token is not yet among them."""
    if token in stop_ids:
        return "stop"
    if n_generated >= max_new_tokens:
        return "length"
    if length >= max_seq_len:
        return "max_seq_len"
    return None


def generate(engine: Engine, prompts: Sequence[Sequence[int]], max_new_tokens: int = 256,
             sampling: Optional[SamplingParams] = None, stop_ids: Optional[Sequence[int]] = None,
             on_tokens: Optional[Callable[[List[int], List[int]], None]] = None,
             stats: Optional[GenerationStats] = None) -> List[List[int]]:
    """Generates up to max_new_tokens for every prompt (lists of token ids); returns the new
    tokens of each, in the order given. `stop_ids` defaults to the model's eos ids.
    `on_tokens(request_indices, tokens)` is called after every step with what was just sampled."""
    sampling = sampling or SamplingParams()
    stop = set(engine.model.spec.stop_token_ids if stop_ids is None else stop_ids)
    if max_new_tokens < 1:
        raise EngineError("max_new_tokens must be at least 1")
    for i, p in enumerate(prompts):
        if len(p) == 0:
            raise EngineError(f"prompt {i} is empty")
        if len(p) >= engine.max_seq_len + 1:
            raise EngineError(f"prompt {i} has {len(p)} tokens, more than max_seq_len {engine.max_seq_len}")
    stats = stats if stats is not None else GenerationStats()
    outputs: List[List[int]] = [[] for _ in prompts]
    cache = engine.cache
    dev = engine.device
    host_tokens = torch.empty(max(engine.max_batch, 1), dtype=torch.int32).pin_memory()
    next_request = 0
    while next_request < len(prompts):
        waiting = [len(p) for p in prompts[next_request:]]
        k = plan_batch(waiting, max_new_tokens, cache.free_slots(), cache.free_pages(), cache.page_size,
                       engine.max_seq_len)
        if k == 0:
            raise EngineError(f"request {next_request} ({waiting[0]} prompt tokens + {max_new_tokens} new) does "
                              "not fit the cache even alone; raise max_tokens or max_seq_len")
        batch = list(range(next_request, next_request + k))
        next_request += k
        stats.batches += 1
        _run_batch(engine, prompts, batch, outputs, max_new_tokens, sampling, stop, on_tokens, stats, host_tokens)
    return outputs


def _run_batch(engine, prompts, batch, outputs, max_new_tokens, sampling, stop, on_tokens, stats, host_tokens):
    cache = engine.cache
    dev = engine.device
    slots = [engine.open() for _ in batch]
    live = list(range(len(batch)))                  # indices into batch / slots
    try:
        # --- prompts, one step
        t0 = torch.cuda.Event(enable_timing=True)
        t1 = torch.cuda.Event(enable_timing=True)
        t0.record()
        trace.push("Prefill")
        logits = engine.step(slots, [prompts[r] for r in batch], "last")
        n = len(batch)
        sampled = torch.empty(n, dtype=torch.int32, device=dev)
        seq_ids = torch.tensor(batch, dtype=torch.int32, device=dev)
        counters = torch.zeros(n, dtype=torch.int32, device=dev)
        ops.sample(logits, sampled, sampling.temperature, sampling.top_p, sampling.seed, seq_ids, counters)
        host_tokens[:n].copy_(sampled, non_blocking=True)
        trace.pop()
        t1.record()
        t1.synchronize()
        stats.prefill_tokens += sum(len(prompts[r]) for r in batch)
        stats.prefill_seconds += t0.elapsed_time(t1) / 1e3
        new = host_tokens[:n].tolist()

        d0 = torch.cuda.Event(enable_timing=True)
        d1 = torch.cuda.Event(enable_timing=True)
        d0.record()
        trace.push("Decode")
        graph = None
        host_view = host_tokens.numpy()              # the same pinned memory, without tensor overheads
        stream = torch.cuda.current_stream()
        slack = 0          # steps for which no live sequence can end by a length limit (0 = look at each)
        while True:
            # --- the common step: nobody can end by length, nobody drew a stop token, the captured step
            # still serves. The next step is launched first; the bookkeeping runs while it does.
            if slack > 0 and graph is not None and longest < graph.kv_limit and stop.isdisjoint(new):
                in_view[:n] = new
                for s in live_slots:
                    cache.reserve(s, cache.lengths[s] + 1)
                graph.replay()
                if on_tokens is not None:
                    on_tokens([batch[i] for i in live], list(new))
                for i, tok in zip(live, new):
                    outputs[batch[i]].append(tok)
                for s in live_slots:
                    cache.note_appended(s, cache.lengths[s] + 1, device_updated=True)
                slack -= 1
                longest += 1
                stream.synchronize()
                new = out_view[:n].tolist()
                stats.decode_steps += 1
                stats.decode_tokens += n
                continue
            # --- decide on the host
            if on_tokens is not None:
                on_tokens([batch[i] for i in live], list(new))
            still, still_tokens = [], []
            for i, tok in zip(live, new):
                r = batch[i]
                outputs[r].append(tok)
                why = finished_reason(tok, len(outputs[r]), cache.lengths[slots[i]], stop, max_new_tokens,
                                      engine.max_seq_len)
                if why is None:
                    still.append(i)
                    still_tokens.append(tok)
                else:
                    engine.close(slots[i])
                    slots[i] = -1
            changed = still != live
            live = still
            if not live:
                break
            # --- one token each
            n = len(live)
            live_slots = [slots[i] for i in live]
            # the tokens go back in from (pinned) host memory, as the reference writes each sampled id
            # into its device input buffer (main.py:282): the host may have the last word on them
            if engine.use_cuda_graph:
                lanes = bucket_for(n)
                longest = max(cache.lengths[s] for s in live_slots) + 1
                if graph is None or graph.n != lanes or longest > graph.kv_limit:
                    # the upload of the tokens, the draw and the download of the drawn tokens are part of
                    # the captured step: one launch a step. A model with a part that cannot be captured makes
                    # this None and switches the engine to eager steps.
                    graph = engine.try_decode_graph(lanes, longest, sampling, host_io=True)
                    changed = True
                    if graph is not None:
                        in_view, out_view = graph.host_in.numpy(), graph.host_out.numpy()
            if engine.use_cuda_graph:
                for s in live_slots:
                    cache.reserve(s, cache.lengths[s] + 1)
                if changed:
                    graph.set_lanes(live_slots)
                    graph.seq_ids[:n].copy_(torch.tensor([batch[i] for i in live], dtype=torch.int32))
                    graph.counters[:n].copy_(torch.tensor([len(outputs[batch[i]]) for i in live], dtype=torch.int32))
                in_view[:n] = still_tokens
                graph.replay()
                # after this step every live sequence has one token more drawn and one more cached
                slack = min(min(max_new_tokens - len(outputs[batch[i]]), engine.max_seq_len - cache.lengths[slots[i]])
                            for i in live) - 1
                for s in live_slots:
                    cache.note_appended(s, cache.lengths[s] + 1, device_updated=True)
                stream.synchronize()
                new = out_view[:n].tolist()
            else:
                logits = engine.step(live_slots, [[t] for t in still_tokens], "last")
                if changed:
                    seq_ids = torch.tensor([batch[i] for i in live], dtype=torch.int32, device=dev)
                    counters = torch.tensor([len(outputs[batch[i]]) for i in live], dtype=torch.int32, device=dev)
                    sampled = torch.empty(n, dtype=torch.int32, device=dev)
                ops.sample(logits, sampled, sampling.temperature, sampling.top_p, sampling.seed, seq_ids, counters)
                # same stream: the upload in step() has read its pinned buffer before this download writes one
                host_tokens[:n].copy_(sampled[:n], non_blocking=True)
                stream.synchronize()
                new = host_view[:n].tolist()
            stats.decode_steps += 1
            stats.decode_tokens += n
        trace.pop()
        d1.record()
        d1.synchronize()
        stats.decode_seconds += d0.elapsed_time(d1) / 1e3
        ops.check_tc_status(dev)         # a kernel that gave up a bounded wait leaves a code here
    finally:
        for s in slots:
            if s >= 0 and cache.slots.is_held(s):
                engine.close(s)
