"""The engine: a model, its cache, and the one step function that everything above uses.

`step()` runs exactly the tokens it is given, as one batch, from the cache that earlier steps
left, and returns float32 logits at the wanted places. Sequences of a batch may have unequal
lengths; prompts go in one step, then one token each. Generation (`generate.py`) and trace
replay (`bin/trace_run`) both drive this function; there is no second forward pass.

The reference's step is `Llama3.forward(tokens[B, S], start_pos, kv_cache)` with one shared
start position and equal lengths (src/model.py:145-185), and its decode graph is B = 1 with
host rewrites per token (src/cuda_graph.py:57-70). Here a one-token step for a batch bucket is
captured once with all per-step inputs (tokens, slots, lengths) in device memory.
"""
from __future__ import annotations

import array
import gc
import itertools
import sys
from typing import Dict, List, Optional, Sequence, Union

import numpy as np
import torch

from ..cache.cache import Cache
from ..kernels import ops, trace
from ..weights.loader import build_model
from .context import StepContext

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


DEFAULT_MAX_SEQ_LEN = 4096


class EngineError(RuntimeError):
    pass


def resolve_dtype(dtype: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.float32, torch.bfloat16):
            raise EngineError(f"dtype {dtype} is not supported (bfloat16, float32)")
        return dtype
    if dtype not in _DTYPES:
        raise EngineError(f"dtype {dtype!r} is not supported (bfloat16, float32)")
    return _DTYPES[dtype]


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def _flatten_tokens(tokens, lens) -> np.ndarray:
    """All sequences' token ids as one int64 array. Lists of Python ints, numpy arrays and CPU
    tensors are taken; anything that is not an integer is refused."""
    parts = []
    try:
        if max(lens) < 128 and not isinstance(tokens[0], (np.ndarray, torch.Tensor)):
            # many short sequences (one-token steps): one pass over all of them
            return np.frombuffer(array.array("q", itertools.chain.from_iterable(tokens)), dtype=np.int64)
        for seq in tokens:
            if isinstance(seq, torch.Tensor):
                seq = seq.detach().cpu().numpy()
            if isinstance(seq, np.ndarray):
                if seq.dtype.kind not in "iu":
                    raise TypeError(f"token ids of dtype {seq.dtype}")
                parts.append(seq.reshape(-1).astype(np.int64, copy=False))
            else:
                parts.append(np.frombuffer(array.array("q", seq), dtype=np.int64))
    except (TypeError, ValueError, OverflowError) as exc:
        raise EngineError(f"step: token ids must be integers ({exc})") from None
    return parts[0] if len(parts) == 1 else np.concatenate(parts)


class Engine:
    def __init__(self, model_dir: str, dtype: Union[str, torch.dtype] = "bfloat16", device: Union[str, int] = 0,
                 max_batch: int = 8, max_seq_len: Optional[int] = None, max_tokens: Optional[int] = None,
                 cuda_graph: bool = True, nvtx: bool = False, decode_attention: str = "auto"):
        """max_batch: sequences held at once (slots). max_seq_len: longest sequence; the upper bound is the
        model's max_position_embeddings, the default is that bound but at most DEFAULT_MAX_SEQ_LEN (4096, the
        reference's default, main.py:40): a real checkpoint allows 131,072 positions, and a cache sized for
        that by default would take tens of gigabytes. max_tokens: positions all live sequences may hold
        together, in whole pages of 64 (default: max_batch * max_seq_len). nvtx: mark the stages of every
        step with NVTX ranges under the reference's names. decode_attention: "auto", or "split" to keep
        the CUDA-core split-KV kernel for every one-token step (for comparisons)."""
        if not torch.cuda.is_available():
            raise EngineError("no CUDA device: this library runs on a GPU only (there is no CPU path)")
        self.device = torch.device("cuda", device) if isinstance(device, int) else torch.device(device)
        if self.device.type != "cuda":
            raise EngineError(f"device {device!r} is not a CUDA device")
        torch.cuda.set_device(self.device)
        self.dtype = resolve_dtype(dtype)
        if decode_attention not in ("auto", "split"):
            raise EngineError(f"decode_attention must be 'auto' or 'split', got {decode_attention!r}")
        self.decode_attention = decode_attention
        if nvtx:
            trace.enable_ranges(True)
        self.model, self.config = build_model(model_dir, self.dtype, self.device,
                                              DEFAULT_MAX_SEQ_LEN if max_seq_len is None else max_seq_len)
        self.max_seq_len = self.model.runtime.max_positions
        self.max_batch = int(max_batch)
        page = 64
        if max_tokens is None:
            max_tokens = self.max_batch * _round_up(self.max_seq_len, page)
        self.cache = Cache(self.model.unit_requests, self.max_batch, int(max_tokens), self.max_seq_len, self.dtype,
                           self.device)
        self.vocab_size = self.model.vocab_size
        self.use_cuda_graph = bool(cuda_graph)
        from .plan import KernelPlan
        self.kernels = KernelPlan(self)
        self._graphs: Dict[tuple, "DecodeGraph"] = {}
        self._prefill_graphs: Dict[int, object] = {}        # prompt length -> False (seen once) or PrefillGraph
        self.launches = 0
        # a step's index arrays are written into pinned host memory and uploaded in one asynchronous copy
        self._staging_tensor = torch.empty(0, dtype=torch.int32)
        self._staging_done = torch.cuda.Event()

    # ---------------------------------------------------------------- sequences
    def open(self) -> int:
        """Takes a cache slot for a new sequence."""
        return self.cache.take_slot()

    def close(self, slot: int) -> None:
        """Gives the slot and everything it holds back."""
        self.cache.give_back_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.lengths[slot]

    def _staging(self, n_ints: int) -> np.ndarray:
        """A pinned int32 buffer of at least n_ints, free to be written: the upload of the step before
        has finished."""
        self._staging_done.synchronize()
        if self._staging_tensor.numel() < n_ints:
            self._staging_tensor = torch.empty(max(4096, 2 * n_ints), dtype=torch.int32).pin_memory()
        return self._staging_tensor.numpy()

    # ---------------------------------------------------------------- the step
    def step(self, slots: Sequence[int], tokens: Sequence[Sequence[int]],
             want: Union[str, Sequence[Sequence[int]]] = "last") -> torch.Tensor:
        """Appends tokens[i] to the sequence in slots[i] and returns float32 logits [R, vocab] at
        the wanted places: `want[i]` lists indices into tokens[i] ("last" = the last token of each,
        "all" = every token), in the order of the sequences and of `want`."""
        n = len(slots)
        if n == 0 or len(tokens) != n:
            raise EngineError("step: slots and tokens must be non-empty lists of the same length")
        if len(set(slots)) != n:
            raise EngineError("step: a slot appears twice in one step")
        lens = [len(t) for t in tokens]
        if min(lens) < 1:
            raise EngineError("step: every sequence must bring at least one token")
        want_last = isinstance(want, str) and want == "last"
        if want_last:
            pass
        elif isinstance(want, str) and want == "all":
            want = [range(l) for l in lens]
        elif isinstance(want, str):
            raise EngineError(f"step: want must be 'last', 'all' or lists of indices, got {want!r}")
        if not want_last and len(want) != n:
            raise EngineError("step: want must have one list per sequence")
        cache = self.cache
        starts = []
        for s, l in zip(slots, lens):
            if not cache.slots.is_held(s):
                raise EngineError(f"step: slot {s} is not open")
            start = cache.lengths[s]
            if start + l > self.max_seq_len:
                raise EngineError(f"step: slot {s} would hold {start + l} tokens, more than max_seq_len "
                                  f"{self.max_seq_len} (an Engine argument; its default is the model's limit, "
                                  f"capped at {DEFAULT_MAX_SEQ_LEN})")
            starts.append(start)
        for s, st, l in zip(slots, starts, lens):
            cache.reserve(s, st + l)

        T = sum(lens)
        flat = _flatten_tokens(tokens, lens)
        if flat.min() < 0 or flat.max() >= self.vocab_size:
            raise EngineError(f"step: token id outside the vocabulary (0..{self.vocab_size - 1})")
        cu = [0] * (n + 1)
        for i, l in enumerate(lens):
            cu[i + 1] = cu[i] + l
        if want_last:
            rows = cu[1:]
            rows = [r - 1 for r in rows]
        else:
            rows = []
            for i, w in enumerate(want):
                for j in w:
                    if not 0 <= j < lens[i]:
                        raise EngineError(f"step: want index {j} is outside sequence {i}'s {lens[i]} tokens")
                    rows.append(cu[i] + j)
        R = len(rows)
        kvlen = [st + l for st, l in zip(starts, lens)]
        # one packed upload: [tokens | tok_pos | tok_seq | cu_q | seq_slot | seq_start | seq_kvlen | rows]
        sizes = [T, T, T, n + 1, n, n, n, R]
        offs = [0]
        for sz in sizes:
            offs.append(offs[-1] + _round_up(sz, 4))
        packed = self._staging(offs[-1])
        packed[:T] = flat
        if n == 1:
            packed[offs[1]:offs[1] + T] = np.arange(starts[0], starts[0] + T, dtype=np.int32)
            packed[offs[2]:offs[2] + T] = 0
        else:
            tok_seq = np.repeat(np.arange(n, dtype=np.int32), lens)
            shift = np.asarray(starts, dtype=np.int32) - np.asarray(cu[:-1], dtype=np.int32)
            packed[offs[1]:offs[1] + T] = np.arange(T, dtype=np.int32) + shift[tok_seq]
            packed[offs[2]:offs[2] + T] = tok_seq
        for k, vals in ((3, cu), (4, slots), (5, starts), (6, kvlen), (7, rows)):
            packed[offs[k]:offs[k] + sizes[k]] = vals
        # A lone prompt whose length has come before runs as a captured step (see PrefillGraph): no launch work
        # on the host beyond one upload and one replay.
        captured = None
        if self.use_cuda_graph and n == 1 and want_last and T >= PrefillGraph.MIN_TOKENS and trace.timer is None:
            captured = self._prefill_graph_for(T, offs, sizes)
        if captured is not None and captured.graph is not None:
            captured.meta.copy_(self._staging_tensor[:offs[-1]], non_blocking=True)
            self._staging_done.record()
            logits = captured.replay()
            for s, new_len in zip(slots, kvlen):
                cache.note_appended(s, new_len, device_updated=True)
            return logits
        dev = torch.empty(offs[-1], dtype=torch.int32, device=self.device)
        dev.copy_(self._staging_tensor[:offs[-1]], non_blocking=True)
        self._staging_done.record()
        view = [dev[offs[k]:offs[k] + sizes[k]] for k in range(8)]
        max_kv = max(kvlen)
        ctx = StepContext(
            n_tokens=T, n_seqs=n, decode=max(lens) == 1, max_q_len=max(lens), max_kv_len=max_kv,
            tokens=view[0], tok_pos=view[1], tok_seq=view[2], cu_q=view[3], seq_slot=view[4], seq_start=view[5],
            seq_kvlen=view[6], logit_rows=view[7], dtype=self.dtype, device=self.device, kernels=self.kernels,
            all_rows=R == T and rows == list(range(T)))
        if trace.timer is not None:      # the per-kernel timer counts attention work from the real lengths
            ops.STEP_HINT["kv_total"] = sum(kvlen)
            ops.STEP_HINT["pairs"] = sum(l * (st + (l + 1) / 2.0) for st, l in zip(starts, lens))
        trace.push("ModelForward")
        logits = self.model.forward(ctx, cache)
        trace.pop()
        ops.advance_lengths(ctx.seq_slot, ctx.seq_kvlen, cache.seq_lens, n, cache.scratch_slot)
        for s, new_len in zip(slots, kvlen):
            cache.note_appended(s, new_len, device_updated=True)
        if captured is not None:
            captured.capture()               # this length came a second time: later steps of it are replays
        return logits

    def _prefill_graph_for(self, T: int, offs, sizes) -> Optional["PrefillGraph"]:
        """The captured lone-prompt step for prompts of T tokens: None at a length's first occurrence, an
        uncaptured PrefillGraph at its second (the step still runs eagerly and captures afterwards), a ready one
        from then on. The few most recently used lengths are kept."""
        seen = self._prefill_graphs
        entry = seen.pop(T, None)
        if entry is None:
            entry = False                     # seen once
        elif entry is False:
            entry = PrefillGraph(self, T, list(offs), list(sizes))
        seen[T] = entry                       # most recently used last
        while len(seen) > PrefillGraph.KEEP:
            seen.pop(next(iter(seen)))
        return entry or None

    # ---------------------------------------------------------------- captured one-token step
    def decode_graph(self, n_lanes: int, kv_len: Optional[int] = None, sampling=None,
                     host_io: bool = False) -> "DecodeGraph":
        """The captured one-token step for `n_lanes` sequences none of which holds more than `kv_len`
        tokens after the step (default: the engine's limit). Kept per (lanes, length bucket): the
        attention grid of a captured step is sized for the bucket, not for the longest possible sequence.
        With `sampling` (a SamplingParams) the draw of the next tokens is part of the captured step:
        `sampled` then holds them after a replay. Greedy and drawing steps are two captures; temperature,
        top_p and seed of a drawing step live in device memory (`set_sampling`), so one capture serves every
        setting. With `host_io` as well, the captured step begins with the
        upload of `host_in` (pinned) into `tokens` and ends with the download of `sampled` into `host_out`
        (pinned): a generation loop then needs one launch per step and no copy calls of its own."""
        limit = kv_bucket_for(self.max_seq_len if kv_len is None else kv_len, self.max_seq_len)
        if host_io and sampling is None:
            raise EngineError("decode_graph: host_io needs the draw inside the captured step (give sampling)")
        mode = None if sampling is None else ("greedy" if sampling.temperature <= 0 else "draw")
        key = (n_lanes, limit, mode, bool(host_io))
        g = self._graphs.get(key)
        if g is None:
            g = DecodeGraph(self, n_lanes, limit, sampling, host_io)
            self._graphs[key] = g
        elif sampling is not None:
            g.set_sampling(sampling)
        return g

    def try_decode_graph(self, *args, **kwargs) -> Optional["DecodeGraph"]:
        """`decode_graph`, or None when this model's step cannot be captured (`use_cuda_graph` is then off)."""
        try:
            return self.decode_graph(*args, **kwargs)
        except RuntimeError as exc:
            if "captur" not in str(exc).lower() and "graph" not in str(exc).lower():
                raise
            capture_failed(self, "the one-token step", exc)
            return None

    def weight_bytes_per_step(self) -> int:
        return self.model.weight_bytes_per_step()

    def kv_bytes_per_token(self) -> int:
        """Cache bytes one position of one sequence occupies, over all units."""
        esize = 2 if self.dtype == torch.bfloat16 else 4
        total = 0
        for reqs in self.model.unit_requests:
            for r in reqs:
                if hasattr(r, "n_kv_heads"):
                    total += 2 * r.n_kv_heads * r.head_dim * esize
        return total


BUCKETS = (1, 2, 4, 8, 16, 32, 64, 128, 256)


def bucket_for(n: int) -> int:
    """The smallest lane count a captured step is kept for that holds n sequences."""
    for b in BUCKETS:
        if b >= n:
            return b
    return n


def kv_bucket_for(kv_len: int, limit: int) -> int:
    """Length buckets of captured steps: 512, 1024, 2048, ... capped by the engine's limit."""
    b = 512
    while b < kv_len:
        b *= 2
    return min(b, limit)


class PrefillGraph:
    """The captured step of ONE prompt of T tokens whose last row's logits are wanted, at any start position
    and in any slot: every index array of the step lives in one device buffer (`meta`, laid out as the eager
    step's packed upload) that is filled before each replay, and every kernel of the step takes its positions,
    slot and lengths from there. A prompt step is some 150 launches; replayed, the host's share of it is one
    upload and one launch. Prompt lengths repeat where prompts are cut into pieces of a fixed size or come
    from templates; a length is captured when it comes the second time, and the KEEP most recently used
    lengths are kept (each holds the activations of a T-token step)."""
    MIN_TOKENS = 16
    KEEP = 4

    def __init__(self, engine: Engine, n_tokens: int, offs, sizes):
        self.engine, self.T = engine, n_tokens
        self.offs, self.sizes = offs, sizes
        self.meta = torch.zeros(offs[-1], dtype=torch.int32, device=engine.device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.logits: Optional[torch.Tensor] = None

    def _forward(self) -> torch.Tensor:
        e, T = self.engine, self.T
        v = [self.meta[self.offs[k]:self.offs[k] + self.sizes[k]] for k in range(8)]
        ctx = StepContext(
            n_tokens=T, n_seqs=1, decode=False, max_q_len=T, max_kv_len=e.max_seq_len, tokens=v[0], tok_pos=v[1],
            tok_seq=v[2], cu_q=v[3], seq_slot=v[4], seq_start=v[5], seq_kvlen=v[6], logit_rows=v[7], dtype=e.dtype,
            device=e.device, kernels=e.kernels, all_rows=False)
        logits = e.model.forward(ctx, e.cache)
        ops.advance_lengths(ctx.seq_slot, ctx.seq_kvlen, e.cache.seq_lens, 1, e.cache.scratch_slot)
        return logits

    def capture(self) -> None:
        """Records the step; nothing runs. Called right after an eager step of the same length, so every kernel
        library is loaded and the allocator's pools are warm."""
        if self.graph is not None:
            return
        torch.cuda.synchronize(self.engine.device)
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()                      # see DecodeGraph._capture
        try:
            with torch.cuda.graph(graph):
                self.logits = self._forward()
        except RuntimeError as exc:
            capture_failed(self.engine, f"the prompt step of {self.T} tokens", exc)
            return
        finally:
            if gc_was_on:
                gc.enable()
        self.launches_per_replay = ops.LAUNCHES - before
        self.graph = graph

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        ops.LAUNCHES += self.launches_per_replay
        return self.logits.clone()        # the captured buffer is written again by the next replay


def capture_failed(engine: Engine, what: str, exc: BaseException) -> None:
    """A part that reads device memory on the host in its forward (a registered part written with plain tensor
    code may) cannot be recorded into a graph. The engine then runs every step eagerly from here on."""
    engine.use_cuda_graph = False
    torch.cuda.synchronize(engine.device)
    print(f"[llm_infer_engine_b200] {what} could not be captured as a CUDA graph ({type(exc).__name__}: "
          f"{str(exc).splitlines()[0] if str(exc) else ''}); steps run eagerly from here on", file=sys.stderr)


class DecodeGraph:
    """One captured one-token step for `n_lanes` sequences. Inputs live in device buffers:
    `tokens[n_lanes]`, `slots[n_lanes]` (padding lanes name the scratch slot), and the lengths in
    the cache's `seq_lens`; the step derives positions from them, so replaying needs no host
    writes beyond the two buffers when the set of sequences changes. `logits` is [n_lanes, vocab]."""

    def __init__(self, engine: Engine, n_lanes: int, kv_limit: Optional[int] = None, sampling=None,
                 host_io: bool = False):
        self.engine = engine
        self.n = n_lanes
        self.sampling = sampling
        self.host_io = bool(host_io)
        self.kv_limit = engine.max_seq_len if kv_limit is None else kv_limit     # lengths this capture serves
        dev = engine.device
        cache = engine.cache
        i32 = dict(dtype=torch.int32, device=dev)
        self.tokens = torch.zeros(n_lanes, **i32)
        self.slots = torch.full((n_lanes,), cache.scratch_slot, **i32)
        self.tok_pos = torch.zeros(n_lanes, **i32)
        self.tok_seq = torch.zeros(n_lanes, **i32)
        self.cu_q = torch.zeros(n_lanes + 1, **i32)
        self.seq_start = torch.zeros(n_lanes, **i32)
        self.seq_kvlen = torch.zeros(n_lanes, **i32)
        self.rows = torch.arange(n_lanes, **i32)
        # with sampling in the captured step: the drawn tokens, and per lane the request's number and how
        # many tokens it has drawn so far (they name the uniform number of each draw)
        self.sampled = torch.zeros(n_lanes, **i32)
        self.seq_ids = torch.zeros(n_lanes, **i32)
        self.counters = torch.zeros(n_lanes, **i32)
        # temperature, top_p and seed of a drawing step, read by the sampling kernel when it runs
        self.draws = sampling is not None and sampling.temperature > 0
        self.sample_params = torch.zeros(4, **i32) if self.draws else None
        self._uploaded = None
        if self.draws:
            self.set_sampling(sampling)
        # pinned host memory that the captured step reads its tokens from and leaves the drawn ones in
        self.host_in = torch.zeros(n_lanes, dtype=torch.int32).pin_memory() if self.host_io else None
        self.host_out = torch.zeros(n_lanes, dtype=torch.int32).pin_memory() if self.host_io else None
        self.logits: Optional[torch.Tensor] = None
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._lane_slots: List[int] = [cache.scratch_slot] * n_lanes
        self._capture()

    def _run(self) -> torch.Tensor:
        if self.host_io:
            self.tokens.copy_(self.host_in, non_blocking=True)
        logits = self._forward()
        if self.draws:
            ops.sample(logits, self.sampled, seq_ids=self.seq_ids, counters=self.counters, params=self.sample_params)
        elif self.sampling is not None:
            ops.sample(logits, self.sampled)
        if self.host_io:
            self.host_out.copy_(self.sampled, non_blocking=True)
        return logits

    def _forward(self) -> torch.Tensor:
        e = self.engine
        ops.prepare_decode(self.slots, e.cache.seq_lens, self.tok_pos, self.tok_seq, self.cu_q, self.seq_start,
                           self.seq_kvlen, self.n)
        ctx = StepContext(
            n_tokens=self.n, n_seqs=self.n, decode=True, max_q_len=1, max_kv_len=self.kv_limit, tokens=self.tokens,
            tok_pos=self.tok_pos, tok_seq=self.tok_seq, cu_q=self.cu_q, seq_slot=self.slots, seq_start=self.seq_start,
            seq_kvlen=self.seq_kvlen, logit_rows=self.rows, dtype=e.dtype, device=e.device, kernels=e.kernels,
            all_rows=True)
        logits = e.model.forward(ctx, e.cache)
        ops.advance_lengths(self.slots, self.seq_kvlen, e.cache.seq_lens, self.n, e.cache.scratch_slot)
        return logits

    def _capture(self) -> None:
        # a first eager run on the scratch slot loads every kernel library and sizes the pools
        side = torch.cuda.Stream(device=self.engine.device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            self._run()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize(self.engine.device)
        self.graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES
        # No garbage collection inside the capture: collecting an engine that is no longer used frees its
        # pinned memory, for which the allocator records an event on the default stream, and work on the
        # default stream while another stream is capturing invalidates the capture.
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            with torch.cuda.graph(self.graph):
                self.logits = self._run()
        finally:
            if gc_was_on:
                gc.enable()
        self.launches_per_replay = ops.LAUNCHES - before      # this library's kernels inside one replay

    def set_sampling(self, sampling) -> None:
        """The settings the next replays draw with. A greedy capture takes only greedy settings and a
        drawing capture only temperatures above zero: the two differ in their kernels."""
        if (sampling.temperature > 0) != self.draws:
            raise EngineError("set_sampling: a greedy and a drawing step are different captures")
        if self.draws and sampling != self._uploaded:
            self.sample_params.copy_(torch.tensor(ops.sampling_words(sampling.temperature, sampling.top_p,
                                                                     sampling.seed), dtype=torch.int32))
            self._uploaded = sampling
        self.sampling = sampling

    def set_lanes(self, slots: Sequence[int]) -> None:
        """Which sequences the lanes continue; the rest are padding."""
        if len(slots) > self.n:
            raise EngineError(f"{len(slots)} sequences do not fit a graph of {self.n} lanes")
        lane_slots = list(slots) + [self.engine.cache.scratch_slot] * (self.n - len(slots))
        if lane_slots != self._lane_slots:
            self.slots.copy_(torch.tensor(lane_slots, dtype=torch.int32))
            self._lane_slots = lane_slots

    def replay(self) -> torch.Tensor:
        self.graph.replay()
        ops.LAUNCHES += self.launches_per_replay
        return self.logits
