"""Python faces of the CUDA kernels: argument checks, then one ctypes call per launch.

Every function takes CUDA tensors, checks dtype / shape / contiguity on the host (the checks
stand in for a memory checker: no kernel is ever launched on sizes it was not written for),
launches on torch's current stream and returns without synchronising. There is no CPU or
library fallback: a tensor that is not on a GPU, or a kernel library that cannot be built,
raises.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build, trace

_c_int, _c_float, _c_void_p = ctypes.c_int, ctypes.c_float, ctypes.c_void_p
_ERRORS = {-1: "bad argument", -2: "size not supported by this kernel", -3: "pointer not aligned",
           -4: "dtype not supported"}
F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}

_fn_cache = {}


class KernelError(RuntimeError):
    pass


PDL = True        # programmatic dependent launch between this library's kernels (see csrc/common.cuh)


def set_pdl(on: bool) -> None:
    """Turns programmatic dependent launch on or off for every kernel library, loaded or yet to be."""
    global PDL
    PDL = bool(on)
    for family in list(_pdl_state):
        _apply_pdl(family)


_pdl_state = {}


def _apply_pdl(family: str) -> None:
    if _pdl_state.get(family) != PDL:
        lib = build.load(family)
        lib.llmie_set_pdl.argtypes = [_c_int]
        lib.llmie_set_pdl.restype = None
        lib.llmie_set_pdl(1 if PDL else 0)
        _pdl_state[family] = PDL


def _fn(family: str, name: str, argtypes, query: bool = False):
    """The exported function `name` of a kernel family. `query=True` marks a host-side question (no launch),
    which the per-kernel timer leaves alone."""
    key = (family, name)
    f = _fn_cache.get(key)
    if f is None:
        lib = build.load(family)
        raw = getattr(lib, name)
        raw.argtypes = argtypes
        raw.restype = _c_int
        _apply_pdl(family)
        short = name[6:] if name.startswith("llmie_") else name
        if query:
            _fn_cache[key] = raw
            return raw

        def f(*args, _raw=raw, _name=short):
            t = trace.timer
            return _raw(*args) if t is None else t.run(_name, _raw, args)

        _fn_cache[key] = f
    return f


def _work(nbytes: float = 0.0, flops: float = 0.0) -> None:
    """Tells an installed per-kernel timer what the next launch moves and computes."""
    if trace.timer is not None:
        trace.timer.note(nbytes, flops)


def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if t is not None)


def library_mm(x: torch.Tensor, w: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
    """x [T, K] @ w[N, K]^T through the library GEMM (cuBLAS), for the products the reference leaves to
    nn.Linear; seen by the per-kernel timer like this library's own launches."""
    def run():
        if out_dtype == x.dtype:
            return torch.mm(x, w.t())
        return torch.mm(x, w.t(), out_dtype=out_dtype)
    t = trace.timer
    if t is None:
        return run()
    T, K = x.shape
    N = w.shape[0]
    t.note(_nbytes(x, w) + T * N * (2 if out_dtype == torch.bfloat16 else 4), 2.0 * T * N * K)
    return t.run("library_mm", run, ())


LAUNCHES = 0      # kernels of this library launched so far (captured launches count once, at capture)


def _check(status: int, name: str) -> None:
    if status == 0:
        global LAUNCHES
        LAUNCHES += 1
        return
    if status < 0:
        raise KernelError(f"{name}: {_ERRORS.get(status, 'error ' + str(status))}")
    raise KernelError(f"{name}: CUDA error {status} at launch")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


_get_device = getattr(torch._C, "_cuda_getDevice", None)


def _stream() -> int:
    """The current CUDA stream of the current device as a raw handle."""
    if _raw_stream is not None:
        return _raw_stream(_get_device() if _get_device is not None else torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor, what: str) -> int:
    code = _DT.get(t.dtype)
    if code is None:
        raise KernelError(f"{what}: dtype {t.dtype} is not supported (float32 or bfloat16)")
    return code


def _need(t: torch.Tensor, what: str, dtype=None, shape=None) -> None:
    """The checks every launch makes of every tensor it is given (written for speed: an eager step makes
    several hundred of them)."""
    if not t.is_cuda:
        raise KernelError(f"{what}: must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{what}: must be contiguous")
    if dtype is not None and t.dtype is not dtype:
        raise KernelError(f"{what}: dtype {t.dtype}, expected {dtype}")
    if shape is not None:
        have = t.shape
        bad = len(have) != len(shape)
        if not bad:
            for want, got in zip(shape, have):
                if want is not None and want != got:
                    bad = True
                    break
        if bad:
            raise KernelError(f"{what}: shape {tuple(have)}, expected {tuple(shape)}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


# ------------------------------------------------------------------------------------------
def embedding(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t] = table[tokens[t]] as float32. tokens int32 [T]; table [V, d]; out float32 [T, d]."""
    T = tokens.shape[0]
    V, d = table.shape
    _need(tokens, "tokens", torch.int32, (T,))
    _need(table, "table")
    _need(out, "out", torch.float32, (T, d))
    _work(T * 4 + T * d * table.element_size() + _nbytes(out))
    f = _fn("elementwise", "llmie_embedding",
            [_c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(tokens.data_ptr(), table.data_ptr(), _dt(table, "table"), out.data_ptr(), T, d, V, _stream()),
           "embedding")
    return out


def add_rmsnorm(h: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h += delta (float32, in place, when rows is None); out = rmsnorm(h) * weight.

    h float32 [T, d]; delta [T, d] of out's dtype or None; weight float32 [d]; out [n_out, d].
    With `rows` (int32 [n_out]) only those rows of h (+ delta) are normalised and h is left as it is."""
    T, d = h.shape
    n_out = T if rows is None else rows.shape[0]
    _need(h, "h", torch.float32)
    _need(weight, "weight", torch.float32, (d,))
    _need(out, "out", None, (n_out, d))
    if delta is not None:
        _need(delta, "delta", out.dtype, (T, d))
    if rows is not None:
        _need(rows, "rows", torch.int32, (n_out,))
    _work((2 * _nbytes(h) if rows is None else n_out * d * 4) + _nbytes(delta, out))
    f = _fn("elementwise", "llmie_add_rmsnorm",
            [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_float, _c_int, _c_void_p])
    _check(f(h.data_ptr(), _ptr(delta), weight.data_ptr(), out.data_ptr(), _ptr(rows), n_out, d, float(eps),
             _dt(out, "out"), _stream()), "add_rmsnorm")
    return out


def residual_add(h: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    """h += delta; h float32, delta float32 or bfloat16 of the same shape."""
    _need(h, "h", torch.float32)
    _need(delta, "delta", None, tuple(h.shape))
    f = _fn("elementwise", "llmie_residual_add", [_c_void_p, _c_void_p, ctypes.c_longlong, _c_int, _c_void_p])
    _check(f(h.data_ptr(), delta.data_ptr(), h.numel(), _dt(delta, "delta"), _stream()), "residual_add")
    return h


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[t, j] = silu(gate_up[t, j]) * gate_up[t, ff + j]; gate_up [T, 2 ff], out [T, ff]."""
    T, ff = out.shape
    _need(out, "out")
    _need(gate_up, "gate_up", out.dtype, (T, 2 * ff))
    _work(_nbytes(gate_up, out))
    f = _fn("elementwise", "llmie_swiglu", [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(gate_up.data_ptr(), out.data_ptr(), T, ff, _dt(out, "out"), _stream()), "swiglu")
    return out


def rope_store(qkv, q_out, k_cache, v_cache, table, tok_pos, tok_seq, seq_slot, block_table, page_size: int,
               n_q: int, n_kv: int, head_dim: int, rot_dim: int, write_kv: bool = True):
    """Rotates q and k by position and writes k, v into the paged cache.

    qkv [T, (n_q + 2 n_kv) hd]; q_out [T, n_q hd]; caches [n_pages, n_kv, page_size, hd] (same dtype);
    table float32 [max_pos, rot_dim / 2, 2] of (cos, sin) or None for no rotation;
    tok_pos, tok_seq int32 [T]; seq_slot int32 [n]; block_table int32 [n_slots, max_pages]."""
    T = qkv.shape[0]
    _need(qkv, "qkv", None, (T, (n_q + 2 * n_kv) * head_dim))
    _need(q_out, "q_out", qkv.dtype, (T, n_q * head_dim))
    _need(tok_pos, "tok_pos", torch.int32)
    _need(tok_seq, "tok_seq", torch.int32)
    _need(seq_slot, "seq_slot", torch.int32)
    _need(block_table, "block_table", torch.int32)
    if tok_pos.shape[0] < T or tok_seq.shape[0] < T:
        raise KernelError("rope_store: tok_pos / tok_seq shorter than the token count")
    table_len = 0
    if table is not None:
        _need(table, "table", torch.float32, (None, rot_dim // 2, 2))
        table_len = table.shape[0]
    if write_kv:
        _need(k_cache, "k_cache", qkv.dtype, (None, n_kv, page_size, head_dim))
        _need(v_cache, "v_cache", qkv.dtype, tuple(k_cache.shape))
    _work(_nbytes(qkv, q_out) + (2 * T * n_kv * head_dim * qkv.element_size() if write_kv else 0))
    f = _fn("elementwise", "llmie_rope_store",
            [_c_void_p] * 9 + [_c_int] * 10 + [_c_void_p])
    _check(f(qkv.data_ptr(), q_out.data_ptr(), _ptr(k_cache) if write_kv else None,
             _ptr(v_cache) if write_kv else None, _ptr(table), tok_pos.data_ptr(), tok_seq.data_ptr(),
             seq_slot.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, T, n_q,
             n_kv, head_dim, rot_dim, table_len, 1 if write_kv else 0, _dt(qkv, "qkv"), _stream()), "rope_store")
    return q_out


def attention_paged(q, k_cache, v_cache, out, tok_pos, tok_seq, seq_slot, block_table, page_size: int,
                    n_q: int, n_kv: int, head_dim: int, scale: float, window: int = 0):
    """Plain attention over the paged cache, one warp per (token, query head).
    q, out [T, n_q hd]; caches [n_pages, n_kv, page_size, hd]; window 0 = all earlier keys."""
    T = q.shape[0]
    _need(q, "q", None, (T, n_q * head_dim))
    _need(out, "out", q.dtype, (T, n_q * head_dim))
    _need(k_cache, "k_cache", q.dtype, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", q.dtype, tuple(k_cache.shape))
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if head_dim % 16 or head_dim > 256:
        raise KernelError(f"attention_paged: head_dim {head_dim} must be a multiple of 16 and at most 256")
    _work(2 * _nbytes(q) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * q.element_size(),
          4.0 * n_q * head_dim * STEP_HINT["pairs"])
    f = _fn("attention_simt", "llmie_attention_paged",
            [_c_void_p] * 8 + [_c_int] * 6 + [_c_float, _c_int, _c_int, _c_void_p])
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), tok_pos.data_ptr(),
             tok_seq.data_ptr(), seq_slot.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, T,
             n_q, n_kv, head_dim, float(scale), int(window), _dt(q, "q"), _stream()), "attention_paged")
    return out


def attention_decode_supported(head_dim: int, dtype: torch.dtype) -> bool:
    code = _DT.get(dtype)
    if code is None:
        return False
    lib = build.load("attention_decode")
    lib.llmie_attention_decode_supported.argtypes = [_c_int, _c_int]
    lib.llmie_attention_decode_supported.restype = _c_int
    return bool(lib.llmie_attention_decode_supported(head_dim, code))


def attention_decode_run_len(n_seqs: int, head_dim: int, dtype: torch.dtype) -> int:
    """Keys per block that attention_decode wants for this many sequences (a multiple of the page size)."""
    lib = build.load("attention_decode")
    lib.llmie_attention_decode_run_len.argtypes = [_c_int, _c_int, _c_int]
    lib.llmie_attention_decode_run_len.restype = _c_int
    return int(lib.llmie_attention_decode_run_len(n_seqs, head_dim, _DT[dtype]))


def decode_scratch_floats(n_seqs: int, n_q: int, head_dim: int, n_runs: int) -> int:
    """float32 elements of scratch that attention_decode needs."""
    return n_seqs * n_q * n_runs * (head_dim + 2)


def decode_counter_ints(n_seqs: int, n_q: int, n_kv: int) -> int:
    """int32 counters that the one-launch form of attention_decode needs (all zero, left zero)."""
    g = n_q // n_kv
    return n_seqs * n_kv * ((g + 3) // 4 if g <= 4 else (g + 7) // 8)


def attention_decode(q, k_cache, v_cache, out, seq_slot, seq_kvlen, block_table, page_size: int, n_q: int,
                     n_kv: int, head_dim: int, scale: float, window: int, run_len: int, n_runs: int,
                     scratch: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None):
    """Split-KV attention for a step in which every sequence brings one token.

    q, out [n, n_q hd]; seq_kvlen int32 [n] = keys each sequence holds INCLUDING this step's;
    n_runs * run_len must be at least the longest length that seq_kvlen can name; run_len is the
    page size. scratch: float32 with decode_scratch_floats(...) elements (allocated here if None).
    With `counters` (int32 zeros, decode_counter_ints(...) of them) the runs are merged by the last
    block of the same launch instead of a second kernel."""
    n = q.shape[0]
    _need(q, "q", None, (n, n_q * head_dim))
    _need(out, "out", q.dtype, (n, n_q * head_dim))
    _need(k_cache, "k_cache", q.dtype, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", q.dtype, tuple(k_cache.shape))
    for name, t in (("seq_slot", seq_slot), ("seq_kvlen", seq_kvlen), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if seq_slot.numel() < n or seq_kvlen.numel() < n:
        raise KernelError("attention_decode: seq_slot / seq_kvlen shorter than the number of sequences")
    need = decode_scratch_floats(n, n_q, head_dim, n_runs)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    _need(scratch, "scratch", torch.float32)
    if scratch.numel() < need:
        raise KernelError(f"attention_decode: scratch holds {scratch.numel()} floats, {need} are needed")
    n_ml = n * n_q * n_runs
    base = scratch.data_ptr()
    if counters is not None:
        _need(counters, "counters", torch.int32)
        if counters.numel() < decode_counter_ints(n, n_q, n_kv):
            raise KernelError("attention_decode: too few counters")
        _work(2 * _nbytes(q) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * q.element_size(),
              4.0 * n_q * head_dim * STEP_HINT["pairs"])
        f = _fn("attention_decode", "llmie_attention_decode_fused",
                [_c_void_p] * 11 + [_c_int] * 6 + [_c_float] + [_c_int] * 4 + [_c_void_p])
        _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), base, base + 4 * n_ml,
                 base + 8 * n_ml, counters.data_ptr(), seq_slot.data_ptr(), seq_kvlen.data_ptr(),
                 block_table.data_ptr(), block_table.shape[1], page_size, n, n_q, n_kv, head_dim, float(scale),
                 int(window), int(run_len), int(n_runs), _dt(q, "q"), _stream()), "attention_decode")
        return out
    f = _fn("attention_decode", "llmie_attention_decode",
            [_c_void_p] * 10 + [_c_int] * 6 + [_c_float] + [_c_int] * 4 + [_c_void_p])
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), base, base + 4 * n_ml,
             base + 8 * n_ml, seq_slot.data_ptr(), seq_kvlen.data_ptr(), block_table.data_ptr(),
             block_table.shape[1], page_size, n, n_q, n_kv, head_dim, float(scale), int(window), int(run_len),
             int(n_runs), _dt(q, "q"), _stream()), "attention_decode")
    return out


# What a step's attention really reads is known to the caller, not to the launcher (which is sized for upper
# bounds): when a per-kernel timer is installed the engine leaves here, for the timer's counts, the keys all
# sequences of the step hold together and the (query, key) pairs the step's causal attention visits.
STEP_HINT = {"kv_total": 0, "pairs": 0}

MMA_MAX_BLOCKS = 148 * 2        # blocks the decode attention aims at: two per SM


def attention_decode_mma_supported(head_dim: int, dtype: torch.dtype, page_size: int) -> bool:
    if dtype != torch.bfloat16:
        return False
    f = _fn("attention_decode_mma", "llmie_attention_decode_mma_supported", [_c_int] * 3, query=True)
    return bool(f(head_dim, _DT[dtype], page_size))


def attention_decode_mma_pages(n_seqs: int, n_q: int, n_kv: int, max_kv_len: int,
                               max_blocks: Optional[int] = None) -> int:
    """Cache pages per block that attention_decode_mma wants for this step's shape."""
    groups = n_kv * ((n_q // n_kv + 15) // 16)
    f = _fn("attention_decode_mma", "llmie_attention_decode_mma_pages", [_c_int] * 4, query=True)
    return int(f(n_seqs, groups, max_kv_len, MMA_MAX_BLOCKS if max_blocks is None else max_blocks))


def attention_decode_mma(q, k_cache, v_cache, out, seq_slot, seq_kvlen, block_table, page_size: int, n_q: int,
                         n_kv: int, head_dim: int, scale: float, window: int, pages_per_run: int, n_runs: int,
                         counters: Optional[torch.Tensor] = None, scratch: Optional[torch.Tensor] = None):
    """Attention for a one-token step on the tensor cores (bfloat16): a warp per cache page, the warps of a
    block merged in shared memory. Arguments as attention_decode; n_runs * pages_per_run pages must cover
    the longest sequence. With n_runs == 1 neither scratch nor counters are touched."""
    n = q.shape[0]
    _need(q, "q", torch.bfloat16, (n, n_q * head_dim))
    _need(out, "out", torch.bfloat16, (n, n_q * head_dim))
    _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    for name, t in (("seq_slot", seq_slot), ("seq_kvlen", seq_kvlen), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if seq_slot.numel() < n or seq_kvlen.numel() < n:
        raise KernelError("attention_decode_mma: seq_slot / seq_kvlen shorter than the number of sequences")
    base = n_ml = 0
    cptr = None
    if n_runs > 1:
        need = decode_scratch_floats(n, n_q, head_dim, n_runs)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=q.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError(f"attention_decode_mma: scratch holds {scratch.numel()} floats, {need} are needed")
        if counters is None or counters.numel() < n * n_kv * ((n_q // n_kv + 15) // 16):
            raise KernelError("attention_decode_mma: counters are needed when a sequence spans several runs")
        _need(counters, "counters", torch.int32)
        base, n_ml, cptr = scratch.data_ptr(), n * n_q * n_runs, counters.data_ptr()
    _work(2 * _nbytes(q) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * 2, 4.0 * n_q * head_dim * STEP_HINT["pairs"])
    f = _fn("attention_decode_mma", "llmie_attention_decode_mma",
            [_c_void_p] * 11 + [_c_int] * 6 + [_c_float] + [_c_int] * 3 + [_c_void_p])
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), base or None,
             (base + 4 * n_ml) or None, (base + 8 * n_ml) or None, cptr, seq_slot.data_ptr(), seq_kvlen.data_ptr(),
             block_table.data_ptr(), block_table.shape[1], page_size, n, n_q, n_kv, head_dim, float(scale),
             int(window), int(pages_per_run), int(n_runs), _stream()), "attention_decode_mma")
    return out


def attention_decode_mma_rope(qkv, k_cache, v_cache, out, table, seq_slot, seq_kvlen, block_table, page_size: int,
                              n_q: int, n_kv: int, head_dim: int, scale: float, window: int, pages_per_run: int,
                              n_runs: int, write_kv: bool = True, counters: Optional[torch.Tensor] = None,
                              scratch: Optional[torch.Tensor] = None):
    """attention_decode_mma with the position encoding and the cache write inside: qkv bfloat16
    [n, (n_q + 2 n_kv) hd] holds the step's raw q, k and v heads; table float32 [max_pos, hd / 2, 2] is the
    (cos, sin) table of a rotation over the whole head size. Sequence i's new key and value are taken for
    position seq_kvlen[i] - 1 and, with write_kv, written into the cache there."""
    n = qkv.shape[0]
    _need(qkv, "qkv", torch.bfloat16, (n, (n_q + 2 * n_kv) * head_dim))
    _need(out, "out", torch.bfloat16, (n, n_q * head_dim))
    _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _need(table, "table", torch.float32, (None, head_dim // 2, 2))
    for name, t in (("seq_slot", seq_slot), ("seq_kvlen", seq_kvlen), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if seq_slot.numel() < n or seq_kvlen.numel() < n:
        raise KernelError("attention_decode_mma_rope: seq_slot / seq_kvlen shorter than the number of sequences")
    base = n_ml = 0
    cptr = None
    if n_runs > 1:
        need = decode_scratch_floats(n, n_q, head_dim, n_runs)
        if scratch is None:
            scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
        _need(scratch, "scratch", torch.float32)
        if scratch.numel() < need:
            raise KernelError(f"attention_decode_mma_rope: scratch holds {scratch.numel()} floats, {need} are needed")
        if counters is None or counters.numel() < n * n_kv * ((n_q // n_kv + 15) // 16):
            raise KernelError("attention_decode_mma_rope: counters are needed when a sequence spans several runs")
        _need(counters, "counters", torch.int32)
        base, n_ml, cptr = scratch.data_ptr(), n * n_q * n_runs, counters.data_ptr()
    _work(_nbytes(qkv, out) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * 2, 4.0 * n_q * head_dim * STEP_HINT["pairs"])
    f = _fn("attention_decode_mma", "llmie_attention_decode_mma_rope",
            [_c_void_p] * 5 + [_c_int] + [_c_void_p] * 7 + [_c_int] * 6 + [_c_float] + [_c_int] * 4 + [_c_void_p])
    _check(f(qkv.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), table.data_ptr(), table.shape[0],
             base or None, (base + 4 * n_ml) or None, (base + 8 * n_ml) or None, cptr, seq_slot.data_ptr(),
             seq_kvlen.data_ptr(), block_table.data_ptr(), block_table.shape[1], page_size, n, n_q, n_kv, head_dim,
             float(scale), int(window), int(pages_per_run), int(n_runs), 1 if write_kv else 0, _stream()),
           "attention_decode_mma_rope")
    return out


def gemm_f32_nt(a: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FMA on CUDA cores, fixed summation order)."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", torch.float32)
    _need(w, "w", torch.float32, (N, K))
    if out is None:
        out = torch.empty((M, N), dtype=torch.float32, device=a.device)
    _need(out, "out", torch.float32, (M, N))
    _work(_nbytes(a, w) + a.shape[0] * w.shape[0] * 4, 2.0 * a.shape[0] * w.shape[0] * w.shape[1])
    f = _fn("gemm_simt", "llmie_gemm_f32_nt", [_c_void_p] * 3 + [_c_int] * 6 + [_c_void_p])
    _check(f(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, K, K, N, _stream()), "gemm_f32_nt")
    return out


SKINNY_STORE_BF16, SKINNY_STORE_F32, SKINNY_ADD_F32, SKINNY_SWIGLU = 0, 1, 2, 3
SKINNY_MAX_BATCH = 32          # what the kernel takes
SKINNY_BEST_BATCH = 8          # up to here it beats the library GEMM (measured on B200)
SKINNY_ADD_BEST_BATCH = 16     # the `h +=` form saves a pass over h as well: 3.7 / 9.6 us against 5.5 / 13.2 us for the
                               # library product of the output / down projection at 16 rows (1B shape); equal at 32


def gemm_skinny_add_wins(rows: int, n: int, k: int, device) -> bool:
    """Whether `h += x w^T` is better done by gemm_skinny than by the library product followed by the add in the
    next norm kernel. Up to 8 rows always. From 9 to 16 rows only for up to one block (16 weight rows) an SM, the
    1B shape's 2,048 outputs: there it takes 4.0 / 9.3 us (output / down projection, 16 rows) against the library's
    5.7 / 12.9 us. Wider outputs were measured inside whole steps (3B shape, 16 sequences of 1,400 tokens): library
    for both 2.254 ms a step, this kernel for the output projection 2.286 ms, for both 2.329 ms, although alone the
    kernel is level with the library there (3,072 x 3,072: 6.6 against 7.0 us)."""
    if rows <= SKINNY_BEST_BATCH:
        return True
    return rows <= SKINNY_ADD_BEST_BATCH and n // 16 <= _sms(device)


def gemm_skinny_ok(batch: int, n: int, k: int, epilogue: int = SKINNY_STORE_BF16) -> bool:
    """Whether gemm_skinny takes this shape (else the caller uses a tiled GEMM)."""
    if not 0 < batch <= SKINNY_MAX_BATCH or k % 32:
        return False
    return (n % 2 == 0 and (n // 2) % 8 == 0) if epilogue == SKINNY_SWIGLU else n % 16 == 0


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> torch.Tensor:
    """y = x w^T for a few rows of x and a large bfloat16 w [N, K] that is read once.

    epilogue SKINNY_STORE_BF16 / SKINNY_STORE_F32: out [batch, N] = y;  SKINNY_ADD_F32: out (float32) += y;
    SKINNY_SWIGLU: w = [gate rows; up rows], out bfloat16 [batch, N / 2] = silu(gate) * up."""
    batch, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16, (N, K))
    if not gemm_skinny_ok(batch, N, K, epilogue):
        raise KernelError(f"gemm_skinny: shape batch={batch}, N={N}, K={K} is not supported")
    cols = N // 2 if epilogue == SKINNY_SWIGLU else N
    want = torch.float32 if epilogue in (SKINNY_STORE_F32, SKINNY_ADD_F32) else torch.bfloat16
    _need(out, "out", want, (batch, cols))
    _work(_nbytes(x, w, out), 2.0 * x.shape[0] * w.shape[0] * w.shape[1])
    f = _fn("gemm_skinny", "llmie_gemm_skinny", [_c_void_p] * 3 + [_c_int] * 5 + [_c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), out.data_ptr(), batch, N, K, cols, epilogue, _stream()), "gemm_skinny")
    return out


def norm_gemm_supported(batch: int, k: int) -> bool:
    """Whether the fused norm + product kernels of one-token steps take this many rows and this width."""
    return 1 <= batch <= 8 and k % 32 == 0 and 8 * (k + 32) * 2 + 12 * 1024 <= 200 * 1024


def _norm_gemm_common(h, norm_w, w, what):
    batch, K = h.shape
    _need(h, "h", torch.float32)
    _need(norm_w, "norm_w", torch.float32, (K,))
    _need(w, "w", torch.bfloat16, (None, K))
    if not norm_gemm_supported(batch, K):
        raise KernelError(f"{what}: {batch} rows of width {K} are not supported")
    return batch, K


def norm_gate_swiglu(h, norm_w, eps: float, w_gate_up, act):
    """act[b, j] = silu(x Wg^T) * (x Wu^T) with x = rmsnorm(h) * norm_w, in one kernel.
    h float32 [batch <= 8, K]; w_gate_up bfloat16 [2 ff, K] = [gate rows; up rows]; act bfloat16 [batch, ff]."""
    batch, K = _norm_gemm_common(h, norm_w, w_gate_up, "norm_gate_swiglu")
    ff = w_gate_up.shape[0] // 2
    _need(act, "act", torch.bfloat16, (batch, ff))
    if w_gate_up.shape[0] % 2 or ff % 8:
        raise KernelError("norm_gate_swiglu: the feed-forward width must be a multiple of 8")
    _work(_nbytes(h, w_gate_up, act), 2.0 * batch * w_gate_up.shape[0] * K)
    f = _fn("gemm_fused_decode", "llmie_norm_gate_swiglu",
            [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(h.data_ptr(), norm_w.data_ptr(), float(eps), w_gate_up.data_ptr(), act.data_ptr(), batch, ff, K,
             _stream()), "norm_gate_swiglu")
    return act


def norm_gemm_f32(h, norm_w, eps: float, w, out):
    """out[batch, N] float32 = (rmsnorm(h) * norm_w) w^T in one kernel (final norm + LM head)."""
    batch, K = _norm_gemm_common(h, norm_w, w, "norm_gemm_f32")
    N = w.shape[0]
    _need(out, "out", torch.float32, (batch, N))
    if N % 16:
        raise KernelError("norm_gemm_f32: N must be a multiple of 16")
    _work(_nbytes(h, w, out), 2.0 * batch * w.shape[0] * K)
    f = _fn("gemm_fused_decode", "llmie_norm_gemm_f32",
            [_c_void_p, _c_void_p, _c_float, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p])
    _check(f(h.data_ptr(), norm_w.data_ptr(), float(eps), w.data_ptr(), out.data_ptr(), batch, N, K, _stream()),
           "norm_gemm_f32")
    return out


def norm_qkv_rope(h, norm_w, eps: float, w_qkv, q_out, k_cache, v_cache, table, tok_pos, tok_seq, seq_slot,
                  block_table, page_size: int, n_q: int, n_kv: int, head_dim: int, write_kv: bool = True):
    """RMSNorm, the packed q/k/v product, rotation of q and k and the KV-cache write in one kernel.
    h float32 [batch <= 8, K]; w_qkv bfloat16 [(n_q + 2 n_kv) hd, K]; q_out bfloat16 [batch, n_q hd];
    table float32 [max_pos, hd / 2, 2] (the whole head is rotated)."""
    batch, K = _norm_gemm_common(h, norm_w, w_qkv, "norm_qkv_rope")
    if w_qkv.shape[0] != (n_q + 2 * n_kv) * head_dim or head_dim % 16:
        raise KernelError("norm_qkv_rope: weight rows do not match the head layout")
    _need(q_out, "q_out", torch.bfloat16, (batch, n_q * head_dim))
    _need(table, "table", torch.float32, (None, head_dim // 2, 2))
    for name, t in (("tok_pos", tok_pos), ("tok_seq", tok_seq), ("seq_slot", seq_slot), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if write_kv:
        _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
        _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    _work(_nbytes(h, w_qkv, q_out) + 2 * batch * n_kv * head_dim * 2, 2.0 * batch * w_qkv.shape[0] * K)
    f = _fn("gemm_fused_decode", "llmie_norm_qkv_rope",
            [_c_void_p, _c_void_p, _c_float] + [_c_void_p] * 9 + [_c_int] * 9 + [_c_void_p])
    _check(f(h.data_ptr(), norm_w.data_ptr(), float(eps), w_qkv.data_ptr(), q_out.data_ptr(),
             _ptr(k_cache) if write_kv else None, _ptr(v_cache) if write_kv else None, table.data_ptr(),
             tok_pos.data_ptr(), tok_seq.data_ptr(), seq_slot.data_ptr(), block_table.data_ptr(),
             block_table.shape[1], page_size, batch, n_q, n_kv, head_dim, K, table.shape[0], 1 if write_kv else 0,
             _stream()), "norm_qkv_rope")
    return q_out


_tc_status = {}
_TC_STATUS_TEXT = {1: "a TMA load did not arrive", 2: "the tensor cores did not release a stage",
                   3: "the accumulators were not completed"}


def tc_status_word(device) -> torch.Tensor:
    """One int32 per device that the tensor-core kernels set when a bounded wait gives up."""
    key = torch.device(device).index or 0
    t = _tc_status.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=device)
        _tc_status[key] = t
    return t


def check_tc_status(device) -> None:
    """Reads the status word (this synchronises) and raises if a tensor-core kernel gave up a wait."""
    t = tc_status_word(device)
    code = int(t.item())
    if code:
        t.zero_()
        raise KernelError(f"a tensor-core kernel timed out: {_TC_STATUS_TEXT.get(code, code)}")


def tc_wait_probe(device, limit: int = 1000) -> None:
    """Launches one block that waits, for at most `limit` polls, on a barrier at which nothing arrives, gives
    up, records the status of a load that did not arrive, frees its tensor memory and returns. The next
    `check_tc_status` then raises. For tests of the give-up path; it never hangs."""
    f = _fn("gemm_tc", "llmie_tc_wait_probe", [_c_void_p, _c_int, _c_void_p])
    with torch.cuda.device(device):
        _check(f(tc_status_word(device).data_ptr(), int(limit), _stream()), "tc_wait_probe")


def attention_prefill_tc_supported(head_dim: int, page_size: int, dtype: torch.dtype) -> bool:
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size == 64


def attention_prefill_tc(q, k_cache, v_cache, out, cu_q, seq_slot, seq_start, block_table, page_size: int,
                         n_seqs: int, max_q_len: int, n_q: int, n_kv: int, head_dim: int, scale: float,
                         window: int = 0):
    """Causal attention for runs of new tokens on the tcgen05 tensor cores, K and V read from the
    paged cache by TMA. q, out bfloat16 [T, n_q hd] with sequences packed (cu_q int32 [n + 1]);
    seq_start int32 [n]: tokens each sequence held before this step. The caches' last page must be
    a scratch page. head_dim 64 or 128, pages of 64."""
    T = q.shape[0]
    _need(q, "q", torch.bfloat16, (T, n_q * head_dim))
    _need(out, "out", torch.bfloat16, (T, n_q * head_dim))
    _need(k_cache, "k_cache", torch.bfloat16, (None, n_kv, page_size, head_dim))
    _need(v_cache, "v_cache", torch.bfloat16, tuple(k_cache.shape))
    for name, t in (("cu_q", cu_q), ("seq_slot", seq_slot), ("seq_start", seq_start), ("block_table", block_table)):
        _need(t, name, torch.int32)
    if not attention_prefill_tc_supported(head_dim, page_size, q.dtype):
        raise KernelError(f"attention_prefill_tc: head_dim {head_dim} / page size {page_size} is not supported")
    if cu_q.numel() < n_seqs + 1 or seq_slot.numel() < n_seqs or seq_start.numel() < n_seqs:
        raise KernelError("attention_prefill_tc: a per-sequence array is shorter than n_seqs")
    if not scale > 0:
        raise KernelError(f"attention_prefill_tc: the scale must be positive, got {scale}")
    _work(2 * _nbytes(q) + 2.0 * STEP_HINT["kv_total"] * n_kv * head_dim * 2, 4.0 * n_q * head_dim * STEP_HINT["pairs"])
    f = _fn("attention_prefill_tc", "llmie_attention_prefill_tc",
            [_c_void_p] * 8 + [_c_int] * 8 + [_c_float, _c_int, _c_void_p, _c_void_p])
    _check(f(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), cu_q.data_ptr(),
             seq_slot.data_ptr(), seq_start.data_ptr(), block_table.data_ptr(), block_table.shape[1],
             k_cache.shape[0], T, n_seqs, max_q_len, n_q, n_kv, head_dim, float(scale), int(window),
             tc_status_word(q.device).data_ptr(), _stream()), "attention_prefill_tc")
    return out


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T on the tcgen05 tensor cores; a, w bfloat16, out bfloat16 or float32."""
    M, K = a.shape
    N = w.shape[0]
    _need(a, "a", torch.bfloat16)
    _need(w, "w", torch.bfloat16, (N, K))
    _need(out, "out", None, (M, N))
    if K % 8 or N % 8:
        raise KernelError(f"gemm_tc: K ({K}) and N ({N}) must be multiples of 8")
    _work(_nbytes(a, w, out), 2.0 * M * N * K)
    f = _fn("gemm_tc", "llmie_gemm_tc", [_c_void_p] * 3 + [_c_int] * 5 + [_c_void_p, _c_void_p])
    _check(f(a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, N, _dt(out, "out"),
             tc_status_word(a.device).data_ptr(), _stream()), "gemm_tc")
    return out


_argmax_parts = {}


STREAM_STORE_BF16, STREAM_STORE_F32, STREAM_ADD_F32 = 0, 1, 2
STREAM_MAX_ROWS = 64
_sm_count = {}


def _sms(device) -> int:
    key = torch.device(device).index or 0
    n = _sm_count.get(key)
    if n is None:
        n = torch.cuda.get_device_properties(key).multi_processor_count
        _sm_count[key] = n
    return n


def gemm_stream_ok(rows: int, n: int, k: int) -> bool:
    """Whether gemm_stream takes this shape: up to 64 rows, K a multiple of 8."""
    return 0 < rows <= STREAM_MAX_ROWS and k % 8 == 0 and n > 0


def gemm_stream_wins(rows: int, n: int, k: int) -> bool:
    """Where gemm_stream beat the library GEMM when measured on a B200 (captured launches, weights rotated through
    more than the L2 holds): only very tall matrices at 33 to 64 rows (a 128,256 x 2,048 head: 84 us against
    92 us). From 9 to 32 rows and for the layer matrices (2,048 to 28,672 rows of weights) the library is equal
    or faster (qkv 6 us against 9-12 us, down 13 us against 13-18 us), so those stay with it."""
    return 32 < rows <= STREAM_MAX_ROWS and k % 8 == 0 and n * k >= 128 * 1024 * 1024


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: int = STREAM_STORE_BF16,
                splits: int = 0) -> torch.Tensor:
    """out = x @ w^T (mode STREAM_STORE_BF16 / STREAM_STORE_F32) or out += x @ w^T (STREAM_ADD_F32, out float32)
    for up to 64 rows of x, on the tcgen05 tensor cores with the weights as the streamed operand. x [M, K] and
    w [N, K] bfloat16. Needs no workspace: slices of K meet in the shared memory of a thread-block cluster.
    splits: 0 = the launcher chooses into how many slices K is cut; 1, 2, 4 or 8 fixes it."""
    M, K = x.shape
    N = w.shape[0]
    _need(x, "x", torch.bfloat16)
    _need(w, "w", torch.bfloat16, (N, K))
    _need(out, "out", torch.bfloat16 if mode == STREAM_STORE_BF16 else torch.float32, (M, N))
    if not gemm_stream_ok(M, N, K):
        raise KernelError(f"gemm_stream: {M} rows x K {K} is not supported (up to {STREAM_MAX_ROWS} rows, K % 8 == 0)")
    _work(_nbytes(x, w, out) + (_nbytes(out) if mode == STREAM_ADD_F32 else 0), 2.0 * M * N * K)
    f = _fn("gemm_stream", "llmie_gemm_stream", [_c_void_p] * 3 + [_c_int] * 6 + [_c_void_p, _c_void_p])
    _check(f(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, int(mode), _sms(x.device), int(splits),
             tc_status_word(x.device).data_ptr(), _stream()), "gemm_stream")
    return out


def _check_query(status: int, name: str) -> None:
    if status != 0:
        raise KernelError(f"{name}: {_ERRORS.get(status, 'error ' + str(status))}")


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Greedy token per row of float32 logits [R, V] (lowest index wins a tie), many blocks per row."""
    R, V = logits.shape
    _need(logits, "logits", torch.float32)
    _need(out, "out", torch.int32)
    if out.shape[0] < R:
        raise KernelError("argmax: out is shorter than the number of rows")
    slices = max(1, min(128, V // 1024, max(8, 1184 // R)))     # about a thousand blocks, each with a few thousand logits
    key = (logits.device, R * slices)
    parts = _argmax_parts.get(key)
    if parts is None:        # kept: a generation loop calls this once per step (calls on one stream are ordered)
        parts = (torch.empty(R * slices, dtype=torch.float32, device=logits.device),
                 torch.empty(R * slices, dtype=torch.int32, device=logits.device))
        _argmax_parts[key] = parts
    part_val, part_idx = parts
    _work(R * V * 4)
    f = _fn("sampling", "llmie_argmax", [_c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p,
                                         _c_void_p])
    _check(f(logits.data_ptr(), R, V, logits.stride(0), slices, part_val.data_ptr(), part_idx.data_ptr(),
             out.data_ptr(), _stream()), "argmax")
    return out


def sampling_words(temperature: float, top_p: float, seed: int) -> list:
    """The four 32-bit words (as Python ints) that `sample(..., params=)` reads from device memory."""
    import struct
    t, p = struct.unpack("<2I", struct.pack("<2f", float(temperature), float(top_p)))
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    as_i32 = lambda w: w - (1 << 32) if w >= (1 << 31) else w
    return [as_i32(t), as_i32(p), as_i32(seed & 0xFFFFFFFF), as_i32(seed >> 32)]


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: float = 0.0, top_p: float = 1.0, seed: int = 0,
           seq_ids: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
           params: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One token per row of float32 logits [R, V]: argmax when temperature <= 0 (lowest index wins a
    tie), else a draw from softmax(logits / T) cut by top_p, with the uniform number of
    (seed, seq_ids[r], counters[r]); counters[r] is then incremented. out int32 [R].
    With `params` (int32 [4] on the device, filled from `sampling_words`) temperature, top_p and seed
    are read from there when the kernel runs, so a captured launch serves any setting."""
    R, V = logits.shape
    if params is not None:
        _need(params, "params", torch.int32, (4,))
        if seq_ids is None or counters is None:
            raise KernelError("sample: seq_ids and counters are required with params")
    elif temperature <= 0 and V >= 4096 and logits.is_contiguous():
        return argmax(logits, out)
    _need(logits, "logits", torch.float32)
    _need(out, "out", torch.int32)
    if out.shape[0] < R:
        raise KernelError("sample: out is shorter than the number of rows")
    if temperature > 0 or params is not None:
        if seq_ids is None or counters is None:
            raise KernelError("sample: seq_ids and counters are required when temperature > 0")
        _need(seq_ids, "seq_ids", torch.int32)
        _need(counters, "counters", torch.int32)
        if seq_ids.shape[0] < R or counters.shape[0] < R:
            raise KernelError("sample: seq_ids / counters shorter than the number of rows")
    _work(R * V * 4)
    f = _fn("sampling", "llmie_sample",
            [_c_void_p, _c_int, _c_int, _c_int, _c_float, _c_float, ctypes.c_ulonglong, _c_void_p, _c_void_p,
             _c_void_p, _c_void_p, _c_void_p])
    _check(f(logits.data_ptr(), R, V, logits.stride(0), float(temperature), float(top_p),
             int(seed) & 0xFFFFFFFFFFFFFFFF, _ptr(params), _ptr(seq_ids), _ptr(counters), out.data_ptr(), _stream()),
           "sample")
    return out


def copy_int(src: torch.Tensor, dst: torch.Tensor, n: int) -> None:
    _need(src, "src", torch.int32)
    _need(dst, "dst", torch.int32)
    if src.numel() < n or dst.numel() < n:
        raise KernelError("copy_int: n exceeds a buffer")
    f = _fn("sampling", "llmie_copy_int", [_c_void_p, _c_void_p, _c_int, _c_void_p])
    _check(f(src.data_ptr(), dst.data_ptr(), n, _stream()), "copy_int")


def prepare_decode(slots, seq_lens, tok_pos, tok_seq, cu_q, seq_start, seq_kvlen, n: int) -> None:
    """Per-lane metadata of a one-token step from the device-resident lengths."""
    for name, t in (("slots", slots), ("seq_lens", seq_lens), ("tok_pos", tok_pos), ("tok_seq", tok_seq),
                    ("cu_q", cu_q), ("seq_start", seq_start), ("seq_kvlen", seq_kvlen)):
        _need(t, name, torch.int32)
    if min(slots.numel(), tok_pos.numel(), tok_seq.numel(), seq_start.numel(), seq_kvlen.numel()) < n \
            or cu_q.numel() < n + 1:
        raise KernelError("prepare_decode: a buffer is shorter than n")
    f = _fn("elementwise", "llmie_prepare_decode", [_c_void_p] * 7 + [_c_int, _c_void_p])
    _check(f(slots.data_ptr(), seq_lens.data_ptr(), tok_pos.data_ptr(), tok_seq.data_ptr(), cu_q.data_ptr(),
             seq_start.data_ptr(), seq_kvlen.data_ptr(), n, _stream()), "prepare_decode")


def advance_lengths(slots, seq_kvlen, seq_lens, n: int, scratch_slot: int) -> None:
    """seq_lens[slots[i]] = seq_kvlen[i] for the n lanes of a step, except the scratch slot."""
    for name, t in (("slots", slots), ("seq_kvlen", seq_kvlen), ("seq_lens", seq_lens)):
        _need(t, name, torch.int32)
    f = _fn("elementwise", "llmie_advance_lengths", [_c_void_p] * 3 + [_c_int, _c_int, _c_void_p])
    _check(f(slots.data_ptr(), seq_kvlen.data_ptr(), seq_lens.data_ptr(), n, scratch_slot, _stream()),
           "advance_lengths")
