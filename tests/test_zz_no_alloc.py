"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some callers cannot allocate device memory at the moment they need attention: all of it is
already in a pool of their own, or they sit in a loop where a cudaMalloc stall is not allowed, or
they are C programs with no tensor library. `llmie_attention_decode_noalloc` serves them from a
fixed scratch array inside the library. Its results must be those of the ordinary entry point,
call after call (the array is shared and keeps the previous call's contents), and a problem
larger than the array must be refused, not run. This file is named to be collected last.
"""
import ctypes

import pytest
import torch

from test_kernels_gpu import Paged, ref_attention

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _symbol():
    from llm_infer_engine_b200.kernels import build
    lib = build.load("attention_decode")
    fn = lib.llmie_attention_decode_noalloc
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int] * 6 + [ctypes.c_float] + [ctypes.c_int] * 4 + [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    cap = lib.llmie_attention_decode_noalloc_capacity
    cap.restype = ctypes.c_ulonglong
    return fn, int(cap())


def _case(seed, lens, n_q, n_kv, hd, dtype):
    pg = Paged(lens, n_kv, hd, dtype, seed=seed)
    pg.fill()
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(len(lens), n_q * hd, generator=g).to(dtype).to(DEV)
    k, v, bt = pg.dev()
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    kvlen = torch.tensor(lens, dtype=torch.int32, device=DEV)
    return pg, q, k, v, bt, slots, kvlen


def _plain(pg, q, lens, n_q, hd, window):
    """Plain float32 attention of each sequence's one query over its own dense keys."""
    rows = []
    for i, n in enumerate(lens):
        qi = q[i].float().cpu().view(1, n_q, hd)
        rows.append(ref_attention(qi, pg.dense_k[i].float(), pg.dense_v[i].float(), [n - 1], hd ** -0.5, window)
                    .reshape(-1))
    return torch.stack(rows)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_no_alloc_matches_ordinary_entry_point_twice(dtype):
    from llm_infer_engine_b200.kernels import ops
    fn, capacity = _symbol()
    assert capacity == 16 * 1024 * 1024
    n_q, n_kv, hd, run_len = 12, 4, 64, 64
    code = 0 if dtype == torch.float32 else 1
    # calls in a row with different data, shapes and windows: each finds the leftovers of the one before in
    # the shared array and must not be disturbed by them. Lengths at page edges (64, 128) and one beyond,
    # and a window that starts inside a page, are the places where a run count or an offset would slip.
    for seed, lens, window in ((1, [5, 130, 700, 64, 333], 0), (2, [901, 17, 256], 0), (3, [64, 128, 129, 65, 1], 0),
                               (4, [300, 64, 128, 40], 100)):
        pg, q, k, v, bt, slots, kvlen = _case(seed, lens, n_q, n_kv, hd, dtype)
        n_runs = (1024 + run_len - 1) // run_len
        want = torch.empty_like(q)
        ops.attention_decode(q, k, v, want, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, window, run_len, n_runs)
        got = torch.full_like(q, float("nan"))
        stream = torch.cuda.current_stream().cuda_stream
        torch.cuda.synchronize()
        allocs_before = torch.cuda.memory_stats()["allocation.all.allocated"]
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), got.data_ptr(), slots.data_ptr(), kvlen.data_ptr(),
                bt.data_ptr(), bt.shape[1], 64, len(lens), n_q, n_kv, hd, hd ** -0.5, window, run_len, n_runs, code,
                stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == allocs_before    # nothing through torch
        assert torch.cuda.mem_get_info()[0] >= free_before                               # nothing from the driver
        # the same kernels on the same inputs: the two entry points agree bit for bit
        assert torch.equal(got, want), float((got.float() - want.float()).abs().max())
        # and both agree with plain attention written in torch
        plain_out = _plain(pg, q, lens, n_q, hd, window)
        tol = 2e-5 if dtype == torch.float32 else 2e-2
        assert torch.allclose(got.float().cpu(), plain_out, atol=tol), float((got.float().cpu() - plain_out).abs().max())


def test_no_alloc_sequence_without_keys_gives_zeros():
    """A length of zero names no keys: the rows of that sequence are zeros, whatever the array held."""
    fn, _ = _symbol()
    n_q, n_kv, hd = 8, 2, 32
    lens = [70, 1, 200]
    pg, q, k, v, bt, slots, kvlen = _case(9, lens, n_q, n_kv, hd, torch.float32)
    kvlen[1] = 0
    out = torch.full_like(q, float("nan"))
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), slots.data_ptr(), kvlen.data_ptr(),
            bt.data_ptr(), bt.shape[1], 64, len(lens), n_q, n_kv, hd, hd ** -0.5, 0, 64, 4, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert bool((out[1] == 0).all())
    plain_out = _plain(pg, q, lens, n_q, hd, 0)
    assert torch.allclose(out[[0, 2]].cpu(), plain_out[[0, 2]], atol=2e-5)


def test_no_alloc_refuses_a_run_length_other_than_a_page():
    fn, _ = _symbol()
    pg, q, k, v, bt, slots, kvlen = _case(5, [10, 20], 8, 2, 32, torch.float32)
    out = torch.full_like(q, 7.0)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), slots.data_ptr(), kvlen.data_ptr(),
            bt.data_ptr(), bt.shape[1], 64, 2, 8, 2, 32, 32 ** -0.5, 0, 128, 2, 0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -2
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())


def test_no_alloc_refuses_what_does_not_fit():
    fn, capacity = _symbol()
    n_q, n_kv, hd, run_len = 32, 8, 64, 64
    lens = [10, 20]
    _, q, k, v, bt, slots, kvlen = _case(3, lens, n_q, n_kv, hd, torch.bfloat16)
    n_runs = capacity // 4 // (len(lens) * n_q * (hd + 2)) + 1          # one run too many for the array
    out = torch.full_like(q, 7.0)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), slots.data_ptr(), kvlen.data_ptr(),
            bt.data_ptr(), bt.shape[1], 64, len(lens), n_q, n_kv, hd, hd ** -0.5, 0, run_len, n_runs, 1,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -5
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())         # nothing ran
