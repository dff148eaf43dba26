"""The engine against the plain implementation, on the GPU, in 32-bit and in bfloat16:
each request alone and whole; with the last 32 tokens one by one; in batches of unequal
lengths whose shorter requests end earlier, one batch after another so that slots are used again."""
import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu

# The bounds are helpers.logit_bound's: float32 agrees to rounding; bfloat16 within 1.5 % of the request's
# largest logit, the same for every way of cutting the work. Random small weights give nearly flat attention, so
# on these models a lost key hides inside the bfloat16 bound; test_far_keys_and_page_edges_matter (sharpened
# weights, all three configurations) is where a lost key shows in both precisions.
LENGTHS = {"a": [5, 11, 17, 40, 64, 65, 100], "b": [1, 9, 33, 70, 128, 129, 200], "c": [3, 127, 128, 129, 300, 700, 64]}

_engines = {}


def engine_for(tag, dtype):
    from llm_infer_engine_b200 import Engine
    key = (tag, dtype)
    if key not in _engines:
        _engines[key] = Engine(helpers.model_folder(tag), dtype=dtype, max_batch=8, max_tokens=64 * 40,
                               cuda_graph=False)
    return _engines[key]


def requests_for(tag):
    cfg = helpers.TINY[tag]["cfg"]
    lens = [l for l in LENGTHS[tag] if l <= cfg["max_position_embeddings"]]
    return {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=100 + i) for i, n in enumerate(lens)}


def oracle(tag, requests):
    folder = helpers.model_folder(tag)
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    return {rid: plain.logits(w, cfg, toks) for rid, toks in requests.items()}


def check(got, want, dtype, what):
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid, got[rid].shape, want[rid].shape)
        diff = (got[rid] - want[rid]).abs()
        worst = int(diff.max(dim=1).values.argmax())
        tol = helpers.logit_bound(dtype, want[rid])
        assert float(diff.max()) <= tol, (f"{what}: request {rid} differs by {float(diff.max()):.3e} "
                                          f"(tolerance {tol}), first at token {int((diff.max(dim=1).values > tol).nonzero()[0])}, "
                                          f"worst at token {worst} of {len(diff)}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["a", "b", "c"])
@pytest.mark.parametrize("mode", ["whole", "tail", "batched"])
def test_replay_matches_plain(tag, dtype, mode):
    requests = requests_for(tag)
    want = oracle(tag, requests)
    if mode == "whole":
        steps = helpers.plan_whole(requests)
    elif mode == "tail":
        steps = helpers.plan_tail(requests, 32)
    else:
        steps = helpers.plan_batched(requests, batch_size=3)
    engine = engine_for(tag, dtype)
    got = helpers.run_plan_engine(engine, steps)
    check(got, want, dtype, f"{tag}/{dtype}/{mode}")
    if dtype == "bfloat16":
        from llm_infer_engine_b200.kernels import ops
        ops.check_tc_status("cuda")
    assert engine.cache.free_slots() == engine.cache.n_slots
    assert engine.cache.free_pages() == engine.cache.n_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run_program(dtype):
    """bin/trace_run itself, as a subprocess, on batches of unequal lengths."""
    tag = "b"
    requests = requests_for(tag)
    want = oracle(tag, requests)
    steps = helpers.plan_batched(requests, batch_size=4)
    got = helpers.run_plan_trace_run(helpers.model_folder(tag), dtype, steps, helpers.max_tokens_for(steps),
                                     helpers.TINY[tag]["cfg"]["vocab_size"])
    check(got, want, dtype, f"trace_run/{dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_requests", [13, 40])
def test_wide_batches_match_plain(dtype, n_requests):
    """Batches of 13 and of 40 sequences decoded together: above 8 rows the bfloat16 step takes other
    kernels (the library product for most projections, the add-into product up to 16 rows, other block
    forms of the decode attention) than the batches of the other tests."""
    from llm_infer_engine_b200 import Engine
    tag = "c"
    folder = helpers.model_folder(tag)
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    g = torch.Generator().manual_seed(n_requests)
    lens = [int(x) for x in torch.randint(2, 150, (n_requests,), generator=g)]
    lens[0], lens[1] = 129, 64
    requests = {f"w{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=300 + i) for i, n in enumerate(lens)}
    want = {rid: plain.logits(w, cfg, toks) for rid, toks in requests.items()}
    steps = helpers.plan_batched(requests, batch_size=n_requests, prompt_frac=0.8)
    engine = Engine(folder, dtype=dtype, max_batch=n_requests, max_tokens=64 * 3 * n_requests, cuda_graph=False)
    got = helpers.run_plan_engine(engine, steps)
    check(got, want, dtype, f"{tag}/{dtype}/wide{n_requests}")
    if dtype == "bfloat16":
        from llm_infer_engine_b200.kernels import ops
        ops.check_tc_status("cuda")
    assert engine.cache.free_slots() == engine.cache.n_slots
