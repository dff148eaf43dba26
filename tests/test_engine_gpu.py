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


AWKWARD = [
    # head size 48 (no tensor-core attention), width and feed-forward no multiples of 16, an odd vocabulary
    dict(num_hidden_layers=2, hidden_size=136, num_attention_heads=3, num_key_value_heads=1, head_dim=48,
         intermediate_size=200, vocab_size=1001, rope_theta=30000.0, rope_scaling=None, rms_norm_eps=3e-6,
         tie_word_embeddings=True, max_position_embeddings=192),
    # head size 80, five query heads on five KV heads, untied head, widths that are multiples of 8 only
    dict(num_hidden_layers=1, hidden_size=200, num_attention_heads=5, num_key_value_heads=5, head_dim=80,
         intermediate_size=328, vocab_size=777, rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5,
         tie_word_embeddings=False, max_position_embeddings=160),
    # head size 112 and 144 do not exist in the fast kernels either; 7 query heads on one KV head
    dict(num_hidden_layers=1, hidden_size=96, num_attention_heads=7, num_key_value_heads=1, head_dim=112,
         intermediate_size=72, vocab_size=130, rope_theta=500000.0,
         rope_scaling={"rope_type": "llama3", "factor": 2.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                       "original_max_position_embeddings": 32},
         rms_norm_eps=1e-5, tie_word_embeddings=True, max_position_embeddings=150),
    # sizes the tensor-core kernels DO take, at their edges: 20 query heads on one KV head of 64 (two chunks of 16
    # query heads per KV head in the decode attention, only the first of which writes the cache) ...
    dict(num_hidden_layers=2, hidden_size=128, num_attention_heads=20, num_key_value_heads=1, head_dim=64,
         intermediate_size=160, vocab_size=300, rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5,
         tie_word_embeddings=True, max_position_embeddings=200),
    # ... and as many KV heads as query heads, head size 128
    dict(num_hidden_layers=1, hidden_size=64, num_attention_heads=3, num_key_value_heads=3, head_dim=128,
         intermediate_size=96, vocab_size=200, rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5,
         tie_word_embeddings=False, max_position_embeddings=200),
    # a width, a feed-forward width and a vocabulary that are no multiples of 8: no 16-byte loads anywhere
    dict(num_hidden_layers=2, hidden_size=100, num_attention_heads=5, num_key_value_heads=5, head_dim=16,
         intermediate_size=60, vocab_size=51, rope_theta=10000.0, rope_scaling=None, rms_norm_eps=1e-5,
         tie_word_embeddings=True, max_position_embeddings=140),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", [0, 1, 2, 3, 4, 5])
def test_unusual_sizes(which, dtype):
    """Head sizes in steps of 16 that the tensor-core kernels do not take, widths that are no multiples of 16 or 8, an
    odd vocabulary, any number of heads and groups (the plain kernels of the same math serve them), and the edges of
    what the tensor-core kernels do take (more than 16 query heads per KV head, one query head per KV head). Whole, one
    by one, in batches of 3 and of 10, in pieces; never a wrong result."""
    from llm_infer_engine_b200 import Engine, write_random_model
    cfg = dict(plain.TINY_A, **AWKWARD[which])
    folder = helpers.scratch_folder("llmie_awkward_")
    write_random_model(cfg, folder, seed=20 + which, std=0.08, norm_range=(0.8, 1.2))
    w = helpers.plain_weights(folder)
    lens = [l for l in (1, 9, 64, 65, 130, 12, 31, 100, 7, 50) if l <= cfg["max_position_embeddings"]]
    requests = {f"k{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=50 + i) for i, n in enumerate(lens)}
    want = {rid: plain.logits(w, cfg, toks) for rid, toks in requests.items()}
    engine = Engine(folder, dtype=dtype, max_batch=10, max_tokens=64 * 24, cuda_graph=False)
    # batches of 3 and of 10: one-token steps of up to 8 rows and of more take different kernels
    for plan in (helpers.plan_whole(requests), helpers.plan_tail(requests, 32), helpers.plan_batched(requests, 3),
                 helpers.plan_batched(requests, 10), helpers.plan_chunked(requests, 33)):
        check(helpers.run_plan_engine(engine, plan), want, dtype, f"awkward {which}/{dtype}")
    # and through the captured step and the loop
    from llm_infer_engine_b200 import generate
    engine2 = Engine(folder, dtype=dtype, max_batch=3, cuda_graph=True)
    prompts = [requests["k1"], requests["k2"][:20], requests["k0"]]
    out = generate(engine2, prompts, max_new_tokens=5, stop_ids=[])
    out_eager = generate(engine, prompts, max_new_tokens=5, stop_ids=[])
    if dtype == "float32":
        assert out == out_eager
    for p, o in zip(prompts, out):
        seq = list(p)
        for tok in o:
            row = plain.logits(w, cfg, seq)[-1]
            best = int(row.argmax())
            assert tok == best or float(row[best] - row[tok]) < (1e-5 if dtype == "float32" else 0.03) * max(1.0, float(row.abs().max()))
            seq.append(tok)
