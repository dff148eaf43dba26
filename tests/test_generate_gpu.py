"""Generation through the Python entry point and the command line, on the GPU: greedy tokens
against the plain implementation, batches of unequal prompts, stop tokens, sequences that end
earlier, batch after batch on few slots, captured steps against eager steps, seeded sampling
that does not depend on batching, long decoding, and weights made so that far keys matter."""
import os
import subprocess
import sys

import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu


def plain_greedy(w, cfg, prompt, n_new, stop=()):
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = plain.greedy(plain.logits(w, cfg, seq)[-1])
        out.append(tok)
        seq.append(tok)
        if tok in stop:
            break
    return out


def agree_or_near_tie(w, cfg, prompt, got, want_fn, gap):
    """Greedy tokens must match the plain implementation; where they part, the plain logits of
    the two candidates must be within `gap` (a near-tie). The engine's token is then followed, so
    that every later token is still compared, each against the plain logits of the engine's own history."""
    seq = list(prompt)
    for tok in got:
        row = plain.logits(w, cfg, seq)[-1]
        best = plain.greedy(row)
        if tok != best:
            assert float(row[best] - row[tok]) < gap, (len(seq), tok, best, float(row[best] - row[tok]))
        seq.append(tok)


@pytest.mark.parametrize("dtype,gap", [("float32", 1e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("tag", ["a", "b"])
@pytest.mark.parametrize("graph", [True, False])
def test_greedy_generation_matches_plain(tag, dtype, gap, graph):
    from llm_infer_engine_b200 import Engine, GenerationStats, generate
    folder = helpers.model_folder(tag)
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    lens = [5, 11, 17, 3, 40, 1, 9] if tag == "a" else [1, 9, 33, 70, 2, 64, 65]
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=200 + i) for i, n in enumerate(lens)]
    engine = Engine(folder, dtype=dtype, max_batch=3, max_tokens=64 * 9, cuda_graph=graph)   # 7 requests, 3 slots
    stats = GenerationStats()
    out = generate(engine, prompts, max_new_tokens=12, stop_ids=[], stats=stats)
    assert stats.batches >= 3 and stats.prefill_tokens == sum(lens)
    assert [len(o) for o in out] == [12] * len(prompts)
    for p, o in zip(prompts, out):
        agree_or_near_tie(w, cfg, p, o, None, gap)
    engine.cache.check()
    assert engine.cache.free_slots() == 3 and engine.cache.free_pages() == engine.cache.n_pages
    # the same requests in another grouping give the same tokens (float32: exactly)
    engine2 = Engine(folder, dtype=dtype, max_batch=7, cuda_graph=graph)
    out2 = generate(engine2, prompts, max_new_tokens=12, stop_ids=[])
    if dtype == "float32":
        assert out2 == out


def test_stop_tokens_and_early_finish():
    from llm_infer_engine_b200 import Engine, generate
    folder = helpers.model_folder("b")
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=300 + i) for i, n in enumerate([4, 20, 8, 50])]
    free = [plain_greedy(w, cfg, p, 16) for p in prompts]
    # stop ids chosen from what the sequences really produce, at different depths
    stop = {free[0][2], free[2][9]}
    want = [plain_greedy(w, cfg, p, 16, stop) for p in prompts]
    assert len({len(x) for x in want}) > 1                      # they do end at different steps
    engine = Engine(folder, dtype="float32", max_batch=4, cuda_graph=True)
    seen = []
    got = generate(engine, prompts, max_new_tokens=16, stop_ids=sorted(stop),
                   on_tokens=lambda reqs, toks: seen.append((list(reqs), list(toks))))
    assert got == want                                          # the stop token is part of the output
    assert [t for reqs, toks in seen for r, t in zip(reqs, toks) if r == 1] == got[1]
    assert len(seen[-1][0]) < len(seen[0][0])                   # later steps carry fewer sequences
    assert engine.cache.free_slots() == 4
    # default stop ids come from the model's eos_token_id
    got_default = generate(engine, prompts, max_new_tokens=16)
    for seq in got_default:
        assert all(t not in (2, 3) for t in seq[:-1])
    # the per-sequence limit ends a sequence (main.py:274 of the reference)
    small = Engine(folder, dtype="float32", max_batch=1, max_seq_len=64, cuda_graph=False)
    out = generate(small, [helpers.random_tokens(cfg["vocab_size"], 60, seed=1)], max_new_tokens=50, stop_ids=[])
    assert len(out[0]) == 5                                     # 60 + 4 cached, the fifth sampled token has no room


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_step_equals_eager_step(dtype):
    """Logits of the captured one-token step against the eager step, lane by lane, with padding."""
    from llm_infer_engine_b200 import Engine
    folder = helpers.model_folder("b")
    cfg = helpers.read_config(folder)
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=400 + i) for i, n in enumerate([3, 64, 29])]
    nxt = [[7], [8], [9]]
    eager = Engine(folder, dtype=dtype, max_batch=4, cuda_graph=False)
    slots = [eager.open() for _ in prompts]
    eager.step(slots, prompts)
    want = eager.step(slots, nxt).cpu()
    graphed = Engine(folder, dtype=dtype, max_batch=4, cuda_graph=True)
    slots = [graphed.open() for _ in prompts]
    graphed.step(slots, prompts)
    g = graphed.decode_graph(4)                                  # one padding lane
    g.set_lanes(slots)
    g.tokens[:3].copy_(torch.tensor([7, 8, 9], dtype=torch.int32))
    for s in slots:
        graphed.cache.reserve(s, graphed.cache.lengths[s] + 1)
    got = g.replay()[:3].cpu()
    diff = (got - want).abs()
    assert torch.equal(got, want), (diff.max(dim=1).values.tolist(), (diff > 0).sum(dim=1).tolist(),
                                    bool(torch.isnan(got).any()), bool(torch.isnan(want).any()))
    assert graphed.cache.seq_lens.cpu().tolist()[:3] == [4, 65, 30]
    assert int(graphed.cache.seq_lens[graphed.cache.scratch_slot]) == 0


def test_capture_survives_a_collectable_engine():
    """An engine that only the garbage collector can free (a reference cycle) holds pinned memory; if
    it were collected in the middle of a graph capture, the capture would be invalidated. The capture
    collects first and keeps the collector off meanwhile, however eager the collector is set."""
    import gc
    from llm_infer_engine_b200 import Engine
    folder = helpers.model_folder("c")
    cfg = helpers.read_config(folder)
    prompt = helpers.random_tokens(cfg["vocab_size"], 40, seed=77)
    old = Engine(folder, dtype="bfloat16", max_batch=2, cuda_graph=False)
    s = old.open()
    old.step([s], [prompt])                       # its pinned upload buffer has been used by a copy
    old.close(s)
    old.keeps_itself_alive = old
    del old
    thresholds = gc.get_threshold()
    gc.set_threshold(1)                           # collect at every opportunity
    try:
        engine = Engine(folder, dtype="bfloat16", max_batch=2, cuda_graph=True)
        slot = engine.open()
        engine.step([slot], [prompt])
        g = engine.decode_graph(2)
        g.set_lanes([slot])
        g.tokens[:1].copy_(torch.tensor([5], dtype=torch.int32))
        engine.cache.reserve(slot, engine.cache.lengths[slot] + 1)
        logits = g.replay()[:1].cpu()
    finally:
        gc.set_threshold(*thresholds)
    assert torch.isfinite(logits).all()


def test_seeded_sampling_does_not_depend_on_batching():
    from llm_infer_engine_b200 import Engine, SamplingParams, generate, uniform_for
    folder = helpers.model_folder("b", std=0.12)                 # livelier logits than N(0, 0.03) gives
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=500 + i) for i, n in enumerate([1, 9, 33, 70])]
    sp = SamplingParams(temperature=0.8, top_p=0.9, seed=99)
    together = generate(Engine(folder, dtype="float32", max_batch=4), prompts, 12, sp, stop_ids=[])
    one_by_one = generate(Engine(folder, dtype="float32", max_batch=1, cuda_graph=False), prompts, 12, sp, stop_ids=[])
    assert together == one_by_one
    assert together != generate(Engine(folder, dtype="float32", max_batch=4), prompts, 12,
                                SamplingParams(temperature=0.8, top_p=0.9, seed=100), stop_ids=[])
    # each token is the plain draw at the uniform number of (seed, request index, draw index). The kernel draws
    # in float32 and the plain implementation in float64: they may part only where the uniform number lies within
    # 1e-5 of an edge of the cumulative distribution, or top_p within 1e-5 of a mass at which a token is cut.
    # After such an edge the engine's own token is followed, so every later draw is still compared.
    edges = 0
    for r, (p, out) in enumerate(zip(prompts, together)):
        seq = list(p)
        for i, tok in enumerate(out):
            row = plain.logits(w, cfg, seq)[-1]
            u = uniform_for(99, r, i)
            want = plain.sample_with_uniform(row, 0.8, 0.9, u)
            if tok != want:
                draw_gap, cut_gap = plain.sample_margins(row, 0.8, 0.9, u)
                assert min(draw_gap, cut_gap) < 1e-5, (r, i, tok, want, draw_gap, cut_gap)
                edges += 1
            seq.append(tok)
    assert edges <= 2, edges
    assert sum(len(set(o)) for o in together) > 20               # it does sample, not repeat one token


# per configuration: the factor on the q and k projections, the lengths, the bfloat16 bound. Sharper scores cost
# bfloat16 accuracy by themselves (a score of 30 carries the rounding of q and k as 0.1), so the factor is
# chosen per model to keep the bound several times below what a lost page of keys would change.
SHARP = {"a": (12.0, [128, 65, 100, 64], 0.03), "b": (6.0, [200, 130, 256, 65], 0.08),
         "c": (2.0, [300, 130, 700, 65], 0.08)}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["a", "b", "c"])
def test_far_keys_and_page_edges_matter(tag, dtype):
    """Random small weights give nearly flat attention, which would hide a lost key. Here q and k
    projections are scaled up so that each query looks hard at a few keys, many of them far away
    or across page edges; one token at a time over several pages, slots used again."""
    from safetensors.torch import load_file, save_file
    import json
    from llm_infer_engine_b200 import Engine
    scale, lens, tol = SHARP[tag]
    if dtype == "float32":
        tol = 1e-4
    src = helpers.model_folder(tag)
    t = load_file(os.path.join(src, "model.safetensors"))
    for name in t:
        if "q_proj" in name or "k_proj" in name:
            t[name] = (t[name].float() * scale).to(torch.bfloat16)
    folder = helpers.scratch_folder("llmie_sharp_")
    save_file(t, os.path.join(folder, "model.safetensors"))
    json.dump(helpers.read_config(src), open(os.path.join(folder, "config.json"), "w"))
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    requests = {f"s{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=600 + i) for i, n in enumerate(lens)}
    want = {rid: plain.logits(w, cfg, toks) for rid, toks in requests.items()}
    engine = Engine(folder, dtype=dtype, max_batch=2, max_tokens=64 * 16, cuda_graph=False)
    worst = 0.0
    for plan in (helpers.plan_whole(requests), helpers.plan_tail(requests, 100), helpers.plan_batched(requests, 2, 0.3),
                 helpers.plan_chunked(requests, 50)):
        got = helpers.run_plan_engine(engine, plan)
        for rid in requests:
            err = float((got[rid] - want[rid]).abs().max())
            worst = max(worst, err)
            assert err <= tol, (rid, err)
    print(f"sharp {tag} {dtype}: worst {worst:.3e}")
    # and the sharpness is real: dropping the first page of keys changes the logits by far more than tol
    toks = requests["s0"]
    full = plain.logits(w, cfg, toks)[-1]
    cut = plain.logits(w, cfg, toks[64:])[-1]
    assert float((full - cut).abs().max()) > 5 * tol, float((full - cut).abs().max())


def test_long_decoding_in_float32():
    """Several hundred one-token steps (graph replays) against one whole-sequence pass."""
    from llm_infer_engine_b200 import Engine, generate
    folder = helpers.model_folder("b")
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    prompt = helpers.random_tokens(cfg["vocab_size"], 3, seed=700)
    engine = Engine(folder, dtype="float32", max_batch=2, cuda_graph=True)
    out = generate(engine, [prompt, prompt[:1]], max_new_tokens=250, stop_ids=[])
    for p, o in zip([prompt, prompt[:1]], out):
        seq = p + o
        ref = plain.logits(w, cfg, seq[:-1])
        picks = ref[len(p) - 1:].argmax(-1).tolist()
        for i, (a, b) in enumerate(zip(o, picks)):
            if a != b:
                row = ref[len(p) - 1 + i]
                assert float(row[b] - row[a]) < 1e-5, (i, a, b)
                break


def test_command_line_with_prompt_ids(tmp_path):
    folder = helpers.model_folder("a")
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    prompt = helpers.random_tokens(cfg["vocab_size"], 9, seed=800)
    env = dict(os.environ, LLM_MAX_NEW_TOKENS="6")
    proc = subprocess.run([sys.executable, os.path.join(helpers.ROOT, "main.py"), "--model", folder, "--prompt-ids",
                           ",".join(map(str, prompt)), "--dtype", "float32", "--env-file", str(tmp_path / "none")],
                          capture_output=True, text=True, env=env, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    out = proc.stdout
    assert "Prefill:" in out and "(9 tokens)" in out and "TPS:" in out and "Total:" in out
    block = out.split("OUTPUT")[1].split("=" * 70)[1]
    ids = [int(x) for x in block.split()]
    want = plain_greedy(w, cfg, prompt, 6, stop=(2,))
    assert ids == want


def test_one_captured_step_serves_every_sampling_setting():
    """Temperature, top-p and seed live in device memory beside the captured step: calls with other settings reuse the
    capture (a greedy and a drawing one per lane count and length bucket, however many settings come) and draw what an
    engine that has seen only that setting draws."""
    from llm_infer_engine_b200 import Engine, SamplingParams, generate
    folder = helpers.model_folder("b", std=0.12)
    cfg = helpers.read_config(folder)
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=900 + n) for n in (7, 21)]
    settings = [SamplingParams(0.8, 0.9, 1), SamplingParams(0.8, 0.9, 2), SamplingParams(1.3, 0.5, 2), SamplingParams(),
                SamplingParams(0.3, 1.0, 77), SamplingParams(0.8, 0.9, 1)]
    engine = Engine(folder, dtype="float32", max_batch=2)
    outs = [generate(engine, prompts, 10, sp, stop_ids=[]) for sp in settings]
    assert len(engine._graphs) == 2, sorted(engine._graphs)          # (2 lanes, 512, greedy) and (2 lanes, 512, draw)
    assert outs[0] == outs[5] and outs[0] != outs[1]                  # the seed matters, and nothing else sticks
    for sp, out in zip(settings, outs):
        fresh = generate(Engine(folder, dtype="float32", max_batch=2), prompts, 10, sp, stop_ids=[])
        assert out == fresh, sp
