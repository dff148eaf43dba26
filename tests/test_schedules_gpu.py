"""Ways of cutting the work that the replay plans of the other files do not produce, each against the
plain implementation: prompts taken in pieces (several tokens at a start position above zero), steps that
mix such a piece with one-token sequences, captured steps of more than 8 lanes with padding lanes, a
generation that outgrows its captured step's length bucket, and the length stops of the captured loop."""
import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu

_engines = {}
_oracles = {}


def engine_for(tag, dtype, graph=False, max_batch=8):
    from llm_infer_engine_b200 import Engine
    key = (tag, dtype, graph, max_batch)
    if key not in _engines:
        _engines[key] = Engine(helpers.model_folder(tag), dtype=dtype, max_batch=max_batch,
                               max_tokens=64 * 6 * max_batch, cuda_graph=graph)
    return _engines[key]


def setup(tag, lens, seed0):
    key = (tag, tuple(lens), seed0)
    if key not in _oracles:
        folder = helpers.model_folder(tag)
        w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
        requests = {f"r{i}": helpers.random_tokens(cfg["vocab_size"], n, seed=seed0 + i) for i, n in enumerate(lens)}
        _oracles[key] = (requests, {rid: plain.logits(w, cfg, toks) for rid, toks in requests.items()})
    return _oracles[key]


def check(got, want, dtype, what):
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid, got[rid].shape, want[rid].shape)
        diff = (got[rid] - want[rid]).abs().max(dim=1).values
        bound = helpers.logit_bound(dtype, want[rid])
        assert float(diff.max()) <= bound, (f"{what}: request {rid} differs by {float(diff.max()):.3e} (bound "
                                            f"{bound:.3e}), first at token {int((diff > bound).nonzero()[0])} of {len(diff)}")


LENS = {"b": [200, 70, 129, 33], "c": [300, 129, 64, 700]}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["b", "c"])
@pytest.mark.parametrize("chunk", [7, 64, 100])
def test_prompts_in_pieces_match_plain(tag, dtype, chunk):
    requests, want = setup(tag, LENS[tag], 400)
    engine = engine_for(tag, dtype)
    got = helpers.run_plan_engine(engine, helpers.plan_chunked(requests, chunk))
    check(got, want, dtype, f"{tag}/{dtype}/chunks of {chunk}")
    assert engine.cache.free_slots() == engine.cache.n_slots and engine.cache.free_pages() == engine.cache.n_pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("tag", ["b", "c"])
@pytest.mark.parametrize("chunk", [5, 64])
def test_a_prompt_in_pieces_beside_one_token_sequences(tag, dtype, chunk):
    """One step holds a piece of a prompt (many tokens, start above zero) and sequences that bring one
    token each: every token must see exactly the keys of its own sequence up to its own position."""
    requests, want = setup(tag, LENS[tag], 400)
    engine = engine_for(tag, dtype)
    got = helpers.run_plan_engine(engine, helpers.plan_mixed(requests, chunk))
    check(got, want, dtype, f"{tag}/{dtype}/mixed, pieces of {chunk}")
    if dtype == "bfloat16":
        from llm_infer_engine_b200.kernels import ops
        ops.check_tc_status("cuda")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_requests,lanes", [(13, 16), (40, 64), (130, 256)])
def test_captured_steps_of_many_lanes(dtype, n_requests, lanes):
    """13 sequences in a captured step of 16 lanes, 40 in one of 64 and 130 in one of 256 (the rest are padding
    lanes on the scratch slot): the last 6 tokens of every request go through the captured step and are compared with
    the plain implementation and, in float32, bit for bit with the same steps run eagerly."""
    tag, tail = "c", 6
    g = torch.Generator().manual_seed(n_requests)
    lens = [int(x) for x in torch.randint(8, 150, (n_requests,), generator=g)]
    lens[0], lens[1], lens[2] = 129 + tail, 64 + tail, 65 + tail
    requests, want = setup(tag, lens, 3000)
    ids = list(requests)
    engine = engine_for(tag, dtype, graph=True, max_batch=n_requests)
    cache = engine.cache

    def run(captured: bool):
        slots = [engine.open() for _ in ids]
        engine.step(slots, [requests[r][:-tail] for r in ids], "last")
        rows = []
        graph = engine.decode_graph(lanes, max(lens)) if captured else None
        if captured:
            assert graph.n == lanes
            graph.set_lanes(slots)
        for t in range(tail):
            toks = [requests[r][len(requests[r]) - tail + t] for r in ids]
            if captured:
                graph.tokens[:len(ids)].copy_(torch.tensor(toks, dtype=torch.int32))
                for s in slots:
                    cache.reserve(s, cache.lengths[s] + 1)
                rows.append(graph.replay()[:len(ids)].clone())
                for s in slots:
                    cache.note_appended(s, cache.lengths[s] + 1, device_updated=True)
            else:
                rows.append(engine.step(slots, [[x] for x in toks], "last").clone())
        for s in slots:
            engine.close(s)
        return torch.stack(rows, dim=1).float()          # [request, tail, vocab]

    captured = run(True)
    for i, rid in enumerate(ids):
        ref = want[rid][-tail:]
        err = float((captured[i].cpu() - ref).abs().max())
        assert err <= helpers.logit_bound(dtype, want[rid]), (rid, lens[i], err)
    if dtype == "float32":
        eager = run(False)
        assert torch.equal(captured, eager), float((captured - eager).abs().max())
    cache.check()
    assert cache.free_slots() == cache.n_slots


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_generation_across_a_length_bucket(dtype):
    """A 505-token prompt and 24 new tokens: the sequence outgrows the 512-token captured step in the
    middle of the run and goes on in the 1024-token one. Captured and eager loops draw the same tokens,
    and they are the plain implementation's greedy tokens."""
    from llm_infer_engine_b200 import Engine, generate
    tag = "c"
    folder = helpers.model_folder(tag)
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=5000 + n) for n in (505, 490)]
    outs = {}
    for graph in (True, False):
        engine = Engine(folder, dtype=dtype, max_batch=2, cuda_graph=graph)
        outs[graph] = generate(engine, prompts, max_new_tokens=24, stop_ids=[])
        if graph:
            limits = sorted({key[1] for key in engine._graphs})
            assert limits == [512, 1024], limits                 # both buckets were really used
    assert outs[True] == outs[False]
    gap = 1e-5 if dtype == "float32" else 0.02
    for p, o in zip(prompts, outs[True]):
        assert len(o) == 24
        seq = list(p)
        for tok in o:            # follow the engine's tokens; each must be the plain argmax or tie with it
            row = plain.logits(w, cfg, seq)[-1]
            best = int(row.argmax())
            assert tok == best or float(row[best] - row[tok]) < gap * max(1.0, float(row.abs().max())), (len(seq), tok, best)
            seq.append(tok)


@pytest.mark.parametrize("graph", [True, False])
def test_length_stops_of_the_loop(graph):
    """max_new_tokens of 1 and 2, and the stop at max_seq_len, with the captured loop and the eager one:
    the counts are exact, the tokens are those of an unlimited run, and the cache is given back whole."""
    from llm_infer_engine_b200 import Engine, generate
    tag = "b"
    folder = helpers.model_folder(tag)
    cfg = helpers.read_config(folder)
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=6000 + n) for n in (9, 30, 17)]
    engine = Engine(folder, dtype="float32", max_batch=4, max_seq_len=40, cuda_graph=graph)
    full = generate(engine, prompts, max_new_tokens=64, stop_ids=[])
    # a sequence may hold max_seq_len tokens in the cache; the token drawn after the last one is still returned
    assert [len(o) for o in full] == [40 - 9 + 1, 40 - 30 + 1, 40 - 17 + 1]
    for n in (1, 2, 5):
        out = generate(engine, prompts, max_new_tokens=n, stop_ids=[])
        assert [len(o) for o in out] == [n, n, n]
        assert out == [o[:n] for o in full]
    engine.cache.check()
    assert engine.cache.free_slots() == engine.cache.n_slots and engine.cache.free_pages() == engine.cache.n_pages


def test_superseded_counters_stay_valid_for_earlier_captures():
    """A captured step keeps the address of the attention counters it was captured with. When a later,
    wider step needs more counters than were allocated, the earlier capture must go on working: replayed
    after the wider step ran, it still equals the eager step."""
    from llm_infer_engine_b200 import Engine
    tag = "c"
    folder = helpers.model_folder(tag)
    cfg = helpers.read_config(folder)
    engine = Engine(folder, dtype="bfloat16", max_batch=48, max_tokens=64 * 3 * 48 + 64 * 12, cuda_graph=True)
    plan = engine.kernels
    plan.MIN_COUNTERS = 2                            # as if little had been allocated: a wider step outgrows it
    cache = engine.cache
    prompt = helpers.random_tokens(cfg["vocab_size"], 600, seed=7000)      # long enough for several runs
    slot = engine.open()
    engine.step([slot], [prompt], "last")
    small = engine.decode_graph(1, 700)
    small.set_lanes([slot])
    first_ptr, first_len = plan._counters.data_ptr(), plan._counters.numel()
    assert first_len < 64
    others = [engine.open() for _ in range(40)]
    engine.step(others, [helpers.random_tokens(cfg["vocab_size"], 70, seed=7100 + i) for i in range(40)], "last")
    wide = engine.decode_graph(64, 700)
    wide.set_lanes(others)
    assert plan._counters.data_ptr() != first_ptr, "the wide step did not outgrow the counters"
    assert plan._retired and plan._retired[0].data_ptr() == first_ptr
    for s in others:
        cache.reserve(s, cache.lengths[s] + 1)
    wide.replay()
    for s in others:
        cache.note_appended(s, cache.lengths[s] + 1, device_updated=True)
    junk = [torch.full((first_len,), 7, dtype=torch.int32, device="cuda") for _ in range(64)]   # would land on freed counters
    tok = 5
    small.tokens[:1].copy_(torch.tensor([tok], dtype=torch.int32))
    cache.reserve(slot, cache.lengths[slot] + 1)
    got = small.replay()[:1].float().clone()
    cache.note_appended(slot, cache.lengths[slot] + 1, device_updated=True)
    # the same token eagerly on a second sequence with the same history
    twin = engine.open()
    engine.step([twin], [prompt], "last")
    want = engine.step([twin], [[tok]], "last").float()
    assert torch.equal(got, want), float((got - want).abs().max())
    assert int(plan._retired[0].abs().sum()) == 0    # the earlier capture left its counters clean
    del junk


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_lone_prompt_steps(dtype):
    """A lone prompt of a length that has come before runs as a captured step. Its logits are those of the
    eager step whatever changes between replays: the tokens, the slot, the start position (a second piece of
    the same length that goes on at position 70) and what the cache holds; other lengths and other `want`
    forms stay eager; only a few lengths are kept."""
    from llm_infer_engine_b200 import Engine
    from llm_infer_engine_b200.engine.engine import PrefillGraph
    tag, T = "c", 70
    folder = helpers.model_folder(tag)
    w, cfg = helpers.plain_weights(folder), helpers.read_config(folder)
    engine = Engine(folder, dtype=dtype, max_batch=4, max_tokens=64 * 16, cuda_graph=True)
    eager = Engine(folder, dtype=dtype, max_batch=4, max_tokens=64 * 16, cuda_graph=False)
    seqs = [helpers.random_tokens(cfg["vocab_size"], 2 * T, seed=8000 + i) for i in range(4)]
    held = engine.open()                                   # so that later requests get other slots
    for i, toks in enumerate(seqs):
        want = plain.logits(w, cfg, toks)
        a, b = engine.open(), eager.open()
        for piece in (toks[:T], toks[T:]):                 # the second piece starts at position 70
            got = engine.step([a], [piece], "last")
            ref = eager.step([b], [piece], "last")
            assert torch.equal(got, ref), (i, float((got - ref).abs().max()))
        err = float((got.float().cpu() - want[-1:]).abs().max())
        assert err <= helpers.logit_bound(dtype, want), (i, err)
        state = engine._prefill_graphs.get(T)
        assert isinstance(state, PrefillGraph) and state.graph is not None      # captured at the second piece of length 70
        engine.close(a)
        eager.close(b)
    engine.close(held)
    # other forms of the same length are not served by the capture
    slot = engine.open()
    all_rows = engine.step([slot], [seqs[0][:T]], "all")
    assert all_rows.shape[0] == T
    engine.close(slot)
    # lengths beyond the few that are kept push the oldest out
    for n in range(20, 20 + PrefillGraph.KEEP + 2):
        for _ in range(2):
            slot = engine.open()
            engine.step([slot], [seqs[1][:n]], "last")
            engine.close(slot)
    assert len(engine._prefill_graphs) == PrefillGraph.KEEP and T not in engine._prefill_graphs
    engine.cache.check()
    assert engine.cache.free_slots() == engine.cache.n_slots
    # a slot that was given back names the scratch page in every entry of its block table again, never a page
    # that another sequence may hold by now
    for group in engine.cache._groups.values():
        assert bool((group.block_table == engine.cache.n_pages).all())
