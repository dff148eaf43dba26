"""The single-kernel one-token step (csrc/decode_stack.cu, engine/stacked.py) against the plain
implementation and against the part-by-part step: several lanes with a padding lane, sequences that
cross a page boundary, a first decoded token, slots that were used before, and the real 1B / 3B / 8B
layer shapes. Models whose parts the kernel does not know must not be given to it."""
import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def stacked_on(monkeypatch):
    monkeypatch.setenv("LLMIE_STACKED_DECODE", "1")      # off by default: it is the slower path so far


def decode_with_graph(engine, prompts, steps, feed, lanes):
    """Prompts in one eager step, then `steps` captured one-token steps fed with feed[i][t].
    Returns per request the logits of every decode step, [steps, vocab]."""
    slots = [engine.open() for _ in prompts]
    engine.step(slots, prompts)
    longest = max(len(p) for p in prompts) + steps
    g = engine.decode_graph(lanes, longest)
    g.set_lanes(slots)
    outs = [[] for _ in prompts]
    for t in range(steps):
        g.tokens[:len(prompts)].copy_(torch.tensor([f[t] for f in feed], dtype=torch.int32))
        for s in slots:
            engine.cache.reserve(s, engine.cache.lengths[s] + 1)
        logits = g.replay()
        for s in slots:
            engine.cache.note_appended(s, engine.cache.lengths[s] + 1, device_updated=True)
        rows = logits[:len(prompts)].cpu()
        for i in range(len(prompts)):
            outs[i].append(rows[i].clone())
    from llm_infer_engine_b200.kernels import ops
    ops.check_tc_status(engine.device)
    lens = engine.cache.seq_lens.cpu().tolist()
    for s, p in zip(slots, prompts):
        assert lens[s] == len(p) + steps
    for s in slots:
        engine.close(s)
    return [torch.stack(o) for o in outs], g


def test_only_known_stacks_are_taken():
    from llm_infer_engine_b200 import Engine
    assert Engine(helpers.model_folder("c"), dtype="bfloat16", max_batch=2).stacked_decode() is not None
    assert Engine(helpers.model_folder("c"), dtype="float32", max_batch=2).stacked_decode() is None
    # head sizes 16 and 32 are not the kernel's
    assert Engine(helpers.model_folder("a"), dtype="bfloat16", max_batch=2).stacked_decode() is None


@pytest.mark.parametrize("lanes", [1, 4, 8])
def test_stacked_step_matches_plain_and_eager(lanes):
    from llm_infer_engine_b200 import Engine
    folder = helpers.model_folder("c")
    cfg, w = helpers.read_config(folder), helpers.plain_weights(folder)
    n_req = {1: 1, 4: 3, 8: 8}[lanes]
    lengths = [61, 3, 127, 64, 1, 200, 65, 30][:n_req]           # 61 + 5 steps crosses a page boundary
    steps = 5
    prompts = [helpers.random_tokens(cfg["vocab_size"], n, seed=700 + i) for i, n in enumerate(lengths)]
    feed = [helpers.random_tokens(cfg["vocab_size"], steps, seed=800 + i) for i in range(n_req)]
    engine = Engine(folder, dtype="bfloat16", max_batch=8, max_seq_len=512)
    for round_ in range(2):                                      # the second round takes slots that were used
        got, g = decode_with_graph(engine, prompts, steps, feed, lanes)
        assert g.stacked is not None and g.launches_per_replay == 1
        for i, (p, f) in enumerate(zip(prompts, feed)):
            want = plain.logits(w, cfg, list(p) + list(f))[len(p):]
            err = float((got[i] - want).abs().max())
            assert err <= 3e-2, (lanes, round_, i, err)
    # the same steps part by part: the same math in another order of summation
    eager = Engine(folder, dtype="bfloat16", max_batch=8, max_seq_len=512, cuda_graph=False)
    slots = [eager.open() for _ in prompts]
    eager.step(slots, prompts)
    for t in range(steps):
        rows = eager.step(slots, [[f[t]] for f in feed]).cpu()
        for i in range(n_req):
            assert float((rows[i] - got[i][t]).abs().max()) <= 2e-2


def test_stacked_step_over_many_pages():
    """A sequence of 330 positions (six pages, the last one partly filled) with livelier weights than
    the default, so that the scores are peaked and a page that was skipped or misplaced shows."""
    from llm_infer_engine_b200 import Engine
    folder = helpers.model_folder("c", std=0.08)
    cfg, w = helpers.read_config(folder), helpers.plain_weights(folder)
    prompt = helpers.random_tokens(cfg["vocab_size"], 330, seed=11)
    feed = [helpers.random_tokens(cfg["vocab_size"], 3, seed=12)]
    engine = Engine(folder, dtype="bfloat16", max_batch=2, max_seq_len=512)
    got, _ = decode_with_graph(engine, [prompt], 3, feed, 1)
    want = plain.logits(w, cfg, list(prompt) + list(feed[0]))[len(prompt):]
    assert float((got[0] - want).abs().max()) <= max(3e-2, 0.015 * float(want.abs().max()))


@pytest.mark.parametrize("tag", ["1b", "3b", "8b"])
def test_stacked_step_real_shapes(tag):
    import test_real_shapes_gpu as real
    from llm_infer_engine_b200 import Engine
    folder, requests, want = real.setup(tag)
    engine = Engine(folder, dtype="bfloat16", max_batch=4, max_seq_len=512, max_tokens=64 * 12)
    ids = list(requests)
    tail = 4
    prompts = [requests[r][:-tail] for r in ids]
    feed = [requests[r][-tail:] for r in ids]
    got, g = decode_with_graph(engine, prompts, tail, feed, 4)
    assert g.stacked is not None
    for i, r in enumerate(ids):
        ref = want[r][-tail:]
        err = float((got[i] - ref).abs().max())
        assert err <= 0.015 * float(want[r].abs().max()), (tag, r, err)
