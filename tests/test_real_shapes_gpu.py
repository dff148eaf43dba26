"""The layer shapes of real Llama models (1B, 3B, 8B), a few layers each, random weights:
the float32 engine must match the plain implementation closely however the work is cut, and the
bfloat16 engine (tensor-core attention, fused one-token kernels, head size 128, 128256-token
vocabulary) must stay within bfloat16 rounding of it."""
import copy

import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu

LLAMA3 = {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
          "original_max_position_embeddings": 8192}
BASE = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "rope_theta": 500000.0, "rope_scaling": LLAMA3,
        "rms_norm_eps": 1e-5, "max_position_embeddings": 131072, "hidden_act": "silu", "attention_bias": False,
        "mlp_bias": False, "eos_token_id": 128001, "torch_dtype": "bfloat16", "vocab_size": 128256}
SHAPES = {
    "1b": dict(BASE, num_hidden_layers=2, hidden_size=2048, num_attention_heads=32, num_key_value_heads=8, head_dim=64,
               intermediate_size=8192, tie_word_embeddings=True),
    "3b": dict(BASE, num_hidden_layers=1, hidden_size=3072, num_attention_heads=24, num_key_value_heads=8, head_dim=128,
               intermediate_size=8192, tie_word_embeddings=True),
    "8b": dict(BASE, num_hidden_layers=1, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
               intermediate_size=14336, tie_word_embeddings=False,
               rope_scaling=dict(LLAMA3, factor=8.0)),
}
_cache = {}


def setup(tag):
    if tag not in _cache:
        from llm_infer_engine_b200 import write_random_model
        folder = helpers.scratch_folder(f"llmie_{tag}_")
        write_random_model(SHAPES[tag], folder, seed=2, std=0.02)
        w = helpers.plain_weights(folder)
        requests = {f"q{i}": helpers.random_tokens(128256, n, seed=900 + i) for i, n in enumerate([70, 9, 150])}
        want = {rid: plain.logits(w, SHAPES[tag], toks) for rid, toks in requests.items()}
        _cache[tag] = (folder, requests, want)
    return _cache[tag]


@pytest.mark.parametrize("tag", ["1b", "3b", "8b"])
# float32: 1e-3 absolute, the bound this benchmark shape is quoted with. bfloat16: rounding grows with the width of the sums and the
# size of the logits, so the bound is relative to the largest logit of the request (1.5 %).
@pytest.mark.parametrize("dtype,tol", [("float32", 1e-3), ("bfloat16", 0.015)])
def test_real_shapes(tag, dtype, tol):
    from llm_infer_engine_b200 import Engine
    from llm_infer_engine_b200.kernels import ops
    folder, requests, want = setup(tag)
    engine = Engine(folder, dtype=dtype, max_batch=4, max_seq_len=512, max_tokens=64 * 12, cuda_graph=False)
    for plan in (helpers.plan_whole(requests), helpers.plan_tail(requests, 32), helpers.plan_batched(requests, 3)):
        got = helpers.run_plan_engine(engine, plan)
        for rid in requests:
            err = float((got[rid] - want[rid]).abs().max())
            bound = tol if dtype == "float32" else tol * float(want[rid].abs().max())
            assert err <= bound, (tag, dtype, rid, err, bound)
            if dtype == "float32":      # identical greedy tokens, except where the plain top two nearly tie
                a, b = got[rid].argmax(-1), want[rid].argmax(-1)
                for t in (a != b).nonzero().flatten().tolist():
                    top2 = want[rid][t].topk(2).values
                    assert float(top2[0] - top2[1]) < 1e-5, (tag, rid, t)
    if dtype == "bfloat16":
        ops.check_tc_status("cuda")
    del engine
    torch.cuda.empty_cache()


def test_long_context_1b_shape():
    """A 2,400-token sequence at the 1B layer shape in bfloat16: the prompt in one step (tensor-core
    attention over 19 key tiles), then 24 tokens one by one (decode attention over 38 pages, cut into
    runs that are merged), eagerly and through the captured step, against the plain implementation at
    the last positions."""
    from llm_infer_engine_b200 import Engine
    from llm_infer_engine_b200.kernels import ops
    folder, _, _ = setup("1b")
    cfg = SHAPES["1b"]
    w = helpers.plain_weights(folder)
    tokens = helpers.random_tokens(128256, 2400, seed=77)
    tail = 24
    hidden = plain.hidden_states(w, cfg, tokens)[-(tail + 1):]      # logits at the last tail + 1 positions only
    want = plain.rms_norm(hidden, w["model.norm.weight"], cfg["rms_norm_eps"]) @ plain.head_weight(w, cfg).T
    bound = 0.015 * float(want.abs().max())
    engine = Engine(folder, dtype="bfloat16", max_batch=2, max_seq_len=4096, max_tokens=2 * 4096)
    # eager steps
    slot = engine.open()
    got = [engine.step([slot], [tokens[:-tail]], "last").float().cpu()]
    for t in tokens[-tail:]:
        got.append(engine.step([slot], [[t]], "last").float().cpu())
    engine.close(slot)
    err = float((torch.cat(got) - want).abs().max())
    assert err <= bound, ("eager", err, bound)
    # the captured step
    slot = engine.open()
    engine.step([slot], [tokens[:-tail]], "last")
    g = engine.decode_graph(1, len(tokens))
    g.set_lanes([slot])
    rows = []
    for t in tokens[-tail:]:
        g.tokens[:1].copy_(torch.tensor([t], dtype=torch.int32))
        engine.cache.reserve(slot, engine.cache.lengths[slot] + 1)
        rows.append(g.replay()[:1].float().cpu().clone())
        engine.cache.note_appended(slot, engine.cache.lengths[slot] + 1, device_updated=True)
    engine.close(slot)
    err = float((torch.cat(rows) - want[1:]).abs().max())
    assert err <= bound, ("graph", err, bound)
    ops.check_tc_status("cuda")


def test_full_depth_1b_float32():
    """All 16 layers of the 1B shape in float32: one 150-token request whole, then again with its last 32
    tokens one by one, within 1e-3 of the plain implementation at every position, so that the growth of
    rounding differences over the full depth is pinned, not only the widths."""
    from llm_infer_engine_b200 import Engine, write_random_model
    cfg = dict(SHAPES["1b"], num_hidden_layers=16)
    folder = helpers.scratch_folder("llmie_1b_full_")
    write_random_model(cfg, folder, seed=2, std=0.02)
    w = helpers.plain_weights(folder)
    requests = {"full": helpers.random_tokens(128256, 150, seed=950)}
    want = plain.logits(w, cfg, requests["full"])
    del w
    engine = Engine(folder, dtype="float32", max_batch=1, max_seq_len=256, max_tokens=256, cuda_graph=False)
    for plan in (helpers.plan_whole(requests), helpers.plan_tail(requests, 32)):
        got = helpers.run_plan_engine(engine, plan)["full"]
        err = float((got - want).abs().max())
        assert err <= 1e-3, err
        a, b = got.argmax(-1), want.argmax(-1)
        for t in (a != b).nonzero().flatten().tolist():
            top2 = want[t].topk(2).values
            assert float(top2[0] - top2[1]) < 1e-5, t
    del engine
    torch.cuda.empty_cache()
