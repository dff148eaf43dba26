"""Host side of the part interfaces: how a layer names its parts, how a block declares its roles, how a cache
unit holds several named requests, and the stage names of traces. No GPU."""
import pytest
import torch

from llm_infer_engine_b200.cache import Cache, KVRequest, StateRequest
from llm_infer_engine_b200.config import LayerSpec, PartSpec
from llm_infer_engine_b200.kernels import trace
from llm_infer_engine_b200.parts import Block, Runtime, lookup


def test_layer_spec_forms():
    a, b, n = PartSpec("gqa_attention", {"x": 1}), PartSpec("swiglu", {}), PartSpec("rmsnorm", {"size": 4, "eps": 1e-5})
    names = {"mixer": "attn", "feed_forward": "mlp", "mixer_norm": "n1", "feed_forward_norm": "n2"}
    positional = LayerSpec("pre_norm", a, b, n, n, names)
    keywords = LayerSpec(block="pre_norm", mixer=a, feed_forward=b, mixer_norm=n, feed_forward_norm=n, names=names)
    mapping = LayerSpec("pre_norm", parts={"mixer": a, "feed_forward": b, "mixer_norm": n, "feed_forward_norm": n}, names=names)
    for spec in (positional, keywords, mapping):
        assert spec.block == "pre_norm" and dict(spec.parts) == dict(positional.parts) and spec.mixer is a
        assert spec.names["feed_forward_norm"] == "n2"
    other = LayerSpec("my_block", parts={"mixer": a, "post_norm": n}, names={"mixer": "m", "post_norm": "pn"})
    assert other.post_norm is n and sorted(other.parts) == ["mixer", "post_norm"]
    with pytest.raises(AttributeError, match="no role 'feed_forward'"):
        other.feed_forward
    with pytest.raises(AttributeError, match="read-only"):
        other.block = "x"
    with pytest.raises(ValueError, match="no checkpoint sub-name"):
        LayerSpec("my_block", parts={"mixer": a}, names={})
    with pytest.raises(TypeError, match="given twice"):
        LayerSpec("pre_norm", a, mixer=a, names=names)
    with pytest.raises(TypeError, match="must be a PartSpec"):
        LayerSpec("my_block", parts={"mixer": "gqa"}, names={"mixer": "m"})


def test_block_checks_its_roles():
    pre_norm = lookup("block", "pre_norm")
    assert sorted(pre_norm.ROLES) == ["feed_forward", "feed_forward_norm", "mixer", "mixer_norm"]
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32, max_positions=8)
    with pytest.raises(ValueError, match="missing .*feed_forward_norm"):
        pre_norm({"mixer": object(), "feed_forward": object(), "mixer_norm": object()}, rt)
    with pytest.raises(ValueError, match="unknown .*extra"):
        pre_norm({"mixer": 1, "feed_forward": 2, "mixer_norm": 3, "feed_forward_norm": 4, "extra": 5}, rt)

    class Clash(Block):
        ROLES = {"parts": "mixer"}

    with pytest.raises(ValueError, match="collide"):
        Clash({"parts": object()}, rt)


def test_a_unit_holds_several_named_requests():
    unit0 = [KVRequest(2, 16, 0, name="attn.kv"), StateRequest("rec.s", (5,)), StateRequest("rec.t", (2, 3), torch.float32)]
    unit1 = [KVRequest(2, 16, 0), KVRequest(2, 16, 8, name="local")]          # two requests, two groups
    unit2 = [KVRequest(2, 16, 0, name="a"), KVRequest(2, 16, 0, name="b")]    # two requests of one geometry
    cache = Cache([unit0, unit1, unit2], n_slots=3, max_tokens=64 * 4, max_seq_len=128, dtype=torch.float32, device="cpu")
    assert sorted(r.geometry() for r in cache.groups()) == [(2, 16, 0), (2, 16, 8)]
    u0, u1, u2 = cache.unit(0), cache.unit(1), cache.unit(2)
    assert sorted(u0.kvs) == ["attn.kv"] and u0.kv is u0.kvs["attn.kv"]        # the only one there is
    assert u0.scoped("rec").state["s"].shape == (4, 5) and u0.scoped("rec").state["t"].shape == (4, 2, 3)
    assert u0.scoped("attn").kv is not None and u0.scoped("rec").kv is None
    assert u1.kv is u1.kvs["kv"] and u1.kvs["local"].window == 8
    assert u2.kv is None and u2.kvs["a"].k.data_ptr() != u2.kvs["b"].k.data_ptr()
    # members of one group share the block table, each has storage of its own
    assert u2.kvs["a"].block_table.data_ptr() == u1.kvs["kv"].block_table.data_ptr() == u0.kv.block_table.data_ptr()
    assert len({u0.kv.k.data_ptr(), u1.kv.k.data_ptr(), u2.kvs["a"].k.data_ptr(), u2.kvs["b"].k.data_ptr()}) == 4
    slot = cache.take_slot()
    u0.state["rec.s"][slot] = 7.0
    cache.give_back_slot(slot)
    assert cache.take_slot() == slot and float(u0.state["rec.s"][slot].abs().sum()) == 0.0      # zeroed on reuse
    with pytest.raises(ValueError, match="two KVRequests are named"):
        Cache([[KVRequest(1, 16), KVRequest(1, 16, 4)]], 1, 64, 64, torch.float32, "cpu")
    with pytest.raises(TypeError, match="unknown request"):
        Cache([["kv"]], 1, 64, 64, torch.float32, "cpu")


def test_trace_stage_names():
    assert not trace.active()
    trace.push("Attn_3")                      # no tracing: nothing is kept
    assert trace.generic_stage() == ""
    trace.pop()
    trace.timer = trace.KernelTimer.__new__(trace.KernelTimer)       # as inside `timing()`, without a device
    try:
        trace.push("Layers")
        trace.push("Attn_12")
        trace.push("QKV_proj")
        assert trace.generic_stage() == "QKV_proj"
        trace.pop()
        assert trace.generic_stage() == "Attn"                        # the layer number is taken off
        trace.pop()
        trace.pop()
        assert trace.generic_stage() == ""
    finally:
        trace.timer = None
