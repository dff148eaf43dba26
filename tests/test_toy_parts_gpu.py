"""Generality of the parts, shown with toy parts that exist only in this file.

A toy architecture is registered here without touching the library: its layers are chosen
one by one from the configuration (a recurrent mixer with a fixed-size state of its own, or the
library's attention with a window), its feed-forwards differ per layer (the library's SwiGLU, or
a toy routed one), and its run order names a layer twice and lets one entry read another's
cache. It is built through the same registry, loader, random mode, cache and step function as
Llama and is checked against a whole-sequence restatement written beside it.
"""
import math
from dataclasses import dataclass
from typing import Tuple

import pytest
import torch

import helpers
import plain_llama as plain

pytestmark = pytest.mark.gpu


# ------------------------------------------------------------------------------------------ toy parts
def _register():
    from llm_infer_engine_b200.cache import StateRequest
    from llm_infer_engine_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture
    from llm_infer_engine_b200.parts import (FeedForward, Linear, Mixer, ParamSpec, register_feed_forward,
                                             register_mixer)

    class DecayMixer(Mixer):
        """s_t = decay * s_{t-1} + x_t W_in^T ;  y_t = s_t W_out^T. The state s is per sequence,
        of fixed size, kept in the cache's state area between steps."""

        def __init__(self, params, runtime):
            super().__init__(params, runtime)
            self.hidden, self.width, self.decay = int(params["hidden"]), int(params["width"]), float(params["decay"])

        def param_specs(self):
            return {"in_proj.weight": ParamSpec((self.width, self.hidden)),
                    "out_proj.weight": ParamSpec((self.hidden, self.width))}

        def load(self, tensors):
            self.w_in, self.w_out = Linear(tensors["in_proj.weight"]), Linear(tensors["out_proj.weight"])

        def cache_requests(self):
            return [StateRequest("s", (self.width,))]

        def forward(self, x, ctx, unit, owns_cache):
            u = self.w_in(x).float()                            # [T, width]
            state = unit.state["s"]                             # [slots + 1, width] float32
            cu, slots = ctx.cu_q.tolist(), ctx.seq_slot.tolist()
            s_all = torch.empty_like(u)
            for i, slot in enumerate(slots):                    # a stateful mixer walks each sequence in order
                s = state[slot].clone()
                for t in range(cu[i], cu[i + 1]):
                    s = self.decay * s + u[t]
                    s_all[t] = s
                if owns_cache:
                    state[slot] = s
            return self.w_out(s_all.to(x.dtype))

    class Top1Routed(FeedForward):
        """Router logits in float32, the best expert per token, y = softmax weight * W2_e relu(W1_e x)."""

        def __init__(self, params, runtime):
            super().__init__(params, runtime)
            self.hidden, self.inner, self.n = int(params["hidden"]), int(params["inner"]), int(params["experts"])

        def param_specs(self):
            specs = {"router.weight": ParamSpec((self.n, self.hidden))}
            for e in range(self.n):
                specs[f"experts.{e}.up.weight"] = ParamSpec((self.inner, self.hidden))
                specs[f"experts.{e}.down.weight"] = ParamSpec((self.hidden, self.inner))
            return specs

        def load(self, tensors):
            self.router = tensors["router.weight"].float()
            self.up = [Linear(tensors[f"experts.{e}.up.weight"]) for e in range(self.n)]
            self.down = [Linear(tensors[f"experts.{e}.down.weight"]) for e in range(self.n)]

        def forward(self, x, ctx):
            probs = torch.softmax(x.float() @ self.router.T, dim=-1)
            weight, expert = probs.max(dim=-1)
            out = torch.zeros_like(x)
            for e in range(self.n):
                rows = (expert == e).nonzero().flatten()
                if rows.numel():
                    y = self.down[e](torch.relu(self.up[e](x[rows].contiguous())))
                    out[rows] = (y.float() * weight[rows, None]).to(x.dtype)
            return out

    register_mixer("toy_decay", DecayMixer)
    register_feed_forward("toy_top1", Top1Routed)

    @dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        vocab: int
        layer_types: Tuple[str, ...]
        schedule: Tuple[Tuple[int, int], ...]      # (layer, cache_of or -1)
        width: int
        decay: float
        heads: int
        kv_heads: int
        head_dim: int
        window: int
        inner: int
        experts: int
        eps: float
        max_pos: int

        @staticmethod
        def from_dict(d):
            return ToyConfig(d["hidden"], d["vocab"], tuple(d["layer_types"]), tuple(tuple(s) for s in d["schedule"]),
                             d["width"], d["decay"], d["heads"], d["kv_heads"], d["head_dim"], d["window"], d["inner"],
                             d["experts"], d["eps"], d["max_pos"])

    def to_spec(c: ToyConfig) -> ModelSpec:
        norm = PartSpec("rmsnorm", {"size": c.hidden, "eps": c.eps})
        names = {"mixer": "mix", "feed_forward": "ff", "mixer_norm": "n1", "feed_forward_norm": "n2"}
        layers = []
        for i, kind in enumerate(c.layer_types):
            if kind == "recurrent":
                mixer = PartSpec("toy_decay", {"hidden": c.hidden, "width": c.width, "decay": c.decay})
            else:
                mixer = PartSpec("gqa_attention", {
                    "hidden": c.hidden, "n_heads": c.heads, "n_kv_heads": c.kv_heads, "head_dim": c.head_dim,
                    "window": c.window if kind == "window_attention" else 0, "scale": None,
                    "position": PartSpec("rope", {"rot_dim": c.head_dim // 2, "theta": 100.0, "scaling": None})})
            ff = PartSpec("toy_top1", {"hidden": c.hidden, "inner": c.inner, "experts": c.experts}) if i % 2 else \
                PartSpec("swiglu", {"hidden": c.hidden, "intermediate": c.inner})
            layers.append(LayerSpec("pre_norm", mixer, ff, norm, norm, names))
        return ModelSpec(hidden_size=c.hidden, vocab_size=c.vocab, max_position=c.max_pos, layers=layers,
                         schedule=[LayerCall(l, None if co < 0 else co) for l, co in c.schedule], final_norm=norm,
                         tie_head=True, embedding_name="emb.weight", layer_prefix="blocks.{i}.",
                         final_norm_name="final", head_name="head.weight")

    register_architecture("ToyForCausalLM", ToyConfig, to_spec)


TOY = {
    "architectures": ["ToyForCausalLM"], "hidden": 48, "vocab": 97,
    "layer_types": ["recurrent", "attention", "window_attention", "recurrent"],
    # layer 1 runs three times: entries 1 and 5 each own a cache unit, entry 3 READS entry 1's unit
    # (it computes queries only)
    "schedule": [[0, -1], [1, -1], [2, -1], [1, 1], [3, -1], [1, -1]],
    "width": 24, "decay": 0.9, "heads": 4, "kv_heads": 2, "head_dim": 16, "window": 20, "inner": 64, "experts": 3,
    "eps": 1e-5, "max_pos": 256,
}


# ------------------------------------------------------------------------------------------ plain restatement
def toy_plain_logits(w, cfg, tokens):
    T, d = len(tokens), cfg["hidden"]
    hd, H, Hkv = cfg["head_dim"], cfg["heads"], cfg["kv_heads"]
    rot = hd // 2
    inv = plain.inv_frequencies(rot, 100.0, None)
    cos, sin = plain.rotation_tables(torch.arange(T), inv)

    def rope(x):                                            # [heads, T, hd]; only the first rot elements turn
        return torch.cat([plain.rotate_half(x[..., :rot], cos, sin), x[..., rot:]], dim=-1)

    h = w["emb.weight"][torch.tensor(tokens)]
    kv_of_entry = {}
    for entry, (layer, cache_of) in enumerate(cfg["schedule"]):
        p = f"blocks.{layer}."
        kind = cfg["layer_types"][layer]
        x = plain.rms_norm(h, w[p + "n1.weight"], cfg["eps"])
        if kind == "recurrent":
            u = x @ w[p + "mix.in_proj.weight"].T
            s, rows = torch.zeros(cfg["width"]), []
            for t in range(T):
                s = cfg["decay"] * s + u[t]
                rows.append(s)
            mixed = torch.stack(rows) @ w[p + "mix.out_proj.weight"].T
        else:
            q = (x @ w[p + "mix.q_proj.weight"].T).view(T, H, hd).transpose(0, 1)
            q = rope(q)
            if cache_of < 0:
                k = rope((x @ w[p + "mix.k_proj.weight"].T).view(T, Hkv, hd).transpose(0, 1))
                v = (x @ w[p + "mix.v_proj.weight"].T).view(T, Hkv, hd).transpose(0, 1)
                kv_of_entry[entry] = (k, v)
            else:
                k, v = kv_of_entry[cache_of]
            k2, v2 = k.repeat_interleave(H // Hkv, 0), v.repeat_interleave(H // Hkv, 0)
            s = q @ k2.transpose(-1, -2) / math.sqrt(hd)
            i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
            mask = j > i
            if kind == "window_attention":
                mask = mask | (j < i - cfg["window"] + 1)
            s = s.masked_fill(mask, float("-inf"))
            mixed = (torch.softmax(s, -1) @ v2).transpose(0, 1).reshape(T, H * hd) @ w[p + "mix.o_proj.weight"].T
        h = h + mixed
        x = plain.rms_norm(h, w[p + "n2.weight"], cfg["eps"])
        if layer % 2:
            probs = torch.softmax(x @ w[p + "ff.router.weight"].T, -1)
            weight, expert = probs.max(-1)
            out = torch.zeros_like(x)
            for t in range(T):
                e = int(expert[t])
                out[t] = weight[t] * (torch.relu(x[t] @ w[p + f"ff.experts.{e}.up.weight"].T)
                                      @ w[p + f"ff.experts.{e}.down.weight"].T)
            h = h + out
        else:
            g = x @ w[p + "ff.gate_proj.weight"].T
            h = h + ((g * torch.sigmoid(g)) * (x @ w[p + "ff.up_proj.weight"].T)) @ w[p + "ff.down_proj.weight"].T
    return plain.rms_norm(h, w["final.weight"], cfg["eps"]) @ w["emb.weight"].T


@pytest.fixture(scope="module")
def toy_folder(tmp_path_factory):
    _register()
    from llm_infer_engine_b200 import write_random_model
    folder = str(tmp_path_factory.mktemp("toy"))
    write_random_model(TOY, folder, seed=11, std=0.15, norm_range=(0.7, 1.3))
    return folder


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 0.15)])
def test_toy_architecture_steps_like_its_plain_restatement(toy_folder, dtype, tol):
    from llm_infer_engine_b200 import Engine
    engine = Engine(toy_folder, dtype=dtype, max_batch=4, max_tokens=64 * 12, cuda_graph=False)
    model = engine.model
    # the run order is data: six entries over four layers, five cache units (entry 3 borrows entry 1's)
    assert len(model.blocks) == 4 and len(model.spec.schedule) == 6 and len(model.unit_requests) == 5
    assert model.unit_of_entry == [0, 1, 2, 1, 3, 4]
    # two groups of keys and values with storage of their own (all keys; a window), and state units
    kinds = sorted((r.n_kv_heads, r.head_dim, r.window) for r in engine.cache.groups())
    assert kinds == [(2, 16, 0), (2, 16, 20)]
    assert engine.cache.unit(0).kv is None and "s" in engine.cache.unit(0).state
    w = helpers.plain_weights(toy_folder)
    requests = {f"t{i}": helpers.random_tokens(TOY["vocab"], n, seed=40 + i) for i, n in enumerate([7, 30, 90, 150, 64])}
    want = {rid: toy_plain_logits(w, TOY, toks) for rid, toks in requests.items()}
    scale = max(float(v.abs().max()) for v in want.values())
    for plan in (helpers.plan_whole(requests), helpers.plan_tail(requests, 32), helpers.plan_batched(requests, 3)):
        got = helpers.run_plan_engine(engine, plan)
        for rid in requests:
            err = (got[rid] - want[rid]).abs().max(dim=1).values
            if dtype == "float32":
                assert float(err.max()) <= tol * max(1.0, scale), (rid, float(err.max()), scale)
            else:
                # in bfloat16 a token whose two best experts nearly tie may be routed the other way;
                # such tokens are few, and every other token must be close
                assert float((err <= tol * max(1.0, scale)).float().mean()) >= 0.95, (rid, err, scale)
    assert engine.cache.free_slots() == 4 and engine.cache.free_pages() == engine.cache.n_pages


def test_a_part_that_cannot_be_captured_falls_back_to_eager_steps(toy_folder, capsys):
    """The toy recurrent mixer reads lengths on the host in its forward, which no CUDA graph can record. An engine with
    captured steps switched on (the default) notices at its first capture, says so once, and goes on eagerly: the
    generated tokens are those of an engine that was eager from the start, and the cache is given back whole."""
    from llm_infer_engine_b200 import Engine, generate
    prompts = [helpers.random_tokens(TOY["vocab"], n, seed=90 + n) for n in (20, 5, 20)]
    eager = Engine(toy_folder, dtype="float32", max_batch=2, max_tokens=64 * 4, cuda_graph=False)
    want = generate(eager, prompts, max_new_tokens=6, stop_ids=[])
    engine = Engine(toy_folder, dtype="float32", max_batch=2, max_tokens=64 * 4, cuda_graph=True)
    got = generate(engine, prompts, max_new_tokens=6, stop_ids=[])
    assert got == want
    assert engine.use_cuda_graph is False
    assert "could not be captured" in capsys.readouterr().err
    # lone prompts of a repeating length would be captured too: they also simply run
    again = generate(engine, [prompts[0], prompts[0], prompts[0]], max_new_tokens=3, stop_ids=[])
    assert again[0] == again[1] == again[2] == want[0][:3]
    engine.cache.check()
    assert engine.cache.free_slots() == 2 and engine.cache.free_pages() == engine.cache.n_pages


def test_state_is_reset_when_a_slot_is_used_again(toy_folder):
    from llm_infer_engine_b200 import Engine
    engine = Engine(toy_folder, dtype="float32", max_batch=1, max_tokens=64 * 4, cuda_graph=False)
    w = helpers.plain_weights(toy_folder)
    for seed in (1, 2):                        # the single slot serves both requests, one after the other
        toks = helpers.random_tokens(TOY["vocab"], 40, seed=seed)
        slot = engine.open()
        assert slot == 0
        got = engine.step([slot], [toks], "all").cpu()
        engine.close(slot)
        assert float((got - toy_plain_logits(w, TOY, toks)).abs().max()) < 5e-5


# ------------------------------------------------------------------------------------------ other arrangements
# A second toy architecture for the edges of the part interfaces: a block with THREE norms (one of them on the
# mixer's output), a block with TWO mixers behind ONE shared norm whose three branches run in parallel (its
# cache unit holds keys and values for one mixer and a state for the other), another position encoding (pairs of
# neighbouring elements, written with plain tensor code including its cache write), learned absolute positions and a
# scale right after the embedding, and a cap on the logits after the head. All of it is defined here.
def _register_arrangements():
    from llm_infer_engine_b200.config import LayerCall, LayerSpec, ModelSpec, PartSpec, register_architecture
    from llm_infer_engine_b200.parts import (Block, ParamSpec, Pointwise, PositionEncoding, call_branch,
                                             register_block, register_pointwise, register_position_encoding)

    class SandwichBlock(Block):
        """h += post_norm(mixer(norm(h))); h += feed_forward(norm(h))."""
        ROLES = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "mixer_post_norm": "norm",
                 "feed_forward_norm": "norm"}

        def forward(self, h, pending, ctx, unit, owns_cache):
            x = self.mixer_norm.forward(h, pending)
            mixed = call_branch(self.mixer, x, ctx, unit, owns_cache)            # no residual: the output is normed first
            mixed = self.mixer_post_norm.forward(mixed.float().contiguous(), None)
            x = self.feed_forward_norm.forward(h, mixed)
            return h, call_branch(self.feed_forward, x, ctx, residual=h)

    class ParallelBlock(Block):
        """x = norm(h); h += attn(x) + rec(x) + feed_forward(x)."""
        ROLES = {"attn": "mixer", "rec": "mixer", "feed_forward": "feed_forward", "norm": "norm"}

        def forward(self, h, pending, ctx, unit, owns_cache):
            x = self.norm.forward(h, pending)
            a = call_branch(self.attn, x, ctx, unit.scoped("attn"), owns_cache)
            r = call_branch(self.rec, x, ctx, unit.scoped("rec"), owns_cache)
            f = call_branch(self.feed_forward, x, ctx)
            return h, (a.float() + r.float() + f.float()).to(x.dtype)

    class ScaleAndPositions(Pointwise):
        def __init__(self, params, runtime):
            super().__init__(params, runtime)
            self.scale, self.hidden, self.max_pos = float(params["scale"]), int(params["hidden"]), int(params["max_pos"])

        def param_specs(self):
            return {"positions.weight": ParamSpec((self.max_pos, self.hidden))}

        def load(self, tensors):
            self.table = tensors["positions.weight"].float()

        def forward(self, x, ctx, rows=None):
            return (x * self.scale + self.table[ctx.tok_pos.long()]).contiguous()

    class SoftCap(Pointwise):
        def forward(self, x, ctx, rows=None):
            cap = float(self.params["cap"])
            return cap * torch.tanh(x / cap)

    class InterleavedRotary(PositionEncoding):
        """Another position encoding: neighbouring elements (2i, 2i + 1) of a head are rotated as a pair (the
        library's own pairs element i with i + head_dim / 2), written with plain tensor code, the cache write
        included: the page of every token is looked up in the unit's block table."""

        def __init__(self, params, runtime):
            super().__init__(params, runtime)
            self.theta = float(params["theta"])

        def encode_and_store(self, qkv, ctx, kv, n_q, n_kv, head_dim, write_kv):
            T = qkv.shape[0]
            inv = 1.0 / (self.theta ** (torch.arange(0, head_dim, 2, device=qkv.device).float() / head_dim))
            angle = ctx.tok_pos.float()[:, None] * inv[None, :]                   # [T, hd / 2]
            cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]

            def turn(x):                                                           # [T, heads, hd]
                x = x.float()
                even, odd = x[..., 0::2], x[..., 1::2]
                return torch.stack([even * cos - odd * sin, odd * cos + even * sin], dim=-1).flatten(-2).to(qkv.dtype)

            q = turn(qkv[:, :n_q * head_dim].view(T, n_q, head_dim))
            if write_kv:
                k = turn(qkv[:, n_q * head_dim:(n_q + n_kv) * head_dim].view(T, n_kv, head_dim))
                v = qkv[:, (n_q + n_kv) * head_dim:].view(T, n_kv, head_dim)
                pos = ctx.tok_pos.long()
                slot = ctx.seq_slot.long()[ctx.tok_seq.long()]
                page = kv.block_table[slot, pos // kv.page_size].long()
                kv.k[page, :, pos % kv.page_size] = k
                kv.v[page, :, pos % kv.page_size] = v
            return q.reshape(T, n_q * head_dim).contiguous()

    register_position_encoding("toy_interleaved_rotary", InterleavedRotary)
    register_block("toy_sandwich", SandwichBlock)
    register_block("toy_parallel", ParallelBlock)
    register_pointwise("toy_scale_positions", ScaleAndPositions)
    register_pointwise("toy_softcap", SoftCap)

    @dataclass(frozen=True)
    class Config:
        d: dict

        @staticmethod
        def from_dict(d):
            return Config(dict(d))

    def to_spec(c) -> ModelSpec:
        c = c.d
        norm = PartSpec("rmsnorm", {"size": c["hidden"], "eps": c["eps"]})
        attn = PartSpec("gqa_attention", {
            "hidden": c["hidden"], "n_heads": c["heads"], "n_kv_heads": c["kv_heads"], "head_dim": c["head_dim"],
            "window": 0, "scale": None, "position": PartSpec("rope", {"rot_dim": c["head_dim"], "theta": 100.0,
                                                                     "scaling": None})})
        rec = PartSpec("toy_decay", {"hidden": c["hidden"], "width": c["width"], "decay": c["decay"]})
        ff = PartSpec("swiglu", {"hidden": c["hidden"], "intermediate": c["inner"]})
        attn2 = PartSpec("gqa_attention", dict(attn.params, position=PartSpec("toy_interleaved_rotary", {"theta": 50.0})))
        sandwich2 = LayerSpec("toy_sandwich", parts={"mixer": attn2, "feed_forward": ff, "mixer_norm": norm,
                                                      "mixer_post_norm": norm, "feed_forward_norm": norm},
                              names={"mixer": "mix", "feed_forward": "ff", "mixer_norm": "n1", "mixer_post_norm": "n1b",
                                     "feed_forward_norm": "n2"})
        sandwich = LayerSpec("toy_sandwich", parts={"mixer": attn, "feed_forward": ff, "mixer_norm": norm,
                                                     "mixer_post_norm": norm, "feed_forward_norm": norm},
                             names={"mixer": "mix", "feed_forward": "ff", "mixer_norm": "n1", "mixer_post_norm": "n1b",
                                    "feed_forward_norm": "n2"})
        parallel = LayerSpec("toy_parallel", parts={"attn": attn, "rec": rec, "feed_forward": ff, "norm": norm},
                             names={"attn": "attn", "rec": "rec", "feed_forward": "ff", "norm": "n"})
        return ModelSpec(hidden_size=c["hidden"], vocab_size=c["vocab"], max_position=c["max_pos"],
                         layers=[sandwich, parallel, sandwich2], schedule=[LayerCall(0), LayerCall(1), LayerCall(2)],
                         final_norm=norm, tie_head=False, embedding_name="emb.weight", layer_prefix="blocks.{i}.",
                         final_norm_name="final", head_name="head.weight",
                         after_embedding=PartSpec("toy_scale_positions", {"scale": c["emb_scale"], "hidden": c["hidden"],
                                                                          "max_pos": c["max_pos"]}),
                         after_head=PartSpec("toy_softcap", {"cap": c["cap"]}), after_embedding_name="pre")

    register_architecture("ToyArrangementsForCausalLM", Config, to_spec)


ARR = {"architectures": ["ToyArrangementsForCausalLM"], "hidden": 40, "vocab": 61, "heads": 2, "kv_heads": 1,
       "head_dim": 32, "width": 12, "decay": 0.8, "inner": 56, "eps": 1e-5, "max_pos": 200, "emb_scale": 3.0, "cap": 2.0}


def arrangements_plain_logits(w, cfg, tokens):
    T, hd, H, Hkv = len(tokens), cfg["head_dim"], cfg["heads"], cfg["kv_heads"]
    cos, sin = plain.rotation_tables(torch.arange(T), plain.inv_frequencies(hd, 100.0, None))
    norm = lambda x, name: plain.rms_norm(x, w[name + ".weight"], cfg["eps"])

    inv2 = 1.0 / (50.0 ** (torch.arange(0, hd, 2).float() / hd))
    cos2, sin2 = torch.cos(torch.arange(T).float()[:, None] * inv2), torch.sin(torch.arange(T).float()[:, None] * inv2)

    def pairs(x):                                           # [heads, T, hd]: elements (2i, 2i + 1) turn together
        even, odd = x[..., 0::2], x[..., 1::2]
        return torch.stack([even * cos2 - odd * sin2, odd * cos2 + even * sin2], dim=-1).flatten(-2)

    def attention(x, p, turn=None):
        turn = turn or (lambda t: plain.rotate_half(t, cos, sin))
        q = turn((x @ w[p + "q_proj.weight"].T).view(T, H, hd).transpose(0, 1))
        k = turn((x @ w[p + "k_proj.weight"].T).view(T, Hkv, hd).transpose(0, 1))
        v = (x @ w[p + "v_proj.weight"].T).view(T, Hkv, hd).transpose(0, 1)
        return plain.causal_gqa_attention(q, k, v).transpose(0, 1).reshape(T, H * hd) @ w[p + "o_proj.weight"].T

    def recurrent(x, p):
        u = x @ w[p + "in_proj.weight"].T
        s, rows = torch.zeros(cfg["width"]), []
        for t in range(T):
            s = cfg["decay"] * s + u[t]
            rows.append(s)
        return torch.stack(rows) @ w[p + "out_proj.weight"].T

    def swiglu(x, p):
        g = x @ w[p + "gate_proj.weight"].T
        return ((g * torch.sigmoid(g)) * (x @ w[p + "up_proj.weight"].T)) @ w[p + "down_proj.weight"].T

    h = w["emb.weight"][torch.tensor(tokens)] * cfg["emb_scale"] + w["pre.positions.weight"][:T]
    for layer in (0, 1, 2):
        p = f"blocks.{layer}."
        if layer == 1:
            x = norm(h, p + "n")
            h = h + attention(x, p + "attn.") + recurrent(x, p + "rec.") + swiglu(x, p + "ff.")
        else:
            h = h + norm(attention(norm(h, p + "n1"), p + "mix.", pairs if layer == 2 else None), p + "n1b")
            h = h + swiglu(norm(h, p + "n2"), p + "ff.")
    logits = norm(h, "final") @ w["head.weight"].T
    return cfg["cap"] * torch.tanh(logits / cfg["cap"])


@pytest.mark.parametrize("dtype,tol", [("float32", 5e-5), ("bfloat16", 0.05)])
def test_other_arrangements_need_only_additions(tmp_path_factory, dtype, tol):
    """Three norms in a block, two mixers and one shared norm in another, parts outside the layers: built from
    registrations made in this file, stepped whole, one by one and in batches, like its plain restatement."""
    _register()
    _register_arrangements()
    from llm_infer_engine_b200 import Engine, write_random_model
    folder = str(tmp_path_factory.mktemp("arrangements"))
    write_random_model(ARR, folder, seed=5, std=0.2, norm_range=(0.7, 1.3))
    engine = Engine(folder, dtype=dtype, max_batch=3, max_tokens=64 * 9, cuda_graph=False)
    # the parallel layer's unit holds keys and values for one mixer and a state for the other, under the roles' names
    unit = engine.cache.unit(1)
    assert sorted(unit.kvs) == ["attn.kv"] and sorted(unit.state) == ["rec.s"]
    assert unit.scoped("rec").state["s"].shape[-1] == ARR["width"] and unit.scoped("attn").kv is not None
    assert sorted(engine.model.blocks[0].parts()) == ["feed_forward", "feed_forward_norm", "mixer", "mixer_norm",
                                                      "mixer_post_norm"]
    w = helpers.plain_weights(folder)
    assert "blocks.0.n1b.weight" in w and "pre.positions.weight" in w and "blocks.1.rec.in_proj.weight" in w
    requests = {f"a{i}": helpers.random_tokens(ARR["vocab"], n, seed=70 + i) for i, n in enumerate([9, 70, 130, 64])}
    want = {rid: arrangements_plain_logits(w, ARR, toks) for rid, toks in requests.items()}
    for plan in (helpers.plan_whole(requests), helpers.plan_tail(requests, 32), helpers.plan_batched(requests, 3),
                 helpers.plan_chunked(requests, 50)):
        got = helpers.run_plan_engine(engine, plan)
        for rid in requests:
            err = float((got[rid] - want[rid]).abs().max())
            assert err <= tol * max(1.0, float(want[rid].abs().max())), (rid, err)
    assert engine.cache.free_slots() == 3 and engine.cache.free_pages() == engine.cache.n_pages
