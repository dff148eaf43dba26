"""Each built-in part alone, built through its registry with sizes of its own and driven with a hand-made step
context and cache unit, against the plain function of the same formula: norm, position encoding, feed-forward,
attention mixer (prompts of unequal lengths, then one token each, eagerly like the engine does), and the
pre-norm block. float32 and bfloat16."""
import types

import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def runtime(dtype, max_positions=512):
    from llm_infer_engine_b200.parts import Runtime
    return Runtime(device=torch.device(DEV), dtype=DTYPES[dtype], max_positions=max_positions)


def build(group, kind, params, dtype, tensors=None, seed=0, std=0.1):
    """A part from its registry with random tensors of its own declaration (rounded to bfloat16, kept in the
    engine's precision as the loader would); returns (part, float32 copies by local name)."""
    from llm_infer_engine_b200.config import PartSpec
    from llm_infer_engine_b200.parts import build_part
    part = build_part(group, PartSpec(kind, params), runtime(dtype))
    g = torch.Generator().manual_seed(seed)
    host = {}
    for name, ps in part.param_specs().items():
        t = torch.rand(ps.shape, generator=g) + 0.5 if ps.role == "vector" else torch.randn(ps.shape, generator=g) * std
        host[name] = t.to(torch.bfloat16).float()
    part.load({n: t.to(DEV, DTYPES[dtype]) for n, t in host.items()})
    return part, host


def tol(dtype, scale):
    return (2e-5 if dtype == "float32" else 2e-2) * max(1.0, scale)


def make_ctx(lens, starts, slots, dtype, kernels=None):
    from llm_infer_engine_b200.engine.context import StepContext
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    T, n = sum(lens), len(lens)
    cu = [0]
    for l in lens:
        cu.append(cu[-1] + l)
    tok_pos = [s + j for s, l in zip(starts, lens) for j in range(l)]
    tok_seq = [i for i, l in enumerate(lens) for _ in range(l)]
    return StepContext(n_tokens=T, n_seqs=n, decode=max(lens) == 1, max_q_len=max(lens),
                       max_kv_len=max(s + l for s, l in zip(starts, lens)), tokens=i32([0] * T), tok_pos=i32(tok_pos),
                       tok_seq=i32(tok_seq), cu_q=i32(cu), seq_slot=i32(slots), seq_start=i32(starts),
                       seq_kvlen=i32([s + l for s, l in zip(starts, lens)]), logit_rows=i32(list(range(T))),
                       dtype=DTYPES[dtype], device=torch.device(DEV), kernels=kernels, all_rows=True)


def kernel_plan(dtype):
    from llm_infer_engine_b200.engine.plan import KernelPlan
    return KernelPlan(types.SimpleNamespace(dtype=DTYPES[dtype], decode_attention="auto"))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_part(dtype):
    norm, w = build("norm", "rmsnorm", {"size": 136, "eps": 3e-6}, dtype, seed=1)
    g = torch.Generator().manual_seed(2)
    h = torch.randn(11, 136, generator=g) * 3
    delta = (torch.randn(11, 136, generator=g)).to(DTYPES[dtype])
    hd_ = h.clone().to(DEV)
    x = norm.forward(hd_, delta.to(DEV))
    want_h = h + delta.float()
    assert torch.allclose(hd_.cpu(), want_h, atol=1e-6)                       # the residual stream is float32 in both
    want = plain.rms_norm(want_h, w["weight"], 3e-6)
    assert x.dtype == DTYPES[dtype]
    assert float((x.float().cpu() - want).abs().max()) <= tol(dtype, float(want.abs().max()))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    some = norm.forward(hd_, None, rows=rows)                                  # only the wanted rows, h untouched
    assert float((some.float().cpu() - want[[7, 0, 3]]).abs().max()) <= tol(dtype, float(want.abs().max()))
    assert torch.allclose(hd_.cpu(), want_h, atol=1e-6)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rot,hd,scaling", [(48, 48, None), (16, 32, None),
                                            (64, 64, {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0,
                                                      "high_freq_factor": 4.0, "original_max_position_embeddings": 64})])
def test_position_encoding_part(dtype, rot, hd, scaling):
    from llm_infer_engine_b200.cache import Cache, KVRequest
    n_q, n_kv = 4, 2
    rope, _ = build("position_encoding", "rope", {"rot_dim": rot, "theta": 30000.0, "scaling": scaling}, dtype)
    cache = Cache([[KVRequest(n_kv, hd)]], 3, 64 * 6, 512, DTYPES[dtype], DEV)
    slots = [cache.take_slot() for _ in range(2)]
    lens, starts = [70, 3], [0, 0]
    for s, l in zip(slots, lens):
        cache.reserve(s, l)
    ctx = make_ctx(lens, starts, slots, dtype)
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(sum(lens), (n_q + 2 * n_kv) * hd, generator=g).to(DTYPES[dtype])
    kv = cache.unit(0).kv
    q = rope.encode_and_store(qkv.to(DEV), ctx, kv, n_q, n_kv, hd, True).float().cpu()
    inv = plain.inv_frequencies(rot, 30000.0, scaling)
    row = 0
    for i, l in enumerate(lens):
        cos, sin = plain.rotation_tables(torch.arange(l), inv)
        x = qkv[row:row + l].float()
        turn = lambda t: torch.cat([plain.rotate_half(t[..., :rot], cos, sin), t[..., rot:]], dim=-1)   # [heads, T, hd]
        q_want = turn(x[:, :n_q * hd].view(l, n_q, hd).transpose(0, 1)).transpose(0, 1).reshape(l, -1)
        k_want = turn(x[:, n_q * hd:(n_q + n_kv) * hd].view(l, n_kv, hd).transpose(0, 1))
        v_want = x[:, (n_q + n_kv) * hd:].view(l, n_kv, hd).transpose(0, 1)
        assert float((q[row:row + l] - q_want).abs().max()) <= tol(dtype, 4.0)
        table = kv.block_table[slots[i]].cpu()
        for pos in (0, l // 2, l - 1):
            page = int(table[pos // 64])
            assert float((kv.k[page, :, pos % 64].float().cpu() - k_want[:, pos]).abs().max()) <= tol(dtype, 4.0)
            assert float((kv.v[page, :, pos % 64].float().cpu() - v_want[:, pos]).abs().max()) <= tol(dtype, 4.0)
        row += l


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("rows", [3, 12, 70])
def test_feed_forward_part(dtype, rows):
    """3 rows take the one-kernel forms of the bfloat16 engine, 12 the add-into product, 70 the library product."""
    ff, w = build("feed_forward", "swiglu", {"hidden": 96, "intermediate": 200}, dtype, seed=4)
    g = torch.Generator().manual_seed(5)
    x = torch.randn(rows, 96, generator=g).to(DTYPES[dtype])
    want = plain.swiglu_mlp(x.float(), {"mlp." + k: v for k, v in w.items()}, "")
    ctx = make_ctx([rows], [0], [0], dtype)
    y = ff.forward(x.to(DEV), ctx)
    assert float((y.float().cpu() - want).abs().max()) <= tol(dtype, float(want.abs().max()))
    h = torch.randn(rows, 96, generator=g)
    hd_ = h.clone().to(DEV)
    out = ff.forward(x.to(DEV), ctx, residual=hd_)                              # may add into the residual stream itself
    total = hd_.cpu() if out is None else h + out.float().cpu()
    assert float((total - (h + want)).abs().max()) <= tol(dtype, float(want.abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n_q,n_kv,hd,window", [(4, 2, 32, 0), (6, 2, 64, 0), (3, 1, 48, 40)])
def test_attention_mixer_part(dtype, n_q, n_kv, hd, window):
    """Prompts of 5, 70 and 130 tokens in one step, then three steps of one token each, through the part's own
    forward with a cache of its own request; every output row against plain attention over the whole sequence."""
    from llm_infer_engine_b200.cache import Cache
    from llm_infer_engine_b200.config import PartSpec
    hidden = 80
    params = {"hidden": hidden, "n_heads": n_q, "n_kv_heads": n_kv, "head_dim": hd, "window": window, "scale": None,
              "position": PartSpec("rope", {"rot_dim": hd, "theta": 10000.0, "scaling": None})}
    mixer, w = build("mixer", "gqa_attention", params, dtype, seed=6, std=0.15)
    cache = Cache([mixer.cache_requests()], 4, 64 * 12, 512, DTYPES[dtype], DEV)
    unit = cache.unit(0)
    plan = kernel_plan(dtype)
    lens, extra = [5, 70, 130], 3
    g = torch.Generator().manual_seed(7)
    xs = [torch.randn(l + extra, hidden, generator=g).to(DTYPES[dtype]) for l in lens]
    cfg = {"num_attention_heads": n_q, "num_key_value_heads": n_kv, "head_dim": hd, "hidden_size": hidden}
    pw = {"self_attn." + k: v for k, v in w.items()}
    inv = plain.inv_frequencies(hd, 10000.0, None)
    want = []
    for x in xs:
        cos, sin = plain.rotation_tables(torch.arange(x.shape[0]), inv)
        if window:
            # plain attention with a window: restated here, the library's plain function has none
            T = x.shape[0]
            xf = x.float()
            q = plain.rotate_half((xf @ pw["self_attn.q_proj.weight"].T).view(T, n_q, hd).transpose(0, 1), cos, sin)
            k = plain.rotate_half((xf @ pw["self_attn.k_proj.weight"].T).view(T, n_kv, hd).transpose(0, 1), cos, sin)
            v = (xf @ pw["self_attn.v_proj.weight"].T).view(T, n_kv, hd).transpose(0, 1)
            k, v = k.repeat_interleave(n_q // n_kv, 0), v.repeat_interleave(n_q // n_kv, 0)
            s = q @ k.transpose(-1, -2) / hd ** 0.5
            i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
            s = s.masked_fill((j > i) | (j < i - window + 1), float("-inf"))
            want.append((torch.softmax(s, -1) @ v).transpose(0, 1).reshape(T, n_q * hd) @ pw["self_attn.o_proj.weight"].T)
        else:
            want.append(plain.attention_layer(x.float(), pw, "", cfg, cos, sin))
    slots = [cache.take_slot() for _ in lens]
    bound = tol(dtype, max(float(t.abs().max()) for t in want))

    def step(step_lens, starts, rows_of):
        for s, st, l in zip(slots, starts, step_lens):
            cache.reserve(s, st + l)
        ctx = make_ctx(step_lens, starts, slots, dtype, plan)
        x = torch.cat([xs[i][st:st + l] for i, (st, l) in enumerate(zip(starts, step_lens))]).to(DEV)
        y = mixer.forward(x, ctx, unit, True).float().cpu()
        row = 0
        for i, (st, l) in enumerate(zip(starts, step_lens)):
            err = float((y[row:row + l] - want[i][st:st + l]).abs().max())
            assert err <= bound, (rows_of, i, st, err, bound)
            row += l
            cache.note_appended(slots[i], st + l, device_updated=False)

    step(lens, [0, 0, 0], "prompts")
    for t in range(extra):
        step([1, 1, 1], [l + t for l in lens], f"token {t}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_pre_norm_block(dtype):
    """The arrangement alone: two blocks in a row (so that the branch output travelling as `pending` is added by the
    next block's norm), prompts of unequal lengths, against the plain block."""
    from llm_infer_engine_b200.cache import Cache
    from llm_infer_engine_b200.config import PartSpec
    from llm_infer_engine_b200.parts import lookup
    hidden, n_q, n_kv, hd, inter = 64, 4, 2, 16, 112
    cfg = {"num_attention_heads": n_q, "num_key_value_heads": n_kv, "head_dim": hd, "hidden_size": hidden,
           "rms_norm_eps": 1e-5}
    specs = {"mixer": ("mixer", "gqa_attention", {"hidden": hidden, "n_heads": n_q, "n_kv_heads": n_kv, "head_dim": hd,
                                                  "window": 0, "scale": None,
                                                  "position": PartSpec("rope", {"rot_dim": hd, "theta": 10000.0, "scaling": None})}),
             "feed_forward": ("feed_forward", "swiglu", {"hidden": hidden, "intermediate": inter}),
             "mixer_norm": ("norm", "rmsnorm", {"size": hidden, "eps": 1e-5}),
             "feed_forward_norm": ("norm", "rmsnorm", {"size": hidden, "eps": 1e-5})}
    names = {"mixer": "self_attn.", "feed_forward": "mlp.", "mixer_norm": "input_layernorm.",
             "feed_forward_norm": "post_attention_layernorm."}
    blocks, pw = [], {}
    for layer in range(2):
        parts = {}
        for role, (group, kind, params) in specs.items():
            parts[role], w = build(group, kind, params, dtype, seed=10 * layer + len(role), std=0.12)
            pw.update({f"model.layers.{layer}.{names[role]}{k}": v for k, v in w.items()})
        blocks.append(lookup("block", "pre_norm")(parts, runtime(dtype)))
    cache = Cache([b.cache_requests() for b in blocks], 3, 64 * 6, 512, DTYPES[dtype], DEV)
    lens = [33, 70]
    slots = [cache.take_slot() for _ in lens]
    for s, l in zip(slots, lens):
        cache.reserve(s, l)
    ctx = make_ctx(lens, [0, 0], slots, dtype, kernel_plan(dtype))
    g = torch.Generator().manual_seed(11)
    hs = [torch.randn(l, hidden, generator=g) for l in lens]
    h = torch.cat(hs).to(DEV)
    pending = None
    for i, b in enumerate(blocks):
        h, pending = b.forward(h, pending, ctx, cache.unit(i), True)
    got = h.cpu() + (pending.float().cpu() if pending is not None else 0)
    inv = plain.inv_frequencies(hd, 10000.0, None)
    row = 0
    for l, h0 in zip(lens, hs):
        cos, sin = plain.rotation_tables(torch.arange(l), inv)
        ref = plain.block(plain.block(h0, pw, 0, cfg, cos, sin), pw, 1, cfg, cos, sin)
        err = float((got[row:row + l] - ref).abs().max())
        assert err <= tol(dtype, float(ref.abs().max())), (l, err)
        row += l
