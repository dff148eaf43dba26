"""Each CUDA kernel alone against a plain float32 torch restatement of the same op, at sizes
other than the engine's tiny models (widths that are no power of two, odd head counts, several
head sizes, pages in scrambled order)."""
import math

import pytest
import torch

import plain_llama as plain

pytestmark = pytest.mark.gpu

DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, f32=1e-5, bf16=2e-2):
    return f32 if dtype == torch.float32 else bf16


def ops():
    from llm_infer_engine_b200.kernels import ops as o
    return o


# ------------------------------------------------------------------------------------------ elementwise
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,vocab", [(96, 301), (2048, 1000), (40, 17)])
def test_embedding(dtype, d, vocab):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, d, generator=g).to(dtype).to(DEV)
    tokens = torch.randint(0, vocab, (37,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(37, d, dtype=torch.float32, device=DEV)
    ops().embedding(tokens, table, out)
    assert torch.equal(out.cpu(), table.float().cpu()[tokens.cpu().long()])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [64, 96, 1000, 2048, 5120])
def test_add_rmsnorm(dtype, d):
    g = torch.Generator().manual_seed(1)
    T, eps = 19, 3e-6
    h = torch.randn(T, d, generator=g) * 3
    delta = torch.randn(T, d, generator=g).to(dtype)
    w = torch.rand(d, generator=g) + 0.5
    h_dev = h.clone().to(DEV)
    out = torch.empty(T, d, dtype=dtype, device=DEV)
    ops().add_rmsnorm(h_dev, delta.to(DEV), w.to(DEV), eps, out)
    h_ref = h + delta.float()
    y_ref = plain.rms_norm(h_ref, w, eps)
    assert torch.allclose(h_dev.cpu(), h_ref, atol=1e-6, rtol=1e-6)           # the sum is float32
    assert torch.allclose(out.float().cpu(), y_ref, atol=tol(dtype, 2e-6, 3e-2), rtol=tol(dtype, 2e-6, 1e-2))
    # no delta
    h2 = h.clone().to(DEV)
    ops().add_rmsnorm(h2, None, w.to(DEV), eps, out)
    assert torch.equal(h2.cpu(), h)
    assert torch.allclose(out.float().cpu(), plain.rms_norm(h, w, eps), atol=tol(dtype, 2e-6, 3e-2), rtol=1e-2)
    # gathered rows: h is left alone
    rows = torch.tensor([18, 0, 7], dtype=torch.int32, device=DEV)
    h3 = h.clone().to(DEV)
    out3 = torch.empty(3, d, dtype=dtype, device=DEV)
    ops().add_rmsnorm(h3, delta.to(DEV), w.to(DEV), eps, out3, rows)
    assert torch.equal(h3.cpu(), h)
    assert torch.allclose(out3.float().cpu(), y_ref[[18, 0, 7]], atol=tol(dtype, 2e-6, 3e-2), rtol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [8, 264, 2048, 3080, 4096])
def test_add_rmsnorm_many_rows(dtype, d):
    """A prompt's worth of rows (more blocks than the GPU holds at once), one row far from the others' scale,
    also with gathered rows."""
    g = torch.Generator().manual_seed(2)
    T, eps = 1030, 1e-5
    h = torch.randn(T, d, generator=g) * 2
    h[5] *= 40.0                                                # one row far from the others' scale
    delta = torch.randn(T, d, generator=g).to(dtype)
    w = torch.rand(d, generator=g) + 0.5
    h_dev = h.clone().to(DEV)
    out = torch.empty(T, d, dtype=dtype, device=DEV)
    ops().add_rmsnorm(h_dev, delta.to(DEV), w.to(DEV), eps, out)
    h_ref = h + delta.float()
    y_ref = plain.rms_norm(h_ref, w, eps)
    assert torch.allclose(h_dev.cpu(), h_ref, atol=1e-6, rtol=1e-6)
    assert torch.allclose(out.float().cpu(), y_ref, atol=tol(dtype, 3e-6, 3e-2), rtol=tol(dtype, 3e-6, 1e-2))
    h2 = h.clone().to(DEV)
    ops().add_rmsnorm(h2, None, w.to(DEV), eps, out)
    assert torch.equal(h2.cpu(), h)
    assert torch.allclose(out.float().cpu(), plain.rms_norm(h, w, eps), atol=tol(dtype, 3e-6, 3e-2), rtol=1e-2)
    rows = torch.randperm(T, generator=g)[:1024].to(torch.int32)
    h3 = h.clone().to(DEV)
    out3 = torch.empty(1024, d, dtype=dtype, device=DEV)
    ops().add_rmsnorm(h3, delta.to(DEV), w.to(DEV), eps, out3, rows.to(DEV))
    assert torch.equal(h3.cpu(), h)
    assert torch.allclose(out3.float().cpu(), y_ref[rows.long()], atol=tol(dtype, 3e-6, 3e-2), rtol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("ff", [192, 250, 8192])
def test_swiglu(dtype, ff):
    g = torch.Generator().manual_seed(2)
    gu = (torch.randn(11, 2 * ff, generator=g) * 2).to(dtype)
    out = torch.empty(11, ff, dtype=dtype, device=DEV)
    ops().swiglu(gu.to(DEV), out)
    gate, up = gu.float()[:, :ff], gu.float()[:, ff:]
    ref = gate * torch.sigmoid(gate) * up
    assert torch.allclose(out.float().cpu(), ref, atol=tol(dtype, 1e-6, 2e-2), rtol=tol(dtype, 1e-5, 1e-2))


@pytest.mark.parametrize("M,N,K", [(1, 300, 96), (5, 64, 50), (17, 129, 200), (70, 384, 96), (200, 2048, 513)])
def test_gemm_f32(M, N, K):
    g = torch.Generator().manual_seed(3)
    a, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    out = ops().gemm_f32_nt(a.to(DEV), w.to(DEV)).cpu()
    ref = (a.double() @ w.double().T).float()
    assert torch.allclose(out, ref, atol=1e-4, rtol=1e-5)
    # a row's result does not depend on the other rows of the launch
    one = ops().gemm_f32_nt(a[M // 2:M // 2 + 1].contiguous().to(DEV), w.to(DEV)).cpu()
    assert torch.equal(one[0], out[M // 2])


# ------------------------------------------------------------------------------------------ paged cache helpers
class Paged:
    """Dense per-sequence K/V laid into scrambled pages, with the index arrays the kernels want."""

    def __init__(self, seq_lens, n_kv, hd, dtype, page_size=64, seed=0, extra_slots=3):
        g = torch.Generator().manual_seed(seed)
        self.page_size, self.n_kv, self.hd = page_size, n_kv, hd
        n = len(seq_lens)
        n_slots = n + extra_slots
        pages_per = [(l + page_size - 1) // page_size for l in seq_lens]
        max_pages = max(pages_per) + 1
        n_pages = sum(pages_per) + 5
        perm = torch.randperm(n_pages, generator=g).tolist()
        self.slots = torch.randperm(n_slots, generator=g)[:n].tolist()
        self.block_table = torch.full((n_slots, max_pages), n_pages - 1, dtype=torch.int32)
        nxt = 0
        for i, s in enumerate(self.slots):
            for p in range(pages_per[i]):
                self.block_table[s, p] = perm[nxt]
                nxt += 1
        self.k = torch.zeros(n_pages, n_kv, page_size, hd, dtype=dtype)
        self.v = torch.zeros(n_pages, n_kv, page_size, hd, dtype=dtype)
        self.dense_k = [torch.randn(l, n_kv, hd, generator=g).to(dtype) for l in seq_lens]
        self.dense_v = [torch.randn(l, n_kv, hd, generator=g).to(dtype) for l in seq_lens]

    def fill(self, upto=None):
        """Writes the dense tensors into their pages (positions < upto[i] if given)."""
        for i, s in enumerate(self.slots):
            L = self.dense_k[i].shape[0] if upto is None else upto[i]
            for pos in range(L):
                page = int(self.block_table[s, pos // self.page_size])
                self.k[page, :, pos % self.page_size] = self.dense_k[i][pos]
                self.v[page, :, pos % self.page_size] = self.dense_v[i][pos]

    def dev(self):
        return self.k.to(DEV), self.v.to(DEV), self.block_table.to(DEV)


def ref_attention(q, k, v, positions, scale, window):
    """q [T, Hq, hd] at absolute `positions`; k, v [L, Hkv, hd] float32; plain softmax attention."""
    Hq, Hkv = q.shape[1], k.shape[1]
    out = torch.zeros_like(q)
    for t, p in enumerate(positions):
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(Hq):
            kk, vv = k[lo:p + 1, h // (Hq // Hkv)], v[lo:p + 1, h // (Hq // Hkv)]
            s = (kk @ q[t, h]) * scale
            out[t, h] = torch.softmax(s, dim=0) @ vv
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,hd", [(4, 2, 16), (3, 1, 32), (6, 2, 48), (8, 8, 64), (5, 5, 80), (4, 1, 128)])
def test_rope_store_and_paged_attention(dtype, n_q, n_kv, hd):
    """Ragged prefill at nonzero start positions: rotate + cache write, then plain attention."""
    o = ops()
    starts, news = [0, 70, 3], [50, 9, 130]
    totals = [s + n for s, n in zip(starts, news)]
    pg = Paged(totals, n_kv, hd, dtype, seed=hd)
    pg.fill(upto=starts)              # what earlier steps left; this step's keys come from rope_store
    theta, rot = 10000.0, hd
    inv = plain.inv_frequencies(rot, theta, None)
    max_pos = 256
    cos, sin = plain.rotation_tables(torch.arange(max_pos), inv)
    table = torch.stack([cos, sin], dim=-1).contiguous()
    T = sum(news)
    g = torch.Generator().manual_seed(5)
    qkv = torch.randn(T, (n_q + 2 * n_kv) * hd, generator=g).to(dtype)
    tok_seq = torch.repeat_interleave(torch.arange(3), torch.tensor(news)).int()
    tok_pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, news)]).int()
    k_dev, v_dev, bt = pg.dev()
    q_out = torch.empty(T, n_q * hd, dtype=dtype, device=DEV)
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    o.rope_store(qkv.to(DEV), q_out, k_dev, v_dev, table.to(DEV), tok_pos.to(DEV), tok_seq.to(DEV), slots, bt, 64,
                 n_q, n_kv, hd, rot)
    # reference rotation in float32
    qf = qkv.float()[:, :n_q * hd].view(T, n_q, hd)
    kf = qkv.float()[:, n_q * hd:(n_q + n_kv) * hd].view(T, n_kv, hd)
    vf = qkv.float()[:, (n_q + n_kv) * hd:].view(T, n_kv, hd)
    c, s = cos[tok_pos.long()][:, None, :], sin[tok_pos.long()][:, None, :]
    rot_q = plain.rotate_half(qf, c, s)
    rot_k = plain.rotate_half(kf, c, s)
    assert torch.allclose(q_out.float().cpu().view(T, n_q, hd), rot_q, atol=tol(dtype, 1e-6, 3e-2))
    k_host, v_host = k_dev.cpu(), v_dev.cpu()
    off = 0
    for i, (st, n) in enumerate(zip(starts, news)):
        for j in range(n):
            pos = st + j
            page = int(pg.block_table[pg.slots[i], pos // 64])
            assert torch.allclose(k_host[page, :, pos % 64].float(), rot_k[off + j], atol=tol(dtype, 1e-6, 3e-2))
            assert torch.equal(v_host[page, :, pos % 64].float(), vf[off + j].to(dtype).float())
            # pages hold exactly what the dense history holds from here on
            pg.dense_k[i][pos] = k_host[page, :, pos % 64]
            pg.dense_v[i][pos] = v_host[page, :, pos % 64]
        off += n
    # attention over the cache, with and without a window
    for window in (0, 40):
        out = torch.empty(T, n_q * hd, dtype=dtype, device=DEV)
        o.attention_paged(q_out, k_dev, v_dev, out, tok_pos.to(DEV), tok_seq.to(DEV), slots, bt, 64, n_q, n_kv, hd,
                          hd ** -0.5, window)
        off = 0
        for i, n in enumerate(news):
            ref = ref_attention(q_out.float().cpu().view(T, n_q, hd)[off:off + n], pg.dense_k[i].float(),
                                pg.dense_v[i].float(), tok_pos[off:off + n].tolist(), hd ** -0.5, window)
            got = out.float().cpu().view(T, n_q, hd)[off:off + n]
            assert torch.allclose(got, ref, atol=tol(dtype, 2e-5, 2e-2)), (window, i, float((got - ref).abs().max()))
            off += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,hd", [(4, 2, 16), (3, 1, 32), (32, 8, 64), (24, 8, 128), (12, 2, 64), (16, 1, 64)])
@pytest.mark.parametrize("run_len", [64])
def test_attention_decode(dtype, n_q, n_kv, hd, run_len):
    """Split-KV decode against the plain formula: unequal lengths from 1 to several runs, a
    window, and a far key made to stand out so that a lost run or page cannot hide."""
    o = ops()
    assert o.attention_decode_supported(hd, dtype)
    lens = [1, 63, 64, 65, 300, 777, 1024]
    pg = Paged(lens, n_kv, hd, dtype, seed=7 + hd)
    g = torch.Generator().manual_seed(11)
    q = torch.randn(len(lens), n_q, hd, generator=g)
    # needle: in the longest sequences one early key matches the query strongly
    for i, L in enumerate(lens):
        if L >= 300:
            needle = 3 + i
            qh = q[i, ::(n_q // n_kv)]                                           # first query head of each group
            gain = 24.0 / ((qh * qh).sum(-1, keepdim=True) * hd ** -0.5)          # its score becomes 24
            pg.dense_k[i][needle, :, :] = (qh * gain).to(dtype)
            pg.dense_v[i][needle, :, :] = 5.0
    pg.fill()
    k_dev, v_dev, bt = pg.dev()
    qd = q.to(dtype).reshape(len(lens), n_q * hd).to(DEV)
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    kvlen = torch.tensor(lens, dtype=torch.int32, device=DEV)
    max_len = 1100
    n_runs = (max_len + run_len - 1) // run_len
    for window in (0, 100):
        out = torch.full((len(lens), n_q * hd), float("nan"), dtype=dtype, device=DEV)
        o.attention_decode(qd, k_dev, v_dev, out, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, window, run_len,
                           n_runs)
        plain_out = torch.empty_like(out)
        tok_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
        tok_seq = torch.arange(len(lens), dtype=torch.int32, device=DEV)
        o.attention_paged(qd, k_dev, v_dev, plain_out, tok_pos, tok_seq, slots, bt, 64, n_q, n_kv, hd, hd ** -0.5, window)
        for i, L in enumerate(lens):
            ref = ref_attention(qd.float().cpu().view(len(lens), n_q, hd)[i:i + 1], pg.dense_k[i].float(),
                                pg.dense_v[i].float(), [L - 1], hd ** -0.5, window)[0]
            got = out.float().cpu().view(len(lens), n_q, hd)[i]
            assert torch.allclose(got, ref, atol=tol(dtype, 2e-5, 3e-2)), (window, L, float((got - ref).abs().max()))
            if window == 0 and L >= 300:
                assert float(got[::n_q // n_kv].mean()) > 4.5      # the needle's value is what comes out
        assert torch.allclose(out.float(), plain_out.float(), atol=tol(dtype, 2e-5, 3e-2))


# ------------------------------------------------------------------------------------------ sampling
def test_argmax_ties_and_sizes():
    o = ops()
    for V in (17, 384, 1000, 128256):
        g = torch.Generator().manual_seed(V)
        logits = torch.randn(5, V, generator=g)
        logits[1, 7] = logits[1].max() + 1
        logits[2, [3, V - 1]] = 50.0              # a tie: the lowest index wins
        logits[3, V - 1] = 60.0
        out = torch.empty(5, dtype=torch.int32, device=DEV)
        o.sample(logits.to(DEV), out)
        assert out.cpu().tolist() == [plain.greedy(r) for r in logits]
        assert out.cpu().tolist()[2] == 3
    # many blocks per row: 16-byte loads (row length a multiple of 4) and plain ones (5003), few rows and many
    # (the grid is cut differently), ties inside one 16-byte group, across groups and across slices
    for V, R in ((4100, 3), (5003, 3), (128256, 64), (50000, 33)):
        g = torch.Generator().manual_seed(V + R)
        logits = torch.randn(R, V, generator=g)
        logits[0, [V // 2 + 1, V // 2 + 2]] = 40.0
        logits[1, [9, V - 2]] = 41.0
        logits[2, [V // 3, V // 3 + 4]] = 42.0
        out = torch.empty(R, dtype=torch.int32, device=DEV)
        o.sample(logits.to(DEV), out)
        assert out.cpu().tolist() == [plain.greedy(r) for r in logits]
        assert out.cpu().tolist()[:3] == [V // 2 + 1, 9, V // 3]


@pytest.mark.parametrize("top_p", [1.0, 0.9, 0.3, 0.0])
@pytest.mark.parametrize("V", [384, 5000])
def test_temperature_sampling_matches_plain_draw(top_p, V):
    from llm_infer_engine_b200.sampling import uniform_for
    o = ops()
    g = torch.Generator().manual_seed(13)
    R, temperature, seed = 24, 0.8, 1234
    logits = torch.randn(R, V, generator=g) * 3
    seq_ids = torch.arange(100, 100 + R, dtype=torch.int32)
    counters = torch.arange(R, dtype=torch.int32) % 5
    out = torch.empty(R, dtype=torch.int32, device=DEV)
    cnt_dev = counters.clone().to(DEV)
    o.sample(logits.to(DEV), out, temperature, top_p, seed, seq_ids.to(DEV), cnt_dev)
    assert cnt_dev.cpu().tolist() == (counters + 1).tolist()
    got = out.cpu().tolist()
    for r in range(R):
        u = uniform_for(seed, int(seq_ids[r]), int(counters[r]))
        want = plain.sample_with_uniform(logits[r], temperature, top_p, u)
        if got[r] != want:
            # float32 vs float64 cumulative sums may put u on the other side of a boundary: then
            # the two tokens must be neighbours in the kept set and u within rounding of the edge
            probs = torch.softmax(logits[r].double() / temperature, dim=-1)
            keep = plain.kept_by_top_p(probs, top_p)
            assert bool(keep[got[r]]), (r, got[r], want)
            cdf = torch.cumsum(torch.where(keep, probs, torch.zeros_like(probs)), 0) / probs[keep].sum()
            edge = float(cdf[min(got[r], want)])
            assert abs(edge - u) < 1e-5, (r, got[r], want, edge, u)
    if top_p == 0.0:
        assert got == [plain.greedy(r) for r in logits]
    # the same sequence id and counter give the same draw whatever row it sits in
    out2 = torch.empty(R, dtype=torch.int32, device=DEV)
    perm = torch.randperm(R, generator=g)
    o.sample(logits[perm].to(DEV), out2, temperature, top_p, seed, seq_ids[perm].to(DEV), counters[perm].clone().to(DEV))
    assert out2.cpu().tolist() == [got[i] for i in perm.tolist()]


# ------------------------------------------------------------------------------------------ skinny GEMM
@pytest.mark.parametrize("batch", [1, 3, 8, 9, 16, 27, 32])
@pytest.mark.parametrize("N,K", [(96, 64), (3072, 2048), (384, 96), (2048, 8192)])
def test_gemm_skinny_epilogues(batch, N, K):
    o = ops()
    g = torch.Generator().manual_seed(batch * 1000 + N)
    x = torch.randn(batch, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T                       # exact product of the bfloat16 values
    assert o.gemm_skinny_ok(batch, N, K)
    xd, wd = x.to(DEV), w.to(DEV)
    out32 = torch.full((batch, N), float("nan"), dtype=torch.float32, device=DEV)
    o.gemm_skinny(xd, wd, out32, o.SKINNY_STORE_F32)
    assert torch.allclose(out32.cpu().double(), ref, atol=2e-4, rtol=1e-4), float((out32.cpu().double() - ref).abs().max())
    out16 = torch.empty((batch, N), dtype=torch.bfloat16, device=DEV)
    o.gemm_skinny(xd, wd, out16, o.SKINNY_STORE_BF16)
    assert torch.equal(out16.cpu(), out32.cpu().to(torch.bfloat16))           # one rounding of the same sums
    h = torch.randn(batch, N, generator=g)
    hd_ = h.clone().to(DEV)
    o.gemm_skinny(xd, wd, hd_, o.SKINNY_ADD_F32)
    assert torch.allclose(hd_.cpu(), h + out32.cpu(), atol=1e-6)
    # gate/up pairing: the weight is [gate rows; up rows]
    ff = N // 2
    if ff % 8 == 0:
        act = torch.empty((batch, ff), dtype=torch.bfloat16, device=DEV)
        o.gemm_skinny(xd, wd, act, o.SKINNY_SWIGLU)
        gate, up = ref[:, :ff], ref[:, ff:]
        want = gate * torch.sigmoid(gate) * up
        assert torch.allclose(act.cpu().double(), want, atol=2e-2, rtol=2e-2)
    # rows do not depend on their neighbours in the batch
    if batch > 1:
        one = torch.empty((1, N), dtype=torch.float32, device=DEV)
        o.gemm_skinny(xd[batch // 2:batch // 2 + 1].contiguous(), wd, one, o.SKINNY_STORE_F32)
        assert torch.equal(one[0].cpu(), out32[batch // 2].cpu())


def test_gemm_skinny_refuses_other_shapes():
    o = ops()
    assert not o.gemm_skinny_ok(33, 64, 64) and not o.gemm_skinny_ok(4, 60, 64) and not o.gemm_skinny_ok(4, 64, 48)
    assert not o.gemm_skinny_ok(4, 24, 64, o.SKINNY_SWIGLU) and o.gemm_skinny_ok(4, 48, 64, o.SKINNY_SWIGLU)
    x = torch.zeros(4, 48, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(64, 48, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(Exception, match="not supported"):
        o.gemm_skinny(x, w, torch.zeros(4, 64, dtype=torch.bfloat16, device=DEV), o.SKINNY_STORE_BF16)


# ------------------------------------------------------------------------------------------ tcgen05 GEMM
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 128, 256), (256, 384, 2048), (100, 200, 72), (2048, 3072, 2048),
                                   (1, 128, 64), (333, 1000, 520)])
def test_gemm_tc(M, N, K):
    o = ops()
    g = torch.Generator().manual_seed(M + N + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = a.double() @ w.double().T
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), out32)
    o.check_tc_status(DEV)
    err = float((out32.cpu().double() - ref).abs().max())
    assert err < 5e-4, err
    out16 = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    o.gemm_tc(a.to(DEV), w.to(DEV), out16)
    o.check_tc_status(DEV)
    assert torch.equal(out16.cpu(), out32.cpu().to(torch.bfloat16))


@pytest.mark.parametrize("M", [1, 9, 16, 17, 33, 64])
@pytest.mark.parametrize("N,K,splits", [(3072, 2048, 0), (2048, 8192, 0), (2048, 2048, 8), (200, 520, 0), (1000, 72, 2),
                                        (16384, 512, 0), (130, 4096, 4), (40000, 256, 1)])
def test_gemm_stream(M, N, K, splits):
    """The weight-streaming tcgen05 product for up to 64 rows: every store mode, K cut into 1 to 8 slices that meet in
    the cluster's shared memory, widths and depths that are no multiples of the tiles (the TMA loads fill with zeros,
    the stores are masked), clusters that take several tiles each, and twice in a row on the same output."""
    o = ops()
    g = torch.Generator().manual_seed(M * 7 + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    ref = x.double() @ w.double().T
    xd, wd = x.to(DEV), w.to(DEV)
    out32 = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    o.gemm_stream(xd, wd, out32, o.STREAM_STORE_F32, splits=splits)
    o.check_tc_status(DEV)
    err = float((out32.cpu().double() - ref).abs().max())
    assert err < 1e-3, err
    again = torch.full_like(out32, float("nan"))
    o.gemm_stream(xd, wd, again, o.STREAM_STORE_F32, splits=splits)
    assert torch.equal(again, out32)                    # slices are added in slice order: no run differs from another
    out16 = torch.empty((M, N), dtype=torch.bfloat16, device=DEV)
    o.gemm_stream(xd, wd, out16, o.STREAM_STORE_BF16, splits=splits)
    assert torch.equal(out16.cpu(), out32.cpu().to(torch.bfloat16))
    h = torch.randn(M, N, generator=g)
    hd_ = h.to(DEV)
    o.gemm_stream(xd, wd, hd_, o.STREAM_ADD_F32, splits=splits)
    o.check_tc_status(DEV)
    assert torch.equal(hd_.cpu(), h + out32.cpu())      # one rounding: h + (the float32 sum)


def test_gemm_stream_refuses_what_it_cannot_take():
    o = ops()
    x = torch.zeros(65, 64, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(128, 64, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(o.KernelError, match="not supported"):
        o.gemm_stream(x, w, torch.zeros(65, 128, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(o.KernelError, match="not supported"):
        o.gemm_stream(x[:4, :60].contiguous(), w[:, :60].contiguous(), torch.zeros(4, 128, dtype=torch.bfloat16, device=DEV))


def test_a_bounded_wait_that_runs_out_is_reported_and_leaves_the_device_usable():
    """The give-up path of the tensor-core kernels' bounded waits: a block waits (at most 1,000 polls) on a
    barrier at which nothing arrives. It must give up, leave the code of the wait in the status word, free
    its tensor memory and return; the host then raises once, the word is clean again, and the next
    tensor-core product (which needs the tensor memory the block held) is correct."""
    import time
    o = ops()
    o.check_tc_status(DEV)                       # clean before
    t0 = time.time()
    o.tc_wait_probe(DEV, limit=1000)
    with pytest.raises(o.KernelError, match="timed out: a TMA load did not arrive"):
        o.check_tc_status(DEV)
    assert time.time() - t0 < 5.0                # it gave up after its polls; it did not hang
    assert int(o.tc_status_word(DEV).item()) == 0
    o.check_tc_status(DEV)                       # raised once, clean again
    # tensor memory was freed and the context is intact: a full-size product right after is right
    g = torch.Generator().manual_seed(1)
    a = torch.randn(256, 512, generator=g).to(torch.bfloat16)
    w = (torch.randn(384, 512, generator=g) / math.sqrt(512)).to(torch.bfloat16)
    out = torch.full((256, 384), float("nan"), dtype=torch.float32, device=DEV)
    for _ in range(3):                           # several blocks per SM over time: none finds the memory still held
        o.gemm_tc(a.to(DEV), w.to(DEV), out)
    o.check_tc_status(DEV)
    assert float((out.cpu().double() - a.double() @ w.double().T).abs().max()) < 5e-4


# ------------------------------------------------------------------------------------------ tcgen05 prefill attention
@pytest.mark.parametrize("n_q,n_kv,hd", [(4, 2, 64), (3, 1, 64), (8, 8, 64), (4, 1, 128), (6, 2, 128)])
def test_attention_prefill_tc(n_q, n_kv, hd):
    """Ragged runs of new tokens at nonzero start positions, across key tiles and cache pages,
    against the plain formula and the plain kernel; with and without a window; a far key made
    to dominate so that a lost tile cannot hide."""
    o = ops()
    dtype = torch.bfloat16
    assert o.attention_prefill_tc_supported(hd, 64, dtype)
    # the last two run over six and eight key tiles: both score buffers and every barrier phase come round again
    starts, news = [0, 70, 3, 200, 0, 130, 0, 600], [50, 9, 300, 129, 1, 128, 700, 300]
    totals = [s + n for s, n in zip(starts, news)]
    pg = Paged(totals, n_kv, hd, dtype, seed=hd + n_q)
    T = sum(news)
    g = torch.Generator().manual_seed(17)
    q = torch.randn(T, n_q, hd, generator=g)
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    # needle: sequence 2 (303 keys, three key tiles): its last query looks hard at key 5
    G = n_q // n_kv
    qi = cu[3] - 1
    qh = q[qi, ::G]
    pg.dense_k[2][5] = (qh * (24.0 / ((qh * qh).sum(-1, keepdim=True) * hd ** -0.5))).to(dtype)
    pg.dense_v[2][5] = 5.0
    pg.fill()
    k_dev, v_dev, bt = pg.dev()
    # the kernel wants the last page to be readable scratch: Paged leaves spare pages, the last is unused
    qd = q.to(dtype).reshape(T, n_q * hd).to(DEV)
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    cu_dev = torch.tensor(cu, dtype=torch.int32, device=DEV)
    st_dev = torch.tensor(starts, dtype=torch.int32, device=DEV)
    tok_seq = torch.repeat_interleave(torch.arange(len(news)), torch.tensor(news)).int().to(DEV)
    tok_pos = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, news)]).int().to(DEV)
    for window in (0, 100):
        out = torch.full((T, n_q * hd), float("nan"), dtype=dtype, device=DEV)
        o.attention_prefill_tc(qd, k_dev, v_dev, out, cu_dev, slots, st_dev, bt, 64, len(news), max(news), n_q, n_kv, hd,
                               hd ** -0.5, window)
        o.check_tc_status(DEV)
        plain_out = torch.empty_like(out)
        o.attention_paged(qd, k_dev, v_dev, plain_out, tok_pos, tok_seq, slots, bt, 64, n_q, n_kv, hd, hd ** -0.5, window)
        got = out.float().cpu().view(T, n_q, hd)
        assert not torch.isnan(got).any()
        for i, n in enumerate(news):
            ref = ref_attention(qd.float().cpu().view(T, n_q, hd)[cu[i]:cu[i + 1]], pg.dense_k[i].float(),
                                pg.dense_v[i].float(), list(range(starts[i], starts[i] + n)), hd ** -0.5, window)
            # outputs are bfloat16: one unit in the last place is 2^-8 of the value's magnitude
            assert torch.allclose(got[cu[i]:cu[i + 1]], ref, atol=2e-2, rtol=1.6e-2), \
                (window, i, float((got[cu[i]:cu[i + 1]] - ref).abs().max()))
        assert torch.allclose(out.float(), plain_out.float(), atol=2e-2, rtol=1.6e-2)
        if window == 0:
            assert float(got[qi, ::G].mean()) > 4.5


# ------------------------------------------------------------------------------------------ fused one-token kernels
@pytest.mark.parametrize("batch", [1, 3, 8])
@pytest.mark.parametrize("K,ff", [(64, 96), (160, 224), (2048, 8192), (96, 256)])
def test_norm_gate_swiglu(batch, K, ff):
    o = ops()
    g = torch.Generator().manual_seed(batch + K)
    h = torch.randn(batch, K, generator=g) * 2
    nw = torch.rand(K, generator=g) + 0.5
    w = (torch.randn(2 * ff, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    eps = 1e-5
    assert o.norm_gemm_supported(batch, K)
    act = torch.full((batch, ff), float("nan"), dtype=torch.bfloat16, device=DEV)
    o.norm_gate_swiglu(h.to(DEV), nw.to(DEV), eps, w.to(DEV), act)
    x = plain.rms_norm(h, nw, eps)
    y = x.double() @ w.double().T
    want = (y[:, :ff] * torch.sigmoid(y[:, :ff]) * y[:, ff:]).float()
    assert torch.allclose(act.float().cpu(), want, atol=3e-2, rtol=3e-2), float((act.float().cpu() - want).abs().max())


@pytest.mark.parametrize("batch,N,K", [(1, 256, 64), (5, 384, 96), (8, 128256, 2048), (2, 512, 160)])
def test_norm_gemm_f32(batch, N, K):
    o = ops()
    g = torch.Generator().manual_seed(batch + N)
    h = torch.randn(batch, K, generator=g) * 3
    nw = torch.rand(K, generator=g) + 0.5
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16)
    out = torch.full((batch, N), float("nan"), dtype=torch.float32, device=DEV)
    o.norm_gemm_f32(h.to(DEV), nw.to(DEV), 1e-6, w.to(DEV), out)
    want = (plain.rms_norm(h, nw, 1e-6).double() @ w.double().T).float()
    assert torch.allclose(out.cpu(), want, atol=2e-2, rtol=2e-2), float((out.cpu() - want).abs().max())


@pytest.mark.parametrize("batch", [1, 4, 8])
@pytest.mark.parametrize("n_q,n_kv,hd,K", [(4, 2, 16, 64), (3, 1, 32, 96), (6, 2, 64, 160), (32, 8, 64, 2048), (4, 1, 128, 256)])
def test_norm_qkv_rope(batch, n_q, n_kv, hd, K):
    """Against the unfused pair: norm kernel + product + rotary/cache-write kernel."""
    o = ops()
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(batch * 7 + hd)
    starts = [int(x) for x in torch.randint(0, 150, (batch,), generator=g)]
    pg = Paged([s + 1 for s in starts], n_kv, hd, dtype, seed=hd)
    k_dev, v_dev, bt = pg.dev()
    k2, v2 = k_dev.clone(), v_dev.clone()
    h = torch.randn(batch, K, generator=g) * 2
    nw = torch.rand(K, generator=g) + 0.5
    w = (torch.randn((n_q + 2 * n_kv) * hd, K, generator=g) / math.sqrt(K)).to(dtype)
    inv = plain.inv_frequencies(hd, 10000.0, None)
    cos, sin = plain.rotation_tables(torch.arange(256), inv)
    table = torch.stack([cos, sin], dim=-1).contiguous().to(DEV)
    tok_pos = torch.tensor(starts, dtype=torch.int32, device=DEV)
    tok_seq = torch.arange(batch, dtype=torch.int32, device=DEV)
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    q = torch.full((batch, n_q * hd), float("nan"), dtype=dtype, device=DEV)
    o.norm_qkv_rope(h.to(DEV), nw.to(DEV), 1e-5, w.to(DEV), q, k_dev, v_dev, table, tok_pos, tok_seq, slots, bt, 64,
                    n_q, n_kv, hd)
    # the unfused path
    xn = torch.empty(batch, K, dtype=dtype, device=DEV)
    o.add_rmsnorm(h.clone().to(DEV), None, nw.to(DEV), 1e-5, xn)
    qkv = (xn.float() @ w.to(DEV).float().T).to(dtype)
    q2 = torch.empty_like(q)
    o.rope_store(qkv, q2, k2, v2, table, tok_pos, tok_seq, slots, bt, 64, n_q, n_kv, hd, hd)
    assert torch.allclose(q.float(), q2.float(), atol=3e-2, rtol=3e-2), float((q.float() - q2.float()).abs().max())
    assert torch.allclose(k_dev.float(), k2.float(), atol=3e-2, rtol=3e-2)
    assert torch.allclose(v_dev.float(), v2.float(), atol=3e-2, rtol=3e-2)
    # and it wrote exactly the cache rows the unfused path wrote
    assert torch.equal((k_dev != pg.dev()[0]).any(-1), (k2 != pg.dev()[0]).any(-1))
    # against plain torch: norm and product in float64 on the bfloat16 weights, plain rotation by position
    x64 = h.double()
    x64 = x64 * torch.rsqrt((x64 * x64).mean(-1, keepdim=True) + 1e-5) * nw.double()
    qkv64 = x64 @ w.double().T
    for b in range(batch):
        c, s_ = cos[starts[b]].double(), sin[starts[b]].double()
        rot = lambda v: torch.cat([v[..., :hd // 2] * c - v[..., hd // 2:] * s_, v[..., hd // 2:] * c + v[..., :hd // 2] * s_], -1)
        q_ref = rot(qkv64[b, :n_q * hd].view(n_q, hd))
        k_ref = rot(qkv64[b, n_q * hd:(n_q + n_kv) * hd].view(n_kv, hd))
        v_ref = qkv64[b, (n_q + n_kv) * hd:].view(n_kv, hd)
        page = int(pg.block_table[pg.slots[b], starts[b] // 64])
        k_got = k_dev[page, :, starts[b] % 64].double().cpu()
        v_got = v_dev[page, :, starts[b] % 64].double().cpu()
        # bfloat16 outputs of values a few units large: half a unit in the last place is 2^-8 of the value
        for name, got_t, ref_t in (("q", q[b].double().cpu().view(n_q, hd), q_ref), ("k", k_got, k_ref), ("v", v_got, v_ref)):
            err = float((got_t - ref_t).abs().max())
            assert err <= 2e-2 * max(1.0, float(ref_t.abs().max())), (name, b, err, float(ref_t.abs().max()))


@pytest.mark.parametrize("n_q,n_kv,hd", [(6, 2, 64), (32, 8, 64), (4, 1, 128), (24, 8, 128)])
@pytest.mark.parametrize("window,pages", [(0, 0), (100, 0), (0, 4)])
def test_decode_attention_with_rotation_and_cache_write_inside(n_q, n_kv, hd, window, pages):
    """One-token attention straight from the raw projections (rotation of q and k and the cache write inside the
    kernel) against the two separate kernels, for sequences whose newest position is a page's first row, its
    last, the first of a half page, and deep in a long sequence cut into runs; and against plain attention."""
    o = ops()
    dtype = torch.bfloat16
    lens = [1, 64, 65, 97, 128, 700, 333, 33, 1500]
    n = len(lens)
    pg = Paged(lens, n_kv, hd, dtype, seed=hd + n_q)
    pg.fill(upto=[l - 1 for l in lens])                # everything but the newest position, which the step brings
    g = torch.Generator().manual_seed(3)
    qkv = torch.randn(n, (n_q + 2 * n_kv) * hd, generator=g).to(dtype).to(DEV)
    inv = plain.inv_frequencies(hd, 10000.0, None)
    cos, sin = plain.rotation_tables(torch.arange(2048), inv)
    table = torch.stack([cos, sin], dim=-1).contiguous().to(DEV)
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    kvlen = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([l - 1 for l in lens], dtype=torch.int32, device=DEV)
    tok_seq = torch.arange(n, dtype=torch.int32, device=DEV)
    max_kv = 2048
    pages = pages or o.attention_decode_mma_pages(n, n_q, n_kv, max_kv)     # 4: long sequences are merged from 8 runs
    n_runs = ((max_kv + 63) // 64 + pages - 1) // pages
    counters = torch.zeros(o.decode_counter_ints(n, n_q, n_kv) + 64, dtype=torch.int32, device=DEV)
    # the two separate kernels
    k1, v1, bt = pg.dev()
    q1 = torch.empty(n, n_q * hd, dtype=dtype, device=DEV)
    o.rope_store(qkv, q1, k1, v1, table, tok_pos, tok_seq, slots, bt, 64, n_q, n_kv, hd, hd)
    want = torch.empty_like(q1)
    o.attention_decode_mma(q1, k1, v1, want, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, window, pages, n_runs,
                           counters=counters)
    # one kernel
    k2, v2, _ = pg.dev()
    got = torch.full_like(want, float("nan"))
    o.attention_decode_mma_rope(qkv, k2, v2, got, table, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, window, pages,
                                n_runs, True, counters=counters)
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2), float((got.float() - want.float()).abs().max())
    assert torch.allclose(k2.float(), k1.float(), atol=1e-2, rtol=1e-2) and torch.equal(v2, v1)
    assert torch.equal((k2 != pg.dev()[0]).any(-1), (k1 != pg.dev()[0]).any(-1))     # the same cache rows were written
    assert int(counters.abs().sum()) == 0
    # without the cache write the cache is left alone and the output is the same
    k3, v3, _ = pg.dev()
    again = torch.empty_like(want)
    o.attention_decode_mma_rope(qkv, k3, v3, again, table, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, window, pages,
                                n_runs, False, counters=counters)
    assert torch.equal(again, got) and torch.equal(k3, pg.dev()[0]) and torch.equal(v3, pg.dev()[1])
    # plain attention over the dense keys (the newest one rotated in float32)
    for i, L in enumerate(lens):
        row = qkv[i].float().cpu()
        qf = row[:n_q * hd].view(n_q, 1, hd)
        kf = row[n_q * hd:(n_q + n_kv) * hd].view(n_kv, 1, hd)
        vf = row[(n_q + n_kv) * hd:].view(n_kv, hd)
        c, s_ = cos[L - 1:L], sin[L - 1:L]
        qr = plain.rotate_half(qf, c, s_).view(1, n_q, hd).to(dtype).float()
        kd, vd = pg.dense_k[i].float().clone(), pg.dense_v[i].float().clone()
        kd[L - 1] = plain.rotate_half(kf, c, s_).view(n_kv, hd).to(dtype).float()
        vd[L - 1] = vf
        ref = ref_attention(qr, kd, vd, [L - 1], hd ** -0.5, window).reshape(-1)
        assert torch.allclose(got[i].float().cpu(), ref, atol=3e-2), (i, L, float((got[i].float().cpu() - ref).abs().max()))


def test_attention_decode_merge_reads_fresh_partials():
    """The block that merges the runs of a sequence must see the other blocks' partial results of THIS
    launch. Few query heads make the partial maxima of many sequences share a 128-byte line, the scratch
    area is reused launch after launch with other inputs, and many merging blocks share an SM: a merge
    that read a line through a stale L1 copy would be far from the merge by a second kernel."""
    o = ops()
    dtype, n_q, n_kv, hd = torch.bfloat16, 3, 1, 32
    g = torch.Generator().manual_seed(5)
    lens = [int(x) for x in torch.randint(65, 256, (300,), generator=g)]
    pg = Paged(lens, n_kv, hd, dtype, seed=9)
    pg.fill()
    k_dev, v_dev, bt = pg.dev()
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    kvlen = torch.tensor(lens, dtype=torch.int32, device=DEV)
    n_runs = 4
    counters = torch.zeros(o.decode_counter_ints(len(lens), n_q, n_kv), dtype=torch.int32, device=DEV)
    scratch = torch.zeros(o.decode_scratch_floats(len(lens), n_q, hd, n_runs), dtype=torch.float32, device=DEV)
    for it in range(12):
        q = (torch.randn(len(lens), n_q * hd, generator=g) * (1 + it)).to(dtype).to(DEV)
        fused = torch.empty_like(q)
        o.attention_decode(q, k_dev, v_dev, fused, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, 0, 64, n_runs,
                           scratch=scratch, counters=counters)
        two = torch.empty_like(q)
        o.attention_decode(q, k_dev, v_dev, two, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, 0, 64, n_runs)
        assert torch.allclose(fused.float(), two.float(), atol=3e-2, rtol=3e-2), (it, float((fused.float() - two.float()).abs().max()))
    assert int(counters.abs().sum()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n_q,n_kv,hd", [(32, 8, 64), (6, 2, 128), (4, 4, 16)])
def test_attention_decode_many_sequences(dtype, n_q, n_kv, hd):
    """Many sequences of unequal lengths in one launch, merged in the same launch or by the second kernel."""
    o = ops()
    g = torch.Generator().manual_seed(3 + hd)
    lens = [int(x) for x in torch.randint(1, 700, (40,), generator=g)]
    lens[0], lens[1], lens[2] = 1, 256, 257
    pg = Paged(lens, n_kv, hd, dtype, seed=hd)
    pg.fill()
    q = torch.randn(len(lens), n_q, hd, generator=g)
    k_dev, v_dev, bt = pg.dev()
    qd = q.to(dtype).reshape(len(lens), n_q * hd).to(DEV)
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    kvlen = torch.tensor(lens, dtype=torch.int32, device=DEV)
    run_len = o.attention_decode_run_len(len(lens), hd, dtype)
    assert run_len % 64 == 0 and run_len >= 64
    n_runs = (768 + run_len - 1) // run_len
    counters = torch.zeros(o.decode_counter_ints(len(lens), n_q, n_kv), dtype=torch.int32, device=DEV)
    for window in (0, 90):
        for fused in (True, False):
            out = torch.full((len(lens), n_q * hd), float("nan"), dtype=dtype, device=DEV)
            o.attention_decode(qd, k_dev, v_dev, out, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, window, run_len,
                               n_runs, counters=counters if fused else None)
            got = out.float().cpu().view(len(lens), n_q, hd)
            assert not torch.isnan(got).any()
            for i in (0, 1, 2, 7, 23, 39):
                ref = ref_attention(qd.float().cpu().view(len(lens), n_q, hd)[i:i + 1], pg.dense_k[i].float(),
                                    pg.dense_v[i].float(), [lens[i] - 1], hd ** -0.5, window)[0]
                assert torch.allclose(got[i], ref, atol=tol(dtype, 2e-5, 3e-2)), (window, fused, i)
        assert int(counters.abs().sum()) == 0          # left clean


def test_attention_decode_mma_page_choice():
    o = ops()
    # a whole sequence per block while a warp takes at most four pages in turn
    assert o.attention_decode_mma_pages(8, 32, 8, 512) == 8
    assert o.attention_decode_mma_pages(8, 32, 8, 1024) == 16
    assert o.attention_decode_mma_pages(64, 32, 8, 1024) == 16
    assert o.attention_decode_mma_pages(8, 32, 8, 4096) == 32          # two runs, 128 blocks
    assert o.attention_decode_mma_pages(256, 32, 8, 4096) == 64        # enough blocks already
    assert o.attention_decode_mma_pages(1, 32, 8, 3500) == 7           # one long sequence: cut on, 64 blocks
    assert o.attention_decode_mma_pages(4, 32, 8, 3500) == 14          # 128 blocks; eight runs would be 256
    for n, kv in ((1, 64), (1, 131072), (48, 640), (64, 8192), (256, 131072)):
        pp = o.attention_decode_mma_pages(n, 32, 8, kv)
        assert 1 <= pp <= (kv + 63) // 64


@pytest.mark.parametrize("n_q,n_kv,hd", [(32, 8, 64), (6, 2, 128), (40, 2, 64), (3, 3, 64)])
@pytest.mark.parametrize("n_seqs,pages_per_run", [(36, 16), (36, 4), (5, 16), (5, 8), (2, 1)])
def test_attention_decode_mma(n_q, n_kv, hd, n_seqs, pages_per_run):
    check_attention_decode_mma(n_q, n_kv, hd, n_seqs, pages_per_run)


@pytest.mark.parametrize("n_q,n_kv,hd,n_seqs", [(32, 8, 64, 64), (32, 8, 64, 80), (6, 2, 128, 80), (6, 2, 128, 200)])
def test_attention_decode_mma_block_forms(n_q, n_kv, hd, n_seqs):
    """Grids that make the launcher take three and two warps per block."""
    check_attention_decode_mma(n_q, n_kv, hd, n_seqs, 16)


def check_attention_decode_mma(n_q, n_kv, hd, n_seqs, pages_per_run):
    """A warp per page on the tensor cores: whole sequences in one block (written straight to the output)
    and several runs (merged by the last block), few and many blocks (8 or 4 warps), groups of more than
    16 query heads, with and without a window, lengths on, before and after a page boundary."""
    o = ops()
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(11 + hd + pages_per_run + n_seqs)
    lens = [int(x) for x in torch.randint(1, 1000, (n_seqs,), generator=g)]
    special = [1, 1000, 64, 65, 128]
    for i in range(min(n_seqs, len(special))):
        lens[i] = special[i]
    pg = Paged(lens, n_kv, hd, dtype, seed=hd)
    pg.fill()
    q = torch.randn(len(lens), n_q, hd, generator=g) * 2.0        # peaked scores: a skipped page would show
    k_dev, v_dev, bt = pg.dev()
    qd = q.to(dtype).reshape(len(lens), n_q * hd).to(DEV)
    slots = torch.tensor(pg.slots, dtype=torch.int32, device=DEV)
    kvlen = torch.tensor(lens, dtype=torch.int32, device=DEV)
    n_runs = (16 + pages_per_run - 1) // pages_per_run            # 16 pages hold 1024 keys
    counters = torch.zeros(max(64, len(lens) * n_kv * 4), dtype=torch.int32, device=DEV)
    assert o.attention_decode_mma_supported(hd, dtype, 64)
    for window in (0, 90):
        out = torch.full((len(lens), n_q * hd), float("nan"), dtype=dtype, device=DEV)
        o.attention_decode_mma(qd, k_dev, v_dev, out, slots, kvlen, bt, 64, n_q, n_kv, hd, hd ** -0.5, window,
                               pages_per_run, n_runs, counters=counters)
        got = out.float().cpu().view(len(lens), n_q, hd)
        assert not torch.isnan(got).any()
        for i in sorted(set([0, 1, 2, 3, 4, 7, 23, 35, n_seqs - 1]) & set(range(n_seqs))):
            ref = ref_attention(qd.float().cpu().view(len(lens), n_q, hd)[i:i + 1], pg.dense_k[i].float(),
                                pg.dense_v[i].float(), [lens[i] - 1], hd ** -0.5, window)[0]
            assert torch.allclose(got[i], ref, atol=3e-2), (window, i, float((got[i] - ref).abs().max()))
    assert int(counters.abs().sum()) == 0          # left clean


@pytest.mark.parametrize("hd,window", [(64, 0), (128, 0), (64, 256)])
def test_attention_prefill_tc_is_repeatable(hd, window):
    """The prompt kernel overlaps a key tile's second product with the next tile's softmax and reuses its score
    buffers for other data; a missing wait would show as outputs that change from run to run. Twelve runs of
    unequal sequences at start positions above zero must agree bit for bit."""
    o = ops()
    n_q, n_kv, P = 8, 2, 64
    lens, starts = [700, 129, 1000, 64, 1], [0, 300, 77, 1000, 5]
    n = len(lens)
    pages_per = max((s + l + P - 1) // P for s, l in zip(starts, lens))
    g = torch.Generator().manual_seed(31)
    k = torch.randn(n * pages_per + 1, n_kv, P, hd, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(n * pages_per + 1, n_kv, P, hd, generator=g).to(torch.bfloat16).to(DEV)
    bt = torch.randperm(n * pages_per, generator=g).to(torch.int32).view(n, pages_per).contiguous().to(DEV)
    T = sum(lens)
    q = torch.randn(T, n_q * hd, generator=g).to(torch.bfloat16).to(DEV)
    cu = torch.tensor([0] + torch.tensor(lens).cumsum(0).tolist(), dtype=torch.int32, device=DEV)
    slots = torch.arange(n, dtype=torch.int32, device=DEV)
    st = torch.tensor(starts, dtype=torch.int32, device=DEV)
    first = None
    for _ in range(12):
        out = torch.full((T, n_q * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        o.attention_prefill_tc(q, k, v, out, cu, slots, st, bt, P, n, max(lens), n_q, n_kv, hd, hd ** -0.5, window)
        if first is None:
            first = out
            assert not torch.isnan(out.float()).any()
        else:
            assert torch.equal(out, first)
    o.check_tc_status(DEV)
