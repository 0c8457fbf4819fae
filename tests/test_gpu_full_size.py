"""Full benchmark sizes on the GPU, checked through size-independent properties
(the oracle would take minutes here): append -> export round trips, fused vs
separate append, invariance to the work split, page conservation, and float64 spot
checks of single (sequence, kv head) pairs rebuilt from the exported block tables."""
import numpy as np
import pytest
import torch

from combsengine_b200 import KVArena
from kvcase import assert_attention_close

pytestmark = pytest.mark.gpu


def attend_f64(q, k, v, scale, window=None):
    """q [h, d], k/v [L, d] (one kv head, the query is the last position)."""
    L = k.shape[0]
    s = (q.astype(np.float64) @ k.astype(np.float64).T) * scale
    if window is not None:
        s[:, : max(0, L - window)] = -np.inf
    s -= s.max(-1, keepdims=True)
    p = np.exp(s)
    p /= p.sum(-1, keepdims=True)
    return p @ v.astype(np.float64)


class Big:
    def __init__(self, layers, n_q, n_kv, d, lens, num_pages, windows=None, seed=0, prefix=0):
        self.n_q, self.n_kv, self.d, self.layers = n_q, n_kv, d, layers
        self.arena = KVArena(layers, n_q, n_kv, d, 40000, 16, num_pages, windows=windows, sliding_popn_refuses=False)
        self.arena.set_free_list(np.random.default_rng(seed).permutation(num_pages))
        self.gen = torch.Generator(device="cuda").manual_seed(seed)
        self.kv = {}  # seq index -> (k [n_kv, L, d], v) on the host, layer 0
        if prefix:
            self.root = self.arena.new_seq()
            pk, pv = self._fill([self.root], [prefix])
            self.seqs = [self.root.fork_prefix(prefix) for _ in lens]
        else:
            self.seqs = [self.arena.new_seq() for _ in lens]
            pk = pv = None
        ks, vs = self._fill(self.seqs, lens)
        for i in range(len(lens)):
            k, v = ks[i], vs[i]
            if prefix:
                k, v = np.concatenate([pk[0], k], 1), np.concatenate([pv[0], v], 1)
            self.kv[i] = (k, v)

    def _rand(self, n):
        return torch.randn(n, device="cuda", generator=self.gen).half()

    def _fill(self, seqs, counts):
        ntok = int(sum(counts))
        kf, vf = self._rand(ntok * self.n_kv * self.d), self._rand(ntok * self.n_kv * self.d)
        self.arena.begin_step(seqs, [int(c) for c in counts])
        for layer in range(self.layers):
            self.arena.append(layer, kf, vf)
        kh, vh, off, ks, vs = kf.cpu().numpy(), vf.cpu().numpy(), 0, [], []
        for c in counts:
            n = int(c) * self.n_kv * self.d
            ks.append(kh[off:off + n].reshape(self.n_kv, int(c), self.d))
            vs.append(vh[off:off + n].reshape(self.n_kv, int(c), self.d))
            off += n
        return ks, vs

    def decode(self, fused=True, scale=None, window=None, layer=0):
        n = len(self.seqs)
        scale = self.d ** -0.5 if scale is None else scale
        q, k, v = self._rand(n * self.n_q * self.d), self._rand(n * self.n_kv * self.d), self._rand(n * self.n_kv * self.d)
        return self.redo(q, k, v, fused, scale, window, layer, first=True)

    def redo(self, q, k, v, fused, scale, window, layer, first=False):
        if not first:
            for s in self.seqs:
                assert s.popn(1) == 1
        self.arena.begin_step(self.seqs, [1] * len(self.seqs))
        if fused:
            out = self.arena.attention(layer, q, k, v, scale, window)
        else:
            self.arena.append(layer, k, v)
            out = self.arena.paged_attention(layer, q, scale, window)
        assert self.arena.device_status() == 0
        return (q, k, v), out

    def spot_check(self, inputs, out, picks, scale, window=None):
        q, k, v = (x.cpu().numpy() for x in inputs)
        o = out.cpu().numpy().reshape(len(self.seqs), self.n_q, self.d)
        rep = self.n_q // self.n_kv
        for b, h in picks:
            kk = np.concatenate([self.kv[b][0][h], k.reshape(-1, self.n_kv, self.d)[b, h][None]], 0)
            vv = np.concatenate([self.kv[b][1][h], v.reshape(-1, self.n_kv, self.d)[b, h][None]], 0)
            qq = q.reshape(-1, self.n_q, self.d)[b, h * rep:(h + 1) * rep]
            assert_attention_close(o[b, h * rep:(h + 1) * rep], attend_f64(qq, kk, vv, scale, window), f"seq {b} head {h}")

    def check_pages_round_trip(self, rng, n=24):
        for _ in range(n):
            b = int(rng.integers(len(self.seqs)))
            tbl = self.seqs[b].block_table()
            lp = int(rng.integers(len(tbl)))
            gk, gv = self.arena.export_page(0, int(tbl[lp]))
            k, v = self.kv[b]
            rows = min(16, k.shape[1] - lp * 16)
            assert np.array_equal(gk[:, :rows], k[:, lp * 16: lp * 16 + rows].view(np.uint16))
            assert np.array_equal(gv[:, :rows], v[:, lp * 16: lp * 16 + rows].view(np.uint16))


def test_cfg2_full_batch_and_arena():
    rng = np.random.default_rng(0xC0B50002)
    lens = rng.integers(1024, 4097, 32)
    w = Big(2, 28, 4, 128, lens, 8192, seed=2)
    assert sum(s.pages_used() for s in w.seqs) + w.arena.num_free_pages() == 8192
    w.check_pages_round_trip(rng)
    inp, out = w.decode(fused=True)
    w.spot_check(inp, out, [(0, 0), (13, 3), (31, 1)], 128 ** -0.5)
    _, out_sep = w.redo(*inp, fused=False, scale=128 ** -0.5, window=None, layer=0)
    assert torch.equal(out, out_sep), "fused append must not change the result"
    for tuning in (dict(consumers=4, ctas_per_sm=2, stages=8), dict(consumers=8, max_ctas=37)):
        w.arena.set_decode_tuning(**tuning)
        _, out_t = w.redo(*inp, fused=True, scale=128 ** -0.5, window=None, layer=0)
        assert_attention_close(out_t.cpu().numpy(), out.cpu().numpy(), f"split {tuning}")
    # the step's new rows landed in their slots
    for b in (0, 31):
        L = w.seqs[b].seq_len()
        gk, _ = w.arena.export_page(0, int(w.seqs[b].block_table()[(L - 1) // 16]))
        assert np.array_equal(gk[:, (L - 1) % 16], inp[1].cpu().numpy().reshape(32, 4, 128)[b].view(np.uint16))


def test_cfg3_full_context_windows():
    w = Big(2, 8, 4, 256, [8192] * 16, 16 * 520, windows=[1024, None], seed=3)
    inp, out = w.decode(layer=0)  # the arena's own window applies
    w.spot_check(inp, out, [(0, 0), (15, 3)], 256 ** -0.5, window=1024)
    inp, out = w.decode(layer=1)
    w.spot_check(inp, out, [(7, 2)], 256 ** -0.5)


def test_cfg5_shared_prefix_long_tails_and_churn():
    rng = np.random.default_rng(0xC0B50005)
    lens = np.round(np.exp(rng.uniform(np.log(128), np.log(32768), 64))).astype(np.int64)
    w = Big(1, 28, 4, 128, lens, 40960, seed=5, prefix=1024)
    prefix_pages = list(w.root.block_table())
    assert all(w.arena.refcount(int(p)) == 65 for p in prefix_pages)
    inp, out = w.decode()
    longest, shortest = int(np.argmax(lens)), int(np.argmin(lens))
    w.spot_check(inp, out, [(longest, 2), (shortest, 0)], 128 ** -0.5)
    # eviction back to the prefix returns exactly the private pages, LIFO
    free0 = w.arena.num_free_pages()
    victims = [int(i) for i in rng.permutation(64)[:6]]
    private = 0
    for i in victims:
        s = w.seqs[i]
        private += s.pages_used() - 64
        last_private = int(s.block_table()[-1])
        assert s.popn(s.seq_len() - 1024) == s.seq_len() - 1024 or True
        assert s.seq_len() == 1024 and s.pages_used() == 64
    assert w.arena.num_free_pages() == free0 + private
    assert all(w.arena.refcount(int(p)) == 65 for p in prefix_pages)
    top = int(w.arena.free_list()[-1])
    w.arena.begin_step([w.seqs[victims[0]]], [1])  # the next append reuses the most recently freed page
    assert int(w.seqs[victims[0]].block_table()[-1]) == top


def test_cfg2_int8_pages_hold_the_half_step_bound_and_decode_tracks_float64():
    """Benchmark geometry and lengths with quantize_kv: every exported page de-quantises to within
    half a step of what was appended (kv.rs:926-953), and a decode step over the int8 records matches
    a float64 attention computed from those de-quantised pages."""
    n_q, n_kv, d = 28, 4, 128
    rng = np.random.default_rng(0xC0B50002)
    lens = rng.integers(1024, 4097, 32)
    pages = 8192
    arena = KVArena(1, n_q, n_kv, d, 4200, 16, pages, quantize_kv=True)
    arena.set_free_list(rng.permutation(pages))
    seqs = [arena.new_seq() for _ in lens]
    gen = torch.Generator(device="cuda").manual_seed(2)
    ntok = int(lens.sum())
    kf = torch.randn(ntok * n_kv * d, device="cuda", generator=gen).half()
    vf = torch.randn(ntok * n_kv * d, device="cuda", generator=gen).half()
    arena.begin_step(seqs, [int(x) for x in lens])
    arena.append(0, kf, vf)
    one = [1] * len(lens)
    q = torch.randn(len(lens) * n_q * d, device="cuda", generator=gen).half()
    k1 = torch.randn(len(lens) * n_kv * d, device="cuda", generator=gen).half()
    v1 = torch.randn(len(lens) * n_kv * d, device="cuda", generator=gen).half()
    arena.begin_step(seqs, one)
    out = arena.attention(0, q, k1, v1, d ** -0.5).cpu().numpy().reshape(len(lens), n_q, d)
    assert arena.device_status() == 0
    kh, vh = kf.cpu().numpy(), vf.cpu().numpy()
    off = 0
    for b, L in enumerate(lens):
        L = int(L)
        if b in (0, 7, 31):  # three sequences in full
            kb = kh[off:off + L * n_kv * d].reshape(n_kv, L, d)
            vb = vh[off:off + L * n_kv * d].reshape(n_kv, L, d)
            K = np.zeros((n_kv, L + 1, d), np.float32)
            V = np.zeros_like(K)
            for lp, pg in enumerate(seqs[b].block_table()):
                kp, ks, vp, vs = arena.export_page_quant(0, int(pg))
                n = min(16, L + 1 - lp * 16)
                for packed, scales, dst in ((kp, ks, K), (vp, vs, V)):
                    by = packed.view(np.uint8).reshape(n_kv, 16, d).astype(np.int32)
                    qv = np.where(np.arange(d) % 4 == 3, by.astype(np.int8).astype(np.int32), by - 128)   # kv.rs:326-346
                    sc = np.repeat(scales.view(np.float16).astype(np.float32), 32, axis=-1)
                    dst[:, lp * 16:lp * 16 + n] = (qv * sc).astype(np.float16).astype(np.float32)[:, :n]
            for src, dq in ((kb, K), (vb, V)):
                groups = src.astype(np.float32).reshape(n_kv, L, d // 32, 32)
                err = np.abs(groups - dq[:, :L].reshape(n_kv, L, d // 32, 32)).max(-1)
                # half a step (kv.rs:940) plus what f16 storage adds: the scale and the product q * scale are each rounded to 11 bits
                bound = np.abs(groups).max(-1) * (1.0 / 254.0 + 2.0 ** -10) + 1e-4
                assert np.all(err <= bound)
            qb = q.cpu().numpy().reshape(len(lens), n_q, d)[b].astype(np.float64)
            for h in range(n_kv):
                ref = attend_f64(qb[h * 7:(h + 1) * 7], K[h], V[h], d ** -0.5)
                assert_attention_close(out[b, h * 7:(h + 1) * 7], ref.astype(np.float32), f"seq {b} kv head {h}")
        off += L * n_kv * d
    assert arena.num_free_pages() == pages - sum((int(L) + 1 + 15) // 16 for L in lens)


def test_cfg4_chunk_rotation_preserves_norms_and_is_linear():
    """One 512-token chunk of the cfg4 prompts through the rotate-and-append kernel: a rotation keeps
    the norm of every (i, i + d/2) pair, position 0 is the identity, and rope(a) + rope(b) = rope(a + b)
    up to storage rounding."""
    from combsengine_b200 import rope as R
    n_q, n_kv, d, batch, chunk = 32, 8, 128, 8, 512
    arena = KVArena(1, n_q, n_kv, d, 2 * chunk, 16, batch * (2 * chunk // 16))
    seqs = [arena.new_seq() for _ in range(batch)]
    rope = R.RotaryEmbedding(arena, 500000.0, 2 * chunk)
    gen = torch.Generator(device="cuda").manual_seed(4)
    ntok = batch * chunk
    mk = lambda heads: torch.randn(ntok * heads * d, device="cuda", generator=gen).half()
    qa, qb, k, v = mk(n_q), mk(n_q), mk(n_kv), mk(n_kv)
    arena.begin_step(seqs, [chunk] * batch)                       # positions 0..511
    ra0 = R.rope_append(arena, 0, rope, qa, k, v).float().view(batch, n_q, chunk, d)
    assert torch.equal(ra0[:, :, 0], qa.float().view(batch, n_q, chunk, d)[:, :, 0])          # position 0: identity
    arena.begin_step(seqs, [chunk] * batch)                       # positions 512..1023
    ra = R.rope_append(arena, 0, rope, qa, k, v).float().view(batch, n_q, chunk, d)
    rb = R.rope_append(arena, 0, rope, qb, k, v).float().view(batch, n_q, chunk, d)
    rab = R.rope_append(arena, 0, rope, (qa.float() + qb.float()).half(), k, v).float().view(batch, n_q, chunk, d)
    x = qa.float().view(batch, n_q, chunk, d)
    pair = lambda t: t[..., : d // 2] ** 2 + t[..., d // 2:] ** 2
    assert torch.allclose(pair(ra), pair(x), rtol=6e-3, atol=6e-3)
    assert torch.allclose(ra + rb, rab, rtol=0, atol=2e-2)
    assert arena.device_status() == 0
    # v is a bit copy into the page slots of positions 512 + 80 .. 512 + 95 of sequence 3
    pg = int(seqs[3].block_table()[chunk // 16 + 5])
    gk, gv = arena.export_page(0, pg)
    assert np.array_equal(gv, v.view(batch, n_kv, chunk, d)[3, :, 80:96].cpu().numpy().view(np.uint16))
    kr = gk.view(np.float16).astype(np.float32)
    kx = k.view(batch, n_kv, chunk, d)[3, :, 80:96].float().cpu().numpy()
    assert np.allclose(kr[..., : d // 2] ** 2 + kr[..., d // 2:] ** 2, kx[..., : d // 2] ** 2 + kx[..., d // 2:] ** 2, rtol=6e-3, atol=6e-3)


def causal_rows_f64(q_rows, k, v, scale, q_pos, window=None):
    """q_rows [n, d] at absolute position q_pos; k/v [L, d] with L > q_pos: keys 0..q_pos are visible
    (bottom-right aligned causal mask, kv.rs:247-251), with a window only (q_pos - w, q_pos] (kv.rs:252-257)."""
    lo = 0 if window is None else max(0, q_pos - window + 1)
    kk, vv = k[lo:q_pos + 1].astype(np.float64), v[lo:q_pos + 1].astype(np.float64)
    s = (q_rows.astype(np.float64) @ kk.T) * scale
    s -= s.max(-1, keepdims=True)
    p = np.exp(s)
    return (p / p.sum(-1, keepdims=True)) @ vv


@pytest.mark.parametrize("chunk_kernel", [3, 2, 1])
def test_cfg4_chunked_prefill_at_full_context(chunk_kernel):
    """The cfg4 shape at its real length: Llama-3-8B geometry, prompts of 8192 tokens in 16 chunks of 512
    (one layer, two prompts).  After chunks 0, 7 and 15 a handful of (prompt, kv head, query row) triples
    are recomputed in float64 from host copies of K and V; the last chunk is repeated with a window."""
    n_q, n_kv, d, batch, prompt, chunk = 32, 8, 128, 2, 8192, 512
    rep, scale = n_q // n_kv, d ** -0.5
    arena = KVArena(1, n_q, n_kv, d, prompt + 64, 16, batch * (prompt // 16 + 4), sliding_popn_refuses=False)
    arena.set_free_list(np.random.default_rng(44).permutation(arena.num_pages))
    arena.set_chunk_kernel(chunk_kernel)
    seqs = [arena.new_seq() for _ in range(batch)]
    gen = torch.Generator(device="cuda").manual_seed(0xC0B50004 + chunk_kernel)
    K = np.zeros((batch, n_kv, prompt, d), np.float16)
    V = np.zeros_like(K)
    rng = np.random.default_rng(chunk_kernel)
    ntok = batch * chunk

    def check(c, q, out, window=None):
        qh = q.cpu().numpy().reshape(batch, n_q, chunk, d)
        oh = out.cpu().numpy().reshape(batch, n_q, chunk, d)
        rows = [0, 1, 127, 128, 300, chunk - 1] + [int(x) for x in rng.integers(0, chunk, 3)]
        for r in rows:
            b, h = int(rng.integers(batch)), int(rng.integers(n_kv))
            ref = causal_rows_f64(qh[b, h * rep:(h + 1) * rep, r], K[b, h], V[b, h], scale, c * chunk + r, window)
            assert_attention_close(oh[b, h * rep:(h + 1) * rep, r], ref, f"chunk {c} prompt {b} kv head {h} row {r} window {window}")

    for c in range(prompt // chunk):
        q = torch.randn(ntok * n_q * d, device="cuda", generator=gen).half()
        k = torch.randn(ntok * n_kv * d, device="cuda", generator=gen).half()
        v = torch.randn(ntok * n_kv * d, device="cuda", generator=gen).half()
        K[:, :, c * chunk:(c + 1) * chunk] = k.cpu().numpy().reshape(batch, n_kv, chunk, d)
        V[:, :, c * chunk:(c + 1) * chunk] = v.cpu().numpy().reshape(batch, n_kv, chunk, d)
        arena.begin_step(seqs, [chunk] * batch, [c * chunk] * batch)
        out = arena.attention(0, q, k, v, scale)
        if c in (0, 7, 15):
            assert arena.device_status() == 0
            check(c, q, out)
    # the last chunk once more with a sliding window (keys (p - 1000, p]): same pages, paged attention only
    for s in seqs:
        assert s.popn(chunk) == chunk
    arena.begin_step(seqs, [chunk] * batch)
    arena.append(0, k, v)
    out = arena.paged_attention(0, q, scale, 1000)
    assert arena.device_status() == 0
    check(prompt // chunk - 1, q, out, window=1000)
    # pages of the last chunk hold exactly what was appended
    tbl = seqs[1].block_table()
    gk, gv = arena.export_page(0, int(tbl[-1]))
    assert np.array_equal(gk, K[1, :, -16:].view(np.uint16)) and np.array_equal(gv, V[1, :, -16:].view(np.uint16))


@pytest.mark.parametrize("chunk_kernel", [3, 2])
def test_chunk_attention_beyond_the_staged_block_table(chunk_kernel):
    """A context longer than the 2560 block-table entries the tensor-core chunk kernels stage in shared
    memory (40960 tokens): the entries past them are read from global memory while the kernel runs."""
    n_q, n_kv, d, ctx, chunk = 4, 1, 128, 41472, 512
    scale = d ** -0.5
    arena = KVArena(1, n_q, n_kv, d, ctx + chunk, 16, (ctx + chunk) // 16 + 8)
    arena.set_free_list(np.random.default_rng(45).permutation(arena.num_pages))
    arena.set_chunk_kernel(chunk_kernel)
    seq = arena.new_seq()
    gen = torch.Generator(device="cuda").manual_seed(45)
    kf = torch.randn(ctx * n_kv * d, device="cuda", generator=gen).half()
    vf = torch.randn(ctx * n_kv * d, device="cuda", generator=gen).half()
    arena.begin_step([seq], [ctx])
    arena.append(0, kf, vf)
    q = torch.randn(chunk * n_q * d, device="cuda", generator=gen).half()
    k = torch.randn(chunk * n_kv * d, device="cuda", generator=gen).half()
    v = torch.randn(chunk * n_kv * d, device="cuda", generator=gen).half()
    arena.begin_step([seq], [chunk], [ctx])
    out = arena.attention(0, q, k, v, scale).cpu().numpy().reshape(n_q, chunk, d)
    assert arena.device_status() == 0
    K = np.concatenate([kf.cpu().numpy().reshape(ctx, d), k.cpu().numpy().reshape(chunk, d)])
    V = np.concatenate([vf.cpu().numpy().reshape(ctx, d), v.cpu().numpy().reshape(chunk, d)])
    qh = q.cpu().numpy().reshape(n_q, chunk, d)
    for r in (0, 255, 256, chunk - 1):
        assert_attention_close(out[:, r], causal_rows_f64(qh[:, r], K, V, scale, ctx + r), f"row {r}")
    # the same chunk through a window that starts beyond the staged entries' reach as well
    assert seq.popn(chunk) == chunk
    arena.begin_step([seq], [chunk], [ctx])
    out = arena.attention(0, q, k, v, scale, 41000).cpu().numpy().reshape(n_q, chunk, d)
    assert arena.device_status() == 0
    for r in (0, chunk - 1):
        assert_attention_close(out[:, r], causal_rows_f64(qh[:, r], K, V, scale, ctx + r, 41000), f"window row {r}")
