"""Shared driver for the GPU parity tests: runs one history on the CUDA path
(through the C ABI) and on the oracle, on identical seeded f16 inputs."""
from __future__ import annotations

import numpy as np
import torch

from combsengine_b200 import KVArena
from oracle import OracleArena

ATOL, RTOL = 2e-3, 1e-2  # f16 storage, f32 accumulation


def assert_attention_close(got: np.ndarray, ref: np.ndarray, what: str = "") -> None:
    """|got - ref| <= 2e-3 + 1e-2 |ref| element-wise, and 2e-3 relative in the Frobenius norm."""
    g, r = got.astype(np.float64), ref.astype(np.float64)
    assert np.isfinite(g).all(), f"{what}: non-finite output"
    err = np.abs(g - r)
    bad = err > ATOL + RTOL * np.abs(r)
    assert not bad.any(), f"{what}: max err {err.max():.3e} at {np.unravel_index(err.argmax(), err.shape)}"
    denom = np.linalg.norm(r)
    if denom > 0:
        assert np.linalg.norm(g - r) / denom < 2e-3, f"{what}: relative error {np.linalg.norm(g - r) / denom:.3e}"


class Pair:
    """A CUDA arena and an oracle arena kept in lock-step."""

    def __init__(self, layers, n_q, n_kv, d, max_seq_len, num_pages=0, page_size=16, windows=None, seed=0,
                 shuffle_free_list=False, popn_refuses=True, tuning=None, chunk_kernel=None, quantize_kv=False):
        self.layers, self.n_q, self.n_kv, self.d = layers, n_q, n_kv, d
        self.g = KVArena(layers, n_q, n_kv, d, max_seq_len, page_size, num_pages, windows,
                         sliding_popn_refuses=popn_refuses, quantize_kv=quantize_kv)
        # sliding layers live in pages on both sides so that page contents can be compared
        self.o = OracleArena(layers, n_kv, d, max_seq_len, page_size, num_pages, windows=windows, rolling=False, dtype="f16",
                             quantize_kv=quantize_kv)
        self.windows = windows
        if tuning:
            self.g.set_decode_tuning(**tuning)
        if chunk_kernel is not None:
            self.g.set_chunk_kernel(chunk_kernel)
        self.rng = np.random.default_rng(seed)
        self.seqs = []
        if shuffle_free_list:
            perm = self.rng.permutation(self.g.num_pages)
            self.g.set_free_list(perm)
            self.o.set_free_list(perm)

    def new_seq(self):
        pair = (self.g.new_seq(), self.o.new_seq())
        self.seqs.append(pair)
        return pair

    def fork(self, pair, n_tokens):
        child = (pair[0].fork_prefix(n_tokens), pair[1].fork_prefix(n_tokens))
        self.seqs.append(child)
        return child

    def drop(self, pair):
        self.seqs.remove(pair)
        pair[0].close()
        pair[1].close()

    def rand(self, heads, tokens):
        return self.rng.standard_normal((heads, tokens, self.d)).astype(np.float16)

    def step(self, pairs, new_tokens, scale=None, window=None, fused=True, check=True, layers=None):
        """One forward pass over `pairs`; returns the CUDA outputs per layer (packed)."""
        scale = 1.0 / np.sqrt(self.d) if scale is None else scale
        gs, os_ = [p[0] for p in pairs], [p[1] for p in pairs]
        pos = [s.seq_len() for s in gs]
        self.g.begin_step(gs, new_tokens, pos)
        self.o.batch_begin(os_, new_tokens)
        outs = []
        for layer in (range(self.layers) if layers is None else layers):
            q = [self.rand(self.n_q, n) for n in new_tokens]
            k = [self.rand(self.n_kv, n) for n in new_tokens]
            v = [self.rand(self.n_kv, n) for n in new_tokens]
            pk = lambda xs: np.concatenate([x.reshape(-1) for x in xs])
            qd, kd, vd = (torch.from_numpy(pk(x)).cuda() for x in (q, k, v))
            if fused:
                out = self.g.attention(layer, qd, kd, vd, scale, window)
            else:
                self.g.append(layer, kd, vd)
                out = self.g.paged_attention(layer, qd, scale, window)
            got = out.cpu().numpy()
            assert self.g.device_status() == 0
            if check:
                ref = self.o.batch_layer(os_, new_tokens, layer, pk(q), pk(k), pk(v), self.n_q, scale, window)
                assert_attention_close(got, ref, f"layer {layer} new_tokens {list(new_tokens)[:4]}")
            else:
                self.o.batch_layer(os_, new_tokens, layer, pk(q), pk(k), pk(v), self.n_q, scale, window)
            outs.append(got)
        return outs

    def assert_state_equal(self, pages="all"):
        """Bit-exact: block tables, free-list order, refcounts and page contents."""
        assert list(self.g.free_list()) == list(self.o.free_list())
        used = set()
        for gs, os_ in self.seqs:
            assert gs.seq_len() == os_.seq_len()
            assert list(gs.block_table()) == list(os_.block_table())
            used.update(int(x) for x in gs.block_table())
        check = range(self.g.num_pages) if pages == "all" else sorted(used)
        for layer in range(self.layers):
            for pg in check:
                if self.g.layer_is_quantized(layer):  # packed words and scales, bit for bit
                    got, want = self.g.export_page_quant(layer, pg), self.o.page_quant(layer, pg)
                    for name, x, y in zip(("K words", "K scales", "V words", "V scales"), got, want):
                        y = y if y.dtype == np.int32 else y.view(np.uint16)
                        assert np.array_equal(x, y), f"{name} of page {pg} layer {layer}"
                    continue
                gk, gv = self.g.export_page(layer, pg)
                ok, ov = self.o.page(layer, pg)
                assert np.array_equal(gk, ok.view(np.uint16)), f"K page {pg} layer {layer}"
                assert np.array_equal(gv, ov.view(np.uint16)), f"V page {pg} layer {layer}"
        for pg in range(self.g.num_pages):
            assert self.g.refcount(pg) == self.o.refcount(pg)
