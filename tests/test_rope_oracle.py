"""The rotary/QK-norm oracle against the known-answer tests the reference keeps beside the code it
restates (engine/core/combs-models/src/rope.rs:211-330)."""
import math

import numpy as np

import oracle


def test_tables_match_known_math():          # rope.rs:215-244
    cos, sin = oracle.rope_tables(8, 10000.0, 4)
    inv = [1.0, 0.1, 0.01, 0.001]
    for pos in range(4):
        for i in range(4):
            angle = pos * inv[i]
            for idx in (i, i + 4):           # half-split layout: i and i + half share the frequency
                assert abs(float(cos[pos, idx]) - math.cos(angle)) < 1e-5
                assert abs(float(sin[pos, idx]) - math.sin(angle)) < 1e-5
    assert np.all(np.abs(cos[0] - 1.0) < 1e-6) and np.all(np.abs(sin[0]) < 1e-6)


def test_linear_scaling_divides_frequencies():   # rope.rs:248-256
    inv, ms = oracle.rope_inv_freq(8, 10000.0, {"kind": "linear", "factor": 2.0})
    assert np.all(np.abs(inv - np.array([0.5, 0.05, 0.005, 0.0005])) < 1e-12) and ms == 1.0


def test_llama3_scaling_matches_reference():     # rope.rs:258-283
    inv, ms = oracle.rope_inv_freq(64, 500000.0, {"kind": "llama3", "factor": 32.0, "low_freq_factor": 1.0,
                                                   "high_freq_factor": 4.0, "original_max_position_embeddings": 8192})
    for i, e in [(0, 1.0), (8, 0.037606030931), (16, 0.000429556797), (24, 1.661967e-06), (31, 9.4183e-08)]:
        assert abs((inv[i] - e) / e) < 1e-6, (i, inv[i])
    assert ms == 1.0


def test_yarn_scaling_matches_reference():       # rope.rs:285-309
    inv, ms = oracle.rope_inv_freq(128, 1e6, {"kind": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768,
                                              "beta_fast": 32.0, "beta_slow": 1.0})
    for i, e in [(0, 1.0), (16, 0.03162277660168379), (32, 0.0006029411764705882), (48, 7.905694150420949e-06),
                 (63, 3.102344401879299e-07)]:
        assert abs((inv[i] - e) / e) < 1e-6, (i, inv[i])
    assert abs(ms - 1.138629436112) < 1e-9


def test_longrope_scaling_matches_reference():   # rope.rs:311-346
    sc = {"kind": "longrope", "short_factor": [1.0, 2.0, 4.0, 8.0], "original_max_position_embeddings": 4096, "factor": 32.0}
    inv, ms = oracle.rope_inv_freq(8, 10000.0, sc)
    assert np.all(np.abs(inv - np.array([1.0, 0.05, 0.0025, 0.000125])) < 1e-15)
    assert abs(ms - math.sqrt(17.0 / 12.0)) < 1e-12
    sc = {"kind": "longrope", "short_factor": [1.0] * 4, "original_max_position_embeddings": 4096, "factor": 1.0}
    assert oracle.rope_inv_freq(8, 10000.0, sc)[1] == 1.0


def test_scaled_tables_apply_mscale():           # rope.rs:348-362
    cos, sin = oracle.rope_tables(8, 10000.0, 2, {"kind": "yarn", "factor": 4.0, "original_max_position_embeddings": 32768,
                                                  "beta_fast": 32.0, "beta_slow": 1.0, "attention_factor": 1.25})
    assert abs(float(cos[0, 0]) - 1.25) < 1e-6 and abs(float(sin[0, 0])) < 1e-6


def test_apply_is_a_rotation_and_position_zero_is_identity():
    rng = np.random.default_rng(3)
    cos, sin = oracle.rope_tables(64, 10000.0, 40)
    x = rng.standard_normal((3, 7, 64)).astype(np.float32)
    assert np.array_equal(oracle.rope_apply(x[:, :1], 0, cos, sin), x[:, :1])
    y = oracle.rope_apply(x, 5, cos, sin)
    assert np.allclose(np.linalg.norm(y, axis=-1), np.linalg.norm(x, axis=-1), rtol=1e-5)
    # against the textbook complex form on the (i, i + half) pairs
    z = x[..., :32] + 1j * x[..., 32:]
    ang = (np.arange(5, 12)[:, None] * (10000.0 ** (-2.0 * np.arange(32) / 64)))[None]
    zr = z * np.exp(1j * ang)
    assert np.allclose(y[..., :32], zr.real, atol=1e-5) and np.allclose(y[..., 32:], zr.imag, atol=1e-5)


def test_rms_norm_flavours():
    rng = np.random.default_rng(4)
    x = rng.standard_normal((5, 128)).astype(np.float32)
    w = rng.standard_normal(128).astype(np.float32) * 0.1
    ref = x / np.sqrt((x.astype(np.float64) ** 2).mean(-1, keepdims=True) + 1e-6)
    assert np.allclose(oracle.rms_norm(x, w, 1e-6), ref * w, atol=1e-5)
    assert np.allclose(oracle.rms_norm(x, w, 1e-6, gemma=True), ref * (1 + w), atol=1e-5)
    xh = x.astype(np.float16)
    assert np.allclose(oracle.rms_norm(xh, w.astype(np.float16), 1e-6).astype(np.float32), ref * w, atol=4e-3)
