"""CPU tests: the oracle against the golden vectors and against its own numpy twin."""
import hashlib
from pathlib import Path

import numpy as np
import pytest

from oracle import exl3_oracle as O

GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.mark.parametrize("rate", [3, 4, 6])
def test_decode_matches_reference_golden(oracle, rate):
    g = np.load(GOLDEN / f"decode_k{rate}.npz")
    rows, cols = int(g["rows"]), int(g["cols"])
    want = g["fp16_bits"]
    assert (oracle.decode_matrix(g["data"], rows, cols, rate) == want).all()
    assert (O.decode_matrix_bits(g["data"], rows, cols, rate) == want).all()


def test_mul1_codebook_all_states(oracle):
    g = np.load(GOLDEN / "mul1.npz")
    states = np.arange(65536, dtype=np.uint32)
    table = O.mul1_bits(states)
    assert hashlib.sha256(table.tobytes()).digest() == g["table_sha256"].tobytes()
    c_table = np.array([oracle.lib.exl3_mul1_bits(int(s)) for s in states], dtype=np.uint16)
    assert (c_table == table).all()
    assert (table[g["samples"]] == g["sample_bits"]).all()
    v = table.view(np.float16).astype(np.float64)
    assert abs(v.mean()) < 5e-3 and abs(v.std() - 1.0) < 5e-3 and np.abs(v).max() < 3.6


def test_tile_permutation_is_a_permutation(oracle):
    perm = O.tile_permutation()
    assert sorted(perm.reshape(-1).tolist()) == list(range(256))
    for i in range(16):
        for o in range(16):
            assert oracle.lib.exl3_index(i, o) == perm[i, o]
    # the 32 positions of one output row-pair are contiguous: what the kernels' lane ownership relies on
    for g in range(8):
        rows = perm[:, [g, g + 8]].reshape(-1)
        assert sorted(rows.tolist()) == list(range(32 * g, 32 * g + 32))


@pytest.mark.skipif(not O.RefWeight.available(), reason="reference decoder library not built (needs the reference checkout)")
@pytest.mark.parametrize("rate", [3, 4, 6])
def test_decode_matches_reference_source_on_host(oracle, rate):
    ref = O.RefWeight()
    rng = np.random.Generator(np.random.Philox(key=rate))
    data, _, _ = O.synthetic_matrix(rng, 64, 128, rate)
    ours = oracle.decode_matrix(data, 64, 128, rate).view(np.float16).astype(np.float32)
    assert (ours == ref.decode_matrix(data, 64, 128, rate)).all()


def test_bf16_and_fp16_conversions(oracle):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1.0, 300.0, 7e4)])
    x = np.concatenate([x, np.array([0.0, -0.0, 65504.0, 65519.9, 65520.0, 6e-8, 2.98e-8, 2.9802322e-8, np.inf, -np.inf], np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = np.array([oracle.lib.exl3_f32_to_f16_bits(float(v)) for v in x], dtype=np.uint16)
    assert (got == want).all()
    back = np.array([oracle.lib.exl3_f16_bits_to_f32(int(h)) for h in want[:2000]], dtype=np.float32)
    assert (back == want[:2000].view(np.float16).astype(np.float32)).all()
    twin = O.bf16_round(x[np.isfinite(x)])
    c = np.array([oracle.lib.exl3_bf16_round(float(v)) for v in x[np.isfinite(x)]], dtype=np.float32)
    assert (twin.view(np.uint32) == c.view(np.uint32)).all()
    assert ((twin.view(np.uint32) & 0xFFFF) == 0).all()


def test_linear_golden_and_forms_agree(oracle):
    g = np.load(GOLDEN / "layer_math.npz")
    rows, cols, rate = int(g["rows"]), int(g["cols"]), int(g["rate"])
    m = oracle.matrix(g["data"], g["suh"], g["svh"], rows, cols, rate)
    y, bad = oracle.linear(m, g["x"])
    assert not bad and (y.view(np.uint32) == g["y"].view(np.uint32)).all()
    y16, bad = oracle.linear(m, g["x"], f16_form=True)
    assert not bad
    y64 = O.linear_f64(g["data"], rows, cols, rate, g["suh"], g["svh"], g["x"])
    scale = np.abs(y64).max()
    assert np.abs(y - y64).max() / scale < 4e-3  # at most one BF16 step
    assert np.abs(y16 - y64).max() / scale < 4e-3
    xt, bad = oracle.input_had(m, g["x"])
    assert not bad and (xt == O.input_had(g["x"], g["suh"])).all()


def test_hadamard_is_orthonormal_and_self_inverse():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((3, 128)).astype(np.float32)
    h = O.hadamard128(x)
    assert np.allclose(O.hadamard128(h), x, atol=1e-5)
    assert np.allclose((h ** 2).sum(-1), (x ** 2).sum(-1), rtol=1e-5)


def test_silu_table_and_routing_golden(oracle):
    g = np.load(GOLDEN / "layer_math.npz")
    table = oracle.silu_table()
    assert hashlib.sha256(table.tobytes()).digest() == g["silu_sha256"].tobytes()
    assert (table[::257] == g["silu_samples"]).all()
    bits = np.array([0x3F80, 0xBF80, 0x0000, 0x4040], dtype=np.uint16)  # 1, -1, 0, 3
    vals = (table[bits].astype(np.uint32) << 16).view(np.float32)
    expect = np.array([1 / (1 + np.exp(-1.0)), -1 / (1 + np.exp(1.0)), 0.0, 3 / (1 + np.exp(-3.0))])
    assert np.allclose(vals, expect, rtol=4e-3, atol=1e-6)
    ids, w, bad = oracle.route(g["logits"])
    assert not bad and (ids == g["route_ids"]).all() and (w == g["route_weights"]).all()
    assert (np.diff(ids, axis=1) > 0).all() and np.allclose(w.sum(1), 1.0, atol=2e-2)
    # top-8 really are the eight largest logits
    for t in range(ids.shape[0]):
        assert set(ids[t].tolist()) == set(np.argsort(-g["logits"][t], kind="stable")[:8].tolist())


def test_activate_and_combine_follow_bf16_boundaries(oracle):
    import ctypes as C

    rng = np.random.default_rng(2)
    gate = O.bf16_round(rng.standard_normal(512).astype(np.float32) * 3)
    up = O.bf16_round(rng.standard_normal(512).astype(np.float32))
    g2 = gate.copy()
    bad = oracle.lib.exl3_activate(g2.ctypes.data_as(C.POINTER(C.c_float)), up.ctypes.data_as(C.POINTER(C.c_float)), 512)
    assert not bad
    table = oracle.silu_table()
    silu = (table[(gate.view(np.uint32) >> 16)].astype(np.uint32) << 16).view(np.float32)
    assert (g2 == O.bf16_round(silu * up)).all()
    hidden = 256
    x = O.bf16_round(rng.standard_normal(hidden).astype(np.float32))
    down = O.bf16_round(rng.standard_normal((8, hidden)).astype(np.float32))
    w = O.bf16_round(rng.uniform(0.05, 0.3, 8).astype(np.float32))
    want = np.zeros(hidden, np.float32)
    for s in range(8):
        want = O.bf16_round(want + O.bf16_round(down[s] * w[s]))
    want = O.bf16_round(x + want)
    got = x.copy()
    f = lambda a: a.ctypes.data_as(C.POINTER(C.c_float))
    assert not oracle.lib.exl3_combine(f(got), f(down), f(w), hidden)
    assert (got == want).all()


def test_group_and_schedule(oracle):
    rng = np.random.default_rng(3)
    for tokens in (1, 4, 33, 257):
        ids = np.stack([np.sort(rng.choice(64, 8, replace=False)) for _ in range(tokens)]).astype(np.int32)
        groups, counts, bad = oracle.group(ids, tokens)
        assert not bad and counts.sum() == tokens * 8
        for e in range(64):
            mine = groups[e * tokens: e * tokens + counts[e]]
            assert (np.diff(mine) > 0).all() and (ids.reshape(-1)[mine] == e).all()
        tiles, bad = oracle.schedule(counts, tokens)
        assert not bad and tiles[:, 2].sum() == tokens * 8 and (tiles[:, 2] <= 32).all() and (tiles[:, 2] >= 1).all()
        assert (np.diff(tiles[:, 0]) >= 0).all()
    dup = np.tile(np.arange(8, dtype=np.int32), (2, 1))
    dup[1, 1] = 0
    assert oracle.group(dup, 2)[2] == 1  # a token may not use an expert twice
    assert oracle.schedule(np.zeros(64, np.int32), 4)[1] == 1  # counts must add up to tokens*8


def test_moe_layer_small(oracle):
    """One tiny layer (hidden 256, inter 128): the composed layer equals its parts."""
    host = O.HostMatrices(1, 256, 128, 4, seed=5)
    rng = np.random.default_rng(4)
    x = O.bf16_round(rng.standard_normal((2, 256)).astype(np.float32))
    ids, w, _ = oracle.route(O.bf16_round(rng.standard_normal((2, 64)).astype(np.float32)))
    out, bad, caps = oracle.moe_layer(host.table, 0, ids, w, x, 256, 128, capture=True)
    assert not bad and np.isfinite(out).all() and (out != x).any()
    e = int(ids[1, 3])
    data, suh, svh = host.get(0, e, 1)
    m = oracle.matrix(data, suh, svh, 128, 256, 4)
    y, _ = oracle.linear(m, x[1])
    assert (caps[1][1 * 8 + 3] == y).all()
    out16, bad16 = oracle.moe_layer(host.table, 0, ids, w, x, 256, 128, f16_form=True)
    assert not bad16
    assert np.abs(out - out16).max() <= 1e-2 * np.abs(out).max()


def test_norm_restatements_against_float64(oracle):
    """The compensated RMS norms of the oracle against a float64 evaluation of the same formulas: the variance and the
    inverse root to FP32 rounding, x exactly, normalized within one BF16 step per rounding (two roundings)."""
    rng = np.random.default_rng(5)
    hidden, rows = 2304, 3
    x = O.bf16_round((3.0 * rng.standard_normal((rows, hidden))).astype(np.float32))
    residual = O.bf16_round(rng.standard_normal((rows, hidden)).astype(np.float32))
    wb = (O.bf16_round((1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)).view(np.uint32) >> 16).astype(np.uint16)
    weight = (wb.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    got_x, got_n, stats, bad = oracle.residual_norm(x, residual, wb)
    assert not bad
    want_x = O.bf16_round((x.astype(np.float64) + residual).astype(np.float32))
    assert np.array_equal(got_x, want_x)
    variance = (want_x.astype(np.float64) ** 2).mean(axis=1)
    inv = 1.0 / np.sqrt(variance + 1e-6)
    assert np.allclose(stats[:, 0], variance, rtol=3e-7) and np.allclose(stats[:, 1], inv, rtol=3e-7)
    want_n = want_x.astype(np.float64) * inv[:, None] * weight
    assert np.allclose(got_n, want_n, rtol=2 ** -7, atol=1e-30)
    # the fused combine + norm equals combine followed by the norm without a residual
    down = O.bf16_round((4.0 * rng.standard_normal((rows, 8, hidden))).astype(np.float32))
    routing = O.bf16_round(np.full((rows, 8), 0.125, dtype=np.float32))
    fused_x, fused_n, fused_s, bad = oracle.combine_norm(x, down, routing, wb)
    step_x, bad2 = oracle.combine(x, down, routing)
    step_x, step_n, step_s, bad3 = oracle.residual_norm(step_x, None, wb)
    assert not (bad or bad2 or bad3)
    assert np.array_equal(fused_x, step_x) and np.array_equal(fused_n, step_n) and np.array_equal(fused_s, step_s)
