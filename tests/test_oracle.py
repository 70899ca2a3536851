"""CPU tests of the oracle itself: the C restatement is checked against (a) independent float64
numpy formulas, (b) its own per-preset restatements of the reference's test lambdas, and (c) the
golden fixtures the reference's Python produced (tests/golden/make_golden.py)."""
import json
import os

import numpy as np
import pytest

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _rand_bf16(o, rng, shape, scale=1.0):
    return o.f32_to_bf16((rng.standard_normal(shape) * scale).astype(np.float32))


def _f(o, bits):
    return o.bf16_to_f32(bits)


def test_bf16_round_to_nearest_even(oracle):
    o = oracle
    # 1 + 2^-8 is a tie between 1.0 (even mantissa) and 1+2^-7: RNE picks 1.0
    x = np.array([1.0, 1.0 + 2 ** -8, 1.0 + 2 ** -8 + 2 ** -16, 1.0 + 3 * 2 ** -8, -2.5, 0.0,
                  3.4028234663852886e38], dtype=np.float32)
    b = o.f32_to_bf16(x)
    back = o.bf16_to_f32(b)
    assert back[0] == 1.0
    assert back[1] == 1.0                      # tie -> even
    assert back[2] == np.float32(1.0 + 2 ** -7)  # just above the tie -> up
    assert back[3] == np.float32(1.0 + 2 ** -6)  # tie with odd lower neighbour -> up to even
    assert back[4] == -2.5 and back[5] == 0.0
    assert np.isinf(back[6])                   # rounds past the largest finite bf16
    # matches torch's conversion on random data
    import torch
    r = np.random.default_rng(0).standard_normal(4096).astype(np.float32) * 37.0
    tb = torch.from_numpy(r).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(o.f32_to_bf16(r), tb)


def test_gemm_bf16_against_float64(oracle):
    o = oracle
    rng = np.random.default_rng(1)
    for (M, N, K) in [(5, 7, 9), (33, 130, 257), (64, 2050, 128)]:
        A = _rand_bf16(o, rng, (M, K))
        B = _rand_bf16(o, rng, (K, N), K ** -0.5)
        C = o.gemm_bf16(A, B)
        ref = _f(o, A).astype(np.float64) @ _f(o, B).astype(np.float64)
        assert np.abs(C - ref).max() < 1e-4 * max(1.0, np.abs(ref).max())


def test_gemm_s8_exact(oracle):
    o = oracle
    rng = np.random.default_rng(2)
    for (M, N, K) in [(3, 5, 7), (37, 129, 300), (8, 2049, 64)]:
        A = rng.integers(-128, 128, (M, K), dtype=np.int8)
        B = rng.integers(-128, 128, (K, N), dtype=np.int8)
        C = o.gemm_s8(A, B)
        assert np.array_equal(C, (A.astype(np.int64) @ B.astype(np.int64)).astype(np.int32))


def test_gemm_s8_extreme_values_no_overflow(oracle):
    # |acc| <= K*128*128: all -128 x -128 at K=1024 stays far below 2^31
    A = np.full((2, 1024), -128, np.int8)
    B = np.full((1024, 3), -128, np.int8)
    assert (oracle.gemm_s8(A, B) == 1024 * 16384).all()


@pytest.fixture(scope="module")
def small(oracle):
    rng = np.random.default_rng(3)
    M, N, K = 24, 64, 48
    A = _rand_bf16(oracle, rng, (M, K))
    B = _rand_bf16(oracle, rng, (K, N), K ** -0.5)
    acc = oracle.gemm_bf16(A, B)
    d = dict(M=M, N=N, K=K, acc=acc, rng=rng,
             scale=rng.uniform(0.5, 1.5, M).astype(np.float32),
             gamma=rng.uniform(0.8, 1.2, N).astype(np.float32),
             bias=rng.normal(0, 0.02, N).astype(np.float32),
             residual=_rand_bf16(oracle, rng, (M, N)),
             cos_sin=oracle.rope_table(M, N, 10000.0))
    return d


def test_flat_program_equals_preset_lambdas(oracle, small):
    """The canonical step order reproduces every preset formula bit for bit."""
    o, s = oracle, small
    acc = s["acc"]
    assert np.array_equal(o.epilogue(acc, row=s["scale"]), o.preset_k1(acc, s["scale"]))
    assert np.array_equal(o.epilogue(acc, row=s["scale"], pair="swiglu"), o.preset_k2(acc, s["scale"]))
    assert np.array_equal(o.epilogue(acc, row=s["scale"], pair="geglu"),
                          o.preset_k2(acc, s["scale"], geglu=True))
    assert np.array_equal(o.epilogue(acc, pair="rope", cos_sin=s["cos_sin"]),
                          o.preset_k4(acc, None, s["cos_sin"]))
    assert np.array_equal(o.epilogue(acc, row=s["scale"], pair="rope", cos_sin=s["cos_sin"]),
                          o.preset_k4(acc, s["scale"], s["cos_sin"]))
    assert np.array_equal(o.epilogue(acc, residual=s["residual"], col=s["gamma"]),
                          o.preset_k0a(acc, s["residual"], s["gamma"]))
    acc_i = (acc * 1000).astype(np.int32)
    st = s["scale"] * 0.01
    sc = s["gamma"] * 0.01
    assert np.array_equal(o.epilogue(acc_i, row=st, col=sc), o.preset_w8a8(acc_i, st, sc))
    assert np.array_equal(o.epilogue(acc_i, row=st, col=sc, bias=s["bias"]),
                          o.preset_w8a8(acc_i, st, sc, s["bias"]))


def test_epilogue_against_float64_formulas(oracle, small):
    o, s = oracle, small
    acc = s["acc"].astype(np.float64)
    R = s["scale"].astype(np.float64)[:, None]
    # k2 compact: silu(gate*R) * (up*R)
    x = acc * R
    g, u = x[:, 0::2], x[:, 1::2]
    want = g / (1 + np.exp(-g)) * u
    _, got = o.epilogue(s["acc"], row=s["scale"], pair="swiglu", compact=True, want_f32=True)
    assert got.shape == (s["M"], s["N"] // 2)
    assert np.abs(got - want).max() < 1e-5
    # duplicated layout holds the same value in both columns of a pair
    _, dup = o.epilogue(s["acc"], row=s["scale"], pair="swiglu", want_f32=True)
    assert np.array_equal(dup[:, 0::2], dup[:, 1::2]) and np.allclose(dup[:, 0::2], got)
    # rope with a per-head table (period 16) equals rope with the table tiled across N
    P = 16
    tab = o.rope_table(s["M"], P, 500000.0)
    full = np.tile(tab, (1, s["N"] // P))
    a = o.epilogue(s["acc"], row=s["scale"], pair="rope", cos_sin=tab, cos_sin_period=P)
    b = o.epilogue(s["acc"], row=s["scale"], pair="rope", cos_sin=full)
    assert np.array_equal(a, b)
    c, sn = full[:, 0::2].astype(np.float64), full[:, 1::2].astype(np.float64)
    e, od = x[:, 0::2], x[:, 1::2]
    _, rf = o.epilogue(s["acc"], row=s["scale"], pair="rope", cos_sin=full, want_f32=True)
    assert np.abs(rf[:, 0::2] - (e * c + od * sn)).max() < 1e-5
    assert np.abs(rf[:, 1::2] - (-e * sn + od * c)).max() < 1e-5
    # rotation preserves the norm of each pair
    assert np.allclose(rf[:, 0::2] ** 2 + rf[:, 1::2] ** 2, e ** 2 + od ** 2, rtol=1e-4, atol=1e-6)
    # unary activations
    from math import erf
    for name, fn in [("gelu", lambda v: v * 0.5 * (1 + np.vectorize(erf)(v / np.sqrt(2)))),
                     ("gelu_tanh", lambda v: v * 0.5 * (1 + np.tanh(0.7978845608028654 * (v + 0.044715 * v ** 3)))),
                     ("silu", lambda v: v / (1 + np.exp(-v))),
                     ("relu", lambda v: np.maximum(v, 0)),
                     ("sigmoid", lambda v: 1 / (1 + np.exp(-v)))]:
        y = acc + s["bias"].astype(np.float64)[None, :]
        _, got = o.epilogue(s["acc"], bias=s["bias"], unary=name, want_f32=True)
        assert np.abs(got - fn(y)).max() < 1e-5, name
    # dual output: aux holds bf16(acc + residual), D = that fp32 sum * gamma
    d, aux = o.epilogue(s["acc"], residual=s["residual"], col=s["gamma"], want_aux=True)
    sm = s["acc"] + o.bf16_to_f32(s["residual"])
    assert np.array_equal(aux, o.f32_to_bf16(sm))
    assert np.array_equal(d, o.f32_to_bf16(sm * s["gamma"][None, :]))


def test_ragged_and_empty_edges(oracle):
    o = oracle
    # odd N: the last column has no partner and is only scaled (tests/test_k4.cpp:149-152)
    acc = np.arange(15, dtype=np.float32).reshape(3, 5)
    sc = np.array([1.0, 2.0, 0.5], np.float32)
    cs = o.rope_table(3, 6, 10000.0)[:, :5].copy()
    cs_full = np.zeros((3, 5), np.float32)
    cs_full[:, :5] = cs
    out = o.preset_k4(acc, sc, cs_full)
    assert np.array_equal(out[:, 4], o.f32_to_bf16(acc[:, 4] * sc))
    # M = 1 and K = 1 degenerate GEMM
    A = o.f32_to_bf16(np.array([[2.0]], np.float32))
    B = o.f32_to_bf16(np.array([[1.0, -3.0, 0.5]], np.float32))
    assert np.array_equal(o.gemm_bf16(A, B), np.array([[2.0, -6.0, 1.0]], np.float32))


def test_rstd_and_quantisers(oracle):
    o = oracle
    rng = np.random.default_rng(5)
    x = _rand_bf16(o, rng, (9, 200), 3.0)
    xf = _f(o, x).astype(np.float64)
    r = o.compute_rstd(x, 1e-6)
    assert np.allclose(r, 1 / np.sqrt((xf ** 2).mean(axis=1) + 1e-6), rtol=1e-6)
    xq, st = o.rstd_and_quantize(x, r)
    normed = xf * r[:, None]
    assert np.allclose(st, np.abs(normed).max(axis=1) / 127 + 1e-8, rtol=1e-5)
    assert xq.min() >= -128 and xq.max() <= 127 and np.abs(xq).max() == 127
    assert np.abs(xq * st[:, None] - normed).max() <= st.max() * 0.5001 + 1e-6
    # all-zero row: scale is the 1e-8 guard, quantised row is zero
    z = np.zeros((1, 16), np.uint16)
    zq, zs = o.quantize_rows(z)
    assert (zq == 0).all() and zs[0] == np.float32(1e-8)
    # weight columns
    W = _rand_bf16(o, rng, (64, 24), 0.1)
    Wq, sc = o.quantize_weight_cols(W)
    Wf = _f(o, W).astype(np.float64)
    assert np.allclose(sc, np.abs(Wf).max(axis=0) / 127 + 1e-8, rtol=1e-5)
    assert np.abs(Wq * sc[None, :] - Wf).max() <= sc.max() * 0.5001
    # round half AWAY from zero (sycl::round), not half-to-even
    h = o.f32_to_bf16(np.array([[2.5, -2.5, 127.0]], np.float32))  # scale = 1 + 1e-8
    hq, hs = o.quantize_rows(h)
    assert hq.tolist() == [[3, -3, 127]]


def test_offline_quantiser_matches_reference_golden(oracle):
    """Pinned: fixture produced by the reference's quantize_columns()."""
    g = np.load(os.path.join(GOLD, "quantize_columns.npz"))
    Wq, sc = oracle.quantize_columns_offline(g["W"])
    assert np.array_equal(Wq, g["Wq"])
    assert np.array_equal(sc, g["scale"])
    assert sc[7] == np.float32(1e-8) and (Wq[:, 7] == 0).all()


def test_rope_table_matches_reference_generator(oracle):
    # tests/test_k4.cpp:81-92 with theta=10000 over the whole N
    M, N = 7, 12
    cs = oracle.rope_table(M, N, 10000.0)
    for m in range(M):
        for kp in range(N // 2):
            freq = np.float32(1.0) / np.float32(np.power(np.float32(10000.0), np.float32(2.0 * kp / N)))
            ang = np.float32(m) * freq
            assert abs(cs[m, 2 * kp] - np.cos(ang)) < 2e-6
            assert abs(cs[m, 2 * kp + 1] - np.sin(ang)) < 2e-6


def test_golden_fixture_inventory():
    k = json.load(open(os.path.join(GOLD, "kernel_presets.json")))
    assert {"k0a", "k1", "k2", "k2_geglu", "k3", "k4", "k4v2", "w8a8_dequant",
            "w8a8_dequant_biased", "k1v2", "k2v2", "k2v2_geglu"} <= set(k["presets"])
    assert {"sa_scale_rows", "sa_residual_gamma", "sa_swiglu", "sa_rope_scaled"} <= set(k["standalone"])
    t = json.load(open(os.path.join(GOLD, "tile_selector.json")))
    assert len(t["tiles"]) == 30
    m = json.load(open(os.path.join(GOLD, "model_presets.json")))
    assert (m["llama3_70b"]["H"], m["llama3_70b"]["H_kv"], m["llama3_70b"]["I"]) == (8192, 1024, 28672)
    assert (m["llama3_8b"]["H"], m["llama3_8b"]["H_kv"], m["llama3_8b"]["I"]) == (4096, 1024, 14336)
