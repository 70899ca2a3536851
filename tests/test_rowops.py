"""Engine-style stand-alone passes (xf_ve_*): the comparison arm of the reference's generated
pipelines (include/xe-fuse/standalone/vllm_ops.hpp).  The oracle restates the reference's loops;
CPU tests hold the oracle to float64 numpy formulas, GPU tests hold the kernels to the oracle
within one bf16 rounding of the fp32 result."""
import numpy as np
import pytest


def _bf(o, a):
    return o.f32_to_bf16(np.asarray(a, np.float32))


def _f(o, bits):
    return o.bf16_to_f32(bits).astype(np.float64)


def _close(o, got_bits, want_bits, ulps=1.0, atol=1e-6):
    """bf16 results agree within `ulps` roundings of the larger magnitude (2^-8 relative), with an
    absolute floor for values that cancel (erf-GeLU of a large negative gate is 1 + erf(x) with
    erf(x) near -1: the device's and the host's erff differ by an fp32 ulp there)."""
    g, w = _f(o, got_bits), _f(o, want_bits)
    tol = ulps * 2.0 ** -7 * np.maximum(np.abs(g), np.abs(w)) + atol
    bad = np.abs(g - w) > tol
    return int(bad.sum()), float(np.abs(g - w).max())


# ------------------------------------------------------------------ oracle vs float64 formulas (CPU)
def test_oracle_rms_norm_formula(oracle):
    rng = np.random.default_rng(0)
    x, w = _bf(oracle, rng.standard_normal((7, 96))), _bf(oracle, rng.normal(1, 0.1, 96))
    xf, wf = _f(oracle, x), _f(oracle, w)
    want = xf / np.sqrt((xf ** 2).mean(1, keepdims=True) + 1e-6) * wf
    nbad, _ = _close(oracle, oracle.ve_rms_norm(x, w), _bf(oracle, want))
    assert nbad == 0


def test_oracle_fused_add_rms_norm_formula(oracle):
    rng = np.random.default_rng(1)
    x, r = _bf(oracle, rng.standard_normal((5, 64))), _bf(oracle, rng.standard_normal((5, 64)))
    w = _bf(oracle, rng.normal(1, 0.1, 64))
    s = _f(oracle, x) + _f(oracle, r)
    out, res = oracle.ve_fused_add_rms_norm(x, r, w)
    assert np.array_equal(res, _bf(oracle, s))                       # residual = bf16(sum), exactly
    want = _f(oracle, res) / np.sqrt((s ** 2).mean(1, keepdims=True) + 1e-6) * _f(oracle, w)
    assert _close(oracle, out, _bf(oracle, want))[0] == 0


@pytest.mark.parametrize("gelu", [False, True])
def test_oracle_act_and_mul_formula(gelu, oracle):
    from math import erf
    rng = np.random.default_rng(2)
    x = _bf(oracle, rng.standard_normal((4, 48)) * 2)
    g, u = _f(oracle, x[:, :24]), _f(oracle, x[:, 24:])
    act = g * 0.5 * (1 + np.vectorize(erf)(g / np.sqrt(2))) if gelu else g / (1 + np.exp(-g))
    assert _close(oracle, oracle.ve_act_and_mul(x, gelu), _bf(oracle, act * u))[0] == 0


def test_oracle_rotary_neox_formula(oracle):
    rng = np.random.default_rng(3)
    M, heads, hs = 6, 3, 16
    q = _bf(oracle, rng.standard_normal((M, heads * hs)))
    ang = rng.uniform(0, 6.28, (M, hs // 2))
    cache = np.concatenate([np.cos(ang), np.sin(ang)], 1).astype(np.float32)
    qf = _f(oracle, q).reshape(M, heads, hs)
    x, y = qf[..., :hs // 2], qf[..., hs // 2:]
    c, s = cache[:, None, :hs // 2].astype(np.float64), cache[:, None, hs // 2:].astype(np.float64)
    want = np.concatenate([x * c - y * s, y * c + x * s], -1).reshape(M, heads * hs)
    assert _close(oracle, oracle.ve_rotary_neox(q, cache, hs), _bf(oracle, want))[0] == 0


def test_oracle_dequant_forms_match_the_preset_restatements(oracle):
    """dequant + rotary == the w8a8 preset followed by the fused path's own RoPE pair op."""
    rng = np.random.default_rng(4)
    M, N = 9, 32
    acc = rng.integers(-20000, 20000, (M, N), dtype=np.int32)
    st, sc = rng.uniform(0.001, 0.01, M).astype(np.float32), rng.uniform(0.001, 0.01, N).astype(np.float32)
    cs = oracle.rope_table(M, N, 10000.0)
    got = oracle.ve_dequant_rotary(acc, st, sc, cs)
    want = oracle.epilogue(acc, row=st, col=sc, pair="rope", cos_sin=cs)
    assert np.array_equal(got, want)
    # dequant + act*mul over halves == dequant, then act_and_mul on the bf16-free fp32 values
    x = acc.astype(np.float64) * st[:, None] * sc[None, :]
    g, u = x[:, :N // 2], x[:, N // 2:]
    r = _bf(oracle, g / (1 + np.exp(-g)) * u)
    out = oracle.ve_dequant_act_mul(acc, st, sc)
    assert _close(oracle, out[:, :N // 2], r)[0] == 0 and np.array_equal(out[:, :N // 2], out[:, N // 2:])


# ------------------------------------------------------------------ kernels vs oracle (GPU)
def _dev(torch, dev, bits):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(dev)


def _host(t):
    import torch
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


@pytest.mark.gpu
@pytest.mark.parametrize("M,N", [(64, 4096), (33, 8192), (5, 200), (3, 7), (2, 65536)])
def test_rms_norm_and_fused_add(M, N, capi, oracle, cuda):
    import torch
    rng = np.random.default_rng(N)
    x, r = _bf(oracle, rng.standard_normal((M, N))), _bf(oracle, rng.standard_normal((M, N)))
    w = _bf(oracle, rng.normal(1, 0.1, N))
    X, R, W = _dev(torch, cuda, x), _dev(torch, cuda, r), _dev(torch, cuda, w)
    out = torch.empty_like(X)
    capi.ve_rms_norm(out, X, W)
    assert _close(oracle, _host(out), oracle.ve_rms_norm(x, w))[0] == 0
    Xi = X.clone()
    capi.ve_rms_norm(Xi, Xi, W)                                      # in place
    assert torch.equal(Xi.view(torch.int16), out.view(torch.int16))
    want_x, want_r = oracle.ve_fused_add_rms_norm(x, r, w)
    capi.ve_fused_add_rms_norm(X, R, W)
    torch.cuda.synchronize()
    assert np.array_equal(_host(R), want_r)                          # bf16(sum): exact
    assert _close(oracle, _host(X), want_x)[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("gelu", [False, True])
@pytest.mark.parametrize("M,d", [(128, 14336), (7, 100), (3, 5)])
def test_act_and_mul(M, d, gelu, capi, oracle, cuda):
    import torch
    x = _bf(oracle, np.random.default_rng(d).standard_normal((M, 2 * d)) * 2)
    out = torch.empty((M, d), dtype=torch.bfloat16, device=cuda)
    capi.ve_act_and_mul(out, _dev(torch, cuda, x), gelu)
    torch.cuda.synchronize()
    nbad, mabs = _close(oracle, _host(out), oracle.ve_act_and_mul(x, gelu), ulps=2, atol=1e-3 if gelu else 1e-6)
    assert nbad == 0, mabs


@pytest.mark.gpu
@pytest.mark.parametrize("M,nq,nk,hs,rot", [(64, 32, 8, 128, 128), (17, 4, 0, 128, 128), (9, 3, 2, 24, 12),
                                            (5, 2, 1, 64, 32)])
def test_rotary_embedding(M, nq, nk, hs, rot, capi, oracle, cuda):
    import torch
    rng = np.random.default_rng(M)
    q = _bf(oracle, rng.standard_normal((M, nq * hs)))
    k = _bf(oracle, rng.standard_normal((M, nk * hs))) if nk else None
    ang = rng.uniform(0, 6.28, (M, rot // 2))
    cache = np.concatenate([np.cos(ang), np.sin(ang)], 1).astype(np.float32)
    Q = _dev(torch, cuda, q)
    Kt = _dev(torch, cuda, k) if nk else None
    capi.ve_rotary_embedding(Q, Kt, torch.from_numpy(cache).to(cuda), hs, rot)
    torch.cuda.synchronize()
    assert _close(oracle, _host(Q), oracle.ve_rotary_neox(q, cache, hs, rot))[0] == 0
    if nk:
        assert _close(oracle, _host(Kt), oracle.ve_rotary_neox(k, cache, hs, rot))[0] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("L,M,N", [(1, 64, 4096), (2, 9, 40), (1, 5, 6), (1, 4, 7)])
def test_dequant_merged_kernels(L, M, N, capi, oracle, cuda):
    import torch
    rng = np.random.default_rng(N)
    acc = rng.integers(-300000, 300000, (L, M, N), dtype=np.int32)
    st = rng.uniform(1e-4, 1e-3, L * M).astype(np.float32)
    sc = rng.uniform(1e-3, 1e-2, L * N).astype(np.float32)
    cs = np.stack([oracle.rope_table(M, N + (N & 1), 10000.0)[:, :N] for _ in range(L)])
    A, ST, SC = (torch.from_numpy(a).to(cuda) for a in (acc, st, sc))
    out = torch.empty((L, M, N), dtype=torch.bfloat16, device=cuda)
    capi.ve_dequant_rotary(out, A, ST, SC, torch.from_numpy(np.ascontiguousarray(cs)).to(cuda))
    torch.cuda.synchronize()
    assert _close(oracle, _host(out), oracle.ve_dequant_rotary(acc, st, sc, cs))[0] == 0
    if N % 2 == 0:
        for gelu in (False, True):
            capi.ve_dequant_act_mul(out, A, ST, SC, gelu)
            torch.cuda.synchronize()
            nbad, mabs = _close(oracle, _host(out), oracle.ve_dequant_act_mul(acc, st, sc, gelu), ulps=2,
                               atol=1e-3 if gelu else 1e-6)
            assert nbad == 0, mabs


@pytest.mark.gpu
def test_rowops_reject_bad_arguments(capi, cuda):
    import torch
    x = torch.zeros((4, 64), dtype=torch.bfloat16, device=cuda)
    L = capi.lib()
    assert L.xf_ve_rms_norm(None, x.data_ptr(), x.data_ptr(), 4, 64, 1e-6, None) == 4
    assert L.xf_ve_rotary_embedding(x.data_ptr(), None, x.data_ptr(), 16, 4, 0, 15, 4, None) == 4   # odd rot_dim
    assert L.xf_ve_act_and_mul(x.data_ptr(), x.data_ptr(), 0, 4, 0, None) == 4
