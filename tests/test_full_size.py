"""Parity at the full sizes of the five benchmark configurations, where the CPU oracle cannot redo the whole
GEMM in seconds.  Each case checks (a) sampled rows -- first/last row of CTA tiles plus random
ones -- element by element against the oracle, and (b) size-independent properties over the whole
output: exact row/column checksums of the int32 accumulator, the two output layouts of one kernel
agreeing bit for bit, RoPE preserving pair norms, the fused result agreeing with the unfused
GEMM + stand-alone kernel."""
import numpy as np
import pytest

import parity_cases as pc

pytestmark = pytest.mark.gpu


def _rows(M, n_random=24, seed=0):
    edge = [0, 1, 127, 128, 255, 256, 257, M // 2 - 1, M // 2, M - 257, M - 256, M - 129, M - 128, M - 1]
    rng = np.random.default_rng(seed)
    r = sorted(set(int(x) for x in edge if 0 <= x < M) | set(rng.integers(0, M, n_random).tolist()))
    return np.array(r, dtype=np.int64)


def _bits(t):
    from conftest import bf16_bits
    return bf16_bits(t)


def _gen_bf16(torch, dev, M, N, K, seed):
    g = torch.Generator(device=dev).manual_seed(seed)
    X = torch.randn(M, K, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    W = (torch.randn(K, N, generator=g, device=dev, dtype=torch.float32) * K ** -0.5).to(torch.bfloat16)
    R = torch.rsqrt((X.float() ** 2).mean(dim=1) + 1e-6).contiguous()
    return X, W, R


def test_config1_k1_whole_output(capi, oracle, cuda):
    """k1, M=512 N=4096 K=4096: small enough for the oracle to redo completely."""
    import torch
    M, N, K = 512, 4096, 4096
    X, W, R = _gen_bf16(torch, cuda, M, N, K, 1)
    D = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    plan = capi.GemmPlan(X, W, D, row_scale=R)
    plan.run()
    torch.cuda.synchronize()
    want = oracle.epilogue(oracle.gemm_bf16(_bits(X), _bits(W)), row=R.cpu().numpy())
    nbad, mabs, mrel = pc.compare_bf16(oracle, _bits(D), want)
    assert nbad == 0, (plan.kernel_name, mabs, mrel)


def test_config2_k2_llama8b_ffn(capi, oracle, cuda):
    """k2, M=4096 K=4096 N=28672 -> [4096,14336]."""
    import torch
    M, N, K = 4096, 28672, 4096
    X, W, R = _gen_bf16(torch, cuda, M, N, K, 2)
    Dc = torch.empty(M, N // 2, dtype=torch.bfloat16, device=cuda)
    Dd = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    pc_ = capi.GemmPlan(X, W, Dc, row_scale=R, pair="swiglu", compact=True)
    pd_ = capi.GemmPlan(X, W, Dd, row_scale=R, pair="swiglu")
    pc_.run(); pd_.run()
    torch.cuda.synchronize()
    assert pc_.device_status() == 0 and pd_.device_status() == 0
    # property: compact output == either column of the duplicated layout, bit for bit, everywhere
    assert torch.equal(Dc.view(torch.int16), Dd[:, 0::2].contiguous().view(torch.int16))
    assert torch.equal(Dc.view(torch.int16), Dd[:, 1::2].contiguous().view(torch.int16))
    # property: fused == bare GEMM + stand-alone kernels up to the intermediate bf16 roundings
    U = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    capi.GemmPlan(X, W, U).run()
    capi.sa_scale_rows(U, R)
    capi.sa_swiglu(U)
    torch.cuda.synchronize()
    diff = (U.float() - Dd.float()).abs()
    assert bool((diff <= 3e-2 + 3e-2 * Dd.float().abs()).all())
    # sampled rows against the oracle
    rows = _rows(M)
    Xs = X[torch.from_numpy(rows).to(cuda)]
    acc = oracle.gemm_bf16(_bits(Xs), _bits(W))
    want = oracle.epilogue(acc, row=R.cpu().numpy()[rows], pair="swiglu", compact=True)
    nbad, mabs, mrel = pc.compare_bf16(oracle, _bits(Dc)[rows], want)
    assert nbad == 0, (mabs, mrel)


@pytest.mark.parametrize("N", [4096, 1024])
def test_config3_k4v2_llama8b_qk(N, capi, oracle, cuda):
    """k4v2, M=4096 (positions 0..4095), K=4096, N=4096 / 1024, table [4096,128], theta=5e5."""
    import torch
    M, K = 4096, 4096
    X, W, R = _gen_bf16(torch, cuda, M, N, K, 3)
    table = oracle.rope_table(M, 128, 500000.0)
    cs = torch.from_numpy(table).to(cuda)
    D = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    plan = capi.GemmPlan(X, W, D, row_scale=R, pair="rope", cos_sin=cs, cos_sin_period=128)
    plan.run()
    # property: a rotation keeps the norm of every (even, odd) pair of the scaled accumulator
    S = torch.empty(M, N, dtype=torch.float32, device=cuda)
    capi.GemmPlan(X, W, S, row_scale=R).run()
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    n_in = S[:, 0::2] ** 2 + S[:, 1::2] ** 2
    Df = D.float()
    n_out = Df[:, 0::2] ** 2 + Df[:, 1::2] ** 2
    assert bool(((n_in - n_out).abs() <= 2e-2 * n_in + 1e-3).all())
    # position 0 has angle 0: the first row passes through unrotated
    assert bool(((Df[0] - S[0]).abs() <= 2e-2 + 1e-2 * S[0].abs()).all())
    rows = _rows(M)
    acc = oracle.gemm_bf16(_bits(X[torch.from_numpy(rows).to(cuda)]), _bits(W))
    want = oracle.epilogue(acc, row=R.cpu().numpy()[rows], pair="rope", cos_sin=table[rows], cos_sin_period=128)
    nbad, mabs, mrel = pc.compare_bf16(oracle, _bits(D)[rows], want)
    assert nbad == 0, (mabs, mrel)


def test_config4_w8a8_llama70b_down(capi, oracle, cuda):
    """w8a8_dequant_biased, M=8192 K=28672 N=8192: int32 accumulators exact, bf16 output in tolerance."""
    import torch
    M, N, K = 8192, 8192, 28672
    g = torch.Generator(device=cuda).manual_seed(4)
    Xf = torch.randn(M, K, generator=g, device=cuda).to(torch.bfloat16).float()
    st = (Xf.abs().amax(dim=1) / 127.0 + 1e-8).contiguous()
    A = torch.clamp(torch.round(Xf / st[:, None]), -128, 127).to(torch.int8)
    del Xf
    Wf = (torch.randn(K, N, generator=g, device=cuda) * K ** -0.5).to(torch.bfloat16).float()
    sc = (Wf.abs().amax(dim=0) / 127.0 + 1e-8).contiguous()
    B = torch.clamp(torch.round(Wf / sc[None, :]), -128, 127).to(torch.int8)
    del Wf
    bias = (torch.randn(N, generator=g, device=cuda) * 0.02).to(torch.bfloat16)
    acc = torch.empty(M, N, dtype=torch.int32, device=cuda)
    D = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    capi.GemmPlan(A, B, acc).run()
    plan = capi.GemmPlan(A, B, D, row_scale=st, col_scale=sc, bias=bias)
    plan.run()
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    # exact checksums over the whole accumulator: sum_n acc[m,n] = A[m,:] . rowsum(B), and
    # sum_m acc[m,n] = colsum(A) . B[:,n], in 64-bit integers
    b_rowsum = B.to(torch.int64).sum(dim=1)
    a_colsum = A.to(torch.int64).sum(dim=0)
    want_rows = (A.to(torch.float64) @ b_rowsum.to(torch.float64)).to(torch.int64)   # |.| < 2^53: exact
    want_cols = (a_colsum.to(torch.float64) @ B.to(torch.float64)).to(torch.int64)
    assert torch.equal(acc.to(torch.int64).sum(dim=1), want_rows)
    assert torch.equal(acc.to(torch.int64).sum(dim=0), want_cols)
    # sampled rows: accumulators bit-exact, dequantised output within the parity bar
    rows = _rows(M, n_random=10)
    ridx = torch.from_numpy(rows).to(cuda)
    want_acc = oracle.gemm_s8(A[ridx].cpu().numpy(), B.cpu().numpy())
    assert np.array_equal(acc[ridx].cpu().numpy(), want_acc)
    want = oracle.epilogue(want_acc, row=st.cpu().numpy()[rows], col=sc.cpu().numpy(),
                           bias=oracle.bf16_to_f32(_bits(bias)))
    nbad, mabs, mrel = pc.compare_bf16(oracle, _bits(D)[rows], want)
    assert nbad == 0, (mabs, mrel)
    # property: the fused epilogue == dequant + bias_add on the exact accumulator (one extra rounding)
    U = torch.empty(M, N, dtype=torch.bfloat16, device=cuda)
    capi.sa_dequant_w8a8(U, acc, st, sc)
    capi.sa_bias_add(U, bias.float())
    torch.cuda.synchronize()
    assert bool(((U.float() - D.float()).abs() <= 2e-2 + 1e-2 * D.float().abs()).all())


def test_config5_llama70b_layer_stages(capi, oracle, cuda):
    """The four stages of the 70B layer chain at M=8192, sampled rows per stage; the down
    projection consumes the gate/up stage's output."""
    import torch
    M, H, HKV, I = 8192, 8192, 1024, 28672
    rows = _rows(M, n_random=6, seed=5)
    ridx = torch.from_numpy(rows).to(cuda)
    table = oracle.rope_table(M, 128, 500000.0)
    cs = torch.from_numpy(table).to(cuda)
    # QKV: k4v2 over all 10240 columns (RoPE applied per 128-column head, V included)
    X, W, R = _gen_bf16(torch, cuda, M, H + 2 * HKV, H, 51)
    D = torch.empty(M, H + 2 * HKV, dtype=torch.bfloat16, device=cuda)
    capi.GemmPlan(X, W, D, row_scale=R, pair="rope", cos_sin=cs, cos_sin_period=128).run()
    torch.cuda.synchronize()
    want = oracle.epilogue(oracle.gemm_bf16(_bits(X[ridx]), _bits(W)), row=R.cpu().numpy()[rows], pair="rope",
                           cos_sin=table[rows], cos_sin_period=128)
    assert pc.compare_bf16(oracle, _bits(D)[rows], want)[0] == 0
    # O projection: k0a with a bf16 residual and gamma ~ N(1, 0.02)
    g = torch.Generator(device=cuda).manual_seed(52)
    X, W, _ = _gen_bf16(torch, cuda, M, H, H, 52)
    res = torch.randn(M, H, generator=g, device=cuda).to(torch.bfloat16)
    gamma = (1 + 0.02 * torch.randn(H, generator=g, device=cuda)).contiguous()
    D = torch.empty(M, H, dtype=torch.bfloat16, device=cuda)
    capi.GemmPlan(X, W, D, residual=res, col_scale=gamma).run()
    torch.cuda.synchronize()
    want = oracle.epilogue(oracle.gemm_bf16(_bits(X[ridx]), _bits(W)), residual=_bits(res)[rows],
                           col=gamma.cpu().numpy())
    assert pc.compare_bf16(oracle, _bits(D)[rows], want)[0] == 0
    del res
    # gate/up: k2 compact, N = 2 x 28672
    X, W, R = _gen_bf16(torch, cuda, M, 2 * I, H, 53)
    G = torch.empty(M, I, dtype=torch.bfloat16, device=cuda)
    capi.GemmPlan(X, W, G, row_scale=R, pair="swiglu", compact=True).run()
    torch.cuda.synchronize()
    want_g = oracle.epilogue(oracle.gemm_bf16(_bits(X[ridx]), _bits(W)), row=R.cpu().numpy()[rows], pair="swiglu",
                             compact=True)
    assert pc.compare_bf16(oracle, _bits(G)[rows], want_g)[0] == 0
    del X, W
    # down: k0a with K = 28672, A = the gate/up output
    g = torch.Generator(device=cuda).manual_seed(54)
    W = (torch.randn(I, H, generator=g, device=cuda) * I ** -0.5).to(torch.bfloat16)
    res = torch.randn(M, H, generator=g, device=cuda).to(torch.bfloat16)
    D = torch.empty(M, H, dtype=torch.bfloat16, device=cuda)
    capi.GemmPlan(G, W, D, residual=res, col_scale=gamma).run()
    torch.cuda.synchronize()
    want = oracle.epilogue(oracle.gemm_bf16(_bits(G)[rows], _bits(W)), residual=_bits(res)[rows],
                           col=gamma.cpu().numpy())
    assert pc.compare_bf16(oracle, _bits(D)[rows], want)[0] == 0
