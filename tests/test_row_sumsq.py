"""The row_sumsq side output of the fused GEMM and its finishing pass (the reference's K0a_CR,
kernels/gemm_residual_gamma_colred.hpp): per row, partial sums of squares of the final fp32 values,
then rstd[m] = 1/sqrt(sum/N + eps).  Checked against the oracle's unrounded epilogue result."""
import ctypes as C

import numpy as np
import pytest

import parity_cases as pc
from test_gemm_parity import _t, _variant_flags

pytestmark = pytest.mark.gpu


def _run(capi, oracle, dev, M, N, K, seed, flags=0, with_residual=True):
    import torch
    from conftest import bf16_bits
    d = pc.make_inputs(oracle, "k0a", M, N, K, seed)
    A, B = _t(torch, d["A"], dev, True), _t(torch, d["B"], dev, True)
    D = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    count = capi.lib().xf_row_sumsq_count(M, N, 1)
    assert count == ((N + 31) // 32) * M
    partials = torch.full((count,), float("nan"), dtype=torch.float32, device=dev)   # no zeroing needed
    kw = dict(col_scale=_t(torch, d["gamma"], dev))
    okw = dict(col=d["gamma"])
    if with_residual:
        kw["residual"] = _t(torch, d["residual"], dev, True)
        okw["residual"] = d["residual"]
    plan = capi.GemmPlan(A, B, D, row_sumsq=partials, flags=flags, **kw)
    plan.run()
    rstd = torch.empty(M, dtype=torch.float32, device=dev)
    capi.reduce_partials_rsqrt(partials, rstd, M, N)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    want_bits, want_f32 = oracle.epilogue(oracle.gemm_bf16(d["A"], d["B"]), want_f32=True, **okw)
    nbad, mabs, mrel = pc.compare_bf16(oracle, bf16_bits(D), want_bits)
    assert nbad == 0, (plan.kernel_name, mabs, mrel)
    assert not torch.isnan(partials).any()                     # every slot was written
    want_rstd = 1.0 / np.sqrt((want_f32.astype(np.float64) ** 2).mean(axis=1) + 1e-6)
    got = rstd.cpu().numpy()
    assert np.allclose(got, want_rstd, rtol=2e-5), (plan.kernel_name, np.abs(got / want_rstd - 1).max())
    return plan, D, rstd


@pytest.mark.parametrize("shape", [(384, 768, 512), (200, 336, 208), (128, 40, 64), (1, 16, 16)])
def test_row_sumsq_matches_the_unrounded_epilogue(shape, capi, oracle, cuda):
    _run(capi, oracle, cuda, *shape, seed=31)


@pytest.mark.parametrize("flags_name", ["1cta_bn128_ks1", "2cta_bn128_ks2", "1cta_bn256_ks1", "2cta_bn256_ks2", "direct"])
def test_row_sumsq_every_variant(flags_name, capi, oracle, cuda):
    _run(capi, oracle, cuda, 512, 1024, 320, seed=32, flags=_variant_flags(capi, flags_name))


def test_row_sumsq_with_split_k(capi, oracle, cuda):
    """Units of a split tile are finished by different CTAs; each slot is still written once."""
    plan, _, _ = _run(capi, oracle, cuda, 640, 2048, 6144, seed=33,
                      flags=_variant_flags(capi, "2cta_bn256") | capi.FLAG_NO_CLUSTER_SPLIT)
    assert "ksplit" in plan.kernel_name


def test_row_sumsq_agrees_with_the_separate_pass(capi, oracle, cuda):
    """rstd from the fused side output vs compute_rstd over the bf16 output: the same up to the
    rounding of D to bf16."""
    import torch
    _, D, rstd = _run(capi, oracle, cuda, 512, 4096, 1024, seed=34)
    sep = torch.empty_like(rstd)
    capi.compute_rstd(D, sep)
    torch.cuda.synchronize()
    assert torch.allclose(rstd, sep, rtol=2e-3)


def test_row_sumsq_is_refused_with_pair_ops(capi, cuda):
    import torch
    A = torch.zeros((128, 64), dtype=torch.bfloat16, device=cuda)
    B = torch.zeros((64, 128), dtype=torch.bfloat16, device=cuda)
    D = torch.zeros((128, 128), dtype=torch.bfloat16, device=cuda)
    partials = torch.zeros(4 * 128, dtype=torch.float32, device=cuda)
    with pytest.raises(capi.XfError) as e:
        capi.GemmPlan(A, B, D, pair="swiglu", row_sumsq=partials)
    assert "row_sumsq" in str(e.value)
    assert capi.lib().xf_reduce_partials_rsqrt(None, None, 4, 4, 1, C.c_float(1e-6), None) == 4
