"""GPU parity: the fused tcgen05 GEMM, called through the C ABI, against the CPU oracle on the same
seeded inputs.  int32 accumulators must be bit-exact; bf16 outputs within abs 2e-2 or rel 1e-2."""
import numpy as np
import pytest

import parity_cases as pc

pytestmark = pytest.mark.gpu


def _t(torch, a, dev, bf16=False):
    if a is None:
        return None
    if bf16:
        return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16).to(dev)
    return torch.from_numpy(np.ascontiguousarray(a)).to(dev)


def run_gpu(capi, o, preset, d, dev, flags=0, out_dtype=None):
    import torch
    int8 = pc.is_int8(preset)
    A = _t(torch, d["A"], dev, bf16=not int8)
    B = _t(torch, d["B"], dev, bf16=not int8)
    k = pc.epilogue_kwargs(o, preset, d)
    M, N = A.shape[0], B.shape[1]
    compact = bool(k.get("compact"))
    n_out = N // 2 if compact else N
    D = torch.full((M, n_out), float("nan"), dtype=out_dtype or torch.bfloat16, device=dev)
    aux = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev) if k.get("want_aux") else None
    bias = None
    if "bias" in k:
        bias = _t(torch, d["bias_bf16"], dev, bf16=True) if preset == "w8a8_biased_bf16bias" else _t(torch, k["bias"], dev)
    plan = capi.GemmPlan(
        A, B, D,
        residual=_t(torch, k.get("residual"), dev, bf16=True), aux_store=aux,
        row_scale=_t(torch, k.get("row"), dev), col_scale=_t(torch, k.get("col"), dev), bias=bias,
        unary=k.get("unary", "none"), pair=k.get("pair", "none"),
        cos_sin=_t(torch, k.get("cos_sin"), dev), cos_sin_period=k.get("cos_sin_period", 0),
        compact=compact, flags=flags)
    plan.run()
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    from conftest import bf16_bits
    res = bf16_bits(D) if D.dtype == torch.bfloat16 else D.cpu().numpy()
    return plan, res, (bf16_bits(aux) if aux is not None else None)


def check(capi, o, preset, M, N, K, dev, flags=0, seed=0):
    d = pc.make_inputs(o, preset, M, N, K, seed)
    _, want = pc.expected(o, preset, d)
    plan, got, aux = run_gpu(capi, o, preset, d, dev, flags)
    want_aux = None
    if isinstance(want, tuple):
        want, want_aux = want
    nbad, mabs, mrel = pc.compare_bf16(o, got, want)
    assert nbad == 0, f"{preset} {M}x{N}x{K} {plan.kernel_name}: {nbad} bad, max abs {mabs}, max rel {mrel}"
    if want_aux is not None:
        nb2, ma2, _ = pc.compare_bf16(o, aux, want_aux)
        assert nb2 == 0, f"{preset} aux store: {nb2} bad, max abs {ma2}"
    return plan


@pytest.mark.parametrize("preset", pc.PRESETS)
def test_presets_aligned(preset, capi, oracle, cuda):
    """Every preset at a tile-aligned shape spanning several CTA tiles and k-blocks."""
    check(capi, oracle, preset, 384, 768, 512, cuda)


@pytest.mark.parametrize("preset", ["k1", "k2", "k2_compact", "k4v2", "k0a", "k0_dual",
                                    "w8a8_dequant_biased", "bias_gelu"])
def test_presets_ragged(preset, capi, oracle, cuda):
    """M, N, K not multiples of any tile: tails are zero-filled on load and clipped on store."""
    check(capi, oracle, preset, 200, 336, 208, cuda)


def _variant_flags(capi, name):
    f = 0
    f |= capi.FLAG_FORCE_1CTA if "1cta" in name else capi.FLAG_FORCE_2CTA if "2cta" in name else 0
    f |= capi.FLAG_FORCE_BN256 if "bn256" in name else capi.FLAG_FORCE_BN128 if "bn128" in name else 0
    f |= capi.FLAG_FORCE_KS1 if "ks1" in name else capi.FLAG_FORCE_KS2 if "ks2" in name else 0
    f |= capi.FLAG_DIRECT_STORE if "direct" in name else 0
    return f


@pytest.mark.parametrize("flags_name", ["2cta_bn256_ks1", "2cta_bn256_ks2", "1cta_bn256_ks1", "2cta_bn128_ks1",
                                        "2cta_bn128_ks2", "1cta_bn128_ks1", "1cta_bn128_ks2", "direct"])
@pytest.mark.parametrize("preset", ["k2_compact", "k4v2_table", "k0a"])
def test_every_kernel_variant(preset, flags_name, capi, oracle, cuda):
    """Each compiled tile variant: 1 or 2 CTAs per tile, 128/256 columns, 1 or 2 K slabs per stage;
    K = 320 is not a multiple of either stage depth."""
    plan = check(capi, oracle, preset, 512, 1024, 320, cuda, flags=_variant_flags(capi, flags_name))
    if flags_name != "direct":
        assert ("cta2" in plan.kernel_name) == ("2cta" in flags_name)


@pytest.mark.parametrize("flags_name", ["2cta_bn256_ks1", "2cta_bn256_ks2", "1cta_bn256_ks1", "1cta_bn128_ks1",
                                        "1cta_bn128_ks2"])
def test_int8_variants(flags_name, capi, oracle, cuda):
    check(capi, oracle, "w8a8_dequant_biased", 512, 1024, 640, cuda, flags=_variant_flags(capi, flags_name))


@pytest.mark.parametrize("shape", [(384, 768, 1024), (200, 336, 208), (128, 256, 128), (1, 16, 16)])
@pytest.mark.parametrize("flags", [0, 2, 4])
def test_int32_accumulator_bit_exact(shape, flags, capi, oracle, cuda):
    """Raw int32 accumulators (empty epilogue, int32 D) equal the exact integer GEMM."""
    import torch
    M, N, K = shape
    rng = np.random.default_rng(11)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    want = oracle.gemm_s8(A, B)
    D = torch.full((M, N), -7, dtype=torch.int32, device=cuda)
    plan = capi.GemmPlan(torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda), D, flags=flags)
    plan.run()
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    assert np.array_equal(D.cpu().numpy(), want), plan.kernel_name


def test_int32_extremes(capi, oracle, cuda):
    """All -128 inputs: the largest magnitude products, K up to the Llama-70B FFN depth."""
    import torch
    M, N, K = 128, 256, 28672
    A = torch.full((M, K), -128, dtype=torch.int8, device=cuda)
    B = torch.full((K, N), -128, dtype=torch.int8, device=cuda)
    D = torch.zeros((M, N), dtype=torch.int32, device=cuda)
    plan = capi.GemmPlan(A, B, D)
    plan.run()
    torch.cuda.synchronize()
    assert int(D.min()) == int(D.max()) == K * 16384


def test_fp32_accumulator_output(capi, oracle, cuda):
    """fp32 D with an empty epilogue returns the accumulator itself."""
    import torch
    d = pc.make_inputs(oracle, "identity", 256, 512, 384, 3)
    acc = oracle.gemm_bf16(d["A"], d["B"])
    _, got, _ = run_gpu(capi, oracle, "identity", d, cuda, out_dtype=torch.float32)
    assert np.abs(got - acc).max() < 1e-4 * np.abs(acc).max()


def test_batched_L(capi, oracle, cuda):
    """L > 1 with per-batch A, B, D and vectors; and a shared weight (batch stride 0)."""
    import torch
    from conftest import bf16_bits
    L, M, N, K = 3, 160, 256, 192
    rng = np.random.default_rng(5)
    A = oracle.f32_to_bf16(rng.standard_normal((L, M, K)).astype(np.float32))
    B = oracle.f32_to_bf16((rng.standard_normal((L, K, N)) * K ** -0.5).astype(np.float32))
    R = rng.uniform(0.5, 1.5, (L, M)).astype(np.float32)
    tA, tB = _t(torch, A, cuda, True), _t(torch, B, cuda, True)
    D = torch.zeros((L, M, N), dtype=torch.bfloat16, device=cuda)
    plan = capi.GemmPlan(tA, tB, D, row_scale=_t(torch, R.reshape(-1), cuda), pair="swiglu")
    plan.run()
    torch.cuda.synchronize()
    got = bf16_bits(D)
    for l in range(L):
        want = oracle.epilogue(oracle.gemm_bf16(A[l], B[l]), row=R[l], pair="swiglu")
        assert pc.compare_bf16(oracle, got[l], want)[0] == 0
    # shared B: 2-D weight tensor => batch stride 0
    D2 = torch.zeros((L, M, N), dtype=torch.bfloat16, device=cuda)
    plan2 = capi.GemmPlan(tA, tB[1].contiguous(), D2, row_scale=_t(torch, R.reshape(-1), cuda))
    plan2.run()
    torch.cuda.synchronize()
    got2 = bf16_bits(D2)
    for l in range(L):
        want = oracle.epilogue(oracle.gemm_bf16(A[l], B[1]), row=R[l])
        assert pc.compare_bf16(oracle, got2[l], want)[0] == 0


def test_null_vector_uses_null_default(capi, oracle, cuda):
    """A broadcast node with a null pointer contributes its null_default (ColBroadcast semantics)."""
    import torch
    import ctypes as C
    from conftest import bf16_bits
    d = pc.make_inputs(oracle, "k1", 128, 256, 128, 9)
    A, B = _t(torch, d["A"], cuda, True), _t(torch, d["B"], cuda, True)
    D = torch.zeros((128, 256), dtype=torch.bfloat16, device=cuda)
    plan = capi.GemmPlan(A, B, D)
    plan.close()
    desc = plan.desc
    desc.epi.row_scale.enabled = 1
    desc.epi.row_scale.ptr = None
    desc.epi.row_scale.dtype = capi.DT_F32
    desc.epi.row_scale.null_default = 0.5
    h = C.c_void_p()
    capi.check(capi.lib().xf_gemm_plan_create(C.byref(desc), plan.workspace.data_ptr(), C.byref(h)))
    capi.check(capi.lib().xf_gemm_run(h, None))
    torch.cuda.synchronize()
    capi.lib().xf_plan_destroy(h)
    want = oracle.epilogue(oracle.gemm_bf16(d["A"], d["B"]), row=np.full(128, 0.5, np.float32))
    assert pc.compare_bf16(oracle, bf16_bits(D), want)[0] == 0


def test_rerun_is_idempotent(capi, oracle, cuda):
    """run() is re-entrant with the same plan: 20 back-to-back launches leave the same bits."""
    import torch
    from conftest import bf16_bits
    d = pc.make_inputs(oracle, "k0a", 512, 512, 256, 4)
    plan, first, _ = run_gpu(capi, oracle, "k0a", d, cuda)
    for _ in range(20):
        plan.run()
    torch.cuda.synchronize()
    D = plan._keep[2]
    assert np.array_equal(bf16_bits(D), first)


def test_canary_rows_and_columns_untouched(capi, oracle, cuda):
    """D embedded in a larger buffer (ldd > N, rows after M): nothing outside [M,N] is written."""
    import torch
    from conftest import bf16_bits
    M, N, K, LDD = 200, 328, 136, 344
    d = pc.make_inputs(oracle, "k1", M, N, K, 6)
    A, B = _t(torch, d["A"], cuda, True), _t(torch, d["B"], cuda, True)
    for flags in (0, capi.FLAG_DIRECT_STORE):
        buf = torch.full((M + 8, LDD), 777.0, dtype=torch.bfloat16, device=cuda)
        D = buf[:M, :N]
        plan = capi.GemmPlan(A, B, D, row_scale=_t(torch, d["scale"], cuda), flags=flags)
        plan.run()
        torch.cuda.synchronize()
        want = oracle.epilogue(oracle.gemm_bf16(d["A"], d["B"]), row=d["scale"])
        assert pc.compare_bf16(oracle, bf16_bits(buf[:M, :N].contiguous()), want)[0] == 0
        assert bool((buf[M:, :] == 777.0).all()) and bool((buf[:, N:] == 777.0).all())


@pytest.mark.parametrize("flags_name", ["pdl", "no_pdl"])
def test_dependent_launches_stay_ordered(flags_name, capi, oracle, cuda):
    """A chain D1 = A*B1, D2 = D1*B2 launched back to back with no host synchronisation, many times
    over with D1 overwritten in between: with programmatic dependent launch the second kernel's
    set-up overlaps the first one's tail, but it must not read D1 before the first has finished."""
    import torch
    from conftest import bf16_bits
    M, K, N1, N2 = 256, 512, 1024, 512
    rng = np.random.default_rng(77)
    A = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    B1 = oracle.f32_to_bf16((rng.standard_normal((K, N1)) * K ** -0.5).astype(np.float32))
    B2 = oracle.f32_to_bf16((rng.standard_normal((N1, N2)) * N1 ** -0.5).astype(np.float32))
    tA, tB1, tB2 = (_t(torch, x, cuda, True) for x in (A, B1, B2))
    D1 = torch.zeros((M, N1), dtype=torch.bfloat16, device=cuda)
    D2 = torch.zeros((M, N2), dtype=torch.bfloat16, device=cuda)
    flags = capi.FLAG_NO_PDL if flags_name == "no_pdl" else 0
    p1 = capi.GemmPlan(tA, tB1, D1, flags=flags)
    p2 = capi.GemmPlan(D1, tB2, D2, flags=flags)
    poison = capi.GemmPlan(tA, tB1, D1, row_scale=torch.zeros(M, device=cuda), flags=flags)   # writes D1 = 0
    for _ in range(25):
        poison.run()
        p1.run()
        p2.run()
    torch.cuda.synchronize()
    assert p1.device_status() == 0 and p2.device_status() == 0
    d1 = oracle.epilogue(oracle.gemm_bf16(A, B1))
    want = oracle.epilogue(oracle.gemm_bf16(d1, B2))
    assert np.array_equal(bf16_bits(D1), d1) or pc.compare_bf16(oracle, bf16_bits(D1), d1)[0] == 0
    assert pc.compare_bf16(oracle, bf16_bits(D2), oracle.epilogue(oracle.gemm_bf16(bf16_bits(D1), B2)))[0] == 0
    assert pc.compare_bf16(oracle, bf16_bits(D2), want)[0] == 0


@pytest.mark.parametrize("preset,shape", [
    ("k4v2_table", (512, 1024, 512)),      # per-head table, one tile per CTA pair
    ("k4v2_table", (300, 640, 264)),       # ragged rows and K
    ("k0a", (384, 768, 512)),              # residual tile
    ("k0a", (200, 336, 208)),              # ragged: the staged tile's columns beyond N read as zero
    ("k0_dual", (384, 768, 512)),          # residual + aux store
    ("k0a", (2048, 4096, 512)),            # 128 paired tiles on 74 pairs: staged only for each CTA's last tile
    ("k4v2_table", (4096, 1024, 256)),
])
def test_tail_operand_staging_is_bit_identical(preset, shape, capi, oracle, cuda):
    """A CTA's last tile takes its residual / cos_sin operand from shared memory (TMA-staged while
    the main loop drains) instead of global loads: same bits out, and inside the parity bar."""
    M, N, K = shape
    d = pc.make_inputs(oracle, preset, M, N, K, seed=3)
    plan_a, got_a, aux_a = run_gpu(capi, oracle, preset, d, cuda)
    plan_b, got_b, aux_b = run_gpu(capi, oracle, preset, d, cuda, flags=capi.FLAG_NO_TAIL_STAGING)
    assert np.array_equal(got_a, got_b), plan_a.kernel_name
    if aux_a is not None:
        assert np.array_equal(aux_a, aux_b)
    _, want = pc.expected(oracle, preset, d)
    if isinstance(want, tuple):
        want = want[0]
    assert pc.compare_bf16(oracle, got_a, want)[0] == 0


@pytest.mark.parametrize("preset,shape,extra", [
    ("k0a", (384, 768, 512), 0),
    ("k0a", (200, 336, 208), 0),               # ragged rows and columns: boxes past the edges read as zero
    ("k0a", (2048, 4096, 512), 0),             # several tiles per CTA: staged last tile + TMA slices before it
    ("k0a", (2048, 4096, 512), "no_tail"),     # every tile through the per-slice TMA loads
    ("k0_dual", (384, 768, 512), 0),           # residual + aux store
    ("k0a", (512, 4096, 4096), 0),             # cluster split-K variant (partials from the partner pair)
    ("k0a", (640, 2304, 8192), 0),             # remainder wave split along K (partials from the workspace)
])
def test_residual_through_tma_is_bit_identical(preset, shape, extra, capi, oracle, cuda):
    """The residual of a 32-column slice comes by TMA into the buffer its result is stored from
    (default) or through per-thread 16-byte loads (XF_FLAG_NO_RESIDUAL_TMA): same bits out."""
    M, N, K = shape
    base = capi.FLAG_NO_TAIL_STAGING if extra == "no_tail" else 0
    d = pc.make_inputs(oracle, preset, M, N, K, seed=5)
    plan_a, got_a, aux_a = run_gpu(capi, oracle, preset, d, cuda, flags=base)
    plan_b, got_b, aux_b = run_gpu(capi, oracle, preset, d, cuda, flags=base | capi.FLAG_NO_RESIDUAL_TMA)
    assert plan_a.device_status() == 0 and plan_b.device_status() == 0
    assert np.array_equal(got_a, got_b), plan_a.kernel_name
    if aux_a is not None:
        assert np.array_equal(aux_a, aux_b)
    _, want = pc.expected(oracle, preset, d)
    if isinstance(want, tuple):
        want = want[0]
    assert pc.compare_bf16(oracle, got_a, want)[0] == 0


@pytest.mark.parametrize("shape,with_residual,L", [
    ((384, 768, 512), True, 1),
    ((200, 336, 208), True, 1),          # ragged: the TMA store clips rows beyond M and columns beyond N
    ((2048, 4096, 512), True, 1),        # several tiles per CTA
    ((1024, 2048, 256), False, 1),       # auxiliary output of the bare accumulator
    ((200, 384, 160), True, 3),          # batched
])
def test_aux_store_through_tma_is_bit_identical(shape, with_residual, L, capi, oracle, cuda):
    """The second (auxiliary) output leaves through a staging buffer and a TMA store (default) or
    through per-thread stores (XF_FLAG_NO_RESIDUAL_TMA): same bits in D and in the auxiliary tensor."""
    import torch
    from conftest import bf16_bits
    M, N, K = shape
    rng = np.random.default_rng(29)
    A = oracle.f32_to_bf16(rng.standard_normal((L, M, K)).astype(np.float32))
    B = oracle.f32_to_bf16((rng.standard_normal((L, K, N)) * K ** -0.5).astype(np.float32))
    res = oracle.f32_to_bf16(rng.standard_normal((L, M, N)).astype(np.float32))
    gamma = rng.normal(1.0, 0.02, (L, N)).astype(np.float32)
    tA, tB = _t(torch, A, cuda, True), _t(torch, B, cuda, True)
    outs = {}
    for flags in (0, capi.FLAG_NO_RESIDUAL_TMA):
        D = torch.full((L, M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
        aux = torch.full((L, M, N), float("nan"), dtype=torch.bfloat16, device=cuda)
        plan = capi.GemmPlan(tA, tB, D, residual=_t(torch, res, cuda, True) if with_residual else None, aux_store=aux,
                             col_scale=_t(torch, gamma.reshape(-1), cuda), flags=flags)
        plan.run()
        torch.cuda.synchronize()
        assert plan.device_status() == 0
        outs[flags] = (bf16_bits(D).copy(), bf16_bits(aux).copy())
    assert np.array_equal(outs[0][0], outs[capi.FLAG_NO_RESIDUAL_TMA][0])
    assert np.array_equal(outs[0][1], outs[capi.FLAG_NO_RESIDUAL_TMA][1])
    for l in range(L):
        acc = oracle.gemm_bf16(A[l], B[l])
        want, want_aux = oracle.epilogue(acc, residual=res[l] if with_residual else None, col=gamma[l], want_aux=True)
        assert pc.compare_bf16(oracle, outs[0][0][l], want)[0] == 0
        assert pc.compare_bf16(oracle, outs[0][1][l], want_aux)[0] == 0


@pytest.mark.parametrize("preset", pc.PRESETS)
@pytest.mark.parametrize("shape", [(384, 768, 512), (200, 336, 208), (2048, 2048, 256)],
                         ids=["aligned", "ragged", "several_tiles"])
def test_class_instance_matches_the_generic_one(preset, shape, capi, oracle, cuda):
    """A plan launches the kernel instance compiled for its epilogue class (scales only, residual,
    GLU pair, RoPE, or everything); XF_FLAG_GENERIC_EPILOGUE forces the all-in-one instance.  Same
    bits out for every preset, aligned, ragged and with several tiles per CTA."""
    M, N, K = shape
    if pc.is_int8(preset) and (N % 16 or K % 16):
        N, K = 352, 208
    if preset == "k4v2_table" and N % 128:
        N = 384           # whole 128-column heads for the per-head table
    d = pc.make_inputs(oracle, preset, M, N, K, seed=11)
    plan_a, got_a, aux_a = run_gpu(capi, oracle, preset, d, cuda)
    plan_b, got_b, aux_b = run_gpu(capi, oracle, preset, d, cuda, flags=capi.FLAG_GENERIC_EPILOGUE)
    assert np.array_equal(got_a, got_b), (preset, plan_a.kernel_name)
    if aux_a is not None:
        assert np.array_equal(aux_a, aux_b)


def test_residual_through_tma_in_place(capi, oracle, cuda):
    """D aliases the residual (x += A @ B, the reference's O-projection use): a slice's residual is
    read before the same slice is stored, whichever way it is fetched."""
    import torch
    from conftest import bf16_bits
    M, N, K = 1024, 2048, 512
    rng = np.random.default_rng(23)
    A = oracle.f32_to_bf16(rng.standard_normal((M, K)).astype(np.float32))
    B = oracle.f32_to_bf16((rng.standard_normal((K, N)) * K ** -0.5).astype(np.float32))
    res = oracle.f32_to_bf16(rng.standard_normal((M, N)).astype(np.float32))
    want = oracle.epilogue(oracle.gemm_bf16(A, B), residual=res)
    tA, tB = _t(torch, A, cuda, True), _t(torch, B, cuda, True)
    for flags in (0, capi.FLAG_NO_RESIDUAL_TMA):
        X = _t(torch, res, cuda, True).clone()
        plan = capi.GemmPlan(tA, tB, X, residual=X, flags=flags)
        plan.run()
        torch.cuda.synchronize()
        assert plan.device_status() == 0
        assert pc.compare_bf16(oracle, bf16_bits(X), want)[0] == 0


def test_batched_full_matrix_operands(capi, oracle, cuda):
    """L > 1 with a residual (batch stride M*N) and with a per-head RoPE table (batch stride M*P):
    the staged operand of the last tile takes its batch from the tile's batch index."""
    import torch
    from conftest import bf16_bits
    L, M, N, K, P = 3, 200, 384, 160, 128
    rng = np.random.default_rng(17)
    A = oracle.f32_to_bf16(rng.standard_normal((L, M, K)).astype(np.float32))
    B = oracle.f32_to_bf16((rng.standard_normal((L, K, N)) * K ** -0.5).astype(np.float32))
    res = oracle.f32_to_bf16(rng.standard_normal((L, M, N)).astype(np.float32))
    gamma = rng.normal(1.0, 0.02, (L, N)).astype(np.float32)
    cs = np.stack([oracle.rope_table(M, P, 500000.0 * (l + 1)) for l in range(L)])
    R = rng.uniform(0.5, 1.5, (L, M)).astype(np.float32)
    tA, tB = _t(torch, A, cuda, True), _t(torch, B, cuda, True)
    outs = {}
    for flags in (0, capi.FLAG_NO_TAIL_STAGING):
        D1 = torch.zeros((L, M, N), dtype=torch.bfloat16, device=cuda)
        p1 = capi.GemmPlan(tA, tB, D1, residual=_t(torch, res, cuda, True), col_scale=_t(torch, gamma.reshape(-1), cuda),
                           flags=flags)
        p1.run()
        D2 = torch.zeros((L, M, N), dtype=torch.bfloat16, device=cuda)
        p2 = capi.GemmPlan(tA, tB, D2, row_scale=_t(torch, R.reshape(-1), cuda), pair="rope",
                           cos_sin=_t(torch, cs, cuda), cos_sin_period=P, flags=flags)
        p2.run()
        torch.cuda.synchronize()
        assert p1.device_status() == 0 and p2.device_status() == 0
        outs[flags] = (bf16_bits(D1).copy(), bf16_bits(D2).copy())
    assert np.array_equal(outs[0][0], outs[capi.FLAG_NO_TAIL_STAGING][0])
    assert np.array_equal(outs[0][1], outs[capi.FLAG_NO_TAIL_STAGING][1])
    for l in range(L):
        acc = oracle.gemm_bf16(A[l], B[l])
        want1 = oracle.epilogue(acc, residual=res[l], col=gamma[l])
        assert pc.compare_bf16(oracle, outs[0][0][l], want1)[0] == 0
        want2 = oracle.epilogue(acc, row=R[l], pair="rope", cos_sin=cs[l], cos_sin_period=P)
        assert pc.compare_bf16(oracle, outs[0][1][l], want2)[0] == 0
