"""Split-K of the remainder wave.

When the tile count is not a multiple of the scheduling units, the tiles of the last wave are cut
into K slices; each slice publishes its raw accumulator and the last one to arrive sums them in
slice order and runs the epilogue.  These cases force that path (the kernel name then carries
"ksplitS") and hold it to the same bar as whole tiles: bf16 outputs inside the parity tolerance of
the host oracle, int32 accumulators bit-exact, repeated launches identical.
"""
import numpy as np
import pytest

import parity_cases as pc
from test_gemm_parity import check, _variant_flags

pytestmark = pytest.mark.gpu


# The planner splits only where its time estimate says the shorter last wave outweighs the trip of
# the partials through L2, i.e. for long K; "2cta_bn256" pins the tile where a narrower one would
# have won without a split.
@pytest.mark.parametrize("preset,shape,flags_name", [
    ("k1", (512, 2048, 8192), ""),                       # 16 paired tiles on 74 units: 4 slices each
    ("k2_compact", (128, 256, 4096), ""),                # two tiles
    ("k4v2_table", (500, 4000, 4160), "2cta_bn256"),     # ragged M, N and K; RoPE pairs after the sum
    ("k0_dual", (512, 2048, 8192), ""),                  # aux store and D both written after the sum
    ("k0a", (640, 2048, 6144), "2cta_bn256"),            # 24 tiles, 3 slices: uneven K ranges
    ("w8a8_dequant_biased", (512, 4096, 16384), "2cta_bn256"),
    ("bias_gelu", (256, 1024, 8192), ""),
])
def test_split_presets(preset, shape, flags_name, capi, oracle, cuda):
    M, N, K = shape
    plan = check(capi, oracle, preset, M, N, K, cuda, flags=(_variant_flags(capi, flags_name) | capi.FLAG_NO_CLUSTER_SPLIT))
    assert "ksplit" in plan.kernel_name, plan.kernel_name


@pytest.mark.parametrize("flags_name", ["1cta_bn128_ks1", "1cta_bn128_ks2", "1cta_bn256_ks1", "2cta_bn128_ks2",
                                        "2cta_bn256_ks1", "direct"])
def test_split_every_variant(flags_name, capi, oracle, cuda):
    plan = check(capi, oracle, "k2_compact", 384, 2304, 6144, cuda, flags=(_variant_flags(capi, flags_name) | capi.FLAG_NO_CLUSTER_SPLIT))
    assert "ksplit" in plan.kernel_name, plan.kernel_name


@pytest.mark.parametrize("shape,flags_name", [((512, 4096, 16384), "2cta_bn256"), ((128, 256, 16384), ""),
                                              ((200, 1008, 8208), "")])
def test_split_int32_bit_exact_and_repeatable(shape, flags_name, capi, oracle, cuda):
    """Integer partial sums are exact in any order; the counters return to zero after each launch,
    so a second and third launch of the same plan give the same answer."""
    import torch
    M, N, K = shape
    rng = np.random.default_rng(5)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    want = oracle.gemm_s8(A, B)
    D = torch.empty((M, N), dtype=torch.int32, device=cuda)
    flags = (_variant_flags(capi, flags_name) | capi.FLAG_NO_CLUSTER_SPLIT)
    plan = capi.GemmPlan(torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda), D, flags=flags)
    assert "ksplit" in plan.kernel_name, plan.kernel_name
    for _ in range(3):
        D.fill_(-7)
        plan.run()
        torch.cuda.synchronize()
        assert plan.device_status() == 0
        assert np.array_equal(D.cpu().numpy(), want), plan.kernel_name
    # the same problem as whole tiles
    D2 = torch.empty_like(D)
    whole = capi.GemmPlan(torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda), D2,
                          flags=flags | capi.FLAG_NO_SPLIT)
    assert "ksplit" not in whole.kernel_name
    whole.run()
    torch.cuda.synchronize()
    assert np.array_equal(D2.cpu().numpy(), want)


def test_split_bf16_is_deterministic(capi, oracle, cuda):
    """fp32 partials are summed in slice order whichever slice finishes last: bit-identical reruns."""
    import torch
    from conftest import bf16_bits
    d = pc.make_inputs(oracle, "k1", 512, 2048, 8192, 3)
    A = torch.from_numpy(d["A"].view(np.int16)).view(torch.bfloat16).to(cuda)
    B = torch.from_numpy(d["B"].view(np.int16)).view(torch.bfloat16).to(cuda)
    D = torch.empty((512, 2048), dtype=torch.bfloat16, device=cuda)
    plan = capi.GemmPlan(A, B, D, flags=capi.FLAG_NO_CLUSTER_SPLIT)
    assert "ksplit" in plan.kernel_name
    outs = []
    for _ in range(4):
        D.zero_()
        plan.run()
        torch.cuda.synchronize()
        outs.append(bf16_bits(D).copy())
    assert all(np.array_equal(outs[0], o) for o in outs[1:])


def test_small_workspace_falls_back_to_whole_tiles(capi, oracle, cuda):
    """A caller that promises only the 16-byte status word gets whole tiles, not a write past it."""
    import ctypes as C
    import torch
    d = pc.make_inputs(oracle, "k1", 512, 2048, 8192, 4)
    A = torch.from_numpy(d["A"].view(np.int16)).view(torch.bfloat16).to(cuda)
    B = torch.from_numpy(d["B"].view(np.int16)).view(torch.bfloat16).to(cuda)
    D = torch.empty((512, 2048), dtype=torch.bfloat16, device=cuda)
    plan = capi.GemmPlan(A, B, D, flags=capi.FLAG_NO_CLUSTER_SPLIT)
    desc = capi.XfGemmDesc.from_buffer_copy(plan.desc)
    desc.workspace_bytes = 0
    ws = torch.zeros(16, dtype=torch.uint8, device=cuda)
    h = C.c_void_p()
    capi.check(capi.lib().xf_gemm_plan_create(C.byref(desc), ws.data_ptr(), C.byref(h)))
    assert b"ksplit" not in capi.lib().xf_gemm_plan_kernel_name(h)
    capi.check(capi.lib().xf_gemm_run(h, None))
    torch.cuda.synchronize()
    capi.lib().xf_plan_destroy(h)
    from conftest import bf16_bits
    want = oracle.epilogue(oracle.gemm_bf16(d["A"], d["B"]))
    assert pc.compare_bf16(oracle, bf16_bits(D), want)[0] == 0


def test_split_wait_gives_up_and_the_plan_recovers(capi, oracle, cuda):
    """The give-up side of a bounded wait, made on purpose without a fault: the counter a K slice
    polls for the other slices' partials is set so far below zero that it cannot reach its target;
    with XF_FLAG_SHORT_WAITS every waiting warp gives up after about a millisecond, the kernel ends
    normally with code 5 in the status word, the host reads it, and the same plan then runs
    correctly again."""
    import torch
    from conftest import bf16_bits
    d = pc.make_inputs(oracle, "k1", 512, 2048, 8192, 6)
    A = torch.from_numpy(d["A"].view(np.int16)).view(torch.bfloat16).to(cuda)
    B = torch.from_numpy(d["B"].view(np.int16)).view(torch.bfloat16).to(cuda)
    D = torch.empty((512, 2048), dtype=torch.bfloat16, device=cuda)
    plan = capi.GemmPlan(A, B, D, flags=capi.FLAG_SHORT_WAITS | capi.FLAG_NO_CLUSTER_SPLIT)
    assert "ksplit" in plan.kernel_name
    plan.run()
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    good = bf16_bits(D).copy()
    counters = plan.workspace[256:256 + 32].view(torch.int32)   # first split tile, first CTA
    counters[0] = -1000000                                       # "published" can never reach its target
    torch.cuda.synchronize()
    plan.run()
    torch.cuda.synchronize()                                     # returns: the wait is bounded
    with pytest.raises(capi.XfError) as e:
        plan.device_status()
    assert "device code 5" in str(e.value)
    assert plan.device_status() == 0                             # reported once, then cleared
    D.zero_()
    plan.run()
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    assert np.array_equal(bf16_bits(D), good)
