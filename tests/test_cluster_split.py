"""Cluster split-K: the variants for small problems (at most one 256 x 256 tile per four SMs).

A cluster of four CTAs holds two MMA pairs that accumulate the two halves of one tile's K range in
their own tensor memory, swap partial accumulators through distributed shared memory and finish
half of the tile's columns each.  The kernel name then ends in "kc2".  Held to the same bar as
every other path: bf16 outputs inside the parity tolerance of the host oracle, int32 accumulators
bit-exact, repeated launches identical.
"""
import numpy as np
import pytest

import parity_cases as pc
from test_gemm_parity import check

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("preset,shape", [
    ("k1", (512, 4096, 4096)),                   # BASELINE configuration 1: 32 tiles, chosen by the planner
    ("k2_compact", (256, 1024, 2048)),           # compact output: two output units per K group
    ("k2", (500, 1000, 2056)),                   # ragged M, N and K; duplicated pair layout
    ("k4v2_table", (512, 1024, 4096)),           # RoPE pairs after the sum, per-head table
    ("k4", (300, 520, 1536)),                    # full-width cos_sin, ragged
    ("k0_dual", (512, 2048, 2048)),              # residual, aux store and D all after the sum
    ("k0a", (256, 264, 1024)),                   # second column tile almost empty
    ("bias_gelu", (128, 256, 1024)),             # one tile, second CTA of each pair has no valid rows
    ("w8a8_dequant_biased", (512, 2048, 8192)),
    ("w8a8_swiglu", (384, 1008, 4112)),
])
def test_cluster_split_presets(preset, shape, capi, oracle, cuda):
    M, N, K = shape
    plan = check(capi, oracle, preset, M, N, K, cuda, flags=capi.FLAG_FORCE_CLUSTER_SPLIT)
    assert plan.kernel_name.split("_s")[0].endswith("kc2"), plan.kernel_name


def test_planner_picks_cluster_split_for_config_1(capi, cuda):
    import torch
    A = torch.zeros((512, 4096), dtype=torch.bfloat16, device=cuda)
    B = torch.zeros((4096, 4096), dtype=torch.bfloat16, device=cuda)
    D = torch.zeros((512, 4096), dtype=torch.bfloat16, device=cuda)
    assert "kc2" in capi.GemmPlan(A, B, D).kernel_name
    assert "kc2" not in capi.GemmPlan(A, B, D, flags=capi.FLAG_NO_CLUSTER_SPLIT).kernel_name
    # short K: a K group would not fill its pipeline
    A2 = torch.zeros((512, 256), dtype=torch.bfloat16, device=cuda)
    B2 = torch.zeros((256, 4096), dtype=torch.bfloat16, device=cuda)
    assert "kc2" not in capi.GemmPlan(A2, B2, D, flags=capi.FLAG_FORCE_CLUSTER_SPLIT).kernel_name


def test_more_tiles_than_clusters_queue(capi, oracle, cuda):
    """Forced onto a problem with more tiles than co-resident clusters: the clusters are independent
    of one another, so the extra ones simply start later."""
    plan = check(capi, oracle, "k2_compact", 2048, 2048, 1024, cuda, flags=capi.FLAG_FORCE_CLUSTER_SPLIT)
    assert "kc2" in plan.kernel_name


@pytest.mark.parametrize("shape", [(512, 2048, 4096), (200, 1008, 8208), (128, 256, 2048)])
def test_cluster_split_int32_bit_exact_and_repeatable(shape, capi, oracle, cuda):
    import torch
    M, N, K = shape
    rng = np.random.default_rng(7)
    A = rng.integers(-128, 128, (M, K), dtype=np.int8)
    B = rng.integers(-128, 128, (K, N), dtype=np.int8)
    want = oracle.gemm_s8(A, B)
    D = torch.empty((M, N), dtype=torch.int32, device=cuda)
    plan = capi.GemmPlan(torch.from_numpy(A).to(cuda), torch.from_numpy(B).to(cuda), D,
                         flags=capi.FLAG_FORCE_CLUSTER_SPLIT)
    assert "kc2" in plan.kernel_name, plan.kernel_name
    for _ in range(3):
        D.fill_(-7)
        plan.run()
        torch.cuda.synchronize()
        assert plan.device_status() == 0
        assert np.array_equal(D.cpu().numpy(), want), plan.kernel_name


def test_cluster_split_bf16_matches_whole_tiles_closely_and_repeats(capi, oracle, cuda):
    """fp32 partials of the two K halves are added once, in a fixed order: reruns are bit-identical,
    and the fp32 result differs from the whole-tile kernel's only by that one extra rounding."""
    import torch
    d = pc.make_inputs(oracle, "k1", 512, 2048, 4096, 9)
    A = torch.from_numpy(d["A"].view(np.int16)).view(torch.bfloat16).to(cuda)
    B = torch.from_numpy(d["B"].view(np.int16)).view(torch.bfloat16).to(cuda)
    D = torch.empty((512, 2048), dtype=torch.float32, device=cuda)
    plan = capi.GemmPlan(A, B, D, flags=capi.FLAG_FORCE_CLUSTER_SPLIT)
    assert "kc2" in plan.kernel_name
    outs = []
    for _ in range(3):
        D.zero_()
        plan.run()
        torch.cuda.synchronize()
        outs.append(D.cpu().numpy().copy())
    assert all(np.array_equal(outs[0], o) for o in outs[1:])
    D2 = torch.empty_like(D)
    whole = capi.GemmPlan(A, B, D2, flags=capi.FLAG_NO_CLUSTER_SPLIT | capi.FLAG_NO_SPLIT)
    whole.run()
    torch.cuda.synchronize()
    assert np.allclose(outs[0], D2.cpu().numpy(), rtol=0, atol=1e-4 * float(np.abs(outs[0]).max()))
