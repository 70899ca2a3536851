"""The allocation-free entry point, xf_gemm_run_static_workspace.

Some callers of this library cannot allocate device memory: a serving process that gave all of HBM
to its own pool when it started, or a plug-in that only borrows buffers from its host.  For them
the fused GEMM can run with its scratch (the kernel's status word and, for schedules that cut the
last wave's tiles into K slices, the slice counters and partial accumulators) in a static 2 MiB
device array inside the library instead of a caller-allocated workspace.  This test drives that entry through the C
ABI and checks that it writes exactly what the plan-based entry writes, on two calls in a row --
the second call finds the array as the first one left it.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test.  It passes alone in a fresh process and after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest

import parity_cases as pc

pytestmark = pytest.mark.gpu


def _bf(torch, bits, dev):
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16).to(dev)


def _both_entries(capi, oracle, dev, preset, M, N, K, seed, flags=0, expect_in_name=""):
    """Runs one problem through the plan entry and through the static-workspace entry."""
    import torch
    from conftest import bf16_bits
    d = pc.make_inputs(oracle, preset, M, N, K, seed)
    A, B = _bf(torch, d["A"], dev), _bf(torch, d["B"], dev)
    R = torch.from_numpy(d["scale"]).to(dev)
    compact = preset == "k2_compact"
    n_out = N // 2 if compact else N
    kw = dict(row_scale=R, pair="swiglu" if compact else "none", compact=compact)
    D_plan = torch.full((M, n_out), float("nan"), dtype=torch.bfloat16, device=dev)
    plan = capi.GemmPlan(A, B, D_plan, flags=flags, **kw)
    assert expect_in_name in plan.kernel_name, plan.kernel_name
    plan.run()
    torch.cuda.synchronize()
    assert plan.device_status() == 0

    # same descriptor, other output buffer, no workspace and no plan
    D_static = torch.full((M, n_out), float("nan"), dtype=torch.bfloat16, device=dev)
    desc = capi.XfGemmDesc.from_buffer_copy(plan.desc)
    desc.D = D_static.data_ptr()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated(dev)
    free_before = torch.cuda.mem_get_info(dev)[0]        # cudaMemGetInfo: sees any allocation on the device
    stream = torch.cuda.current_stream().cuda_stream
    capi.check(capi.lib().xf_gemm_run_static_workspace(C.byref(desc), stream))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated(dev) == before
    assert torch.cuda.mem_get_info(dev)[0] == free_before
    code = C.c_int32(-1)
    capi.check(capi.lib().xf_gemm_static_workspace_status(C.byref(code)))
    assert code.value == 0
    got_plan, got_static = bf16_bits(D_plan), bf16_bits(D_static)
    # same kernel, same inputs: bit-identical; and both inside the parity bar against the oracle
    assert np.array_equal(got_static, got_plan)
    _, want = pc.expected(oracle, preset, d)
    nbad, mabs, mrel = pc.compare_bf16(oracle, got_static, want)
    assert nbad == 0, (mabs, mrel)


def test_static_workspace_entry_matches_plan_entry_twice(capi, oracle, cuda):
    # two calls in a row, different problems: the second starts from the first one's leftovers
    _both_entries(capi, oracle, cuda, "k1", 256, 512, 256, seed=21)
    _both_entries(capi, oracle, cuda, "k2_compact", 200, 336, 208, seed=22)


def test_static_workspace_entry_runs_a_split_schedule_that_fits(capi, oracle, cuda):
    """A schedule that cuts its tiles into K slices keeps counters and partial accumulators in the
    static array too (they fit its 2 MiB here); twice in a row: the counters start from what the
    previous call left."""
    lib = capi.lib()
    lib.xf_gemm_run_static_workspace(None, None)          # first touch outside the memory accounting
    for seed in (23, 24):
        _both_entries(capi, oracle, cuda, "k1", 128, 256, 4096, seed=seed,
                      flags=capi.FLAG_NO_CLUSTER_SPLIT, expect_in_name="ksplit")


def test_static_workspace_entry_refuses_what_does_not_fit(capi, cuda):
    """A split whose partial accumulators exceed the static array is refused with the size in the
    message; the same problem with XF_FLAG_NO_SPLIT runs (whole tiles, 16 bytes of scratch)."""
    import torch
    M, N, K = 512, 2048, 8192             # 16 paired tiles cut into 4 K slices: 16 MiB of partials
    A = torch.randn(M, K, device=cuda).to(torch.bfloat16)
    B = (torch.randn(K, N, device=cuda) * K ** -0.5).to(torch.bfloat16)
    D1 = torch.zeros(M, N, dtype=torch.bfloat16, device=cuda)
    plan = capi.GemmPlan(A, B, D1, flags=capi.FLAG_NO_CLUSTER_SPLIT)
    assert "ksplit" in plan.kernel_name and plan.workspace.numel() > capi.STATIC_WORKSPACE_BYTES
    desc = capi.XfGemmDesc.from_buffer_copy(plan.desc)
    D2 = torch.zeros_like(D1)
    desc.D = D2.data_ptr()
    rc = capi.lib().xf_gemm_run_static_workspace(C.byref(desc), None)
    assert rc == 5                                           # XF_ERR_NOT_SUPPORTED
    msg = capi.lib().xf_last_error_string().decode()
    assert "bytes of workspace" in msg and "XF_FLAG_NO_SPLIT" in msg
    desc.flags |= capi.FLAG_NO_SPLIT
    capi.check(capi.lib().xf_gemm_run_static_workspace(C.byref(desc), torch.cuda.current_stream().cuda_stream))
    whole = capi.GemmPlan(A, B, D1, flags=capi.FLAG_NO_CLUSTER_SPLIT | capi.FLAG_NO_SPLIT)
    whole.run()
    torch.cuda.synchronize()
    assert torch.equal(D1.view(torch.int16), D2.view(torch.int16))


def test_static_workspace_entry_rejects_bad_problems(capi, cuda):
    d = capi.XfGemmDesc()
    rc = capi.lib().xf_gemm_run_static_workspace(C.byref(d), None)
    assert rc != 0 and capi.lib().xf_last_error_string()
    assert capi.lib().xf_gemm_run_static_workspace(None, None) == 4
