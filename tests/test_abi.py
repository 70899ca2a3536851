"""CPU-only checks of the C ABI: the shared library loads, exports every symbol the header
declares, and the host-side argument validation returns the documented status codes (these entry
points never touch the GPU)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "xefuse_b200.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"XF_API\s+[\w\s\*]+?\b(xf_\w+)\s*\(", text)))


def test_header_declares_what_the_binding_lists(capi):
    assert declared_symbols() == sorted(capi.EXPORTS)


def test_library_exports_every_declared_symbol(capi):
    L = capi.lib()
    for name in declared_symbols():
        assert hasattr(L, name), f"{name} declared in include/xefuse_b200.h but not exported"
    assert L.xf_version() >= 100
    assert L.xf_compiled_arch() == 100


def test_struct_layout_matches_header(capi):
    # sizes the C compiler gives the PODs (LP64): guards the ctypes mirrors against drift
    import subprocess
    import tempfile
    src = '#include "xefuse_b200.h"\n#include <stdio.h>\nint main(){printf("%zu %zu %zu %zu\\n",' \
          'sizeof(xf_vec),sizeof(xf_mat),sizeof(xf_epilogue_desc),sizeof(xf_gemm_desc));return 0;}\n'
    with tempfile.TemporaryDirectory() as td:
        c = os.path.join(td, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(td, "s")
        subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe])
        sizes = list(map(int, subprocess.check_output([exe]).split()))
    assert sizes == [C.sizeof(capi.XfVec), C.sizeof(capi.XfMat), C.sizeof(capi.XfEpilogueDesc),
                     C.sizeof(capi.XfGemmDesc)]


def base_desc(capi):
    d = capi.XfGemmDesc()
    d.dtype_ab, d.dtype_d = capi.DT_BF16, capi.DT_BF16
    d.M, d.N, d.K, d.L = 256, 512, 128, 1
    d.A, d.lda = 0x10000, 128
    d.B, d.ldb = 0x20000, 512
    d.D, d.ldd = 0x30000, 512
    return d


def status(capi, d):
    return capi.lib().xf_gemm_can_implement(C.byref(d))


def test_can_implement_accepts_a_plain_problem(capi):
    assert status(capi, base_desc(capi)) == 0


@pytest.mark.parametrize("mutate,code", [
    (lambda d: setattr(d, "M", 0), 4),                 # invalid problem
    (lambda d: setattr(d, "A", None), 4),
    (lambda d: setattr(d, "dtype_ab", 2), 2),          # fp32 inputs: invalid data type
    (lambda d: setattr(d, "lda", 64), 3),              # lda < K: invalid layout
    (lambda d: setattr(d, "lda", 132), 1),             # 264-byte pitch: misaligned operand
    (lambda d: setattr(d, "B", 0x20002), 1),           # unaligned base
    (lambda d: setattr(d, "ldd", 100), 3),             # ldd < N
    (lambda d: setattr(d, "dtype_d", 3), 5),           # int32 out from bf16 in: not supported
    (lambda d: setattr(d.epi, "pair", 9), 5),
    (lambda d: setattr(d.epi, "out_layout", 1), 5),    # compact without a gated pair op
])
def test_can_implement_rejections(capi, mutate, code):
    d = base_desc(capi)
    mutate(d)
    assert status(capi, d) == code
    assert capi.lib().xf_last_error_string()  # a reason is recorded


def test_pair_ops_need_even_n_and_rope_needs_a_table(capi):
    d = base_desc(capi)
    d.N, d.ldb, d.ldd = 504, 504, 504
    d.epi.pair = capi.PAIR["swiglu"]
    assert status(capi, d) == 0
    d.N = 503
    assert status(capi, d) == 4
    d = base_desc(capi)
    d.epi.pair = capi.PAIR["rope"]
    assert status(capi, d) == 4                         # cos_sin pointer missing
    d.epi.cos_sin.ptr, d.epi.cos_sin.dtype, d.epi.cos_sin.ld = 0x40000, capi.DT_F32, 512
    assert status(capi, d) == 0
    d.epi.cos_sin_period, d.epi.cos_sin.ld = 48, 48     # period must be a multiple of 32
    assert status(capi, d) == 5
    d.epi.cos_sin_period, d.epi.cos_sin.ld = 128, 128
    assert status(capi, d) == 0


def test_int8_alignment_is_sixteen_elements(capi):
    d = base_desc(capi)
    d.dtype_ab = capi.DT_S8
    d.lda, d.K = 136, 136    # 136 bytes: not a multiple of 16
    assert status(capi, d) == 1
    d.lda, d.K = 144, 144
    assert status(capi, d) == 0
    d.dtype_d = capi.DT_S32  # raw accumulators allowed for int8 with an empty epilogue
    assert status(capi, d) == 0
    d.epi.row_scale.enabled = 1
    d.epi.row_scale.dtype = capi.DT_F32
    assert status(capi, d) == 5


def test_workspace_size_and_status_strings(capi):
    L = capi.lib()
    d = base_desc(capi)
    n = C.c_size_t(123)
    assert L.xf_gemm_workspace_size(C.byref(d), C.byref(n)) == 0 and n.value == 16
    assert L.xf_status_string(0) == b"Success"
    assert L.xf_status_string(1) == b"Error Misaligned Operand"
    assert L.xf_status_string(5) == b"Error Not Supported"
    assert L.xf_gemm_run(None, None) == 4


def test_every_reference_tile_string_is_a_valid_hint(capi):
    """tile_selector's 30 Xe tile strings are hints; any of them must be accepted."""
    import json
    t = json.load(open(os.path.join(ROOT, "tests", "golden", "tile_selector.json")))
    for s in t["tiles"]:
        tm, tn, tk = [int(x.strip().lstrip("_")) for x in s.split(",")]
        d = base_desc(capi)
        d.tile_m, d.tile_n, d.tile_k = tm, tn, tk
        assert status(capi, d) == 0, s


def test_plan_create_without_gpu_fails_loudly(capi):
    """No CPU fallback: on a box without a B200 plan creation reports an error, never success."""
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present: covered by the gpu tests")
    d = base_desc(capi)
    h = C.c_void_p()
    rc = capi.lib().xf_gemm_plan_create(C.byref(d), None, C.byref(h))
    assert rc != 0 and not h.value


def test_diagnostic_flags_need_an_opt_in(capi, monkeypatch):
    """The XF_FLAG_DIAG_* flags leave D garbage: refused unless the environment opts in."""
    d = base_desc(capi)
    d.flags = capi.FLAG_DIAG_NO_MMA
    monkeypatch.delenv("XEFUSE_ALLOW_DIAG", raising=False)
    assert status(capi, d) == 5
    assert b"XEFUSE_ALLOW_DIAG" in capi.lib().xf_last_error_string()
    monkeypatch.setenv("XEFUSE_ALLOW_DIAG", "1")
    assert status(capi, d) == 0
    d.flags = capi.FLAG_NO_CLUSTER_SPLIT | capi.FLAG_NO_TAIL_STAGING | capi.FLAG_NO_ACC_PREFETCH   # plain tuning flags
    monkeypatch.delenv("XEFUSE_ALLOW_DIAG", raising=False)
    assert status(capi, d) == 0


def test_static_workspace_entries_reject_null_arguments(capi):
    L = capi.lib()
    assert L.xf_gemm_run_static_workspace(None, None) == 4
    assert L.xf_gemm_static_workspace_status(None) == 4
    assert L.xf_gemm_cluster_capacity(capi.DT_F32, None, None) == 4
