"""The B200 tile selector behind the reference selector's interface, and the kernel runner."""
import importlib.util
import json
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _selector():
    p = os.path.join(ROOT, "xe-fuse_b200", "autotune", "tile_selector.py")
    spec = importlib.util.spec_from_file_location("xf_tile_selector", p)
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_select_tile_keeps_the_reference_interface():
    ts = _selector()
    gold = json.load(open(os.path.join(ROOT, "tests", "golden", "tile_selector.json")))
    extents = set()
    for s in gold["tiles"]:
        extents |= {int(x.strip().lstrip("_")) for x in s.split(",")}
    for g in gold["grid"]:                       # every (m, n, k, kernel) the fixture covers
        out = ts.select_tile(g["m"], g["n"], g["k"], g["kernel"])
        assert re.fullmatch(r"_\d+, _\d+, _\d+", out), out
        assert {int(x.strip().lstrip("_")) for x in out.split(",")} <= extents   # only known extents
    assert ts.select_tile(4096, 28672, 4096, "k2") == "_256, _256, _32"
    assert ts.select_tile(512, 4096, 4096, "k1") == "_128, _128, _32"
    assert ts.native_tile(8192, 8192, 28672, "s8") == (256, 256, 2, 256)


@pytest.mark.gpu
def test_selector_mirrors_the_library_choice(capi, cuda):
    import torch
    ts = _selector()
    sms = torch.cuda.get_device_properties(cuda).multi_processor_count
    for (M, N, K) in [(4096, 28672, 4096), (4096, 4096, 4096), (4096, 1024, 4096), (512, 4096, 4096),
                      (128, 512, 256), (8192, 3584, 4096), (1024, 2048, 1024), (4096, 7168, 4096),
                      (128, 4096, 4096), (4096, 512, 14336), (128, 256, 8192)]:
        for dt, tdt in (("bf16", torch.bfloat16), ("s8", torch.int8)):
            A = torch.zeros((M, K), dtype=tdt, device=cuda)
            B = torch.zeros((K, N), dtype=tdt, device=cuda)
            D = torch.zeros((M, N), dtype=torch.bfloat16, device=cuda)
            plan = capi.GemmPlan(A, B, D)
            # the library's name also carries the pipeline depth ("_s3"), which the mirror leaves out
            assert re.sub(r"_s\d+", "", plan.kernel_name) == ts.kernel_name(M, N, K, dt, sm_count=sms), (M, N, K, dt)
