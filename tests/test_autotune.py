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
    assert ts.select_tile(512, 4096, 4096, "k1") == "_256, _256, _32"      # cluster split-K variant
    assert ts.kernel_name(512, 4096, 4096) == "bf16_256x256_cta2_k128_kc2"
    assert ts.native_tile(8192, 8192, 28672, "s8") == (256, 256, 2, 256)


@pytest.mark.gpu
def test_selector_mirrors_the_library_choice(capi, cuda):
    import torch
    ts = _selector()
    sms = torch.cuda.get_device_properties(cuda).multi_processor_count
    cap = {"bf16": capi.cluster_capacity(capi.DT_BF16), "s8": capi.cluster_capacity(capi.DT_S8)}
    for (M, N, K) in [(4096, 28672, 4096), (4096, 4096, 4096), (4096, 1024, 4096), (512, 4096, 4096),
                      (128, 512, 256), (8192, 3584, 4096), (1024, 2048, 1024), (4096, 7168, 4096),
                      (128, 4096, 4096), (4096, 512, 14336), (128, 256, 8192)]:
        for dt, tdt in (("bf16", torch.bfloat16), ("s8", torch.int8)):
            A = torch.zeros((M, K), dtype=tdt, device=cuda)
            B = torch.zeros((K, N), dtype=tdt, device=cuda)
            D = torch.zeros((M, N), dtype=torch.bfloat16, device=cuda)
            plan = capi.GemmPlan(A, B, D)
            # the library's name also carries the pipeline depth ("_s3"), which the mirror leaves out
            want = ts.kernel_name(M, N, K, dt, sm_count=sms, pairs=cap[dt][0], quads=cap[dt][1])
            assert re.sub(r"_s\d+(?=_|$)", "", plan.kernel_name) == want, (M, N, K, dt)


def test_split_planner_invariants():
    """The Python mirror of the planner over a sweep of shapes: a split factor is 0 or 2..8, leaves
    at least 4 K blocks per slice, never creates more slice items than scheduling units, and each
    slice finishes whole 32-output-column units of its tile."""
    ts = _selector()
    import itertools
    seen_split = 0
    for M, N, K in itertools.product([128, 512, 2048, 4096, 8192], [256, 1024, 3584, 7168, 28672],
                                     [256, 1024, 4096, 14336]):
        for dt, es, variants in (("bf16", 2, ts.BF16_VARIANTS), ("s8", 1, ts.S8_VARIANTS)):
            rows, bn, ctas, kstage, split, kc = ts.native_tile(M, N, K, dt, with_split=True)
            if kc > 1:        # cluster split-K: whole tiles, one per cluster, no global split
                assert split == 0 and -(-M // rows) * -(-N // bn) <= ts.SM_COUNT // 4
                assert -(-K // kstage) >= ts.MIN_KB_PER_GROUP * kc
                continue
            units = ts.SM_COUNT // ctas
            tiles = -(-M // rows) * -(-N // bn)
            if split:
                seen_split += 1
                num_kb = -(-K // kstage)
                assert 2 <= split <= 8 and num_kb // split >= 4, (M, N, K, dt, split)
                assert (tiles % units) * split <= units
            else:
                assert split == 0
    assert seen_split > 20


def test_work_item_order_covers_every_item_once():
    """Model of the kernel's schedule (schedule_item in csrc/xf_gemm_kernel.cuh): unit u runs items
    u, u+U, ...; a unit that owns a K slice runs it first.  Every whole tile and every slice is run
    exactly once, and a unit's slice comes before all of its whole tiles."""
    def order(unit, U, split_first, total_items, split_s):
        out = []
        for w in range(unit, total_items, U):
            if split_s == 0 or unit >= total_items - split_first or split_first == 0:
                out.append(w)
            else:
                out.append(split_first + unit if w == unit else w - U)
        return out
    for T, U, S in [(224, 74, 8), (448, 74, 8), (1792, 74, 4), (256, 74, 2), (32, 74, 2), (1, 148, 8), (75, 74, 8),
                    (148, 148, 0), (300, 148, 0)]:
        rem = T % U
        split_tiles = rem if S else 0
        split_first = T - split_tiles
        total_items = split_first + split_tiles * max(S, 1)
        units = min(total_items, U)
        ran = []
        for u in range(units):
            o = order(u, units, split_first, total_items, S)
            ran += o
            slices = [w for w in o if S and w >= split_first]
            assert len(slices) <= 1 and (not slices or o[0] == slices[0]), (T, U, S, u, o)
        assert sorted(ran) == list(range(total_items)), (T, U, S)
