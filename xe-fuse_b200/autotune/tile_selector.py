"""B200 tile selection, behind the reference selector's interface.

`select_tile(M, N, K, kernel="bare", groups=1) -> str` keeps the signature and the return format
(a `cute::Shape<>` argument string such as "_256, _256, _32") of the reference's
autotune/tile_selector.py:48, so generate_kernel.py / generate_pipeline.py can import this module
in its place.  On B200 the TileShape of a kernel is only a hint: the library maps it to a native
CTA tile.  `native_tile()` mirrors that choice (select_variant in csrc/xf_gemm.cu): the cost of a
variant is waves x tile area / measured efficiency, over the compiled variants; the tiles of a
partly filled last wave are cut into K slices (split_factor), which shortens that wave

    (columns, CTAs per tile, 128-byte K slabs per stage): rows = 128 x CTAs

The efficiencies were measured on a 4096 x 28672 x 4096 bf16 GEMM on B200.
"""
from math import ceil

SM_COUNT = 148

# (bn, ctas, ks) -> relative throughput; order = the library's variant table
BF16_VARIANTS = [((256, 2, 1), 0.91), ((256, 2, 2), 1.00), ((256, 1, 1), 0.84), ((128, 2, 1), 0.48),
                 ((128, 2, 2), 0.67), ((128, 1, 1), 0.55), ((128, 1, 2), 0.72)]
S8_VARIANTS = [((256, 2, 1), 0.91), ((256, 2, 2), 1.00), ((256, 1, 1), 0.84), ((128, 1, 1), 0.55),
               ((128, 1, 2), 0.72)]


MAX_SPLIT, MIN_KB_PER_SLICE = 8, 4


def tile_time_us(bn, eff, K, es):
    """Microseconds one scheduling unit spends on one tile (tile_time_us in csrc/xf_gemm.cu)."""
    return (2.0 + 0.0029 * K * es) * (bn / 256.0) / eff


def split_overhead_us(bn, whole_waves):
    """Cost of passing the partial accumulators through L2; partly hidden behind the next tile when
    the unit has whole tiles to run after its slice."""
    if whole_waves:
        return 7.0 if bn == 256 else 5.0
    return 10.0 if bn == 256 else 7.0


def split_factor(tiles, units, K, es, bn, ks, eff, compact=False):
    """K slices per tile of the remainder wave (0 = whole tiles); split_factor in csrc/xf_gemm.cu."""
    rem = tiles % units
    if rem == 0:
        return 0
    num_kb = ceil(K / ((128 // es) * ks))
    s = min(units // rem, num_kb // MIN_KB_PER_SLICE, MAX_SPLIT, bn // (64 if compact else 32))
    if s < 2:
        return 0
    return s if tile_time_us(bn, eff, K, es) * (1.0 - 1.0 / s) > split_overhead_us(bn, tiles >= units) else 0


def native_tile(M, N, K, dtype="bf16", L=1, sm_count=SM_COUNT, compact=False, with_split=False):
    """(rows, columns, ctas, k_elements_per_stage) of the kernel variant the library picks; with
    with_split also the number of K slices the tiles of the remainder wave are cut into."""
    best, best_cost, best_split = None, None, 0
    es = 1 if dtype in ("s8", "int8") else 2
    for (bn, ctas, ks), eff in (S8_VARIANTS if es == 1 else BF16_VARIANTS):
        tiles = ceil(M / (128 * ctas)) * ceil(N / bn) * L
        units = sm_count // ctas
        split = split_factor(tiles, units, K, es, bn, ks, eff, compact)
        t = tile_time_us(bn, eff, K, es)
        cost = (tiles // units) * t
        if tiles % units:
            cost += (t / split + split_overhead_us(bn, tiles >= units)) if split else t
        if best is None or cost < best_cost * 0.999:
            best, best_cost, best_split = (bn, ctas, ks), cost, split
    bn, ctas, ks = best
    kslab = 128 // es
    if with_split:
        return 128 * ctas, bn, ctas, ks * kslab, best_split
    return 128 * ctas, bn, ctas, ks * kslab


def kernel_name(M, N, K, dtype="bf16", L=1, sm_count=SM_COUNT, compact=False):
    """Name the library reports for that variant (xf_gemm_plan_kernel_name without the stage count)."""
    rows, bn, ctas, kstage, split = native_tile(M, N, K, dtype, L, sm_count, compact, with_split=True)
    name = f"{'s8' if dtype in ('s8', 'int8') else 'bf16'}_{rows}x{bn}_cta{ctas}_k{kstage}"
    return name + (f"_ksplit{split}" if split else "")


def select_tile(M: int, N: int, K: int, kernel: str = "bare", groups: int = 1) -> str:
    """TileShape string for the kernel generators: the native (rows, columns) with the reference's
    K extent of 32 -- every value is one of the extents the reference's tile list uses."""
    dtype = "s8" if "w8a8" in kernel else "bf16"
    rows, bn, _, _ = native_tile(M, N, K, dtype)
    return f"_{rows}, _{bn}, _32"
