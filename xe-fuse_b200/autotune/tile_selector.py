"""B200 tile selection, behind the reference selector's interface.

`select_tile(M, N, K, kernel="bare", groups=1) -> str` keeps the signature and the return format
(a `cute::Shape<>` argument string such as "_256, _256, _32") of the reference's
autotune/tile_selector.py:48, so generate_kernel.py / generate_pipeline.py can import this module
in its place.  On B200 the TileShape of a kernel is only a hint: the library maps it to a native
CTA tile.  `native_tile()` mirrors that choice (select_variant in csrc/xf_gemm.cu): the cost of a
variant is waves x tile area / measured efficiency, over the compiled variants; the tiles of a
partly filled last wave are cut into K slices (split_factor), which shortens that wave; problems
of at most one 256 x 256 tile per four SMs may run a cluster split-K variant (two CTA pairs per
tile, partial accumulators swapped through distributed shared memory)

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
# cluster split-K variant: K groups per cluster, exchange cost, K blocks each group needs
CLUSTER_KC, CLUSTER_EXCHANGE_US, MIN_KB_PER_GROUP = 2, 1.0, 4


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
    s = min(units // rem, num_kb // MIN_KB_PER_SLICE, MAX_SPLIT)
    if s < 2:
        return 0
    return s if tile_time_us(bn, eff, K, es) * (1.0 - 1.0 / s) > split_overhead_us(bn, tiles >= units) else 0


def _choose(M, N, K, dtype, L, sm_count, compact, pairs, quads):
    """((bn, ctas, ks), K slices of the remainder wave, K groups per cluster)."""
    best, best_cost, best_split, best_kc = None, None, 0, 1
    es = 1 if dtype in ("s8", "int8") else 2
    pairs = sm_count // 2 if pairs is None else pairs
    quads = sm_count // 4 if quads is None else quads
    order = list(S8_VARIANTS if es == 1 else BF16_VARIANTS)
    for entry, eff in order + [((256, 2, 2, CLUSTER_KC), 1.00)]:   # the library's table order
        bn, ctas, ks = entry[:3]
        kc = entry[3] if len(entry) > 3 else 1
        tiles = ceil(M / (128 * ctas)) * ceil(N / bn) * L
        if kc > 1:
            num_kb = ceil(K / ((128 // es) * ks))
            if num_kb < MIN_KB_PER_GROUP * kc or tiles > quads:
                continue
            cost, split = tile_time_us(bn, eff, ceil(K / kc), es) + CLUSTER_EXCHANGE_US, 0
        else:
            units = pairs if ctas == 2 else sm_count
            split = split_factor(tiles, units, K, es, bn, ks, eff, compact)
            t = tile_time_us(bn, eff, K, es)
            cost = (tiles // units) * t
            if tiles % units:
                cost += (t / split + split_overhead_us(bn, tiles >= units)) if split else t
        if best is None or cost < best_cost * 0.999:
            best, best_cost, best_split, best_kc = (bn, ctas, ks), cost, split, kc
    return best, best_split, best_kc


def native_tile(M, N, K, dtype="bf16", L=1, sm_count=SM_COUNT, compact=False, with_split=False,
                pairs=None, quads=None):
    """(rows, columns, ctas, k_elements_per_stage) of the kernel variant the library picks; with
    with_split also the number of K slices the tiles of the remainder wave are cut into and the
    number of K groups per cluster (1 = no cluster split-K).  `pairs` / `quads`: the CTA pairs and
    4-CTA clusters the device holds at once (xf_gemm_cluster_capacity); default sm_count / 2, / 4."""
    (bn, ctas, ks), split, kc = _choose(M, N, K, dtype, L, sm_count, compact, pairs, quads)
    kslab = 128 // (1 if dtype in ("s8", "int8") else 2)
    if with_split:
        return 128 * ctas, bn, ctas, ks * kslab, split, kc
    return 128 * ctas, bn, ctas, ks * kslab


def kernel_name(M, N, K, dtype="bf16", L=1, sm_count=SM_COUNT, compact=False, pairs=None, quads=None):
    """Name the library reports for that variant (xf_gemm_plan_kernel_name without the stage count)."""
    rows, bn, ctas, kstage, split, kc = native_tile(M, N, K, dtype, L, sm_count, compact, with_split=True,
                                                    pairs=pairs, quads=quads)
    name = f"{'s8' if dtype in ('s8', 'int8') else 'bf16'}_{rows}x{bn}_cta{ctas}_k{kstage}"
    return name + (f"_kc{kc}" if kc > 1 else "") + (f"_ksplit{split}" if split else "")


def select_tile(M: int, N: int, K: int, kernel: str = "bare", groups: int = 1) -> str:
    """TileShape string for the kernel generators: the native (rows, columns) with the reference's
    K extent of 32 -- every value is one of the extents the reference's tile list uses."""
    dtype = "s8" if "w8a8" in kernel else "bf16"
    rows, bn, _, _ = native_tile(M, N, K, dtype)
    return f"_{rows}, _{bn}, _32"
