"""Generates the golden fixtures under tests/golden/ by IMPORTING the reference's own Python
(autotune/*.py of IntelLabs/Xe-Fuse).  Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/Xe-Fuse

The fixtures are committed; the tests read only the fixtures.  What can be pinned this way is what
the reference implements in Python: its tile selector (every tile string the selector can emit has
to be accepted as a TileShape hint), its model-shape presets (the GEMM shapes of the benchmark
configurations), the preset table of the kernel generator (EVT alias spelling + aux buffers per preset; the
generator's emitted argument code is NOT stored)
and its offline per-column int8 weight quantiser.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "autotune"))
    import generate_kernel as gk
    import model_presets as mp
    import quantize_weights_quaRot as qw
    import tile_selector as ts

    # 1. tile selector: the tile list and a grid of decisions
    grid = []
    for kernel in ["k0a", "k1", "k2", "k3", "k4"]:
        for m in [1, 8, 16, 64, 128, 512, 1024, 4096, 8192, 16384]:
            for n, k in [(1024, 4096), (4096, 4096), (8192, 8192), (14336, 4096), (28672, 4096),
                         (57344, 8192), (8192, 28672)]:
                grid.append({"m": m, "n": n, "k": k, "kernel": kernel,
                             "tile": ts.select_tile(m, n, k, kernel)})
    tiles = ts.TILES if hasattr(ts, "TILES") else sorted({g["tile"] for g in grid})
    tiles = list(tiles.values()) if isinstance(tiles, dict) else list(tiles)
    with open(os.path.join(HERE, "tile_selector.json"), "w") as f:
        json.dump({"tiles": tiles, "grid": grid}, f, indent=0, sort_keys=True)

    # 2. model presets
    with open(os.path.join(HERE, "model_presets.json"), "w") as f:
        json.dump(mp.MODEL_PRESETS, f, indent=1, sort_keys=True)

    # 3. kernel-generator presets: EVT typedef text, aux buffers, element types
    presets = {}
    for name, p in gk.PRESETS.items():
        presets[name] = {k: p[k] for k in p if k in (
            "name", "evt_description", "tile_shape", "evt_typedefs", "aux_data",
            "element_a", "element_b", "element_d", "element_acc", "element_compute",
            "alignment_ab", "alignment_cd")}
    sa = {name: {k: v for k, v in p.items() if k in ("name", "evt_description", "aux_data", "standalone")}
          for name, p in gk.STANDALONE_PRESETS.items()}
    with open(os.path.join(HERE, "kernel_presets.json"), "w") as f:
        json.dump({"presets": presets, "standalone": sa}, f, indent=1, sort_keys=True)

    # 4. offline per-column int8 quantiser on seeded weights
    rng = np.random.default_rng(1234)
    W = (rng.standard_normal((96, 40)) / np.sqrt(96)).astype(np.float32)
    W[:, 7] = 0.0  # an all-zero column exercises the zero-scale guard
    Wq, sc = qw.quantize_columns(W)
    np.savez_compressed(os.path.join(HERE, "quantize_columns.npz"), W=W, Wq=Wq, scale=sc)
    print("wrote fixtures to", HERE)


if __name__ == "__main__":
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("XEFUSE_REFERENCE_ROOT")
    if not ref_root:
        sys.exit("usage: make_golden.py <reference checkout>   (or set XEFUSE_REFERENCE_ROOT)")
    main(ref_root)
