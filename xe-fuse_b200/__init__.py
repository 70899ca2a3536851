"""xe-fuse_b200: B200 (sm_100a) fused GEMM + epilogue kernels behind Xe-Fuse's builder API.

The directory name carries a hyphen (it mirrors the reference project's name), so it is loaded by
path: see `load()` in the repository's `xefuse_loader.py`, or

    import importlib.util, sys
    spec = importlib.util.spec_from_file_location("xefuse_b200", ".../xe-fuse_b200/__init__.py",
                                                  submodule_search_locations=[".../xe-fuse_b200"])

Contents:
  csrc/      hand-written CUDA (tcgen05 / TMEM / TMA) and the C ABI of include/xefuse_b200.h
  include/   header-only C++17 front end: xe_fuse::builder, xe_fuse::Gemm*, harness shims
  capi.py    ctypes binding used by the tests and bench.py
  sharding.py  column sharding of a stage over the GPUs of a box + the output all-gather
  build.py   nvcc build of libxefuse_b200.so
"""
from . import capi  # noqa: F401
from . import sharding  # noqa: F401
from .build import build  # noqa: F401
