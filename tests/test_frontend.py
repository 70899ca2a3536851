"""The header-only C++ front end (xe-fuse_b200/include): xe_fuse::builder aliases, named kernel
structs, harness shims.

CPU: the lowering of every preset's visitor tree to the flat epilogue program; trees outside the
     program are refused; where the reference checkout is present, the text its generators emit and
     its own test mains compile and link UNMODIFIED against these headers.
GPU: a harness main in the reference's style runs each preset through the builder API and prints
     "Disposition: Passed".
"""
import os
import shutil
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CPP = os.path.join(ROOT, "tests", "cpp")
BUILD = os.path.join(CPP, "build")
FE = os.path.join(ROOT, "xe-fuse_b200", "include")
LIBDIR = os.path.join(ROOT, "xe-fuse_b200")
REF = os.environ.get("XEFUSE_REFERENCE_ROOT", "")   # a checkout of the reference, if any
CUDA = "/usr/local/cuda"


def _newest(path):
    t = 0
    for d, _, fs in os.walk(path):
        for f in fs:
            t = max(t, os.path.getmtime(os.path.join(d, f)))
    return t


def compile_cpp(src, out, syntax_only=False):
    cmd = ["g++", "-std=c++17", "-O1", "-fopenmp", "-I", FE, "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(CUDA, "include"), src]
    if syntax_only:
        cmd += ["-fsyntax-only"]
    else:
        cmd += ["-o", out, "-L", LIBDIR, "-lxefuse_b200", "-L", os.path.join(CUDA, "lib64"), "-lcudart",
                f"-Wl,-rpath,{LIBDIR}"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0, f"{' '.join(cmd)}\n{r.stdout[-4000:]}"


def built(name, capi):
    """Builds tests/cpp/<name>.cpp into tests/cpp/build/<name> when stale; returns the path."""
    os.makedirs(BUILD, exist_ok=True)
    src, out = os.path.join(CPP, name + ".cpp"), os.path.join(BUILD, name)
    newest = max(os.path.getmtime(src), _newest(FE), os.path.getmtime(os.path.join(ROOT, "include", "xefuse_b200.h")))
    if not os.path.exists(out) or os.path.getmtime(out) < newest:
        compile_cpp(src, out)
    return out


def parse_lowering(text):
    rows = {}
    for line in text.strip().splitlines():
        name, *kv = line.split()
        rows[name] = dict(x.split("=", 1) for x in kv)
    return rows


def test_lowering_of_every_preset_tree(capi):
    exe = built("lowering_check", capi)
    rows = parse_lowering(subprocess.check_output([exe], text=True))
    ok = lambda n: rows[n]["lower"] == "0" and rows[n]["can"] == "0"
    for n in ["k1", "k2", "k2_compact", "k8", "k3", "k4", "k4v2_table", "k0a", "k0_dual", "w8a8", "w8a8_biased",
              "w8a8_rope", "w8a8_swiglu", "w8a8_geglu", "bias_gelu", "scale_silu", "null_row", "bare", "bare_alpha2"]:
        assert ok(n), (n, rows[n])
    r = rows
    assert r["k1"]["row"] == "1@1000/1" and r["k1"]["pair"] == "0" and r["k1"]["tile"] == "256,256,32"
    assert r["k2"]["pair"] == "1" and r["k2"]["layout"] == "0" and r["k2_compact"]["layout"] == "1"
    assert r["k8"]["row"].startswith("0@") and r["k8"]["pair"] == "1"
    assert r["k3"]["pair"] == "3" and r["k3"]["cs"] == "4000" and r["k3"]["row"].startswith("0@")
    assert r["k4"]["pair"] == "3" and r["k4"]["row"] == "1@1000/1" and r["k4v2_table"]["period"] == "128"
    assert r["k0a"]["res"] == "1@5000" and r["k0a"]["col"] == "1@2000" and r["k0a"]["aux"] == "0@0"
    assert ok("k0a_cr") and r["k0a_cr"]["res"] == "1@5000" and r["k0a_cr"]["col"] == "1@2000"
    assert r["k0a_cr"]["sumsq"] == "7000" and ok("k0a_cr_null") and r["k0a_cr_null"]["sumsq"] == "0"
    assert r["k0_dual"]["aux"] == "1@6000" and r["k0_dual"]["res"] == "1@5000" and r["k0_dual"]["col"] == "1@2000"
    assert r["w8a8"]["ab"] == "1" and r["w8a8"]["row"] == "1@1000/1" and r["w8a8"]["col"] == "1@2000"
    assert r["w8a8_biased"]["bias"] == "1@3000"
    assert r["w8a8_rope"]["pair"] == "3" and r["w8a8_swiglu"]["pair"] == "1" and r["w8a8_geglu"]["pair"] == "2"
    assert r["bias_gelu"]["bias"] == "1@3000" and r["bias_gelu"]["unary"] == "1"
    assert r["scale_silu"]["unary"] == "3" and r["scale_silu"]["row"] == "1@1000/1"
    assert r["null_row"]["row"] == "1@0/0.5"            # null pointer -> null_default broadcast
    assert r["bare"]["row"].startswith("0@") and r["bare_alpha2"]["row"] == "1@0/2"
    # B is [K,N] row-major: ldb is the N extent although make_shape is called with (N,K,L)
    assert r["k1"]["lda"] == "128" and r["k1"]["ldb"] == "512" and r["k1"]["ldd"] == "512"
    for n in ["bad_beta", "bad_scale_after_unary", "bad_residual_after_scale", "bad_hadamard", "bad_acc_twice",
              "bad_cr_no_source", "bad_unused_source"]:
        assert rows[n]["lower"] == "5" and rows[n]["can"] == "5", (n, rows[n])   # kErrorNotSupported


def test_harness_compiles(capi):
    built("harness", capi)


needs_reference = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "autotune")),
                                     reason="reference checkout not present on this machine")


@needs_reference
def test_reference_generated_kernels_compile_unmodified(capi, tmp_path):
    """generate_kernel.py --preset <each> emits text that compiles and links against this front end."""
    presets = ["k1", "k3", "k4", "k4v2", "k0a", "k2", "k2_geglu", "k1v2", "k2v2", "k2v2_geglu",
               "w8a8_dequant", "w8a8_dequant_biased", "sa_scale_rows", "sa_residual_gamma", "sa_swiglu",
               "sa_rope_scaled"]
    for p in presets:
        src = tmp_path / f"{p}.cpp"
        subprocess.check_call([sys.executable, "generate_kernel.py", "--preset", p, "--output", str(src)],
                              cwd=os.path.join(REF, "autotune"), stdout=subprocess.DEVNULL)
        compile_cpp(str(src), str(tmp_path / p))
    # a tile picked by the reference's selector round-trips through --tile auto
    src = tmp_path / "k2_auto.cpp"
    subprocess.check_call([sys.executable, "generate_kernel.py", "--preset", "k2", "--tile", "auto", "--output",
                           str(src)], cwd=os.path.join(REF, "autotune"), stdout=subprocess.DEVNULL)
    compile_cpp(str(src), str(tmp_path / "k2_auto"))


@needs_reference
def test_reference_generated_pipelines_compile_unmodified(capi, tmp_path):
    """generate_pipeline.py (bf16 and W8A8, SwiGLU and GeGLU models) emits whole-layer benchmarks --
    fused stages, the engine-style arm (vllm_ops.hpp) and the naive arm -- that build as they are."""
    for preset, extra in [("llama3_8b", []), ("llama3_8b", ["--int8-mode", "w8a8"]), ("gemma2_9b", []),
                          ("llama3_70b", ["--autotune"])]:
        name = preset + "".join(extra).replace("-", "_")
        src = tmp_path / f"{name}.cpp"
        subprocess.check_call([sys.executable, "generate_pipeline.py", "--preset", preset, "--output", str(src)]
                              + extra, cwd=os.path.join(REF, "autotune"), stdout=subprocess.DEVNULL,
                              stderr=subprocess.DEVNULL)
        compile_cpp(str(src), str(tmp_path / name))


@needs_reference
def test_reference_test_mains_compile_unmodified(capi, tmp_path):
    """tests/test_k*.cpp and the MoE examples of the reference build against the front end as they are."""
    for t in ["tests/test_k1.cpp", "tests/test_k2.cpp", "tests/test_k3.cpp", "tests/test_k4.cpp",
              "tests/test_k0a.cpp", "tests/test_k0a_colred.cpp", "tests/test_k8.cpp", "tests/test_k2_w8a8.cpp",
              "tests/test_k4_w8a8.cpp",
              "examples/moe_expert_builder.cpp", "examples/moe_expert_fused.cpp"]:
        compile_cpp(os.path.join(REF, t), str(tmp_path / os.path.basename(t)[:-4]))


HARNESS_PRESETS = ["k1", "k1v2", "k2", "k2_compact", "k2_geglu", "k2v2", "k8", "k3", "k4", "k4v2", "k0a", "k0",
                   "bias_gelu", "w8a8", "w8a8_biased", "w8a8_rope", "w8a8_swiglu", "w8a8_geglu", "unsupported"]


@pytest.mark.gpu
@pytest.mark.parametrize("preset", HARNESS_PRESETS)
def test_harness_presets_on_gpu(preset, capi, cuda):
    exe = built("harness", capi)
    r = subprocess.run([exe, f"--preset={preset}", "--m=384", "--n=512", "--k=256"], stdout=subprocess.PIPE,
                       stderr=subprocess.STDOUT, text=True, timeout=300)
    assert r.returncode == 0 and "Disposition: Passed" in r.stdout, r.stdout[-3000:]


@pytest.mark.gpu
def test_harness_batched_moe_and_ragged_on_gpu(capi, cuda):
    exe = built("harness", capi)
    for args in (["--preset=moe", "--m=128", "--n=256", "--k=128", "--l=4"],
                 ["--preset=k4", "--m=200", "--n=328", "--k=136"],
                 ["--preset=w8a8_biased", "--m=200", "--n=336", "--k=208"]):
        r = subprocess.run([exe] + args, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
        assert r.returncode == 0 and "Disposition: Passed" in r.stdout, (args, r.stdout[-3000:])
