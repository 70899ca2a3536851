"""Builds the reference's OWN harness programs, unmodified, against this repo's front end.

Test infrastructure, not product: nothing under xe-fuse_b200/ or bench.py's timed path uses it.

The reference (IntelLabs/Xe-Fuse) holds no golden vectors; what pins its arithmetic are the checks
inside its own programs: tests/test_k*.cpp rebuild the expected output with a naive device GEMM plus
a per-element lambda and compare at a relative tolerance (tests/test_k2.cpp:108-170,
tests/test_k4.cpp:127-179, tests/test_k4_w8a8.cpp:146-232), and the text generate_pipeline.py emits
verifies every stage the same way (autotune/pipeline_template.cpp.j2:345-488).  This script compiles
those sources WHERE THEY LIE in a checkout of the reference (nothing is copied into this repo) with
g++ against xe-fuse_b200/include and links them to libxefuse_b200.so.  The binaries land in
oracle/_ref/ (git-ignored), together with manifest.json; tests/test_reference_mains.py runs them
on a GPU and requires each program's own verdict to be "Passed".

Usage:  python oracle/build_ref_mains.py [--reference /path/to/Xe-Fuse] [--only NAME ...]
The reference root defaults to the XEFUSE_REFERENCE_ROOT environment variable.
"""
import argparse
import concurrent.futures
import json
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
OUT = os.path.join(HERE, "_ref")
FE = os.path.join(ROOT, "xe-fuse_b200", "include")
LIBDIR = os.path.join(ROOT, "xe-fuse_b200")
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")

# reference sources compiled as they are
TEST_MAINS = ["tests/test_k1.cpp", "tests/test_k2.cpp", "tests/test_k3.cpp", "tests/test_k4.cpp",
              "tests/test_k0a.cpp", "tests/test_k0a_colred.cpp", "tests/test_k8.cpp",
              "tests/test_k2_w8a8.cpp", "tests/test_k4_w8a8.cpp",
              "examples/moe_expert_builder.cpp", "examples/moe_expert_fused.cpp"]
# generate_kernel.py --preset <name>
KERNEL_PRESETS = ["k1", "k3", "k4", "k4v2", "k0a", "k2", "k2_geglu", "k1v2", "k2v2", "k2v2_geglu",
                  "w8a8_dequant", "w8a8_dequant_biased", "sa_scale_rows", "sa_residual_gamma",
                  "sa_swiglu", "sa_rope_scaled"]
# generate_pipeline.py --preset <model> [extra]
PIPELINES = [("llama3_8b", []), ("llama3_70b", []), ("gemma2_9b", []),
             ("llama3_8b", ["--int8-mode", "w8a8"]), ("llama3_70b", ["--int8-mode", "w8a8"]),
             ("gemma2_9b", ["--int8-mode", "w8a8"]), ("llama3_70b", ["--autotune"])]


def compile_one(src, out):
    cmd = ["g++", "-std=c++17", "-O2", "-fopenmp", "-I", FE, "-I", os.path.join(ROOT, "include"),
           "-I", os.path.join(CUDA, "include"), src, "-o", out, "-L", LIBDIR, "-lxefuse_b200",
           "-L", os.path.join(CUDA, "lib64"), "-lcudart",
           "-Wl,-rpath,$ORIGIN/../../xe-fuse_b200", f"-Wl,-rpath,{os.path.join(CUDA, 'lib64')}"]
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    return r.returncode, r.stdout[-3000:]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("XEFUSE_REFERENCE_ROOT", ""))
    ap.add_argument("--only", nargs="*", default=None, help="build only these output names")
    a = ap.parse_args()
    ref = a.reference
    if not ref or not os.path.isdir(os.path.join(ref, "autotune")):
        sys.exit("no reference checkout: pass --reference or set XEFUSE_REFERENCE_ROOT")
    if not os.path.exists(os.path.join(LIBDIR, "libxefuse_b200.so")):
        sys.exit("build the library first: python xe-fuse_b200/build.py")
    os.makedirs(OUT, exist_ok=True)
    gen = tempfile.mkdtemp(prefix="xf_refgen_")
    jobs = []   # (name, kind, origin, source path)
    for t in TEST_MAINS:
        jobs.append(("ref_" + os.path.basename(t)[:-4], "main", t, os.path.join(ref, t)))
    for p in KERNEL_PRESETS:
        src = os.path.join(gen, f"gen_{p}.cpp")
        subprocess.check_call([sys.executable, "generate_kernel.py", "--preset", p, "--output", src],
                              cwd=os.path.join(ref, "autotune"), stdout=subprocess.DEVNULL)
        jobs.append((f"gen_{p}", "generated_kernel", f"autotune/generate_kernel.py --preset {p}", src))
    for model, extra in PIPELINES:
        name = "pipe_" + model + "".join("_" + e.strip("-").replace("-", "_") for e in extra)
        src = os.path.join(gen, name + ".cpp")
        subprocess.check_call([sys.executable, "generate_pipeline.py", "--preset", model, "--output", src] + extra,
                              cwd=os.path.join(ref, "autotune"), stdout=subprocess.DEVNULL,
                              stderr=subprocess.DEVNULL)
        jobs.append((name, "generated_pipeline",
                     f"autotune/generate_pipeline.py --preset {model} {' '.join(extra)}".strip(), src))
    if a.only is not None:
        jobs = [j for j in jobs if j[0] in a.only]
    manifest, failed = [], []
    with concurrent.futures.ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        futs = {ex.submit(compile_one, j[3], os.path.join(OUT, j[0])): j for j in jobs}
        for f in concurrent.futures.as_completed(futs):
            name, kind, origin, _ = futs[f]
            rc, log = f.result()
            if rc != 0:
                failed.append((name, log))
            else:
                manifest.append({"name": name, "kind": kind, "origin": origin})
    manifest.sort(key=lambda m: m["name"])
    mpath = os.path.join(OUT, "manifest.json")
    if a.only is not None and os.path.exists(mpath):
        old = {m["name"]: m for m in json.load(open(mpath))}
        old.update({m["name"]: m for m in manifest})
        manifest = sorted(old.values(), key=lambda m: m["name"])
    json.dump(manifest, open(mpath, "w"), indent=1)
    for name, log in failed:
        sys.stderr.write(f"--- {name} failed to build\n{log}\n")
    print(f"{len(manifest)} programs in {OUT}; {len(failed)} failed to build")
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
