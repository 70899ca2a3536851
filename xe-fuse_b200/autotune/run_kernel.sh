#!/bin/bash
# Compile one generated kernel (.cpp written by the reference's generate_kernel.py /
# generate_pipeline.py, or by hand against xe_fuse::builder) with the B200 front end and run it.
# Counterpart of the reference's autotune/run_kernel.sh (icpx + Intel Xe): same BUILD:/SPILLS:
# lines, so tooling that parses them keeps working.
#
#   usage: run_kernel.sh kernel.cpp [args passed to the kernel, e.g. --m=4096 --iterations=100]
set -u
KERNEL_SRC=${1:?usage: run_kernel.sh kernel.cpp [kernel args]}
shift
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
PKG="$(dirname "$HERE")"
ROOT="$(dirname "$PKG")"
CUDA_HOME=${CUDA_HOME:-/usr/local/cuda}
BUILD_DIR=$(mktemp -d)
BINARY="$BUILD_DIR/kernel"

echo "=== xe-fuse kernel (B200 back end) ==="
echo "Source: $KERNEL_SRC"
echo ""
[ -f "$PKG/libxefuse_b200.so" ] || python "$PKG/build.py" > /dev/null || { echo "BUILD: FAILED (library)"; exit 1; }

echo "--- Compiling ---"
g++ -std=c++17 -O2 -fopenmp -I "$PKG/include" -I "$ROOT/include" -I "$CUDA_HOME/include" \
    "$KERNEL_SRC" -o "$BINARY" -L "$PKG" -lxefuse_b200 -L "$CUDA_HOME/lib64" -lcudart \
    -Wl,-rpath,"$PKG" > "$BUILD_DIR/build.log" 2>&1
if [ $? -ne 0 ]; then
    echo "BUILD: FAILED"
    cat "$BUILD_DIR/build.log"
    rm -rf "$BUILD_DIR"
    exit 1
fi
echo "BUILD: OK"
# device code is pre-compiled in the library; its kernels have no register spills (nvcc -Xptxas -v)
echo "SPILLS: 0"
echo ""
echo "--- Running ---"
"$BINARY" "$@"
RC=$?
rm -rf "$BUILD_DIR"
exit $RC
