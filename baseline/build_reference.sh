#!/bin/sh
# Installs the unmodified reference (Neil456/Redline) into baseline/_ref for the
# reference arm of bench.py: its Python tooling by pip (offline, no dependencies
# resolved), its engine and command-line programs by its own CMake build for sm_100.
# Usage: baseline/build_reference.sh /path/to/reference
set -e
if [ -z "$1" ] || [ ! -d "$1" ]; then
    echo "usage: $0 /path/to/reference (a checkout of Neil456/Redline)" >&2
    exit 2
fi
REF=$1
HERE=$(cd "$(dirname "$0")" && pwd)
SRC=$(mktemp -d)/reference
cp -r "$REF" "$SRC"      # the build writes into the source tree; the original may be read-only
python -m pip install --no-index --no-build-isolation --no-deps --find-links /opt/wheelhouse \
    --target "$HERE/_ref" --upgrade "$SRC"
cmake -S "$SRC" -B "$HERE/_ref/build" -DCMAKE_BUILD_TYPE=Release -DCMAKE_CUDA_ARCHITECTURES=100 \
    -DREDLINE_BUILD_TESTS=OFF
cmake --build "$HERE/_ref/build" -j8 --target redline_bench redline_generate redline_ref
rm -rf "$HERE/_ref/build/CMakeFiles" "$HERE"/_ref/build/*.a
echo "reference installed under $HERE/_ref"
