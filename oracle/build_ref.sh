#!/usr/bin/env bash
# Builds the reference project itself (CPU only: its tessiq:0 device) from the sources where they
# lie, into oracle/_ref/, so that tests can hold the oracle port and the golden vectors against the
# reference's own answers. The reference tree is read-only, so it is copied to a scratch directory
# first; nothing of it is copied into this repository (oracle/_ref/ is ignored by git).
#
#   oracle/build_ref.sh [/path/to/reference]      (without an argument: the checkout this script is set up for, REFERENCE below)
#
# Takes about two minutes on 8 cores. Needs cmake, ninja, a host g++ with a shared libstdc++
# (/usr/bin/g++), pybind11 and the PyTorch the reference pins.
set -euo pipefail
REFERENCE="${1:-/root/reference}"
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
OUT="$HERE/_ref"
SCRATCH="$(mktemp -d /tmp/tessiq_ref.XXXXXX)"
trap 'rm -rf "$SCRATCH"' EXIT
if [ ! -f "$REFERENCE/CMakeLists.txt" ]; then
  echo "no reference tree at $REFERENCE" >&2
  exit 2
fi
cp -r "$REFERENCE" "$SCRATCH/src"
chmod -R u+w "$SCRATCH/src"
cmake -S "$SCRATCH/src" -B "$SCRATCH/build" -G Ninja \
  -DCMAKE_C_COMPILER=/usr/bin/gcc -DCMAKE_CXX_COMPILER=/usr/bin/g++ \
  -DTESSIQ_BUILD_TESTS=OFF -DTESSIQ_BUILD_PYTHON=ON -DTESSIQ_ENABLE_CUDA=OFF \
  -DCMAKE_BUILD_TYPE=RelWithDebInfo -DTESSIQ_WARNINGS_AS_ERRORS=OFF \
  -DPython_EXECUTABLE="$(command -v python)" > "$SCRATCH/configure.log" 2>&1 || { tail -40 "$SCRATCH/configure.log" >&2; exit 1; }
cmake --build "$SCRATCH/build" -j"$(nproc)" > "$SCRATCH/build.log" 2>&1 || { tail -60 "$SCRATCH/build.log" >&2; exit 1; }
rm -rf "$OUT"
mkdir -p "$OUT"
cp -r "$SCRATCH/src/python/tessiq" "$OUT/tessiq"
find "$SCRATCH/build" -name '_C*.so' -exec cp {} "$OUT/tessiq/" \;
find "$SCRATCH/build" -name 'libtessiq*.so*' -exec cp -P {} "$OUT/tessiq/" \; 2>/dev/null || true
PYTHONPATH="$OUT" python -c "import tessiq; print('reference', tessiq.__version__, 'devices', tessiq.device_count())"
