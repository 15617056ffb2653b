"""Builds libtessiq_b200.so, in tree, for sm_100a.

    python -m tessiq_b200.build [--force] [--verbose]

Each `csrc/*.cu` is compiled to an object with nvcc (in parallel) and the objects are linked into
`tessiq_b200/libtessiq_b200.so` with the CUDA runtime linked statically. NVRTC (used to instantiate
fused elementwise kernels) is opened at run time, so the library loads on a machine without a GPU
or a driver. Objects are rebuilt only when a source or header is newer.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
ROOT = PACKAGE.parent
CSRC = PACKAGE / "csrc"
OBJECTS = CSRC / "build"
LIBRARY = PACKAGE / "libtessiq_b200.so"

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = [
    "-O3",
    "-std=c++17",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "--extended-lambda",
    "-Xcompiler",
    "-fPIC,-Wall,-Wno-unknown-pragmas",
    f"-I{ROOT / 'include'}",
    f"-I{CSRC}",
]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found; tessiq_b200 has no CPU build")
    return found


def _newest_header() -> float:
    headers = list(CSRC.glob("*.h")) + list((ROOT / "include").glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile(source: Path, force: bool, verbose: bool) -> Path:
    target = OBJECTS / (source.stem + ".o")
    stamp = max(source.stat().st_mtime, _newest_header(), Path(__file__).stat().st_mtime)
    if not force and target.exists() and target.stat().st_mtime >= stamp:
        return target
    command = [nvcc(), *ARCH, *COMMON, "-c", str(source), "-o", str(target)]
    if verbose:
        command.insert(1, "-Xptxas=-v")
        print(" ".join(command), flush=True)
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{result.stdout}\n{result.stderr}")
    if verbose or result.stderr.strip():
        sys.stderr.write(result.stderr)
    return target


def build(force: bool = False, verbose: bool = False) -> Path:
    OBJECTS.mkdir(parents=True, exist_ok=True)
    sources = sorted(CSRC.glob("*.cu"))
    if not sources:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        objects = list(pool.map(lambda s: _compile(s, force, verbose), sources))
    newest = max(o.stat().st_mtime for o in objects)
    if force or not LIBRARY.exists() or LIBRARY.stat().st_mtime < newest:
        command = [
            nvcc(), *ARCH, "-shared", "-o", str(LIBRARY), *map(str, objects),
            "-cudart", "static", "-Xcompiler", "-fPIC", "-ldl", "-lpthread",
        ]
        result = subprocess.run(command, capture_output=True, text=True)
        if result.returncode != 0:
            raise RuntimeError(f"linking {LIBRARY.name} failed:\n{result.stdout}\n{result.stderr}")
    return LIBRARY


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--force", action="store_true")
    parser.add_argument("--verbose", action="store_true", help="print commands and ptxas -v output")
    arguments = parser.parse_args()
    print(build(arguments.force, arguments.verbose))


if __name__ == "__main__":
    main()
