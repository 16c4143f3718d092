"""Builds the CUDA library for sm_100a with nvcc, in tree.

`python -m mmh3_b200.build` compiles every source under `mmh3_b200/csrc` into
`mmh3_b200/lib/libmmh3_attn_b200.so` (and the test-only UMMA self-test library next to it). nvcc
cross-compiles without a GPU. A source is recompiled when it or any header is newer than its object.
"""

from __future__ import annotations

import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys

ROOT = pathlib.Path(__file__).resolve().parent
REPO = ROOT.parent
CSRC = ROOT / "csrc"
LIB_DIR = ROOT / "lib"
OBJ_DIR = LIB_DIR / "obj"
LIBRARY = LIB_DIR / "libmmh3_attn_b200.so"
SELFTEST_LIBRARY = LIB_DIR / "libmmh3_b200_selftest.so"

# The arch is spelled out: the shorthand -arch=sm_100a assembles for plain sm_100 with this nvcc
# and rejects every tcgen05 `.kind`.
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
]


def nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: the CUDA library cannot be built")
    return found


def _newest_header() -> float:
    headers = list(CSRC.glob("*.cuh")) + list((REPO / "include").glob("*.h"))
    return max(path.stat().st_mtime for path in headers)


def _compile(source: pathlib.Path, obj: pathlib.Path, verbose: bool) -> None:
    command = [nvcc(), *NVCC_FLAGS, "-c", str(source), "-o", str(obj)]
    if verbose:
        command.insert(1, "-Xptxas")
        command.insert(2, "-v")
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed on {source.name}:\n{result.stdout}\n{result.stderr}")
    if verbose:
        sys.stderr.write(result.stderr)


def _link(objects: list[pathlib.Path], library: pathlib.Path) -> None:
    command = [nvcc(), *NVCC_FLAGS, "-shared", "-o", str(library), *map(str, objects)]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link of {library.name} failed:\n{result.stdout}\n{result.stderr}")


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    """Compiles what is stale and returns the path of the library."""
    OBJ_DIR.mkdir(parents=True, exist_ok=True)
    header_time = _newest_header()
    sources = sorted(CSRC.glob("*.cu")) + [REPO / "tests" / "csrc" / "umma_selftest.cu"]
    jobs = []
    objects = {}
    for source in sources:
        obj = OBJ_DIR / (source.stem + ".o")
        objects[source.stem] = obj
        stale = (
            force
            or not obj.exists()
            or obj.stat().st_mtime < max(source.stat().st_mtime, header_time)
        )
        if stale:
            jobs.append((source, obj))
    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as pool:
            list(pool.map(lambda job: _compile(job[0], job[1], verbose), jobs))
    product = [obj for stem, obj in objects.items() if stem != "umma_selftest"]
    if jobs or not LIBRARY.exists():
        _link(product, LIBRARY)
    if jobs or not SELFTEST_LIBRARY.exists():
        _link([objects["umma_selftest"], objects["common"]], SELFTEST_LIBRARY)
    return LIBRARY


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
