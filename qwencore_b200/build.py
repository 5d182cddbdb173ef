"""In-tree build of the sm_100a shared library.

`python -m qwencore_b200.build` compiles every translation unit under csrc/ with nvcc for
sm_100a and links `qwencore_b200/libqwc_b200.so`.  Nothing is JIT-compiled at import
time: the built library travels with the tree.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
BUILD_DIR = PACKAGE_DIR / "_build"
LIBRARY = PACKAGE_DIR / "libqwc_b200.so"

# QWC_NVCC_DEFINES="-DQWC_STREAMK_TRACE" builds the projection kernel with its CTA timeline
EXTRA_DEFINES = os.environ.get("QWC_NVCC_DEFINES", "").split()

NVCC_FLAGS = [
    *EXTRA_DEFINES,
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-std=c++17",
    "-O3",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
]


def _nvcc() -> str:
    found = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(found):
        raise RuntimeError("nvcc not found: the CUDA extension cannot be built")
    return found


def sources() -> list[Path]:
    return sorted(list((CSRC / "kernels").glob("*.cu")) + list((CSRC / "host").glob("*.cpp")) +
                  list((CSRC / "host").glob("*.cu")))


def _headers() -> list[Path]:
    return sorted(list(CSRC.rglob("*.cuh")) + list(CSRC.rglob("*.h")) +
                  list((PACKAGE_DIR.parent / "include").glob("*.h")))


def _stamp(source: Path, extra_flags: list[str]) -> str:
    digest = hashlib.sha256()
    digest.update(source.read_bytes())
    for header in _headers():
        digest.update(header.read_bytes())
    digest.update(" ".join(NVCC_FLAGS + extra_flags).encode())
    return digest.hexdigest()


def _compile(source: Path, verbose: bool, ptxas_info: bool) -> Path:
    BUILD_DIR.mkdir(exist_ok=True)
    obj = BUILD_DIR / (source.stem + ".o")
    stamp_file = BUILD_DIR / (source.stem + ".stamp")
    extra = ["-Xptxas", "-v"] if ptxas_info else []
    stamp = _stamp(source, extra)
    if obj.exists() and stamp_file.exists() and stamp_file.read_text() == stamp and not ptxas_info:
        return obj
    command = [_nvcc(), *NVCC_FLAGS, *extra, "-x", "cu", "-I", str(PACKAGE_DIR.parent / "include"), "-c",
               str(source), "-o", str(obj)]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"nvcc failed for {source.name}:\n{result.stdout}\n{result.stderr}")
    if verbose or ptxas_info:
        sys.stderr.write(result.stderr)
    stamp_file.write_text(stamp)
    return obj


def build(verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile (only what changed) and link the shared library; returns its path."""
    files = sources()
    if not files:
        raise RuntimeError("no sources under csrc/")
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(files))) as pool:
        objects = list(pool.map(lambda s: _compile(s, verbose, ptxas_info), files))
    newest = max(o.stat().st_mtime for o in objects)
    if LIBRARY.exists() and LIBRARY.stat().st_mtime >= newest:
        return LIBRARY
    command = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(LIBRARY),
               *[str(o) for o in objects], "-Xlinker", "-Bsymbolic", "-lcudart", "-ldl", "-lpthread"]
    result = subprocess.run(command, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError(f"link failed:\n{result.stdout}\n{result.stderr}")
    return LIBRARY


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
