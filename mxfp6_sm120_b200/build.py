"""In-tree build of ``libmxfp6_b200.so`` (sm_100a only).

``python -m mxfp6_sm120_b200.build`` compiles every ``csrc/*.cu`` with nvcc into
objects under ``csrc/_obj`` and links ``lib/libmxfp6_b200.so`` next to the
package.  nvcc cross-compiles, so no GPU is needed to build.
"""

from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
OBJ = CSRC / "_obj"
LIB_DIR = PACKAGE_DIR / "lib"
LIB_PATH = LIB_DIR / "libmxfp6_b200.so"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    candidate = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(candidate).exists():
        raise RuntimeError("nvcc not found; the library can only be built with the CUDA toolkit")
    return candidate


def _stale(target: Path, sources: list[Path]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(src.stat().st_mtime > stamp for src in sources)


def build(verbose: bool = False, force: bool = False, ptxas_info: bool = False) -> Path:
    """Compile and link the library; returns its path."""
    nvcc = _nvcc()
    OBJ.mkdir(parents=True, exist_ok=True)
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    headers = sorted(CSRC.glob("*.cuh")) + [PACKAGE_DIR.parent / "include" / "mxfp6_b200.h"]
    sources = sorted(CSRC.glob("*.cu"))
    jobs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd: list[str]) -> None:
        if verbose:
            print(" ".join(cmd), flush=True)
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")
        if ptxas_info or verbose:
            sys.stderr.write(proc.stderr)

    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        list(pool.map(run, jobs))

    objects = [OBJ / (src.stem + ".o") for src in sources]
    if force or jobs or _stale(LIB_PATH, objects):
        run(
            [
                nvcc,
                "-shared",
                "-o",
                str(LIB_PATH),
                *map(str, objects),
                "-cudart",
                "static",
                "-Xlinker",
                "--no-undefined",
            ]
        )
    return LIB_PATH


if __name__ == "__main__":
    path = build(verbose="-v" in sys.argv, force="-f" in sys.argv, ptxas_info="--ptxas" in sys.argv)
    print(path)
