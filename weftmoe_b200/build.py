"""In-tree nvcc build of libweftmoe_b200.so for sm_100a (no JIT cache, no fallback).

The reference builds its native runtime lazily with nvcc behind `weftmoe/jit.py:183-246`; here
the build is one explicit step whose output sits beside the package so that it is the file the
process loads.  `python -m weftmoe_b200.build` rebuilds; `build()` is idempotent.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIBRARY = PACKAGE / "libweftmoe_b200.so"
OBJECTS = PACKAGE / "build"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
          "-Xcompiler", "-fvisibility=hidden", "-Xcompiler", "-Wall"]


def _nvcc() -> str:
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    candidate = Path(cuda_home) / "bin" / "nvcc"
    path = str(candidate) if candidate.is_file() else shutil.which("nvcc")
    if not path:
        raise RuntimeError("nvcc not found: set CUDA_HOME")
    return path


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, inputs: list[Path]) -> bool:
    if not target.is_file():
        return True
    stamp = target.stat().st_mtime_ns
    return any(p.stat().st_mtime_ns > stamp for p in inputs)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    """Compile every .cu under csrc/ for sm_100a and link the shared library."""
    nvcc = _nvcc()
    headers = sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h")) + \
        sorted((PACKAGE.parent / "include").glob("*.h"))
    OBJECTS.mkdir(exist_ok=True)
    jobs = []
    for src in sources():
        obj = OBJECTS / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *ARCH_FLAGS, *COMMON, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        if verbose:
            print(" ".join(cmd), flush=True)
        done = subprocess.run(cmd, capture_output=True, text=True)
        if done.returncode:
            raise RuntimeError(f"nvcc failed:\n{' '.join(cmd)}\n{done.stdout}\n{done.stderr}")
        return done.stderr

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        logs = list(pool.map(run, jobs))
    if ptxas_info:
        print("\n".join(logs))
    objects = [OBJECTS / (src.stem + ".o") for src in sources()]
    if force or jobs or _stale(LIBRARY, objects):
        run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(LIBRARY), *map(str, objects),
             "-cudart", "static", "-Xcompiler", "-fPIC"])
    return LIBRARY


if __name__ == "__main__":
    out = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas" in sys.argv)
    print(f"built {out}")
