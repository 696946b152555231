"""In-tree build of libb200moe.so (hand-written sm_100a CUDA behind a C ABI).

``python -m llm_gpu_kernels_b200.build`` compiles every ``csrc/*.cu`` with nvcc
for ``sm_100a`` only and links ``llm_gpu_kernels_b200/libb200moe.so``. nvcc
cross-compiles, so this works on a machine without a GPU. Nothing is compiled
at import or at prepare time: a missing library is an error, never a fallback.
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
LIBRARY = PACKAGE / "libb200moe.so"
OBJ_DIR = PACKAGE / "build"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if candidate and Path(candidate).is_file():
            return candidate
    raise RuntimeError("nvcc not found; set NVCC or put it on PATH")


def sources():
    return sorted(CSRC.glob("*.cu"))


def _stale(target: Path, deps) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any(Path(d).stat().st_mtime > stamp for d in deps)


def build(force: bool = False, verbose: bool = False, ptxas_info: bool = False) -> Path:
    nvcc = find_nvcc()
    OBJ_DIR.mkdir(exist_ok=True)
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + [PACKAGE.parent / "include" / "b200moe.h"]
    jobs = []
    for src in sources():
        obj = OBJ_DIR / (src.stem + ".o")
        if force or _stale(obj, [src, *headers]):
            cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
            if ptxas_info:
                cmd[1:1] = ["-Xptxas", "-v"]
            jobs.append(cmd)

    def run(cmd):
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise RuntimeError("nvcc failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
        if verbose or ptxas_info:
            sys.stderr.write(proc.stdout + proc.stderr)

    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as pool:
        list(pool.map(run, jobs))
    objects = [str(OBJ_DIR / (src.stem + ".o")) for src in sources()]
    if force or jobs or _stale(LIBRARY, objects):
        run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-o", str(LIBRARY), *objects,
             "-cudart", "static"])
    return LIBRARY


if __name__ == "__main__":
    path = build(force="--force" in sys.argv, verbose=True, ptxas_info="--ptxas-info" in sys.argv)
    print(path)
