"""Builds the CUDA library in-tree: ``dashmag_b200/csrc/libdash_attn_b200.so`` for sm_100a.

``python -m dashmag_b200.build`` (or ``build()``) compiles every ``csrc/*.cu`` with nvcc and links
them into one shared library with a static CUDA runtime, so that the library loads on a machine
without a GPU (only launches need one).  Objects are rebuilt when their source or any header is
newer.
"""
from __future__ import annotations

import concurrent.futures
import os
import pathlib
import shutil
import subprocess
import sys

HERE = pathlib.Path(__file__).resolve().parent
CSRC = HERE / "csrc"
OBJ = CSRC / "build"
LIB = CSRC / "libdash_attn_b200.so"
INCLUDE = HERE.parent / "include"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and pathlib.Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: the CUDA library cannot be built")


def build(force: bool = False, verbose: bool = False) -> pathlib.Path:
    sources = sorted(CSRC.glob("*.cu"))
    headers = list(CSRC.glob("*.h")) + list(CSRC.glob("*.cuh")) + list(INCLUDE.glob("*.h"))
    newest_header = max(h.stat().st_mtime for h in headers)
    OBJ.mkdir(exist_ok=True)
    nvcc = _nvcc()
    host_cc = "/usr/bin/g++" if pathlib.Path("/usr/bin/g++").exists() else None

    def compile_one(src: pathlib.Path):
        obj = OBJ / (src.stem + ".o")
        if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, newest_header):
            return obj, ""
        cmd = [nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
        if host_cc:
            cmd[1:1] = ["-ccbin", host_cc]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        return obj, r.stderr

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
        results = list(pool.map(compile_one, sources))
    objs = [o for o, _ in results]
    logs = "".join(log for _, log in results)
    if logs:
        (OBJ / "ptxas.log").write_text(logs)
        if verbose:
            print(logs)
    if force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs):
        cmd = [nvcc, "-shared", "-o", str(LIB), *map(str, objs), "-cudart", "static"]
        if host_cc:
            cmd[1:1] = ["-ccbin", host_cc]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
