"""In-tree build of liblrnnx_b200.so (nvcc, sm_100a only).

``python -m lrnnx_b200.build`` compiles every ``csrc/*.cu`` to an object file
(in parallel, skipping up-to-date ones) and links ``lib/liblrnnx_b200.so``.
nvcc cross-compiles without a GPU, so this also runs on CPU-only hosts.
"""
from __future__ import annotations

import concurrent.futures as cf
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent
CSRC = ROOT / "csrc"
OBJ = ROOT / "lib" / "obj"
LIB = ROOT / "lib" / "liblrnnx_b200.so"

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-lineinfo",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-Xcompiler", "-fPIC", "-Xptxas", "-v",
    "--expt-relaxed-constexpr",
]


def _newest_header() -> float:
    hs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.inc")) + [ROOT.parent / "include" / "lrnnx_b200.h"]
    return max(h.stat().st_mtime for h in hs)


def _compile(src: Path, force: bool) -> tuple[Path, str]:
    obj = OBJ / (src.stem + ".o")
    if not force and obj.exists() and obj.stat().st_mtime > max(src.stat().st_mtime, _newest_header()):
        return obj, ""
    cmd = ["nvcc", *NVCC_FLAGS, "-c", str(src), "-o", str(obj)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{r.stdout}\n{r.stderr}")
    (OBJ / (src.stem + ".ptxas.log")).write_text(r.stderr)
    return obj, r.stderr


def build_library(force: bool = False, verbose: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sorted(CSRC.glob("*.cu"))
    with cf.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
        results = list(ex.map(lambda s: _compile(s, force), srcs))
    objs = [o for o, _ in results]
    rebuilt = any(log for _, log in results)
    if rebuilt or not LIB.exists() or force:
        cmd = ["nvcc", "-shared", "-o", str(LIB), *map(str, objs), "-gencode", "arch=compute_100a,code=sm_100a",
               "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    if verbose:
        for _, log in results:
            if log:
                print(log)
    return LIB


if __name__ == "__main__":
    p = build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(p)
