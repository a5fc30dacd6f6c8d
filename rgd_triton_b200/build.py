"""Build librgd_b200.so in-tree with nvcc for sm_100a.

    python -m rgd_triton_b200.build [--force] [--verbose]

Every ``csrc/*.cu`` is compiled to an object file under ``csrc/build/`` (in
parallel, skipped when the object is newer than the source and the headers) and
linked into ``rgd_triton_b200/librgd_b200.so``.  No GPU is needed to build.
"""
from __future__ import annotations

import argparse
import concurrent.futures as cf
import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
OBJ = CSRC / "build"
LIB = PKG / "librgd_b200.so"
INCLUDE = PKG.parent / "include"

NVCC_FLAGS = [
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-Xcompiler", "-fPIC",
    "--expt-relaxed-constexpr",
]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found: set NVCC or put /usr/local/cuda/bin on PATH")


def _deps_mtime() -> float:
    hdrs = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(INCLUDE.glob("*.h"))
    return max((h.stat().st_mtime for h in hdrs), default=0.0)


def _compile(src: Path, force: bool, verbose: bool, ptxas_v: bool) -> tuple[Path, str]:
    obj = OBJ / (src.stem + ".o")
    newest_dep = max(src.stat().st_mtime, _deps_mtime(), Path(__file__).stat().st_mtime)
    if not force and obj.exists() and obj.stat().st_mtime >= newest_dep:
        return obj, ""
    cmd = [_nvcc(), *NVCC_FLAGS, f"-I{INCLUDE}", "-c", str(src), "-o", str(obj)]
    if ptxas_v:
        cmd[1:1] = ["-Xptxas", "-v"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed for {src.name}:\n{res.stdout}\n{res.stderr}")
    return obj, res.stderr


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def build(force: bool = False, verbose: bool = False, ptxas_v: bool = False) -> Path:
    """Compile and link the library; returns its path."""
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    if not srcs:
        raise RuntimeError(f"no CUDA sources under {CSRC}")
    logs = []
    with cf.ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as ex:
        futs = [ex.submit(_compile, s, force, verbose, ptxas_v) for s in srcs]
        objs = []
        for f in futs:
            o, log = f.result()
            objs.append(o)
            if log:
                logs.append(log)
    if ptxas_v:
        print("\n".join(logs))
    need_link = force or not LIB.exists() or any(o.stat().st_mtime > LIB.stat().st_mtime for o in objs)
    if need_link:
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", str(LIB), *map(str, objs)]
        if verbose:
            print(" ".join(cmd), flush=True)
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--ptxas-v", action="store_true", help="print registers / spills / shared memory per kernel")
    a = ap.parse_args(argv)
    lib = build(a.force, a.verbose, a.ptxas_v)
    print(lib)
    return 0


if __name__ == "__main__":
    sys.exit(main())
