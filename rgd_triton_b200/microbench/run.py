"""Build and run one of the micro-benchmarks of this folder on the current GPU.

    python -m rgd_triton_b200.microbench.run mma_rate | l2_reduction | alu_rate

They are stand-alone programs (not part of librgd_b200.so): measurements that shaped the
kernels and that the notes under profiles/ quote.  Each runs for a few seconds on one GPU.
"""
from __future__ import annotations

import subprocess
import sys
import tempfile
from pathlib import Path

from ..build import NVCC_FLAGS, _nvcc

HERE = Path(__file__).resolve().parent
NAMES = ("mma_rate", "l2_reduction", "alu_rate")


def main(argv=None) -> int:
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) != 1 or argv[0] not in NAMES:
        print(f"usage: python -m rgd_triton_b200.microbench.run {{{' | '.join(NAMES)}}}")
        return 2
    src = HERE / (argv[0] + ".cu")
    with tempfile.TemporaryDirectory() as tmp:
        exe = Path(tmp) / argv[0]
        flags = [f for f in NVCC_FLAGS if f not in ("-Xcompiler", "-fPIC")]
        cmd = [_nvcc(), *flags, f"-I{HERE.parent / 'csrc'}", f"-I{HERE.parent.parent / 'include'}", str(src), "-o", str(exe)]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            print(res.stdout + res.stderr)
            return 1
        return subprocess.run([str(exe)]).returncode


if __name__ == "__main__":
    raise SystemExit(main())
