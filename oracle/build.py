"""Compile the CPU oracle (test infrastructure) into oracle/libfos_oracle.so with gcc."""

from __future__ import annotations

import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
SRC = HERE / "fos_oracle.c"
OUT = HERE / "libfos_oracle.so"

# -ffp-contract=off: every multiply and add must round separately, as eager fp32 tensor
# arithmetic does.  No -ffast-math, no -march=native (the library is built on one
# machine and run on another).
FLAGS = [
    "-std=c11", "-O3", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off",
    "-fno-fast-math", "-mavx2", "-mf16c",
]


def build(force: bool = False) -> Path:
    if not force and OUT.exists() and OUT.stat().st_mtime >= SRC.stat().st_mtime:
        return OUT
    cmd = ["gcc", *FLAGS, "-o", str(OUT), str(SRC), "-lm"]
    subprocess.run(cmd, check=True)
    return OUT


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
