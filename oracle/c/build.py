"""Compiles oracle/c/oracle.c into oracle/c/liboracle.so with gcc (test infrastructure only)."""

import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB = HERE / "liboracle.so"


def build(force=False):
    src = HERE / "oracle.c"
    if force or not LIB.exists() or LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-std=c11", "-ffp-contract=off", "-fPIC", "-shared", "-o", str(LIB), str(src), "-lm"],
                       check=True)
    return LIB


if __name__ == "__main__":
    print(build(force=True))
