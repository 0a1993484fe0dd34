"""Builds libdlmrt_b200.so in-tree with nvcc for sm_100a (cross-compiles without a GPU).

    python -m dlmrt_b200.build [--verbose]

The library is plain CUDA C++ behind an extern "C" boundary (include/dlmrt_b200.h); it links the CUDA runtime
statically and resolves the one driver symbol it needs (cuTensorMapEncodeTiled) at run time, so it has no link-time
dependency on libcuda or on torch.
"""

import subprocess
import sys
from pathlib import Path

PACKAGE = Path(__file__).resolve().parent
CSRC = PACKAGE / "csrc"
LIB = PACKAGE / "libdlmrt_b200.so"
SOURCES = ["api.cu", "reduce.cu", "rowpar_bf16.cu", "rowpar_nvfp4.cu", "moe_front.cu", "device_loop.cu"]
FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--expt-relaxed-constexpr",
         "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]


def stale():
    if not LIB.exists():
        return True
    built = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [PACKAGE.parent / "include" / "dlmrt_b200.h"]
    return any(d.stat().st_mtime > built for d in deps)


def build(verbose=False, force=False):
    """Compile every CUDA source of the package into one shared library; returns its path."""
    if not force and not stale():
        return LIB
    objects = []
    out_dir = PACKAGE / "build"
    out_dir.mkdir(exist_ok=True)
    procs = []
    for src in SOURCES:
        obj = out_dir / (src + ".o")
        cmd = ["nvcc", *FLAGS, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        objects.append(str(obj))
    failed = False
    for src, proc in procs:
        log, _ = proc.communicate()
        if proc.returncode or verbose:
            print(f"--- {src}\n{log}", file=sys.stderr)
        failed |= bool(proc.returncode)
    if failed:
        raise RuntimeError("nvcc failed; see the log above")
    link = ["nvcc", "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC", "-o", str(LIB),
            *objects]
    subprocess.run(link, check=True)
    return LIB


if __name__ == "__main__":
    print(build(verbose="--verbose" in sys.argv, force=True))
