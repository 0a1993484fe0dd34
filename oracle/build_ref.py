"""Builds the REFERENCE's own fused-reduction extension into oracle/_ref/ (test infrastructure only).

    python oracle/build_ref.py [/path/to/reference]     (default: $DLMRT_REFERENCE, else ../reference)

The source file dlmrt/ops/csrc/tp_comm.cu is compiled where it lies in the reference tree, with the flags the
reference's own loader uses (dlmrt/ops/extensions.py:46-50: -O3 -std=c++17 -gencode=arch=compute_100a,code=sm_100a);
only the outputs land here. No reference source is copied. The resulting module (a torch extension exporting
`reduce`, `reduce_norm`, `reduce_norm_residual`) runs only on a GPU; the GPU tests use it to pin oracle.reduce and
this library's kernels against the reference's kernel on the same seeded inputs, and bench.py times it as the
"kernel to beat". oracle/_ref/ is git-ignored.
"""

import os
import sys
from pathlib import Path

NAME = "dlmrt_tp_comm_sm100a"
OUT = Path(__file__).resolve().parent / "_ref"


def reference_tree():
    """Where the reference's sources lie: $DLMRT_REFERENCE, else a `reference` folder beside this repository.
    None when neither exists (a machine that only carries the prebuilt oracle/_ref)."""
    candidates = [os.environ.get("DLMRT_REFERENCE"), Path(__file__).resolve().parent.parent.parent / "reference"]
    for c in candidates:
        if c and (Path(c) / "dlmrt" / "ops" / "csrc" / "tp_comm.cu").exists():
            return Path(c)
    return None


def build(reference):
    from torch.utils.cpp_extension import load

    src = Path(reference) / "dlmrt" / "ops" / "csrc" / "tp_comm.cu"
    if not src.exists():
        raise FileNotFoundError(src)
    OUT.mkdir(exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    load(name=NAME, sources=[str(src)], build_directory=str(OUT), is_python_module=False, verbose=False,
         extra_cuda_cflags=["-O3", "-std=c++17", "-gencode=arch=compute_100a,code=sm_100a"])
    return OUT / f"{NAME}.so"


def load_built():
    """Import the prebuilt module (GPU box: no reference tree, no compiler run). None when it was never built."""
    so = OUT / f"{NAME}.so"
    if not so.exists():
        return None
    import importlib.util

    import torch  # noqa: F401  (the extension links against torch)

    spec = importlib.util.spec_from_file_location(NAME, so)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else reference_tree()))
