"""dlmrt_b200: the tensor-parallel row-parallel hot path of a block-diffusion denoise round, B200-native.

    dlmrt_b200.distributed.parallel   init(), Group: the reduction entry point (mirror of dlmrt/distributed/parallel.py)
    dlmrt_b200.layers.linear          Linear: the row-parallel projection (mirror of dlmrt/layers/linear.py)
    dlmrt_b200.quantization.nvfp4     NVFP4 expert format and the expert down-projection entry point
    dlmrt_b200.ops.block_graph        BlockGraph / LoopGraph / StagedLoopGraph: the device-side loop around captured rounds
    dlmrt_b200.build                  compiles csrc/ into libdlmrt_b200.so (sm_100a)

Everything numeric runs in hand-written CUDA behind the C ABI declared in include/dlmrt_b200.h.
"""

__version__ = "0.1.0"
