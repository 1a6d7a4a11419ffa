"""B200 (sm_100a) producer of the integer MoE block and the fused-dequant integer matmul.

``qk_cuda``  host-array bridge with the reference bridge's function names (ctypes over the C-ABI)
``device``   device-tensor (PyTorch) front end over the same library
``build``    in-tree nvcc build of ``lib/libnmc_qk_cuda.so``
"""
__all__ = ["qk_cuda", "device", "build"]
