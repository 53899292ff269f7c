"""tennis_b200: the int8 quantized-convolution path of TenniS on NVIDIA B200 (sm_100a).

``quantize`` -> ``conv2d_quantized`` (+ add_bias, relu / leaky_relu, optional requantize), written as CUDA
kernels behind the C ABI in include/tennis_b200.h.  ``tennis_b200.ops`` mirrors the TenniS operator interface
for Python callers; ``tennis_b200/plugin`` holds the C++ operator classes that register on TenniS's "gpu"
device.  Importing the package does not load the CUDA library; the first operator call does, and fails
loudly when it is missing.
"""
from . import _lib  # noqa: F401

__all__ = ["_lib", "ops", "workloads", "build"]
