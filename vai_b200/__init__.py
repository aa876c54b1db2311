"""B200 (sm_100a) backend for vAi's Linear node.

The package mirrors the part of `pyvai` that the Linear path uses (Dtype, Epilogue,
ResidualOrder, Tensor, NeuralNet, nodes.LinearNode); the arithmetic runs in
hand-written CUDA kernels behind the C ABI in include/vaicu.h.
"""
from . import nodes
from .engine import Device, DeviceBuffer, Dtype, Epilogue, NeuralNet, Node, ResidualOrder, Tensor

__all__ = ["Device", "DeviceBuffer", "Dtype", "Epilogue", "NeuralNet", "Node", "ResidualOrder", "Tensor", "nodes"]
