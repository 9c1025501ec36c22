"""Host runtime: stream-owned launches over the C ABI, raw or with torch tensors."""

from .kernel import KernelLaunch
from .device import CUDA

__all__ = ["KernelLaunch", "CUDA", "TorchRuntime", "TensorKernel"]


def __getattr__(name):
    if name in ("TorchRuntime", "TensorKernel"):
        from . import torch as _torch

        return getattr(_torch, name)
    raise AttributeError(name)
