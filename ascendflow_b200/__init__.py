"""B200 (sm_100a) sparse MLA attention behind the reference's launch ABI.

Only what the operator path needs lives here: the CUDA sources and C ABI
(`csrc/`), the build recipe, the host runtime that mirrors the reference's
`KernelLaunch` / `TensorKernel` / `TorchRuntime`, the PyTorch op, request /
query sharding for several GPUs, and seeded workload generators.
"""

from .diagnostics import CompileError, ErrorKind, require

__all__ = ["CompileError", "ErrorKind", "require"]
