"""Tensor calls on torch's current CUDA stream, through the compiled launch ABI.

Mirrors the reference's `TensorKernel` / `TorchRuntime` (`src/runtime/torch.py:60-288`):
the signature, dtypes, shapes and the disjointness contract come from the
library's `kernel_metadata_<name>` JSON; one workspace arena exists per
(stream, runtime sizes); outputs are passed explicitly; every violated contract
raises `CompileError` before anything is enqueued. Differences are those of
the device: tensors live on the current CUDA device instead of "npu:0", the
metadata target is "sm_100a", and every layout is linear.
"""

import ctypes as ct
import hashlib
import inspect
import json
from itertools import pairwise
from os import PathLike, fsdecode
from pathlib import Path

from ..diagnostics import require
from .kernel import KernelLaunch

TARGET = "sm_100a"
_DTYPES = {"f16": "float16", "bf16": "bfloat16", "f32": "float32", "i32": "int32", "i64": "int64"}
_LIBRARIES = {}


def _library(value):
    """Load a library once per path and refuse a file that changed underneath a loaded handle."""
    if not isinstance(value, (str, bytes, PathLike)):
        return value
    path = Path(fsdecode(value)).resolve()
    identity = hashlib.sha256(path.read_bytes()).hexdigest()
    if path in _LIBRARIES:
        previous, library = _LIBRARIES[path]
        require(previous == identity, "loaded kernel library changed; build into a new output directory")
        return library
    library = ct.CDLL(str(path))
    _LIBRARIES[path] = (identity, library)
    return library


def _extent(expression, parameters):
    """Evaluate a metadata shape entry: int, parameter name, {"mul": [a, b]} or {"add": [a, b]}."""
    if type(expression) is int:
        return expression
    if isinstance(expression, str):
        require(expression in parameters, f"missing runtime parameter {expression}; pass it by name")
        return parameters[expression]
    require(
        isinstance(expression, dict) and len(expression) == 1 and next(iter(expression)) in ("mul", "add"),
        "invalid compiled tensor extent",
    )
    (operator, operands), = expression.items()
    require(isinstance(operands, list) and len(operands) == 2, "invalid compiled tensor extent operands")
    left, right = (_extent(item, parameters) for item in operands)
    return left * right if operator == "mul" else left + right


class TensorKernel:
    """One compiled signature; arenas are isolated by stream and scalar binding."""

    def __init__(self, runtime, library, name):
        self.runtime = runtime
        self.library = _library(library)
        require(hasattr(self.library, "kernel_metadata_" + name),
                "compiled tensor metadata is missing; rebuild the kernel")
        query = getattr(self.library, "kernel_metadata_" + name)
        query.argtypes, query.restype = [], ct.c_char_p
        self.metadata = json.loads(query())
        require(self.metadata["version"] == 1 and self.metadata["name"] == name,
                "compiled kernel ABI version/name differs")
        require(self.metadata["target"] == TARGET, f"tensor runtime requires {TARGET}")
        self.name = name
        self.tensors = tuple(item["name"] for item in self.metadata["tensors"])
        self.parameters = tuple(item["name"] for item in self.metadata["parameters"])
        positional = inspect.Parameter.POSITIONAL_OR_KEYWORD
        self.__signature__ = inspect.Signature(
            [inspect.Parameter(n, positional) for n in self.tensors]
            + [inspect.Parameter(n, inspect.Parameter.KEYWORD_ONLY, default=None) for n in self.parameters]
        )
        self._bindings = {}

    @property
    def workspace_nbytes(self):
        return sum(binding.workspace_nbytes for binding in self._bindings.values())

    def bind(self, *args, **kwargs):
        """Validate once; bound tensors must keep their shape, dtype and storage."""
        require(not self.runtime._closed, "kernel runtime is closed")
        torch = self.runtime.torch
        values = self.__signature__.bind(*args, **kwargs).arguments
        parameters = {n: values[n] for n in self.parameters if values.get(n) is not None}
        require(all(type(n) is int and 0 <= n < 1 << 63 for n in parameters.values()),
                "runtime parameters require nonnegative int64 integers")
        tensors = tuple(values[n] for n in self.tensors)
        device, intervals, pointers = None, [], []
        for tensor, spec in zip(tensors, self.metadata["tensors"]):
            name = spec["name"]
            require(isinstance(tensor, torch.Tensor), f"{name}: expected a Torch tensor")
            require(tensor.device.type == "cuda", f"{name}: expected a CUDA tensor")
            device = tensor.device if device is None else device
            require(tensor.device == device, "kernel tensors must share one device")
            require(tensor.is_contiguous(), f"{name}: expected contiguous tensor storage")
            require(spec["layout"] == "linear", f"{name}: unsupported compiled tensor layout")
            require(tensor.dtype == getattr(torch, _DTYPES[spec["dtype"]]),
                    f"{name}: tensor dtype differs from compiled ABI")
            require(len(tensor.shape) == len(spec["shape"]), f"{name}: tensor rank differs from compiled ABI")
            for actual, dimension in zip(tensor.shape, spec["shape"]):
                if isinstance(dimension, str):
                    if dimension in parameters:
                        require(parameters[dimension] == actual,
                                f"{name}: conflicting runtime dimension {dimension}")
                    else:
                        parameters[dimension] = int(actual)
            pointer = tensor.data_ptr()
            pointers.append(pointer)
            nbytes = tensor.numel() * tensor.element_size()
            if nbytes:
                intervals.append((pointer, pointer + nbytes, name))
        require(device.index == self.runtime.current_device(),
                "kernel tensors must live on the current CUDA device")
        for spec, tensor in zip(self.metadata["tensors"], tensors):
            expected = tuple(_extent(n, parameters) for n in spec["shape"])
            require(tuple(tensor.shape) == expected, f"{spec['name']}: tensor shape differs from compiled ABI")
        for spec in self.metadata["parameters"]:
            name = spec["name"]
            require(name in parameters, f"missing runtime parameter {name}; pass it by name")
            value = parameters[name]
            require(spec["minimum"] <= value < 1 << 63 and value % spec["multiple"] == 0,
                    f"{name}: runtime input contract differs")
        if self.metadata["disjoint_external"]:
            ordered = sorted(intervals)
            require(all(a[1] <= b[0] for a, b in pairwise(ordered)),
                    "external tensors violate the compiled disjoint contract")
        sizes = tuple(parameters[n] for n in self.parameters)
        recorded_streams = set()

        def invoke():
            require(not self.runtime._closed, "kernel runtime is closed")
            context = self.runtime._context(device)
            key = (context.stream.value, sizes)
            if key not in self._bindings:
                self._bindings[key] = KernelLaunch(context, self.library, self.name, parameters=sizes)
            # Inputs made on another stream: their allocations must outlive this consumer.
            # Readiness of their contents stays the caller's business.
            if context.stream.value not in recorded_streams:
                for tensor in tensors:
                    tensor.record_stream(context.torch_stream)
                recorded_streams.add(context.stream.value)
            self._bindings[key](*pointers)
            return self._bindings[key]

        return invoke

    def __call__(self, *args, **kwargs):
        return self.bind(*args, **kwargs)()


class _StreamContext:
    def __init__(self, owner, stream, device):
        self.owner, self.torch_stream, self.device = owner, stream, device
        self.stream = ct.c_void_p(stream.cuda_stream)
        self.allocations = []

    @property
    def _closed(self):
        return self.owner._closed

    @property
    def resources(self):
        return self.owner.resources

    def allocate_uninitialized(self, nbytes):
        torch = self.owner.torch
        with torch.cuda.stream(self.torch_stream):
            storage = torch.empty(max(nbytes, 1) + 511, dtype=torch.uint8, device=self.device)
        storage.record_stream(self.torch_stream)
        self.allocations.append(storage)
        return ct.c_void_p((storage.data_ptr() + 511) // 512 * 512)


class TorchRuntime:
    """Own compiled tensor calls and their per-stream arenas until close()."""

    def __init__(self, torch=None):
        if torch is None:
            import torch
        self.torch = torch
        self._closed = False
        self._streams = {}

    def current_device(self):
        return self.torch.cuda.current_device()

    @property
    def resources(self):
        from types import SimpleNamespace

        require(not self._closed, "kernel runtime is closed")
        count = self.torch.cuda.get_device_properties(self.current_device()).multi_processor_count
        return SimpleNamespace(cube_cores=count, vector_cores=count, multiprocessors=count)

    def _context(self, device):
        stream = self.torch.cuda.current_stream(device)
        key = (device.index, stream.cuda_stream)
        if key not in self._streams:
            self._streams[key] = _StreamContext(self, stream, device)
        return self._streams[key]

    def kernel(self, library=None, name="sparse_mla"):
        require(not self._closed, "kernel runtime is closed")
        if library is None:
            from ..build import library_path

            library = library_path()
        return TensorKernel(self, library, name)

    def close(self):
        if not self._closed:
            for context in self._streams.values():
                context.torch_stream.synchronize()
            for context in self._streams.values():
                context.allocations.clear()
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *error):
        self.close()
