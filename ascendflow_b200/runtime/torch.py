"""Calls with torch CUDA tensors on torch's current stream, over the launch ABI.

The user-facing surface is the reference's (`src/runtime/torch.py:60-288`, described in its
`docs/guide/runtime.md:60-95`): `TorchRuntime().kernel(library, name)` gives a callable that
takes the kernel's tensors by position or name (outputs are passed explicitly), accepts size
parameters by keyword, validates everything against the library's metadata before anything is
enqueued, and launches on the current stream with one workspace arena per device, stream and
size binding. `bind(...)` validates once and returns a callable for repeated launches.
`close()` synchronises the streams used and frees the arenas. Tensors live on the current CUDA
device (the reference has a single "npu:0").
"""

import ctypes as ct
import hashlib
import inspect
import os
from pathlib import Path
from types import SimpleNamespace

from ..diagnostics import require
from .kernel import KernelLaunch
from .signature import TARGET, Signature  # noqa: F401  (TARGET is part of this module's surface)

_loaded = {}  # resolved path -> (sha256 of the file when loaded, CDLL)


def _library(value):
    """Load a library once per path. A file that changed after it was loaded is refused: the
    dynamic loader would keep serving the old image under the new file's name."""
    if not isinstance(value, (str, bytes, os.PathLike)):
        return value
    path = Path(os.fsdecode(value)).resolve()
    digest = hashlib.sha256(path.read_bytes()).hexdigest()
    known = _loaded.get(path)
    if known is None:
        known = _loaded[path] = (digest, ct.CDLL(str(path)))
    require(known[0] == digest, "loaded kernel library changed; build into a new output directory")
    return known[1]


class BoundCall:
    """Validated arguments of one kernel; calling it launches on the then-current stream."""

    def __init__(self, kernel, device, tensors, sizes):
        self.kernel, self.device, self.tensors, self.sizes = kernel, device, tensors, sizes
        self.pointers = tuple(tensor.data_ptr() for tensor in tensors)
        self._streams_seen = set()

    def __call__(self):
        kernel = self.kernel
        require(not kernel.runtime._closed, "kernel runtime is closed")
        context = kernel.runtime._context(self.device)
        launch = kernel._launch_for(self.device, context, self.sizes)
        handle = context.stream.value
        if handle not in self._streams_seen:
            # Arguments produced on another stream: the caching allocator must not recycle their
            # memory before this stream is done with it. Their contents being ready is the
            # caller's business, as with any stream-ordered call.
            for tensor in self.tensors:
                tensor.record_stream(context.torch_stream)
            self._streams_seen.add(handle)
        launch(*self.pointers)
        return launch


class TensorKernel:
    """One kernel of a library with its declared signature."""

    def __init__(self, runtime, library, name):
        self.runtime, self.name = runtime, name
        self.library = _library(library)
        symbol = getattr(self.library, f"kernel_metadata_{name}", None)
        require(symbol is not None, "compiled tensor metadata is missing; rebuild the kernel")
        symbol.restype, symbol.argtypes = ct.c_char_p, []
        self.signature = Signature(symbol(), name)
        self.metadata = self.signature.raw
        self.tensors, self.parameters = self.signature.tensor_names, self.signature.size_names
        positional, keyword = inspect.Parameter.POSITIONAL_OR_KEYWORD, inspect.Parameter.KEYWORD_ONLY
        self.__signature__ = inspect.Signature(
            [inspect.Parameter(n, positional) for n in self.tensors]
            + [inspect.Parameter(n, keyword, default=None) for n in self.parameters])
        self._bindings = {}  # (device index, stream handle, sizes) -> KernelLaunch

    @property
    def workspace_nbytes(self):
        return sum(launch.workspace_nbytes for launch in self._bindings.values())

    def _launch_for(self, device, context, sizes):
        # The legacy default stream has handle 0 on every GPU: the device is part of the key, or
        # a second GPU would be handed the first one's workspace.
        key = (device.index, context.stream.value, sizes)
        if key not in self._bindings:
            self._bindings[key] = KernelLaunch(context, self.library, self.name, parameters=sizes)
        return self._bindings[key]

    def bind(self, *args, **kwargs):
        """Validate once; the bound tensors must keep their shape, dtype and storage."""
        require(not self.runtime._closed, "kernel runtime is closed")
        torch, signature = self.runtime.torch, self.signature
        arguments = self.__signature__.bind(*args, **kwargs).arguments
        tensors = tuple(arguments[name] for name in self.tensors)
        for spec, tensor in zip(signature.tensors, tensors):
            signature.check_tensor(torch, spec, tensor)
        device = tensors[0].device
        require(all(t.device == device for t in tensors), "kernel tensors must share one device")
        require(device.index == self.runtime.current_device(),
                "kernel tensors must live on the current CUDA device")
        given = {n: arguments[n] for n in self.parameters if arguments.get(n) is not None}
        sizes = signature.solve_sizes(tensors, given)
        signature.check_shapes_and_sizes(tensors, sizes)
        signature.check_disjoint(tensors)
        return BoundCall(self, device, tensors, tuple(sizes[n] for n in self.parameters))

    def __call__(self, *args, **kwargs):
        return self.bind(*args, **kwargs)()


class _StreamContext:
    """What a `KernelLaunch` needs from its owner: the stream handle, device resources, arenas."""

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
        """512-byte aligned device memory that lives until the runtime is closed."""
        torch = self.owner.torch
        with torch.cuda.stream(self.torch_stream):
            block = torch.empty(max(nbytes, 1) + 511, dtype=torch.uint8, device=self.device)
        block.record_stream(self.torch_stream)
        self.allocations.append(block)
        return ct.c_void_p(-(-block.data_ptr() // 512) * 512)


class TorchRuntime:
    """Owns tensor kernels and their per-stream arenas until `close()`."""

    def __init__(self, torch=None):
        if torch is None:
            import torch
        self.torch, self._closed, self._streams = torch, False, {}

    def current_device(self):
        return self.torch.cuda.current_device()

    @property
    def resources(self):
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
        """`library` None selects this package's own built library."""
        require(not self._closed, "kernel runtime is closed")
        if library is None:
            from ..build import library_path

            library = library_path()
        return TensorKernel(self, library, name)

    def close(self):
        if self._closed:
            return
        for context in self._streams.values():
            context.torch_stream.synchronize()
        for context in self._streams.values():
            context.allocations.clear()
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *error):
        self.close()
