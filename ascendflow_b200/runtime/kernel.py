"""One kernel of a launch library, bound to a stream and to fixed runtime sizes.

The launch ABI is the reference's (generated at `src/backend/structured.py:626-649` and
`src/backend/workspace.py:93-130`, consumed by its `KernelLaunch`, `src/runtime/kernel.py:9-63`):
per kernel `<name>` a library exports `kernel_config_<name>`, `workspace_size_<name>` and
`launch_<name>(stream, tensor pointers..., workspace, int64 sizes...)`. A `KernelLaunch`
here plays the same part with the same constructor and call convention, so the two are
interchangeable over either side's libraries: it reads the configuration, sizes the workspace
once, keeps that arena for its lifetime and forwards calls. One binding belongs to one stream;
launches on other streams need bindings of their own.
"""

import ctypes as ct
import os

from ..diagnostics import require

_INT64_LIMIT = 1 << 63
_CONFIG_WORDS = 5  # tensors, size parameters, has workspace, two device-resource words


def _is_size(value):
    return type(value) is int and 0 <= value < _INT64_LIMIT


def _open(library):
    """A path is loaded; anything else is taken to be a loaded library already."""
    if isinstance(library, (str, bytes, os.PathLike)):
        return ct.CDLL(os.fspath(library))
    return library


class KernelLaunch:
    def __init__(self, runtime, library, name, *, parameters=()):
        sizes = tuple(parameters)
        require(all(map(_is_size, sizes)), "kernel size parameters must be nonnegative int64 integers")
        self.runtime, self.name, self.parameters = runtime, name, sizes
        self.stream = ct.c_void_p(runtime.stream.value)
        self.library = _open(library)
        self.tensors, has_workspace = self._read_configuration()
        self.workspace, self.workspace_nbytes = None, 0
        self.query = None
        if has_workspace:
            self._size_workspace()
        pointer_count = 1 + self.tensors + (self.query is not None)
        self.launch = getattr(self.library, f"launch_{name}")
        self.launch.restype = ct.c_int
        self.launch.argtypes = [ct.c_void_p] * pointer_count + [ct.c_int64] * len(sizes)

    def _read_configuration(self):
        """Tensor count and workspace flag; the size-parameter count and device words are checked."""
        symbol = getattr(self.library, f"kernel_config_{self.name}")
        symbol.restype, symbol.argtypes = ct.c_int, [ct.POINTER(ct.c_int64)]
        words = (ct.c_int64 * _CONFIG_WORDS)()
        require(symbol(words) == 0, "failed to read compiled kernel configuration")
        tensors, expected, has_workspace, *device_words = words
        require(expected == len(self.parameters), f"kernel expects {expected} size parameters")
        if any(device_words):  # a library built for one device shape; this one exports zeros
            have = self.runtime.resources
            require(tuple(device_words) == (have.cube_cores, have.vector_cores),
                    "compiled device resources differ from the runtime device; rebuild for this device")
        return int(tensors), bool(has_workspace)

    def _size_workspace(self):
        self.query = getattr(self.library, f"workspace_size_{self.name}")
        self.query.restype = ct.c_int
        self.query.argtypes = [ct.POINTER(ct.c_uint64)] + [ct.c_int64] * len(self.parameters)
        nbytes = ct.c_uint64()
        require(self.query(ct.byref(nbytes), *self.parameters) == 0,
                f"{self.name}: workspace byte extent exceeds int64 or is invalid")
        self.workspace_nbytes = nbytes.value
        self.workspace = self.runtime.allocate_uninitialized(nbytes.value)

    def __call__(self, *tensors):
        require(not self.runtime._closed, "kernel runtime is closed")
        require(len(tensors) == self.tensors, f"kernel expects {self.tensors} tensor pointers")
        arguments = [self.stream, *tensors]
        if self.query is not None:
            arguments.append(self.workspace)
        status = self.launch(*arguments, *self.parameters)
        if status != 0:
            raise RuntimeError(f"kernel launch failed with status {status}; device retries are disabled")

    def status(self):
        """Synchronise the stream and return the workspace's status block as a tuple of ints
        (word 0: 0 ok, 1 bad block-table entry, 2 an on-chip wait expired)."""
        require(self.workspace is not None, "kernel has no workspace status block")
        read = self.library.read_status_sparse_mla
        read.restype = ct.c_int
        read.argtypes = [ct.c_void_p, ct.c_void_p, ct.POINTER(ct.c_int32)]
        words = (ct.c_int32 * 8)()
        code = read(self.stream, self.workspace, words)
        if code != 0:
            raise RuntimeError(f"status read failed with CUDA error {code}; device retries are disabled")
        return tuple(words)
