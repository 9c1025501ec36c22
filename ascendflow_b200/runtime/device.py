"""Raw CUDA runtime adapter: device memory, one stream, events, kernel bindings.

The CUDA counterpart of the reference's `ACL` ctypes wrapper
(`src/device.py:63-186`), used where a test or tool wants raw pointers, guard
bytes behind every buffer and no tensor library in the way
(`benchmarks/attention/run_sparse.py:171-338` drives its device runs this way).
Every failed runtime call raises; nothing is retried.
"""

import ctypes as ct
from types import SimpleNamespace

from ..diagnostics import ErrorKind, require
from .kernel import KernelLaunch

_H2D, _D2H = 1, 2


def _load_cudart():
    names = ["libcudart.so.12", "libcudart.so", "/usr/local/cuda/lib64/libcudart.so"]
    try:  # torch ships the runtime it was built with; prefer that copy when torch is present
        import os
        import torch

        base = os.path.join(os.path.dirname(torch.__file__), "..", "nvidia", "cuda_runtime", "lib")
        names.insert(0, os.path.join(base, "libcudart.so.12"))
    except Exception:
        pass
    for name in names:
        try:
            return ct.CDLL(name, mode=ct.RTLD_GLOBAL)
        except OSError:
            continue
    require(False, "libcudart not found", kind=ErrorKind.RESOURCE)


class CUDA:
    """One device, one stream. `close()` synchronises and frees what it allocated."""

    def __init__(self, device=0):
        self.lib = _load_cudart()
        self._closed = False
        self.allocations = []
        self.device = int(device)
        self.call("cudaSetDevice", [ct.c_int], self.device)
        self.stream = ct.c_void_p()
        self.call("cudaStreamCreate", [ct.POINTER(ct.c_void_p)], ct.byref(self.stream))

    def call(self, name, types, *arguments):
        fn = getattr(self.lib, name)
        fn.argtypes, fn.restype = types, ct.c_int
        status = fn(*arguments)
        if status:
            raise RuntimeError(f"{name} failed with CUDA error {status}; device retries are disabled")

    @property
    def resources(self):
        count = ct.c_int()
        self.call("cudaDeviceGetAttribute", [ct.POINTER(ct.c_int), ct.c_int, ct.c_int],
                  ct.byref(count), 16, self.device)  # cudaDevAttrMultiProcessorCount
        return SimpleNamespace(cube_cores=count.value, vector_cores=count.value, multiprocessors=count.value)

    def allocate_uninitialized(self, nbytes):
        require(not self._closed, "kernel runtime is closed")
        pointer = ct.c_void_p()
        self.call("cudaMalloc", [ct.POINTER(ct.c_void_p), ct.c_size_t], ct.byref(pointer), max(int(nbytes), 1))
        self.allocations.append(pointer)
        return pointer

    def allocate(self, data):
        data = bytes(data)
        pointer = self.allocate_uninitialized(len(data))
        if data:
            self.call("cudaMemcpy", [ct.c_void_p, ct.c_char_p, ct.c_size_t, ct.c_int],
                      pointer, data, len(data), _H2D)
        return pointer

    def read(self, pointer, nbytes):
        buffer = ct.create_string_buffer(int(nbytes))
        self.synchronize()
        if nbytes:
            self.call("cudaMemcpy", [ct.c_void_p, ct.c_void_p, ct.c_size_t, ct.c_int],
                      buffer, pointer, int(nbytes), _D2H)
        return buffer.raw

    def free(self, pointer):
        self.call("cudaFree", [ct.c_void_p], pointer)
        self.allocations = [p for p in self.allocations if p.value != pointer.value]

    def event(self):
        handle = ct.c_void_p()
        self.call("cudaEventCreate", [ct.POINTER(ct.c_void_p)], ct.byref(handle))
        return handle

    def record(self, event):
        self.call("cudaEventRecord", [ct.c_void_p, ct.c_void_p], event, self.stream)

    def elapsed_us(self, start, end):
        value = ct.c_float()
        self.call("cudaEventElapsedTime", [ct.POINTER(ct.c_float), ct.c_void_p, ct.c_void_p],
                  ct.byref(value), start, end)
        return value.value * 1000.0

    def synchronize(self):
        self.call("cudaStreamSynchronize", [ct.c_void_p], self.stream)

    def kernel(self, library, name, parameters=()):
        require(not self._closed, "kernel runtime is closed")
        return KernelLaunch(self, library, name, parameters=parameters)

    def close(self):
        if self._closed:
            return
        self.synchronize()
        for pointer in self.allocations:
            self.call("cudaFree", [ct.c_void_p], pointer)
        self.allocations = []
        self.call("cudaStreamDestroy", [ct.c_void_p], self.stream)
        self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *error):
        self.close()
