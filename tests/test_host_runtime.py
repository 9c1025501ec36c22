"""Host runtime without a device: C-ABI exports, metadata, sizing, binding rules.

Follows the reference's host ABI tests (`tests/runtime/test_tensor_kernel.py`,
`test_launcher.py`, `test_workspace.py`): the real library is loaded and its non-compute
symbols are called; argument order, stream forwarding, arena reuse and every `TensorKernel`
rejection are checked against a small host-only library with a fake tensor class.
"""

import ctypes as ct
import json
import re
import subprocess
from pathlib import Path
from types import SimpleNamespace

import pytest

from ascendflow_b200.build import build_library
from ascendflow_b200.diagnostics import CompileError
from ascendflow_b200.runtime.kernel import KernelLaunch
from ascendflow_b200.runtime.torch import TensorKernel

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def library():
    return ct.CDLL(str(build_library()))


def declared_symbols():
    header = (ROOT / "include/sparse_mla.h").read_text()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    return sorted(set(re.findall(r"\b((?:kernel_config|kernel_metadata|workspace_size|launch|read_status)_\w+)\s*\(", header)))


def test_library_exports_every_declared_symbol(library):
    names = declared_symbols()
    assert {"launch_sparse_mla", "kernel_config_sparse_mla", "kernel_metadata_sparse_mla",
            "workspace_size_sparse_mla", "launch_sparse_mla_f16"} <= set(names)
    for name in names:
        assert hasattr(library, name), name


@pytest.mark.parametrize("name,dtype", [("sparse_mla", "bf16"), ("sparse_mla_f16", "f16")])
def test_config_and_metadata(library, name, dtype):
    config = getattr(library, "kernel_config_" + name)
    config.argtypes, config.restype = [ct.POINTER(ct.c_int64)], ct.c_int
    values = (ct.c_int64 * 5)()
    assert config(values) == 0 and list(values) == [13, 6, 1, 0, 0]
    assert config(None) == -1
    query = getattr(library, "kernel_metadata_" + name)
    query.restype = ct.c_char_p
    meta = json.loads(query())
    assert meta["version"] == 1 and meta["name"] == name and meta["target"] == "sm_100a"
    assert meta["disjoint_external"] is True and meta["workspace"] is True
    assert [t["name"] for t in meta["tensors"]] == [
        "q", "ori_kv", "cmp_kv", "cmp_sparse_indices", "ori_block_table", "cmp_block_table",
        "cu_seqlens_q", "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length",
        "sinks", "attention_out"]
    assert [t["dtype"] for t in meta["tensors"]] == [dtype] * 3 + ["i32"] * 8 + ["f32", dtype]
    assert [t["access"] for t in meta["tensors"]] == ["read"] * 12 + ["write"]
    assert [p["name"] for p in meta["parameters"]] == ["B", "T", "PAGES", "ORI_BLOCKS", "CMP_BLOCKS", "CMP_PAGE"]
    assert meta["tensors"][0]["shape"] == ["T", 64, 512]
    assert meta["tensors"][2]["shape"] == ["CMP_BLOCKS", "CMP_PAGE", 1, 512]
    assert meta["tensors"][6]["shape"] == [{"add": ["B", 1]}]


def test_workspace_size_contract(library):
    query = library.workspace_size_sparse_mla
    query.argtypes = [ct.POINTER(ct.c_uint64)] + [ct.c_int64] * 6
    query.restype = ct.c_int
    size = ct.c_uint64(123)
    assert query(ct.byref(size), 4, 16, 32, 128, 128, 64) == 0
    assert size.value > 0 and size.value % 512 == 0
    assert query(None, 4, 16, 32, 128, 128, 64) == -1
    for position in range(6):
        arguments = [4, 16, 32, 128, 128, 64]
        arguments[position] = -1
        assert query(ct.byref(size), *arguments) == -1 and size.value == 0
    assert query(ct.byref(size), 4, 1 << 62, 32, 128, 128, 64) == -1
    assert query(ct.byref(size), 4, 16, 32, 1 << 60, 128, 64) == -1
    assert query(ct.byref(size), 0, 0, 0, 0, 0, 0) == 0


def test_launch_rejects_impossible_sizes_before_touching_a_device(library):
    launch = library.launch_sparse_mla
    launch.argtypes = [ct.c_void_p] * 15 + [ct.c_int64] * 6
    launch.restype = ct.c_int
    pointers = [None] * 15
    assert launch(*pointers, 4, 16, 32, 128, 128, 64) == -1  # no workspace
    pointers[14] = 4096
    assert launch(*pointers, 0, 16, 32, 128, 128, 64) == -1
    assert launch(*pointers, 4, 16, 32, 128, 128, 32) == -1  # compressed page must be 64 or 128


# ---- binding rules against a host-only library and fake tensors --------------------------------

@pytest.fixture(scope="module")
def probe(tmp_path_factory):
    output = tmp_path_factory.mktemp("probe") / "libprobe.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-fsanitize=undefined", "-fno-sanitize-recover",
                    "-o", str(output), str(ROOT / "tests/fake_kernel.c")], check=True)
    return ct.CDLL(str(output))


class FakeDType:
    def __init__(self, name, size):
        self.name, self.size = name, size


class FakeTorch:
    float32, int32, float16, bfloat16, int64 = (FakeDType(n, s) for n, s in (
        ("float32", 4), ("int32", 4), ("float16", 2), ("bfloat16", 2), ("int64", 8)))

    class Tensor:
        def __init__(self, shape, dtype, pointer, device=("cuda", 0), contiguous=True):
            self.shape, self.dtype, self.pointer, self.contiguous = tuple(shape), dtype, pointer, contiguous
            self.device = SimpleNamespace(type=device[0], index=device[1])
            self.recorded = []

        def is_contiguous(self): return self.contiguous
        def data_ptr(self): return self.pointer
        def element_size(self): return self.dtype.size
        def record_stream(self, stream): self.recorded.append(stream)
        def numel(self):
            count = 1
            for extent in self.shape:
                count *= extent
            return count


FakeTorch.Tensor.__eq__ = object.__eq__


class FakeRuntime:
    """What TensorKernel needs from TorchRuntime, with host memory standing in for arenas."""

    def __init__(self, stream=0x5000):
        self.torch, self._closed, self.arenas, self.stream_value = FakeTorch, False, [], stream

    def current_device(self): return getattr(self, "device_index", 0)

    def _context(self, device):
        owner = self

        class Context:
            torch_stream = ("stream", owner.stream_value)
            stream = ct.c_void_p(owner.stream_value)
            _closed = False
            resources = SimpleNamespace(cube_cores=0, vector_cores=0)

            def allocate_uninitialized(self, nbytes):
                buffer = ct.create_string_buffer(nbytes + 512)
                owner.arenas.append(buffer)
                return ct.c_void_p((ct.addressof(buffer) + 511) // 512 * 512)

        if not hasattr(self, "_cached") or self._cached[0] != self.stream_value:
            self._cached = (self.stream_value, Context())
        return self._cached[1]


def tensors(n=4, x_pointer=0x10000, y_pointer=0x20000):
    x = FakeTorch.Tensor((n, 4), FakeTorch.float32, x_pointer)
    x.device = y_device = SimpleNamespace(type="cuda", index=0)
    y = FakeTorch.Tensor((2 * n,), FakeTorch.int32, y_pointer)
    y.device = y_device
    return x, y


def last_call(probe):
    out = (ct.c_int64 * 5)()
    probe.probe_last_call(out)
    return list(out)


def test_argument_order_stream_and_workspace_reuse(probe):
    runtime = FakeRuntime()
    kernel = TensorKernel(runtime, probe, "probe")
    assert kernel.tensors == ("x", "y") and kernel.parameters == ("N",)
    x, y = tensors()
    before = probe.probe_launches()
    kernel(x, y)
    kernel(x=x, y=y)
    assert probe.probe_launches() == before + 2
    stream, px, py, workspace, n = last_call(probe)
    assert (stream, px, py, n) == (0x5000, 0x10000, 0x20000, 4)
    assert workspace % 512 == 0 and len(runtime.arenas) == 1
    assert kernel.workspace_nbytes == 512
    # record_stream once per bound call and stream (two separate binds above).
    assert x.recorded == [("stream", 0x5000)] * 2 and y.recorded == [("stream", 0x5000)] * 2
    bound = kernel.bind(x, y)
    bound(), bound(), bound()
    assert len(x.recorded) == 3
    # Other sizes or another stream get their own arena.
    kernel(*tensors(8))
    assert len(runtime.arenas) == 2 and kernel.workspace_nbytes == 512 + 1024
    runtime.stream_value = 0x6000
    kernel(x, y)
    assert last_call(probe)[0] == 0x6000 and len(runtime.arenas) == 3


@pytest.mark.parametrize("mutate,message", [
    (lambda x, y: setattr(x, "dtype", FakeTorch.float16), "dtype differs"),
    (lambda x, y: setattr(x, "contiguous", False), "contiguous"),
    (lambda x, y: setattr(x, "shape", (4, 4, 1)), "rank differs"),
    (lambda x, y: setattr(y, "shape", (9,)), "shape differs"),
    (lambda x, y: setattr(x, "shape", (3, 4)), "shape differs|contract differs"),
    (lambda x, y: setattr(x, "device", SimpleNamespace(type="cpu", index=None)), "CUDA tensor"),
    (lambda x, y: setattr(y, "pointer", x.pointer + 16), "disjoint"),
])
def test_rejections_happen_before_any_launch(probe, mutate, message):
    kernel = TensorKernel(FakeRuntime(), probe, "probe")
    x, y = tensors()
    mutate(x, y)
    before = probe.probe_launches()
    with pytest.raises(CompileError, match=message):
        kernel(x, y)
    assert probe.probe_launches() == before


def test_other_device_conflicting_parameter_closed_runtime_and_failed_launch(probe):
    runtime = FakeRuntime()
    kernel = TensorKernel(runtime, probe, "probe")
    x, y = tensors()
    with pytest.raises(CompileError, match="conflicting runtime dimension"):
        kernel(x, y, N=6)
    with pytest.raises(CompileError, match="expected a Torch tensor"):
        kernel(object(), y)
    other = SimpleNamespace(type="cuda", index=1)
    x.device = y.device = other
    with pytest.raises(CompileError, match="current CUDA device"):
        kernel(x, y)
    x, y = tensors()
    y.device = other
    with pytest.raises(CompileError, match="share one device"):
        kernel(x, y)
    with pytest.raises(RuntimeError, match="status 7; device retries are disabled"):
        kernel(*tensors(666))
    runtime._closed = True
    with pytest.raises(CompileError, match="closed"):
        kernel(*tensors())


def test_kernel_launch_checks_parameter_count_and_pointer_count(probe):
    context = FakeRuntime()._context(None)
    with pytest.raises(CompileError, match="expects 1 size parameters"):
        KernelLaunch(context, probe, "probe", parameters=())
    with pytest.raises(CompileError, match="nonnegative int64"):
        KernelLaunch(context, probe, "probe", parameters=(-2,))
    with pytest.raises(CompileError, match="workspace byte extent"):
        KernelLaunch(context, probe, "probe", parameters=((1 << 63) - 1,))
    binding = KernelLaunch(context, probe, "probe", parameters=(4,))
    with pytest.raises(CompileError, match="expects 2 tensor pointers"):
        binding(1)


def test_wrong_target_or_name_is_refused(probe):
    with pytest.raises(CompileError, match="metadata is missing"):
        TensorKernel(FakeRuntime(), probe, "absent")


def test_two_devices_with_the_same_stream_handle_get_separate_arenas(probe):
    """The legacy default stream is handle 0 on every GPU: a call on a second device with the same
    sizes must not reuse the binding (and workspace) made for the first."""
    runtime = FakeRuntime(stream=0)
    kernel = TensorKernel(runtime, probe, "probe")
    kernel(*tensors())
    first = last_call(probe)[3]
    runtime.device_index = 1
    x, y = tensors(x_pointer=0x30000, y_pointer=0x40000)
    x.device = y.device = SimpleNamespace(type="cuda", index=1)
    kernel(x, y)
    assert len(runtime.arenas) == 2 and last_call(probe)[3] != first
    runtime.device_index = 0
    kernel(*tensors())
    assert len(runtime.arenas) == 2 and last_call(probe)[3] == first
