"""The reference project's own, unmodified `KernelLaunch` binds this repository's libraries.

`src/runtime/kernel.py:9-63` of the reference is loaded from a reference checkout as it is
(its one import, `..diagnostics.require`, comes from the checkout too) and is given a library
built here: the host-only probe library on CPU, the sm_100a attention library on a GPU. That
is the drop-in claim at its narrowest point: the four exported symbols per kernel, their
argument order and their return codes are what the reference's runtime expects. Skipped where
no reference checkout is present (looked for beside this repository, or at the path in
ASCENDFLOW_REFERENCE).
"""

import ctypes as ct
import importlib.util
import os
import subprocess
import sys
import types
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]
REFERENCE = Path(os.environ.get("ASCENDFLOW_REFERENCE", ROOT.parent / "reference"))


@pytest.fixture(scope="module")
def reference_kernel_launch():
    source = REFERENCE / "src/runtime/kernel.py"
    if not source.exists():
        pytest.skip("no reference checkout here")
    # A bare package tree under a private name, so that the relative import resolves to the
    # checkout's own diagnostics module and nothing else of the reference is imported.
    root = types.ModuleType("_reference_ascendflow")
    root.__path__ = []
    runtime = types.ModuleType("_reference_ascendflow.runtime")
    runtime.__path__ = []
    sys.modules.update({root.__name__: root, runtime.__name__: runtime})
    for name, path in (("_reference_ascendflow.diagnostics", REFERENCE / "src/diagnostics.py"),
                       ("_reference_ascendflow.runtime.kernel", source)):
        spec = importlib.util.spec_from_file_location(name, path)
        module = importlib.util.module_from_spec(spec)
        sys.modules[name] = module
        spec.loader.exec_module(module)
    return sys.modules["_reference_ascendflow.runtime.kernel"].KernelLaunch


def test_reference_class_binds_the_probe_library(reference_kernel_launch, tmp_path):
    output = tmp_path / "libprobe.so"
    subprocess.run(["gcc", "-shared", "-fPIC", "-O1", "-o", str(output), str(ROOT / "tests/fake_kernel.c")], check=True)
    probe = ct.CDLL(str(output))
    arenas = []

    def allocate(nbytes):
        arenas.append(ct.create_string_buffer(nbytes + 512))
        return ct.c_void_p((ct.addressof(arenas[-1]) + 511) // 512 * 512)

    context = SimpleNamespace(stream=ct.c_void_p(0x7000), _closed=False, allocate_uninitialized=allocate,
                              resources=SimpleNamespace(cube_cores=0, vector_cores=0))
    binding = reference_kernel_launch(context, probe, "probe", parameters=(4,))
    assert binding.tensors == 2 and binding.workspace_nbytes == 512 and len(arenas) == 1
    before = probe.probe_launches()
    binding(0x10000, 0x20000)
    assert probe.probe_launches() == before + 1
    seen = (ct.c_int64 * 5)()
    probe.probe_last_call(seen)
    assert list(seen)[:3] == [0x7000, 0x10000, 0x20000] and seen[4] == 4 and seen[3] % 512 == 0


def test_reference_class_reads_this_librarys_configuration(reference_kernel_launch):
    """No device needed: the constructor only reads the configuration and sizes the workspace."""
    from ascendflow_b200.build import build_library

    library = ct.CDLL(str(build_library()))
    sizes = (4, 16, 32, 128, 128, 64)  # B, T, PAGES, ORI_BLOCKS, CMP_BLOCKS, CMP_PAGE
    taken = []
    context = SimpleNamespace(stream=ct.c_void_p(0), _closed=False,
                              allocate_uninitialized=lambda n: taken.append(n) or ct.c_void_p(512),
                              resources=SimpleNamespace(cube_cores=0, vector_cores=0))
    binding = reference_kernel_launch(context, library, "sparse_mla", parameters=sizes)
    assert binding.tensors == 13 and taken == [1024] and binding.workspace_nbytes == 1024
    assert len(binding.launch.argtypes) == 1 + 13 + 1 + 6


@pytest.mark.gpu
def test_reference_class_launches_the_attention_kernel(reference_kernel_launch):
    import torch

    from ascendflow_b200.build import library_path
    from oracle import sparse_mla_oracle as O
    from tests import support as S

    policy = O.make_policy(4, 16, max_seq=4096, blocks=128)
    data = O.validation_inputs(policy, "mixed")
    tensors, _ = S.to_device(data, policy)
    stream = torch.cuda.current_stream()
    arenas = []

    def allocate(nbytes):
        arenas.append(torch.empty(nbytes + 512, dtype=torch.uint8, device="cuda"))
        return ct.c_void_p((arenas[-1].data_ptr() + 511) // 512 * 512)

    count = torch.cuda.get_device_properties(0).multi_processor_count
    context = SimpleNamespace(stream=ct.c_void_p(stream.cuda_stream), _closed=False, allocate_uninitialized=allocate,
                              resources=SimpleNamespace(cube_cores=count, vector_cores=count))
    sizes = (policy["B"], policy["T"], policy["MAX_SEQ"] // 128, policy["ORI_BLOCKS"], policy["CMP_BLOCKS"],
             128 // policy["RATIO"])
    binding = reference_kernel_launch(context, str(library_path()), "sparse_mla", parameters=sizes)
    binding(*(tensors[name].data_ptr() for name in S.TENSOR_ORDER))
    torch.cuda.synchronize()
    actual = S.output_to_numpy(tensors["attention_out"], "bf16")
    S.assert_close(actual, O.reference_fp32_from_data(data, policy), "reference KernelLaunch / mixed")
    assert np.isfinite(actual).all()
