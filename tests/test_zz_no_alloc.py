"""The launch entry that allocates nothing, against the ordinary entry, through the C ABI.

`launch_sparse_mla_static_workspace` is for callers that cannot allocate device memory around
the call (an engine step under an allocator freeze, a plugin given a fixed arena): its workspace
is a static device array inside the library. This file is collected last on purpose, so that a
run that stops at the first failure has already run every other test. It must pass alone in a
fresh process and after the other tests.
"""

import ctypes as ct

import numpy as np
import pytest

from oracle import sparse_mla_oracle as O
from tests import support as S

pytestmark = pytest.mark.gpu


def test_static_workspace_entry_matches_the_ordinary_entry_twice_in_a_row():
    import torch

    from ascendflow_b200 import ops
    from ascendflow_b200.build import library_path
    from ascendflow_b200.runtime.torch import _library

    library = _library(library_path())
    launch = library.launch_sparse_mla_static_workspace
    launch.argtypes = [ct.c_void_p] * 14 + [ct.c_int64] * 6
    launch.restype = ct.c_int
    library.read_status_sparse_mla.argtypes = [ct.c_void_p, ct.c_void_p, ct.POINTER(ct.c_int32)]
    library.read_status_sparse_mla.restype = ct.c_int

    policy = O.make_policy(4, 16, max_seq=4096, blocks=128)
    stream = torch.cuda.current_stream().cuda_stream
    for call, case in enumerate(("mixed", "sink")):  # two calls in a row share the static array
        data = O.validation_inputs(policy, case)
        tensors, _ = S.to_device(data, policy)
        ops.sparse_mla(*(tensors[name] for name in S.TENSOR_ORDER))
        expected = tensors["attention_out"].clone()
        tensors["attention_out"].fill_(float("nan"))
        allocated = torch.cuda.memory_allocated()
        status = launch(stream, *(tensors[name].data_ptr() for name in S.TENSOR_ORDER),
                        policy["B"], policy["T"], policy["MAX_SEQ"] // 128, policy["ORI_BLOCKS"],
                        policy["CMP_BLOCKS"], 128 // policy["RATIO"])
        assert status == 0, f"call {call}: status {status}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated
        words = (ct.c_int32 * 8)()
        assert library.read_status_sparse_mla(ct.c_void_p(stream), None, words) == 0
        assert words[0] == 0, f"call {call}: status block {list(words)}"
        actual = S.output_to_numpy(tensors["attention_out"], "bf16")
        # Same kernel on the same inputs: identical, and within the suite's bars of the reference.
        assert np.array_equal(actual, S.output_to_numpy(expected, "bf16")), f"call {call}"
        S.assert_close(actual, O.reference_fp32_from_data(data, policy), f"static workspace / {case}")


def test_static_workspace_entry_refuses_bad_sizes_without_launching():
    from ascendflow_b200.build import library_path
    from ascendflow_b200.runtime.torch import _library

    launch = _library(library_path()).launch_sparse_mla_static_workspace
    launch.argtypes = [ct.c_void_p] * 14 + [ct.c_int64] * 6
    launch.restype = ct.c_int
    assert launch(*([None] * 14), 4, -1, 32, 128, 128, 64) == -1
    assert launch(*([None] * 14), 4, 1 << 62, 32, 128, 128, 64) == -1
