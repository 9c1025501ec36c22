"""PyTorch surface of the operator: a function and a registered custom op.

`sparse_mla(...)` takes the thirteen tensors of the reference entry
(`examples/sparse_attention/attention.py:210-224`) in the same order with the
same names, layouts and dtypes, the output passed explicitly
(`docs/guide/runtime.md:88-89` of the reference). It launches on torch's current
CUDA stream through the C ABI. There is no CPU or eager fallback: a missing
library or a non-CUDA tensor raises.
"""

from __future__ import annotations

import torch

from .runtime.torch import TorchRuntime

TENSORS = (
    "q", "ori_kv", "cmp_kv", "cmp_sparse_indices", "ori_block_table", "cmp_block_table",
    "cu_seqlens_q", "seqused_ori_kv", "seqused_cmp_kv", "cmp_residual_kv", "ori_topk_length",
    "sinks", "attention_out",
)

_runtime = None
_kernels = {}


def runtime():
    global _runtime
    if _runtime is None or _runtime._closed:
        _runtime = TorchRuntime(torch)
        _kernels.clear()
    return _runtime


def kernel(name="sparse_mla"):
    owner = runtime()
    if name not in _kernels:
        _kernels[name] = owner.kernel(None, name)
    return _kernels[name]


def sparse_mla(q, ori_kv, cmp_kv, cmp_sparse_indices, ori_block_table, cmp_block_table,
               cu_seqlens_q, seqused_ori_kv, seqused_cmp_kv, cmp_residual_kv, ori_topk_length,
               sinks, attention_out):
    """Run sparse MLA attention into `attention_out` on the current stream; returns it."""
    name = "sparse_mla_f16" if q.dtype == torch.float16 else "sparse_mla"
    kernel(name)(q, ori_kv, cmp_kv, cmp_sparse_indices, ori_block_table, cmp_block_table,
                 cu_seqlens_q, seqused_ori_kv, seqused_cmp_kv, cmp_residual_kv, ori_topk_length,
                 sinks, attention_out)
    return attention_out


@torch.library.custom_op("ascendflow_b200::sparse_mla", mutates_args=("attention_out",),
                         device_types="cuda")
def _sparse_mla_op(q: torch.Tensor, ori_kv: torch.Tensor, cmp_kv: torch.Tensor,
                   cmp_sparse_indices: torch.Tensor, ori_block_table: torch.Tensor,
                   cmp_block_table: torch.Tensor, cu_seqlens_q: torch.Tensor,
                   seqused_ori_kv: torch.Tensor, seqused_cmp_kv: torch.Tensor,
                   cmp_residual_kv: torch.Tensor, ori_topk_length: torch.Tensor,
                   sinks: torch.Tensor, attention_out: torch.Tensor) -> None:
    sparse_mla(q, ori_kv, cmp_kv, cmp_sparse_indices, ori_block_table, cmp_block_table,
               cu_seqlens_q, seqused_ori_kv, seqused_cmp_kv, cmp_residual_kv, ori_topk_length,
               sinks, attention_out)


def resolve_rows(cmp_sparse_indices, ori_block_table, cmp_block_table, cu_seqlens_q,
                 seqused_ori_kv, seqused_cmp_kv, cmp_residual_kv, ori_topk_length, *,
                 ori_blocks, cmp_blocks, cmp_page):
    """Export the gathered index set `[T, 640]` int32 (physical cache row or -1 per slot)."""
    import ctypes as ct

    from .build import library_path
    from .diagnostics import require
    from .runtime.torch import _library

    library = _library(library_path())
    tensors = (cmp_sparse_indices, ori_block_table, cmp_block_table, cu_seqlens_q, seqused_ori_kv,
               seqused_cmp_kv, cmp_residual_kv, ori_topk_length)
    for tensor in tensors:
        require(tensor.is_cuda and tensor.is_contiguous() and tensor.dtype == torch.int32,
                "index-set export expects contiguous int32 CUDA tensors")
    tokens, batches, pages = cmp_sparse_indices.shape[0], ori_block_table.shape[0], ori_block_table.shape[1]
    resolved = torch.empty((tokens, 640), dtype=torch.int32, device=cmp_sparse_indices.device)
    workspace = torch.empty(1024, dtype=torch.uint8, device=cmp_sparse_indices.device)
    launch = library.launch_sparse_mla_resolve_rows
    launch.argtypes = [ct.c_void_p] * 11 + [ct.c_int64] * 6
    launch.restype = ct.c_int
    stream = torch.cuda.current_stream(cmp_sparse_indices.device).cuda_stream
    status = launch(stream, *(t.data_ptr() for t in tensors), resolved.data_ptr(), workspace.data_ptr(),
                    batches, tokens, pages, int(ori_blocks), int(cmp_blocks), int(cmp_page))
    if status:
        raise RuntimeError(f"kernel launch failed with status {status}; device retries are disabled")
    return resolved
