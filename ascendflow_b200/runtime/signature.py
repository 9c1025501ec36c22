"""The tensor signature a launch library declares, and the checks a call must pass.

A library describes each kernel in a JSON document returned by `kernel_metadata_<name>`
(format of the reference's `src/backend/abi.py:43-59`; checked by its `TensorKernel.bind`,
`src/runtime/torch.py:100-168`): ordered tensors with dtype, shape and access, named int64 size
parameters with a minimum and a multiple, and whether external tensors must be disjoint. A
shape entry is an integer, the name of a size parameter, or `{"mul": [a, b]}` /
`{"add": [a, b]}` over such entries. Sizes the caller does not pass are read off the tensors.

Every failed check raises `CompileError` and happens before anything is enqueued: no implicit
cast, copy or padding is ever made.
"""

import json
from dataclasses import dataclass

from ..diagnostics import require

TARGET = "sm_100a"
DTYPE_NAMES = {"f16": "float16", "bf16": "bfloat16", "f32": "float32", "i32": "int32", "i64": "int64"}
_INT64_LIMIT = 1 << 63


@dataclass(frozen=True)
class TensorSpec:
    name: str
    dtype: str
    shape: tuple
    layout: str
    access: str


@dataclass(frozen=True)
class SizeSpec:
    name: str
    minimum: int
    multiple: int


def evaluate(entry, sizes):
    """Value of one shape entry under the size assignment `sizes`."""
    if type(entry) is int:
        return entry
    if isinstance(entry, str):
        require(entry in sizes, f"missing runtime parameter {entry}; pass it by name")
        return sizes[entry]
    well_formed = isinstance(entry, dict) and len(entry) == 1 and set(entry) <= {"mul", "add"}
    require(well_formed, "invalid compiled tensor extent")
    (operator, operands), = entry.items()
    require(isinstance(operands, list) and len(operands) == 2, "invalid compiled tensor extent operands")
    first, second = evaluate(operands[0], sizes), evaluate(operands[1], sizes)
    return first + second if operator == "add" else first * second


class Signature:
    """Parsed metadata of one kernel."""

    def __init__(self, document, name):
        data = json.loads(document)
        require(data["version"] == 1 and data["name"] == name, "compiled kernel ABI version/name differs")
        require(data["target"] == TARGET, f"tensor runtime requires {TARGET}")
        self.raw = data
        self.name = name
        self.tensors = tuple(TensorSpec(t["name"], t["dtype"], tuple(t["shape"]), t["layout"], t["access"])
                             for t in data["tensors"])
        self.sizes = tuple(SizeSpec(s["name"], s["minimum"], s["multiple"]) for s in data["parameters"])
        self.disjoint = bool(data["disjoint_external"])

    @property
    def tensor_names(self):
        return tuple(spec.name for spec in self.tensors)

    @property
    def size_names(self):
        return tuple(spec.name for spec in self.sizes)

    def check_tensor(self, torch, spec, tensor):
        """Type, placement, storage and rank of one argument."""
        name = spec.name
        require(isinstance(tensor, torch.Tensor), f"{name}: expected a Torch tensor")
        require(tensor.device.type == "cuda", f"{name}: expected a CUDA tensor")
        require(tensor.is_contiguous(), f"{name}: expected contiguous tensor storage")
        require(spec.layout == "linear", f"{name}: unsupported compiled tensor layout")
        require(tensor.dtype == getattr(torch, DTYPE_NAMES[spec.dtype]),
                f"{name}: tensor dtype differs from compiled ABI")
        require(len(tensor.shape) == len(spec.shape), f"{name}: tensor rank differs from compiled ABI")

    def solve_sizes(self, tensors, given):
        """Complete `given` from the dimensions that are plain size names; returns name -> value."""
        require(all(type(v) is int and 0 <= v < _INT64_LIMIT for v in given.values()),
                "runtime parameters require nonnegative int64 integers")
        sizes = dict(given)
        for spec, tensor in zip(self.tensors, tensors):
            for extent, entry in zip(tensor.shape, spec.shape):
                if not isinstance(entry, str):
                    continue
                if entry in sizes:
                    require(sizes[entry] == extent, f"{spec.name}: conflicting runtime dimension {entry}")
                else:
                    sizes[entry] = int(extent)
        return sizes

    def check_shapes_and_sizes(self, tensors, sizes):
        for spec, tensor in zip(self.tensors, tensors):
            wanted = tuple(evaluate(entry, sizes) for entry in spec.shape)
            require(tuple(tensor.shape) == wanted, f"{spec.name}: tensor shape differs from compiled ABI")
        for spec in self.sizes:
            require(spec.name in sizes, f"missing runtime parameter {spec.name}; pass it by name")
            value = sizes[spec.name]
            require(spec.minimum <= value < _INT64_LIMIT and value % spec.multiple == 0,
                    f"{spec.name}: runtime input contract differs")

    def check_disjoint(self, tensors):
        """No two non-empty arguments may overlap in memory (the kernels assume it)."""
        if not self.disjoint:
            return
        spans = sorted((t.data_ptr(), t.data_ptr() + t.numel() * t.element_size())
                       for t in tensors if t.numel())
        clash = any(later[0] < earlier[1] for earlier, later in zip(spans, spans[1:]))
        require(not clash, "external tensors violate the compiled disjoint contract")
