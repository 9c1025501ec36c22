"""Regenerate `tests/golden/sparse_mla_golden.npz` from the reference project itself.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

The reference's oracle module (`benchmarks/attention/sparse_reference.py`) and
its b16 codec (`benchmarks/validation/dtypes.py`) are imported UNMODIFIED. Their
only non-stdlib dependency is `ascendflow.diagnostics`, so an empty `ascendflow`
package is registered and `src/diagnostics.py` is loaded under that name; the
rest of the compiler (which needs xdsl) is never imported. `make_inputs` lives in
a module whose imports need the compiler and an Ascend runtime, so that one
function is cut out of `benchmarks/attention/sparse_performance.py` by its AST
node and executed as written, with only the names it uses supplied.

Nothing here is used at test time except the `.npz` it writes.
"""

from __future__ import annotations

import ast
import hashlib
import importlib.util
import sys
import types
from pathlib import Path

import numpy as np


def load_reference(root: Path):
    package = types.ModuleType("ascendflow")
    package.__path__ = []
    sys.modules["ascendflow"] = package
    spec = importlib.util.spec_from_file_location("ascendflow.diagnostics", root / "src/diagnostics.py")
    module = importlib.util.module_from_spec(spec)
    sys.modules["ascendflow.diagnostics"] = module
    spec.loader.exec_module(module)
    sys.path.insert(0, str(root))
    import benchmarks.attention.sparse_reference as reference
    import benchmarks.validation.dtypes as codec

    source = (root / "benchmarks/attention/sparse_performance.py").read_text()
    tree = ast.parse(source)
    node = next(n for n in tree.body if isinstance(n, ast.FunctionDef) and n.name == "make_inputs")
    namespace = {
        "np": np,
        "require": module.require,
        "decode": codec.decode,
        "encode": codec.encode,
    }
    exec(compile(ast.Module([node], []), "sparse_performance.make_inputs", "exec"), namespace)
    return reference, codec, namespace["make_inputs"]


def digest(array) -> str:
    array = np.ascontiguousarray(array)
    return hashlib.sha256(str(array.dtype).encode() + str(array.shape).encode() + array.tobytes()).hexdigest()


def policy_of(b, t, h, d, page, ratio, max_seq, window, topk, dtype, blocks):
    return {
        "B": b, "T": t, "H": h, "D": d, "PAGE": page, "RATIO": ratio, "MAX_SEQ": max_seq,
        "ORI_BLOCKS": blocks, "CMP_BLOCKS": blocks, "WINDOW": window, "TOPK": topk,
        "S": window + topk, "DTYPE": dtype, "SCALE": float(d) ** -0.5,
    }


# name -> policy arguments. Small shapes keep the fixture a few hundred KB; the
# last one has the CUDA kernel's compile-time geometry (H64, D512, window 128, TopK 512).
SMALL = {
    "c2_bf16": (4, 16, 4, 32, 16, 2, 128, 8, 16, "bf16", 32),
    "c1_bf16": (4, 16, 4, 32, 16, 1, 128, 8, 16, "bf16", 32),
    "c2_f16": (3, 11, 2, 16, 8, 2, 64, 8, 8, "f16", 24),
    "kernel_geometry": (4, 8, 64, 512, 128, 2, 1024, 128, 512, "bf16", 32),
}
SUBSAMPLE = 61  # stride of the stored output sample for the kernel-geometry policy


def main(root: Path, destination: Path):
    reference, codec, make_inputs = load_reference(root)
    store = {}
    for name, arguments in SMALL.items():
        policy = policy_of(*arguments)
        for case in reference.CASES:
            data = reference.inputs(policy, case)
            key = f"validation/{name}/{case}"
            for field, value in data.items():
                store[f"{key}/input_sha256/{field}"] = np.array(digest(value))
            kv, bias = reference.gather_oracle(data, policy)
            store[f"{key}/gather_kv_sha256"] = np.array(digest(kv))
            store[f"{key}/gather_live"] = np.packbits(np.isfinite(bias))
            out = reference.oracle(data, policy)
            bits = np.frombuffer(codec.encode(out, policy["DTYPE"]), dtype="<u2").reshape(out.shape)
            if name == "kernel_geometry":
                store[f"{key}/output_bits_sample"] = bits.reshape(-1)[::SUBSAMPLE].copy()
            else:
                store[f"{key}/output_bits"] = bits
        # Ragged explicit query lengths, including empty requests.
        lens = [0, 2, 0, arguments[1] - 2] if arguments[0] == 4 else [0, 2, arguments[1] - 2]
        if name != "kernel_geometry":
            data = reference.inputs(policy, "mixed", lens)
            key = f"validation/{name}/mixed_query_lens"
            store[f"{key}/query_lens"] = np.array(lens, dtype=np.int32)
            kv, bias = reference.gather_oracle(data, policy)
            store[f"{key}/gather_kv_sha256"] = np.array(digest(kv))
            store[f"{key}/gather_live"] = np.packbits(np.isfinite(bias))
            out = reference.oracle(data, policy)
            store[f"{key}/output_bits"] = np.frombuffer(
                codec.encode(out, policy["DTYPE"]), dtype="<u2"
            ).reshape(out.shape)

    # Measurement-input generator: B1 prefill and multi-request decode, C1 and C2.
    for name, (b, t, ratio, context, seed) in {
        "prefill_c2": (1, 8, 2, 8, 41),
        "prefill_c1": (1, 8, 1, 8, 41),
        "chunk_c2": (1, 8, 2, 13, 7),
        "decode_c2": (3, 9, 2, 16, 11),
    }.items():
        policy = policy_of(b, t, 2, 4, 4, ratio, 16, 3, 4, "bf16", 4 * b)
        arrays, patches, valid = make_inputs(policy, context, seed)
        key = f"performance/{name}"
        store[f"{key}/arguments"] = np.array([b, t, ratio, context, seed], dtype=np.int64)
        for field, value in arrays.items():
            store[f"{key}/array_sha256/{field}"] = np.array(digest(value))
        store[f"{key}/valid"] = np.packbits(valid)
        for cache, page in (("ori_kv", 4), ("cmp_kv", 4 // ratio)):
            shape = (4 * b, page, 1, 4)
            raw = bytearray(int(np.prod(shape)) * 2)
            for offset, value in patches[cache]:
                raw[offset : offset + len(value)] = value
            store[f"{key}/cache_bits/{cache}"] = np.frombuffer(bytes(raw), dtype="<u2").reshape(shape).copy()

    # b16 codec on awkward values: ties, subnormals, large magnitudes.
    probe = np.array(
        [0.0, -0.0, 1.0, 1.00390625, 1.01171875, -1.00390625, 3.0e38, -3.0e38, 1e-40, 65504.0,
         0.333333343, 2.0 ** -24, 1.0 + 2.0 ** -8, 1.0 + 3 * 2.0 ** -9],
        dtype=np.float32,
    )
    probe = np.concatenate([probe, np.random.default_rng(5).normal(0, 4, 4096).astype(np.float32)])
    store["codec/probe"] = probe
    for dtype in ("bf16", "f16"):
        with np.errstate(over="ignore"):
            store[f"codec/{dtype}"] = np.frombuffer(codec.encode(probe, dtype), dtype="<u2").copy()

    np.savez_compressed(destination, **store)
    print(f"wrote {destination} ({destination.stat().st_size} bytes, {len(store)} entries)")


if __name__ == "__main__":
    reference_root = Path(sys.argv[1]) if len(sys.argv) > 1 else Path(__file__).resolve().parents[3] / "reference"
    main(reference_root, Path(__file__).with_name("sparse_mla_golden.npz"))
