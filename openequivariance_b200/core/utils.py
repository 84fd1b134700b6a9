"""Small shared helpers: dtype enums, the supported-problem guard, layout transposes, hashing.

Mirrors the parts of openequivariance/openequivariance/core/utils.py that the hot path's
callers rely on (``DTypeEnum`` :13-22, ``filter_and_analyze_problem`` :81-117,
``torch_to_oeq_dtype`` :120-138, ``hash_str_64`` :208-209, ``transpose_irrep_layout`` :212-260).
"""

from __future__ import annotations

import hashlib
import math
from enum import IntEnum

import numpy as np

from .irreps import Irreps
from .problem import TPProblem
from .wigner import wigner_3j


class DTypeEnum(IntEnum):
    """Numeric dtype tags shared with the native library (``include/oeq_b200.h``)."""

    FLOAT32 = 1
    FLOAT64 = 2
    INT32 = 3
    INT64 = 4
    UINT8 = 5


dtype_to_enum = {}
for _np_type, _tag in ((np.float32, DTypeEnum.FLOAT32), (np.float64, DTypeEnum.FLOAT64),
                       (np.int32, DTypeEnum.INT32), (np.int64, DTypeEnum.INT64), (np.uint8, DTypeEnum.UINT8)):
    dtype_to_enum[_np_type] = _tag
    dtype_to_enum[np.dtype(_np_type)] = _tag


def calc_weight_offsets(tpp: TPProblem) -> list:
    """Start of every instruction's weight block in the flat weight vector (unweighted ones take no room)."""
    offsets, cursor = [], 0
    for ins in tpp.instructions:
        offsets.append(cursor)
        if ins.has_weight:
            cursor += math.prod(ins.path_shape)
    return offsets


def count_cg_non_zero(l1: int, l2: int, l3: int) -> int:
    return int(np.count_nonzero(wigner_3j(l1, l2, l3)))


def filter_and_analyze_problem(problem: TPProblem) -> dict:
    """Rejects (``AssertionError``) the configurations the kernels do not handle, exactly the set the
    reference rejects: mixed connection modes, unweighted paths, modes other than uvu/uvw,
    ir_mul with uvw, differing irrep/weight dtypes, internal weights, no instructions."""
    assert len(problem.instructions) > 0, "Tensor product has no valid instructions!"
    first_mode = problem.instructions[0].connection_mode
    for i, inst in enumerate(problem.instructions):
        assert inst.connection_mode == first_mode, (
            f"All instructions must have the same connection mode, got {inst.connection_mode} and {first_mode}")
        assert inst.has_weight, f"All instructions must have trainable weights, got {inst.has_weight} at index {i}"
    assert first_mode in ["uvu", "uvw"], f"Connection mode must be 'uvu' or 'uvw', got {first_mode}"
    if problem.layout == "ir_mul":
        assert first_mode == "uvu", "layout='ir_mul' is only supported for pure 'uvu' problems"
    assert problem.irrep_dtype == problem.weight_dtype, (
        f"irrep_dtype and weight_dtype must be the same, got {problem.irrep_dtype} and {problem.weight_dtype}")
    assert not problem.internal_weights, (
        f"Openequivariance does not support internal weights, got {problem.internal_weights}")
    return {"is_uvw": first_mode == "uvw"}


def torch_to_oeq_dtype(torch_dtype):
    """torch.float32 / torch.float64 -> np.float32 / np.float64 (the types ``TPProblem`` takes)."""
    import torch

    if torch_dtype == torch.float32:
        return np.float32
    if torch_dtype == torch.float64:
        return np.float64
    raise ValueError("Unsupported torch dtype!")


def oeq_to_torch_dtype(oeq_dtype):
    import torch

    if oeq_dtype == np.float32:
        return torch.float32
    if oeq_dtype == np.float64:
        return torch.float64
    raise ValueError("Unsupported numpy dtype!")


def hash_str_64(s: str) -> int:
    """56-bit key derived from sha256, small enough for a torch ``int`` op argument."""
    return int.from_bytes(hashlib.sha256(s.encode()).digest()[:7], "big")


def transpose_irrep_layout(array: np.ndarray, irreps: Irreps, src_layout: str, dst_layout: str) -> np.ndarray:
    """NumPy transpose of ``[..., irreps.dim]`` features between ``mul_ir`` ([mul][2l+1] per block) and
    ``ir_mul`` ([2l+1][mul] per block).  Always returns a new array."""
    for name, layout in (("src_layout", src_layout), ("dst_layout", dst_layout)):
        if layout not in ("mul_ir", "ir_mul"):
            raise ValueError(f"Unsupported {name}: {layout}")
    x = np.asarray(array)
    out = np.empty_like(x)
    if src_layout == dst_layout:
        out[...] = x
        return out
    lead = x.shape[:-1]
    for seg, (mul, ir) in zip(irreps.slices(), irreps):
        block = x[..., seg]
        inner = (ir.dim, mul) if src_layout == "ir_mul" else (mul, ir.dim)
        out[..., seg] = block.reshape(*lead, *inner).swapaxes(-1, -2).reshape(*lead, mul * ir.dim)
    return out
