"""``transpose_irreps``: differentiable ``mul_ir`` <-> ``ir_mul`` transposition of irrep-packed features
(behaviour of openequivariance/openequivariance/_torch/utils.py:81-147)."""

import torch

from ..core.irreps import Irreps


def transpose_irreps(array: torch.Tensor, irreps: Irreps, src_layout: str, dst_layout: str) -> torch.Tensor:
    r"""
    Transposes ``[..., irreps.dim]`` features block by block between ``mul_ir`` (``[mul][2l+1]``) and
    ``ir_mul`` (``[2l+1][mul]``).  Leading dimensions are preserved and gradients flow through.
    Equal layouts return a copy.

    :raises TypeError: if ``array`` is not a ``torch.Tensor``.
    :raises ValueError: for a layout name other than ``"mul_ir"`` / ``"ir_mul"``.
    """
    if src_layout not in ("mul_ir", "ir_mul"):
        raise ValueError(f"Unsupported src_layout: {src_layout}")
    if dst_layout not in ("mul_ir", "ir_mul"):
        raise ValueError(f"Unsupported dst_layout: {dst_layout}")
    if not isinstance(array, torch.Tensor):
        raise TypeError(f"Expected torch.Tensor, got {type(array)}")
    if src_layout == dst_layout:
        return array.clone()
    lead = array.shape[:-1]
    pieces = []
    for seg, (mul, ir) in zip(Irreps(irreps).slices(), Irreps(irreps)):
        inner = (ir.dim, mul) if src_layout == "ir_mul" else (mul, ir.dim)
        pieces.append(array[..., seg].reshape(*lead, *inner).transpose(-1, -2).reshape(*lead, mul * ir.dim))
    return torch.cat(pieces, dim=-1) if pieces else array.clone()
