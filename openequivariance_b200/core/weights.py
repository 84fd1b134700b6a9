"""The kernel-side ("OEQ") weight order and its conversion from / to e3nn's order.

e3nn stores each instruction's weights row-major in ``(u, v)`` (``uvu``) or ``(u, v, w)`` (``uvw``).
The reference's kernels consume them re-tiled: every multiplicity axis is cut into chunks of 32,
the tiles of one instruction follow each other in ``(u-chunk, v-chunk[, w-chunk])`` row-major order,
and inside a tile the two leading axes are swapped, i.e. a tile is ``[v][u]`` / ``[v][u][w]``
(openequivariance/openequivariance/core/ComputationSchedule.py:185-343 and :651-712,
openequivariance/openequivariance/_torch/utils.py:8-59).  The kernels of this package read weights
in exactly that order, so weights prepared for the reference work unchanged.

This module expresses the whole conversion as one index permutation ``perm`` with
``W_oeq[..., k] = W_e3nn[..., perm[k]]``.
"""

from __future__ import annotations

from math import prod

import numpy as np

from .problem import TPProblem

CHUNK = 32  # multiplicity tile edge; equals the warp width the reference tiles for


def _chunks(n: int):
    return [slice(s, min(s + CHUNK, n)) for s in range(0, n, CHUNK)]


def oeq_weight_permutation(problem: TPProblem) -> np.ndarray:
    """``perm`` (int64, length ``weight_numel``) such that ``W_oeq = W_e3nn[..., perm]``."""
    pieces = []
    for idx, ins in enumerate(problem.instructions):
        start, stop, shape = problem.weight_range_and_shape_for_instruction(idx)
        flat = np.arange(start, stop, dtype=np.int64).reshape(shape)
        if ins.connection_mode == "uvu":
            for us in _chunks(shape[0]):
                for vs in _chunks(shape[1]):
                    pieces.append(flat[us, vs].T.ravel())
        elif ins.connection_mode == "uvw":
            for us in _chunks(shape[0]):
                for vs in _chunks(shape[1]):
                    for ws in _chunks(shape[2]):
                        pieces.append(flat[us, vs, ws].transpose(1, 0, 2).ravel())
        else:
            pieces.append(flat.ravel())
    perm = np.concatenate(pieces) if pieces else np.zeros(0, dtype=np.int64)
    assert perm.shape[0] == problem.weight_numel == sum(prod(i.path_shape) for i in problem.instructions)
    return perm


def _apply(weights, index: np.ndarray, scatter: bool):
    """Gather (``out = w[..., index]``) or scatter (``out[..., index] = w``) along the last axis, for
    numpy arrays and torch tensors alike; the result has the input's type, dtype and device."""
    try:
        import torch
    except ImportError:  # pragma: no cover - torch is a hard dependency of the op layer only
        torch = None
    if torch is not None and isinstance(weights, torch.Tensor):
        idx = torch.as_tensor(index, device=weights.device)
        if not scatter:
            return weights.index_select(-1, idx)
        out = torch.zeros_like(weights)
        out.index_copy_(-1, idx, weights)
        return out
    w = np.asarray(weights)
    if not scatter:
        return w[..., index].copy()
    out = np.zeros_like(w)
    out[..., index] = w
    return out


def reorder_weights(problem: TPProblem, weights, direction: str, perm: np.ndarray = None):
    """``direction="forward"``: e3nn order -> kernel order; ``"backward"``: kernel order -> e3nn order."""
    assert direction in ("forward", "backward")
    if perm is None:
        perm = oeq_weight_permutation(problem)
    return _apply(weights, perm, scatter=(direction == "backward"))
