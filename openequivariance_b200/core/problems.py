"""Problem constructors used by models, tests and benchmarks.

Same names and semantics as openequivariance/openequivariance/benchmark/problems.py
(``FullyConnectedTPProblem`` :14-33, ``ChannelwiseTPP`` :122-170, ``SingleInstruction`` :172-196,
model zoos :292-347), which follow e3nn's ``FullyConnectedTensorProduct`` and MACE's channelwise
instruction builder.
"""

from __future__ import annotations

from typing import Optional

import numpy as np

from .irreps import Irreps
from .problem import TPProblem


class FullyConnectedTPProblem(TPProblem):
    """Every (in1, in2, out) triple allowed by the selection rules, mode ``uvw`` (NequIP / e3nn style)."""

    def __init__(self, irreps_in1, irreps_in2, irreps_out, **kwargs) -> None:
        L1, L2, L3 = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
        instructions = []
        for a, (_, ir_a) in enumerate(L1):
            for b, (_, ir_b) in enumerate(L2):
                allowed = set(ir_a * ir_b)
                for o, (_, ir_o) in enumerate(L3):
                    if ir_o in allowed:
                        instructions.append((a, b, o, "uvw", True, 1.0))
        super().__init__(L1, L2, L3, instructions, **kwargs)


class ChannelwiseTPP(TPProblem):
    """MACE-style channelwise product: one ``uvu`` path per allowed (l1, l2, l3), output blocks sorted by
    irrep, per-item (unshared) weights.  The requested ``irreps_out`` only filters which irreps survive."""

    def __init__(self, irreps_in1, irreps_in2, irreps_out, label: Optional[str] = None,
                 irrep_dtype=np.float32, weight_dtype=np.float32):
        L1, L2, keep = Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_out)
        blocks, paths = [], []
        for a, (mul, ir_a) in enumerate(L1):
            for b, (_, ir_b) in enumerate(L2):
                for ir_o in ir_a * ir_b:
                    if ir_o in keep:
                        paths.append((a, b, len(blocks)))
                        blocks.append((mul, ir_o))
        sorted_out, new_index, _ = Irreps(blocks).sort()
        instructions = sorted(((a, b, new_index[o], "uvu", True) for a, b, o in paths), key=lambda t: t[2])
        super().__init__(L1, L2, sorted_out, instructions, internal_weights=False, shared_weights=False,
                         label=label, irrep_dtype=irrep_dtype, weight_dtype=weight_dtype)


class SingleInstruction(TPProblem):
    """One instruction ``(0, 0, 0, mode, True)`` between single-block irreps, unshared weights."""

    def __init__(self, irreps_in1, irreps_in2, irreps_in3, mode: str, label: Optional[str] = None):
        super().__init__(Irreps(irreps_in1), Irreps(irreps_in2), Irreps(irreps_in3), [(0, 0, 0, mode, True)],
                         internal_weights=False, shared_weights=False, label=label)


FCTPP = FullyConnectedTPProblem
CTPP = ChannelwiseTPP


def mace_problems():
    return [
        CTPP("128x0e+128x1o+128x2e", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e+128x3o", "mace-large"),
        CTPP("128x0e+128x1o", "1x0e+1x1o+1x2e+1x3o", "128x0e+128x1o+128x2e", "mace-medium"),
    ]


def nequip_problems():
    lips = "32x0o + 32x0e + 32x1o + 32x1e + 32x2o + 32x2e"
    aspirin = "64x0o + 64x0e + 64x1o + 64x1e"
    toluene = "64x0o + 64x0e + 64x1o + 64x1e + 64x2o + 64x2e"
    benzene = "64x0o + 64x0e + 64x1o + 64x1e + 64x2o + 64x2e + 64x3o + 64x3e"
    water = "32x0o + 32x0e + 32x1o + 32x1e"
    return [
        CTPP(lips, "0e + 1o + 2e", lips, "nequip-lips"),
        CTPP(aspirin, "0e + 1o", aspirin, "nequip-revmd17-aspirin"),
        CTPP(toluene, "0e + 1o + 2e", toluene, "nequip-revmd17-toluene"),
        CTPP(benzene, "0e + 1o + 2e + 3o", benzene, "nequip-revmd17-benzene"),
        CTPP(water, "0e + 1o", water, "nequip-water"),
    ]


def e3nn_torch_tetris_poly_problems():
    return [
        FCTPP("1x0e + 1x1o + 1x2e + 1x3o", "1x0e + 1x1o + 1x2e + 1x3o",
              "64x0e + 24x1e + 24x1o + 16x2e + 16x2o", label="tetris-poly-1"),
        FCTPP("64x0e + 24x1e + 24x1o + 16x2e + 16x2o", "1x0e + 1x1o + 1x2e", "0o + 6x0e", label="tetris-poly-2"),
    ]


def diffdock_problems():
    feats = "10x1o + 10x1e + 48x0e + 48x0o"
    return [
        FCTPP(feats, "1x0e + 1x1o", feats, shared_weights=False, label="DiffDock-L=1"),
        FCTPP(feats, "1x0e + 1x1o + 1x2e", feats, shared_weights=False, label="DiffDock-L=2"),
    ]


# ---- the three signatures the headline benchmarks are quoted on -------------------------------------------

def readme_problem(dtype=np.float32) -> TPProblem:
    """``1x2e (x) 1x3e -> 1x2e``, one ``uvu`` path, per-item weights: the reference README's first example."""
    return TPProblem(Irreps("1x2e"), Irreps("1x3e"), Irreps("1x2e"), [(0, 0, 0, "uvu", True)],
                     shared_weights=False, internal_weights=False, irrep_dtype=dtype, weight_dtype=dtype)


def mace_like_problem(dtype=np.float32) -> TPProblem:
    """128 channels of l<=3 features times l<=3 edge harmonics, every allowed output with l<=3 (23 ``uvu`` paths)."""
    feats = "128x0e+128x1o+128x2e+128x3o"
    return ChannelwiseTPP(feats, "1x0e+1x1o+1x2e+1x3o", feats, "mace-like", irrep_dtype=dtype, weight_dtype=dtype)


def nequip_like_problem(dtype=np.float32) -> TPProblem:
    """32 channels of both parities for l<=2, l<=2 edge harmonics, all 30 ``uvw`` paths, shared weights."""
    feats = "32x0e+32x0o+32x1e+32x1o+32x2e+32x2o"
    return FullyConnectedTPProblem(feats, "1x0e+1x1o+1x2e", feats, shared_weights=True, label="nequip-like",
                                   irrep_dtype=dtype, weight_dtype=dtype)
