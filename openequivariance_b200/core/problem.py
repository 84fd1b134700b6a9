"""``TPProblem``: the specification of one weighted Clebsch-Gordan tensor product.

Same constructor signature, attributes and normalisation rule as the reference's
``TPProblem`` (openequivariance/openequivariance/core/e3nn_lite.py:363-653), which in turn
restates e3nn's ``o3.TensorProduct`` bookkeeping: every instruction
``(i_in1, i_in2, i_out, mode, has_weight[, path_weight])`` receives the coefficient
``sqrt(alpha)`` where

* ``alpha`` starts at the irrep-normalisation factor (``component``: ``2*l_out+1``;
  ``norm``: ``(2*l_1+1)(2*l_2+1)``; ``none``: 1),
* is divided by the path-normalisation denominator (``element``: the sum over all
  instructions that write the same output block of ``in1_var*in2_var*fan``; ``path``:
  this instruction's ``in1_var*in2_var*fan`` times the number of such instructions),
  where ``fan`` counts the products summed into one output element
  (``uvu``: mul(in2); ``uvw``: mul(in1)*mul(in2); ...),
* and is multiplied by ``out_var[i_out]`` and the user's path weight.

Weights are laid out instruction after instruction, each block row-major in its
``path_shape`` ((u,v) for ``uvu``, (u,v,w) for ``uvw``): e3nn's order.
"""

from __future__ import annotations

import copy
from math import prod, sqrt
from typing import Any, List, NamedTuple, Optional, Tuple

import numpy as np

from .irreps import Irreps, _MulIr

_MODES = ("uvw", "uvu", "uvv", "uuw", "uuu", "uvuv", "uvu<v", "u<vw")


class Instruction(NamedTuple):
    i_in1: int
    i_in2: int
    i_out: int
    connection_mode: str
    has_weight: bool
    path_weight: float
    path_shape: tuple


def _path_shape(mode: str, m1: int, m2: int, mo: int) -> tuple:
    if mode == "uvw":
        return (m1, m2, mo)
    if mode in ("uvu", "uvv", "uvuv"):
        return (m1, m2)
    if mode == "uuw":
        return (m1, mo)
    if mode == "uuu":
        return (m1,)
    if mode == "uvu<v":
        return (m1 * (m2 - 1) // 2,)
    if mode == "u<vw":
        return (m1 * (m2 - 1) // 2, mo)
    raise KeyError(mode)


def _fan_in(mode: str, m1: int, m2: int) -> int:
    """Number of (in1, in2) products accumulated into one output element by a path."""
    return {
        "uvw": m1 * m2,
        "uvu": m2,
        "uvv": m1,
        "uuw": m1,
        "uuu": 1,
        "uvuv": 1,
        "uvu<v": 1,
        "u<vw": m1 * (m2 - 1) // 2,
    }[mode]


def _variances(given, count: int, what: str) -> List[float]:
    if given is None:
        return [1.0] * count
    out = [float(v) for v in given]
    assert len(out) == count, f"Len of {what} must be equal to len of the matching irreps"
    return out


class TPProblem:
    """
    Specification for a CG tensor product. All parameters of e3nn's ``o3.TensorProduct`` are
    available, plus the datatypes of irreps and weights and the memory layout.

    :param irreps_in1: Irreps of the first argument.
    :param irreps_in2: Irreps of the second argument.
    :param irreps_out: Irreps of the output.
    :param instructions: list of ``(i_in1, i_in2, i_out, mode, has_weight[, path_weight])``.
    :param irrep_dtype: ``np.float32`` (default) or ``np.float64``.
    :param weight_dtype: ``np.float32`` (default) or ``np.float64``.
    :param shared_weights: one weight vector for the whole batch (True, default) or one per item.
    :param internal_weights: must be False; no weights are owned by this package.
    :param irrep_normalization: "component" (default), "norm" or "none".
    :param path_normalization: "element" (default), "path" or "none".
    :param layout: "mul_ir" (default) or "ir_mul".
    """

    instructions: List[Any]
    shared_weights: bool
    internal_weights: bool
    weight_numel: int
    label: str
    layout: str

    def __init__(
        self,
        irreps_in1,
        irreps_in2,
        irreps_out,
        instructions: List[tuple],
        in1_var: Optional[List[float]] = None,
        in2_var: Optional[List[float]] = None,
        out_var: Optional[List[float]] = None,
        irrep_normalization: str = "component",
        path_normalization: str = "element",
        internal_weights: Optional[bool] = False,
        shared_weights: Optional[bool] = None,
        label: Optional[str] = None,
        irrep_dtype: type = np.float32,
        weight_dtype: type = np.float32,
        layout: str = "mul_ir",
    ) -> None:
        assert irrep_normalization in ["component", "norm", "none"]
        assert path_normalization in ["element", "path", "none"]
        assert layout in ["mul_ir", "ir_mul"]
        assert issubclass(irrep_dtype, np.generic)
        assert issubclass(weight_dtype, np.generic)

        self.irreps_in1 = Irreps(irreps_in1)
        self.irreps_in2 = Irreps(irreps_in2)
        self.irreps_out = Irreps(irreps_out)
        self.instructions_raw = instructions
        self.in1_var, self.in2_var, self.out_var = in1_var, in2_var, out_var
        self.irrep_normalization = irrep_normalization
        self.path_normalization = path_normalization
        self.label = label if label is not None else ""
        self.layout = layout

        L1, L2, L3 = self.irreps_in1, self.irreps_in2, self.irreps_out
        v1 = _variances(in1_var, len(L1), "in1_var")
        v2 = _variances(in2_var, len(L2), "in2_var")
        vo = _variances(out_var, len(L3), "out_var")

        parsed = []
        for raw in instructions:
            raw = tuple(raw)
            if len(raw) == 5:
                raw = raw + (1.0,)
            a, b, o, mode, has_weight, user_weight = raw
            assert mode in _MODES
            ir1, ir2, iro = L1[a].ir, L2[b].ir, L3[o].ir
            assert ir1.p * ir2.p == iro.p
            assert abs(ir1.l - ir2.l) <= iro.l <= ir1.l + ir2.l
            parsed.append((a, b, o, mode, has_weight, user_weight))

        # variance mass flowing into each output block, used by "element" normalisation
        mass_into = {}
        paths_into = {}
        for a, b, o, mode, _, _ in parsed:
            mass = v1[a] * v2[b] * _fan_in(mode, L1[a].mul, L2[b].mul)
            mass_into[o] = mass_into.get(o, 0.0) + mass
            paths_into[o] = paths_into.get(o, 0) + 1

        self.instructions = []
        for a, b, o, mode, has_weight, user_weight in parsed:
            if irrep_normalization == "component":
                alpha = L3[o].ir.dim
            elif irrep_normalization == "norm":
                alpha = L1[a].ir.dim * L2[b].ir.dim
            else:
                alpha = 1
            if path_normalization == "element":
                denom = mass_into[o]
            elif path_normalization == "path":
                denom = v1[a] * v2[b] * _fan_in(mode, L1[a].mul, L2[b].mul) * paths_into[o]
            else:
                denom = 1
            if denom > 0.0:
                alpha /= denom
            alpha *= vo[o]
            alpha *= user_weight
            self.instructions.append(
                Instruction(a, b, o, mode, has_weight, sqrt(alpha),
                            _path_shape(mode, L1[a].mul, L2[b].mul, L3[o].mul))
            )

        self._in1_dim = L1.dim
        self._in2_dim = L2.dim

        if shared_weights is False and internal_weights is None:
            internal_weights = False
        if shared_weights is None:
            shared_weights = True
        assert shared_weights or not internal_weights
        self.internal_weights = internal_weights
        self.shared_weights = shared_weights

        self.weight_numel = sum(prod(ins.path_shape) for ins in self.instructions if ins.has_weight)
        self.output_mask = None
        self.irrep_dtype = irrep_dtype
        self.weight_dtype = weight_dtype

    def __str__(self) -> str:
        return (f"{self.__class__.__name__}({self.irreps_in1.simplify()} x "
                f"{self.irreps_in2.simplify()}) -> {self.irreps_out.simplify()}")

    def __repr__(self) -> str:
        lines = [str(self),
                 f"irrep_normalization = {self.irrep_normalization!r}",
                 f"path_normalization = {self.path_normalization!r}",
                 f"internal_weights = {self.internal_weights!r}",
                 f"shared_weights = {self.shared_weights!r}",
                 f"in1_var = {self.in1_var!r}", f"in2_var = {self.in2_var!r}", f"out_var = {self.out_var!r}",
                 f"num weights {self.weight_numel}",
                 "| in1 | in2 | out | l1 | l2 | l3 | m1 | m2 | m3 | mode  | weights | path |"]
        for ins in self.instructions:
            a, b, o = self.irreps_in1[ins.i_in1], self.irreps_in2[ins.i_in2], self.irreps_out[ins.i_out]
            assert isinstance(a, _MulIr) and isinstance(b, _MulIr) and isinstance(o, _MulIr)
            lines.append(
                f"| {ins.i_in1:3} | {ins.i_in2:3} | {ins.i_out:3} | {a.ir.l:2} | {b.ir.l:2} | {o.ir.l:2} |"
                f" {a.mul:3} | {b.mul:3} | {o.mul:3} | {ins.connection_mode:<5} | {str(ins.has_weight):<7} |"
                f" {ins.path_weight:<4.2f} |")
        return "\n".join(lines) + "\n"

    def weight_range_and_shape_for_instruction(self, instruction: int) -> Tuple[int, int, tuple]:
        """``(start, stop, shape)`` of an instruction's block inside the flat e3nn-ordered weight vector."""
        ins = self.instructions[instruction]
        if not ins.has_weight:
            raise ValueError(f"Instruction {instruction} has no weights.")
        start = sum(prod(prev.path_shape) for prev in self.instructions[:instruction])
        return start, start + prod(ins.path_shape), ins.path_shape

    def clone(self):
        return copy.deepcopy(self)
