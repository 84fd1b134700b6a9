"""Problem descriptor: the byte payload handed to the native library in place of kernel source.

The reference ships a JSON string holding generated CUDA source, launch configs and ``kernel_prop``
through the ``json_bytes`` op argument (openequivariance/openequivariance/core/LoopUnrollTP.py:100-127,
LoopUnrollConv.py:187-223).  Here the payload is a small line-oriented text record describing the
*problem* (irreps, instructions, folded Clebsch-Gordan nonzeros); the native library parses it,
specialises its hand-written kernel templates for it and caches the result under ``hash``.

Grammar (one record per line, blank-separated, ``#`` starts a comment)::

    OEQB 1
    dtype <1=f32|2=f64>
    layout <0=mul_ir|1=ir_mul>
    shared <0|1>
    mode <uvu|uvw>
    conv <0|1> <deterministic 0|1> <kahan 0|1> <idx dtype enum>
    L1 <nblocks> <dim>            followed by nblocks lines  "<mul> <l> <parity> <offset>"
    L2 ... / L3 ...               likewise
    wn <weight_numel>
    ins <count>
    I <i_in1> <i_in2> <i_out> <weight_offset> <nnz>    followed by nnz lines "<i> <j> <k> <coef>"
    end

``coef`` is ``path_weight * wigner_3j[i, j, k]`` written as a C99 hex float (exact double).
``weight_offset`` is the start of the instruction's block in the kernel-order weight vector.
"""

from __future__ import annotations

import numpy as np

from .problem import TPProblem
from .utils import calc_weight_offsets, dtype_to_enum, filter_and_analyze_problem, hash_str_64
from .wigner import wigner_3j

CG_ZERO_TOL = 1e-12


def folded_cg(problem: TPProblem, ins_index: int):
    """Nonzeros ``(i, j, k, path_weight*C[i,j,k])`` of one instruction, ordered by (j, i, k)."""
    ins = problem.instructions[ins_index]
    l1 = problem.irreps_in1[ins.i_in1].ir.l
    l2 = problem.irreps_in2[ins.i_in2].ir.l
    l3 = problem.irreps_out[ins.i_out].ir.l
    c = wigner_3j(l1, l2, l3)
    ii, jj, kk = np.nonzero(np.abs(c) > CG_ZERO_TOL)
    order = np.lexsort((kk, ii, jj))
    return [(int(ii[n]), int(jj[n]), int(kk[n]), float(c[ii[n], jj[n], kk[n]] * ins.path_weight)) for n in order]


def _irreps_lines(tag: str, irreps) -> list:
    lines = [f"{tag} {len(irreps)} {irreps.dim}"]
    for sl, (mul, ir) in zip(irreps.slices(), irreps):
        lines.append(f"{mul} {ir.l} {ir.p} {sl.start}")
    return lines


def build_descriptor(problem: TPProblem, *, conv: bool = False, deterministic: bool = False,
                     kahan: bool = False, idx_dtype=np.int64) -> str:
    """Serialises ``problem`` (after the supported-problem guard) into the descriptor text."""
    filter_and_analyze_problem(problem)
    mode = problem.instructions[0].connection_mode
    lines = [
        "OEQB 1",
        f"dtype {int(dtype_to_enum[problem.irrep_dtype])}",
        f"layout {1 if problem.layout == 'ir_mul' else 0}",
        f"shared {int(bool(problem.shared_weights))}",
        f"mode {mode}",
        f"conv {int(conv)} {int(deterministic)} {int(kahan)} {int(dtype_to_enum[idx_dtype])}",
    ]
    lines += _irreps_lines("L1", problem.irreps_in1)
    lines += _irreps_lines("L2", problem.irreps_in2)
    lines += _irreps_lines("L3", problem.irreps_out)
    lines.append(f"wn {problem.weight_numel}")
    lines.append(f"ins {len(problem.instructions)}")
    offsets = calc_weight_offsets(problem)
    for n, ins in enumerate(problem.instructions):
        nz = folded_cg(problem, n)
        lines.append(f"I {ins.i_in1} {ins.i_in2} {ins.i_out} {offsets[n]} {len(nz)}")
        lines += [f"{i} {j} {k} {float(c).hex()}" for i, j, k, c in nz]
    lines.append("end")
    return "\n".join(lines) + "\n"


def descriptor_hash(text: str) -> int:
    return hash_str_64(text)
