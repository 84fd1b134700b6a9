"""Symmetric contraction (the node-wise product basis that follows the convolution in MACE) on the library's ragged
grouped product kernels.

Counterpart of openequivariance/openequivariance/_torch/symmetric_contraction/symmetric_contraction.py:

* ``GroupMM`` (reference :7-108) -- the ragged grouped product as a torch custom op with autograd; the work is done by
  ``oeqb_group_mm`` (one kernel launch per call) instead of one cuBLAS strided-batched GEMM per chemical element.
* ``Contraction`` / ``SymmetricContraction`` (reference :233-422) -- the contraction of node features with the
  generalised Clebsch-Gordan tensors ``U`` and element-dependent weights.  The reference builds ``U`` with e3nn
  (``U_matrix_real``, code it takes from MACE); e3nn is not a dependency of this library, so the tensors are an
  argument here: pass the ones MACE / e3nn give you (``U_matrix_real(irreps_in, irreps_out, correlation=nu)[-1]``).

Math (MACE's symmetric contraction), for one output irrep, features ``x [N, F, ell]``, element ``e(n)`` of node ``n``,
correlation order ``nu_max``:  ``out = sum_k U_numax[..., i, k] W_numax[e, k, f] x[n, f, i]`` and then, for
``nu = nu_max - 1 ... 1``:  ``out = sum_i (sum_k U_nu[..., i, k] W_nu[e, k, f] + out[..., i]) x[n, f, i]``.
"""

from __future__ import annotations

import ctypes
from typing import Dict, List, Optional, Sequence

import torch

from .. import native

_DTYPE_ENUM = {torch.float32: 1, torch.float64: 2}


def _check_cuda(t, name):
    if not t.is_cuda:
        raise RuntimeError(f"Tensor '{name}' is not on the GPU.")


@torch.library.custom_op("oeq_b200::group_gemm", mutates_args=(), device_types="cuda")
def group_gemm(A: torch.Tensor, B: torch.Tensor, ragged_counts: torch.Tensor, M: int, K: int, ragged_inner: int,
               num_elements: int) -> torch.Tensor:
    """``ragged_inner == 0``: ``A [G, F, M, K]``, ``B [N, F, K]`` -> ``[N, F, M]``;
    ``ragged_inner == 1``: ``A [N, F, M]``, ``B [N, F, K]`` -> ``[G, F, M, K]``;
    ``ragged_inner == 2``: ``A [G, F, M, K]``, ``B [N, F, M]`` -> ``[N, F, K]`` (mode 0 with transposed weights).
    ``ragged_counts``: CPU int64 ``[G]``, nodes per group (the nodes are sorted by group)."""
    _check_cuda(A, "A")
    _check_cuda(B, "B")
    if A.dtype not in _DTYPE_ENUM or B.dtype != A.dtype:
        raise RuntimeError(f"Dtype mismatch for tensor 'A' / 'B': {A.dtype}, {B.dtype}")
    counts = ragged_counts.detach().to(device="cpu", dtype=torch.int64).contiguous()
    if counts.numel() != num_elements:
        raise RuntimeError(f"Shape mismatch for tensor 'ragged_counts'. Expected: [{num_elements}]. Got: {list(counts.shape)}")
    N, F = B.shape[0], B.shape[1]
    if int(counts.sum()) != N:
        raise RuntimeError(f"ragged_counts sums to {int(counts.sum())} but the node tensors have {N} rows")
    want_A = (N, F, M) if ragged_inner == 1 else (num_elements, F, M, K)
    want_B = (N, F, M) if ragged_inner == 2 else (N, F, K)
    if tuple(A.shape) != want_A or tuple(B.shape) != want_B:
        raise RuntimeError(f"Shape mismatch for tensor 'A' / 'B'. Expected: {list(want_A)}, {list(want_B)}. "
                           f"Got: {list(A.shape)}, {list(B.shape)}")
    a, b = A.contiguous(), B.contiguous()
    shape = {0: (N, F, M), 1: (num_elements, F, M, K), 2: (N, F, K)}[ragged_inner]
    C = torch.empty(shape, device=a.device, dtype=a.dtype)
    if C.numel() == 0:
        return C
    with torch.cuda.device(a.device):
        rc = native.load().oeqb_group_mm(
            _DTYPE_ENUM[a.dtype], ragged_inner, num_elements, F, M, K,
            ctypes.cast(counts.data_ptr(), ctypes.POINTER(ctypes.c_int64)), ctypes.c_void_p(a.data_ptr()),
            ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(C.data_ptr()),
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    native.check(rc, "group_gemm")
    return C


@group_gemm.register_fake
def _(A, B, ragged_counts, M, K, ragged_inner, num_elements):
    if ragged_inner == 0:
        return A.new_empty(B.shape[0], B.shape[1], M)
    if ragged_inner == 2:
        return A.new_empty(B.shape[0], B.shape[1], K)
    return A.new_empty(num_elements, B.shape[1], M, K)


def _group_gemm_setup(ctx, inputs, output):
    ctx.A, ctx.B, ctx.counts, ctx.M, ctx.K, ctx.ragged_inner, ctx.num_elements = inputs


def _group_gemm_backward(ctx, grad):
    A, B, counts, M, K, G = ctx.A, ctx.B, ctx.counts, ctx.M, ctx.K, ctx.num_elements
    if ctx.ragged_inner == 0:      # C[n,f,m] = sum_k A[g,f,m,k] B[n,f,k]
        grad_A = group_gemm(grad, B, counts, M, K, 1, G)
        grad_B = group_gemm(A, grad, counts, M, K, 2, G)
    elif ctx.ragged_inner == 1:    # C[g,f,m,k] = sum_n A[n,f,m] B[n,f,k]
        grad_A = group_gemm(grad, B, counts, M, K, 0, G)
        grad_B = group_gemm(grad, A, counts, M, K, 2, G)
    else:                          # C[n,f,k] = sum_m A[g,f,m,k] B[n,f,m]
        grad_A = group_gemm(B, grad, counts, M, K, 1, G)
        grad_B = group_gemm(A, grad, counts, M, K, 0, G)
    return grad_A, grad_B, None, None, None, None, None


group_gemm.register_autograd(_group_gemm_backward, setup_context=_group_gemm_setup)


class GroupMM:
    """``GroupMM(dtype, num_elements, batch_size)`` of the reference: ``forward(weights [G, F, M, K], vectors [N, F, K],
    bincounts)`` -> ``[N, F, M]``; ``batch_size`` is the number of feature channels ``F``."""

    def __init__(self, dtype, num_elements, batch_size):
        assert dtype in _DTYPE_ENUM, "float32 or float64"
        self.dtype, self.num_elements, self.batch_size = dtype, num_elements, batch_size

    def group_gemm(self, A, B, ragged_counts, M, K, ragged_inner):
        return group_gemm(A, B, ragged_counts, M, K, ragged_inner, self.num_elements)

    def forward(self, weights, vectors, bincounts):
        return group_gemm(weights, vectors, bincounts, weights.shape[2], weights.shape[3], 0, self.num_elements)


class Contraction(torch.nn.Module):
    """Contraction for one output irrep.  ``U_matrices[nu]`` has shape ``[(2L+1,)] + [ell] * nu + [num_params_nu]``
    for ``nu = 1 ... correlation`` (the leading dimension only when the output irrep has ``L > 0``)."""

    def __init__(self, U_matrices: Dict[int, torch.Tensor], num_features: int, num_elements: int,
                 internal_weights: bool = True, weights: Optional[Sequence[torch.Tensor]] = None, dtype=None):
        super().__init__()
        dtype = dtype or torch.get_default_dtype()
        self.correlation = max(U_matrices)
        assert sorted(U_matrices) == list(range(1, self.correlation + 1)), "U_matrices needs every order 1 ... correlation"
        self.num_features, self.num_elements = num_features, num_elements
        for nu, U in U_matrices.items():
            U = U.to(dtype)
            self.register_buffer(f"U_matrix_{nu}", U)
            # [params, everything else]: the weights are applied with one matrix product per order
            self.register_buffer(f"U_permuted_{nu}", U.movedim(-1, 0).reshape(U.shape[-1], -1).contiguous())
        self.groupMM = GroupMM(dtype, num_elements, num_features)
        if internal_weights:
            ws = []
            for nu in range(self.correlation, 0, -1):
                n_par = self.U(nu).shape[-1]
                ws.append(torch.nn.Parameter(torch.randn(num_elements, n_par, num_features, dtype=dtype) / n_par))
            self.weights_max = ws[0]
            self.weights = torch.nn.ParameterList(ws[1:])
        else:
            # the reference's order: orders correlation-1 ... 1, then the highest order last
            assert weights is not None and len(weights) == self.correlation, "one weight tensor per order"
            self.weights = list(weights[:-1])
            self.weights_max = weights[-1]

    def U(self, nu):
        return getattr(self, f"U_matrix_{nu}")

    def forward(self, x: torch.Tensor, bincount: torch.Tensor, sorted_indices: torch.Tensor) -> torch.Tensor:
        """``x [N, F, ell]`` with the nodes sorted by element, ``bincount`` (CPU) nodes per element, ``sorted_indices [N]``
        the element of each (sorted) node."""
        U = self.U(self.correlation)
        n_par, ell = U.shape[-1], U.shape[-2]
        UW = self.weights_max.transpose(1, 2).reshape(-1, n_par) @ getattr(self, f"U_permuted_{self.correlation}")
        out = self.groupMM.forward(UW.view(self.num_elements, self.num_features, -1, ell), x, bincount)
        out = out.view([x.shape[0], self.num_features] + list(U.shape[:-2]))
        for i, W in enumerate(self.weights):
            nu = self.correlation - i - 1
            U = self.U(nu)
            c = W.transpose(1, 2).reshape(-1, W.shape[1]) @ getattr(self, f"U_permuted_{nu}")
            c = c.view([W.shape[0], W.shape[2]] + list(U.shape[:-1]))[sorted_indices] + out
            s = c.shape
            out = (c.reshape(s[0] * s[1], -1, s[-1]) * x.reshape(s[0] * s[1], 1, s[-1])).sum(dim=2).view(s[:-1])
        return out.reshape(out.shape[0], -1)


class SymmetricContraction(torch.nn.Module):
    """``forward(x [N, F, ell], y [N, num_elements] one-hot)`` -> concatenation over the output irreps of
    ``[N, F * (2L+1)]``.  ``U_matrices_per_irrep``: one ``{nu: U}`` dictionary per output irrep (see ``Contraction``)."""

    def __init__(self, U_matrices_per_irrep: List[Dict[int, torch.Tensor]], num_features: int, num_elements: int,
                 internal_weights: bool = True, weights: Optional[List[Sequence[torch.Tensor]]] = None, dtype=None):
        super().__init__()
        self.num_elements = num_elements
        self.contractions = torch.nn.ModuleList(
            Contraction(U, num_features, num_elements, internal_weights, None if weights is None else weights[i], dtype)
            for i, U in enumerate(U_matrices_per_irrep))

    def forward(self, x: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
        indices = torch.argmax(y, dim=1)
        bincount = torch.bincount(indices, minlength=self.num_elements).to("cpu")
        permutation = torch.argsort(indices, stable=True)
        inverse = torch.argsort(permutation)
        xs, sorted_indices = x[permutation], indices[permutation]
        outs = [c(xs, bincount, sorted_indices) for c in self.contractions]
        return torch.cat(outs, dim=-1)[inverse]
