"""``TensorProductConv``: drop-in module for the fused tensor product + graph convolution.

Same constructor (``deterministic``, ``kahan``, ``torch_op``, ``use_opaque``), ``forward(X, Y, W, rows, cols,
sender_perm=None)`` contract, ``workspace_buffer`` attribute and harness hooks as
openequivariance/openequivariance/_torch/TensorProductConv.py:32-277 (+ NPDoubleBackwardMixin.py:140-289).
Mode rules follow core/LoopUnrollConv.py:34-46: ``kahan`` needs ``deterministic``; the deterministic
algorithm does not take shared weights.
"""

from __future__ import annotations

from typing import Optional

import numpy as np
import torch

from ..core.problem import TPProblem
from .TensorProduct import _ProblemModule


class TensorProductConv(_ProblemModule):
    r"""
    Given a directed graph :math:`G=(V,E)`, node features :math:`x_j`, edge features :math:`y_e` and edge
    weights :math:`W_e`, computes :math:`z_i = \sum_{(i,j,e)\in\mathcal N(i)} W_e (x_j \otimes_{CG} y_e)`.

    ``deterministic=False`` scatters with atomics (any edge order).  ``deterministic=True`` needs edges sorted
    by (row, col) and ``sender_perm`` (the permutation taking the row-major edge list to column-major order,
    see ``CoordGraph``); results are then bitwise reproducible and independent of launch geometry.

    :param problem: Specification of the tensor product.
    :param deterministic: use the receiver-sorted algorithm. *Default*: ``False``.
    :param kahan: compensated summation over a receiver's edges (fp32, deterministic only). *Default*: ``False``.
    :param use_opaque: Deprecated, ignored.
    """

    _conv = True

    def __init__(self, problem: TPProblem, *, deterministic: bool = False, kahan: bool = False,
                 torch_op: bool = True, use_opaque: bool = False):
        torch.nn.Module.__init__(self)
        self.input_args = {"problem": problem, "deterministic": deterministic, "kahan": kahan,
                           "torch_op": torch_op, "use_opaque": use_opaque}
        self._init_class()

    def _init_class(self):
        self.deterministic = bool(self.input_args["deterministic"])
        self.kahan = bool(self.input_args["kahan"])
        self.idx_dtype = np.int64
        if self.kahan:
            assert self.deterministic, "kahan=True requires deterministic=True"
            assert self.input_args["problem"].irrep_dtype == np.float32, "kahan=True requires float32"
        if self.deterministic:
            assert not self.input_args["problem"].shared_weights, (
                "Deterministic convolution does not support shared weights")
        self._build(deterministic=self.deterministic, kahan=self.kahan, idx_dtype=self.idx_dtype)
        self.kernel_prop.update({"deterministic": int(self.deterministic), "idx_dtype": 4, "workspace_size": 0})
        # Scratch depends on the graph size, so the op layer sizes it per call (oeqb_conv_workspace_bytes) and
        # allocates from torch's caching allocator when this persistent buffer is too small.  Callers that want
        # allocation-free steps can pre-size it with allocate_workspace().
        self.workspace_size = 0
        self.workspace_buffer = None
        self.dummy_transpose_perm = None
        if torch.cuda.is_available():
            self.allocate_workspace(0)
            self.dummy_transpose_perm = torch.zeros(1, dtype=torch.int64, device="cuda")

    def allocate_workspace(self, size_bytes, device="cuda"):
        self.workspace_size = int(size_bytes)
        self.workspace_buffer = torch.zeros(max(int(size_bytes), 1), dtype=torch.uint8, device=device)
        self.workspace_ptr = self.workspace_buffer.data_ptr()

    @staticmethod
    def name():
        return "B200TensorProductConv"

    def forward(self, X: torch.Tensor, Y: torch.Tensor, W: torch.Tensor, rows: torch.Tensor, cols: torch.Tensor,
                sender_perm: Optional[torch.Tensor] = None) -> torch.Tensor:
        r"""
        :param X: ``[|V|, irreps_in1.dim]``.
        :param Y: ``[|E|, irreps_in2.dim]``.
        :param W: ``[|E|, weight_numel]`` or ``[weight_numel]`` (shared), kernel order.
        :param rows: ``[|E|]`` int64 receiver of each edge (row-major sorted with ``cols`` when deterministic).
        :param cols: ``[|E|]`` int64 sender of each edge.
        :param sender_perm: ``[|E|]`` int64, required when ``deterministic=True``.
        :return: ``[|V|, irreps_out.dim]``.
        """
        if sender_perm is None:
            if self.dummy_transpose_perm is None or self.dummy_transpose_perm.device != X.device:
                self.dummy_transpose_perm = torch.zeros(1, dtype=torch.int64, device=X.device)
            sender_perm = self.dummy_transpose_perm
        if self.workspace_buffer is None or self.workspace_buffer.device != X.device:
            self.allocate_workspace(self.workspace_size, X.device)
        return torch.ops.libtorch_tp_jit.jit_conv_forward(self.kernel, self.hash, X, Y, W, self.L3_dim, rows, cols,
                                                          self.workspace_buffer, sender_perm)

    # -- NumPy harness hooks -----------------------------------------------------------------------------------
    def _graph_tensors(self, graph):
        assert graph.rows.dtype == self.idx_dtype and graph.cols.dtype == self.idx_dtype
        rows = torch.tensor(graph.rows, device="cuda")
        cols = torch.tensor(graph.cols, device="cuda")
        perm = torch.tensor(graph.transpose_perm, device="cuda") if self.deterministic else None
        return rows, cols, perm

    def forward_cpu(self, L1_in, L2_in, weights, L3_out, graph):
        w = self.reorder_weights_from_e3nn(weights, not self.config.shared_weights)
        rows, cols, perm = self._graph_tensors(graph)
        out = self.forward(torch.tensor(L1_in, device="cuda"), torch.tensor(L2_in, device="cuda"),
                           torch.tensor(w, device="cuda"), rows, cols, perm)
        L3_out[:] = out.numpy(force=True)

    def backward_cpu(self, L1_in, L1_grad, L2_in, L2_grad, weights, weights_grad, L3_grad, graph):
        w = self.reorder_weights_from_e3nn(weights, not self.config.shared_weights)
        rows, cols, perm = self._graph_tensors(graph)
        x = torch.tensor(L1_in, requires_grad=True, device="cuda")
        y = torch.tensor(L2_in, requires_grad=True, device="cuda")
        wt = torch.tensor(w, requires_grad=True, device="cuda")
        self.forward(x, y, wt, rows, cols, perm).backward(gradient=torch.tensor(L3_grad, device="cuda"))
        L1_grad[:] = x.grad.numpy(force=True)
        L2_grad[:] = y.grad.numpy(force=True)
        weights_grad[:] = self.reorder_weights_to_e3nn(wt.grad.numpy(force=True), not self.config.shared_weights)
        return L1_grad, L2_grad, weights_grad

    def double_backward_cpu(self, in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad, graph):
        from .TensorProduct import TensorProduct
        assert self.torch_op
        rows, cols, perm = self._graph_tensors(graph)
        call = lambda x, y, w: self.forward(x, y, w, rows, cols, perm)  # noqa: E731
        return TensorProduct._second_order(self, in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad, call)

    def triple_backward_cpu(self, in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad, cotangents, graph):
        from .TensorProduct import TensorProduct
        assert self.torch_op
        rows, cols, perm = self._graph_tensors(graph)
        call = lambda x, y, w: self.forward(x, y, w, rows, cols, perm)  # noqa: E731
        return TensorProduct._second_order(self, in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad,
                                           call, third=cotangents)
