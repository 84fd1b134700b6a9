"""``TensorProduct``: drop-in ``torch.nn.Module`` for the batched Clebsch-Gordan tensor product.

Same constructor, attributes, ``forward`` contract, weight-reordering helpers, ``.to()`` re-specialisation,
pickling and NumPy harness hooks as openequivariance/openequivariance/_torch/TensorProduct.py:19-179 (with the
double / triple backward drivers of _torch/NPDoubleBackwardMixin.py:10-137).  The work is done by the
``libtorch_tp_jit::jit_tp_*`` ops of ``ops.py``.
"""

from __future__ import annotations

import numpy as np
import torch

from ..core.descriptor import build_descriptor, descriptor_hash
from ..core.problem import TPProblem
from ..core.utils import dtype_to_enum, oeq_to_torch_dtype, torch_to_oeq_dtype
from ..core.weights import oeq_weight_permutation, reorder_weights
from . import ops  # noqa: F401  (registers the ops)


def string_to_tensor(text: str) -> torch.Tensor:
    """UTF-8 bytes of ``text`` as a CPU uint8 tensor (the ``json_bytes`` op argument)."""
    return torch.tensor(np.frombuffer(text.encode("utf-8"), dtype=np.uint8).copy(), device="cpu")


class _ProblemModule(torch.nn.Module):
    """Behaviour shared by ``TensorProduct`` and ``TensorProductConv``: descriptor, weight order, dtype moves."""

    _conv = False

    def _build(self, **descriptor_flags):
        problem: TPProblem = self.input_args["problem"]
        self.config = problem.clone()
        self.L1, self.L2, self.L3 = self.config.irreps_in1, self.config.irreps_in2, self.config.irreps_out
        self.torch_op = self.input_args.get("torch_op", True)
        self.kernel_string = build_descriptor(self.config, conv=self._conv, **descriptor_flags)
        self.hash = descriptor_hash(self.kernel_string)
        self.kernel = string_to_tensor(self.kernel_string)
        self.L3_dim = self.L3.dim
        self.weight_numel = self.config.weight_numel
        self.kernel_prop = {
            "L1_dim": self.L1.dim, "L2_dim": self.L2.dim, "L3_dim": self.L3.dim,
            "weight_numel": self.config.weight_numel, "shared_weights": int(self.config.shared_weights),
            "irrep_dtype": dtype_to_enum[self.config.irrep_dtype], "weight_dtype": dtype_to_enum[self.config.weight_dtype],
        }
        self._weight_perm = oeq_weight_permutation(self.config)

    # -- dtype moves re-specialise the kernels, device moves are free (nothing is owned) ----------------------
    def to(self, *args, **kwargs):
        r"""See ``torch.nn.Module.to``; a dtype change rebuilds the problem for that dtype."""
        _, dtype, _, _ = torch._C._nn._parse_to(*args, **kwargs)
        if dtype is not None:
            updated = self.input_args["problem"].clone()
            updated.irrep_dtype = torch_to_oeq_dtype(dtype)
            updated.weight_dtype = torch_to_oeq_dtype(dtype)
            self.input_args["problem"] = updated
            self._init_class()
        torch.nn.Module.to(self, *args, **kwargs)
        return self

    def _apply(self, fn, recurse=True):
        if getattr(self, "_applying", False):
            return super()._apply(fn, recurse)
        current = oeq_to_torch_dtype(self.input_args["problem"].irrep_dtype)
        probe = fn(torch.tensor(0.0, dtype=current))
        if probe.dtype != current and probe.dtype in (torch.float32, torch.float64):
            self._applying = True
            try:
                self.to(probe.dtype)
            finally:
                self._applying = False
        return super()._apply(fn, recurse)

    def __getstate__(self):
        return self.input_args

    def __setstate__(self, state):
        torch.nn.Module.__init__(self)
        self.input_args = state
        self._init_class()

    def reorder_weights_from_e3nn(self, weights, has_batch_dim=True):
        r"""e3nn weight order -> the order the kernels read (numpy in -> numpy out, torch in -> torch out)."""
        return reorder_weights(self.config, weights, "forward", self._weight_perm)

    def reorder_weights_to_e3nn(self, weights, has_batch_dim=True):
        r"""Inverse of :py:meth:`reorder_weights_from_e3nn`."""
        return reorder_weights(self.config, weights, "backward", self._weight_perm)


class TensorProduct(_ProblemModule):
    r"""
    Drop-in replacement for ``o3.TensorProduct`` from e3nn: forward, backward and double backward run as
    hand-written sm_100a kernels specialised for the problem.  Construction fails with ``AssertionError``
    for unsupported specifications (mixed connection modes, unweighted paths, modes other than
    ``uvu``/``uvw``, internal weights, ``ir_mul`` with ``uvw``).

    :param problem: Specification of the tensor product.
    :param use_opaque: Deprecated, ignored.
    """

    def __init__(self, problem: TPProblem, torch_op=True, use_opaque=False):
        torch.nn.Module.__init__(self)
        self.input_args = {"problem": problem, "torch_op": torch_op, "use_opaque": use_opaque}
        self._init_class()

    def _init_class(self):
        self._build()

    @staticmethod
    def name():
        return "B200TensorProduct"

    def forward(self, x: torch.Tensor, y: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
        r"""
        :math:`W (x \otimes_{\textrm{CG}} y)`, identical to ``o3.TensorProduct.forward`` up to weight order.

        :param x: ``[batch, irreps_in1.dim]``, dtype ``problem.irrep_dtype``.
        :param y: ``[batch, irreps_in2.dim]``.
        :param W: ``[batch, weight_numel]`` (``shared_weights=False``) or ``[weight_numel]``, kernel order.
        :return: ``[batch, irreps_out.dim]``.
        """
        return torch.ops.libtorch_tp_jit.jit_tp_forward(self.kernel, self.hash, x, y, W, self.L3_dim)

    # -- NumPy harness hooks (weights arrive in e3nn order, as in the reference's correctness suite) ---------
    def forward_cpu(self, L1_in, L2_in, L3_out, weights) -> None:
        w = self.reorder_weights_from_e3nn(weights, not self.config.shared_weights)
        out = self.forward(torch.tensor(L1_in, device="cuda"), torch.tensor(L2_in, device="cuda"),
                           torch.tensor(w, device="cuda"))
        L3_out[:] = out.numpy(force=True)

    def backward_cpu(self, L1_in, L1_grad, L2_in, L2_grad, L3_grad, weights, weights_grad) -> None:
        w = self.reorder_weights_from_e3nn(weights, not self.config.shared_weights)
        x = torch.tensor(L1_in, requires_grad=True, device="cuda")
        y = torch.tensor(L2_in, requires_grad=True, device="cuda")
        wt = torch.tensor(w, requires_grad=True, device="cuda")
        self.forward(x, y, wt).backward(gradient=torch.tensor(L3_grad, device="cuda"))
        L1_grad[:] = x.grad.numpy(force=True)
        L2_grad[:] = y.grad.numpy(force=True)
        weights_grad[:] = self.reorder_weights_to_e3nn(wt.grad.numpy(force=True), not self.config.shared_weights)

    def _second_order(self, in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad, call, third=None):
        dev = "cuda"
        x = torch.tensor(in1, device=dev, requires_grad=True)
        y = torch.tensor(in2, device=dev, requires_grad=True)
        w = torch.tensor(weights, device=dev, requires_grad=True)
        g = torch.tensor(out_grad, device=dev, requires_grad=True)
        a = torch.tensor(in1_dgrad, device=dev, requires_grad=third is not None)
        b = torch.tensor(in2_dgrad, device=dev, requires_grad=third is not None)
        c = torch.tensor(weights_dgrad, device=dev, requires_grad=third is not None)
        out = call(x, y, w)
        gx, gy, gw = torch.autograd.grad(out, [x, y, w], g, create_graph=True, retain_graph=True)
        second = torch.autograd.grad([gx, gy, gw], [x, y, w, g], [a, b, c], create_graph=third is not None)
        if third is None:
            return tuple(t.detach().cpu().numpy() for t in second)
        cots = [torch.tensor(t, device=dev) for t in third]
        res = torch.autograd.grad(list(second), [x, y, w, g, a, b, c], cots, allow_unused=True)
        return tuple(None if t is None else t.detach().cpu().numpy() for t in res)

    def double_backward_cpu(self, in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad):
        """Kernel-order weights in, ``(in1_grad, in2_grad, weights_grad, out_dgrad)`` out."""
        assert self.torch_op
        return self._second_order(in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad, self.forward)

    def triple_backward_cpu(self, in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad, cotangents):
        """Third order: gradients of ``<cotangents, double_backward outputs>`` w.r.t. all seven inputs."""
        assert self.torch_op
        return self._second_order(in1, in2, out_grad, weights, weights_dgrad, in1_dgrad, in2_dgrad, self.forward,
                                  third=cotangents)
