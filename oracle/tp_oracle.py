"""CPU oracle for the Clebsch-Gordan tensor product and the fused graph convolution.

TEST INFRASTRUCTURE ONLY.  Nothing under ``openequivariance_b200/`` imports this file; it is used by
``tests/``, by ``__graft_entry__.smoke()`` as the checker and by ``bench.py`` for the CPU baseline /
reference arm.  The product path has no CPU fallback.

What it restates.  The reference validates its kernels against third-party e3nn
(``o3.TensorProduct``; call sites openequivariance/openequivariance/_torch/E3NNTensorProduct.py:39-51,69,87
and E3NNConv.py:22-43).  e3nn (unpinned in the reference's pyproject, its spec layer cites e3nn 0.5.3/0.5.4)
is not installed here and cannot be, so this file restates its published algorithm:

* per instruction, with ``C = wigner_3j(l1, l2, l3)`` and ``pw = instruction.path_weight``
  (normalisation rule: openequivariance/openequivariance/core/e3nn_lite.py:518-578),
  ``uvu``:  ``z[b,u,k] += pw * sum_{v,i,j} C[i,j,k] x[b,u,i] y[b,v,j] W[b,u,v]``
  ``uvw``:  ``z[b,w,k] += pw * sum_{u,v,i,j} C[i,j,k] x[b,u,i] y[b,v,j] W[b,u,v,w]``
  (the same contraction the reference's kernels unroll: templates/loop_unroll_tp.cuh:46-96);
* weights flattened instruction by instruction, row-major in ``path_shape`` (e3nn order;
  e3nn_lite.py:594-596, 643-650);
* feature blocks laid out ``[mul][2l+1]`` (``mul_ir``) or ``[2l+1][mul]`` (``ir_mul``);
* convolution: ``Z = scatter_add(TP(X[cols], Y, W), rows)`` (E3NNConv.py:41-43,
  core/ConvolutionBase.py:292-301).

Gradients of every order come from torch autograd on these einsums, which is how the reference's
harness obtains e3nn's (``_torch/NPDoubleBackwardMixin.py:17-137``).

The Wigner-3j tensors come from the product's ``openequivariance_b200.core.wigner.wigner_3j`` (the oracle does not carry a
second construction); that function is pinned entry by entry against the reference's generator (item (1) below), so what this file
adds, and what item (2) pins, is the contraction, the normalisation and the weight layout.

Pinning status: PINNED.  (1) The Wigner-3j tensors, path weights, instruction tables and e3nn->kernel weight
permutations are pinned entry-by-entry against the reference's own generator (tests/golden/wigner_3j.npz,
problems.json, coord_graph.json; made by tests/golden/make_golden.py).  (2) The contraction itself -- forward and
backward of five tensor-product problems (uvu / uvw, unshared / shared weights, two with a non-trivial weight
re-tiling) and of an atomic and a deterministic convolution -- is pinned against outputs of the unmodified reference
run on a B200 through its own JIT CUDA kernels (tests/golden/reference_gpu.npz, made by
tests/golden/make_reference_gpu_golden.py; checked in tests/test_reference_gpu_golden.py to 2e-6 relative L2, the
fp32 rounding of those kernels).  The reference holds no stored golden vectors of its own (its tests call live e3nn,
which is not installable here); O(3)-equivariance and third-order autograd checks complement the pins.
"""

from __future__ import annotations

import numpy as np
import torch

from openequivariance_b200.core.wigner import wigner_3j


def _blocks(problem, t: torch.Tensor, irreps, layout: str):
    """Splits ``t [..., dim]`` into per-block views shaped ``[..., mul, 2l+1]``."""
    out = []
    for sl, (mul, ir) in zip(irreps.slices(), irreps):
        blk = t[..., sl]
        if layout == "ir_mul":
            blk = blk.reshape(*t.shape[:-1], ir.dim, mul).transpose(-1, -2)
        else:
            blk = blk.reshape(*t.shape[:-1], mul, ir.dim)
        out.append(blk)
    return out


def tp_forward(problem, x: torch.Tensor, y: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
    """``o3.TensorProduct.forward`` semantics.  ``W`` is in e3nn order: ``[wn]`` if shared else ``[B, wn]``."""
    dtype = x.dtype
    B = x.shape[0]
    layout = getattr(problem, "layout", "mul_ir")
    xb = _blocks(problem, x, problem.irreps_in1, layout)
    yb = _blocks(problem, y, problem.irreps_in2, layout)
    outs = [None] * len(problem.irreps_out)
    offset = 0
    for ins in problem.instructions:
        mul1, ir1 = problem.irreps_in1[ins.i_in1]
        mul2, ir2 = problem.irreps_in2[ins.i_in2]
        mulo, iro = problem.irreps_out[ins.i_out]
        C = torch.as_tensor(wigner_3j(ir1.l, ir2.l, iro.l), dtype=dtype)
        n = int(np.prod(ins.path_shape))
        w = W[..., offset:offset + n].reshape(*W.shape[:-1], *ins.path_shape)
        offset += n
        a, b = xb[ins.i_in1], yb[ins.i_in2]
        if ins.connection_mode == "uvu":
            if problem.shared_weights:
                r = torch.einsum("ijk,bui,bvj,uv->buk", C, a, b, w)
            else:
                r = torch.einsum("ijk,bui,bvj,buv->buk", C, a, b, w)
        elif ins.connection_mode == "uvw":
            if problem.shared_weights:
                r = torch.einsum("ijk,bui,bvj,uvw->bwk", C, a, b, w)
            else:
                r = torch.einsum("ijk,bui,bvj,buvw->bwk", C, a, b, w)
        else:
            raise NotImplementedError(ins.connection_mode)
        r = r * ins.path_weight
        outs[ins.i_out] = r if outs[ins.i_out] is None else outs[ins.i_out] + r
    flat = []
    for o, (mul, ir) in enumerate(problem.irreps_out):
        blk = outs[o] if outs[o] is not None else torch.zeros(B, mul, ir.dim, dtype=dtype)
        if layout == "ir_mul":
            blk = blk.transpose(-1, -2)
        flat.append(blk.reshape(B, mul * ir.dim))
    return torch.cat(flat, dim=1)


def conv_forward(problem, X, Y, W, rows, cols) -> torch.Tensor:
    """``Z[n] = sum_{e: rows[e]==n} TP(X[cols[e]], Y[e], W[e])`` with ``Z`` of ``X.shape[0]`` rows."""
    messages = tp_forward(problem, X[cols], Y, W)
    Z = torch.zeros(X.shape[0], messages.shape[1], dtype=messages.dtype)
    return Z.index_add(0, rows, messages)


# ---- numpy-in / numpy-out drivers in the shape of the reference's correctness harness ----------------------

def _t(a, dtype, grad=False):
    return torch.tensor(np.asarray(a), dtype=dtype, requires_grad=grad)


def _apply(problem, x, y, W, graph):
    if graph is None:
        return tp_forward(problem, x, y, W)
    return conv_forward(problem, x, y, W, graph[0], graph[1])


def forward(problem, x, y, W, graph=None, dtype=torch.float64):
    g = None if graph is None else (torch.as_tensor(graph[0]), torch.as_tensor(graph[1]))
    with torch.no_grad():
        return _apply(problem, _t(x, dtype), _t(y, dtype), _t(W, dtype), g).numpy()


def backward(problem, x, y, W, out_grad, graph=None, dtype=torch.float64):
    """Returns ``(dx, dy, dW)`` for the cotangent ``out_grad``."""
    g = None if graph is None else (torch.as_tensor(graph[0]), torch.as_tensor(graph[1]))
    xt, yt, wt = _t(x, dtype, True), _t(y, dtype, True), _t(W, dtype, True)
    out = _apply(problem, xt, yt, wt, g)
    out.backward(_t(out_grad, dtype))
    return xt.grad.numpy(), yt.grad.numpy(), wt.grad.numpy()


def double_backward(problem, x, y, W, out_grad, x_dgrad, y_dgrad, W_dgrad, graph=None, dtype=torch.float64):
    """Second-order pullback: with ``(gx, gy, gW) = vjp(out_grad)``, returns the gradients of
    ``<gx, x_dgrad> + <gy, y_dgrad> + <gW, W_dgrad>`` w.r.t. ``(x, y, W, out_grad)``."""
    g = None if graph is None else (torch.as_tensor(graph[0]), torch.as_tensor(graph[1]))
    xt, yt, wt = _t(x, dtype, True), _t(y, dtype, True), _t(W, dtype, True)
    gt = _t(out_grad, dtype, True)
    out = _apply(problem, xt, yt, wt, g)
    gx, gy, gw = torch.autograd.grad(out, [xt, yt, wt], gt, create_graph=True, retain_graph=True)
    res = torch.autograd.grad([gx, gy, gw], [xt, yt, wt, gt],
                              [_t(x_dgrad, dtype), _t(y_dgrad, dtype), _t(W_dgrad, dtype)])
    return tuple(r.numpy() for r in res)
