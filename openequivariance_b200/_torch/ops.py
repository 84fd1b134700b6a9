"""torch operator layer: the six ``libtorch_tp_jit::jit_*`` ops, with the reference's schemas.

Counterpart of openequivariance/openequivariance/extension/torch_core.hpp:274-644 (op bodies, tensor checks,
output allocation, schemas) and of the fake / autograd / autocast registrations in
openequivariance/openequivariance/_torch/TensorProduct.py:182-374 and TensorProductConv.py:280-568.
Each op validates its tensors (same ``RuntimeError`` texts as ``check_tensor``, torch_core.hpp:109-134),
allocates the outputs with the inputs' options, and calls the C ABI of ``liboeq_b200.so`` on the current
CUDA stream with raw device pointers.  ``json_bytes`` carries the problem descriptor (CPU uint8 tensor),
``hash`` the cache key, as in the reference; exported graphs therefore stay self-contained.
"""

from __future__ import annotations

import ctypes

import torch

from .. import native

NS = "libtorch_tp_jit"

_SCHEMAS = {
    "jit_tp_forward": "(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, int L3_dim) -> Tensor",
    "jit_tp_backward": "(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, Tensor L3_grad)"
                       " -> (Tensor, Tensor, Tensor)",
    "jit_tp_double_backward": "(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, Tensor L3_grad,"
                              " Tensor L1_dgrad, Tensor L2_dgrad, Tensor W_dgrad) -> (Tensor, Tensor, Tensor, Tensor)",
    "jit_conv_forward": "(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, int L3_dim, Tensor rows,"
                        " Tensor cols, Tensor workspace, Tensor transpose_perm) -> Tensor",
    "jit_conv_backward": "(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, Tensor L3_grad,"
                         " Tensor rows, Tensor cols, Tensor workspace, Tensor transpose_perm)"
                         " -> (Tensor, Tensor, Tensor)",
    "jit_conv_double_backward": "(Tensor json_bytes, int hash, Tensor L1_in, Tensor L2_in, Tensor W, Tensor L3_grad,"
                                " Tensor L1_dgrad, Tensor L2_dgrad, Tensor W_dgrad, Tensor rows, Tensor cols,"
                                " Tensor workspace, Tensor transpose_perm) -> (Tensor, Tensor, Tensor, Tensor)",
}



def _load_cpp_ops() -> bool:
    """Loads ``csrc/liboeq_b200_torch.so`` (the operators registered from C++: ``csrc/torch_ops.cpp``) when it has been
    built from the current sources.  ``OEQB_PYTHON_OPS=1`` keeps the Python implementation below instead."""
    import os

    from .. import build_native
    if os.environ.get("OEQB_PYTHON_OPS") == "1" or not os.path.exists(build_native.TORCH_LIB):
        return False
    try:
        if build_native.torch_ops_need_build():
            return False
        native.load()                       # the operator library links liboeq_b200.so: have it mapped first
        torch.ops.load_library(build_native.TORCH_LIB)
        return True
    except Exception as exc:  # noqa: BLE001 - the Python implementation below serves instead
        import sys
        print(f"[oeq_b200] operator library not loaded ({exc}); using the Python operator layer", file=sys.stderr)
        return False


CPP_OPS = _load_cpp_ops()
if not CPP_OPS:
    _lib_def = torch.library.Library(NS, "DEF")
    for _name, _schema in _SCHEMAS.items():
        _lib_def.define(_name + _schema)
    _lib_impl = torch.library.Library(NS, "IMPL", "CUDA")

_ENUM_TO_TORCH = {1: torch.float32, 2: torch.float64, 3: torch.int32, 4: torch.int64, 5: torch.uint8}
_TORCH_TO_ENUM = {v: k for k, v in _ENUM_TO_TORCH.items()}

# key -> (descriptor bytes, KernelProp); filled on first sight of a key so the tensor->bytes copy happens once
_PROBLEMS = {}


def _problem(json_bytes: torch.Tensor, key: int):
    hit = _PROBLEMS.get(key)
    if hit is None:
        desc = bytes(json_bytes.detach().cpu().contiguous().numpy().tobytes())
        hit = (desc, native.query(desc, key))
        _PROBLEMS[key] = hit
    return hit


def _check(t: torch.Tensor, shape, dtype, name: str):
    if t.dim() != len(shape) or any(int(t.shape[i]) != int(s) for i, s in enumerate(shape)):
        raise RuntimeError(f"Shape mismatch for tensor '{name}'. Expected: {list(shape)}. Got: {list(t.shape)}")
    if not t.is_cuda:
        raise RuntimeError(f"Tensor '{name}' is not on the GPU.")
    if t.dtype != dtype:
        raise RuntimeError(f"Dtype mismatch for tensor '{name}'. Expected: {_TORCH_TO_ENUM.get(dtype, dtype)}. "
                           f"Got: {_TORCH_TO_ENUM.get(t.dtype, t.dtype)}")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() > 0 else ctypes.c_void_p(0)


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _on_device:
    """Makes ``t``'s device current for the duration of a C-ABI call (cheap no-op when it already is)."""

    def __init__(self, t):
        self.want = t.device.index
        self.guard = None

    def __enter__(self):
        if self.want is not None and self.want != torch.cuda.current_device():
            self.guard = torch.cuda.device(self.want)
            self.guard.__enter__()

    def __exit__(self, *exc):
        if self.guard is not None:
            self.guard.__exit__(*exc)


def _first_dim(t, name):
    if t.dim() < 1:
        raise RuntimeError(f"Shape mismatch for tensor '{name}'. Expected a leading batch dimension. Got: {list(t.shape)}")
    return int(t.shape[0])


def _tp_checks(prop, L1_in, L2_in, W):
    dt = _ENUM_TO_TORCH[prop.irrep_dtype]
    B = _first_dim(L1_in, "L1_in")
    _check(L1_in, (B, prop.L1_dim), dt, "L1_in")
    _check(L2_in, (B, prop.L2_dim), dt, "L2_in")
    wshape = (prop.weight_numel,) if prop.shared_weights else (B, prop.weight_numel)
    _check(W, wshape, _ENUM_TO_TORCH[prop.weight_dtype], "W")
    return B, dt


def jit_tp_forward(json_bytes, hash, L1_in, L2_in, W, L3_dim):
    desc, prop = _problem(json_bytes, hash)
    B, _ = _tp_checks(prop, L1_in, L2_in, W)
    x, y, w = L1_in.contiguous(), L2_in.contiguous(), W.contiguous()
    out = torch.empty((B, prop.L3_dim), dtype=x.dtype, device=x.device)
    with _on_device(x):
        rc = native.load().oeqb_tp_forward(desc, len(desc), hash, B, _ptr(x), _ptr(y), _ptr(w), _ptr(out), _stream())
    native.check(rc, "jit_tp_forward")
    return out


def jit_tp_backward(json_bytes, hash, L1_in, L2_in, W, L3_grad):
    desc, prop = _problem(json_bytes, hash)
    B, dt = _tp_checks(prop, L1_in, L2_in, W)
    _check(L3_grad, (B, prop.L3_dim), dt, "L3_grad")
    x, y, w, g = L1_in.contiguous(), L2_in.contiguous(), W.contiguous(), L3_grad.contiguous()
    dx, dy, dw = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)
    with _on_device(x):
        rc = native.load().oeqb_tp_backward(desc, len(desc), hash, B, _ptr(x), _ptr(y), _ptr(w), _ptr(g),
                                            _ptr(dx), _ptr(dy), _ptr(dw), _stream())
    native.check(rc, "jit_tp_backward")
    return dx, dy, dw


def jit_tp_double_backward(json_bytes, hash, L1_in, L2_in, W, L3_grad, L1_dgrad, L2_dgrad, W_dgrad):
    desc, prop = _problem(json_bytes, hash)
    B, dt = _tp_checks(prop, L1_in, L2_in, W)
    _check(L3_grad, (B, prop.L3_dim), dt, "L3_grad")
    _check(L1_dgrad, (B, prop.L1_dim), dt, "L1_dgrad")
    _check(L2_dgrad, (B, prop.L2_dim), dt, "L2_dgrad")
    _check(W_dgrad, tuple(W.shape), W.dtype, "W_dgrad")
    x, y, w, g = L1_in.contiguous(), L2_in.contiguous(), W.contiguous(), L3_grad.contiguous()
    x2, y2, w2 = L1_dgrad.contiguous(), L2_dgrad.contiguous(), W_dgrad.contiguous()
    dx, dy, dw, dg = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w), torch.empty_like(g)
    with _on_device(x):
        rc = native.load().oeqb_tp_double_backward(desc, len(desc), hash, B, _ptr(x), _ptr(y), _ptr(w), _ptr(g),
                                                   _ptr(x2), _ptr(y2), _ptr(w2), _ptr(dx), _ptr(dy), _ptr(dw),
                                                   _ptr(dg), _stream())
    native.check(rc, "jit_tp_double_backward")
    return dx, dy, dw, dg


# ---- convolution ------------------------------------------------------------------------------------------

def _conv_checks(prop, L1_in, L2_in, W, rows, cols, workspace, perm):
    dt = _ENUM_TO_TORCH[prop.irrep_dtype]
    it = _ENUM_TO_TORCH[prop.idx_dtype]
    N = _first_dim(L1_in, "L1_in")
    E = _first_dim(rows, "rows")
    _check(L1_in, (N, prop.L1_dim), dt, "L1_in")
    _check(L2_in, (E, prop.L2_dim), dt, "L2_in")
    wshape = (prop.weight_numel,) if prop.shared_weights else (E, prop.weight_numel)
    _check(W, wshape, _ENUM_TO_TORCH[prop.weight_dtype], "W")
    _check(rows, (E,), it, "rows")
    _check(cols, (E,), it, "cols")
    if prop.deterministic:
        _check(perm, (E,), it, "transpose_perm")
    _check(workspace, tuple(workspace.shape) if workspace.dim() == 1 else (-1,), torch.uint8, "workspace")
    return N, E, dt


def _scratch(desc, key, direction, N, E, workspace):
    """Returns a uint8 CUDA tensor at least as large as the call needs: the caller's when big enough."""
    need = native.load().oeqb_conv_workspace_bytes(desc, len(desc), key, direction, N, E)
    if need < 0:
        native.check(int(-need), "oeqb_conv_workspace_bytes")
    if workspace.numel() >= need:
        return workspace, int(workspace.numel())
    fresh = torch.empty(int(need), dtype=torch.uint8, device=workspace.device)
    return fresh, int(need)


def jit_conv_forward(json_bytes, hash, L1_in, L2_in, W, L3_dim, rows, cols, workspace, transpose_perm):
    desc, prop = _problem(json_bytes, hash)
    N, E, _ = _conv_checks(prop, L1_in, L2_in, W, rows, cols, workspace, transpose_perm)
    x, y, w = L1_in.contiguous(), L2_in.contiguous(), W.contiguous()
    r, c, p = rows.contiguous(), cols.contiguous(), transpose_perm.contiguous()
    out = torch.empty((N, prop.L3_dim), dtype=x.dtype, device=x.device)
    with _on_device(x):
        ws, nbytes = _scratch(desc, hash, 0, N, E, workspace)
        rc = native.load().oeqb_conv_forward(desc, len(desc), hash, N, E, _ptr(x), _ptr(y), _ptr(w), _ptr(out),
                                             _ptr(r), _ptr(c), _ptr(p) if prop.deterministic else None,
                                             _ptr(ws), nbytes, _stream())
    native.check(rc, "jit_conv_forward")
    return out


def jit_conv_backward(json_bytes, hash, L1_in, L2_in, W, L3_grad, rows, cols, workspace, transpose_perm):
    desc, prop = _problem(json_bytes, hash)
    N, E, dt = _conv_checks(prop, L1_in, L2_in, W, rows, cols, workspace, transpose_perm)
    _check(L3_grad, (N, prop.L3_dim), dt, "L3_grad")
    x, y, w, g = L1_in.contiguous(), L2_in.contiguous(), W.contiguous(), L3_grad.contiguous()
    r, c, p = rows.contiguous(), cols.contiguous(), transpose_perm.contiguous()
    dx, dy, dw = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w)
    with _on_device(x):
        ws, nbytes = _scratch(desc, hash, 1, N, E, workspace)
        rc = native.load().oeqb_conv_backward(desc, len(desc), hash, N, E, _ptr(x), _ptr(y), _ptr(w), _ptr(g),
                                              _ptr(dx), _ptr(dy), _ptr(dw), _ptr(r), _ptr(c),
                                              _ptr(p) if prop.deterministic else None, _ptr(ws), nbytes, _stream())
    native.check(rc, "jit_conv_backward")
    return dx, dy, dw


def jit_conv_double_backward(json_bytes, hash, L1_in, L2_in, W, L3_grad, L1_dgrad, L2_dgrad, W_dgrad, rows, cols,
                             workspace, transpose_perm):
    desc, prop = _problem(json_bytes, hash)
    N, E, dt = _conv_checks(prop, L1_in, L2_in, W, rows, cols, workspace, transpose_perm)
    _check(L3_grad, (N, prop.L3_dim), dt, "L3_grad")
    _check(L1_dgrad, (N, prop.L1_dim), dt, "L1_dgrad")
    _check(L2_dgrad, (E, prop.L2_dim), dt, "L2_dgrad")
    _check(W_dgrad, tuple(W.shape), W.dtype, "W_dgrad")
    x, y, w, g = L1_in.contiguous(), L2_in.contiguous(), W.contiguous(), L3_grad.contiguous()
    x2, y2, w2 = L1_dgrad.contiguous(), L2_dgrad.contiguous(), W_dgrad.contiguous()
    r, c, p = rows.contiguous(), cols.contiguous(), transpose_perm.contiguous()
    dx, dy, dw, dg = torch.empty_like(x), torch.empty_like(y), torch.empty_like(w), torch.empty_like(g)
    with _on_device(x):
        ws, nbytes = _scratch(desc, hash, 2, N, E, workspace)
        rc = native.load().oeqb_conv_double_backward(
            desc, len(desc), hash, N, E, _ptr(x), _ptr(y), _ptr(w), _ptr(g), _ptr(x2), _ptr(y2), _ptr(w2),
            _ptr(dx), _ptr(dy), _ptr(dw), _ptr(dg), _ptr(r), _ptr(c), _ptr(p) if prop.deterministic else None,
            _ptr(ws), nbytes, _stream())
    native.check(rc, "jit_conv_double_backward")
    return dx, dy, dw, dg


if not CPP_OPS:
    for _name, _fn in (("jit_tp_forward", jit_tp_forward), ("jit_tp_backward", jit_tp_backward),
                       ("jit_tp_double_backward", jit_tp_double_backward), ("jit_conv_forward", jit_conv_forward),
                       ("jit_conv_backward", jit_conv_backward), ("jit_conv_double_backward", jit_conv_double_backward)):
        _lib_impl.impl(_name, _fn)


# ---- fake (meta) kernels ----------------------------------------------------------------------------------

@torch.library.register_fake(f"{NS}::jit_tp_forward")
def _(json_bytes, hash, L1_in, L2_in, W, L3_dim):
    return L1_in.new_empty(L1_in.shape[0], L3_dim)


@torch.library.register_fake(f"{NS}::jit_tp_backward")
def _(json_bytes, hash, L1_in, L2_in, W, L3_grad):
    return torch.empty_like(L1_in), torch.empty_like(L2_in), torch.empty_like(W)


@torch.library.register_fake(f"{NS}::jit_tp_double_backward")
def _(json_bytes, hash, L1_in, L2_in, W, L3_grad, L1_dgrad, L2_dgrad, W_dgrad):
    return torch.empty_like(L1_in), torch.empty_like(L2_in), torch.empty_like(W), torch.empty_like(L3_grad)


@torch.library.register_fake(f"{NS}::jit_conv_forward")
def _(json_bytes, hash, L1_in, L2_in, W, L3_dim, rows, cols, workspace, transpose_perm):
    return L1_in.new_empty(L1_in.shape[0], L3_dim)


@torch.library.register_fake(f"{NS}::jit_conv_backward")
def _(json_bytes, hash, L1_in, L2_in, W, L3_grad, rows, cols, workspace, transpose_perm):
    return torch.empty_like(L1_in), torch.empty_like(L2_in), torch.empty_like(W)


@torch.library.register_fake(f"{NS}::jit_conv_double_backward")
def _(json_bytes, hash, L1_in, L2_in, W, L3_grad, L1_dgrad, L2_dgrad, W_dgrad, rows, cols, workspace, transpose_perm):
    return torch.empty_like(L1_in), torch.empty_like(L2_in), torch.empty_like(W), torch.empty_like(L3_grad)


# ---- autograd chain: forward -> backward -> double backward -> (third order, composed) ---------------------
#
# With Q(g; x, y, W) = <g, F(x, y, W)> (F trilinear) the three ops are
#   backward(x, y, W, g)            = (dQ/dx, dQ/dy, dQ/dW)
#   double_backward(x, y, W, g; a, b, c) = gradients of  <a, dQ/dx> + <b, dQ/dy> + <c, dQ/dW>  w.r.t. (x, y, W, g)
# The third order is obtained by rebuilding that scalar from differentiable forward calls and letting autograd
# differentiate it with the ops above, so any higher order keeps working.

def _ops():
    return torch.ops.libtorch_tp_jit


def _register_tp_autograd():
    def fwd_setup(ctx, inputs, output):
        ctx.kernel, ctx.hash, ctx.L1_in, ctx.L2_in, ctx.W, ctx.L3_dim = inputs

    def fwd_backward(ctx, grad_out):
        dx, dy, dw = _ops().jit_tp_backward(ctx.kernel, ctx.hash, ctx.L1_in, ctx.L2_in, ctx.W, grad_out)
        return None, None, dx, dy, dw, None

    torch.library.register_autograd(f"{NS}::jit_tp_forward", fwd_backward, setup_context=fwd_setup)

    def bwd_setup(ctx, inputs, output):
        ctx.kernel, ctx.hash, ctx.L1_in, ctx.L2_in, ctx.W, ctx.L3_grad = inputs

    def bwd_backward(ctx, a, b, c):
        a = torch.zeros_like(ctx.L1_in) if a is None else a
        b = torch.zeros_like(ctx.L2_in) if b is None else b
        c = torch.zeros_like(ctx.W) if c is None else c
        dx, dy, dw, dg = _ops().jit_tp_double_backward(ctx.kernel, ctx.hash, ctx.L1_in, ctx.L2_in, ctx.W,
                                                       ctx.L3_grad, a, b, c)
        return None, None, dx, dy, dw, dg

    torch.library.register_autograd(f"{NS}::jit_tp_backward", bwd_backward, setup_context=bwd_setup)

    def dbl_setup(ctx, inputs, output):
        ctx.kernel, ctx.hash = inputs[0], inputs[1]
        ctx.saved = inputs[2:9]

    def dbl_backward(ctx, t_dx, t_dy, t_dw, t_dg):
        fwd = lambda x, y, w: _ops().jit_tp_forward(ctx.kernel, ctx.hash, x, y, w, int(ctx.saved[3].shape[1]))  # noqa: E731
        return (None, None) + _third_order(fwd, ctx.saved, (t_dx, t_dy, t_dw, t_dg))

    torch.library.register_autograd(f"{NS}::jit_tp_double_backward", dbl_backward, setup_context=dbl_setup)


def _third_order(fwd, saved, cotangents):
    """Gradients of ``<t_dx,dx>+<t_dy,dy>+<t_dw,dw>+<t_dg,dg>`` w.r.t. the seven tensor inputs of a
    double-backward op, where ``fwd(x, y, w)`` is the (differentiable) forward op of the same problem."""
    x, y, w, g, a, b, c = saved
    t_dx, t_dy, t_dw, t_dg = cotangents
    keep = torch.is_grad_enabled()
    with torch.enable_grad():
        leaves = [t.detach().requires_grad_(True) for t in (x, y, w, g, a, b, c)]
        x_, y_, w_, g_, a_, b_, c_ = leaves
        total = None

        def add(term):
            nonlocal total
            total = term if total is None else total + term

        # <t, Bx(y', W', g)> = <g, F(t, y', W')> and likewise for the other two adjoints
        if t_dx is not None:
            add((g_ * (fwd(t_dx, b_, w_) + fwd(t_dx, y_, c_))).sum())
        if t_dy is not None:
            add((g_ * (fwd(a_, t_dy, w_) + fwd(x_, t_dy, c_))).sum())
        if t_dw is not None:
            add((g_ * (fwd(a_, y_, t_dw) + fwd(x_, b_, t_dw))).sum())
        if t_dg is not None:
            add((t_dg * (fwd(a_, y_, w_) + fwd(x_, b_, w_) + fwd(x_, y_, c_))).sum())
        if total is None:
            return tuple(None for _ in leaves)
        grads = torch.autograd.grad(total, leaves, create_graph=keep, allow_unused=True)
    return tuple(grads)


def _register_conv_autograd():
    def fwd_setup(ctx, inputs, output):
        (ctx.kernel, ctx.hash, ctx.L1_in, ctx.L2_in, ctx.W, ctx.L3_dim, ctx.rows, ctx.cols, ctx.workspace,
         ctx.perm) = inputs

    def fwd_backward(ctx, grad_out):
        dx, dy, dw = _ops().jit_conv_backward(ctx.kernel, ctx.hash, ctx.L1_in, ctx.L2_in, ctx.W, grad_out,
                                              ctx.rows, ctx.cols, ctx.workspace, ctx.perm)
        return None, None, dx, dy, dw, None, None, None, None, None

    torch.library.register_autograd(f"{NS}::jit_conv_forward", fwd_backward, setup_context=fwd_setup)

    def bwd_setup(ctx, inputs, output):
        (ctx.kernel, ctx.hash, ctx.L1_in, ctx.L2_in, ctx.W, ctx.L3_grad, ctx.rows, ctx.cols, ctx.workspace,
         ctx.perm) = inputs

    def bwd_backward(ctx, a, b, c):
        a = torch.zeros_like(ctx.L1_in) if a is None else a
        b = torch.zeros_like(ctx.L2_in) if b is None else b
        c = torch.zeros_like(ctx.W) if c is None else c
        dx, dy, dw, dg = _ops().jit_conv_double_backward(ctx.kernel, ctx.hash, ctx.L1_in, ctx.L2_in, ctx.W,
                                                         ctx.L3_grad, a, b, c, ctx.rows, ctx.cols, ctx.workspace,
                                                         ctx.perm)
        return None, None, dx, dy, dw, dg, None, None, None, None

    torch.library.register_autograd(f"{NS}::jit_conv_backward", bwd_backward, setup_context=bwd_setup)

    def dbl_setup(ctx, inputs, output):
        ctx.kernel, ctx.hash = inputs[0], inputs[1]
        ctx.saved = inputs[2:9]
        ctx.rows, ctx.cols, ctx.workspace, ctx.perm = inputs[9:13]

    def dbl_backward(ctx, t_dx, t_dy, t_dw, t_dg):
        l3 = int(ctx.saved[3].shape[1])
        fwd = lambda x, y, w: _ops().jit_conv_forward(ctx.kernel, ctx.hash, x, y, w, l3, ctx.rows, ctx.cols,  # noqa: E731
                                                      ctx.workspace, ctx.perm)
        return (None, None) + _third_order(fwd, ctx.saved, (t_dx, t_dy, t_dw, t_dg)) + (None, None, None, None)

    torch.library.register_autograd(f"{NS}::jit_conv_double_backward", dbl_backward, setup_context=dbl_setup)


_register_tp_autograd()
_register_conv_autograd()

for _name in _SCHEMAS:
    torch.library.register_autocast(f"{NS}::{_name}", "cuda", torch.float32)
