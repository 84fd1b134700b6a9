"""The batched tensor-product configurations at their full benchmark sizes (MACE-like uvu, 200,000 items; NequIP-like uvw,
50,000 items), where the fp64 oracle is too slow to run over the whole batch: the specialised kernels against the general
kernels over every item, the oracle on a slice of items, and linearity of the product in its first argument."""
import pytest
import torch

from helpers import rel_l2
from oracle import tp_oracle

pytestmark = pytest.mark.gpu


def _inputs(problem, B, lmax, seed):
    from openequivariance_b200.core.graph import spherical_harmonics
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(seed)
    x = torch.randn(B, problem.irreps_in1.dim, device=dev, generator=gen)
    v = torch.randn(B, 3, device=dev, generator=gen, dtype=torch.float64)
    y = spherical_harmonics(lmax, v).float().contiguous()
    if problem.shared_weights:
        w = torch.randn(problem.weight_numel, device=dev, generator=gen) / 12.6
    else:
        w = torch.randn(B, problem.weight_numel, device=dev, generator=gen)
    g = torch.randn(B, problem.irreps_out.dim, device=dev, generator=gen)
    return x, y, w, g


@pytest.mark.parametrize("which,B,lmax,option,tol", [("mace_like", 200000, 3, "force_generic", 2e-6),
                                                     ("nequip_like", 50000, 2, "no_tc", 6e-6)])
def test_full_size_batches(which, B, lmax, option, tol):
    import openequivariance_b200 as oeq
    from openequivariance_b200 import native
    from openequivariance_b200.core import problems as P
    problem = P.mace_like_problem() if which == "mace_like" else P.nequip_like_problem()
    tp = oeq.TensorProduct(problem)
    assert native.query(tp.kernel_string.encode(), tp.hash).fast_path in (1, 2)
    ops = torch.ops.libtorch_tp_jit
    x, y, w, g = _inputs(problem, B, lmax, 0)

    def run(xx):
        z = ops.jit_tp_forward(tp.kernel, tp.hash, xx, y, w, problem.irreps_out.dim)
        return (z, *ops.jit_tp_backward(tp.kernel, tp.hash, xx, y, w, g))
    fast = run(x)
    native.set_option(option, "1")
    if which == "nequip_like":
        native.set_option("tc_backward", "0")
    try:
        general = run(x)
    finally:
        native.set_option(option, "0")
        native.set_option("tc_backward", "7")
    for a, b, what in zip(fast, general, ("z", "dx", "dy", "dW")):
        err = float((a.double() - b.double()).norm() / b.double().norm())
        assert err <= tol, (what, err)
    del general
    # the oracle on a slice of items (per-item outputs), and linearity in x over the whole batch
    sl = slice(B // 2, B // 2 + 64)
    wn = w.cpu().numpy() if problem.shared_weights else w[sl].cpu().numpy()
    want = tp_oracle.forward(problem, x[sl].cpu().numpy(), y[sl].cpu().numpy(), tp.reorder_weights_to_e3nn(wn))
    assert rel_l2(fast[0][sl].cpu().numpy(), want) <= 1e-5
    x2 = torch.randn_like(x)
    z12 = ops.jit_tp_forward(tp.kernel, tp.hash, x + x2, y, w, problem.irreps_out.dim)
    z2 = ops.jit_tp_forward(tp.kernel, tp.hash, x2, y, w, problem.irreps_out.dim)
    err = float((z12.double() - fast[0].double() - z2.double()).norm() / z12.double().norm())
    assert err <= 1e-5, err
