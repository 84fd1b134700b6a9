"""The ``ir_mul`` layout both ways, as the reference tests it (tests/batch_test.py:309-380): a module built for ``ir_mul``
directly, and a ``mul_ir`` module wrapped in ``transpose_irreps`` on its inputs and output; forward and gradients agree,
and both agree with the oracle evaluated on the transposed data."""
import pytest
import torch

from helpers import rel_l2, tp_problem_matrix
from oracle import tp_oracle

MATRIX = dict(tp_problem_matrix())


def _problems():
    import openequivariance_b200 as oeq
    out = [MATRIX["mace_medium"].clone()]
    for mul in (5, 13):
        out.append(oeq.TPProblem(f"{mul}x5e", "1x3e", f"{mul}x5e", [(0, 0, 0, "uvu", True)], shared_weights=False,
                                 internal_weights=False, label=f"ir_mul_repr_{mul}x1x{mul}_l535"))
    return out


def test_transpose_irreps_checks_and_roundtrip():
    import openequivariance_b200 as oeq
    irreps = oeq.Irreps("3x1o+2x2e+4x0e")
    x = torch.arange(2 * irreps.dim, dtype=torch.float32).reshape(2, irreps.dim)
    y = oeq.transpose_irreps(x, irreps, "mul_ir", "ir_mul")
    assert y.shape == x.shape and not torch.equal(x, y)
    assert torch.equal(oeq.transpose_irreps(y, irreps, "ir_mul", "mul_ir"), x)
    assert y[0, 1].item() == x[0, 3].item()            # [mul][2l+1] -> [2l+1][mul]: component 0 of channel 1
    same = oeq.transpose_irreps(x, irreps, "mul_ir", "mul_ir")
    assert torch.equal(same, x) and same.data_ptr() != x.data_ptr()
    with pytest.raises(ValueError, match="Unsupported src_layout"):
        oeq.transpose_irreps(x, irreps, "mulir", "ir_mul")
    with pytest.raises(ValueError, match="Unsupported dst_layout"):
        oeq.transpose_irreps(x, irreps, "mul_ir", "irmul")
    with pytest.raises(TypeError):
        oeq.transpose_irreps(x.numpy(), irreps, "mul_ir", "ir_mul")


@pytest.mark.gpu
@pytest.mark.parametrize("index", [0, 1, 2])
def test_ir_mul_native_and_through_the_transpose_wrapper(index):
    import openequivariance_b200 as oeq
    base = _problems()[index]
    native_problem = base.clone()
    native_problem.layout = "ir_mul"
    tp_native = oeq.TensorProduct(native_problem)
    tp_plain = oeq.TensorProduct(base)                   # mul_ir
    B = 257
    gen = torch.Generator(device="cuda").manual_seed(index)
    x = torch.rand(B, base.irreps_in1.dim, device="cuda", generator=gen, requires_grad=True)
    y = torch.rand(B, base.irreps_in2.dim, device="cuda", generator=gen, requires_grad=True)
    w = torch.rand(B, base.weight_numel, device="cuda", generator=gen, requires_grad=True)
    g = torch.rand(B, base.irreps_out.dim, device="cuda", generator=gen)

    def wrapped(x_, y_, w_):   # inputs and output in ir_mul, the module in mul_ir
        z = tp_plain(oeq.transpose_irreps(x_, base.irreps_in1, "ir_mul", "mul_ir"),
                     oeq.transpose_irreps(y_, base.irreps_in2, "ir_mul", "mul_ir"), w_)
        return oeq.transpose_irreps(z, base.irreps_out, "mul_ir", "ir_mul")

    z_native = tp_native(x, y, w)
    grads_native = torch.autograd.grad(z_native, [x, y, w], g)
    z_wrapped = wrapped(x, y, w)
    grads_wrapped = torch.autograd.grad(z_wrapped, [x, y, w], g)
    assert rel_l2(z_native.detach().cpu().numpy(), z_wrapped.detach().cpu().numpy()) <= 2e-6
    for a, b, what in zip(grads_native, grads_wrapped, ("dx", "dy", "dW")):
        assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) <= 2e-6, what
    # and against the oracle, which works in mul_ir
    xm = oeq.transpose_irreps(x.detach(), base.irreps_in1, "ir_mul", "mul_ir").cpu().numpy()
    ym = oeq.transpose_irreps(y.detach(), base.irreps_in2, "ir_mul", "mul_ir").cpu().numpy()
    want = tp_oracle.forward(base, xm, ym, tp_plain.reorder_weights_to_e3nn(w.detach().cpu().numpy()))
    got = oeq.transpose_irreps(z_native.detach(), base.irreps_out, "ir_mul", "mul_ir").cpu().numpy()
    assert rel_l2(got, want) <= 1e-5
