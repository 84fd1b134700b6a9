"""GPU parity of the batched tensor product against the fp64 CPU oracle: forward, backward, double and triple
backward, in the shape of the reference's tests/batch_test.py (batch sizes :66,79,94,113; thresholds :30-36)."""
import numpy as np
import pytest
import torch

from helpers import ABS_LINF, REL_L2, rel_l2, tp_problem_matrix, uniform_inputs, with_dtype
from oracle import tp_oracle

pytestmark = pytest.mark.gpu

MATRIX = tp_problem_matrix()
IDS = [t[0] for t in MATRIX]
FP64_TOO = {"readme", "uvu_m33v3", "uvu_l431", "uvw_m40", "uvw_l431", "uvu_shared", "uvw_shared",
            "uvu_ir_mul", "multi_out", "nequip_like", "mace_medium"}


def _cases():
    for name, p in MATRIX:
        yield pytest.param(name, p, np.float32, id=f"{name}-f32")
        if name in FP64_TOO:
            yield pytest.param(name, p, np.float64, id=f"{name}-f64")


def _module(problem):
    import openequivariance_b200 as oeq
    return oeq.TensorProduct(problem)


def _batch(name, default):
    return {"mace_like": 96, "mace_medium": 96, "nequip_like": 128, "diffdock1": 64, "tetris_poly2": 64}.get(name, default)


@pytest.mark.parametrize("name,problem,dt", list(_cases()))
def test_tp_forward(name, problem, dt):
    p = with_dtype(problem, dt)
    tp = _module(p)
    B = _batch(name, 1000)
    x, y, w, *_ = uniform_inputs(p, B)
    want = tp_oracle.forward(p, x, y, w)
    got = np.zeros((B, p.irreps_out.dim), dtype=dt)
    tp.forward_cpu(x, y, got, w)
    assert rel_l2(got, want) <= REL_L2[dt]
    if dt == np.float32:
        assert np.abs(got - want).max() < ABS_LINF["fwd"] * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("name,problem,dt", list(_cases()))
def test_tp_backward(name, problem, dt):
    p = with_dtype(problem, dt)
    tp = _module(p)
    B = _batch(name, 1000)
    x, y, w, g, *_ = uniform_inputs(p, B)
    want = tp_oracle.backward(p, x, y, w, g)
    dx, dy, dw = np.zeros_like(x), np.zeros_like(y), np.zeros_like(w)
    tp.backward_cpu(x, dx, y, dy, g, w, dw)
    for got, ref, what in zip((dx, dy, dw), want, ("dx", "dy", "dW")):
        assert rel_l2(got, ref) <= REL_L2[dt], what


@pytest.mark.parametrize("name,problem,dt", list(_cases()))
def test_tp_double_backward(name, problem, dt):
    p = with_dtype(problem, dt)
    tp = _module(p)
    B = _batch(name, 200)
    x, y, w, g, x2, y2, w2 = uniform_inputs(p, B)
    # harness works in kernel weight order on both sides: reorder what goes to the oracle
    want = tp_oracle.double_backward(p, x, y, tp.reorder_weights_to_e3nn(w), g, x2, y2, tp.reorder_weights_to_e3nn(w2))
    got = tp.double_backward_cpu(x, y, g, w, w2, x2, y2)
    want = (want[0], want[1], tp.reorder_weights_from_e3nn(want[2]), want[3])
    for a, b, what in zip(got, want, ("dx", "dy", "dW", "dg")):
        assert rel_l2(a, b) <= REL_L2[dt], what


@pytest.mark.parametrize("name", ["readme", "uvu_m5", "uvw_m4", "uvu_shared"])
def test_tp_triple_backward(name):
    p = with_dtype(dict(MATRIX)[name], np.float64)
    tp = _module(p)
    B = 4
    x, y, w, g, x2, y2, w2 = uniform_inputs(p, B)
    rng = np.random.default_rng(5)
    cots = [rng.uniform(size=t.shape) for t in (x, y, w, g)]
    got = tp.triple_backward_cpu(x, y, g, w, w2, x2, y2, cots)

    def t(a, grad=True):
        return torch.tensor(a, dtype=torch.float64, requires_grad=grad)

    xt, yt, gt, at, bt = t(x), t(y), t(g), t(x2), t(y2)
    wt, ct = t(tp.reorder_weights_to_e3nn(w)), t(tp.reorder_weights_to_e3nn(w2))
    out = tp_oracle.tp_forward(p, xt, yt, wt)
    gx, gy, gw = torch.autograd.grad(out, [xt, yt, wt], gt, create_graph=True)
    second = torch.autograd.grad([gx, gy, gw], [xt, yt, wt, gt], [at, bt, ct], create_graph=True)
    cots_t = [t(cots[0], False), t(cots[1], False), t(tp.reorder_weights_to_e3nn(cots[2]), False), t(cots[3], False)]
    third = torch.autograd.grad(list(second), [xt, yt, wt, gt, at, bt, ct], cots_t, allow_unused=True)
    for i, (a, b) in enumerate(zip(got, third)):
        b = np.zeros_like(a) if b is None else b.detach().numpy()
        if i in (2, 6):
            b = tp.reorder_weights_from_e3nn(b)
        a = np.zeros_like(b) if a is None else a
        assert rel_l2(a, b) <= 1e-11, i


def test_equivariance_of_oracle_and_kernel():
    """Rotating inputs by Wigner-D matrices built from the same CG machinery rotates the output: guards the basis
    and sign conventions that no golden vector pins."""
    import openequivariance_b200 as oeq
    from openequivariance_b200.core.graph import spherical_harmonics
    p = with_dtype(dict(MATRIX)["mace_medium"], np.float64)
    B = 16
    gen = torch.Generator().manual_seed(1)
    v = torch.randn(B, 3, generator=gen, dtype=torch.float64)
    q, _ = torch.linalg.qr(torch.randn(3, 3, generator=gen, dtype=torch.float64))
    if torch.det(q) < 0:
        q = -q
    y = spherical_harmonics(3, v)
    y_rot = spherical_harmonics(3, v @ q.T)
    # D^l from harmonics: solve Y_l(Rv) = D_l Y_l(v) on a generic set of directions
    probes = torch.randn(64, 3, generator=gen, dtype=torch.float64)
    Yp, Yr = spherical_harmonics(3, probes), spherical_harmonics(3, probes @ q.T)
    D = {}
    for l in range(4):
        sl = slice(l * l, (l + 1) ** 2)
        D[l] = torch.linalg.lstsq(Yp[:, sl], Yr[:, sl]).solution.T
        assert torch.allclose(D[l] @ D[l].T, torch.eye(2 * l + 1, dtype=torch.float64), atol=1e-9)

    def rotate(feat, irreps):
        out = []
        for sl, (mul, ir) in zip(irreps.slices(), irreps):
            blk = feat[:, sl].reshape(B, mul, ir.dim)
            out.append(torch.einsum("ab,nub->nua", D[ir.l], blk).reshape(B, -1))
        return torch.cat(out, 1)

    x = torch.randn(B, p.irreps_in1.dim, generator=gen, dtype=torch.float64)
    w = torch.randn(B, p.weight_numel, generator=gen, dtype=torch.float64)
    z = tp_oracle.tp_forward(p, x, y, w)
    z_rot = tp_oracle.tp_forward(p, rotate(x, p.irreps_in1), y_rot, w)
    assert torch.allclose(z_rot, rotate(z, p.irreps_out), atol=1e-9)
    tp = oeq.TensorProduct(p)
    zk = tp(rotate(x, p.irreps_in1).cuda(), y_rot.cuda(), w.cuda()).cpu()
    assert torch.allclose(zk, rotate(z, p.irreps_out), atol=1e-9)


def test_weight_reorder_nontrivial_case_end_to_end():
    """16x1e (x) 3x1e 'uvu' has a non-identity kernel weight order; e3nn-ordered weights must give oracle results."""
    p = dict(MATRIX)["uvu_m16v5"]
    tp = _module(p)
    assert not np.array_equal(tp._weight_perm, np.arange(p.weight_numel))
    x, y, w, *_ = uniform_inputs(p, 50)
    got = np.zeros((50, p.irreps_out.dim), dtype=np.float32)
    tp.forward_cpu(x, y, got, w)
    assert rel_l2(got, tp_oracle.forward(p, x, y, w)) <= 1e-5


def test_edge_cases_empty_and_single_item():
    p = dict(MATRIX)["uvu_m5"]
    tp = _module(p)
    x = torch.zeros(0, p.irreps_in1.dim, device="cuda")
    y = torch.zeros(0, p.irreps_in2.dim, device="cuda")
    w = torch.zeros(0, p.weight_numel, device="cuda")
    assert tp(x, y, w).shape == (0, p.irreps_out.dim)
    xs, ys, ws, *_ = uniform_inputs(p, 1)
    got = tp(torch.tensor(xs).cuda(), torch.tensor(ys).cuda(), torch.tensor(ws).cuda()).cpu().numpy()
    assert rel_l2(got, tp_oracle.forward(p, xs, ys, tp.reorder_weights_to_e3nn(ws))) <= 1e-5
    # non-contiguous inputs are accepted (made contiguous inside the op)
    xb, yb, wb, *_ = uniform_inputs(p, 33)
    xt = torch.tensor(np.concatenate([xb, xb], 1)).cuda()[:, : p.irreps_in1.dim]
    got = tp(xt, torch.tensor(yb).cuda(), torch.tensor(wb).cuda()).cpu().numpy()
    assert rel_l2(got, tp_oracle.forward(p, xb, yb, tp.reorder_weights_to_e3nn(wb))) <= 1e-5


def test_uvw_tensor_core_forward_is_used_and_matches_general_kernel():
    """The NequIP-like problem is served by the tcgen05 kernel (fast_path == 2); its 3xTF32 result must agree with
    the fp64 oracle to the fp32 tolerance and with the general CUDA-core kernel to rounding, also on a ragged batch."""
    import openequivariance_b200 as oeq
    from openequivariance_b200 import native
    p = dict(MATRIX)["nequip_like"]
    tp = _module(p)
    assert native.query(tp.kernel_string.encode(), tp.hash).fast_path == 2
    for B in (1, 127, 128, 129, 1000):
        x, y, w, *_ = uniform_inputs(p, B, seed=B)
        args = [torch.tensor(a, device="cuda") for a in (x, y, w)]
        before = native.launch_count()
        got = tp(*args).cpu().numpy()
        assert native.launch_count() == before + 1
        native.set_option("no_tc", "1")
        try:
            ref = tp(*args).cpu().numpy()
        finally:
            native.set_option("no_tc", "0")
        assert rel_l2(got, ref) <= 2e-6
        assert rel_l2(got, tp_oracle.forward(p, x, y, tp.reorder_weights_to_e3nn(w))) <= 1e-5


def _l3_uvw_problem():
    """32 channels of l = 0 ... 3 with parities, shared weights: 7-component blocks on the tensor-core path."""
    from openequivariance_b200.core import problems as P
    feats = "32x0e+32x1o+32x2e+32x3o"
    return P.FullyConnectedTPProblem(feats, "1x0e+1x1o+1x2e+1x3o", feats, shared_weights=True, label="uvw-l3",
                                     irrep_dtype=np.float32, weight_dtype=np.float32)


def _mixed_mul_uvw_problem():
    """64-channel inputs into 32-, 64- and 96-channel outputs: the weight blocks are walked in 32 x 32 tiles, and the 22
    groups of the weight-gradient kernel take two launches."""
    from openequivariance_b200.core import problems as P
    return P.FullyConnectedTPProblem("64x0e+64x0o+64x1e+64x1o+64x2e+64x2o", "1x0e+1x1o+1x2e", "32x0e+64x1o+96x2e",
                                     shared_weights=True, label="uvw-mixed", irrep_dtype=np.float32, weight_dtype=np.float32)


def _uvw_tc_problem(which):
    return {"nequip_like": lambda: dict(MATRIX)["nequip_like"], "l3": _l3_uvw_problem, "mixed": _mixed_mul_uvw_problem}[which]()


@pytest.mark.parametrize("which", ["l3", "mixed"])
def test_uvw_tensor_core_forward_on_other_block_shapes(which):
    """7-component blocks and multiplicities above 32 on the tcgen05 forward: against the general kernel and the oracle."""
    from openequivariance_b200 import native
    p = _uvw_tc_problem(which)
    tp = _module(p)
    assert native.query(tp.kernel_string.encode(), tp.hash).fast_path == 2
    for B in (5, 129, 700):
        x, y, w, *_ = uniform_inputs(p, B, seed=B)
        args = [torch.tensor(a, device="cuda") for a in (x, y, w)]
        got = tp(*args).cpu().numpy()
        native.set_option("no_tc", "1")
        try:
            ref = tp(*args).cpu().numpy()
        finally:
            native.set_option("no_tc", "0")
        # the tensor cores accumulate with truncation: the error grows with the length of the sums (64 channels x 5 paths
        # here: ~3e-6 against 1e-7 for the fp32 FMA kernels); the bound that counts is the oracle's
        assert rel_l2(got, ref) <= 5e-6
        assert rel_l2(got, tp_oracle.forward(p, x, y, tp.reorder_weights_to_e3nn(w))) <= 1e-5


@pytest.mark.parametrize("which", ["nequip_like", "l3", "mixed"])
def test_uvw_tensor_core_backward_is_used_and_matches_general_kernel_and_oracle(which):
    """Backward of the shared-weight 'uvw' problems on the tcgen05 kernels (gradient of x: the forward kernel on transposed
    tables; gradient of y: g W^T on the tensor cores folded with x; gradient of W: a GEMM over the batch with ordered
    partial sums): four launches, results equal to the general CUDA-core kernels to rounding and to the fp64 oracle to
    the fp32 tolerance, on ragged batches around the 64- and 128-item tiles; dW is bitwise reproducible."""
    from openequivariance_b200 import native
    p = _uvw_tc_problem(which)
    tp = _module(p)
    assert native.query(tp.kernel_string.encode(), tp.hash).fast_path == 2
    ops = torch.ops.libtorch_tp_jit
    launches = 5 if which == "mixed" else 4          # dx, dy, dW (16 groups per launch), ordered sum
    for B in (1, 63, 65, 129, 1000, 6000):
        x, y, w, g, *_ = uniform_inputs(p, B, seed=B)
        args = [torch.tensor(a, device="cuda") for a in (x, y, w, g)]
        before = native.launch_count()
        got = [t.cpu().numpy() for t in ops.jit_tp_backward(tp.kernel, tp.hash, *args)]
        assert native.launch_count() == before + launches
        again = ops.jit_tp_backward(tp.kernel, tp.hash, *args)
        assert all(np.array_equal(a, b.cpu().numpy()) for a, b in zip(got, again))
        native.set_option("tc_backward", "0")
        try:
            ref = [t.cpu().numpy() for t in ops.jit_tp_backward(tp.kernel, tp.hash, *args)]
        finally:
            native.set_option("tc_backward", "7")
        for a, b, what in zip(got, ref, ("dx", "dy", "dW")):
            assert rel_l2(a, b) <= 6e-6, (B, what)
        if B <= 1000:
            want = tp_oracle.backward(p, x, y, tp.reorder_weights_to_e3nn(w), g)
            want = (want[0], want[1], tp.reorder_weights_from_e3nn(want[2]))
            for a, b, what in zip(got, want, ("dx", "dy", "dW")):
                assert rel_l2(a, b) <= 1e-5, (B, what)
    native.check(native.load().oeqb_check_status(), "status")


@pytest.mark.parametrize("which", ["nequip_like", "mixed"])
def test_uvw_tensor_core_double_backward_matches_general_kernels(which):
    """The second-order pass of the shared-weight 'uvw' problem runs its five terms on the tensor-core kernels (the later
    ones add to their outputs): same results as the general kernels, to rounding."""
    from openequivariance_b200 import native
    p = _uvw_tc_problem(which)
    tp = _module(p)
    ops = torch.ops.libtorch_tp_jit
    for B in (77, 1500):
        x, y, w, g, *_ = uniform_inputs(p, B, seed=B)
        x2, y2, w2, *_ = uniform_inputs(p, B, seed=B + 1)
        args = [torch.tensor(a, device="cuda") for a in (x, y, w, g, x2, y2, w2)]
        got = [t.cpu().numpy() for t in ops.jit_tp_double_backward(tp.kernel, tp.hash, *args)]
        native.set_option("tc_backward", "0")
        try:
            ref = [t.cpu().numpy() for t in ops.jit_tp_double_backward(tp.kernel, tp.hash, *args)]
        finally:
            native.set_option("tc_backward", "7")
        for a, b, what in zip(got, ref, ("dx", "dy", "dW", "dg")):
            assert rel_l2(a, b) <= 5e-6, (B, what)


def _random_uvw_problem(seed):
    """A seeded random shared-weight 'uvw' problem the tensor-core kernels accept: 2-4 input and output blocks with
    multiplicities from {32, 64, 96, 128} and l <= 3, harmonics up to l = 2 or 3; the selection rules leave some blocks
    without any path (those results are zeroed by the host) and give the paths of a block different shapes."""
    from openequivariance_b200.core import problems as P
    rng = np.random.default_rng(seed)

    def blocks(n):
        out = []
        for _ in range(n):
            l = int(rng.integers(0, 4))
            out.append(f"{int(rng.choice([32, 64, 96, 128]))}x{l}{'e' if rng.integers(0, 2) else 'o'}")
        return "+".join(out)
    lmax = int(rng.integers(2, 4))
    harmonics = "+".join(f"1x{l}{'e' if l % 2 == 0 else 'o'}" for l in range(lmax + 1))
    return P.FullyConnectedTPProblem(blocks(int(rng.integers(2, 5))), harmonics, blocks(int(rng.integers(2, 5))),
                                     shared_weights=True, label=f"uvw-random-{seed}", irrep_dtype=np.float32,
                                     weight_dtype=np.float32)


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 9, 10, 11])
def test_uvw_tensor_core_kernels_on_random_problems(seed):
    """Forward, backward and double backward of random tensor-core-eligible problems: tcgen05 kernels against the general
    kernels (rounding) and the forward / backward against the oracle."""
    from openequivariance_b200 import native
    try:
        p = _random_uvw_problem(seed)
    except AssertionError:
        pytest.skip("the random irreps admit no path")
    if len(p.instructions) == 0:
        pytest.skip("the random irreps admit no path")
    tp = _module(p)
    if native.query(tp.kernel_string.encode(), tp.hash).fast_path != 2:
        pytest.skip("not on the tensor-core path")
    ops = torch.ops.libtorch_tp_jit
    B = 131
    x, y, w, g, *_ = uniform_inputs(p, B, seed=seed)
    x2, y2, w2, *_ = uniform_inputs(p, B, seed=seed + 100)
    a = [torch.tensor(t, device="cuda") for t in (x, y, w, g, x2, y2, w2)]

    def run():
        z = ops.jit_tp_forward(tp.kernel, tp.hash, a[0], a[1], a[2], p.irreps_out.dim)
        first = ops.jit_tp_backward(tp.kernel, tp.hash, *a[:4])
        second = ops.jit_tp_double_backward(tp.kernel, tp.hash, *a)
        return [t.cpu().numpy() for t in (z, *first, *second)]
    got = run()
    native.set_option("no_tc", "1")
    try:
        ref = run()
    finally:
        native.set_option("no_tc", "0")
    names = ("z", "dx", "dy", "dW", "ddx", "ddy", "ddW", "ddg")
    for u, v, what in zip(got, ref, names):
        scale = max(float(np.linalg.norm(v)), 1e-30)
        assert float(np.linalg.norm(u - v)) / scale <= 8e-6 or float(np.abs(v).max()) == 0.0 and float(np.abs(u).max()) == 0.0, what
    we = tp.reorder_weights_to_e3nn(w)
    assert rel_l2(got[0], tp_oracle.forward(p, x, y, we)) <= 1e-5
    want = tp_oracle.backward(p, x, y, we, g)
    want = (want[0], want[1], tp.reorder_weights_from_e3nn(want[2]))
    for u, v, what in zip(got[1:4], want, names[1:4]):
        if float(np.abs(v).max()) == 0.0:
            assert float(np.abs(u).max()) == 0.0, what
        else:
            assert rel_l2(u, v) <= 1e-5, what


def test_uvw_tensor_core_weight_gradient_keeps_its_accuracy_on_long_batches():
    """The tensor cores add into their accumulators with truncation, so a sum over the whole batch loses accuracy with its
    length (it reached 1e-5 at 50,000 items and 8e-5 at 400,000 before the accumulators were emptied per tile).  The weight
    gradient of a 200,000-item batch must stay as accurate as that of a short one: against this library's fp64 kernels."""
    from openequivariance_b200.core import problems as P
    p32, p64 = P.nequip_like_problem(), P.nequip_like_problem(np.float64)
    tp32, tp64 = _module(p32), _module(p64)
    ops = torch.ops.libtorch_tp_jit
    gen = torch.Generator(device="cuda").manual_seed(0)
    B = 200000
    x, y, g = (torch.randn(B, n, device="cuda", generator=gen) for n in (576, 9, 576))
    w = torch.randn(p32.weight_numel, device="cuda", generator=gen) / 12.6
    want = ops.jit_tp_backward(tp64.kernel, tp64.hash, x.double(), y.double(), w.double(), g.double())
    got = ops.jit_tp_backward(tp32.kernel, tp32.hash, x, y, w, g)
    for a, b, what in zip(got, want, ("dx", "dy", "dW")):
        err = float((a.double() - b).norm() / b.norm())
        assert err <= 4e-6, (what, err)
