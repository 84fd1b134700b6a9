"""GPU parity of the fused convolution (atomic, deterministic, Kahan) against the oracle's gather + TP + scatter-add
on a seeded synthetic graph (stands in for the reference's downloaded 1drf graph, tests/conv_test.py:30-41)."""
import numpy as np
import pytest
import torch

from helpers import REL_L2, rel_l2, single, small_graph, tp_problem_matrix, uniform_inputs, with_dtype
from oracle import tp_oracle

pytestmark = pytest.mark.gpu

MATRIX = dict(tp_problem_matrix())
CONV_PROBLEMS = ["readme", "uvu_m33v3", "uvu_l431", "uvw_m4", "uvw_m40", "multi_out", "mace_medium", "nequip_water_uvu",
                 "ctpp_ir_mul", "uvu_ir_mul_fast", "mace_like"]
MODES = ["atomic", "deterministic", "kahan"]


class G:
    pass


@pytest.fixture(scope="module")
def graph():
    g = small_graph()
    out = G()
    out.node_count = g["n_nodes"]
    out.rows = g["rows"].numpy().astype(np.int64)
    out.cols = g["cols"].numpy().astype(np.int64)
    out.transpose_perm = g["transpose_perm"].numpy().astype(np.int64)
    out.nnz = len(out.rows)
    return out


def _conv(problem, mode):
    import openequivariance_b200 as oeq
    return oeq.TensorProductConv(problem, deterministic=mode != "atomic", kahan=mode == "kahan")


def _shuffled(graph, seed=0):
    """The atomic variant takes edges in any order: hand it a random one."""
    rng = np.random.default_rng(seed)
    order = rng.permutation(graph.nnz)
    out = G()
    out.node_count, out.nnz = graph.node_count, graph.nnz
    out.rows, out.cols, out.transpose_perm = graph.rows[order], graph.cols[order], graph.transpose_perm
    return out, order


def _cases():
    for name in CONV_PROBLEMS:
        for mode in MODES:
            # MACE-like in fp64 (the accuracy pass of the partitioned configuration): deterministic mode only, to bound run time
            dts = [np.float32] if (mode == "kahan" or (name == "mace_like" and mode != "deterministic")) else [np.float32, np.float64]
            for dt in dts:
                yield pytest.param(name, mode, dt, id=f"{name}-{mode}-{'f32' if dt == np.float32 else 'f64'}")


@pytest.mark.parametrize("name,mode,dt", list(_cases()))
def test_conv_forward_backward(name, mode, dt, graph):
    p = with_dtype(MATRIX[name], dt)
    conv = _conv(p, mode)
    E, N = graph.nnz, graph.node_count
    x, y, w, g, *_ = uniform_inputs(p, E, n_rows=N)
    order = np.arange(E)
    gr = graph
    if mode == "atomic":
        gr, order = _shuffled(graph)
    want = tp_oracle.forward(p, x, y[order], w if p.shared_weights else w[order], graph=(gr.rows, gr.cols))
    got = np.zeros((N, p.irreps_out.dim), dtype=dt)
    conv.forward_cpu(x, y[order], w if p.shared_weights else w[order], got, gr)
    tol = REL_L2[dt]
    assert rel_l2(got, want) <= tol
    wdx, wdy, wdw = tp_oracle.backward(p, x, y[order], w if p.shared_weights else w[order], g, graph=(gr.rows, gr.cols))
    dx, dy, dw = np.zeros_like(x), np.zeros_like(y), np.zeros_like(w)
    conv.backward_cpu(x, dx, y[order], dy, w if p.shared_weights else w[order], dw, g, gr)
    assert rel_l2(dx, wdx) <= tol, "dx"
    assert rel_l2(dy, wdy) <= tol, "dy"
    assert rel_l2(dw, wdw) <= tol, "dW"


@pytest.mark.parametrize("name,mode,dt", [(n, m, d) for n in ["readme", "uvu_m33v3", "uvw_m4", "mace_medium", "nequip_water_uvu"]
                                          for m in MODES[:2] for d in (np.float64, np.float32)
                                          if d == np.float64 or n in ("mace_medium", "nequip_water_uvu")])
def test_conv_double_backward(name, mode, dt, graph):
    p = with_dtype(MATRIX[name], dt)
    conv = _conv(p, mode)
    E, N = graph.nnz, graph.node_count
    x, y, w, g, x2, y2, w2 = uniform_inputs(p, E, n_rows=N)
    to_e3nn = conv.reorder_weights_to_e3nn
    want = tp_oracle.double_backward(p, x, y, to_e3nn(w), g, x2, y2, to_e3nn(w2), graph=(graph.rows, graph.cols))
    got = conv.double_backward_cpu(x, y, g, w, w2, x2, y2, graph)
    want = (want[0], want[1], conv.reorder_weights_from_e3nn(want[2]), want[3])
    tol = 1e-11 if dt == np.float64 else REL_L2[dt]
    for a, b, what in zip(got, want, ("dx", "dy", "dW", "dg")):
        assert rel_l2(a, b) <= tol, what


def test_deterministic_conv_is_bitwise_reproducible(graph):
    p = MATRIX["mace_medium"]
    conv = _conv(p, "deterministic")
    E, N = graph.nnz, graph.node_count
    x, y, w, g, *_ = uniform_inputs(p, E, n_rows=N)
    t = lambda a, grad=False: torch.tensor(a, device="cuda", requires_grad=grad)  # noqa: E731
    rows, cols, perm = t(graph.rows), t(graph.cols), t(graph.transpose_perm)
    first = None
    for _ in range(5):
        xt, yt, wt = t(x, True), t(y, True), t(w, True)
        out = conv(xt, yt, wt, rows, cols, perm)
        out.backward(t(g))
        snap = [out.detach().cpu(), xt.grad.cpu(), yt.grad.cpu(), wt.grad.cpu()]
        if first is None:
            first = snap
        else:
            for a, b in zip(snap, first):
                assert torch.equal(a, b)


def test_conv_edge_cases():
    """No edges at all; the reference README's 3-node / 4-edge graph; isolated receivers stay exactly zero."""
    import openequivariance_b200 as oeq
    p = MATRIX["uvu_m5"]
    for det in (False, True):
        conv = oeq.TensorProductConv(p, deterministic=det)
        X = torch.rand(3, p.irreps_in1.dim, device="cuda")
        empty = torch.zeros(0, dtype=torch.int64, device="cuda")
        Z = conv(X, torch.zeros(0, p.irreps_in2.dim, device="cuda"), torch.zeros(0, p.weight_numel, device="cuda"),
                 empty, empty, empty if det else None)
        assert Z.shape == (3, p.irreps_out.dim) and float(Z.abs().max()) == 0.0
        rows = torch.tensor([0, 1, 1, 2], device="cuda")
        cols = torch.tensor([1, 0, 2, 1], device="cuda")
        perm = torch.tensor([1, 0, 3, 2], device="cuda")
        Y = torch.rand(4, p.irreps_in2.dim, device="cuda")
        W = torch.rand(4, p.weight_numel, device="cuda")
        Z = conv(X, Y, W, rows, cols, perm if det else None).cpu().numpy()
        want = tp_oracle.forward(p, X.cpu().numpy(), Y.cpu().numpy(), conv.reorder_weights_to_e3nn(W.cpu().numpy()),
                                 graph=(rows.cpu().numpy(), cols.cpu().numpy()))
        assert rel_l2(Z, want) <= 1e-5


def test_isolated_nodes_get_zero_rows(graph):
    p = MATRIX["uvu_m33v3"]
    conv = _conv(p, "deterministic")
    E, N = graph.nnz, graph.node_count
    x, y, w, *_ = uniform_inputs(p, E, n_rows=N)
    got = np.full((N, p.irreps_out.dim), 7.0, dtype=np.float32)
    conv.forward_cpu(x, y, w, got, graph)
    present = np.zeros(N, dtype=bool)
    present[graph.rows] = True
    assert (~present).sum() >= 2
    assert np.all(got[~present] == 0.0)


def test_int32_indices_through_the_c_abi(graph):
    """Descriptors built with idx_dtype=int32 (what a JAX front end would pass; the reference's JAX extension uses int32
    indices) run the same kernels on 32-bit rows / cols / perm."""
    import ctypes
    from openequivariance_b200 import native
    from openequivariance_b200.core.descriptor import build_descriptor, descriptor_hash
    p = MATRIX["mace_medium"]
    E, N = graph.nnz, graph.node_count
    x, y, w, *_ = uniform_inputs(p, E, n_rows=N)
    lib = native.load()
    outs = []
    for idx_np, idx_t in ((np.int64, torch.int64), (np.int32, torch.int32)):
        text = build_descriptor(p, conv=True, deterministic=True, idx_dtype=idx_np)
        desc, key = text.encode(), descriptor_hash(text)
        X, Y, W = (torch.tensor(a, device="cuda") for a in (x, y, w))
        rows, cols, perm = (torch.tensor(a, device="cuda").to(idx_t) for a in (graph.rows, graph.cols, graph.transpose_perm))
        Z = torch.full((N, p.irreps_out.dim), float("nan"), device="cuda")
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        rc = lib.oeqb_conv_forward(desc, len(desc), key, N, E, ptr(X), ptr(Y), ptr(W), ptr(Z), ptr(rows), ptr(cols), ptr(perm),
                                   None, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        native.check(rc, "oeqb_conv_forward")
        outs.append(Z.cpu())
    assert torch.equal(outs[0], outs[1])
    assert rel_l2(outs[1].numpy(), tp_oracle.forward(p, x, y, w, graph=(graph.rows, graph.cols))) <= 1e-5


def test_two_step_backward_equals_the_single_call(graph):
    """oeqb_conv_backward_edges + oeqb_conv_backward_rows (two row ranges, the later rows first, as the partitioned driver
    calls them) against oeqb_conv_backward: identical bits for dX, dY and dW."""
    import ctypes
    from openequivariance_b200 import native
    from openequivariance_b200.core.descriptor import build_descriptor, descriptor_hash
    p = MATRIX["mace_medium"]
    E, N = graph.nnz, graph.node_count
    x, y, w, g, *_ = uniform_inputs(p, E, n_rows=N)
    lib = native.load()
    text = build_descriptor(p, conv=True, deterministic=True)
    desc, key = text.encode(), descriptor_hash(text)
    X, Y, W, G = (torch.tensor(a, device="cuda") for a in (x, y, w, g))
    rows, cols, perm = (torch.tensor(a, device="cuda") for a in (graph.rows, graph.cols, graph.transpose_perm))
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    need = lib.oeqb_conv_workspace_bytes(desc, len(desc), key, 1, N, E)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    ref = [torch.full_like(t, float("nan")) for t in (X, Y, W)]
    native.check(lib.oeqb_conv_backward(desc, len(desc), key, N, E, ptr(X), ptr(Y), ptr(W), ptr(G), ptr(ref[0]), ptr(ref[1]),
                                        ptr(ref[2]), ptr(rows), ptr(cols), ptr(perm), ptr(ws), need, st), "single call")
    got = [torch.full_like(t, float("nan")) for t in (X, Y, W)]
    ws2 = torch.empty(need, dtype=torch.uint8, device="cuda")
    native.check(lib.oeqb_conv_backward_edges(desc, len(desc), key, N, N, E, ptr(X), ptr(Y), ptr(W), ptr(G), ptr(got[1]),
                                              ptr(got[2]), ptr(rows), ptr(cols), ptr(perm), ptr(ws2), need, st), "edges")
    split = N - 11
    native.check(lib.oeqb_conv_backward_rows(desc, len(desc), key, N, E, split, N, ptr(perm), ptr(ws2), need, ptr(got[0]), st), "rows")
    native.check(lib.oeqb_conv_backward_rows(desc, len(desc), key, N, E, 0, split, ptr(perm), ptr(ws2), need, ptr(got[0]), st), "rows")
    torch.cuda.synchronize()
    for a, b, what in zip(got, ref, ("dX", "dY", "dW")):
        assert torch.equal(a, b), what
    # a problem without those kernels is refused
    other = MATRIX["uvw_m4"]
    text = build_descriptor(other, conv=True, deterministic=True)
    rc = lib.oeqb_conv_backward_rows(text.encode(), len(text), descriptor_hash(text), N, E, 0, N, ptr(perm), ptr(ws2), need, ptr(got[0]), st)
    assert rc == 5
