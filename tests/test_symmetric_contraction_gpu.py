"""Ragged grouped products and the symmetric contraction built on them, against plain torch (einsum) in fp64:
forward, both gradients, empty groups, fp32 and fp64.  The generalised Clebsch-Gordan tensors U are random here: the
contraction is linear algebra in U, so any U exercises it (the reference takes U from e3nn, which is not installed)."""
import pytest
import torch

from helpers import rel_l2

pytestmark = pytest.mark.gpu


def _groups(counts, dev):
    return torch.repeat_interleave(torch.arange(len(counts), device=dev), torch.tensor(counts, device=dev))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.float64, 1e-13)])
@pytest.mark.parametrize("M,K", [(256, 16), (37, 9), (5, 1), (130, 25)])
def test_group_gemm_both_modes_and_gradients(dtype, tol, M, K):
    from openequivariance_b200._torch.symmetric_contraction import group_gemm
    dev = "cuda"
    counts = [7, 0, 33, 1, 90]
    G, F, N = len(counts), 6, sum(counts)
    gen = torch.Generator(device=dev).manual_seed(M * 100 + K)
    A = torch.randn(G, F, M, K, device=dev, dtype=dtype, generator=gen, requires_grad=True)
    B = torch.randn(N, F, K, device=dev, dtype=dtype, generator=gen, requires_grad=True)
    cot = torch.randn(N, F, M, device=dev, dtype=dtype, generator=gen)
    bc = torch.tensor(counts, dtype=torch.int64)
    out = group_gemm(A, B, bc, M, K, 0, G)
    gA, gB = torch.autograd.grad(out, [A, B], cot)
    Ad, Bd = A.detach().double().requires_grad_(True), B.detach().double().requires_grad_(True)
    want = torch.einsum("nfmk,nfk->nfm", Ad[_groups(counts, dev)], Bd)
    wA, wB = torch.autograd.grad(want, [Ad, Bd], cot.double())
    for got, ref, what in ((out, want, "C"), (gA, wA, "dA"), (gB, wB, "dB")):
        assert rel_l2(got.detach().cpu().numpy(), ref.detach().cpu().numpy()) <= tol, what
    assert float(gA[1].abs().max()) == 0.0                      # the empty group's weights get an exactly zero gradient
    # mode 1 on its own, and reproducible
    Y = torch.randn(N, F, M, device=dev, dtype=dtype, generator=gen)
    first = group_gemm(Y, B.detach(), bc, M, K, 1, G)
    assert torch.equal(first, group_gemm(Y, B.detach(), bc, M, K, 1, G))
    ref = torch.zeros(G, F, M, K, device=dev, dtype=torch.float64).index_add_(
        0, _groups(counts, dev), torch.einsum("nfm,nfk->nfmk", Y.double(), B.detach().double()))
    assert rel_l2(first.cpu().numpy(), ref.cpu().numpy()) <= tol


def _einsum_contraction(Us, Ws, x, elem):
    """MACE's symmetric contraction written with einsum (the oracle): Us / Ws indexed by order nu."""
    corr = max(Us)
    lead = "w" if Us[corr].dim() == corr + 2 else ""
    idx = "ijlpq"[:corr]
    out = torch.einsum(f"{lead}{idx}k,nkf,nf{idx[-1]}->nf{lead}{idx[:-1]}", Us[corr], Ws[corr][elem], x)
    for nu in range(corr - 1, 0, -1):
        idx = "ijlpq"[:nu]
        c = torch.einsum(f"{lead}{idx}k,nkf->nf{lead}{idx}", Us[nu], Ws[nu][elem]) + out
        out = torch.einsum(f"nf{lead}{idx},nf{idx[-1]}->nf{lead}{idx[:-1]}", c, x)
    return out.reshape(out.shape[0], -1)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.float64, 1e-12)])
def test_symmetric_contraction_matches_einsum(dtype, tol):
    from openequivariance_b200._torch.symmetric_contraction import SymmetricContraction
    dev = "cuda"
    ell, F, E, N, corr = 9, 8, 4, 150, 3
    gen = torch.Generator(device=dev).manual_seed(3)
    rnd = lambda *s: torch.randn(*s, device=dev, dtype=torch.float64, generator=gen)  # noqa: E731
    U_scalar = {nu: rnd(*([ell] * nu), 3 + nu) for nu in range(1, corr + 1)}          # output 0e
    U_vector = {nu: rnd(3, *([ell] * nu), 2 + nu) for nu in range(1, corr + 1)}       # output 1o
    sc = SymmetricContraction([U_scalar, U_vector], F, E, dtype=dtype).to(dev)
    elem = torch.randint(0, E, (N,), device=dev, generator=gen)
    elem[elem == 2] = 1                                                                # one element without nodes
    y = torch.nn.functional.one_hot(elem, E).to(dtype)
    x = torch.randn(N, F, ell, device=dev, dtype=dtype, generator=gen, requires_grad=True)
    out = sc(x, y)
    cot = torch.randn(out.shape, device=dev, dtype=dtype, generator=gen)
    params = [p for p in sc.parameters()]
    grads = torch.autograd.grad(out, [x] + params, cot)
    xd = x.detach().double().requires_grad_(True)
    wants, wparams = [], []
    for c, Us in zip(sc.contractions, (U_scalar, U_vector)):
        Ws = {corr: c.weights_max.detach().double().requires_grad_(True)}
        for i, w in enumerate(c.weights):
            Ws[corr - i - 1] = w.detach().double().requires_grad_(True)
        wants.append(_einsum_contraction(Us, Ws, xd, elem))
        wparams.append(Ws)
    want = torch.cat(wants, dim=-1)
    assert rel_l2(out.detach().cpu().numpy(), want.detach().cpu().numpy()) <= tol
    (wx,) = torch.autograd.grad(want, [xd], cot.double(), retain_graph=True)
    assert rel_l2(grads[0].cpu().numpy(), wx.cpu().numpy()) <= tol
    gw = torch.autograd.grad(want, [wparams[0][corr]], cot.double())[0]
    got_gw = dict(zip([id(p) for p in params], grads[1:]))[id(sc.contractions[0].weights_max)]
    assert rel_l2(got_gw.cpu().numpy(), gw.cpu().numpy()) <= tol
