"""Argument checks of the op layer raise RuntimeError with the reference's messages
(tests/input_validation_test.py:96-140) and the ops run on the current stream and on any visible device."""
import numpy as np
import pytest
import torch

from helpers import tp_problem_matrix, uniform_inputs

pytestmark = pytest.mark.gpu
MATRIX = dict(tp_problem_matrix())


def _tp_and_buffers():
    import openequivariance_b200 as oeq
    p = MATRIX["uvu_m5"]
    x, y, w, *_ = uniform_inputs(p, 8)
    return oeq.TensorProduct(p), [torch.tensor(t, device="cuda") for t in (x, y, w)]


def _conv_and_buffers(det):
    import openequivariance_b200 as oeq
    p = MATRIX["uvu_m5"]
    rows = torch.tensor([0, 1, 1, 2], device="cuda")
    cols = torch.tensor([1, 0, 2, 1], device="cuda")
    perm = torch.tensor([1, 0, 3, 2], device="cuda")
    x, y, w, *_ = uniform_inputs(p, 4, n_rows=3)
    bufs = [torch.tensor(t, device="cuda") for t in (x, y, w)] + [rows, cols] + ([perm] if det else [])
    return oeq.TensorProductConv(p, deterministic=det), bufs


CASES = [("tp", lambda: _tp_and_buffers()), ("conv_atomic", lambda: _conv_and_buffers(False)),
         ("conv_det", lambda: _conv_and_buffers(True))]


@pytest.mark.parametrize("kind,make", CASES, ids=[c[0] for c in CASES])
def test_argument_checks(kind, make):
    exe, bufs = make()
    exe(*bufs)
    for i in range(len(bufs)):
        b = [t.clone() for t in bufs]
        b[i] = b[i].unsqueeze(1)
        with pytest.raises(RuntimeError, match="Shape mismatch"):
            exe(*b)
        b = [t.clone() for t in bufs]
        b[i] = b[i].cpu()
        with pytest.raises(RuntimeError, match="is not on the GPU"):
            exe(*b)
        b = [t.clone() for t in bufs]
        b[i] = b[i].to(torch.bfloat16)
        with pytest.raises(RuntimeError, match="Dtype mismatch"):
            exe(*b)
        if not (kind != "tp" and i == 0):
            for j in range(bufs[i].dim()):
                b = [t.clone() for t in bufs]
                shape = list(b[i].shape)
                shape[j] += 1
                b[i] = torch.zeros(shape, dtype=b[i].dtype, device="cuda")
                with pytest.raises(RuntimeError, match="Shape mismatch"):
                    exe(*b)


def test_runs_on_current_stream_and_module_moves():
    exe, bufs = _tp_and_buffers()
    ref = exe(*bufs)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        out = exe(*bufs)
    s.synchronize()
    assert torch.equal(out, ref)
    # .to(dtype) re-specialises
    exe64 = exe.to(torch.float64)
    out64 = exe64(*[t.double() for t in bufs])
    assert out64.dtype == torch.float64 and torch.allclose(out64.float(), ref, atol=1e-5)


def test_pickle_compile_export_roundtrip(tmp_path):
    import openequivariance_b200 as oeq
    exe, bufs = _tp_and_buffers()
    ref = exe(*bufs)
    torch.save(exe, tmp_path / "tp.pt")
    again = torch.load(tmp_path / "tp.pt", weights_only=True)
    assert torch.equal(again(*bufs), ref)
    exported = torch.export.export(exe, tuple(bufs), strict=False)
    assert torch.equal(exported.module()(*bufs), ref)
    compiled = torch.compile(exe, fullgraph=True)
    xs = [b.clone().requires_grad_(True) for b in bufs]
    out = compiled(*xs)
    out.sum().backward()
    ys = [b.clone().requires_grad_(True) for b in bufs]
    exe(*ys).sum().backward()
    assert torch.allclose(out, ref)
    for a, b in zip(xs, ys):
        assert torch.allclose(a.grad, b.grad)
    assert isinstance(oeq.torch_ext_so_path(), str)
