"""Argument checks of the op layer raise RuntimeError with the reference's messages
(tests/input_validation_test.py:96-140) and the ops run on the current stream and on any visible device."""
import os

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


@pytest.mark.parametrize("det", [False, True], ids=["atomic", "deterministic"])
def test_bad_indices_are_refused_before_any_main_kernel(det):
    """rows / cols / transpose_perm become addresses of bulk copies inside the kernels, so the library checks them on
    the device first (one small kernel, then a wait) and refuses the call; the bad access itself never happens."""
    from openequivariance_b200 import native
    exe, bufs = _conv_and_buffers(det)
    exe(*bufs)
    x, y, w, rows, cols = bufs[:5]

    def refused(*args):
        before = native.launch_count()
        with pytest.raises(RuntimeError, match="must lie in"):
            exe(*args)
        assert native.launch_count() - before == 1          # the checking kernel only
        torch.cuda.synchronize()
        assert native.load().oeqb_check_status() == 0       # and it left no stale failure behind

    bad_cols = cols.clone()
    bad_cols[2] = 3                                           # n_nodes is 3
    refused(x, y, w, rows, bad_cols, *bufs[5:])
    bad_rows = rows.clone()
    bad_rows[0] = -1
    refused(x, y, w, bad_rows, cols, *bufs[5:])
    if det:
        unsorted = torch.tensor([1, 0, 1, 2], device="cuda")
        refused(x, y, w, unsorted, cols, bufs[5])
        bad_perm = bufs[5].clone()
        bad_perm[1] = 4                                       # n_edges is 4: only the backward pass reads it
        xg = x.clone().requires_grad_(True)
        out = exe(xg, y, w, rows, cols, bad_perm)
        with pytest.raises(RuntimeError, match="must lie in"):
            out.sum().backward()
    exe(*bufs)                                                # a good call still works afterwards


@pytest.mark.parametrize("det", [False, True], ids=["atomic", "deterministic"])
def test_conv_pickle_export_compile_roundtrip(det, tmp_path):
    """torch.save / torch.export(strict=False) / torch.compile(fullgraph=True) of the convolution module, forward and
    backward under compile, as the reference tests them (tests/export_test.py:61-116)."""
    exe, bufs = _conv_and_buffers(det)
    ref = exe(*bufs)
    torch.save(exe, tmp_path / "conv.pt")
    again = torch.load(tmp_path / "conv.pt", weights_only=True)
    assert torch.allclose(again(*bufs), ref, atol=1e-6)
    exported = torch.export.export(exe, tuple(bufs), strict=False)
    assert torch.allclose(exported.module()(*bufs), ref, atol=1e-6)
    compiled = torch.compile(exe, fullgraph=True)
    xs = [b.clone().requires_grad_(True) if b.is_floating_point() else b for b in bufs]
    out = compiled(*xs)
    out.sum().backward()
    ys = [b.clone().requires_grad_(True) if b.is_floating_point() else b for b in bufs]
    exe(*ys).sum().backward()
    assert torch.allclose(out, ref, atol=1e-6)
    for a, b in zip(xs[:3], ys[:3]):
        assert torch.allclose(a.grad, b.grad, atol=1e-5)


def test_kernels_are_named_by_pass():
    """Profiler trace of forward + backward + double backward issued on a side stream: the kernels of this library show
    up with names that carry ``forward`` / ``backward`` / ``double_backward`` (the substrings the reference's timing
    helper and stream test select kernels by: core/utils.py:174-203, tests/stream_test.py:97-391)."""
    from torch.profiler import ProfilerActivity, profile
    import openequivariance_b200 as oeq
    p = MATRIX["mace_medium"]
    tp = oeq.TensorProduct(p)
    x, y, w, g, *_ = uniform_inputs(p, 64)
    xt, yt, wt = (torch.tensor(t, device="cuda", requires_grad=True) for t in (x, y, w))
    gt = torch.tensor(g, device="cuda", requires_grad=True)
    side = torch.cuda.Stream()

    def run():
        out = tp(xt, yt, wt)
        gx, gy, gw = torch.autograd.grad(out, [xt, yt, wt], gt, create_graph=True)
        (gx.sum() + gy.sum() + gw.sum()).backward()

    with torch.cuda.stream(side):
        run()                                                  # compile / load outside the trace
    side.synchronize()
    try:
        with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
            with torch.cuda.stream(side):
                run()
            side.synchronize()
        events = [e for e in prof.events() if "oeq_" in e.name]
    except Exception as exc:  # noqa: BLE001 - no CUPTI on this machine: nothing to check
        pytest.skip(f"profiler unavailable: {exc}")
    if not events:
        pytest.skip("the profiler recorded no device kernels on this machine")
    names = {e.name for e in events}
    assert any("forward" in n and "double_backward" not in n and "backward" not in n for n in names), names
    assert any("backward" in n and "double_backward" not in n for n in names), names
    assert any("double_backward" in n for n in names), names


def test_python_operator_layer_still_works():
    """The operators are normally the C++ registrations of csrc/torch_ops.cpp; the equivalent Python implementation
    (used when that library has not been built) must keep producing the same results and the same error texts."""
    import subprocess
    import sys
    from helpers import ROOT
    code = (
        "import torch, numpy as np, sys\n"
        "sys.path.insert(0, 'tests')\n"
        "import openequivariance_b200 as oeq\n"
        "from openequivariance_b200._torch import ops\n"
        "from helpers import tp_problem_matrix, uniform_inputs, rel_l2\n"
        "from oracle import tp_oracle\n"
        "assert not ops.CPP_OPS\n"
        "p = dict(tp_problem_matrix())['uvu_m5']\n"
        "x, y, w, g, *_ = uniform_inputs(p, 32)\n"
        "tp = oeq.TensorProduct(p)\n"
        "xt, yt, wt = (torch.tensor(t, device='cuda', requires_grad=True) for t in (x, y, w))\n"
        "out = tp(xt, yt, wt); out.backward(torch.tensor(g, device='cuda'))\n"
        "assert rel_l2(out.detach().cpu().numpy(), tp_oracle.forward(p, x, y, w)) <= 1e-5\n"
        "assert rel_l2(xt.grad.cpu().numpy(), tp_oracle.backward(p, x, y, w, g)[0]) <= 1e-5\n"
        "try:\n"
        "    tp(xt.unsqueeze(1), yt, wt)\n"
        "except RuntimeError as e:\n"
        "    assert 'Shape mismatch' in str(e)\n"
        "else:\n"
        "    raise SystemExit('no error')\n"
        "print('ok')\n")
    env = dict(os.environ, OEQB_PYTHON_OPS="1")
    r = subprocess.run([sys.executable, "-c", code], cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "ok" in r.stdout, r.stdout[-2000:] + r.stderr[-2000:]


_AOTI_PROBE = r"""
import os, sys, torch
class M(torch.nn.Module):
    def forward(self, x):
        return x * 2 + 1
x = torch.randn(8, 4, device="cuda")
ep = torch.export.export(M(), (x,), strict=False)
path = torch._inductor.aoti_compile_and_package(ep, package_path=sys.argv[1])
m = torch._inductor.aoti_load_package(path)
assert torch.allclose(m(x), x * 2 + 1)
print("aoti ok")
"""
_AOTI_STATE = {}


def _gomp_fix(tmp_path):
    """inductor links its wrapper with -fopenmp; a compiler installed outside the system prefix does not find a
    libgomp.spec by itself.  Point it at torch's own libgomp through a spec file in a scratch directory."""
    fix = tmp_path / "gomp"
    fix.mkdir(exist_ok=True)
    (fix / "libgomp.spec").write_text("*link_gomp: -lgomp %{static: -ldl }\n")
    lib = os.path.join(os.path.dirname(torch.__file__), "lib", "libgomp.so.1")
    if os.path.exists(lib) and not (fix / "libgomp.so").exists():
        os.symlink(lib, fix / "libgomp.so")
    return str(fix) + os.pathsep + os.environ.get("LIBRARY_PATH", "")


def _aoti_package(tmp_path):
    import subprocess
    import sys
    os.environ["LIBRARY_PATH"] = _gomp_fix(tmp_path)
    if "ok" not in _AOTI_STATE:
        # AOTInductor itself has to work on this machine: a package of a model without any custom operator, built and
        # loaded in a child process (a broken tool chain crashes the loader instead of raising)
        r = subprocess.run([sys.executable, "-c", _AOTI_PROBE, str(tmp_path / "probe.pt2")], capture_output=True, text=True,
                           timeout=900)
        _AOTI_STATE["ok"] = r.returncode == 0 and "aoti ok" in r.stdout
        _AOTI_STATE["why"] = f"exit code {r.returncode}: {(r.stderr or r.stdout)[-200:]}"
    if not _AOTI_STATE["ok"]:
        pytest.skip("AOTInductor cannot build and load even a package without custom operators on this machine "
                    f"({_AOTI_STATE['why']})")
    exe, bufs = _tp_and_buffers()
    ep = torch.export.export(exe, tuple(bufs), strict=False)
    path = torch._inductor.aoti_compile_and_package(ep, package_path=str(tmp_path / "tp.pt2"))
    return exe, bufs, path


def test_aoti_package_in_python(tmp_path):
    """torch.export -> AOTInductor package -> load and run (the reference's tests/export_test.py:119-137)."""
    exe, bufs, path = _aoti_package(tmp_path)
    model = torch._inductor.aoti_load_package(path)
    assert torch.allclose(model(*bufs), exe(*bufs), atol=1e-5)


def test_aoti_package_from_cpp(tmp_path):
    """The same package run by a stand-alone C++ program that gets the operators from liboeq_b200_torch.so alone (no
    Python in the process), as the reference's extension/test/load_aoti.cpp does for its own extension."""
    import subprocess
    from torch.utils import cpp_extension as ce
    from helpers import ROOT
    from openequivariance_b200 import build_native
    exe, bufs, path = _aoti_package(tmp_path)
    runner = tmp_path / "run_package"
    lib = ce.library_paths()[0]
    cmd = [os.environ.get("CXX", "g++"), "-O1", "-std=c++17", os.path.join(ROOT, "tests", "aoti", "run_package.cpp"),
           "-o", str(runner), f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}"]
    cmd += [f"-I{p}" for p in ce.include_paths()] + ["-I/usr/local/cuda/include", f"-L{lib}", "-ltorch", "-ltorch_cpu",
                                                      "-ltorch_cuda", "-lc10", "-lc10_cuda", "-ldl", f"-Wl,-rpath,{lib}"]
    build = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    if build.returncode != 0:
        pytest.skip(f"could not compile the C++ runner here: {build.stderr[-300:]}")
    B, L1, L2, wn = bufs[0].shape[0], bufs[0].shape[1], bufs[1].shape[1], bufs[2].shape[1]
    run = subprocess.run([str(runner), build_native.TORCH_LIB, path, str(B), str(L1), str(L2), str(wn)],
                         capture_output=True, text=True, timeout=600)
    assert run.returncode == 0, run.stdout[-1000:] + run.stderr[-2000:]
    got = dict(line.split(" ", 1) for line in run.stdout.strip().splitlines())

    def ramp(rows, cols, scale):
        return torch.sin(torch.arange(rows * cols, dtype=torch.float32, device="cuda") * scale).reshape(rows, cols)

    want = exe(ramp(B, L1, 0.37), ramp(B, L2, 0.11), ramp(B, wn, 0.23)).double().cpu()
    assert got["shape"].split() == [str(want.shape[0]), str(want.shape[1])]
    assert abs(float(got["sum"]) - float(want.sum())) <= 1e-4 * float(want.abs().sum())
    assert abs(float(got["abs"]) - float(want.abs().sum())) <= 1e-5 * float(want.abs().sum())


def test_a_starved_wait_gives_up_and_reports():
    """Every spin on a barrier in the pipelined kernels is bounded.  The library's self-test launches a CTA whose barrier is
    never arrived at: the kernel has to come back by itself (~2 s), all of its threads have to leave through the abort
    flag, and the code has to reach the host through the status word; afterwards the context is usable as before."""
    import ctypes
    import openequivariance_b200 as oeq
    from openequivariance_b200 import native
    p = MATRIX["mace_medium"]
    conv = oeq.TensorProductConv(p, deterministic=True)
    desc = conv.kernel_string.encode()
    lib = native.load()
    assert lib.oeqb_check_status() == 0
    with torch.cuda.device(0):
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        native.check(lib.oeqb_selftest_bounded_wait(desc, len(desc), conv.hash, st), "oeqb_selftest_bounded_wait")
    assert lib.oeqb_check_status() == 0                      # the self-test consumed the code it provoked
    tp = oeq.TensorProduct(p)
    x, y, w, *_ = uniform_inputs(p, 16)
    out = tp(*(torch.tensor(t, device="cuda") for t in (x, y, w)))
    assert torch.isfinite(out).all()


@pytest.mark.parametrize("start", [np.float32, np.float64])
def test_module_follows_its_parent_to_another_dtype(start):
    """``parent.to(dtype)`` re-specialises a TensorProduct / TensorProductConv held as a submodule (the reference's
    tests/batch_test.py:383-451): outputs come back in the new dtype and agree with the oracle."""
    import openequivariance_b200 as oeq
    from helpers import with_dtype
    from oracle import tp_oracle
    problem = with_dtype(MATRIX["mace_medium"], start)

    class Parent(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.tp = oeq.TensorProduct(problem)
            self.conv = oeq.TensorProductConv(problem, deterministic=False)

        def forward(self, x, y, w):
            return self.tp(x, y, w)

    parent = Parent()
    first = torch.float32 if start == np.float32 else torch.float64
    other = torch.float64 if start == np.float32 else torch.float32
    for dtype in (first, other):
        if dtype != first:
            parent.to(dtype)
        npdt = np.float32 if dtype == torch.float32 else np.float64
        x, y, w, *_ = uniform_inputs(with_dtype(problem, npdt), 10, seed=3)
        out = parent(*(torch.tensor(t, device="cuda") for t in (x, y, w)))
        assert out.dtype == dtype
        want = tp_oracle.forward(problem, x, y, parent.tp.reorder_weights_to_e3nn(w))
        assert np.linalg.norm(out.cpu().numpy() - want) / np.linalg.norm(want) <= (1e-5 if dtype == torch.float32 else 1e-12)
        rows = torch.tensor([0, 1, 1, 2], device="cuda")
        cols = torch.tensor([1, 0, 2, 1], device="cuda")
        xs, ys, ws = (torch.tensor(t[:4] if i else t[:3], device="cuda") for i, t in enumerate((x, y, w)))
        z = parent.conv(xs, ys, ws, rows, cols)
        assert z.dtype == dtype and z.shape == (3, problem.irreps_out.dim)
