"""More than one GPU in a machine: the same problem on every visible device, from one process (the library's
per-device bookkeeping: shared-memory opt-in per kernel and device, status word per device) and from one process per
device launched by torchrun, as the reference tests it (tests/multidevice_test.py:7-57).  MACE-large on purpose: its
kernels need more than 48 KB of dynamic shared memory, which has to be enabled on each device separately.
Skipped on a single-GPU machine."""
import os
import subprocess
import sys
import textwrap

import numpy as np
import pytest
import torch

from helpers import ROOT, rel_l2, uniform_inputs
from oracle import tp_oracle

pytestmark = pytest.mark.gpu


def _problem():
    from openequivariance_b200.core import problems as P
    return P.mace_problems()[0]


def _needs_two():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")


def test_same_module_on_every_device_of_one_process():
    _needs_two()
    import openequivariance_b200 as oeq
    p = _problem()
    x, y, w, g, *_ = uniform_inputs(p, 200)
    want = tp_oracle.forward(p, x, y, w)
    tp = oeq.TensorProduct(p)
    outs = []
    for d in range(torch.cuda.device_count()):
        dev = f"cuda:{d}"
        xt, yt, wt = (torch.tensor(t, device=dev, requires_grad=True) for t in (x, y, tp.reorder_weights_from_e3nn(w)))
        out = tp(xt, yt, wt)                       # current device stays 0: the op switches to the tensors' device
        out.backward(torch.tensor(g, device=dev))
        outs.append((out.detach().cpu(), xt.grad.cpu()))
        assert rel_l2(outs[-1][0].numpy(), want) <= 1e-5
    for o, gx in outs[1:]:
        assert torch.equal(o, outs[0][0]) and torch.equal(gx, outs[0][1])


def test_one_process_per_device():
    _needs_two()
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.path.join(ROOT, "tests") + os.pathsep + os.environ.get("PYTHONPATH", ""))
    result = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--standalone", "--local-addr", "127.0.0.1",
                             "--nnodes=1", "--nproc-per-node=2", __file__], capture_output=True, check=False, env=env,
                            timeout=600)
    if result.returncode != 0:
        pytest.fail(textwrap.dedent(f"""
            torchrun failed with code {result.returncode}
            stdout: {result.stdout.decode()[-3000:]}
            stderr: {result.stderr.decode()[-3000:]}"""))


if __name__ == "__main__":
    import openequivariance_b200 as oeq

    local_rank = int(os.environ["LOCAL_RANK"])
    device = f"cuda:{local_rank}"
    p = _problem()
    x, y, w, *_ = uniform_inputs(p, 1000)
    tp = oeq.TensorProduct(p)
    with torch.cuda.device(device):
        out = tp(torch.tensor(x, device=device), torch.tensor(y, device=device),
                 torch.tensor(tp.reorder_weights_from_e3nn(w), device=device))
        torch.cuda.synchronize()
    err = rel_l2(out.cpu().numpy(), tp_oracle.forward(p, x, y, w))
    assert err <= 1e-5, err
    print(f"rank {local_rank} on {device}: rel-L2 {err:.2e}")
