"""Single-irrep sweep over the reference's multiplicities (tests/batch_test.py:144-264): 1 ... 512 for 'uvu', 1 ... 64 for
'uvw', including sizes that are not multiples of 32 and second operands with multiplicity > 1, for three of its irrep
triples (l up to 7).  Forward and backward of each problem against the fp64 oracle, fp32, relative L2 <= 1e-5."""
import numpy as np
import pytest

from helpers import REL_L2, rel_l2, single, uniform_inputs
from oracle import tp_oracle

pytestmark = pytest.mark.gpu

UVU_MULS = [(1, 1, 1), (2, 1, 2), (4, 1, 4), (8, 1, 8), (16, 1, 16), (32, 1, 32), (5, 1, 5), (13, 1, 13), (19, 1, 19),
            (33, 1, 33), (49, 1, 49), (50, 1, 50), (123, 1, 123), (128, 1, 128), (256, 1, 256), (512, 1, 512), (1, 2, 1),
            (1, 4, 1), (1, 16, 1), (1, 32, 1), (16, 3, 16), (16, 9, 16), (24, 24, 24), (32, 32, 32)]
UVW_MULS = [(1, 1, 1), (2, 1, 2), (4, 1, 4), (8, 1, 8), (16, 1, 16), (32, 1, 32), (5, 1, 5), (13, 1, 13), (19, 1, 19),
            (33, 1, 33), (49, 1, 49), (50, 1, 50), (64, 1, 64), (1, 2, 1), (1, 4, 1), (1, 16, 1), (1, 32, 1), (16, 3, 16),
            (16, 9, 16), (24, 24, 24), (32, 32, 32)]
IRS = [(1, 1, 1), (2, 2, 4), (7, 2, 5)]


def _cases():
    for mode, muls in (("uvu", UVU_MULS), ("uvw", UVW_MULS)):
        for m in muls:
            yield pytest.param(mode, m, id=f"{mode}-{m[0]}x{m[1]}x{m[2]}")


@pytest.mark.parametrize("mode,m", list(_cases()))
def test_single_irrep_sweep(mode, m):
    import openequivariance_b200 as oeq
    for i in IRS:
        p = single(f"{m[0]}x{i[0]}e", f"{m[1]}x{i[1]}e", f"{m[2]}x{i[2]}e", mode)
        tp = oeq.TensorProduct(p)
        B = 24 if p.weight_numel > 4096 else 64
        x, y, w, g, *_ = uniform_inputs(p, B)
        # the harness hooks take and return weights in e3nn order, like the oracle
        got = np.zeros((B, p.irreps_out.dim), dtype=np.float32)
        tp.forward_cpu(x, y, got, w)
        assert rel_l2(got, tp_oracle.forward(p, x, y, w)) <= REL_L2[np.float32], (i, "forward")
        dx, dy, dw = np.zeros_like(x), np.zeros_like(y), np.zeros_like(w)
        tp.backward_cpu(x, dx, y, dy, g, w, dw)
        wdx, wdy, wdw = tp_oracle.backward(p, x, y, w, g)
        for a, b, what in ((dx, wdx, "dx"), (dy, wdy, "dy"), (dw, wdw, "dW")):
            assert rel_l2(a, b) <= REL_L2[np.float32], (i, what)
