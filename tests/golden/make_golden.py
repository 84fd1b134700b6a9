"""Regenerates the golden fixtures in this directory from the reference checkout.

Run in a container that has the reference sources (they are imported read-only, torch-free):

    OEQ_NOTORCH=1 PYTHONPATH=/path/to/reference/openequivariance python tests/golden/make_golden.py

Outputs (committed):
  wigner_3j.npz        every real Wigner-3j tensor with l1, l2, l3 <= 5 (plus a few up to l=7), float64
  problems.json        path weights, weight_numel, irreps dims and the e3nn->kernel weight permutation for a
                       list of problems, obtained from the reference's TPProblem / ComputationSchedule classes
  coord_graph.json     rows / cols / transpose_perm of the reference CoordGraph on a small random edge list
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    os.environ["OEQ_NOTORCH"] = "1"
    from openequivariance.core.e3nn_lite import wigner_3j
    from openequivariance.benchmark import problems as rp
    from openequivariance.core.ComputationSchedule import ComputationSchedule
    from openequivariance.core.ConvolutionBase import CoordGraph
    import torch
    from openequivariance._torch.utils import reorder_torch

    w3j = {}
    for l1 in range(8):
        for l2 in range(8):
            for l3 in range(abs(l1 - l2), min(l1 + l2, 7) + 1):
                if max(l1, l2, l3) <= 5 or (l1, l2, l3) in [(7, 2, 5), (5, 2, 7), (6, 1, 7), (7, 7, 0), (3, 4, 7)]:
                    w3j[f"{l1}_{l2}_{l3}"] = wigner_3j(l1, l2, l3)
    np.savez_compressed(os.path.join(HERE, "wigner_3j.npz"), **w3j)

    def spec(name, cls, args, kwargs):
        if cls == "TPProblem":
            p = rp.TPProblem(args[0], args[1], args[2], [tuple(i) for i in args[3]], **kwargs)
        else:
            p = getattr(rp, cls)(*args, **kwargs)
        sched = ComputationSchedule(p, smem_limit=232448, warps_per_block=1, warp_size=32, block_count=1,
                                    direction="forward", irrep_dtype=np.float32, weight_dtype=np.float32,
                                    include_scratch=(p.instructions[0].connection_mode == "uvw"),
                                    stream_weights=(p.instructions[0].connection_mode == "uvw"), schedule_type=3)
        ident = torch.arange(p.weight_numel, dtype=torch.float64)
        batched = not p.shared_weights
        w_in = ident.unsqueeze(0) if batched else ident
        oeq = reorder_torch(sched, w_in, "forward", batched).reshape(-1).to(torch.int64).tolist()
        return {
            "name": name, "cls": cls, "args": args, "kwargs": kwargs,
            "L1_dim": p.irreps_in1.dim, "L2_dim": p.irreps_in2.dim, "L3_dim": p.irreps_out.dim,
            "irreps_out": str(p.irreps_out), "weight_numel": p.weight_numel,
            "shared_weights": bool(p.shared_weights),
            "instructions": [[i.i_in1, i.i_in2, i.i_out, i.connection_mode, bool(i.has_weight),
                              float(i.path_weight), list(i.path_shape)] for i in p.instructions],
            # identity permutations are stored as the string "identity" to keep the fixture small
            "oeq_from_e3nn_perm": "identity" if oeq == list(range(p.weight_numel)) else oeq,
        }

    feats = "128x0e+128x1o+128x2e+128x3o"
    nq = "32x0e+32x0o+32x1e+32x1o+32x2e+32x2o"
    specs = [
        spec("readme", "TPProblem", ["1x2e", "1x3e", "1x2e", [[0, 0, 0, "uvu", True]]], {"shared_weights": False, "internal_weights": False}),
        spec("mace_like", "ChannelwiseTPP", [feats, "1x0e+1x1o+1x2e+1x3o", feats], {}),
        spec("nequip_like", "FullyConnectedTPProblem", [nq, "1x0e+1x1o+1x2e", nq], {"shared_weights": True}),
        spec("uvu_v3", "SingleInstruction", ["16x1e", "3x1e", "16x1e", "uvu"], {}),
        spec("uvu_big", "SingleInstruction", ["70x2e", "33x1o", "70x3o", "uvu"], {}),
        spec("uvw_64", "SingleInstruction", ["64x1e", "1x1e", "64x1e", "uvw"], {}),
        spec("uvw_ragged", "SingleInstruction", ["40x1o", "3x2e", "33x1o", "uvw"], {}),
        spec("diffdock1", "FullyConnectedTPProblem", ["10x1o + 10x1e + 48x0e + 48x0o", "1x0e + 1x1o", "10x1o + 10x1e + 48x0e + 48x0o"], {"shared_weights": False}),
        spec("tetris2", "FullyConnectedTPProblem", ["64x0e + 24x1e + 24x1o + 16x2e + 16x2o", "1x0e + 1x1o + 1x2e", "0o + 6x0e"], {}),
    ]
    specs = [s for s in specs if s is not None]
    # a mixed-normalisation problem, spec layer only (mixed modes are rejected by the kernels, so no schedule)
    p = rp.TPProblem("4x1o+2x2e", "2x1o+1x0e", "4x1o+4x2e+4x0e",
                     [(0, 0, 1, "uvu", True, 2.0), (0, 1, 0, "uvu", True), (0, 0, 2, "uvu", True, 0.5), (1, 1, 1, "uvw", True)],
                     irrep_normalization="norm", path_normalization="path", in1_var=[1.0, 2.0], in2_var=[0.5, 1.5],
                     out_var=[1.0, 3.0, 0.25])
    norm_case = {"path_weights": [float(i.path_weight) for i in p.instructions], "weight_numel": p.weight_numel}
    with open(os.path.join(HERE, "problems.json"), "w") as f:
        json.dump({"problems": specs, "norm_path_case": norm_case}, f)

    rng = np.random.default_rng(7)
    n, e = 12, 60
    rows = rng.integers(0, n, size=e).astype(np.int64)
    cols = rng.integers(0, n, size=e).astype(np.int64)
    g = CoordGraph(np.zeros((n, 3)), rows, cols, "g")
    with open(os.path.join(HERE, "coord_graph.json"), "w") as f:
        json.dump({"n": n, "rows_in": rows.tolist(), "cols_in": cols.tolist(), "rows": g.rows.tolist(),
                   "cols": g.cols.tolist(), "transpose_perm": g.transpose_perm.tolist()}, f)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    sys.exit(main())
