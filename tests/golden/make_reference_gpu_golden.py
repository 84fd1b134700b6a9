"""Runs the UNMODIFIED reference (its own JIT CUDA kernels) on a GPU and records small input/output fixtures, plus
(optionally) its timing on the benchmark workload.

The reference checkout cannot travel to a GPU machine as a dependency of the tests, so this script is run once by hand:

    # on a machine with the reference sources: stage the package (not committed) and pre-build its extension
    cp -r <reference>/openequivariance/openequivariance baseline/_ref/
    # on the GPU machine, from the repository root
    TORCH_EXTENSIONS_DIR=$PWD/baseline/_ref/_torch_ext OEQ_JIT_EXTENSION=1 PYTHONPATH=$PWD/baseline/_ref:$PWD \
        python tests/golden/make_reference_gpu_golden.py --out out/reference_gpu.npz [--bench]

and the resulting ``reference_gpu.npz`` is committed next to this file.  Inputs are seeded; weights are stored in e3nn
order (the reference's ``reorder_weights_from_e3nn`` is applied before its kernels run, ``reorder_weights_to_e3nn``
to its weight gradients).
"""
import argparse
import json
import sys
import time
import warnings

import numpy as np
import torch

warnings.filterwarnings("ignore")


def cases():
    import openequivariance as oeq
    from openequivariance.benchmark.problems import ChannelwiseTPP, FullyConnectedTPProblem, SingleInstruction
    out = []
    out.append(("readme", oeq.TPProblem(oeq.Irreps("1x2e"), oeq.Irreps("1x3e"), oeq.Irreps("1x2e"), [(0, 0, 0, "uvu", True)],
                                       shared_weights=False, internal_weights=False), 6))
    out.append(("uvu_16x1e_3x1e", SingleInstruction("16x1e", "3x1e", "16x1e", "uvu"), 5))
    out.append(("uvw_40_3_33", SingleInstruction("40x1o", "3x2e", "33x1o", "uvw"), 3))
    out.append(("ctpp_32", ChannelwiseTPP("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"), 6))
    out.append(("fc_shared", FullyConnectedTPProblem("8x0e+8x1o+8x1e", "1x0e+1x1o", "8x0e+8x1o+8x1e", shared_weights=True), 7))
    return out


def run_tp(name, problem, batch, store):
    import openequivariance as oeq
    rng = np.random.default_rng(abs(hash(name)) % 1000 + 17)
    x = rng.uniform(size=(batch, problem.irreps_in1.dim)).astype(np.float32)
    y = rng.uniform(size=(batch, problem.irreps_in2.dim)).astype(np.float32)
    wshape = (problem.weight_numel,) if problem.shared_weights else (batch, problem.weight_numel)
    w = rng.uniform(size=wshape).astype(np.float32)
    g = rng.uniform(size=(batch, problem.irreps_out.dim)).astype(np.float32)
    tp = oeq.TensorProduct(problem)
    xt = torch.tensor(x, device="cuda", requires_grad=True)
    yt = torch.tensor(y, device="cuda", requires_grad=True)
    wt = torch.tensor(tp.reorder_weights_from_e3nn(w, not problem.shared_weights), device="cuda", requires_grad=True)
    z = tp(xt, yt, wt)
    z.backward(torch.tensor(g, device="cuda"))
    torch.cuda.synchronize()
    dw = tp.reorder_weights_to_e3nn(wt.grad.cpu().numpy(), not problem.shared_weights)
    for key, val in (("x", x), ("y", y), ("w", w), ("g", g), ("z", z.detach().cpu().numpy()), ("dx", xt.grad.cpu().numpy()),
                     ("dy", yt.grad.cpu().numpy()), ("dw", dw)):
        store[f"tp/{name}/{key}"] = val


def run_conv(store):
    import openequivariance as oeq
    from openequivariance.benchmark.problems import ChannelwiseTPP
    from openequivariance.core.ConvolutionBase import CoordGraph
    problem = ChannelwiseTPP("32x0e+32x1o", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e")
    rng = np.random.default_rng(5)
    n = 14
    pairs = [(i, j) for i in range(n) for j in range(n) if i != j and ((i * 7 + j * 3) % 4 == 0 or (j * 7 + i * 3) % 4 == 0)]
    rows = np.array([p[0] for p in pairs], dtype=np.int64)
    cols = np.array([p[1] for p in pairs], dtype=np.int64)
    graph = CoordGraph(np.zeros((n, 3)), rows, cols, "fixture")
    E = graph.nnz
    x = rng.uniform(size=(n, problem.irreps_in1.dim)).astype(np.float32)
    y = rng.uniform(size=(E, problem.irreps_in2.dim)).astype(np.float32)
    w = rng.uniform(size=(E, problem.weight_numel)).astype(np.float32)
    g = rng.uniform(size=(n, problem.irreps_out.dim)).astype(np.float32)
    store["conv/rows"], store["conv/cols"], store["conv/perm"] = graph.rows, graph.cols, graph.transpose_perm
    for key, val in (("x", x), ("y", y), ("w", w), ("g", g)):
        store[f"conv/{key}"] = val
    for mode, det in (("atomic", False), ("det", True)):
        conv = oeq.TensorProductConv(problem, deterministic=det)
        xt = torch.tensor(x, device="cuda", requires_grad=True)
        yt = torch.tensor(y, device="cuda", requires_grad=True)
        wt = torch.tensor(conv.reorder_weights_from_e3nn(w, True), device="cuda", requires_grad=True)
        r, c = torch.tensor(graph.rows, device="cuda"), torch.tensor(graph.cols, device="cuda")
        p = torch.tensor(graph.transpose_perm, device="cuda") if det else None
        z = conv(xt, yt, wt, r, c, p)
        z.backward(torch.tensor(g, device="cuda"))
        torch.cuda.synchronize()
        store[f"conv/{mode}/z"] = z.detach().cpu().numpy()
        store[f"conv/{mode}/dx"] = xt.grad.cpu().numpy()
        store[f"conv/{mode}/dy"] = yt.grad.cpu().numpy()
        store[f"conv/{mode}/dw"] = conv.reorder_weights_to_e3nn(wt.grad.cpu().numpy(), True)


def second_order_cases():
    """The benchmark signatures themselves (MACE-like channelwise 'uvu', NequIP-like fully connected shared-weight 'uvw') and a
    smaller channelwise problem, each with forward, backward and double backward."""
    from openequivariance.benchmark.problems import ChannelwiseTPP, FullyConnectedTPProblem
    feats = "128x0e+128x1o+128x2e+128x3o"
    ir = "32x0e+32x0o+32x1e+32x1o+32x2e+32x2o"
    return [("mace_like", ChannelwiseTPP(feats, "1x0e+1x1o+1x2e+1x3o", feats), 2),
            ("nequip_like", FullyConnectedTPProblem(ir, "1x0e+1x1o+1x2e", ir, shared_weights=True), 3),
            ("ctpp_32", ChannelwiseTPP("32x0e+32x1o+32x2e", "1x0e+1x1o+1x2e", "32x0e+32x1o+32x2e"), 4)]


def run_second_order(name, problem, batch, store):
    """z, (dx, dy, dw) for the cotangent g, and the gradients of <dx,x2> + <dy,y2> + <dw,w2> w.r.t. (x, y, w, g): what the
    reference's double-backward kernels return.  Weights and weight gradients are stored in e3nn order."""
    import openequivariance as oeq
    rng = np.random.default_rng(abs(hash(name)) % 1000 + 31)
    shared = problem.shared_weights
    wshape = (problem.weight_numel,) if shared else (batch, problem.weight_numel)
    draw = lambda *shape: rng.uniform(-1.0, 1.0, size=shape).astype(np.float32)  # noqa: E731
    x, x2 = draw(batch, problem.irreps_in1.dim), draw(batch, problem.irreps_in1.dim)
    y, y2 = draw(batch, problem.irreps_in2.dim), draw(batch, problem.irreps_in2.dim)
    w, w2 = draw(*wshape), draw(*wshape)
    g = draw(batch, problem.irreps_out.dim)
    tp = oeq.TensorProduct(problem)
    t = lambda a: torch.tensor(a, device="cuda", requires_grad=True)  # noqa: E731
    xt, yt, gt = t(x), t(y), t(g)
    wt = t(tp.reorder_weights_from_e3nn(w, not shared))
    w2t = torch.tensor(tp.reorder_weights_from_e3nn(w2, not shared), device="cuda")
    z = tp(xt, yt, wt)
    dx, dy, dw = torch.autograd.grad(z, [xt, yt, wt], gt, create_graph=True)
    scalar = (dx * torch.tensor(x2, device="cuda")).sum() + (dy * torch.tensor(y2, device="cuda")).sum() + (dw * w2t).sum()
    ddx, ddy, ddw, ddg = torch.autograd.grad(scalar, [xt, yt, wt, gt])
    torch.cuda.synchronize()
    back = lambda a: tp.reorder_weights_to_e3nn(a.detach().cpu().numpy(), not shared)  # noqa: E731
    for key, val in (("x", x), ("y", y), ("w", w), ("g", g), ("x2", x2), ("y2", y2), ("w2", w2), ("z", z.detach().cpu().numpy()),
                     ("dx", dx.detach().cpu().numpy()), ("dy", dy.detach().cpu().numpy()), ("dw", back(dw)),
                     ("ddx", ddx.cpu().numpy()), ("ddy", ddy.cpu().numpy()), ("ddw", back(ddw)), ("ddg", ddg.cpu().numpy())):
        store[f"tp2/{name}/{key}"] = val


def bench(n_nodes, steps):
    """Reference kernels on the benchmark workload (graph and inputs built with this repository's seeded generators)."""
    import openequivariance as oeq
    from openequivariance.benchmark.problems import ChannelwiseTPP
    import os
    os.environ["OEQ_NOTORCH"] = "1"   # import only this repository's torch-free core: both packages own the op namespace
    from openequivariance_b200.core.graph import periodic_radius_graph, spherical_harmonics
    feats = "128x0e+128x1o+128x2e+128x3o"
    problem = ChannelwiseTPP(feats, "1x0e+1x1o+1x2e+1x3o", feats)
    dev = torch.device("cuda", 0)
    g = periodic_radius_graph(n_nodes, mean_degree=32.0, cutoff=5.0, seed=0, device=dev)
    rows, cols, perm = g["rows"], g["cols"], g["transpose_perm"]
    E = rows.numel()
    Y = spherical_harmonics(3, g["vec"]).float().contiguous()
    gen = torch.Generator(device=dev).manual_seed(11)
    X = torch.randn(n_nodes, problem.irreps_in1.dim, device=dev, generator=gen)
    W = torch.randn(E, problem.weight_numel, device=dev, generator=gen)
    G = torch.randn(n_nodes, problem.irreps_out.dim, device=dev, generator=gen)
    ops = torch.ops.libtorch_tp_jit
    results = {}
    for mode, det in (("deterministic", True), ("atomic", False)):
        conv = oeq.TensorProductConv(problem, deterministic=det)
        p = perm if det else conv.dummy_transpose_perm
        if not det:
            shuffle = torch.randperm(E, device=dev)
            r, c, y, w = rows[shuffle].contiguous(), cols[shuffle].contiguous(), Y[shuffle].contiguous(), W
        else:
            r, c, y, w = rows, cols, Y, W

        def fwd():
            return ops.jit_conv_forward(conv.kernel, conv.hash, X, y, w, conv.L3_dim, r, c, conv.workspace_buffer, p)

        def bwd():
            return ops.jit_conv_backward(conv.kernel, conv.hash, X, y, w, G, r, c, conv.workspace_buffer, p)

        for _ in range(3):
            fwd(); bwd()
        torch.cuda.synchronize()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        tf, tb = [], []
        for _ in range(steps):
            ev[0].record(); fwd(); ev[1].record(); bwd(); ev[2].record()
            torch.cuda.synchronize()
            tf.append(ev[0].elapsed_time(ev[1])); tb.append(ev[1].elapsed_time(ev[2]))
        tf.sort(); tb.sort()
        results[mode] = {"forward_ms": tf[len(tf) // 2], "backward_ms": tb[len(tb) // 2],
                         "edges_per_s_fwd_bwd": E / ((tf[len(tf) // 2] + tb[len(tb) // 2]) * 1e-3)}
    results["nodes"], results["edges"] = n_nodes, E
    return results


def bench_tp(steps):
    """Reference kernels on the two batched tensor-product configurations (same shapes and input distributions as
    ``bench.py --workload tp_uvu / tp_uvw``): forward, backward, double backward, median of ``steps`` CUDA-event timings with
    a 256 MB buffer written between iterations."""
    import openequivariance as oeq
    from openequivariance.benchmark.problems import ChannelwiseTPP, FullyConnectedTPProblem
    dev = torch.device("cuda", 0)
    ops = torch.ops.libtorch_tp_jit
    flush = torch.empty(64 << 20, dtype=torch.float32, device=dev)
    feats = "128x0e+128x1o+128x2e+128x3o"
    ir = "32x0e+32x0o+32x1e+32x1o+32x2e+32x2o"
    cases = {
        "tp_uvu": (ChannelwiseTPP(feats, "1x0e+1x1o+1x2e+1x3o", feats), 200000),
        "tp_uvw": (FullyConnectedTPProblem(ir, "1x0e+1x1o+1x2e", ir, shared_weights=True, internal_weights=False), 50000),
    }
    out = {}
    for name, (problem, B) in cases.items():
        gen = torch.Generator(device=dev).manual_seed(5)
        mk = lambda *shape: torch.randn(*shape, device=dev, generator=gen)
        wshape = (problem.weight_numel,) if problem.shared_weights else (B, problem.weight_numel)
        X, Y, W = mk(B, problem.irreps_in1.dim), mk(B, problem.irreps_in2.dim), mk(*wshape)
        G, X2, Y2, W2 = mk(B, problem.irreps_out.dim), mk(B, problem.irreps_in1.dim), mk(B, problem.irreps_in2.dim), mk(*wshape)
        tp = oeq.TensorProduct(problem)
        passes = {
            "forward": lambda: ops.jit_tp_forward(tp.kernel, tp.hash, X, Y, W, tp.L3_dim),
            "backward": lambda: ops.jit_tp_backward(tp.kernel, tp.hash, X, Y, W, G),
            "double_backward": lambda: ops.jit_tp_double_backward(tp.kernel, tp.hash, X, Y, W, G, X2, Y2, W2),
        }
        res = {}
        for pname, fn in passes.items():
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            ts = []
            for _ in range(steps):
                flush.fill_(1.0)
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); r = fn(); b.record()
                torch.cuda.synchronize()
                del r
                ts.append(a.elapsed_time(b))
            ts.sort()
            res[pname + "_ms"] = ts[len(ts) // 2]
        res["batch"] = B
        out[name] = res
        del X, Y, W, G, X2, Y2, W2
        torch.cuda.empty_cache()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="out/reference_gpu.npz")
    ap.add_argument("--bench", action="store_true")
    ap.add_argument("--bench-tp", action="store_true", help="time the reference's batched tensor-product kernels only")
    ap.add_argument("--second-order", default="", help="also write the second-order fixtures (benchmark signatures) to this file")
    ap.add_argument("--nodes", type=int, default=50000)
    ap.add_argument("--steps", type=int, default=5)
    args = ap.parse_args()
    import openequivariance as oeq
    if not oeq.BUILT_EXTENSION:
        print(json.dumps({"reference": "unavailable", "why": str(oeq.BUILT_EXTENSION_ERROR)[:500]}))
        return 1
    if args.bench_tp:
        print(json.dumps({"reference_tp_on_gpu": bench_tp(args.steps)}))
        return 0
    store = {}
    for name, problem, batch in cases():
        run_tp(name, problem, batch, store)
    run_conv(store)
    import os
    os.makedirs(os.path.dirname(os.path.abspath(args.out)), exist_ok=True)
    np.savez_compressed(args.out, **{k.replace("/", "__"): v for k, v in store.items()})
    print("fixtures:", len(store), "arrays ->", args.out)
    if args.second_order:
        store2 = {}
        for name, problem, batch in second_order_cases():
            run_second_order(name, problem, batch, store2)
        np.savez_compressed(args.second_order, **{k.replace("/", "__"): v for k, v in store2.items()})
        print("second-order fixtures:", len(store2), "arrays ->", args.second_order)
    if args.bench:
        t0 = time.time()
        print(json.dumps({"reference_on_gpu": bench(args.nodes, args.steps), "wall_s": round(time.time() - t0, 1)}))
    return 0


if __name__ == "__main__":
    sys.exit(main())
