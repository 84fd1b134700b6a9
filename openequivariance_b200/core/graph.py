"""Graph-side inputs of the fused convolution: adjacency ordering, synthetic graphs, edge harmonics.

* ``CoordGraph`` reproduces the ordering contract of the reference's class of the same name
  (openequivariance/openequivariance/core/ConvolutionBase.py:57-82): edges sorted by (row, col)
  and ``transpose_perm[k]`` = position, in that order, of the k-th edge of the (col, row) order.
* ``periodic_radius_graph`` builds the seeded synthetic periodic point cloud that stands in for the
  molecular-graph pickles the reference downloads for its tests and benchmarks.
* ``spherical_harmonics`` generates component-normalised real harmonics in the same basis as
  ``wigner_3j`` by Clebsch-Gordan recursion (the reference has no harmonics code of its own; it
  takes them from e3nn).
"""

from __future__ import annotations

import math

import numpy as np
import torch

from .wigner import wigner_3j


def sort_edges(rows, cols):
    """Returns ``(order, transpose_perm)`` for index tensors/arrays ``rows, cols``: ``order`` sorts the
    edges by (row, col); ``transpose_perm`` lists, for the (col, row) order, positions in the sorted list."""
    if isinstance(rows, torch.Tensor):
        n = int(max(int(rows.max()), int(cols.max())) + 1) if rows.numel() else 1
        order = torch.argsort(rows.to(torch.int64) * n + cols.to(torch.int64), stable=True)
        r, c = rows[order], cols[order]
        perm = torch.argsort(c.to(torch.int64) * n + r.to(torch.int64), stable=True)
        return order, perm
    order = np.lexsort((cols, rows))
    r, c = rows[order], cols[order]
    perm = np.lexsort((r, c))
    return order, perm


def transpose_permutation(rows, cols):
    """For an edge list in ANY fixed order: positions of its edges listed in (col, row) order (stable)."""
    if isinstance(rows, torch.Tensor):
        n = int(max(int(rows.max()), int(cols.max())) + 1) if rows.numel() else 1
        return torch.argsort(cols.to(torch.int64) * n + rows.to(torch.int64), stable=True)
    return np.lexsort((rows, cols))


def prepare_graph(rows: torch.Tensor, cols: torch.Tensor, n_nodes: int):
    """Edge list in any order -> what the deterministic convolution needs, on the tensors' device and without a host
    synchronisation: ``rows, cols`` sorted by (row, col), ``transpose_perm`` (positions, in that order, of the edges listed
    by (col, row)) and ``order`` (the permutation that was applied, for re-ordering per-edge tensors such as ``Y`` and ``W``).

    Device counterpart of ``CoordGraph`` (``ConvolutionBase.py:57-82`` of the reference sorts a Python list).  CUDA
    tensors (int32 / int64) go through the library's own kernels (``oeqb_prepare_graph``: counting sort by node, then a
    rank-in-segment pass; stable for duplicate edges); CPU tensors take two stable key sorts, for host-side planning
    and tests.  Index dtype preserved."""
    assert rows.shape == cols.shape and rows.dim() == 1
    if rows.is_cuda:
        import ctypes

        from .. import native
        assert rows.dtype == cols.dtype and rows.dtype in (torch.int32, torch.int64), "index arrays must be int32 or int64"
        lib = native.load()
        E = int(rows.numel())
        r_in, c_in = rows.contiguous(), cols.contiguous()
        out = {k: torch.empty_like(r_in) for k in ("rows", "cols", "transpose_perm", "order")}
        if E == 0:
            return out
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731
        with torch.cuda.device(rows.device):
            need = int(lib.oeqb_graph_workspace_bytes(n_nodes, E))
            ws = torch.empty(max(need, 1), dtype=torch.uint8, device=rows.device)
            rc = lib.oeqb_prepare_graph(3 if rows.dtype == torch.int32 else 4, n_nodes, E, ptr(r_in), ptr(c_in),
                                        ptr(out["rows"]), ptr(out["cols"]), ptr(out["order"]), ptr(out["transpose_perm"]),
                                        ptr(ws), need, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        native.check(rc, "oeqb_prepare_graph")
        return out
    r64, c64 = rows.to(torch.int64), cols.to(torch.int64)
    order = torch.argsort(r64 * n_nodes + c64, stable=True)
    r, c = r64[order], c64[order]
    perm = torch.argsort(c * n_nodes + r, stable=True)
    return {"rows": r.to(rows.dtype), "cols": c.to(cols.dtype), "transpose_perm": perm.to(rows.dtype), "order": order}


class CoordGraph:
    """Adjacency of a point cloud, row-major sorted, with the permutation to column-major order.

    ``rows[i]`` is the receiver and ``cols[i]`` the sender of edge ``i``; ``nnz`` counts directed edges."""

    def __init__(self, coords, rows, cols, name):
        assert len(rows) == len(cols)
        self.nnz = len(rows)
        self.node_count = coords.shape[0]
        self.coords = coords
        self.name = name
        rows, cols = np.asarray(rows), np.asarray(cols)
        order, perm = sort_edges(rows, cols)
        self.edge_order = order
        self.rows = rows[order]
        self.cols = cols[order]
        self.transpose_perm = perm.astype(self.rows.dtype)


def box_length(n_nodes: int, mean_degree: float, cutoff: float) -> float:
    """Edge of the periodic cube in which ``n_nodes`` uniform points have ``mean_degree`` neighbours within ``cutoff``."""
    return (n_nodes * (4.0 / 3.0) * math.pi * cutoff**3 / mean_degree) ** (1.0 / 3.0)


def periodic_radius_graph(n_nodes: int, mean_degree: float = 32.0, cutoff: float = 5.0, seed: int = 0,
                          device="cpu"):
    """Seeded uniform points in a periodic cube, neighbours within ``cutoff`` under the minimum-image rule.

    Nodes are numbered in cell order (x-slab major), so contiguous node ranges are spatial slabs.
    Returns ``dict(pos [N,3] f64, rows [E], cols [E] int64 sorted by (row, col), vec [E,3] f64 = pos[col]-pos[row]
    (minimum image), transpose_perm [E], box)``.  The edge set is symmetric: (i, j) present iff (j, i) present.
    """
    box = box_length(n_nodes, mean_degree, cutoff)
    gen = torch.Generator(device="cpu").manual_seed(seed)
    pos = (torch.rand(n_nodes, 3, generator=gen, dtype=torch.float64) * box).to(device)
    ncell = int(box // cutoff)
    if ncell < 3:
        # tiny boxes: all pairs
        i = torch.arange(n_nodes, device=device).repeat_interleave(n_nodes)
        j = torch.arange(n_nodes, device=device).repeat(n_nodes)
    else:
        cs = box / ncell
        cc = torch.clamp((pos / cs).floor().to(torch.int64), 0, ncell - 1)
        cid = (cc[:, 0] * ncell + cc[:, 1]) * ncell + cc[:, 2]
        order0 = torch.argsort(cid, stable=True)
        pos, cc, cid = pos[order0], cc[order0], cid[order0]
        counts = torch.bincount(cid, minlength=ncell**3)
        starts = torch.cumsum(counts, 0) - counts
        me = torch.arange(n_nodes, device=device)
        i_parts, j_parts = [], []
        for dx in (-1, 0, 1):
            for dy in (-1, 0, 1):
                for dz in (-1, 0, 1):
                    off = torch.tensor([dx, dy, dz], device=device)
                    nb = (cc + off) % ncell
                    nid = (nb[:, 0] * ncell + nb[:, 1]) * ncell + nb[:, 2]
                    cnt = counts[nid]
                    ii = me.repeat_interleave(cnt)
                    first = torch.cumsum(cnt, 0) - cnt
                    local = torch.arange(ii.numel(), device=device) - first.repeat_interleave(cnt)
                    i_parts.append(ii)
                    j_parts.append(starts[nid].repeat_interleave(cnt) + local)
        i, j = torch.cat(i_parts), torch.cat(j_parts)
    d = pos[j] - pos[i]
    d = d - box * torch.round(d / box)
    keep = (d.square().sum(1) < cutoff * cutoff) & (i != j)
    i, j, d = i[keep], j[keep], d[keep]
    order, perm = sort_edges(i, j)
    return {"pos": pos, "rows": i[order].contiguous(), "cols": j[order].contiguous(), "vec": d[order].contiguous(),
            "transpose_perm": perm.contiguous(), "box": box, "n_nodes": n_nodes}


def spherical_harmonics(lmax: int, vectors: torch.Tensor, normalize: bool = True) -> torch.Tensor:
    """Real harmonics ``[n, (lmax+1)^2]`` of ``vectors [n,3]``, block l scaled so that its squared norm is 2l+1
    on unit vectors ("component" normalisation).  ``Y_1 = sqrt(3) (y, z, x)``; higher degrees come from
    ``Y_{l+1} ~ C(l,1,l+1) Y_l Y_1``, which fixes the basis to the one of ``wigner_3j``."""
    v = vectors.to(torch.float64)
    if normalize:
        v = v / v.norm(dim=1, keepdim=True)
    y1 = math.sqrt(3.0) * torch.stack([v[:, 1], v[:, 2], v[:, 0]], dim=1)
    blocks = [torch.ones(v.shape[0], 1, dtype=torch.float64, device=v.device)]
    if lmax >= 1:
        blocks.append(y1)
    for l in range(1, lmax):
        c = torch.as_tensor(wigner_3j(l, 1, l + 1), device=v.device)
        blocks.append(torch.einsum("ijk,ni,nj->nk", c, blocks[l], y1) * _recursion_scale(l))
    return torch.cat(blocks[: lmax + 1], dim=1)


_SCALE_CACHE = {}


def _recursion_scale(l: int) -> float:
    """Factor s_l with ``Y_{l+1} = s_l * C(l,1,l+1) Y_l Y_1`` having squared norm 2l+3 on unit vectors.

    Found numerically once per degree on a fixed unit vector; the ratio is direction independent because both
    sides are harmonic polynomials of degree l+1 transforming in the same irrep."""
    if l in _SCALE_CACHE:
        return _SCALE_CACHE[l]
    v = np.array([0.3, -0.5, 0.7])
    v = v / np.linalg.norm(v)
    y1 = math.sqrt(3.0) * np.array([v[1], v[2], v[0]])
    ys = [np.ones(1), y1]
    for m in range(1, l + 1):
        c = wigner_3j(m, 1, m + 1)
        raw = np.einsum("ijk,i,j->k", c, ys[m], y1)
        s = math.sqrt((2 * m + 3) / float(raw @ raw))
        _SCALE_CACHE[m] = s
        ys.append(raw * s)
    return _SCALE_CACHE[l]
