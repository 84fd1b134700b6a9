"""Receiver-partitioned fused convolution across the GPUs of one node.

The reference has no multi-GPU code (its only multi-device test runs independent replicas,
tests/multidevice_test.py:7-57); this module is the partitioned deterministic convolution the benchmark
configuration asks for.

Partition.  Nodes are numbered in spatial (x-slab major) order, so rank ``r`` of ``P`` owns the contiguous receiver
range ``[N*r/P, N*(r+1)/P)`` and, the edge list being receiver-sorted, a contiguous range of edges with their ``Y``,
``W``, ``dY``, ``dW``.  Senders outside the range are the rank's *halo*; they are appended after the owned nodes in the
rank's local numbering, grouped by owner.

Forward.  The rows ``X[halo]`` are fetched from their owners with one grouped send/recv (NCCL over NVLink) on a side
stream while the kernel runs on the *interior* receivers (a contiguous middle range none of whose edges has a halo
sender); the two boundary ranges follow once the halo has landed in local memory.  Every receiver's edges stay in list
order, so ``Z`` is bit-identical to the single-GPU result for any ``P``.

Backward.  ``dY``/``dW`` are local.  ``dX`` is computed for the local numbering; the halo part is sent back to the
owners and added there in rank order.  It is reproducible run to run for a given ``P``; for boundary senders the
association of the floating-point sum differs from the single-GPU one (partials per rank), for all others it is
bit-identical.

Remote rows always land in this GPU's own memory before a kernel reads them; no kernel here reads peer memory.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

from .core.graph import transpose_permutation


def require_fp32_int64(conv, *index_tensors):
    """The partitioned and the streamed drivers allocate fp32 buffers and compute byte offsets for fp32 rows and int64
    indices.  A convolution of another precision, or 32-bit index arrays, would make the kernels read those buffers
    past their end, so both are refused here, before anything is launched."""
    import numpy as np
    dt = np.dtype(conv.config.irrep_dtype)
    if dt != np.dtype(np.float32) or np.dtype(conv.config.weight_dtype) != np.dtype(np.float32):
        raise TypeError(f"partitioned / streamed convolution supports float32 problems only, got {dt}")
    for t in index_tensors:
        if t is not None and t.dtype != torch.int64:
            raise TypeError(f"partitioned / streamed convolution needs int64 index arrays, got {t.dtype}")


def owner_range(n_nodes: int, world: int, rank: int):
    return (n_nodes * rank) // world, (n_nodes * (rank + 1)) // world


@dataclass
class PartitionPlan:
    """Everything rank ``rank`` needs to run its share of a convolution over a globally sorted edge list."""

    rank: int
    world: int
    n_nodes: int
    n0: int
    n1: int
    e0: int
    e1: int
    halo_ids: torch.Tensor                 # global ids of halo senders, ascending (hence grouped by owner)
    recv_counts: List[int]                 # halo rows owned by each peer
    send_ids: List[torch.Tensor]           # per peer: local indices of owned rows that peer needs (ascending)
    rows_local: torch.Tensor               # receiver of each local edge, relative to n0
    cols_local: torch.Tensor               # sender of each local edge in local numbering (owned first, then halo)
    perm_local: torch.Tensor               # sender-major order of the local edges
    interior: tuple = (0, 0)               # receiver sub-range [a, b) (local) whose edges have no halo sender
    interior_edges: tuple = (0, 0)         # matching edge sub-range [ea, eb) (local)
    rows_mid: Optional[torch.Tensor] = None    # rows_local[ea:eb] - a
    rows_right: Optional[torch.Tensor] = None  # rows_local[eb:] - b

    @property
    def n_owned(self) -> int:
        return self.n1 - self.n0

    @property
    def n_halo(self) -> int:
        return int(self.halo_ids.numel())

    @property
    def n_local_edges(self) -> int:
        return self.e1 - self.e0


def _halo_of(rows, cols, n_nodes, world, q):
    n0, n1 = owner_range(n_nodes, world, q)
    e0 = int(torch.searchsorted(rows, torch.tensor(n0, device=rows.device, dtype=rows.dtype)))
    e1 = int(torch.searchsorted(rows, torch.tensor(n1, device=rows.device, dtype=rows.dtype)))
    c = cols[e0:e1]
    outside = c[(c < n0) | (c >= n1)]
    return n0, n1, e0, e1, torch.unique(outside)


def plan_on_device(rows: torch.Tensor, cols: torch.Tensor, n_nodes: int, recv: tuple, own: tuple, bounds: List[int], rank: int):
    """The library's planning kernels (``oeqb_plan_count`` / ``oeqb_plan_fill``) for the holder of receivers ``recv`` who
    owns the sender rows ``own`` (may be empty).  One host synchronisation (the sizes of the lists).  Returns a dict with
    ``e0, e1, a, b, ea, eb, recv_counts, send_counts`` (Python ints / lists) and the tensors ``halo_ids, send_ids``
    (concatenated by owner), ``rows_local, cols_local, perm_local``."""
    import ctypes

    from . import native
    assert rows.is_cuda and rows.dtype == torch.int64 and cols.dtype == torch.int64
    lib, dev = native.load(), rows.device
    rows, cols = rows.contiguous(), cols.contiguous()
    E, world = int(rows.numel()), len(bounds) - 1
    args = (n_nodes, E, ctypes.c_void_p(rows.data_ptr()), ctypes.c_void_p(cols.data_ptr()), recv[0], recv[1], own[0], own[1], world)
    barr = (ctypes.c_int64 * (world + 1))(*bounds)
    with torch.cuda.device(dev):
        st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        need = int(lib.oeqb_plan_workspace_bytes(n_nodes, E, recv[1] - recv[0], own[1] - own[0], world))
        ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
        counts = torch.empty(8 + 2 * world, dtype=torch.int64, device=dev)
        native.check(lib.oeqb_plan_count(*args, rank, barr, ctypes.c_void_p(ws.data_ptr()), need, ctypes.c_void_p(counts.data_ptr()), st),
                     "oeqb_plan_count")
        c = counts.tolist()                                   # the one synchronisation
        e0, e1, n_halo = c[0], c[1], c[2]
        send_counts = c[8 + world:8 + 2 * world]
        i64 = dict(dtype=torch.int64, device=dev)
        halo = torch.empty(n_halo, **i64)
        send = torch.empty(sum(send_counts), **i64)
        rl, cl, pl = (torch.empty(e1 - e0, **i64) for _ in range(3))
        p = lambda t: ctypes.c_void_p(t.data_ptr() if t.numel() else 0)
        native.check(lib.oeqb_plan_fill(*args, barr, e0, e1, n_halo, ctypes.c_void_p(ws.data_ptr()), need, p(halo), p(send), p(rl), p(cl),
                                        p(pl), st), "oeqb_plan_fill")
    return dict(e0=e0, e1=e1, a=c[3], b=c[4], ea=c[5], eb=c[6], recv_counts=c[8:8 + world], send_counts=send_counts, halo_ids=halo,
                send_ids=send, rows_local=rl, cols_local=cl, perm_local=pl)


def build_plan(rows: torch.Tensor, cols: torch.Tensor, n_nodes: int, world: int, rank: int) -> PartitionPlan:
    """Pure index arithmetic on the global, (row, col)-sorted edge list; needs no communication because every rank
    holds the same global ``rows`` / ``cols`` (built from the same seed or broadcast by the caller).  CUDA int64 lists are
    planned by the library's kernels (one pass over the edges, one host synchronisation); CPU lists (host-side tests) by
    the torch restatement below, which is also what the device plan is tested against."""
    if rows.is_cuda and rows.dtype == torch.int64:
        n0, n1 = owner_range(n_nodes, world, rank)
        bounds = [owner_range(n_nodes, world, q)[0] for q in range(world)] + [n_nodes]
        d = plan_on_device(rows, cols, n_nodes, (n0, n1), (n0, n1), bounds, rank)
        send_ids = list(torch.split(d["send_ids"], d["send_counts"]))
        rl, a, b, ea, eb = d["rows_local"], d["a"], d["b"], d["ea"], d["eb"]
        return PartitionPlan(rank=rank, world=world, n_nodes=n_nodes, n0=n0, n1=n1, e0=d["e0"], e1=d["e1"], halo_ids=d["halo_ids"],
                             recv_counts=d["recv_counts"], send_ids=send_ids, rows_local=rl, cols_local=d["cols_local"],
                             perm_local=d["perm_local"], interior=(a, b), interior_edges=(ea, eb),
                             rows_mid=(rl[ea:eb] - a).contiguous(), rows_right=(rl[eb:] - b).contiguous())
    n0, n1, e0, e1, halo = _halo_of(rows, cols, n_nodes, world, rank)
    dev = rows.device
    bounds = torch.tensor([owner_range(n_nodes, world, q)[0] for q in range(world)] + [n_nodes], device=dev)
    owner_of_halo = torch.bucketize(halo, bounds, right=True) - 1
    recv_counts = [int((owner_of_halo == q).sum()) for q in range(world)]
    send_ids = []
    for q in range(world):
        if q == rank:
            send_ids.append(torch.zeros(0, dtype=torch.int64, device=dev))
            continue
        halo_q = _halo_of(rows, cols, n_nodes, world, q)[4]
        mine = halo_q[(halo_q >= n0) & (halo_q < n1)]
        send_ids.append((mine - n0).to(torch.int64))
    c = cols[e0:e1]
    owned = (c >= n0) & (c < n1)
    cols_local = torch.where(owned, c - n0, (n1 - n0) + torch.searchsorted(halo, c))
    rows_local = (rows[e0:e1] - n0).contiguous()
    # the local list keeps the global (row, global col) order, which is not sorted by local col inside a row:
    # take the sender-major permutation of the list as it stands
    perm_local = transpose_permutation(rows_local, cols_local)
    # interior receivers: the longest middle run without any boundary receiver on either side of the split point
    n_owned = n1 - n0
    boundary_rows = torch.unique(rows_local[~owned])
    a, b = 0, n_owned
    if boundary_rows.numel() > 0:
        half = n_owned // 2
        left = boundary_rows[boundary_rows < half]
        right = boundary_rows[boundary_rows >= half]
        a = int(left.max()) + 1 if left.numel() else 0
        b = int(right.min()) if right.numel() else n_owned
    ea = int(torch.searchsorted(rows_local, torch.tensor(a, device=dev, dtype=rows_local.dtype)))
    eb = int(torch.searchsorted(rows_local, torch.tensor(b, device=dev, dtype=rows_local.dtype)))
    return PartitionPlan(rank=rank, world=world, n_nodes=n_nodes, n0=n0, n1=n1, e0=e0, e1=e1, halo_ids=halo,
                         recv_counts=recv_counts, send_ids=send_ids, rows_local=rows_local,
                         cols_local=cols_local.contiguous(), perm_local=perm_local.contiguous(), interior=(a, b),
                         interior_edges=(ea, eb), rows_mid=(rows_local[ea:eb] - a).contiguous(),
                         rows_right=(rows_local[eb:] - b).contiguous())


# ---------------------------------------------------------------------------------------------- halo exchange

def exchange_halo(plan: PartitionPlan, x_local: torch.Tensor, group=None):
    """Fills ``x_local[n_owned:]`` with the halo rows from their owners (grouped send/recv).  Returns the send
    buffers, which must stay alive until the caller has synchronised with the stream this ran on."""
    if plan.world == 1 or (plan.n_halo == 0 and all(s.numel() == 0 for s in plan.send_ids)):
        return []
    ops, keep = [], []
    offset = plan.n_owned
    for q in range(plan.world):
        cnt = plan.recv_counts[q]
        if q != plan.rank and cnt > 0:
            ops.append(dist.P2POp(dist.irecv, x_local[offset:offset + cnt], q, group=group))
        offset += cnt
    for q in range(plan.world):
        ids = plan.send_ids[q]
        if q != plan.rank and ids.numel() > 0:
            buf = x_local.index_select(0, ids)
            keep.append(buf)
            ops.append(dist.P2POp(dist.isend, buf, q, group=group))
    if ops:
        for work in dist.batch_isend_irecv(ops):
            work.wait()
    return keep


def send_halo_gradients(plan: PartitionPlan, dx_local: torch.Tensor, group=None):
    """First half of ``return_halo_gradients``: sends the halo part of ``dx_local`` to the owners and receives what the
    peers computed for this rank's rows.  Returns ``{peer: rows}`` for ``add_halo_gradients``.  Runs on the current
    stream, so a caller can put it on a side stream once the halo rows of ``dx_local`` are final and keep computing."""
    if plan.world == 1:
        return {}
    ops, recv_bufs = [], {}
    for q in range(plan.world):
        ids = plan.send_ids[q]
        if q != plan.rank and ids.numel() > 0:
            recv_bufs[q] = torch.empty((ids.numel(), dx_local.shape[1]), dtype=dx_local.dtype, device=dx_local.device)
            ops.append(dist.P2POp(dist.irecv, recv_bufs[q], q, group=group))
    offset = plan.n_owned
    for q in range(plan.world):
        cnt = plan.recv_counts[q]
        if q != plan.rank and cnt > 0:
            ops.append(dist.P2POp(dist.isend, dx_local[offset:offset + cnt], q, group=group))
        offset += cnt
    if ops:
        for work in dist.batch_isend_irecv(ops):
            work.wait()
    return recv_bufs


def add_halo_gradients(plan: PartitionPlan, dx_local: torch.Tensor, recv_bufs) -> torch.Tensor:
    """Second half: adds the received rows into the owned part, peer by peer in rank order (each peer's row list has
    unique targets, so the result does not depend on timing)."""
    dx_owned = dx_local[:plan.n_owned]
    for q in sorted(recv_bufs):
        dx_owned.index_add_(0, plan.send_ids[q], recv_bufs[q])
    return dx_owned


def return_halo_gradients(plan: PartitionPlan, dx_local: torch.Tensor, group=None) -> torch.Tensor:
    """Sends the halo part of ``dx_local`` back to the owners and adds what arrives into the owned part, peer by
    peer in rank order."""
    return add_halo_gradients(plan, dx_local, send_halo_gradients(plan, dx_local, group))


# ---------------------------------------------------------------------------------------------- GPU execution

class PartitionedConv:
    """One rank's share of a deterministic ``TensorProductConv`` over a partitioned graph.

    ``forward(x_owned, Y, W)`` / ``backward(G)`` work on the rank's owned receivers and local edges; ``Y``, ``W`` are
    the rows of the global per-edge tensors for edges ``[plan.e0, plan.e1)``."""

    def __init__(self, conv, plan: PartitionPlan, device, group=None, exchange: Optional[Callable] = None,
                 give_back: Optional[Callable] = None):
        """``exchange(plan, x_local)`` / ``give_back(plan, dx_local)`` replace the NCCL halo traffic (used by the
        single-GPU emulation test, which plays all ranks in one process)."""
        from . import native
        assert conv.deterministic, "the partitioned convolution is built on the deterministic kernels"
        require_fp32_int64(conv, plan.rows_local, plan.cols_local, plan.perm_local)
        self.conv, self.plan, self.device, self.group = conv, plan, device, group
        self._exchange = exchange or (lambda pl, x: exchange_halo(pl, x, group))
        self._give_back = give_back or (lambda pl, dx: return_halo_gradients(pl, dx, group))
        self.lib = native.load()
        self.native = native
        self.desc = conv.kernel_string.encode()
        self.key = conv.hash
        p = plan
        self.L1, self.L2, self.L3, self.wn = conv.L1.dim, conv.L2.dim, conv.L3.dim, conv.weight_numel
        self.x_local = torch.empty((p.n_owned + p.n_halo, self.L1), dtype=torch.float32, device=device)
        self.comm_stream = torch.cuda.Stream(device=device)
        need = self.lib.oeqb_conv_workspace_bytes(self.desc, len(self.desc), self.key, 1, p.n_owned + p.n_halo, p.n_local_edges)
        self.workspace = torch.empty(max(int(need), 1), dtype=torch.uint8, device=device)
        self._keep = []
        # the two-step backward (halo rows of dX first, their transfer overlapped with the owned rows) needs the
        # channel-parallel deterministic kernels; other problems take the single call
        self.split_backward = native.query(self.desc, self.key).fast_path == 1 and exchange is None and give_back is None

    @staticmethod
    def _p(t, byte_offset=0):
        return ctypes.c_void_p(t.data_ptr() + byte_offset)

    def _forward_range(self, Y, W, Z, recv_lo, recv_hi, e_lo, e_hi, rows_rel, stream):
        """Receivers [recv_lo, recv_hi) (local), edges [e_lo, e_hi) (local), written into Z[recv_lo:recv_hi]."""
        if recv_hi <= recv_lo:
            return
        p = self.plan
        n_e = e_hi - e_lo
        rc = self.lib.oeqb_conv_forward_rect(
            self.desc, len(self.desc), self.key, recv_hi - recv_lo, p.n_owned + p.n_halo, n_e,
            self._p(self.x_local), self._p(Y, e_lo * self.L2 * 4), self._p(W, e_lo * self.wn * 4),
            self._p(Z, recv_lo * self.L3 * 4), self._p(rows_rel), self._p(p.cols_local, e_lo * 8),
            self._p(p.perm_local), self._p(self.workspace), self.workspace.numel(), ctypes.c_void_p(stream.cuda_stream))
        self.native.check(rc, "partitioned conv forward")

    def forward(self, x_owned: Optional[torch.Tensor], Y: torch.Tensor, W: torch.Tensor) -> torch.Tensor:
        """``x_owned`` may be ``None`` when the caller has already written ``self.x_local[:n_owned]``."""
        p = self.plan
        main = torch.cuda.current_stream(self.device)
        if x_owned is not None:
            self.x_local[:p.n_owned].copy_(x_owned)
        Z = torch.empty((p.n_owned, self.L3), dtype=torch.float32, device=self.device)
        # halo rows travel on the side stream while the interior receivers are computed
        self.comm_stream.wait_stream(main)
        with torch.cuda.stream(self.comm_stream):
            self._keep = self._exchange(p, self.x_local)
        a, b = p.interior
        ea, eb = p.interior_edges
        self._forward_range(Y, W, Z, a, b, ea, eb, p.rows_mid, main)
        main.wait_stream(self.comm_stream)
        self._forward_range(Y, W, Z, 0, a, 0, ea, p.rows_local, main)
        self._forward_range(Y, W, Z, b, p.n_owned, eb, p.n_local_edges, p.rows_right, main)
        self.saved = (Y, W)
        return Z

    def backward(self, G: torch.Tensor):
        """Returns ``(dX_owned, dY, dW)`` for the cotangent ``G [n_owned, L3]`` of the last ``forward``."""
        p = self.plan
        Y, W = self.saved
        n_loc = p.n_owned + p.n_halo
        # the kernel indexes G by local receiver, which is always < n_owned: no padding rows are needed
        dx_local = torch.empty((n_loc, self.L1), dtype=torch.float32, device=self.device)
        dY, dW = torch.empty_like(Y), torch.empty_like(W)
        main = torch.cuda.current_stream(self.device)
        st = ctypes.c_void_p(main.cuda_stream)
        if self.split_backward and p.world > 1 and p.n_local_edges > 0 and p.n_halo > 0:
            # per-edge pass, then the halo rows of dX (the last n_halo local rows); they travel to their owners on the side
            # stream while the owned rows are summed; the owners add what arrived at the end, in rank order
            rc = self.lib.oeqb_conv_backward_edges(
                self.desc, len(self.desc), self.key, p.n_owned, n_loc, p.n_local_edges, self._p(self.x_local), self._p(Y),
                self._p(W), self._p(G), self._p(dY), self._p(dW), self._p(p.rows_local), self._p(p.cols_local),
                self._p(p.perm_local), self._p(self.workspace), self.workspace.numel(), st)
            self.native.check(rc, "partitioned conv backward (edges)")
            rc = self.lib.oeqb_conv_backward_rows(self.desc, len(self.desc), self.key, n_loc, p.n_local_edges, p.n_owned, n_loc,
                                                  self._p(p.perm_local), self._p(self.workspace), self.workspace.numel(),
                                                  self._p(dx_local), st)
            self.native.check(rc, "partitioned conv backward (halo rows)")
            self.comm_stream.wait_stream(main)
            with torch.cuda.stream(self.comm_stream):
                received = send_halo_gradients(p, dx_local, self.group)
            rc = self.lib.oeqb_conv_backward_rows(self.desc, len(self.desc), self.key, n_loc, p.n_local_edges, 0, p.n_owned,
                                                  self._p(p.perm_local), self._p(self.workspace), self.workspace.numel(),
                                                  self._p(dx_local), st)
            self.native.check(rc, "partitioned conv backward (owned rows)")
            main.wait_stream(self.comm_stream)
            return add_halo_gradients(p, dx_local, received), dY, dW
        rc = self.lib.oeqb_conv_backward_rect(
            self.desc, len(self.desc), self.key, p.n_owned, n_loc, p.n_local_edges, self._p(self.x_local), self._p(Y), self._p(W),
            self._p(G), self._p(dx_local), self._p(dY), self._p(dW), self._p(p.rows_local), self._p(p.cols_local),
            self._p(p.perm_local), self._p(self.workspace), self.workspace.numel(), st)
        self.native.check(rc, "partitioned conv backward")
        dX = self._give_back(p, dx_local)
        return dX, dY, dW
