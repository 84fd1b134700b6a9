"""Fused convolution over graphs whose per-edge tensors do not fit in device memory.

The largest benchmark configuration of the reference's conv suite (2,000,000 nodes, ~64M edges; its graphs come from
``benchmark/problems.py`` / ``tests/benchmark.py:366-420``) has 754 GB of per-edge weights in fp32.  The reference keeps
all operands resident and cannot run it; this driver walks the receivers in contiguous chunks and hands each chunk to
the deterministic kernels:

* chunk ``c`` owns receivers ``[n0, n1)`` and, the edge list being receiver-sorted, the contiguous edges ``[e0, e1)``;
* its senders are renumbered ``0..S-1`` (sorted unique sender ids), their rows gathered into a small ``X`` block, and the
  sender-major permutation of the chunk's edges is built once (``plan``);
* per step and chunk: the caller's ``weights(c, out)`` fills the chunk's weight rows (generated, loaded, ...), the
  forward kernel writes ``Z[n0:n1]``, the caller's ``cotangent(c, Z_c)`` returns ``dL/dZ`` for the chunk, the backward
  kernels write ``dY``, ``dW`` of the chunk and a dense ``dX`` block that is added to the global ``dX`` rows of the
  chunk's senders.  Chunks run in order, so the result is reproducible; ``Z``, ``dY``, ``dW`` are bit-identical to a
  single resident call, ``dX`` differs only in the association of the per-sender sum (one partial per chunk).

Only the loss must be separable over receivers (each chunk's cotangent is available right after its forward), which
holds for the benchmark's loss and for any per-node readout.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass
from typing import Callable, List, Optional

import torch

from .core.graph import transpose_permutation


@dataclass
class ChunkPlan:
    n0: int
    n1: int
    e0: int
    e1: int
    senders: torch.Tensor      # [S] global ids of the chunk's senders, ascending
    rows_local: torch.Tensor   # [e1-e0] receiver - n0
    cols_local: torch.Tensor   # [e1-e0] index into ``senders``
    perm_local: torch.Tensor   # [e1-e0] sender-major order of the chunk's edges


def plan_chunks(rows: torch.Tensor, cols: torch.Tensor, n_receivers: int, chunk_nodes: int) -> List[ChunkPlan]:
    """``rows`` sorted ascending (ties in any fixed order), values < ``n_receivers``; ``cols`` any node ids."""
    assert chunk_nodes > 0
    plans = []
    bounds = list(range(0, n_receivers, chunk_nodes)) + [n_receivers]
    if rows.is_cuda and rows.dtype == torch.int64 and cols.dtype == torch.int64:
        # the library's planning kernels: per chunk one pass over the edges and one host synchronisation (the list sizes)
        from .partition import plan_on_device
        n_nodes = max(n_receivers, int(cols.max()) + 1 if cols.numel() else 0)
        for n0, n1 in zip(bounds[:-1], bounds[1:]):
            d = plan_on_device(rows, cols, n_nodes, (n0, n1), (0, 0), [0, n_nodes], 0)
            plans.append(ChunkPlan(n0, n1, d["e0"], d["e1"], d["halo_ids"], d["rows_local"], d["cols_local"], d["perm_local"]))
        return plans
    cuts = torch.searchsorted(rows, torch.tensor(bounds, device=rows.device, dtype=rows.dtype)).tolist()
    for (n0, n1), (e0, e1) in zip(zip(bounds[:-1], bounds[1:]), zip(cuts[:-1], cuts[1:])):
        c = cols[e0:e1]
        senders = torch.unique(c)                       # sorted
        cols_local = torch.searchsorted(senders, c)
        rows_local = rows[e0:e1] - n0
        perm = transpose_permutation(rows_local, cols_local) if e1 > e0 else cols_local.clone()
        plans.append(ChunkPlan(n0, n1, e0, e1, senders, rows_local.contiguous(), cols_local.contiguous(),
                               perm.to(rows.dtype).contiguous()))
    return plans


class StreamedConv:
    """Deterministic ``TensorProductConv`` run chunk by chunk (see the module docstring)."""

    def __init__(self, conv, rows: torch.Tensor, cols: torch.Tensor, n_receivers: int, chunk_nodes: int, device):
        from . import native
        from .partition import require_fp32_int64
        assert conv.deterministic, "the streamed convolution is built on the deterministic kernels"
        require_fp32_int64(conv, rows, cols)
        self.native, self.lib = native, native.load()
        self.desc, self.key = conv.kernel_string.encode(), conv.hash
        self.L1, self.L2, self.L3, self.wn = conv.L1.dim, conv.L2.dim, conv.L3.dim, conv.weight_numel
        self.device = device
        self.n_receivers = n_receivers
        self.plans = plan_chunks(rows, cols, n_receivers, chunk_nodes)
        self.max_edges = max((p.e1 - p.e0 for p in self.plans), default=0)
        self.max_senders = max((int(p.senders.numel()) for p in self.plans), default=0)
        self.max_receivers = max((p.n1 - p.n0 for p in self.plans), default=0)
        f32 = dict(dtype=torch.float32, device=device)
        # buffers shared by all chunks
        self.W = torch.empty((max(self.max_edges, 1), self.wn), **f32)
        self.dW = torch.empty_like(self.W)
        self.x_block = torch.empty((max(self.max_senders, 1), self.L1), **f32)
        self.dx_block = torch.empty_like(self.x_block)
        self.Z = torch.empty((max(self.max_receivers, 1), self.L3), **f32)
        need = 1
        for p in self.plans:
            if p.e1 > p.e0:
                need = max(need, int(self.lib.oeqb_conv_workspace_bytes(self.desc, len(self.desc), self.key, 1,
                                                                         int(p.senders.numel()), p.e1 - p.e0)))
        self.workspace = torch.empty(need, dtype=torch.uint8, device=device)

    @staticmethod
    def _p(t, byte_offset=0):
        return ctypes.c_void_p(t.data_ptr() + byte_offset)

    def chunks_touching(self, first_row: int) -> List[int]:
        """Chunks one of whose senders has an id >= ``first_row`` (with ``first_row`` = the number of owned rows of a
        partitioned graph: the chunks that read halo rows and write halo gradients).  One host synchronisation."""
        tops = torch.stack([p.senders[-1] if p.senders.numel() else p.senders.new_tensor(-1) for p in self.plans])
        return [c for c, top in enumerate(tops.tolist()) if top >= first_row]

    def step(self, X: torch.Tensor, Y: torch.Tensor, weights: Callable, cotangent: Callable, dX: torch.Tensor,
             dY: Optional[torch.Tensor] = None, on_chunk: Optional[Callable] = None, order: Optional[List[int]] = None,
             before_chunk: Optional[Callable] = None, after_chunk: Optional[Callable] = None):
        """One forward + backward pass over all chunks.

        ``X [n_nodes, L1]``, ``Y [E, L2]`` resident; ``weights(c, W_c)`` fills ``W_c [E_c, wn]``; ``cotangent(c, Z_c)``
        returns ``G_c`` (may alias ``Z_c``); ``dX [n_nodes, L1]`` is zeroed here and accumulated; ``dY [E, L2]``
        optional.  ``on_chunk(c, plan, Z_c, dW_c)`` sees each chunk's outputs before the buffers are reused.
        ``order`` lists the chunks in the order to run them (default: ascending; any fixed order gives reproducible
        results, the association of the per-sender sums in ``dX`` follows it); ``before_chunk(c)`` / ``after_chunk(c)``
        run on the host around each chunk's launches (a partitioned caller waits for halo rows / starts sending halo
        gradients there)."""
        st = ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)
        dX.zero_()
        for c in (range(len(self.plans)) if order is None else order):
            p = self.plans[c]
            n_e, n_r, n_s = p.e1 - p.e0, p.n1 - p.n0, int(p.senders.numel())
            Z_c = self.Z[:n_r]
            if before_chunk is not None:
                before_chunk(c)
            if n_e == 0:
                Z_c.zero_()
                if on_chunk is not None:
                    on_chunk(c, p, Z_c, self.dW[:0])
                if after_chunk is not None:
                    after_chunk(c)
                continue
            W_c, dW_c = self.W[:n_e], self.dW[:n_e]
            weights(c, W_c)
            torch.index_select(X, 0, p.senders, out=self.x_block[:n_s])
            Y_c = Y[p.e0:p.e1]
            rc = self.lib.oeqb_conv_forward_rect(
                self.desc, len(self.desc), self.key, n_r, n_s, n_e, self._p(self.x_block), self._p(Y_c), self._p(W_c),
                self._p(Z_c), self._p(p.rows_local), self._p(p.cols_local), self._p(p.perm_local),
                self._p(self.workspace), self.workspace.numel(), st)
            self.native.check(rc, "streamed conv forward")
            G_c = cotangent(c, Z_c)
            dY_c = dY[p.e0:p.e1] if dY is not None else torch.empty((n_e, self.L2), dtype=torch.float32, device=self.device)
            rc = self.lib.oeqb_conv_backward_rect(
                self.desc, len(self.desc), self.key, n_r, n_s, n_e, self._p(self.x_block), self._p(Y_c), self._p(W_c),
                self._p(G_c), self._p(self.dx_block), self._p(dY_c), self._p(dW_c), self._p(p.rows_local),
                self._p(p.cols_local), self._p(p.perm_local), self._p(self.workspace), self.workspace.numel(), st)
            self.native.check(rc, "streamed conv backward")
            dX.index_add_(0, p.senders, self.dx_block[:n_s])   # unique indices: one add per row, chunks in order
            if on_chunk is not None:
                on_chunk(c, p, Z_c, dW_c)
            if after_chunk is not None:
                after_chunk(c)
        return dX
