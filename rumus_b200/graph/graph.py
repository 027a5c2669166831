"""CSR graph + SpMM (reference: rumus-graph/src/graph.rs:10-217, ops.rs:18-196).

``Graph.new(num_nodes, src, dst, weights)`` builds the CSR of the adjacency ``A`` (row = dst,
col = src: messages flow src -> dst) and of ``A^T`` once; ``graph.spmm(X)`` computes ``A @ X`` and
its backward is ``A^T @ dY`` on the pre-transposed CSR — the same kernel, no atomics.
"""
from __future__ import annotations

from ctypes import c_int, c_void_p
from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import native
from ..ops._lib import check, count_launch, ptr, stream_ptr

native.register_signature("rb_spmm_csr", [c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                                          c_int, c_int, c_void_p])


@dataclass
class SparseTensor:
    """CSR matrix ``[rows, cols]``: ``rowptr`` int32 [rows+1], ``col`` int32 [nnz], ``val`` fp32 [nnz] or None."""
    rows: int
    cols: int
    rowptr: torch.Tensor
    col: torch.Tensor
    val: Optional[torch.Tensor]

    def to(self, device) -> "SparseTensor":
        return SparseTensor(self.rows, self.cols, self.rowptr.to(device), self.col.to(device),
                            self.val.to(device) if self.val is not None else None)

    def dense(self) -> torch.Tensor:
        out = torch.zeros(self.rows, self.cols, device=self.rowptr.device)
        counts = (self.rowptr[1:] - self.rowptr[:-1]).long()
        r = torch.repeat_interleave(torch.arange(self.rows, device=out.device), counts)
        v = self.val if self.val is not None else torch.ones(self.col.numel(), device=out.device)
        out.index_put_((r, self.col.long()), v, accumulate=True)
        return out


def _build_csr(rows: int, cols: int, r: torch.Tensor, c: torch.Tensor, v: Optional[torch.Tensor]) -> SparseTensor:
    order = torch.argsort(r * cols + c, stable=True)
    r, c = r[order], c[order]
    v = v[order].float() if v is not None else None
    counts = torch.bincount(r, minlength=rows)
    rowptr = torch.zeros(rows + 1, dtype=torch.int64)
    rowptr[1:] = torch.cumsum(counts, 0)
    return SparseTensor(rows, cols, rowptr.int(), c.int(), v)


def _spmm_raw(a: SparseTensor, x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        return a.dense().to(x.dtype) @ x
    x = x.contiguous()
    y = torch.empty((a.rows, x.shape[1]), dtype=x.dtype, device=x.device)
    check(native.lib().rb_spmm_csr(native.dtype_code(x.dtype), ptr(a.rowptr), ptr(a.col), ptr(a.val),
                                   ptr(x), ptr(y), a.rows, x.shape[1], stream_ptr()), "rb_spmm_csr")
    count_launch()
    return y


class _SpmmFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, a, at):
        ctx.at = at
        return _spmm_raw(a, x)

    @staticmethod
    def backward(ctx, dy):
        return _spmm_raw(ctx.at, dy), None, None


def spmm(a: SparseTensor, at: SparseTensor, x: torch.Tensor) -> torch.Tensor:
    return _SpmmFn.apply(x, a, at)


class Graph:
    def __init__(self, num_nodes: int, adj: SparseTensor, adj_t: SparseTensor):
        self.num_nodes, self.adj, self.adj_t = num_nodes, adj, adj_t

    @staticmethod
    def new(num_nodes: int, src, dst, weights=None, device="cpu") -> "Graph":
        src = torch.as_tensor(src, dtype=torch.int64)
        dst = torch.as_tensor(dst, dtype=torch.int64)
        w = torch.as_tensor(weights, dtype=torch.float32) if weights is not None else None
        a = _build_csr(num_nodes, num_nodes, dst, src, w)
        at = _build_csr(num_nodes, num_nodes, src, dst, w)
        return Graph(num_nodes, a.to(device), at.to(device))

    def to(self, device) -> "Graph":
        return Graph(self.num_nodes, self.adj.to(device), self.adj_t.to(device))

    def spmm(self, x: torch.Tensor) -> torch.Tensor:
        """``A @ x`` with ``x [num_nodes, F]`` (reference: Graph::spmm, graph.rs:88)."""
        return spmm(self.adj, self.adj_t, x)
