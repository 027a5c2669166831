"""Tensor parallelism with sequence-parallel activations.

Reference: ``ColumnParallelLinear`` (weight ``[K, N/T]``, replicated input, explicit
``allreduce_grad_x``) and ``RowParallelLinear`` (weight ``[K/T, N]``, partial outputs averaged —
which is wrong for partial sums — bias on rank 0) in rumus-distributed/src/tensor_parallel.rs:20-86,
all staged through the host.

Here the activations between a row-parallel output and the next column-parallel input are
sharded along the token dimension (``[M/T, d]`` per rank), so:

* column-parallel forward  = ALL-GATHER(tokens) -> GEMM          (fused kernel ``rb_ag_gemm``)
* row-parallel forward     = GEMM -> REDUCE-SCATTER(tokens, SUM) (fused kernel ``rb_gemm_rs``)
* column-parallel backward = dgrad GEMM -> REDUCE-SCATTER, wgrad on the gathered input
* row-parallel backward    = ALL-GATHER(dY) -> dgrad GEMM, wgrad on the gathered dY

``mode='nccl'`` runs the same layers with NCCL collectives + separate GEMMs (baseline);
CPU tensors use ``torch.distributed`` (gloo) and PyTorch math, which is how the sharding logic is
tested without GPUs.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..nn.modules import Module, _linear_rng, _uniform
from ..ops import functional as F
from ..ops import native
from ..utils.metrics import trace_range


class TPContext:
    """Process group + (for fused mode) arena staging shared by all TP layers of a model."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, mode: Optional[str] = None,
                 arena=None, max_tokens: int = 0, max_features: int = 0, dtype=torch.bfloat16):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        mode = mode or os.environ.get("RB_BACKEND", "fused")
        if self.world == 1:
            mode = "local"
        self.mode = mode
        self.arena = arena
        self.epoch = 0
        self.dtype = dtype
        if mode == "fused":
            from .symm import SymmArena
            esz = torch.empty((), dtype=dtype).element_size()
            stage_bytes = max_tokens * max_features * esz
            # slot sets of the push-form reduce-scatter: two of [world][max_tokens / world, max_features]
            push_bytes = stage_bytes
            if self.arena is None:
                self.arena = SymmArena(2 * stage_bytes + push_bytes + (64 << 20), group)
            a = self.arena
            self.gather_buf, self.gather_off = a.alloc_bytes(stage_bytes)
            self.partial_buf, self.partial_off = a.alloc_bytes(stage_bytes)
            self.chunk_flags = a.alloc_local_ints(256)
            n_tiles = (max_tokens // 128 + 1) * (max_features // 256 + 1)
            self.tile_flags_off = a.alloc_flags(n_tiles * self.world)
            self.tile_counters = a.alloc_local_ints(n_tiles)
            self.enter_flags = a.alloc_flags(self.world)
            self.bar_flags = a.alloc_flags(self.world)
            self.bar_epoch = 0
            self.stage_bytes = stage_bytes
            self.push_acc = None
            if os.environ.get("RB_TP_PUSH", "1") == "1" and push_bytes > 0:
                try:
                    # the pull form's partial-sum buffer doubles as the first slot set
                    self.push_acc = [self.partial_off, a.alloc_bytes(push_bytes)[1]]
                    self.push_bytes = push_bytes
                    self.push_flags = a.alloc_flags(self.world)
                    self.push_counters = a.alloc_local_ints(self.world)
                    self.push_epoch = 0
                except Exception:       # an arena handed in from outside may have no room: keep the pull form
                    self.push_acc = None
            torch.cuda.synchronize()
            a.barrier()
        self._last_fused = None

    def next_epoch(self) -> int:
        self.epoch += 1
        return self.epoch

    def order_fused(self, kind: str) -> None:
        """Called before a fused operation of ``kind`` ('A' all-gather→GEMM, 'R' GEMM→reduce-scatter).
        Neither kernel ends with a barrier: reuse of the staging buffers is safe because finishing
        one kind needs signals that every peer sends only after its preceding operation of the
        other kind.  Two operations of the same kind in a row do not have that property (checked on
        the model in ``utils/protocol_check.tp_sequence_programs``), so a group barrier goes between
        them."""
        if self._last_fused == kind:
            from . import fused_ops
            self.bar_epoch += 1
            fused_ops.group_barrier(self.arena, self.bar_flags, self.bar_epoch)
        self._last_fused = kind

    # ------------------------------------------------------------ collectives (baseline paths)
    def all_gather_rows(self, x_local: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x_local
        out = torch.empty((x_local.shape[0] * self.world, *x_local.shape[1:]), dtype=x_local.dtype,
                          device=x_local.device)
        dist.all_gather_into_tensor(out, x_local.contiguous(), group=self.group)
        return out

    def reduce_scatter_rows(self, x_full: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return x_full
        out = torch.empty((x_full.shape[0] // self.world, *x_full.shape[1:]), dtype=x_full.dtype,
                          device=x_full.device)
        dist.reduce_scatter_tensor(out, x_full.contiguous(), op=dist.ReduceOp.SUM, group=self.group)
        return out

    def all_reduce(self, x: torch.Tensor, op=dist.ReduceOp.SUM) -> torch.Tensor:
        if self.world > 1:
            dist.all_reduce(x, op=op, group=self.group)
        return x


def _mm(a, b):
    return native.gemm(a, b) if a.is_cuda else a @ b


def _fused_ag_gemm(ctx: TPContext, x_local, w, bias=None, act=None):
    with trace_range("tp.fused.ag_gemm"):
        return _fused_ag_gemm_impl(ctx, x_local, w, bias, act)


def _fused_ag_gemm_impl(ctx: TPContext, x_local, w, bias=None, act=None):
    """x_local [M/T, K] (each rank's rows) , w [K, N] logical -> (y [M, N], gathered x [M, K])."""
    from . import fused_ops
    a = ctx.arena
    Ml, K = x_local.shape
    M = Ml * ctx.world
    N = w.shape[1]
    esz = x_local.element_size()
    shard_bytes = Ml * K * esz
    assert shard_bytes * ctx.world <= ctx.stage_bytes and shard_bytes % 16 == 0
    # a peer may only read my shard after I announced it (src flag); I only overwrite it after
    # everybody consumed the previous contents, which the alternation of gather and reduce
    # operations guarantees and ``order_fused`` enforces otherwise; a host-side group barrier
    # guards the first use.
    ctx.order_fused("A")
    stage = ctx.gather_buf[: shard_bytes * ctx.world].view(x_local.dtype).view(M, K)
    stage[ctx.rank * Ml:(ctx.rank + 1) * Ml].copy_(x_local)
    epoch = ctx.next_epoch()
    _announce(ctx, epoch)
    # chunk = the unit in which GEMM tiles learn that gathered rows have arrived: 256 KB measured best at 4
    # ranks (227 us against 287 us with 1 MB chunks), no difference at 2
    chunk = max(256 << 10, (shard_bytes * ctx.world + 255) // 256)
    chunk = (chunk + 15) // 16 * 16
    out = torch.empty((M, N), dtype=x_local.dtype, device=x_local.device)
    fused_ops.ag_gemm(a, buf_off=ctx.gather_off, shard_bytes=shard_bytes, chunk_flags=ctx.chunk_flags,
                      chunk_bytes=chunk, epoch=epoch, gather_a=True, operand_off=0, other=w, M=M,
                      N=N, K=K, out=out, src_flags_off=ctx.enter_flags, bias=bias, act=act,
                      # with more ranks the gather is a larger share of the kernel (227 vs 238 us at 4 ranks)
                      n_copy_ctas=32 if ctx.world >= 4 else 16)
    return out, stage


def _announce(ctx: TPContext, epoch: int) -> None:
    """Publish 'my shard of the staging buffer holds epoch `epoch`' to every peer (stream ordered)."""
    from . import fused_ops
    fused_ops.signal_peers(ctx.arena, ctx.enter_flags, epoch)


def _fused_gemm_rs(ctx: TPContext, a_mat, w, bias=None, residual=None):
    with trace_range("tp.fused.gemm_rs"):
        return _fused_gemm_rs_impl(ctx, a_mat, w, bias, residual)


def _fused_gemm_rs_impl(ctx: TPContext, a_mat, w, bias=None, residual=None):
    """a_mat [M, K_local], w [K_local, N] -> y_local [M/T, N] (sum over ranks, + bias, + residual:
    both are added by the reducing owner of each output tile)."""
    from . import fused_ops
    M, K = a_mat.shape
    N = w.shape[1]
    out = torch.empty((M // ctx.world, N), dtype=a_mat.dtype, device=a_mat.device)
    ctx.order_fused("R")
    if ctx.push_acc is not None and M * N * a_mat.element_size() <= ctx.push_bytes and N % 8 == 0:
        # tiles stored from the GEMM's epilogue into the owners' per-source slots
        ctx.push_epoch += 1
        fused_ops.gemm_rs_push(ctx.arena, a_mat, w, slots_off=ctx.push_acc[ctx.push_epoch & 1],
                               done_flags_off=ctx.push_flags, owner_counters=ctx.push_counters,
                               epoch=ctx.push_epoch, out=out, bias=bias,
                               residual=residual.contiguous() if residual is not None else None)
        return out
    epoch = ctx.next_epoch()
    fused_ops.gemm_rs(ctx.arena, a_mat, w, partial_off=ctx.partial_off,
                      tile_flags_off=ctx.tile_flags_off, tile_counters=ctx.tile_counters, epoch=epoch,
                      out=out, bias=bias, residual=residual)
    return out


class _ColumnParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, w, bias, tp: TPContext, act):
        if tp.mode == "fused" and x_local.is_cuda and _fusable(tp, x_local.shape[0] * tp.world):
            y, x_full = _fused_ag_gemm(tp, x_local, w, bias, act=None)
            x_full = x_full.clone()
        else:
            x_full = tp.all_gather_rows(x_local)
            y = _mm(x_full, w)
            if bias is not None:
                y = y + bias
        ctx.tp = tp
        ctx.has_bias = bias is not None
        ctx.w_mg = F._main_grad(w)
        ctx.save_for_backward(x_full, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x_full, w = ctx.saved_tensors
        tp = ctx.tp
        dy = dy.contiguous()
        if tp.mode == "fused" and dy.is_cuda and _fusable_rs(tp, dy.shape[0]):
            dx_local = _fused_gemm_rs(tp, dy, w.t())
        else:
            dx_local = tp.reduce_scatter_rows(_mm(dy, w.t()))
        dw = F._wgrad(x_full, dy, ctx.w_mg) if dy.is_cuda else x_full.t() @ dy
        db = None
        if ctx.has_bias:
            db = native.colsum(dy) if dy.is_cuda else dy.sum(0)
        return dx_local, dw, db, None, None


class _RowParallelFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, tp: TPContext, residual=None):
        if tp.mode == "fused" and x.is_cuda and _fusable_rs(tp, x.shape[0]):
            y_local = _fused_gemm_rs(tp, x, w, bias, residual.contiguous() if residual is not None else None)
        else:
            y_local = tp.reduce_scatter_rows(_mm(x, w))
            if bias is not None:
                y_local = y_local + bias
            if residual is not None:
                y_local = y_local + residual
        ctx.tp = tp
        ctx.has_res = residual is not None
        ctx.has_bias = bias is not None
        ctx.w_mg = F._main_grad(w)
        ctx.save_for_backward(x, w)
        return y_local

    @staticmethod
    def backward(ctx, dy_local):
        x, w = ctx.saved_tensors
        tp = ctx.tp
        dy_local = dy_local.contiguous()
        if tp.mode == "fused" and dy_local.is_cuda and _fusable(tp, dy_local.shape[0] * tp.world):
            dx, dy_full = _fused_ag_gemm(tp, dy_local, w.t())
        else:
            dy_full = tp.all_gather_rows(dy_local)
            dx = _mm(dy_full, w.t())
        dw = F._wgrad(x, dy_full, ctx.w_mg) if x.is_cuda else x.t() @ dy_full
        db = None
        if ctx.has_bias:
            db = native.colsum(dy_local) if dy_local.is_cuda else dy_local.sum(0)
        return dx, dw, db, None, (dy_local if ctx.has_res else None)


_fallback_logged = set()


# The PULL form of GEMM -> reduce-scatter cannot overlap its reduction pass with the GEMM (a row block is
# complete only when every rank has computed its partial, and each rank computes its own blocks last):
# measured on the Llama-7B layer shapes it wins at 2 ranks (342 vs 359 us) and loses at 4 (271 vs 259 us),
# so without the push form (the default, see _fused_gemm_rs_impl) the row-parallel side above this group
# size runs the plain GEMM + NCCL reduce-scatter.  RB_TP_FUSE_RS_MAX overrides.
FUSED_RS_MAX_WORLD = int(__import__("os").environ.get("RB_TP_FUSE_RS_MAX", "2"))


def _fusable_rs(tp: TPContext, M: int) -> bool:
    # the push form has no second pass over the partial sums, so it is not limited to small groups
    if getattr(tp, "push_acc", None) is not None:
        return _fusable(tp, M)
    return tp.world <= FUSED_RS_MAX_WORLD and _fusable(tp, M)


def _fusable(tp: TPContext, M: int) -> bool:
    ok = M % (128 * tp.world) == 0
    if not ok and (M, tp.world) not in _fallback_logged:
        _fallback_logged.add((M, tp.world))
        import warnings
        warnings.warn(f"tensor-parallel layer with {M} tokens on {tp.world} ranks: the fused "
                      f"gather/GEMM/reduce-scatter kernels need a multiple of {128 * tp.world} tokens; "
                      "using NCCL collectives + separate GEMMs for this shape", stacklevel=3)
    return ok


def mark_tp_replicated(p: nn.Parameter) -> nn.Parameter:
    """Tags a parameter that every tensor-parallel rank holds in full while its gradient only
    covers that rank's token slab (norm weights in a sequence-parallel region, the bias of a
    row-parallel layer).  ``sync_replicated_grads`` / ``FSDP.reduce_grads`` sum those gradients
    over the group so that the copies stay identical."""
    p._tp_replicated = True
    return p


def sync_replicated_grads(module: nn.Module, tp: TPContext) -> None:
    """SUM all-reduce, over the tensor-parallel group, of ``.grad`` of every parameter tagged by
    ``mark_tp_replicated`` (for models driven by a plain optimizer; flat-arena engines use
    ``FSDP.reduce_grads``).  Collective."""
    if tp.world == 1:
        return
    grads = [p.grad for p in module.parameters() if getattr(p, "_tp_replicated", False) and p.grad is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    dist.all_reduce(flat, group=tp.group)
    o = 0
    for g in grads:
        g.copy_(flat[o:o + g.numel()].view(g.shape))
        o += g.numel()


class ColumnParallelLinear(Module):
    """Weight ``[in, out/T]`` (this rank's output columns).  Input: token-sharded ``[M/T, in]``;
    output ``[M, out/T]``."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = True,
                 device=None, dtype=None):
        super().__init__()
        assert out_features % tp.world == 0
        self.tp = tp
        self.in_features, self.out_features = in_features, out_features
        bound = math.sqrt(1.0 / in_features)
        full = _uniform((in_features, out_features), bound, _linear_rng, device, dtype)
        n = out_features // tp.world
        self.weight = nn.Parameter(full[:, tp.rank * n:(tp.rank + 1) * n].contiguous())
        self.bias = None
        if bias:
            fb = _uniform((out_features,), bound, _linear_rng, device, dtype)
            self.bias = nn.Parameter(fb[tp.rank * n:(tp.rank + 1) * n].contiguous())

    def forward(self, x_local):
        if self.tp.world == 1:
            return F.linear(x_local, self.weight, self.bias)
        return _ColumnParallelFn.apply(x_local, self.weight, self.bias, self.tp, None)


class RowParallelLinear(Module):
    """Weight ``[in/T, out]`` (this rank's input rows).  Input ``[M, in/T]``; output token-sharded
    ``[M/T, out]``, summed over ranks; the bias is added once (by the reducing owner)."""

    def __init__(self, in_features: int, out_features: int, tp: TPContext, bias: bool = True,
                 device=None, dtype=None):
        super().__init__()
        assert in_features % tp.world == 0
        self.tp = tp
        self.in_features, self.out_features = in_features, out_features
        bound = math.sqrt(1.0 / in_features)
        full = _uniform((in_features, out_features), bound, _linear_rng, device, dtype)
        k = in_features // tp.world
        self.weight = nn.Parameter(full[tp.rank * k:(tp.rank + 1) * k].contiguous())
        self.bias = nn.Parameter(_uniform((out_features,), bound, _linear_rng, device, dtype)) if bias else None
        if self.bias is not None:
            mark_tp_replicated(self.bias)

    def forward(self, x, residual=None):
        """``residual``: token-sharded ``[M/T, out]`` tensor added to the reduced output (inside the
        fused kernel's reduction)."""
        if self.tp.world == 1:
            return F.linear(x, self.weight, self.bias, residual=residual)
        return _RowParallelFn.apply(x, self.weight, self.bias, self.tp, residual)


def scatter_rows(x: torch.Tensor, tp: TPContext) -> torch.Tensor:
    """Take this rank's token slab of a replicated ``[M, d]`` tensor (entering a sequence-parallel
    region); its backward all-gathers the gradient."""
    if tp.world == 1:
        return x
    return _ScatterRowsFn.apply(x, tp)


def gather_rows(x_local: torch.Tensor, tp: TPContext) -> torch.Tensor:
    if tp.world == 1:
        return x_local
    return _GatherRowsFn.apply(x_local, tp)


class _ScatterRowsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        n = x.shape[0] // tp.world
        return x[tp.rank * n:(tp.rank + 1) * n].contiguous()

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_gather_rows(g.contiguous()), None


class _GatherRowsFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x_local, tp):
        ctx.tp = tp
        return tp.all_gather_rows(x_local)

    @staticmethod
    def backward(ctx, g):
        n = g.shape[0] // ctx.tp.world
        # every rank computed the same loss contribution pattern downstream: the gradient of a
        # gather is the local slab of the (summed) upstream gradient
        return ctx.tp.reduce_scatter_rows(g.contiguous()), None


# ------------------------------------------------------------------ vocabulary-parallel embedding
class _VocabParallelEmbedFn(torch.autograd.Function):
    """Rows of the table outside this rank's vocabulary slice contribute zeros; the partial results
    are summed over the group — as a reduce-scatter over tokens when the output feeds a
    sequence-parallel region, else as an all-reduce."""

    @staticmethod
    def forward(ctx, weight, tokens, tp, vocab_start, sequence_parallel):
        vloc = weight.shape[0]
        tl = tokens.reshape(-1) - vocab_start
        mine = (tl >= 0) & (tl < vloc)
        idx = tl.clamp(0, vloc - 1)
        out = weight.index_select(0, idx) * mine[:, None].to(weight.dtype)
        ctx.tp, ctx.sp, ctx.vloc = tp, sequence_parallel, vloc
        ctx.save_for_backward(idx, mine)
        if sequence_parallel:
            return tp.reduce_scatter_rows(out)
        return tp.all_reduce(out)

    @staticmethod
    def backward(ctx, g):
        idx, mine = ctx.saved_tensors
        if ctx.sp:
            g = ctx.tp.all_gather_rows(g.contiguous())
        g = g * mine[:, None].to(g.dtype)
        dw = torch.zeros(ctx.vloc, g.shape[1], dtype=torch.float32, device=g.device)
        dw.index_add_(0, idx, g.float())
        return dw.to(g.dtype), None, None, None, None


class VocabParallelEmbedding(Module):
    """Embedding table split along the vocabulary: rank ``r`` of ``T`` holds rows
    ``[r*V/T, (r+1)*V/T)``.  The reference has only the replicated ``Embedding``
    (rumus/src/nn/embedding.rs; no vocabulary-parallel helper in rumus-distributed/src/tensor_parallel.rs);
    for a 7B model on 8 ranks the split table saves 7/8 of 0.26 GB per rank and, more to the point,
    leaves the token embedding in the same layout as the vocabulary-parallel head, so tied weights
    stay possible.

    ``forward(tokens)`` takes the full ``[M]`` token ids (replicated on the group) and returns
    ``[M, d]``, or this rank's ``[M/T, d]`` token slab with ``sequence_parallel=True``.
    The full table is drawn from the same random stream as ``Embedding`` (every rank draws all of
    it) and then sliced, so the values do not depend on the group size."""

    def __init__(self, vocab_size: int, dim: int, tp: TPContext, sequence_parallel: bool = False,
                 device=None, dtype=None):
        super().__init__()
        if vocab_size % tp.world:
            raise ValueError(f"vocab_size {vocab_size} is not divisible by the group size {tp.world}")
        from ..nn.modules import Embedding
        self.tp, self.sp = tp, sequence_parallel
        self.vocab_size, self.dim = vocab_size, dim
        self.vloc = vocab_size // tp.world
        self.vocab_start = tp.rank * self.vloc
        full = Embedding(vocab_size, dim).weight.data
        w = full[self.vocab_start:self.vocab_start + self.vloc].clone()
        self.weight = nn.Parameter(w.to(device=device, dtype=dtype or w.dtype))

    def forward(self, tokens: torch.Tensor) -> torch.Tensor:
        if self.tp.world == 1:
            return self.weight.index_select(0, tokens.reshape(-1))
        return _VocabParallelEmbedFn.apply(self.weight, tokens, self.tp, self.vocab_start, self.sp)


def vocab_parallel_cross_entropy(logits_local: torch.Tensor, targets: torch.Tensor, tp: TPContext) -> torch.Tensor:
    """Mean cross entropy of ``[M, V/T]`` logit slices against full-vocabulary ``targets`` without
    gathering the logits (three small all-reduces: row max, sum of exponentials, target logit)."""
    from ..models.llama_parallel import _VocabParallelCE
    return _VocabParallelCE.apply(logits_local, targets.reshape(-1), tp, tp.rank * logits_local.shape[1])


# ------------------------------------------------------------------ replicated-activation regions
class _CopyToRegionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        ctx.tp = tp
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return ctx.tp.all_reduce(g.contiguous().clone()), None


class _ReduceFromRegionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, tp):
        return tp.all_reduce(x.contiguous().clone())

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_region(x: torch.Tensor, tp: TPContext) -> torch.Tensor:
    """Entry of a tensor-parallel region whose input is replicated: identity in forward, SUM
    all-reduce of the gradient in backward (every rank only sees the contribution of its own
    weight columns).  The reference leaves this to the user as an explicit
    ``ColumnParallelLinear::allreduce_grad_x`` call (rumus-distributed/src/tensor_parallel.rs:39-48)."""
    return x if tp.world == 1 else _CopyToRegionFn.apply(x, tp)


def reduce_from_region(x: torch.Tensor, tp: TPContext) -> torch.Tensor:
    """Exit of a tensor-parallel region with replicated output: SUM all-reduce of the partial
    results in forward (the reference averages, rumus-distributed/src/collective.rs:56-60, which is
    wrong for partial sums), identity in backward."""
    return x if tp.world == 1 else _ReduceFromRegionFn.apply(x, tp)
