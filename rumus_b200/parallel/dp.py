"""Data parallel training: one process per GPU, gradients all-reduced (mean) in buckets.

Reference: ``DataParallel`` replicates a model across devices in one process, scatters the batch,
gathers outputs on device 0 and re-broadcasts weights every step; ``AllReduceSync`` averages each
gradient on the host (rumus/src/nn/parallel.rs:24-250).  Here every rank owns its replica and its
data (SPMD); after backward the flat gradient bucket — which lives in the symmetric arena — is
all-reduced by ONE kernel that also multiplies by ``1/(loss_scale * world)`` and raises a job-wide
non-finite flag (``csrc/comm/fsdp_comm.cu: allreduce_unscale_kernel``); identical optimizer steps
on identical gradients keep the replicas in sync without a broadcast.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..utils.metrics import trace_range
from .flat import _round_up


class GradBucket:
    def __init__(self, params: List[nn.Parameter], world: int, alloc):
        self.params = params
        dtype = params[0].dtype
        offs, off = [], 0
        for p in params:
            offs.append(off)
            off += _round_up(p.numel(), 64)
        self.numel = _round_up(off, 16 * world)
        self.flat = alloc(self.numel, dtype)
        self.offsets = offs
        for p, o in zip(params, offs):
            p.main_grad = self.flat[o:o + p.numel()].view(p.shape)
            p.grad_accumulate = False

    def begin_step(self):
        for p in self.params:
            p.grad_accumulate = False

    def collect(self):
        """Gradients that arrived through plain autograd are moved into the bucket and ``p.grad``
        is re-pointed at the bucket view, so optimizers read reduced values."""
        for p in self.params:
            if p.grad is not None and p.grad.data_ptr() != p.main_grad.data_ptr():
                if p.grad_accumulate:
                    p.main_grad.add_(p.grad)
                else:
                    p.main_grad.copy_(p.grad)
            p.grad = p.main_grad
            p.grad_accumulate = True


class DataParallel:
    """``dp = DataParallel(model); loss.backward(); dp.all_reduce_grads(scaler)`` then step."""

    def __init__(self, model: nn.Module, group: Optional[dist.ProcessGroup] = None,
                 mode: Optional[str] = None, bucket_mb: int = 25, arena=None):
        self.model = model
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        # reverse registration order: backward produces gradients roughly from the last layer to the
        # first, so the first bucket to fill is the first one in the list
        params = [p for p in model.parameters() if p.requires_grad][::-1]
        dev = params[0].device
        mode = mode or os.environ.get("RB_BACKEND", "fused")
        if self.world == 1:
            mode = "local"
        elif dev.type != "cuda":
            mode = "cpu"
        self.mode = mode
        self.arena = arena
        if mode == "fused":
            from .symm import SymmArena
            if self.arena is None:
                need = sum(p.numel() * p.element_size() for p in params) * 1.1 + (16 << 20)
                self.arena = SymmArena(int(need), group)
            alloc = lambda n, dt: self.arena.alloc_flat(n, dt)
        else:
            alloc = lambda n, dt: torch.zeros(n, dtype=dt, device=dev)
        # bucket by dtype and size
        self.buckets: List[GradBucket] = []
        by_dtype = {}
        for p in params:
            by_dtype.setdefault(p.dtype, []).append(p)
        limit = bucket_mb << 20
        for dt, ps in by_dtype.items():
            cur, cur_bytes = [], 0
            for p in ps:
                cur.append(p)
                cur_bytes += p.numel() * p.element_size()
                if cur_bytes >= limit:
                    self.buckets.append(GradBucket(cur, self.world, alloc))
                    cur, cur_bytes = [], 0
            if cur:
                self.buckets.append(GradBucket(cur, self.world, alloc))
        self.epoch = 0
        self.found_inf = torch.zeros(1, dtype=torch.int32, device=dev)
        # overlap with backward: per-parameter hooks count a bucket full and reduce it right away on
        # a side stream (armed per step by ``begin_backward``)
        self._armed = False
        self._inv_scale = None
        self._launched = [False] * len(self.buckets)
        self._pending = [0] * len(self.buckets)
        self._handles = []
        self._cuda = dev.type == "cuda"
        self.comm_stream = (torch.cuda.Stream(device=dev, priority=-1)
                            if self._cuda and self.world > 1 else None)
        for bi, b in enumerate(self.buckets):
            for p in b.params:
                p.register_post_accumulate_grad_hook(self._make_hook(bi))
        if mode == "fused":
            a = self.arena
            self._flags = [(a.alloc_flags(self.world), a.alloc_flags(self.world), a.alloc_flags(self.world))
                           for _ in self.buckets]
            self._counters = [a.alloc_local_ints(1) for _ in self.buckets]
            a.barrier()
        if self.world > 1:
            self.broadcast_weights()

    def broadcast_weights(self) -> None:
        """One-time sync of the replicas (reference: parallel.rs:113-123 does this every step)."""
        for t in list(self.model.parameters()) + list(self.model.buffers()):
            dist.broadcast(t.data, src=dist.get_global_rank(self.group, 0) if self.group else 0,
                           group=self.group)

    def zero_grad(self) -> None:
        for b in self.buckets:
            b.begin_step()
        for p in self.model.parameters():
            p.grad = None

    # ------------------------------------------------------------------ overlap with backward
    def begin_backward(self, inv_scale: Optional[torch.Tensor] = None) -> None:
        """Call right before ``loss.backward()`` of the step whose gradients are to be reduced:
        from then on a bucket is all-reduced (and unscaled by ``inv_scale``, a device scalar) on
        the side stream as soon as backward has produced its last gradient."""
        self.epoch += 1
        self.found_inf.zero_()
        self._armed = True
        self._inv_scale = inv_scale
        self._launched = [False] * len(self.buckets)
        self._pending = [len(b.params) for b in self.buckets]
        self._handles = []

    def _make_hook(self, bi: int):
        def hook(p):
            if not self._armed or self._launched[bi]:
                return
            self._pending[bi] -= 1
            if self._pending[bi] == 0:
                self._launch(bi)
        return hook

    def _launch(self, i: int) -> None:
        with trace_range(f"dp.{self.mode}.bucket{i}"):
            self._launch_bucket(i)

    def _launch_bucket(self, i: int) -> None:
        b = self.buckets[i]
        self._launched[i] = True
        b.collect()
        if self.mode == "fused":
            from . import fused_ops
            ef, xf, nf = self._flags[i]
            cur = torch.cuda.current_stream()
            self.comm_stream.wait_stream(cur)
            with torch.cuda.stream(self.comm_stream):
                fused_ops.allreduce_unscale(self.arena, b.flat, enter_flags_off=ef, exit_flags_off=xf,
                                            inf_flags_off=nf, epoch=self.epoch,
                                            inv_scale=self._inv_scale, extra_scale=1.0 / self.world,
                                            found_inf=self.found_inf, done_counter=self._counters[i])
        elif self.world > 1:
            if self._cuda:
                cur = torch.cuda.current_stream()
                self.comm_stream.wait_stream(cur)
                with torch.cuda.stream(self.comm_stream):
                    self._handles.append(dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group,
                                                         async_op=True))
            else:
                self._handles.append(dist.all_reduce(b.flat, op=dist.ReduceOp.SUM, group=self.group,
                                                     async_op=True))

    def all_reduce_grads(self, inv_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Mean all-reduce of every bucket, fused with the unscale by ``inv_scale`` (device scalar,
        ``1/loss_scale``).  Returns the job-wide non-finite flag (int32 device tensor).  Buckets
        that ``begin_backward`` already reduced during backward are only waited for."""
        if not self._armed:
            self.epoch += 1
            self.found_inf.zero_()
            self._inv_scale = inv_scale
            self._launched = [False] * len(self.buckets)
            self._handles = []
        self._armed = False
        for i in range(len(self.buckets)):
            if not self._launched[i]:
                self._launch(i)
        for h in self._handles:
            h.wait()
        self._handles = []
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        if self.mode != "fused":
            # unscale and non-finite check stay on the device (no host round trip per bucket): the
            # scale is a device scalar, the flag is accumulated with a device-side maximum
            inv = self._inv_scale
            for b in self.buckets:
                if inv is not None:
                    b.flat.mul_((inv / self.world).to(b.flat.dtype))
                elif self.world > 1:
                    b.flat.mul_(1.0 / self.world)
                bad = torch.logical_not(torch.isfinite(b.flat).all()).to(self.found_inf.dtype)
                torch.maximum(self.found_inf, bad.reshape(self.found_inf.shape), out=self.found_inf)
        return self.found_inf
