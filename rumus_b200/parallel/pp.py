"""Pipeline parallelism with a true 1F1B schedule over NCCL (or gloo) point-to-point.

Reference: ``PipelineExecutor::run`` splits a batch into micro-batches, runs one thread per stage
connected by in-process channels, and — despite its name — does all forwards then all backwards
(GPipe order; rumus-distributed/src/pipeline.rs:35-187).  Here every stage is a process:

    warm-up   : ``min(P - 1 - stage, M)`` forwards
    steady    : one forward, one backward, alternating
    cool-down : the remaining backwards

Activations travel with ``isend`` / ``irecv`` (posted early so the transfer overlaps the
neighbouring compute); receives for the next micro-batch are posted before the current compute
starts.  At most ``P - stage`` micro-batches are alive per stage, instead of all ``M``.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch

from ..utils.metrics import trace_range
import torch.distributed as dist


def one_f_one_b_order(stage: int, num_stages: int, num_micro: int) -> List[tuple]:
    """The op sequence of one stage: list of ('F', mb) / ('B', mb).  Pure function (unit tested)."""
    warm = min(num_stages - 1 - stage, num_micro)
    ops = [("F", i) for i in range(warm)]
    f, b = warm, 0
    while f < num_micro:
        ops.append(("F", f)); f += 1
        ops.append(("B", b)); b += 1
    while b < num_micro:
        ops.append(("B", b)); b += 1
    return ops


def bubble_fraction(num_stages: int, num_micro: int) -> float:
    """Idle share of a 1F1B step when every micro-batch stage takes the same time:
    ``(P - 1) / (M + P - 1)`` (P - 1 warm-up and P - 1 drain slots out of M + P - 1 per direction)."""
    return (num_stages - 1) / float(num_micro + num_stages - 1)


class PipelineStage:
    """``forward_fn(x_or_microbatch) -> tensor``; the last stage's ``forward_fn`` returns the loss
    of the micro-batch (already divided by the number of micro-batches by ``run``)."""

    def __init__(self, forward_fn: Callable, stage: int, num_stages: int, prev_rank: Optional[int],
                 next_rank: Optional[int], act_shape: Sequence[int], act_dtype: torch.dtype, device,
                 group: Optional[dist.ProcessGroup] = None):
        self.forward_fn = forward_fn
        self.stage, self.num_stages = stage, num_stages
        self.prev_rank, self.next_rank = prev_rank, next_rank
        self.act_shape, self.act_dtype, self.device = tuple(act_shape), act_dtype, device
        self.group = group

    @property
    def is_first(self) -> bool:
        return self.stage == 0

    @property
    def is_last(self) -> bool:
        return self.stage == self.num_stages - 1

    # ---- p2p helpers: every exchange with a neighbour that has a matching exchange in the
    # opposite direction is issued as ONE batched group, which is what keeps 1F1B deadlock free
    # (stage s "send fwd + recv bwd" meets stage s+1 "send bwd + recv fwd").
    def _exchange(self, send_next=None, send_prev=None, recv_prev=False, recv_next=False):
        ops, r_prev, r_next = [], None, None
        if send_prev is not None:
            ops.append(dist.P2POp(dist.isend, send_prev.contiguous(), self.prev_rank))
        if recv_prev:
            r_prev = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, r_prev, self.prev_rank))
        if send_next is not None:
            ops.append(dist.P2POp(dist.isend, send_next.contiguous(), self.next_rank))
        if recv_next:
            r_next = torch.empty(self.act_shape, dtype=self.act_dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, r_next, self.next_rank))
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        return r_prev, r_next

    def run(self, micro_batches: Sequence, ops_log: Optional[list] = None) -> Optional[torch.Tensor]:
        """Runs one training step (forward + backward of every micro-batch).  ``micro_batches`` is
        consumed by the first stage (inputs) and the last stage (targets, through ``forward_fn``);
        middle stages may pass a list of ``None``.  Returns the mean loss on the last stage."""
        M = len(micro_batches)
        warm = min(self.num_stages - 1 - self.stage, M)
        steady = M - warm
        inputs, outputs = [], []
        total_loss = None

        def fwd(mb, x):
            nonlocal total_loss
            if ops_log is not None:
                ops_log.append(("F", mb))
            if not self.is_first:
                x = x.requires_grad_(True)
            else:
                x = micro_batches[mb]
            with trace_range(f"pp.stage{self.stage}.fwd.mb{mb}"):
                out = self.forward_fn(x) if not self.is_last else self.forward_fn((x, micro_batches[mb]))
            if self.is_last:
                out = out / M
                total_loss = out.detach() if total_loss is None else total_loss + out.detach()
            inputs.append(x)
            outputs.append(out)
            return out

        def bwd(mb, grad_out):
            if ops_log is not None:
                ops_log.append(("B", mb))
            x, out = inputs.pop(0), outputs.pop(0)
            with trace_range(f"pp.stage{self.stage}.bwd.mb{mb}"):
                if self.is_last:
                    out.backward()
                else:
                    torch.autograd.backward(out, grad_out)
            return None if self.is_first else x.grad

        f = b = 0
        x_in = None
        # warm-up forwards
        for _ in range(warm):
            if not self.is_first:
                x_in, _ = self._exchange(recv_prev=True)
            out = fwd(f, x_in); f += 1
            if not self.is_last:
                self._exchange(send_next=out.detach())
        if steady > 0 and not self.is_first:
            x_in, _ = self._exchange(recv_prev=True)
        # steady state: 1 forward, 1 backward
        for i in range(steady):
            out = fwd(f, x_in); f += 1
            g_out = None
            if not self.is_last:
                _, g_out = self._exchange(send_next=out.detach(), recv_next=True)
            g_in = bwd(b, g_out); b += 1
            last = i == steady - 1
            if not self.is_first:
                if last:
                    self._exchange(send_prev=g_in)
                else:
                    x_in, _ = self._exchange(send_prev=g_in, recv_prev=True)
        # cool-down backwards
        for _ in range(warm):
            g_out = None
            if not self.is_last:
                _, g_out = self._exchange(recv_next=True)
            g_in = bwd(b, g_out); b += 1
            if not self.is_first:
                self._exchange(send_prev=g_in)
        return total_loss
