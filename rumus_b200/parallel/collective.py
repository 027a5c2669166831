"""Stand-alone collectives with an asynchronous handle.

Reference: ``CollectiveBarrier::reduce`` (blocking mean over rank threads through host memory,
rumus-distributed/src/collective.rs:16-79), ``CommThread`` (one background thread per device that
maps a staging buffer, joins the barrier and writes the result back, :97-145) and
``async_allreduce`` → ``AllReduceHandle::wait`` (:152-202).

With one process per GPU the background thread becomes a side stream: the collective is enqueued
behind the work that produced the tensor, the caller keeps launching compute, and ``wait()`` makes
the *current stream* depend on the result (an event, not a host block).  On CPU ranks (gloo) the
handle wraps the process group's asynchronous work object.

The gradient paths of the training engines do not go through this module — they use the fused
kernels (``parallel/dp.py``, ``parallel/fsdp.py``); this is the general-purpose entry point the
reference exposes to user code.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

_side_streams = {}


def _side_stream(device: torch.device) -> "torch.cuda.Stream":
    key = (device.type, device.index)
    if key not in _side_streams:
        _side_streams[key] = torch.cuda.Stream(device=device)
    return _side_streams[key]


class AllReduceHandle:
    """Completion handle of ``async_all_reduce``.  ``wait()`` returns the reduced tensor (the one
    that was passed in, reduced in place) once it is safe to use on the current stream."""

    def __init__(self, tensor: torch.Tensor, work=None, event: Optional["torch.cuda.Event"] = None,
                 scale: Optional[float] = None):
        self.tensor, self._work, self._event, self._scale = tensor, work, event, scale
        self._done = work is None and event is None

    def is_completed(self) -> bool:
        if self._done:
            return True
        if self._event is not None:
            return self._event.query()
        return self._work.is_completed()

    def wait(self) -> torch.Tensor:
        if not self._done:
            if self._event is not None:
                torch.cuda.current_stream(self.tensor.device).wait_event(self._event)
            else:
                self._work.wait()
                if self._scale is not None:
                    self.tensor.mul_(self._scale)
            self._done = True
        return self.tensor


def async_all_reduce(tensor: torch.Tensor, average: bool = True,
                     group: Optional[dist.ProcessGroup] = None) -> AllReduceHandle:
    """Starts an in-place all-reduce of ``tensor`` (mean by default, like the reference's barrier;
    ``average=False`` sums) and returns at once."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return AllReduceHandle(tensor)
    if tensor.is_cuda:
        side = _side_stream(tensor.device)
        side.wait_stream(torch.cuda.current_stream(tensor.device))
        with torch.cuda.stream(side):
            dist.all_reduce(tensor, op=dist.ReduceOp.AVG if average else dist.ReduceOp.SUM, group=group)
            ev = torch.cuda.Event()
            ev.record(side)
        tensor.record_stream(side)
        return AllReduceHandle(tensor, event=ev)
    # gloo has no AVG: sum, then scale when the handle is waited on
    work = dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=group, async_op=True)
    return AllReduceHandle(tensor, work=work, scale=(1.0 / world) if average else None)


def all_reduce(tensor: torch.Tensor, average: bool = True,
               group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Blocking form (reference: ``CollectiveBarrier::reduce``)."""
    return async_all_reduce(tensor, average, group).wait()


def barrier(group: Optional[dist.ProcessGroup] = None) -> None:
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.barrier(group)
