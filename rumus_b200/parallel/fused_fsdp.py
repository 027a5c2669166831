"""Fused-kernel communication for the FSDP engine (see ``fsdp.py`` for the step protocol).

Per sharding unit there are two epoch-flag arrays in the arena (``grad_ready[world]``,
``param_ready[world]``) and one local completion counter.  At optimizer step ``t`` (1-based):

* ``reduce_scatter_adam(u)`` launches ``rb_rs_adam`` with epoch ``t``: it announces this rank's
  gradients, waits for every peer's announcement, reduces + updates + rewrites the parameter
  shard, then announces ``param_ready = t``;
* ``all_gather(u)`` launches ``rb_all_gather`` with epoch ``t``: per peer it waits for
  ``param_ready >= t`` and pulls that peer's shard.

Write-after-read safety of the gradient buffers needs no extra barrier: a rank only starts
writing unit ``u``'s gradients for step ``t+1`` after its own all-gather of ``u`` at step ``t``
returned, and that returned only after every peer had published ``param_ready = t``, which each
peer does after it finished reading everybody's gradients of step ``t``.
"""
from __future__ import annotations

import os

from . import fused_ops

# CTAs per communication kernel while the backward pass is still running on the compute stream
# (few, so the persistent GEMMs keep their SMs) and once it has finished (nothing left to overlap
# with: use the whole GPU).
_RS_CTAS = int(os.environ.get("RB_RS_CTAS", "148"))
_AG_CTAS = int(os.environ.get("RB_AG_CTAS", "32"))
_TAIL_RS_CTAS = int(os.environ.get("RB_TAIL_RS_CTAS", "296"))
_TAIL_AG_CTAS = int(os.environ.get("RB_TAIL_AG_CTAS", "148"))


class FusedFsdpComm:
    def __init__(self, engine):
        self.e = engine
        a = engine.arena
        self.arena = a
        self.grad_flags = [a.alloc_flags(a.world) for _ in engine.units]
        self.param_flags = [a.alloc_flags(a.world) for _ in engine.units]
        self.counters = [a.alloc_local_ints(1) for _ in engine.units]
        for u in engine.units:
            home = u.persist if u.persist is not None else u.flat_param
            assert hasattr(home, "arena_offset") and hasattr(u.flat_grad, "arena_offset")
        a.barrier()

    def reduce_scatter_adam(self, idx: int, tail: bool = False) -> None:
        e, u = self.e, self.e.units[idx]
        if u.persist is not None:
            # the kernel writes the updated shard at param_off + shard_lo elements: aim that at the
            # shard's own buffer
            param_off = u.persist.arena_offset - u.shard_range[0] * u.persist.element_size()
        else:
            param_off = u.flat_param.arena_offset
        fused_ops.rs_adam(self.arena, u.dtype, u.flat_grad.arena_offset, param_off,
                          u.shard_range[0], u.shard_numel, u.master, u.exp_avg, u.exp_avg_sq,
                          lr=e.lr, beta1=e.beta1, beta2=e.beta2, eps=e.eps,
                          weight_decay=e.weight_decay, step=e.step_count + 1, adamw=e.adamw,
                          grad_flags_off=self.grad_flags[idx], param_flags_off=self.param_flags[idx],
                          epoch=e.step_count + 1, done_counter=self.counters[idx],
                          ctas=_TAIL_RS_CTAS if tail else _RS_CTAS)

    def all_gather(self, idx: int, tail: bool = False) -> None:
        e, u = self.e, self.e.units[idx]
        esz = u.flat_param.element_size()
        fused_ops.all_gather(self.arena, u.flat_param.arena_offset, u.shard_numel * esz,
                             src_flags_off=self.param_flags[idx], epoch=e.step_count + 1,
                             ctas=_TAIL_AG_CTAS if tail else _AG_CTAS)

    def gather_shards(self, idx: int, dst, tail: bool = False) -> None:
        """Resharded unit: every rank's persistent shard -> the local slot ``dst``.  A peer's shard
        is read once its ``param_ready`` flag shows the update of the last completed step."""
        e, u = self.e, self.e.units[idx]
        esz = u.persist.element_size()
        fused_ops.shard_gather(self.arena, u.persist.arena_offset, dst, u.shard_numel * esz,
                               src_flags_off=self.param_flags[idx], epoch=e.step_count,
                               ctas=_TAIL_AG_CTAS if tail else _AG_CTAS)

    def end_step(self) -> None:
        pass
