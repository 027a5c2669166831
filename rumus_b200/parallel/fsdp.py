"""Fully sharded data parallel training over flat per-block arenas.

Reference behaviour (rumus/src/nn/fsdp.rs:63-312, rumus/src/autograd/backward.rs:1101-1242):
parameters are sharded across ranks, gathered around each linear layer's forward and backward,
gradients are averaged across ranks and each rank keeps its slice, and an ordinary optimizer then
updates the shards.  There every transfer goes through host memory and a mutex rendezvous.

Here each sharding unit (embeddings, one transformer block, final norm + head) is one flat bf16
vector (``flat.FlatUnit``).  Per step and unit:

* backward writes gradients straight into the unit's flat gradient buffer;
* when the unit's backward has finished (an autograd boundary node fires), the side stream runs
  **reduce-scatter + sharded Adam** — in ``fused`` mode ONE kernel (``rs_adam_kernel``, ``csrc/comm/fsdp_comm.cu``)
  that reads this rank's slice of every peer's gradient buffer over NVLink, averages in fp32,
  applies Adam(W) to the fp32 master shard and moments, and writes the bf16 shard in place;
* the updated shards are **all-gathered** for the next forward — in ``fused`` mode by copy CTAs
  that pull peer shards with plain P2P loads (stand-alone kernel, or folded into the unit's first
  consuming GEMM, ``ag_gemm_kernel`` in ``csrc/comm/tp_comm.cu``).

With ``reshard_after_forward`` (the reference's flow, rumus/src/nn/fsdp.rs:117-312: weights are
gathered for a layer's forward, dropped, and gathered again for its backward) a block keeps only
its shard between uses: the full vector of a block lives in one of two rotating slots, the next
block's shards are gathered into the other slot while this block computes, and nothing is gathered
after the update.  Parameter memory is then shards + two block-sized slots instead of every block
in full.  In ``fused`` mode the shards live in the arena and ``shard_gather_kernel`` pulls them into
the local slot with plain peer loads; ``nccl`` and CPU ranks use ``all_gather_into_tensor``.

``nccl`` mode issues ``reduce_scatter_tensor`` / ``all_gather_into_tensor`` plus the fused flat
Adam kernel: that is the comparison baseline.  With a world size of 1 no communication happens.
"""
from __future__ import annotations

import contextlib
import os
from typing import List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import native
from ..utils.metrics import trace_range
from .flat import FlatUnit, build_units, default_units


class _Boundary(torch.autograd.Function):
    """Identity in forward; in backward it tells the engine that every gradient of the unit whose
    *input* this is has been produced."""

    @staticmethod
    def forward(ctx, x, engine, unit_idx):
        ctx.engine, ctx.unit_idx = engine, unit_idx
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.engine._unit_backward_done(ctx.unit_idx)
        return g, None, None


class _PreBackward(torch.autograd.Function):
    """Identity on a unit's *output*; its backward runs before the unit's own backward and makes
    sure the unit's full parameters are back in their slot."""

    @staticmethod
    def forward(ctx, x, engine, unit_idx):
        ctx.engine, ctx.unit_idx = engine, unit_idx
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        ctx.engine._materialize(ctx.unit_idx, direction=-1)
        return g, None, None


class FSDP:
    def __init__(self, model: nn.Module, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999,
                 eps: float = 1e-8, weight_decay: float = 0.0, adamw: bool = False,
                 group: Optional[dist.ProcessGroup] = None, mode: Optional[str] = None,
                 unit_roots: Optional[list] = None, arena=None, local_only: bool = False,
                 reshard_after_forward: bool = False, defer_update: bool = False):
        self.model = model
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps
        self.weight_decay, self.adamw = weight_decay, adamw
        self.group = group
        # ``defer_update``: several backward passes feed one optimizer step (pipeline micro-batches,
        # gradient accumulation), so a unit is only reduced and updated from ``step()``, never from
        # the boundary node that fires at the end of each backward pass
        self._defer = bool(defer_update)
        # ``local_only``: no sharding (the parameters of a tensor/pipeline-parallel stage are
        # already this rank's own); the engine is then just the flat-arena fused optimizer
        self.world = dist.get_world_size(group) if dist.is_initialized() and not local_only else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() and not local_only else 0
        mode = mode or os.environ.get("RB_BACKEND", "fused")
        dev = next(model.parameters()).device
        if self.world == 1:
            mode = "local"
        elif dev.type != "cuda":
            mode = "cpu"   # gloo ranks: same schedule, collectives through torch.distributed
        self.mode = mode
        self.arena = arena
        alloc = None
        self._reshard = bool(reshard_after_forward) and self.world > 1
        param_alloc_for = None
        if mode == "fused":
            from .symm import SymmArena
            total = sum(p.numel() for p in model.parameters())
            blocks = getattr(model, "blocks", None)
            in_blocks = sum(p.numel() for b in blocks for p in b.parameters()) if blocks is not None else 0
            if self._reshard:
                # peer-visible: all gradients, the resident units' parameters, the blocks' shards
                elems = total + (total - in_blocks) + in_blocks // self.world
                plain = lambda n, dt, dev: torch.zeros(n, dtype=dt, device=dev)   # noqa: E731
                param_alloc_for = lambda name: plain if name.startswith("blocks.") else None   # noqa: E731
            else:
                elems = 2 * total
            if self.arena is None:
                self.arena = SymmArena(int(elems * 2 * 1.05) + (64 << 20), group)
            alloc = self.arena.alloc_flat
        self.units: List[FlatUnit] = build_units(model, unit_roots or default_units(model),
                                                 self.world, self.rank, alloc, param_alloc_for)
        self.step_count = 0
        self._pending: List[int] = []
        self._cuda = dev.type == "cuda"
        # highest priority: when SM resources free up, pending communication CTAs are placed before
        # the next compute kernel's, so the collectives run in the shadow of the backward pass
        # instead of piling up behind it
        self.comm_stream = (torch.cuda.Stream(device=dev, priority=-1)
                            if self._cuda and self.world > 1 else None)
        self._unit_events = [None] * len(self.units)
        self._trace = None
        self._install_boundaries()
        self._resharded: List[int] = []
        if self._reshard:
            self._setup_reshard()
        if mode == "fused":
            from .fused_fsdp import FusedFsdpComm
            self.fused = FusedFsdpComm(self)
        else:
            self.fused = None

    # ------------------------------------------------------------------ wiring
    def _install_boundaries(self) -> None:
        """Route the input of every block (and of the tail) through a boundary node."""
        blocks = getattr(self.model, "blocks", None)
        name_to_idx = {u.name: i for i, u in enumerate(self.units)}
        engine = self
        if blocks is not None:
            for i, b in enumerate(blocks):
                idx = name_to_idx.get(f"blocks.{i}")
                if idx is None:
                    continue
                orig = b.forward

                def fwd(x, *a, _orig=orig, _idx=idx, **kw):
                    if torch.is_grad_enabled() and x.requires_grad:
                        x = _Boundary.apply(x, engine, _idx)
                    if not engine._reshard:
                        return _orig(x, *a, **kw)
                    engine._materialize(_idx, direction=+1)
                    out = _orig(x, *a, **kw)
                    if torch.is_grad_enabled() and isinstance(out, torch.Tensor) and out.requires_grad:
                        out = _PreBackward.apply(out, engine, _idx)
                    return out

                b.forward = fwd
        tail_idx = name_to_idx.get("tail")
        ln_final = getattr(self.model, "ln_final", None)
        if tail_idx is not None and ln_final is not None:
            orig = ln_final.forward

            def fwd_tail(x, *a, _orig=orig, **kw):
                if torch.is_grad_enabled() and x.requires_grad:
                    x = _Boundary.apply(x, engine, tail_idx)
                return _orig(x, *a, **kw)

            ln_final.forward = fwd_tail
        self._hooked = {i for n, i in name_to_idx.items() if n.startswith("blocks.") or n == "tail"}
        self._first_hooked = min(self._hooked) if self._hooked else -1

    # ------------------------------------------------------------------ resharding (ZeRO-3 flow)
    def _setup_reshard(self) -> None:
        """Blocks give up their full parameter buffers; embeddings and the tail (used at both ends
        of every step) stay resident."""
        self._resharded = sorted(i for i, u in enumerate(self.units) if u.name.startswith("blocks."))
        if not self._resharded:
            self._reshard = False
            return
        u0 = self.units[self._resharded[0]]
        size = max(self.units[i].padded for i in self._resharded)
        self._slots = [torch.zeros(size, dtype=u0.dtype, device=u0.device) for _ in range(2)]
        self._slot_of = {idx: k % 2 for k, idx in enumerate(self._resharded)}
        self._slot_owner = [None, None]
        self._slot_event = [None, None]
        self.gather_stream = torch.cuda.Stream(device=u0.device) if self._cuda else None
        self.gathers_issued = 0
        # fused mode: peers read the shards, so they live in the arena; the slots stay local
        shard_alloc = self.arena.alloc_flat if self.mode == "fused" else None
        for idx in self._resharded:
            self.units[idx].reshard(self._slots[self._slot_of[idx]], shard_alloc)

    def _gather_into_slot(self, idx: int) -> None:
        s = self._slot_of[idx]
        if self._slot_owner[s] == idx:
            return
        u = self.units[idx]
        slot = self._slots[s][: u.padded]
        if self._cuda:
            # every kernel that still reads the slot's previous owner was enqueued before this point
            self.gather_stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self.gather_stream), trace_range(f"fsdp.gather.{u.name}"):
                if self.mode == "fused":
                    self.fused.gather_shards(idx, slot)
                else:
                    dist.all_gather_into_tensor(slot, u.persist, group=self.group)
                ev = torch.cuda.Event()
                ev.record(self.gather_stream)
            self._slot_event[s] = ev
        else:
            dist.all_gather_into_tensor(slot, u.persist, group=self.group)
        self._slot_owner[s] = idx
        self.gathers_issued += 1

    def _materialize(self, idx: int, direction: int) -> None:
        """Full parameters of unit ``idx`` into its slot (no-op if they are still there), then the
        gather of the unit that runs next in ``direction`` (+1 forward, -1 backward) is started
        into the other slot so that it overlaps this unit's compute."""
        if idx not in self._slot_of:
            return
        self._gather_into_slot(idx)
        if self._cuda and self._slot_event[self._slot_of[idx]] is not None:
            torch.cuda.current_stream().wait_event(self._slot_event[self._slot_of[idx]])
        k = self._resharded.index(idx) + direction
        if 0 <= k < len(self._resharded):
            self._gather_into_slot(self._resharded[k])

    @contextlib.contextmanager
    def summon_full_params(self, writeback: bool = False):
        """Inside the block every parameter of the model holds its full, current value (needed to
        read a state dict, or with ``writeback`` to load one: on exit each rank keeps its shard of
        what was written).  Collective: every rank must enter.  A no-op unless parameters are
        resharded."""
        if not self._reshard:
            yield
            return
        for idx in self._resharded:
            u = self.units[idx]
            full = torch.empty(u.padded, dtype=u.dtype, device=u.device)
            dist.all_gather_into_tensor(full, u.persist, group=self.group)
            u.bind_storage(full)
        try:
            yield
        finally:
            for idx in self._resharded:
                u = self.units[idx]
                if writeback:
                    lo, hi = u.shard_range
                    u.persist.copy_(u.flat_param[lo:hi])
                u.bind_storage(self._slots[self._slot_of[idx]])
            self._slot_owner = [None, None]

    def param_bytes(self) -> int:
        """Bytes of low-precision parameter storage this rank holds between steps."""
        total = 0
        for i, u in enumerate(self.units):
            esz = u.flat_param.element_size()
            total += (u.shard_numel if u.persist is not None else u.padded) * esz
        if self._reshard:
            total += sum(s.numel() * s.element_size() for s in self._slots)
        return total

    # ------------------------------------------------------------------ step protocol
    def zero_grad(self) -> None:
        for u in self.units:
            u.begin_step()
            for p in u.params:
                p.grad = None
        self._done = [False] * len(self.units)

    def _unit_backward_done(self, idx: int) -> None:
        if self._done[idx] or not self._cuda or self._defer:
            # CPU ranks get parameter gradients through plain autograd accumulation, which may
            # run after this node: they finish every unit in step() instead.
            return
        self._done[idx] = True
        # after the first block's backward only the embedding gradient is left to compute: from
        # here on the communication kernels have the GPU to themselves
        self._reduce_and_update(idx, tail=(idx == self._first_hooked))

    def reduce_grads(self, replicated_group: Optional[dist.ProcessGroup] = None,
                     dp_group: Optional[dist.ProcessGroup] = None) -> None:
        """For an engine built with ``local_only`` (a tensor x pipeline parallel stage), between the
        last backward pass and ``step()``:

        * parameters tagged ``_tp_replicated`` (norm weights and row-parallel biases, which every
          tensor-parallel rank holds in full but which only see that rank's token slab) get the SUM
          of their gradients over ``replicated_group``;
        * every gradient is then averaged over ``dp_group`` (replicas that saw different data).

        Both are collectives: every rank of the group has to call this."""
        for u in self.units:
            u.collect_stray_grads()
        if replicated_group is not None and dist.get_world_size(replicated_group) > 1:
            views = [p.main_grad for u in self.units for p in u.params
                     if getattr(p, "_tp_replicated", False)]
            if views:
                flat = torch.cat([v.reshape(-1).float() for v in views])
                dist.all_reduce(flat, group=replicated_group)
                o = 0
                for v in views:
                    v.copy_(flat[o:o + v.numel()].view(v.shape))
                    o += v.numel()
        if dp_group is not None and dist.get_world_size(dp_group) > 1:
            n = dist.get_world_size(dp_group)
            for u in self.units:
                g = u.flat_grad
                if g.is_cuda and g.dtype != torch.float16:
                    dist.all_reduce(g, op=dist.ReduceOp.AVG, group=dp_group)
                else:
                    dist.all_reduce(g, group=dp_group)
                    g.div_(n)

    def step(self) -> None:
        """Call after ``loss.backward()``: finishes the units whose backward did not fire a
        boundary (the embeddings) and makes the updated parameters visible to the next forward."""
        for i in range(len(self.units) - 1, -1, -1):
            if not self._done[i]:
                self._done[i] = True
                self._reduce_and_update(i, tail=True)
        if self.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        if self.fused is not None:
            self.fused.end_step()
        self.step_count += 1

    # ------------------------------------------------------------------ per-unit work
    def _adam_args(self):
        return dict(lr=self.lr, beta1=self.beta1, beta2=self.beta2, eps=self.eps,
                    weight_decay=self.weight_decay, step=self.step_count + 1, adamw=self.adamw)

    def _reduce_and_update(self, idx: int, tail: bool = False) -> None:
        u = self.units[idx]
        u.collect_stray_grads()
        if self.mode == "local":
            if self._cuda:
                native.adam_flat(u.flat_grad, u.master, u.exp_avg, u.exp_avg_sq, u.flat_param,
                                 **self._adam_args())
            else:
                _adam_reference(u.flat_grad.float(), u, **self._adam_args())
            return
        if self.mode == "cpu":
            shard = torch.empty(u.shard_numel, dtype=u.dtype)
            dist.reduce_scatter_tensor(shard, u.flat_grad, op=dist.ReduceOp.SUM, group=self.group)
            _adam_reference(shard.float() / self.world, u, **self._adam_args())
            if u.persist is not None:
                self._invalidate(idx)       # gathered again on next use
            else:
                dist.all_gather_into_tensor(u.flat_param, u.param_shard().clone(), group=self.group)
            return
        cur = torch.cuda.current_stream()
        trace = self._trace
        if trace is not None:
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            ev[0].record(cur)
            trace.append((u.name, ev))
        self.comm_stream.wait_stream(cur)
        with torch.cuda.stream(self.comm_stream), trace_range(f"fsdp.{self.mode}.{u.name}"):
            if trace is not None:
                ev[1].record(self.comm_stream)
            if self.mode == "fused":
                self.fused.reduce_scatter_adam(idx, tail)
                if u.persist is not None:
                    self._invalidate(idx)   # gathered again on next use
                else:
                    self.fused.all_gather(idx, tail)
            else:  # nccl baseline
                shard = u.grad_shard()
                dist.reduce_scatter_tensor(shard, u.flat_grad, op=dist.ReduceOp.AVG, group=self.group)
                native.adam_flat(shard, u.master, u.exp_avg, u.exp_avg_sq, u.param_shard(),
                                 **self._adam_args())
                if u.persist is not None:
                    self._invalidate(idx)   # gathered again on next use
                else:
                    dist.all_gather_into_tensor(u.flat_param, u.param_shard(), group=self.group)
            if trace is not None:
                ev[2].record(self.comm_stream)

    def _invalidate(self, idx: int) -> None:
        s = self._slot_of[idx]
        if self._slot_owner[s] == idx:
            self._slot_owner[s] = None

    def start_trace(self) -> None:
        """Record, for every unit of the following steps, when its backward finished (compute
        stream) and when its reduce-scatter/update/all-gather started and ended (side stream)."""
        self._trace = []

    def stop_trace(self, origin: "torch.cuda.Event"):
        """Returns ``[(unit, backward_done_ms, comm_start_ms, comm_end_ms)]`` relative to ``origin``."""
        torch.cuda.synchronize()
        out = [(n, origin.elapsed_time(e[0]), origin.elapsed_time(e[1]), origin.elapsed_time(e[2]))
               for n, e in (self._trace or [])]
        self._trace = None
        return out

    # ------------------------------------------------------------------ state
    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def get_lr(self) -> float:
        return self.lr

    def optimizer_state(self) -> dict:
        """This rank's shard of the optimizer state (for ``optim-rank{r}.safetensors``)."""
        out = {}
        for u in self.units:
            out[f"{u.name}.master"] = u.master
            out[f"{u.name}.exp_avg"] = u.exp_avg
            out[f"{u.name}.exp_avg_sq"] = u.exp_avg_sq
        return out

    def load_optimizer_state(self, sd: dict) -> None:
        for u in self.units:
            u.master.copy_(sd[f"{u.name}.master"])
            u.exp_avg.copy_(sd[f"{u.name}.exp_avg"])
            u.exp_avg_sq.copy_(sd[f"{u.name}.exp_avg_sq"])
            u.param_shard().copy_(u.master)
        if self.world > 1:
            for i, u in enumerate(self.units):
                if u.persist is not None:
                    self._invalidate(i)
                else:
                    dist.all_gather_into_tensor(u.flat_param, u.param_shard().clone(), group=self.group)


def _adam_reference(g32, u: FlatUnit, *, lr, beta1, beta2, eps, weight_decay, step, adamw):
    m, v, w = u.exp_avg, u.exp_avg_sq, u.master
    m.mul_(beta1).add_(g32, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g32, g32, value=1 - beta2)
    if adamw:
        w.mul_(1 - lr * weight_decay)
    w.sub_(lr * (m / (1 - beta1 ** step)) / ((v / (1 - beta2 ** step)).sqrt() + eps))
    u.param_shard().copy_(w)
