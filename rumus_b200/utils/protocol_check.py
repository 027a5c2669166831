"""Exhaustive interleaving check of the epoch-flag protocols used by the fused collective kernels.

The kernels synchronise through monotonically increasing flags in peer-visible memory
(``st.release.sys`` / ``ld.acquire.sys``, ``csrc/comm/comm_common.cuh``).  Whether a protocol needs
an extra barrier is a question about interleavings, not about one run, so it is answered on a
model: every rank is a straight-line program of atomic actions and the checker walks every
reachable interleaving (memoised on the ranks' program counters — memory contents are a function
of them because the programs are deterministic), reporting

* a read that observes another version than the one the protocol promises,
* a write to a buffer while a peer is in the middle of reading it (write-after-read hazard),
* a deadlock (nobody can move, somebody is not finished).

Actions: ``("write", buf, version)``, ``("set", flag, value)``, ``("wait", flag, value)``
(blocks until ``flag >= value``), ``("begin_read", buf, version)``, ``("end_read", buf)``.
"""
from __future__ import annotations

from typing import Dict, List, Sequence, Tuple

Action = Tuple


class ProtocolViolation(AssertionError):
    pass


def explore(programs: Sequence[Sequence[Action]], max_states: int = 2_000_000) -> int:
    """Walks every interleaving of ``programs``; returns the number of distinct states visited.
    Raises ``ProtocolViolation`` on the first violation."""
    n = len(programs)

    def memory(pcs):
        """(buffer versions, flag values, open reads) implied by the program counters."""
        ver: Dict[str, int] = {}
        flags: Dict[str, int] = {}
        reading: Dict[str, int] = {}
        for r in range(n):
            for a in programs[r][:pcs[r]]:
                if a[0] == "write":
                    ver[a[1]] = max(ver.get(a[1], 0), a[2])
                elif a[0] == "set":
                    flags[a[1]] = max(flags.get(a[1], 0), a[2])
                elif a[0] == "begin_read":
                    reading[a[1]] = reading.get(a[1], 0) + 1
                elif a[0] == "end_read":
                    reading[a[1]] -= 1
        return ver, flags, reading

    seen = set()
    stack: List[Tuple[int, ...]] = [tuple(0 for _ in range(n))]
    while stack:
        pcs = stack.pop()
        if pcs in seen:
            continue
        seen.add(pcs)
        if len(seen) > max_states:
            raise RuntimeError("state space larger than max_states")
        ver, flags, reading = memory(pcs)
        moved = False
        for r in range(n):
            if pcs[r] >= len(programs[r]):
                continue
            a = programs[r][pcs[r]]
            if a[0] == "wait" and flags.get(a[1], 0) < a[2]:
                continue
            if a[0] == "write" and reading.get(a[1], 0) > 0:
                raise ProtocolViolation(f"rank {r} writes {a[1]} (version {a[2]}) while it is being read; pcs={pcs}")
            if a[0] == "begin_read" and ver.get(a[1], 0) != a[2]:
                raise ProtocolViolation(
                    f"rank {r} reads {a[1]} at version {ver.get(a[1], 0)}, expected {a[2]}; pcs={pcs}")
            moved = True
            nxt = list(pcs)
            nxt[r] += 1
            stack.append(tuple(nxt))
        if not moved and any(pcs[r] < len(programs[r]) for r in range(n)):
            raise ProtocolViolation(f"deadlock at pcs={pcs}")
    return len(seen)


def fsdp_unit_programs(world: int, steps: int, wait_param_flags: bool = True,
                       wait_grad_flags: bool = True) -> List[List[Action]]:
    """One sharding unit of the fused FSDP step (``parallel/fused_fsdp.py``): per optimizer step a
    rank writes its gradients, announces them, waits for every announcement, reads its slice of
    every rank's gradients, rewrites its parameter shard, announces it, and pulls every peer's
    shard after that peer's announcement; the next step's gradient write follows in program order.
    The two switches remove one of the waits (used to show that the checker finds the hazard)."""
    progs: List[List[Action]] = []
    for r in range(world):
        p: List[Action] = []
        for t in range(1, steps + 1):
            p.append(("write", f"grad{r}", t))
            for q in range(world):
                p.append(("set", f"grad_ready[{q}][{r}]", t))
            if wait_grad_flags:
                for q in range(world):
                    p.append(("wait", f"grad_ready[{r}][{q}]", t))
            for q in range(world):
                p.append(("begin_read", f"grad{q}", t))
                p.append(("end_read", f"grad{q}"))
            p.append(("write", f"shard{r}", t))
            for q in range(world):
                p.append(("set", f"param_ready[{q}][{r}]", t))
            for q in range(world):
                if q == r:
                    continue
                if wait_param_flags:
                    p.append(("wait", f"param_ready[{r}][{q}]", t))
                p.append(("begin_read", f"shard{q}", t))
                p.append(("end_read", f"shard{q}"))
        progs.append(p)
    return progs


def allreduce_programs(world: int, steps: int, exit_barrier: bool = True) -> List[List[Action]]:
    """The in-place all-reduce + unscale of a gradient bucket (``allreduce_unscale_kernel``): enter
    flags (my bucket is complete), every rank reduces its slice from all peers and writes the
    result back into every peer's bucket, exit flags (my writes are done) before anyone may start
    the next step's gradient writes.  Buffers are modelled per (owner, slice)."""
    progs: List[List[Action]] = []
    for r in range(world):
        p: List[Action] = []
        for t in range(1, steps + 1):
            v_in, v_out = 2 * t - 1, 2 * t
            for s in range(world):
                p.append(("write", f"bucket{r}.slice{s}", v_in))     # backward fills the bucket
            for q in range(world):
                p.append(("set", f"enter[{q}][{r}]", t))
            for q in range(world):
                p.append(("wait", f"enter[{r}][{q}]", t))
            for q in range(world):                                   # reduce my slice from everyone
                p.append(("begin_read", f"bucket{q}.slice{r}", v_in))
                p.append(("end_read", f"bucket{q}.slice{r}"))
            for q in range(world):                                   # broadcast the reduced slice
                p.append(("write", f"bucket{q}.slice{r}", v_out))
            for q in range(world):
                p.append(("set", f"exit[{q}][{r}]", t))
            if exit_barrier:
                for q in range(world):
                    p.append(("wait", f"exit[{r}][{q}]", t))
            for s in range(world):                                   # optimizer reads the reduced bucket
                p.append(("begin_read", f"bucket{r}.slice{s}", v_out))
                p.append(("end_read", f"bucket{r}.slice{s}"))
        progs.append(p)
    return progs


def fsdp_reshard_programs(world: int, steps: int, wait_param_flags: bool = True,
                          wait_grad_flags: bool = True) -> List[List[Action]]:
    """One unit of the FSDP step with parameters resharded between uses (``shard_gather_kernel`` in
    ``csrc/comm/fsdp_comm.cu``): at step ``t`` a rank pulls every peer's persistent shard twice
    (for the forward and again for the backward) once the peer's ``param_ready`` flag shows the
    update of step ``t-1``, then announces its gradients, waits for every announcement, reduces its
    slice, overwrites its own shard and announces ``param_ready = t``.  The gathered copies live in
    local memory and are not modelled.  What keeps a rank from overwriting its shard while a slow
    peer is still gathering it is the gradient announcement: a peer only announces after its
    backward, which comes after its second gather."""
    progs: List[List[Action]] = []
    for r in range(world):
        p: List[Action] = []
        for t in range(1, steps + 1):
            for _use in ("forward", "backward"):
                for q in range(world):
                    if q == r:
                        continue
                    if wait_param_flags:
                        p.append(("wait", f"param_ready[{r}][{q}]", t - 1))
                    p.append(("begin_read", f"shard{q}", t - 1))
                    p.append(("end_read", f"shard{q}"))
            p.append(("write", f"grad{r}", t))
            for q in range(world):
                p.append(("set", f"grad_ready[{q}][{r}]", t))
            if wait_grad_flags:
                for q in range(world):
                    p.append(("wait", f"grad_ready[{r}][{q}]", t))
            for q in range(world):
                p.append(("begin_read", f"grad{q}", t))
                p.append(("end_read", f"grad{q}"))
            p.append(("write", f"shard{r}", t))
            for q in range(world):
                p.append(("set", f"param_ready[{q}][{r}]", t))
        progs.append(p)
    return progs


def rs_push_programs(world: int, steps: int, alternate: bool = True) -> List[List[Action]]:
    """GEMM -> reduce-scatter in its push form (``gemm_rs_push_kernel``): per call every rank adds its
    tiles into each owner's sum buffer (modelled as one sub-buffer per contributing rank), tells the
    owner it is done, and the owner — once everybody said so — reads the sums and puts the buffer back
    to zero.  No barrier follows.  With two buffers used in turn a peer can only reach the next use of a
    buffer after the owner's pass over it (it needs the owner's flag of the call in between, which the
    owner sends after that pass, in program order); with a single buffer (``alternate=False``) a fast
    peer adds the next call's tiles into sums the owner is still reading."""
    progs: List[List[Action]] = []
    for r in range(world):
        p: List[Action] = []
        for t in range(1, steps + 1):
            b = (t & 1) if alternate else 0
            for o in range(world):                                   # epilogue: add my tiles of owner o
                p.append(("write", f"sum{o}.{b}.from{r}", t))
                p.append(("set", f"done[{o}][{r}]", t))
            for q in range(world):                                   # final pass of my own sums
                p.append(("wait", f"done[{r}][{q}]", t))
            for q in range(world):
                p.append(("begin_read", f"sum{r}.{b}.from{q}", t))
                p.append(("end_read", f"sum{r}.{b}.from{q}"))
        progs.append(p)
    return progs


def tp_sequence_programs(world: int, ops: str) -> List[List[Action]]:
    """A sequence of fused tensor-parallel operations on one ``TPContext`` (``parallel/tp.py``,
    ``csrc/comm/tp_comm.cu``).  ``ops`` is a string over

    * ``A`` — all-gather → GEMM: a rank writes its shard of the staging buffer, announces it, and
      pulls every peer's shard after that peer's announcement;
    * ``R`` — GEMM → reduce-scatter: a rank writes partial tiles for every owner into its partial
      buffer, signals the owners, and as an owner reads its tiles from every peer after their signals;
    * ``b`` — a group barrier.

    Neither operation ends with a barrier.  Reusing the staging buffer is safe when ``A`` and ``R``
    alternate (finishing ``R`` needs every peer's tile signal, which a peer sends after its
    preceding ``A`` has completed, and vice versa); two operations of the same kind in a row need
    the barrier between them, which ``TPContext`` inserts."""
    progs: List[List[Action]] = []
    for r in range(world):
        p: List[Action] = []
        for e, op in enumerate(ops, start=1):
            if op == "A":
                p.append(("write", f"stage{r}", e))
                for q in range(world):
                    p.append(("set", f"enter[{q}][{r}]", e))
                for q in range(world):
                    if q == r:
                        continue
                    p.append(("wait", f"enter[{r}][{q}]", e))
                    p.append(("begin_read", f"stage{q}", e))
                    p.append(("end_read", f"stage{q}"))
            elif op == "R":
                for q in range(world):
                    p.append(("write", f"partial{r}.for{q}", e))
                    p.append(("set", f"tile[{q}][{r}]", e))
                for q in range(world):
                    p.append(("wait", f"tile[{r}][{q}]", e))
                    p.append(("begin_read", f"partial{q}.for{r}", e))
                    p.append(("end_read", f"partial{q}.for{r}"))
            elif op == "b":
                for q in range(world):
                    p.append(("set", f"bar[{q}][{r}]", e))
                for q in range(world):
                    p.append(("wait", f"bar[{r}][{q}]", e))
            else:
                raise ValueError(op)
        progs.append(p)
    return progs
