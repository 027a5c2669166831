"""Host model of an intra-kernel mbarrier pipeline: roles as coroutines, barriers with the hardware's
phase-parity semantics, a randomised scheduler, and data-hazard bookkeeping.

A warp-specialised kernel is a handful of roles (copy producers, MMA issuer, conversion warps,
epilogue) that hand shared-memory stages to each other through mbarriers.  Whether the ring indices,
arrival counts and phase parities are right — no deadlock, no stage overwritten before its consumer
is done, no stage consumed before all of its producers have written — can be decided on the host:
the roles below restate the loop structure of a kernel (same stage / parity expressions), the
scheduler interleaves them at random, and every shared-memory stage carries a tag saying what it
holds, which consumers check.

``Mbar`` follows ``mbarrier.try_wait.parity``: a barrier starts in phase 0; ``wait(p)`` succeeds
when the phase of parity ``p`` has completed, i.e. when the current phase's parity differs from
``p`` (so waiting for parity 1 on a fresh barrier succeeds at once — the idiom producers use for
"the stage is free the first time round").  A phase completes when ``count`` arrivals have been
made (a TMA transaction or a ``tcgen05.commit`` counts as one arrival here).

Used for ``csrc/kernels/w4a16_gemm.cu`` (``w4a16_roles``).
"""
from __future__ import annotations

import random
from typing import Callable, Dict, Generator, List


class PipelineError(AssertionError):
    pass


class Mbar:
    def __init__(self, count: int):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self) -> None:
        self.pending -= 1
        if self.pending < 0:
            raise PipelineError("more arrivals than the barrier was initialised for")
        if self.pending == 0:
            self.phase ^= 1
            self.pending = self.count

    def passed(self, parity: int) -> bool:
        return self.phase != parity


Role = Generator[Callable[[], bool], None, None]


def run(roles: Dict[str, Role], seed: int = 0, max_steps: int = 1_000_000) -> int:
    """Runs the roles to completion under a random schedule.  A role yields a predicate when it has
    to wait; it is resumed only once the predicate holds.  Raises on deadlock."""
    rng = random.Random(seed)
    waiting: Dict[str, Callable[[], bool]] = {}
    live = dict(roles)
    for name, g in list(live.items()):      # run every role up to its first wait
        try:
            waiting[name] = next(g)
        except StopIteration:
            del live[name]
    steps = 0
    while live:
        ready = [n for n in live if waiting[n]()]
        if not ready:
            raise PipelineError(f"deadlock: {sorted(live)} all blocked")
        n = rng.choice(ready)
        try:
            waiting[n] = next(live[n])
        except StopIteration:
            del live[n]
            del waiting[n]
        steps += 1
        if steps > max_steps:
            raise PipelineError("did not finish")
    return steps


def w4a16_roles(nkb: int, raw_stages: int = 8, ab_stages: int = 3, dequant_warps: int = 4,
                bug: str = "") -> Dict[str, Role]:
    """The roles of ``w4a16_gemm_kernel`` for one CTA that walks ``nkb`` k-blocks: packed-weight TMA
    (raw ring), activation TMA, ``dequant_warps`` conversion warps (raw ring -> operand stage), the
    MMA issuer, and the epilogue the conversion warps turn into.  Stage contents are tagged with the
    k-block they hold.  ``bug`` plants a defect so that tests can see the model catch it:
    ``"no_stage_wait"`` (conversion warps do not wait for the operand stage to be released),
    ``"raw_count"`` (the raw ring's release barrier expects one arrival too few),
    ``"parity"`` (the weight TMA waits on the wrong parity)."""
    raw_full = [Mbar(1) for _ in range(raw_stages)]
    raw_empty = [Mbar(dequant_warps - (1 if bug == "raw_count" else 0)) for _ in range(raw_stages)]
    a_full = [Mbar(dequant_warps) for _ in range(ab_stages)]
    x_full = [Mbar(1) for _ in range(ab_stages)]
    ab_empty = [Mbar(1) for _ in range(ab_stages)]
    acc_full = Mbar(1)
    raw = [None] * raw_stages                                   # k-block held by each raw stage
    a_tile = [[None] * dequant_warps for _ in range(ab_stages)]  # per conversion warp's quarter
    x_tile = [None] * ab_stages
    consumed: List[int] = []
    state = {"mma_reading": None, "acc_done": False, "epilogues": 0}

    def yield_point():
        return lambda: True

    def tma_w():
        r, ph = 0, 0
        for i in range(nkb):
            yield (lambda r=r, ph=ph: raw_empty[r].passed(ph if bug == "parity" else ph ^ 1))
            # the copy lands some time later: model the landing as a separate step
            yield yield_point()
            raw[r] = i
            raw_full[r].arrive()
            r += 1
            if r == raw_stages:
                r, ph = 0, ph ^ 1

    def tma_x():
        s, ph = 0, 0
        for i in range(nkb):
            yield (lambda s=s, ph=ph: ab_empty[s].passed(ph ^ 1))
            if state["mma_reading"] == s:
                raise PipelineError(f"activation stage {s} overwritten while the MMA reads it")
            yield yield_point()
            x_tile[s] = i
            x_full[s].arrive()
            s += 1
            if s == ab_stages:
                s, ph = 0, ph ^ 1

    def dequant(w: int):
        r = s = 0
        rph = sph = 0
        for i in range(nkb):
            yield (lambda r=r, rph=rph: raw_full[r].passed(rph))
            if raw[r] != i:
                raise PipelineError(f"warp {w}: raw stage {r} holds k-block {raw[r]}, expected {i}")
            words = raw[r]                    # into registers
            raw_empty[r].arrive()
            r += 1
            if r == raw_stages:
                r, rph = 0, rph ^ 1
            if bug != "no_stage_wait":
                yield (lambda s=s, sph=sph: ab_empty[s].passed(sph ^ 1))
            if state["mma_reading"] == s:
                raise PipelineError(f"warp {w}: operand stage {s} overwritten while the MMA reads it")
            a_tile[s][w] = words
            yield yield_point()               # stores, proxy fence
            a_full[s].arrive()
            s += 1
            if s == ab_stages:
                s, sph = 0, sph ^ 1
        yield (lambda: acc_full.passed(0))
        if not state["acc_done"] or len(consumed) != nkb:
            raise PipelineError("epilogue started before the last MMA was committed")
        state["epilogues"] += 1

    def mma():
        s, ph = 0, 0
        for i in range(nkb):
            yield (lambda s=s, ph=ph: a_full[s].passed(ph))
            yield (lambda s=s, ph=ph: x_full[s].passed(ph))
            if any(t != i for t in a_tile[s]) or x_tile[s] != i:
                raise PipelineError(f"MMA {i}: stage {s} holds weights {a_tile[s]} / activations {x_tile[s]}")
            state["mma_reading"] = s
            yield yield_point()               # the MMAs execute asynchronously
            state["mma_reading"] = None
            consumed.append(i)
            ab_empty[s].arrive()              # tcgen05.commit
            s += 1
            if s == ab_stages:
                s, ph = 0, ph ^ 1
        state["acc_done"] = True
        acc_full.arrive()

    roles: Dict[str, Role] = {"tma_w": tma_w(), "tma_x": tma_x(), "mma": mma()}
    for w in range(dequant_warps):
        roles[f"dequant{w}"] = dequant(w)
    roles["_check"] = _final_check(state, consumed, nkb, dequant_warps)
    return roles


def _final_check(state, consumed, nkb, warps) -> Role:
    yield (lambda: state["epilogues"] == warps)
    if consumed != list(range(nkb)):
        raise PipelineError(f"k-blocks consumed out of order: {consumed}")
