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

Used for ``csrc/kernels/w4a16_gemm.cu`` (``w4a16_roles``), the CTA-pair GEMM (``gemm_2cta_roles``) and the
bulk-copy ring of the LayerNorm backward kernel (``norm_ring_roles``) and the window / accumulator
hand-offs of the direct stem convolution's weight-gradient kernel (``conv_stem_wgrad_roles``).
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


def gemm_2cta_roles(num_tiles: int, num_kb: int, stages: int = 6, epi_warps: int = 2, bug: str = "") -> Dict[str, Role]:
    """The CTA pair of ``gemm_pair_body`` (``csrc/kernels/gemm_pair.cuh``, 256 x 256 tiles) walking ``num_tiles`` tiles
    of ``num_kb`` K blocks: a copy producer per CTA (both complete on the leader's ``full`` barrier,
    whose expected byte count the leader alone arms), the leader's MMA issuer (its commits release
    the stage in both CTAs and hand the accumulator to both CTAs' epilogue warps), ``epi_warps``
    epilogue warps per CTA (they release the accumulator on the leader's barrier and finally arrive
    on both CTAs' ``done`` barriers).  Transaction bytes are modelled as a count that may run ahead
    of the arming (a copy of the peer may land first).  ``bug``: ``"peer_not_released"`` (the leader
    forgets the commit into the peer's ``empty`` barrier), ``"half_tx"`` (the leader arms the barrier
    for its own bytes only)."""
    full = [{"bar": Mbar(1), "tx": 0} for _ in range(stages)]          # leader's
    empty = [[Mbar(1) for _ in range(stages)] for _ in range(2)]        # per CTA
    tmem_full = [[Mbar(1) for _ in range(2)] for _ in range(2)]         # per CTA, per accumulator
    tmem_empty = [Mbar(2 * epi_warps) for _ in range(2)]                # leader's
    done = [Mbar(2 * epi_warps) for _ in range(2)]
    stage_tag = [[None] * stages for _ in range(2)]                     # (tile, kb) held by each CTA's stage
    acc_tag = [None, None]                                              # tile held by each accumulator
    state = {"reading": None, "finished": 0}
    PER_CTA_TX = 2                                                      # A box + B box

    def full_complete(s, parity):
        # the phase can only complete after the leader's arrival; bytes must have netted to zero
        return full[s]["bar"].passed(parity)

    def tx_done(s):
        f = full[s]
        if f.get("armed") and f["tx"] == 0:
            f["armed"] = False
            f["bar"].arrive()

    def producer(cta: int):
        stage, phase, issued = 0, 0, 0
        for tile in range(num_tiles):
            for kb in range(num_kb):
                yield (lambda s=stage, ph=phase: empty[cta][s].passed(ph ^ 1))
                issued += 1
                if state["reading"] == stage:
                    raise PipelineError(f"CTA {cta}: stage {stage} overwritten while the MMA reads it")
                if cta == 0:
                    full[stage]["tx"] += PER_CTA_TX if bug == "half_tx" else 2 * PER_CTA_TX
                    full[stage]["armed"] = True
                for _ in range(PER_CTA_TX):
                    yield (lambda: True)                    # the copy lands later
                    full[stage]["tx"] -= 1
                    stage_tag[cta][stage] = (tile, kb)
                    tx_done(stage)
                if cta == 0:
                    tx_done(stage)
                stage += 1
                if stage == stages:
                    stage, phase = 0, phase ^ 1

    def mma():
        stage, phase, acc, acc_phase = 0, 0, 0, 0
        for tile in range(num_tiles):
            yield (lambda a=acc, ph=acc_phase: tmem_empty[a].passed(ph ^ 1))
            for kb in range(num_kb):
                yield (lambda s=stage, ph=phase: full_complete(s, ph))
                if stage_tag[0][stage] != (tile, kb) or stage_tag[1][stage] != (tile, kb):
                    raise PipelineError(f"MMA tile {tile} kb {kb}: stage {stage} holds {stage_tag[0][stage]} / "
                                        f"{stage_tag[1][stage]}")
                state["reading"] = stage
                yield (lambda: True)
                state["reading"] = None
                empty[0][stage].arrive()
                if bug != "peer_not_released":
                    empty[1][stage].arrive()
                stage += 1
                if stage == stages:
                    stage, phase = 0, phase ^ 1
            acc_tag[acc] = tile
            tmem_full[0][acc].arrive()
            tmem_full[1][acc].arrive()
            acc += 1
            if acc == 2:
                acc, acc_phase = 0, acc_phase ^ 1

    def epilogue(cta: int, w: int):
        acc, acc_phase = 0, 0
        for tile in range(num_tiles):
            yield (lambda a=acc, ph=acc_phase: tmem_full[cta][a].passed(ph))
            if acc_tag[acc] != tile:
                raise PipelineError(f"CTA {cta} epilogue {w}: accumulator {acc} holds tile {acc_tag[acc]}, expected {tile}")
            yield (lambda: True)                            # tcgen05.ld + stores
            if acc_tag[acc] != tile:
                raise PipelineError(f"CTA {cta} epilogue {w}: accumulator {acc} overwritten while it was read")
            tmem_empty[acc].arrive()
            acc += 1
            if acc == 2:
                acc, acc_phase = 0, acc_phase ^ 1
        done[0].arrive()
        done[1].arrive()

    def teardown(cta: int):
        yield (lambda: done[cta].passed(0))
        state["finished"] += 1

    roles: Dict[str, Role] = {"producer0": producer(0), "producer1": producer(1), "mma": mma(),
                              "teardown0": teardown(0), "teardown1": teardown(1)}
    for cta in range(2):
        for w in range(epi_warps):
            roles[f"epi{cta}.{w}"] = epilogue(cta, w)
    return roles


def norm_ring_roles(rows: int, stages: int = 4, threads: int = 3, bug: str = "") -> Dict[str, Role]:
    """One row group of ``norm_bwd_ring_kernel`` (``csrc/kernels/norm.cu``): ``stages`` shared-memory
    slots, each filled by bulk copies that complete on the slot's mbarrier; the group's threads wait for
    a slot, take their part of the row into registers, meet at the group's named barrier, and only then
    does one of them request the row ``stages`` ahead into the slot just emptied.  ``threads`` model
    threads stand for the group's 128.  ``bug``: ``"refill_early"`` requests the next row before the
    barrier (a slot may be overwritten while a slower thread still reads it), ``"parity"`` flips the
    phase one trip late."""
    full = [Mbar(1) for _ in range(stages)]
    tag: List = [None] * stages
    reading = [0] * stages
    requests: List = []                     # (slot, row) issued and not yet landed
    state = {"landed": 0, "done_threads": 0, "arrived": 0, "generation": 0}

    def request(slot, row):
        requests.append((slot, row))

    def engine():
        total = rows
        while state["landed"] < total:
            yield (lambda: bool(requests))
            slot, row = requests.pop(0)
            if reading[slot]:
                raise PipelineError(f"row {row} lands in slot {slot} while {reading[slot]} thread(s) still read it")
            tag[slot] = row
            full[slot].arrive()
            state["landed"] += 1

    def thread(t: int):
        if t == 0:
            for s0 in range(min(stages, rows)):
                request(s0, s0)
        slot, phase = 0, 0
        for i in range(rows):
            yield (lambda slot=slot, phase=phase: full[slot].passed(phase))
            if tag[slot] != i:
                raise PipelineError(f"thread {t}: slot {slot} holds row {tag[slot]}, expected {i}")
            reading[slot] += 1
            yield (lambda: True)            # shared-memory loads into registers
            reading[slot] -= 1
            if bug == "refill_early" and t == 0 and i + stages < rows:
                request(slot, i + stages)
            gen = state["generation"]       # the group's named barrier
            state["arrived"] += 1
            if state["arrived"] == threads:
                state["arrived"] = 0
                state["generation"] += 1
            yield (lambda gen=gen: state["generation"] != gen)
            if bug != "refill_early" and t == 0 and i + stages < rows:
                request(slot, i + stages)
            slot += 1
            if slot == stages:
                slot = 0
                if bug != "parity" or i >= stages:
                    phase ^= 1
        state["done_threads"] += 1

    roles: Dict[str, Role] = {"engine": engine()}
    for t in range(threads):
        roles[f"thread{t}"] = thread(t)
    return roles


def conv_stem_wgrad_roles(tiles: int, threads: int = 3, bug: str = "") -> Dict[str, Role]:
    """One CTA of ``conv_stem_wgrad_kernel`` (``csrc/kernels/conv_stem.cu``) walking ``tiles`` tiles: two
    input buffers (image window + dY tile, filled by TMA on ``full[buf]``), one operand tile that the
    threads rebuild for every tile, MMAs that read the operand tile and the dY buffer and commit to
    ``mma_done``.  Per iteration: wait for the previous tile's MMAs, request the next tile into the other
    buffer, wait for this tile's buffer, build, barrier, issue.  ``bug``: ``"no_mma_wait"`` skips the wait
    for the previous MMAs (the operand tile is rebuilt, and the other dY buffer refilled, under them)."""
    full = [Mbar(1), Mbar(1)]
    mma_done = Mbar(1)
    buf_tag: List = [None, None]
    operand = {"tile": None, "writers": 0}
    state = {"mma_reading": None, "landed": 0, "issued_mma": 0, "arrived": 0, "generation": 0}
    requests: List = []

    def barrier():
        gen = state["generation"]
        state["arrived"] += 1
        if state["arrived"] == threads:
            state["arrived"] = 0
            state["generation"] += 1
        return lambda gen=gen: state["generation"] != gen

    def engine():
        while state["landed"] < tiles:
            yield (lambda: bool(requests))
            buf, tile = requests.pop(0)
            if state["mma_reading"] is not None and state["mma_reading"][1] == buf:
                raise PipelineError(f"tile {tile} lands in buffer {buf} while MMAs still read its dY tile")
            buf_tag[buf] = tile
            full[buf].arrive()
            state["landed"] += 1

    def tensor_core():
        for i in range(tiles):
            yield (lambda i=i: state["issued_mma"] > i)
            yield (lambda: True)            # the MMAs execute asynchronously
            state["mma_reading"] = None
            mma_done.arrive()

    def thread(t: int):
        if t == 0 and tiles > 0:
            requests.append((0, 0))
        for it in range(tiles):
            buf = it & 1
            if it > 0 and bug != "no_mma_wait":
                yield (lambda it=it: mma_done.passed((it - 1) & 1))
            yield barrier()
            if t == 0 and it + 1 < tiles:
                requests.append((buf ^ 1, it + 1))
            yield (lambda buf=buf, it=it: full[buf].passed((it >> 1) & 1))
            if buf_tag[buf] != it:
                raise PipelineError(f"thread {t}: buffer {buf} holds tile {buf_tag[buf]}, expected {it}")
            if state["mma_reading"] is not None:
                raise PipelineError(f"thread {t} rebuilds the operand tile while the MMAs of tile "
                                    f"{state['mma_reading'][0]} read it")
            yield (lambda: True)            # build this thread's operand row
            operand["tile"] = it
            yield barrier()
            if t == 0:
                state["mma_reading"] = (it, buf)
                state["issued_mma"] += 1
        if tiles > 0:
            yield (lambda: mma_done.passed((tiles - 1) & 1))

    roles: Dict[str, Role] = {"engine": engine(), "tensor_core": tensor_core()}
    for t in range(threads):
        roles[f"thread{t}"] = thread(t)
    return roles
