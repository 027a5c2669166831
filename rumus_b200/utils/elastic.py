"""Elastic supervision: run a training job as one process per rank, detect a lost rank, stop the
others in a coordinated way and restart from the last checkpoint — with fewer ranks if asked to —
using the re-sharding checkpoint loader (``io/checkpoint.py``).

The reference has no failure handling: a dead rank leaves its peers blocked forever in
``Condvar::wait_while`` (rumus-distributed/src/collective.rs:64-66,
rumus/src/autograd/backward.rs:1205-1207).

Division of labour:

* inside a rank, ``utils/fault.Heartbeat`` (TCP-store heartbeats) raises ``PeerLost`` before the
  next collective once a peer stopped beating, and the bounded device-side waits turn a stuck
  kernel into ``DeviceWaitTimeout``; either ends the rank's process with a non-zero exit code;
* the supervisor below owns the rank processes.  When one exits abnormally it terminates exactly
  the processes it started (by handle — never by name or pattern), waits for them, and starts a new
  generation: same world size, or one rank fewer when ``shrink_on_failure`` is set (a failed GPU
  does not come back).  Workers find the newest checkpoint themselves (``latest_checkpoint``).

A worker is a picklable ``fn(rank, world, generation, *args)`` run under the ``spawn`` start
method; rendezvous is a fresh port on 127.0.0.1 per generation.
"""
from __future__ import annotations

import os
import socket
import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch.multiprocessing as mp


def _free_port() -> int:
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def latest_checkpoint(root: str, verify: bool = False) -> Optional[str]:
    """Newest complete checkpoint directory ``root/step-<n>`` (complete = has ``trainer_state.json``,
    which ``save_checkpoint`` writes last and atomically), or ``None``.  With ``verify`` a
    checkpoint whose files do not match their recorded digests is skipped in favour of an older
    one."""
    from ..io.checkpoint import verify_checkpoint
    best, best_step = None, -1
    if not os.path.isdir(root):
        return None
    for name in os.listdir(root):
        if not name.startswith("step-"):
            continue
        try:
            step = int(name[5:])
        except ValueError:
            continue
        d = os.path.join(root, name)
        if step > best_step and os.path.exists(os.path.join(d, "trainer_state.json")):
            if verify and not verify_checkpoint(d):
                continue
            best, best_step = d, step
    return best


_stop_event = None


def stop_requested() -> bool:
    """True once the supervisor has asked this generation to stop (a peer was lost).  Workers poll
    it between steps, next to ``Heartbeat.check_peers``, and return: a rank that leaves between
    steps has no kernel or collective in flight.  Ranks that do not return within the grace period
    are terminated by process handle."""
    return _stop_event is not None and _stop_event.is_set()


def _entry(fn, rank, world, generation, port, backend_env, args, stop_event=None):
    global _stop_event
    _stop_event = stop_event
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank),
                       "LOCAL_RANK": str(rank), "WORLD_SIZE": str(world),
                       "RB_ELASTIC_GENERATION": str(generation)})
    os.environ.update(backend_env)
    # a supervised rank may be stopped while its peers still run: its memory must never be bound to
    # an NVLink multicast object (neither the arena's nor NCCL's), whatever the caller's environment says
    os.environ["RB_MULTIMEM"] = "0"
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    fn(rank, world, generation, *args)


@dataclass
class GenerationRecord:
    generation: int
    world: int
    exit_codes: List[Optional[int]]
    failed_ranks: List[int] = field(default_factory=list)
    seconds: float = 0.0


class ElasticSupervisor:
    def __init__(self, fn: Callable, world: int, args: tuple = (), max_restarts: int = 3,
                 shrink_on_failure: bool = False, min_world: int = 1, poll_s: float = 0.05,
                 stop_grace_s: float = 5.0, env: Optional[dict] = None):
        self.fn, self.world, self.args = fn, world, args
        self.max_restarts, self.shrink, self.min_world = max_restarts, shrink_on_failure, min_world
        self.poll_s, self.stop_grace_s = poll_s, stop_grace_s
        self.env = dict(env or {})
        self.history: List[GenerationRecord] = []

    def _run_generation(self, generation: int, world: int) -> GenerationRecord:
        ctx = mp.get_context("spawn")
        port = _free_port()
        stop = ctx.Event()
        procs = [ctx.Process(target=_entry, args=(self.fn, r, world, generation, port, self.env, self.args, stop))
                 for r in range(world)]
        t0 = time.time()
        for p in procs:
            p.start()
        failed: List[int] = []
        while True:
            alive = False
            for r, p in enumerate(procs):
                if p.is_alive():
                    alive = True
                elif p.exitcode not in (0, None) and r not in failed:
                    failed.append(r)
            if failed or not alive:
                break
            time.sleep(self.poll_s)
        if failed:
            # coordinated stop of this generation: first ask (workers that poll ``stop_requested``
            # leave between steps), then end what is left — only the processes started above, by handle
            stop.set()
            deadline = time.time() + self.stop_grace_s
            for p in procs:
                p.join(timeout=max(0.0, deadline - time.time()))
            for p in procs:
                if p.is_alive():
                    p.terminate()
            deadline = time.time() + self.stop_grace_s
            for p in procs:
                p.join(timeout=max(0.0, deadline - time.time()))
            for p in procs:
                if p.is_alive():
                    p.kill()
                    p.join(timeout=1.0)
        else:
            for p in procs:
                p.join()
        return GenerationRecord(generation, world, [p.exitcode for p in procs], failed, time.time() - t0)

    def run(self) -> List[GenerationRecord]:
        """Runs generations until one finishes with every rank exiting 0, or ``max_restarts`` is
        used up (then raises ``RuntimeError``).  Returns the record of every generation."""
        world = self.world
        for generation in range(self.max_restarts + 1):
            rec = self._run_generation(generation, world)
            self.history.append(rec)
            if not rec.failed_ranks and all(c == 0 for c in rec.exit_codes):
                return self.history
            if self.shrink and world > self.min_world:
                world -= 1
        raise RuntimeError(f"job did not finish within {self.max_restarts} restarts: "
                           f"{[(r.generation, r.world, r.failed_ranks) for r in self.history]}")
