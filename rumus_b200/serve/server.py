"""HTTP front end: ``POST /v1/generate {"token_ids": [...], "max_new_tokens": n}`` ->
``{"generated_ids": [...], "latency_ms": x}`` — the reference's API (rumus-serve/src/server.rs:22-115),
with the latency actually measured (the reference hard-codes 0.0) plus ``GET /metrics``.

The engine runs on its own thread (the reference's dedicated GPU worker thread,
rumus-serve/src/main.rs:74-88); handlers park on an asyncio future per request; a bounded queue
gives back-pressure (HTTP 503 when full).

CLI keeps the reference's flag names (rumus-serve/src/main.rs:13-62):
``--port --max-batch --batch-timeout-ms --vocab-size --hidden-dim --num-heads --num-layers``.
"""
from __future__ import annotations

import argparse
import asyncio
import itertools
import queue
import threading
import time
from typing import Dict

import torch

from ..models.llama import LlamaConfig
from .engine import Engine, ServeConfig


class EngineWorker:
    """Owns the engine thread.  With tensor parallelism this is rank 0's worker: before every engine
    step it tells the other ranks which requests joined (one host-side broadcast over ``cpu_group``),
    so every rank adds the same requests before the same step; ``follower_loop`` is what the other
    ranks run."""

    def __init__(self, engine: Engine, max_queue: int = 1024, idle_sleep_s: float = 0.0005, cpu_group=None):
        self.engine = engine
        self.cpu_group = cpu_group
        self.inbox: "queue.Queue" = queue.Queue(maxsize=max_queue)
        self.waiters: Dict[int, tuple] = {}
        self.ids = itertools.count(1)
        self.idle_sleep_s = idle_sleep_s
        self.stop_flag = False
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.completed = 0
        self.ttft_ms = []
        self.itl_ms = []          # per request: mean time between output tokens after the first

    def start(self):
        self.thread.start()

    def stop(self):
        self.stop_flag = True
        self.thread.join(timeout=5)

    def _announce(self, new_requests, stop: bool = False) -> None:
        if self.cpu_group is not None:
            import torch.distributed as dist
            dist.broadcast_object_list([("stop",) if stop else ("step", new_requests)], src=0, group=self.cpu_group)

    def submit(self, token_ids, max_new, loop, fut) -> bool:
        try:
            self.inbox.put_nowait((next(self.ids), list(token_ids), int(max_new), loop, fut, time.time()))
            return True
        except queue.Full:
            return False

    def _run(self):
        eng = self.engine
        while not self.stop_flag:
            joined = []
            while True:
                try:
                    rid, toks, max_new, loop, fut, t0 = self.inbox.get_nowait()
                except queue.Empty:
                    break
                if eng.add_request(rid, toks, max_new, arrival=t0):
                    self.waiters[rid] = (loop, fut, t0)
                    joined.append((rid, toks, max_new))
                else:
                    loop.call_soon_threadsafe(fut.set_exception, ValueError("request does not fit the KV pool"))
            if not eng.has_work():
                time.sleep(self.idle_sleep_s)     # the other ranks stay parked in their broadcast
                continue
            self._announce(joined)
            for rid in eng.step():
                req = eng.requests.pop(rid)
                loop, fut, t0 = self.waiters.pop(rid)
                self.completed += 1
                now = time.time()
                if req.first_token_time:
                    self.ttft_ms.append((req.first_token_time - t0) * 1e3)
                    if len(req.output) > 1:
                        self.itl_ms.append((now - req.first_token_time) * 1e3 / (len(req.output) - 1))
                res = {"generated_ids": req.output, "latency_ms": (time.time() - t0) * 1e3}
                loop.call_soon_threadsafe(fut.set_result, res)


def follower_loop(engine: Engine, cpu_group) -> None:
    """Ranks other than 0 of a tensor-parallel server: take rank 0's word for which requests join,
    then run the same engine step (its collectives pair up with rank 0's)."""
    import torch.distributed as dist
    while True:
        box = [None]
        dist.broadcast_object_list(box, src=0, group=cpu_group)
        msg = box[0]
        if msg[0] == "stop":
            return
        for rid, toks, max_new in msg[1]:
            engine.add_request(rid, toks, max_new)
        for rid in engine.step():
            engine.requests.pop(rid, None)


def build_app(worker: EngineWorker):
    from aiohttp import web

    async def generate(request: "web.Request"):
        try:
            body = await request.json()
            toks = body["token_ids"]
            max_new = int(body.get("max_new_tokens", 16))
        except Exception:
            return web.json_response({"error": "bad request"}, status=400)
        if not toks:
            return web.json_response({"error": "token_ids must be non-empty"}, status=400)
        loop = asyncio.get_running_loop()
        fut = loop.create_future()
        if not worker.submit(toks, max_new, loop, fut):
            return web.json_response({"error": "queue full"}, status=503)
        try:
            return web.json_response(await fut)
        except Exception as e:  # noqa: BLE001
            return web.json_response({"error": str(e)}, status=500)

    async def metrics(request):
        e = worker.engine
        tt = sorted(worker.ttft_ms)
        p50 = tt[len(tt) // 2] if tt else 0.0
        it = sorted(worker.itl_ms)
        itl50 = it[len(it) // 2] if it else 0.0
        total_blocks = e.cfg.num_blocks
        txt = (f"rumus_requests_completed {worker.completed}\n"
               f"rumus_tokens_generated {e.tokens_out}\n"
               f"rumus_engine_steps {e.steps}\n"
               f"rumus_kv_free_blocks {e.sched.free_blocks()}\n"
               f"rumus_kv_block_utilisation {1.0 - e.sched.free_blocks() / max(1, total_blocks):.4f}\n"
               f"rumus_queue_waiting {e.sched.num_waiting()}\n"
               f"rumus_running {e.sched.num_running()}\n"
               f"rumus_preemptions {e.sched.preemptions()}\n"
               f"rumus_ttft_p50_ms {p50:.3f}\n"
               f"rumus_inter_token_latency_p50_ms {itl50:.3f}\n")
        return web.Response(text=txt)

    app = web.Application()
    app.router.add_post("/v1/generate", generate)
    app.router.add_get("/metrics", metrics)
    return app


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--port", type=int, default=3000)
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--batch-timeout-ms", type=int, default=5,
                    help="kept for CLI compatibility; continuous batching has no collection deadline")
    ap.add_argument("--vocab-size", type=int, default=32000)
    ap.add_argument("--hidden-dim", type=int, default=512)
    ap.add_argument("--num-heads", type=int, default=4)
    ap.add_argument("--num-layers", type=int, default=2)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--tp", type=int, default=1,
                    help="tensor-parallel degree: start that many ranks with python -m torch.distributed.run; "
                         "rank 0 serves HTTP, the others follow its schedule")
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"])
    a = ap.parse_args(argv)
    import os
    from datetime import timedelta
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if a.tp != world:
        raise SystemExit(f"--tp {a.tp} but {world} rank(s) were started")
    dev = torch.device(a.device)
    cpu_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if dev.type == "cuda":
            dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
            torch.cuda.set_device(dev)
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
        # followers park in a broadcast until rank 0 has a step for them: no timeout to speak of
        cpu_group = dist.new_group(backend="gloo", timeout=timedelta(days=7))
    mc = LlamaConfig(vocab_size=a.vocab_size, d_model=a.hidden_dim, num_heads=a.num_heads,
                     num_kv_heads=a.num_heads, num_layers=a.num_layers, ffn_dim=4 * a.hidden_dim,
                     seq_len=2048)
    cfg = ServeConfig(model=mc, max_batch=a.max_batch, num_blocks=1024, comm_mode=a.comm,
                      dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32,
                      scale_dtype=torch.float16 if dev.type == "cuda" else torch.float32)
    engine = Engine(cfg, dev)
    engine.warmup_graphs()          # every rank: the decode graphs are captured before traffic arrives
    if world > 1 and dist.get_rank() != 0:
        follower_loop(engine, cpu_group)
        dist.destroy_process_group()
        return
    from aiohttp import web
    worker = EngineWorker(engine, cpu_group=cpu_group)
    worker.start()
    try:
        web.run_app(build_app(worker), port=a.port)
    finally:
        worker.stop()
        if world > 1:
            worker._announce([], stop=True)
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
