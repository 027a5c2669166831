"""Poisson load generator / serving benchmark.

Drives an ``Engine`` in-process with requests whose arrival times follow a Poisson process
(default 32 req/s), prompt lengths U[128, 2048] and output lengths U[128, 512], random token ids —
the serving configuration of the benchmark suite.  Reports generated tokens/s and the p50
time-to-first-token.  Under tensor parallelism every rank runs the same schedule (same seed) and
rank 0 reports.

    python -m rumus_b200.serve.loadgen --requests 64            (1 GPU, scaled-down model)
    python -m torch.distributed.run --nproc-per-node 8 -m rumus_b200.serve.loadgen --tp 8 --model 7b --requests 256
"""
from __future__ import annotations

import argparse
import json
import os
import random
import time

import torch
import torch.distributed as dist

from ..models.llama import LlamaConfig
from .engine import Engine, ServeConfig


def native_status() -> int:
    if not torch.cuda.is_available():
        return 0
    from ..ops import native
    return int(native.read_status())


class ArrivalClock:
    """Which requests have arrived by now.  Under tensor parallelism every rank must add the same
    requests before the same engine step, so rank 0's wall clock decides and the count travels to the
    other ranks (one small host-side broadcast per engine step over a gloo group)."""

    def __init__(self, arrivals, t0: float):
        self.arrivals, self.t0 = arrivals, t0
        self.tp = dist.is_initialized() and dist.get_world_size() > 1
        self.rank = dist.get_rank() if self.tp else 0
        self.cpu_group = dist.new_group(backend="gloo") if self.tp else None
        self._box = torch.zeros(2, dtype=torch.int64)

    def arrived(self, have: int):
        """Returns (number of requests arrived so far, rank 0's time in seconds since the start)."""
        now = time.time() - self.t0
        n = have
        while n < len(self.arrivals) and self.arrivals[n][0] <= now:
            n += 1
        if self.tp:
            self._box[0], self._box[1] = n, int(now * 1e6)
            dist.broadcast(self._box, src=0, group=self.cpu_group)
            n, now = int(self._box[0]), float(self._box[1]) / 1e6
        return n, now


def run(engine: Engine, n_requests: int, rate: float, prompt_rng=(128, 2048), out_rng=(128, 512),
        seed: int = 0, vocab: int = 32000):
    rnd = random.Random(seed)
    t, arrivals = 0.0, []
    for i in range(n_requests):
        t += rnd.expovariate(rate)
        arrivals.append((t, i + 1, [rnd.randrange(vocab) for _ in range(rnd.randint(*prompt_rng))],
                         rnd.randint(*out_rng)))
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    t0 = time.time()
    clock = ArrivalClock(arrivals, t0)
    nxt, done, ttft = 0, 0, []
    while done < n_requests:
        n_arrived, now = clock.arrived(nxt)
        while nxt < n_arrived:
            a = arrivals[nxt]
            engine.add_request(a[1], a[2], a[3], arrival=t0 + a[0])
            nxt += 1
        if not engine.has_work():
            if clock.rank == 0:
                time.sleep(min(0.001, max(0.0, arrivals[nxt][0] - now)) if nxt < n_requests else 0.001)
            continue
        for rid in engine.step():
            r = engine.requests.pop(rid)
            ttft.append((r.first_token_time - r.arrival) * 1e3)
            done += 1
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    wall = time.time() - t0
    ttft.sort()
    return {"requests": n_requests, "wall_s": wall, "generated_tokens": engine.tokens_out,
            "tok_per_s": engine.tokens_out / wall, "ttft_p50_ms": ttft[len(ttft) // 2],
            "ttft_p99_ms": ttft[min(len(ttft) - 1, int(len(ttft) * 0.99))], "steps": engine.steps,
            "preemptions": engine.sched.preemptions()}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="small", choices=["small", "7b"])
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--rate", type=float, default=32.0)
    ap.add_argument("--comm", default="fused", choices=["fused", "nccl"],
                    help="tensor-parallel reductions: one-shot arena kernel, or NCCL all-reduce")
    ap.add_argument("--tp", type=int, default=0,
                    help="tensor-parallel degree; must equal the number of ranks started by torch.distributed.run")
    ap.add_argument("--no-graphs", action="store_true",
                    help="launch every decode kernel from the host instead of replaying captured CUDA graphs")
    ap.add_argument("--num-blocks", type=int, default=0,
                    help="KV-cache blocks per rank (0: sized to at most 35%% of device memory)")
    a = ap.parse_args(argv)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local) if torch.cuda.is_available() else torch.device("cpu")
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    if a.tp and a.tp != world:
        raise SystemExit(f"--tp {a.tp} needs {a.tp} ranks (python -m torch.distributed.run --nproc-per-node {a.tp} "
                         f"-m rumus_b200.serve.loadgen ...), found {world}")
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if dev.type == "cuda":
            dist.init_process_group("nccl", device_id=dev)
        else:
            dist.init_process_group("gloo")
    mc = LlamaConfig.llama_7b() if a.model == "7b" else LlamaConfig(
        vocab_size=32000, seq_len=4096, d_model=1024, num_heads=8, num_kv_heads=8, num_layers=4, ffn_dim=2816)
    num_blocks = a.num_blocks or (8192 if a.model == "7b" else 2048)
    if dev.type == "cuda" and not a.num_blocks:
        # bound the KV cache: block bytes = tokens x layers x (K and V) x local kv heads x head dim x 2 B
        block_size = ServeConfig.__dataclass_fields__["block_size"].default
        per_block = block_size * mc.num_layers * 2 * max(1, mc.num_kv_heads // world) * (mc.d_model // mc.num_heads) * 2
        cap = int(0.35 * torch.cuda.get_device_properties(dev).total_memory / per_block)
        num_blocks = max(64, min(num_blocks, cap))
    cfg = ServeConfig(model=mc, num_blocks=num_blocks, max_batch=128,
                      token_budget=8192, comm_mode=a.comm,
                      dtype=torch.bfloat16 if dev.type == "cuda" else torch.float32,
                      scale_dtype=torch.float16 if dev.type == "cuda" else torch.float32)
    if a.no_graphs:
        cfg.cuda_graphs = False
    eng = Engine(cfg, dev)
    eng.warmup_graphs(max_ctx=2048 + 512)       # prompts U[128,2048] + outputs U[128,512]
    res = run(eng, a.requests, a.rate, vocab=mc.vocab_size)
    if int(os.environ.get("RANK", "0")) == 0:
        res.update({"model": a.model, "tp": world, "rate_req_s": a.rate, "weights": "INT4 g128 fp16 scales",
                    "kv_blocks": num_blocks, "comm_mode": a.comm if world > 1 else "local",
                    "decode_graphs": bool(cfg.cuda_graphs and dev.type == "cuda"),
                    "graph_replays": eng.graph_replays, "graphs_captured": len(eng._graphs), "engine_steps": eng.steps,
                    "device_status": native_status()})
        print(json.dumps(res))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
