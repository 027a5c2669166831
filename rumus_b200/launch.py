"""Config-driven training entry point: one process per rank.

    python -m rumus_b200.launch --config tiny-decoder-cpu --steps 50
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \\
        -m rumus_b200.launch --config gpt-1.3b-fsdp --steps 100 --ckpt-dir ckpt --ckpt-every 50

``--config`` is a preset name (``utils/config.PRESETS``) or a YAML file with the same fields.
The run builds the model family of the config (GPT with the sharded-data-parallel engine, ResNet-50
with data parallelism and dynamic loss scaling, Llama with tensor x pipeline parallelism), feeds it
synthetic data of the configured shape or a ``.rrec`` file (``--data``, read by the native batch loader), writes JSONL metrics per rank
(``--metrics-dir``), saves checkpoints (``--ckpt-dir`` / ``--ckpt-every``) and, with ``--resume``,
continues from the newest checkpoint whose digests verify — also when it was written by a different
number of ranks.  Under an ``ElasticSupervisor`` this is the worker a restart re-enters.

The reference has no launcher: jobs are Rust programs that wire modules by hand
(rumus/tests/*.rs); its trainer is rumus/src/train.rs:56-96.
"""
from __future__ import annotations

import argparse
import contextlib
import json
import os
import sys
import time

import torch
import torch.distributed as dist

from .utils.config import TrainConfig, load_config

_DTYPES = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


def _setup():
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dev = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl" if cuda else "gloo")
    return rank, world, dev


def _token_batches(cfg: TrainConfig, rank: int, dev, data_path):
    """Yields ``(inputs [B, S], targets [B, S])`` forever."""
    kw = cfg.model.kwargs
    B, S, V = cfg.seqs_per_gpu, kw["seq_len"], kw["vocab_size"]
    if data_path:
        from .data import NativeBatchLoader
        loader = NativeBatchLoader(data_path, B, shuffle=True, drop_last=True)
        while True:
            for item in loader:
                yield (item.input.to(dev, non_blocking=True).long(),
                       item.target.to(dev, non_blocking=True).long())
    g = torch.Generator().manual_seed(cfg.seed * 1000 + rank)
    pin = dev.type == "cuda"
    while True:
        # a learnable synthetic stream: arithmetic progressions with a random start and stride
        start = torch.randint(0, V, (B, 1), generator=g)
        stride = torch.randint(1, 4, (B, 1), generator=g)
        tok = (start + stride * torch.arange(S + 1)[None]) % V
        if pin:
            tok = tok.pin_memory()
        tok = tok.to(dev, non_blocking=True)
        yield tok[:, :-1], tok[:, 1:]


def _run_gpt(cfg: TrainConfig, a, rank, world, dev) -> dict:
    from .io.checkpoint import load_checkpoint, save_checkpoint
    from .models import GPT, GPTConfig
    from .parallel import FSDP
    from .utils import DeviceTimer, MetricsLogger
    from .utils.elastic import latest_checkpoint
    dtype = _DTYPES[cfg.precision.compute] if dev.type == "cuda" else torch.float32
    model = GPT(GPTConfig(**cfg.model.kwargs), device=dev, dtype=dtype)
    model.init_weights(0.02, seed=cfg.seed)
    mode = None if cfg.parallel.backend == "fused" else cfg.parallel.backend
    engine = FSDP(model, lr=cfg.lr, adamw=cfg.optimizer == "adamw", mode=mode,
                  reshard_after_forward=cfg.parallel.reshard_after_forward)
    resumed = None
    if a.resume and a.ckpt_dir:
        resumed = latest_checkpoint(a.ckpt_dir, verify=True)
        if resumed:
            load_checkpoint(resumed, model, engine)
    log = MetricsLogger(a.metrics_dir, rank=rank) if a.metrics_dir else None
    batches = _token_batches(cfg, rank, dev, a.data)
    steps = a.steps if a.steps is not None else cfg.steps
    tokens_per_step = world * cfg.seqs_per_gpu * cfg.model.kwargs["seq_len"]
    first = last = None
    t0, step0 = time.time(), engine.step_count
    while engine.step_count < steps:
        x, y = next(batches)
        will_log = (engine.step_count + 1) % a.log_every == 0 or engine.step_count + 1 == steps
        timer = DeviceTimer() if will_log else contextlib.nullcontext()
        with timer:      # device-timed (CUDA events) on the steps that are logged; no sync otherwise
            engine.zero_grad()
            loss = model(x, y)
            loss.backward()
            engine.step()
        if will_log:
            last = float(loss.item())
            first = last if first is None else first
            if log:
                rec = dict(step=engine.step_count, loss=last, lr=engine.lr, step_ms=timer.ms,
                           tokens_per_s_device=tokens_per_step / max(1e-9, timer.ms / 1e3),
                           tokens_per_s=tokens_per_step * (engine.step_count - step0) / max(1e-9, time.time() - t0))
                if dev.type == "cuda":
                    rec["hbm_peak_gb"] = torch.cuda.max_memory_allocated(dev) / 2 ** 30
                log.log(**rec)
        if a.ckpt_dir and a.ckpt_every and engine.step_count % a.ckpt_every == 0:
            save_checkpoint(os.path.join(a.ckpt_dir, f"step-{engine.step_count}"), model, engine,
                            extra={"config": cfg.name})
    return {"family": "gpt", "steps": engine.step_count, "first_logged_loss": first, "last_loss": last,
            "mode": engine.mode, "world": world, "resumed_from": resumed}


def _run_resnet(cfg: TrainConfig, a, rank, world, dev) -> dict:
    from .models import ResNet50
    from .ops import functional as F
    from .optim import SGD, GradScaler
    from .parallel.dp import DataParallel
    from .utils import MetricsLogger
    dtype = _DTYPES[cfg.precision.compute] if dev.type == "cuda" else torch.float32
    model = ResNet50(device=dev, dtype=dtype, **cfg.model.kwargs)
    mode = None if cfg.parallel.backend == "fused" else cfg.parallel.backend
    dp = DataParallel(model, mode=mode)
    opt = SGD(model.parameters(), lr=cfg.lr, momentum=cfg.momentum)
    scaler = GradScaler(init_scale=cfg.precision.init_scale) if cfg.precision.loss_scaling else None
    log = MetricsLogger(a.metrics_dir, rank=rank) if a.metrics_dir else None
    B = a.batch or cfg.seqs_per_gpu
    res = a.image_size
    g = torch.Generator().manual_seed(cfg.seed * 1000 + rank)
    steps = a.steps if a.steps is not None else cfg.steps
    last = None
    for step in range(1, steps + 1):
        x = torch.randn(B, 3, res, res, generator=g).to(dev).to(dtype)
        if dev.type == "cuda":
            x = x.contiguous(memory_format=torch.channels_last)
        y = torch.randint(0, cfg.model.kwargs.get("num_classes", 1000), (B,), generator=g).to(dev)
        dp.zero_grad()
        loss = F.cross_entropy_loss(model(x), y)
        if scaler is not None:
            scaler._ensure(dev)
            dp.begin_backward(scaler.inv_scale)
            scaler.scale(loss).backward()
            found = dp.all_reduce_grads()
            opt.grad_scale, opt.skip_flag = None, found
            scaler.found_inf = found
            opt.step()
            scaler.update()
        else:
            dp.begin_backward(None)
            loss.backward()
            dp.all_reduce_grads()
            opt.step()
        if step % a.log_every == 0 or step == steps:
            last = float(loss.item())
            if log:
                log.log(step=step, loss=last, loss_scale=scaler.scale_value if scaler else 1.0)
    return {"family": "resnet50", "steps": steps, "last_loss": last, "mode": dp.mode, "world": world}


def _run_llama(cfg: TrainConfig, a, rank, world, dev) -> dict:
    """Tensor x pipeline parallel Llama: 1F1B over ``parallel.pp`` stages, sequence-parallel
    tensor-parallel blocks, per-stage fused Adam; ``--export-dense`` writes the reference-layout
    ``model.safetensors`` assembled from all shards at the end."""
    from .io.safetensors import save_safetensors
    from .models.llama import LlamaConfig
    from .models.llama_parallel import ParallelLlamaStage
    from .parallel import FSDP
    from .parallel.pp import PipelineStage, bubble_fraction
    from .parallel.topology import build_topology
    from .parallel.tp import TPContext
    from .utils import MetricsLogger
    par = cfg.parallel
    if par.pp < 2:
        raise SystemExit("the Llama launcher path needs pp >= 2 (use FSDP / DP presets otherwise)")
    topo = build_topology(tp=par.tp, pp=par.pp)
    mc = LlamaConfig(**cfg.model.kwargs)
    dtype = _DTYPES[cfg.precision.compute] if dev.type == "cuda" else torch.float32
    global_batch = cfg.global_batch or cfg.seqs_per_gpu * topo.dp * par.micro_batches
    mb_seqs = global_batch // (topo.dp * par.micro_batches)
    mb_tokens = mb_seqs * mc.seq_len
    mode = "nccl" if dev.type != "cuda" else (None if par.backend == "fused" else par.backend)
    tp = TPContext(group=topo.tp_group, mode=mode, max_tokens=mb_tokens, max_features=mc.d_model)
    stage = ParallelLlamaStage(mc, tp, topo.pp_idx, par.pp, device=dev, dtype=dtype)
    stage.init_weights(0.02, seed=cfg.seed)
    stage.set_microbatch_shape(mb_seqs, mc.seq_len)
    units = [(f"blocks.{i}", [b]) for i, b in enumerate(stage.blocks)]
    rest = [p for n, p in stage.named_parameters() if not n.startswith("blocks.")]
    if rest:
        units.append(("edge", rest))
    opt = FSDP(stage, lr=cfg.lr, unit_roots=units, local_only=True, defer_update=True)
    ps = PipelineStage(stage, topo.pp_idx, par.pp, topo.prev_stage_rank, topo.next_stage_rank,
                       (mb_tokens // par.tp, mc.d_model), dtype, dev)
    first, last = topo.pp_idx == 0, topo.pp_idx == par.pp - 1
    g = torch.Generator().manual_seed(cfg.seed * 1000 + topo.dp_idx)
    log = MetricsLogger(a.metrics_dir, rank=rank) if a.metrics_dir else None
    steps = a.steps if a.steps is not None else cfg.steps
    first_loss = last_loss = None
    for step in range(1, steps + 1):
        toks = []
        for _ in range(par.micro_batches):
            start = torch.randint(0, mc.vocab_size, (mb_seqs, 1), generator=g)
            toks.append((start + torch.arange(mc.seq_len + 1)[None]) % mc.vocab_size)
        if first:
            mbs = [t[:, :-1].to(dev) for t in toks]
        elif last:
            mbs = [t[:, 1:].to(dev) for t in toks]
        else:
            mbs = [None] * par.micro_batches
        opt.zero_grad()
        loss = ps.run(mbs)
        # norm weights are replicated over the tensor-parallel group, the whole stage over the
        # data-parallel replicas: sum resp. average those gradients before the update
        opt.reduce_grads(replicated_group=topo.tp_group, dp_group=topo.dp_group)
        opt.step()
        if last and (step % a.log_every == 0 or step == steps):
            last_loss = float(loss)
            first_loss = last_loss if first_loss is None else first_loss
            if log and tp.rank == 0:
                log.log(step=step, loss=last_loss)
    if a.export_dense:
        full = stage.export_dense()
        if rank == 0:
            os.makedirs(os.path.dirname(os.path.abspath(a.export_dense)), exist_ok=True)
            save_safetensors(full, a.export_dense)
    # the loss lives on the last stage: hand it to rank 0 for the summary line
    summary = [None] * world
    dist.all_gather_object(summary, (first_loss, last_loss) if last and tp.rank == 0 else None)
    got = [s for s in summary if s is not None][0]
    return {"family": "llama", "steps": steps, "first_logged_loss": got[0], "last_loss": got[1],
            "parallelism": f"tp{par.tp}xpp{par.pp}xdp{topo.dp}", "mode": tp.mode, "world": world,
            "bubble_fraction_ideal": bubble_fraction(par.pp, par.micro_batches)}


def main(argv=None) -> dict:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True, help="preset name or YAML path")
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--data", default=None, help=".rrec file of (input tokens, target tokens) records")
    ap.add_argument("--metrics-dir", default=None)
    ap.add_argument("--ckpt-dir", default=None)
    ap.add_argument("--ckpt-every", type=int, default=0)
    ap.add_argument("--resume", action="store_true")
    ap.add_argument("--log-every", type=int, default=10)
    ap.add_argument("--batch", type=int, default=None, help="per-rank batch override (vision)")
    ap.add_argument("--image-size", type=int, default=224)
    ap.add_argument("--export-dense", default=None,
                    help="(Llama) write the dense reference-layout model.safetensors here at the end")
    a = ap.parse_args(argv)
    cfg = load_config(a.config)
    rank, world, dev = _setup()
    if cfg.model.family == "gpt":
        out = _run_gpt(cfg, a, rank, world, dev)
    elif cfg.model.family == "resnet50":
        out = _run_resnet(cfg, a, rank, world, dev)
    elif cfg.model.family == "llama":
        out = _run_llama(cfg, a, rank, world, dev)
    else:
        raise SystemExit(f"unknown model family {cfg.model.family!r}")
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
    sys.exit(0)
