"""Training checkpoints: model weights in the reference's safetensors layout plus what a resume
needs and the reference never saves (rumus/src/nn/io.rs stores weights only): sharded optimizer
state, step counter, LR, loss scale, RNG seed, and the world layout — with a loader that
re-shards the optimizer state for a different world size.

Layout of a checkpoint directory:
  model.safetensors            fp32, reference tensor names, [in, out] Linear weights (rank 0)
  optim-rank{r}.safetensors    fp32 master / exp_avg / exp_avg_sq shards of every flat unit
  trainer_state.json           step, lr, betas, world size, per-unit (numel, padded, shard) sizes,
                               SHA-256 of every other file
All files are written to a temporary name and renamed (atomic on POSIX); ``trainer_state.json`` is
written last, after every rank's shard is on disk, so its presence marks a complete checkpoint and
its digests let a loader reject a damaged one.
"""
from __future__ import annotations

import contextlib
import hashlib
import json
import os
from typing import Optional

import torch
import torch.distributed as dist

from .safetensors import load_safetensors, load_into, save_safetensors


def _atomic_json(obj, path):
    tmp = f"{path}.tmp.{os.getpid()}"
    with open(tmp, "w") as f:
        json.dump(obj, f, indent=1)
        f.flush()
        os.fsync(f.fileno())
    os.replace(tmp, path)


class CheckpointCorrupt(IOError):
    pass


def _sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        for chunk in iter(lambda: f.read(1 << 22), b""):
            h.update(chunk)
    return h.hexdigest()


def verify_checkpoint(directory: str) -> bool:
    """True when ``trainer_state.json`` exists and every file it lists has the recorded digest."""
    try:
        with open(os.path.join(directory, "trainer_state.json")) as f:
            st = json.load(f)
        for name, digest in st.get("files", {}).items():
            if _sha256(os.path.join(directory, name)) != digest:
                return False
        return True
    except (OSError, ValueError):
        return False


def save_checkpoint(directory: str, model: torch.nn.Module, engine, extra: Optional[dict] = None) -> None:
    """``engine`` is a ``parallel.FSDP`` (any world size, including 1)."""
    os.makedirs(directory, exist_ok=True)
    rank, world = engine.rank, engine.world
    mine = {}
    # with resharded parameters every rank takes part in gathering them for the writer
    with getattr(engine, "summon_full_params", contextlib.nullcontext)():
        if rank == 0:
            save_safetensors(model.state_dict(), os.path.join(directory, "model.safetensors"))
            mine["model.safetensors"] = _sha256(os.path.join(directory, "model.safetensors"))
    shard_name = f"optim-rank{rank}.safetensors"
    save_safetensors(engine.optimizer_state(), os.path.join(directory, shard_name))
    mine[shard_name] = _sha256(os.path.join(directory, shard_name))
    files = dict(mine)
    if world > 1 and dist.is_initialized():
        # every shard is on disk (and its digest known to rank 0) before the state file appears
        gathered = [None] * world
        dist.all_gather_object(gathered, mine, group=engine.group)
        files = {k: v for d in gathered for k, v in d.items()}
    if rank == 0:
        state = {"step": engine.step_count, "lr": engine.lr, "beta1": engine.beta1, "beta2": engine.beta2,
                 "eps": engine.eps, "weight_decay": engine.weight_decay, "adamw": engine.adamw,
                 "world": world,
                 "units": [{"name": u.name, "numel": u.numel, "padded": u.padded, "shard": u.shard_numel}
                           for u in engine.units],
                 "files": files,
                 "extra": extra or {}}
        _atomic_json(state, os.path.join(directory, "trainer_state.json"))
    if world > 1 and dist.is_initialized():
        dist.barrier(engine.group)


def load_checkpoint(directory: str, model: torch.nn.Module, engine, verify: bool = True) -> dict:
    """Restores weights, optimizer shards (re-sharded if the saved world size differs), step and
    hyper-parameters.  Returns the ``extra`` dict that was saved.  With ``verify`` the files are
    checked against the digests in ``trainer_state.json`` first (``CheckpointCorrupt``)."""
    with open(os.path.join(directory, "trainer_state.json")) as f:
        st = json.load(f)
    if verify and not verify_checkpoint(directory):
        raise CheckpointCorrupt(f"{directory}: a file does not match its recorded SHA-256")
    summon = getattr(engine, "summon_full_params", None)
    with (summon(writeback=True) if summon is not None else contextlib.nullcontext()):
        load_into(model, os.path.join(directory, "model.safetensors"))
    old_world = st["world"]
    if old_world == engine.world:
        sd = load_safetensors(os.path.join(directory, f"optim-rank{engine.rank}.safetensors"))
        sd = {k: v.to(engine.units[0].master.device) for k, v in sd.items()}
    else:
        shards = [load_safetensors(os.path.join(directory, f"optim-rank{r}.safetensors"))
                  for r in range(old_world)]
        sd = {}
        saved_units = {u["name"]: u for u in st["units"]}
        for u in engine.units:
            su = saved_units[u.name]
            assert su["numel"] == u.numel, f"unit {u.name} changed size"
            for part in ("master", "exp_avg", "exp_avg_sq"):
                full = torch.cat([s[f"{u.name}.{part}"] for s in shards])[: u.numel]
                padded = torch.zeros(u.padded)
                padded[: u.numel] = full
                lo, hi = u.shard_range
                sd[f"{u.name}.{part}"] = padded[lo:hi].to(u.master.device)
    for u in engine.units:
        u.master.copy_(sd[f"{u.name}.master"])
        u.exp_avg.copy_(sd[f"{u.name}.exp_avg"])
        u.exp_avg_sq.copy_(sd[f"{u.name}.exp_avg_sq"])
    # the low-precision parameters were restored from model.safetensors (identical on all ranks);
    # for fp32 models make the flat parameters bit-identical to the master shards
    for u in engine.units:
        if u.dtype == torch.float32:
            u.param_shard().copy_(u.master)
    engine.step_count = st["step"]
    engine.lr, engine.beta1, engine.beta2 = st["lr"], st["beta1"], st["beta2"]
    engine.eps, engine.weight_decay, engine.adamw = st["eps"], st["weight_decay"], st["adamw"]
    return st.get("extra", {})
