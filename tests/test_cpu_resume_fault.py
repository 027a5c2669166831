"""Checkpoint resume identity / re-sharding, config presets, heartbeat-based failure detection
with host-side fault injection (CPU ranks; no GPU involved)."""
import json
import os
import time

import pytest
import torch
import torch.distributed as dist

from dist_utils import run_ranks


def _make():
    from rumus_b200.models import GPT, GPTConfig
    cfg = GPTConfig(vocab_size=64, seq_len=16, d_model=32, num_heads=2, num_layers=2, ffn_dim=64)
    torch.manual_seed(0)
    return GPT(cfg)


def _data():
    g = torch.Generator().manual_seed(9)
    return torch.randint(0, 64, (6, 4, 17), generator=g)


def _step(model, eng, tok):
    eng.zero_grad()
    loss = model(tok[:, :-1], tok[:, 1:])
    loss.backward()
    eng.step()
    return loss.item()


def test_resume_continues_bit_identically(tmp_path):
    from rumus_b200.io.checkpoint import load_checkpoint, save_checkpoint
    from rumus_b200.parallel import FSDP
    data = _data()
    m = _make(); e = FSDP(m, lr=1e-2)
    for s in range(3):
        _step(m, e, data[s])
    save_checkpoint(str(tmp_path), m, e, extra={"seed": 9})
    cont = [_step(m, e, data[s]) for s in range(3, 6)]
    m2 = _make()
    with torch.no_grad():
        for p in m2.parameters():
            p.add_(1.0)       # make sure everything really comes from the checkpoint
    e2 = FSDP(m2, lr=123.0)
    extra = load_checkpoint(str(tmp_path), m2, e2)
    assert extra == {"seed": 9} and e2.step_count == 3 and e2.lr == 1e-2
    again = [_step(m2, e2, data[s]) for s in range(3, 6)]
    assert again == cont                     # bit-identical loss curve
    st = json.load(open(tmp_path / "trainer_state.json"))
    assert st["world"] == 1 and st["units"][0]["name"] == "embeddings"
    assert sorted(os.listdir(tmp_path)) == ["model.safetensors", "optim-rank0.safetensors", "trainer_state.json"]


def _save_worker(rank, world, d):
    from rumus_b200.io.checkpoint import save_checkpoint
    from rumus_b200.parallel import FSDP
    m = _make(); e = FSDP(m, lr=1e-2)
    data = _data()
    for s in range(3):
        _step(m, e, data[s][rank * 2:(rank + 1) * 2])
    save_checkpoint(d, m, e)
    return [_step(m, e, data[s][rank * 2:(rank + 1) * 2]) for s in range(3, 5)]


def test_reshard_world2_checkpoint_into_world1(tmp_path):
    from rumus_b200.io.checkpoint import load_checkpoint
    from rumus_b200.parallel import FSDP
    d = str(tmp_path)
    run_ranks(_save_worker, 2, d)
    assert os.path.exists(os.path.join(d, "optim-rank1.safetensors"))
    m = _make(); e = FSDP(m, lr=1.0)
    load_checkpoint(d, m, e)
    assert e.world == 1 and e.step_count == 3
    # the re-assembled optimizer state equals a single-process run on the same global batches
    ref = _make(); er = FSDP(ref, lr=1e-2)
    data = _data()
    for s in range(3):
        _step(ref, er, data[s])
    for u, ur in zip(e.units, er.units):
        # parameters whose exact gradient is zero (attention key biases) only carry rounding noise,
        # which Adam normalises to +-lr: allow that handful of outliers
        bad = (u.master[: u.numel] - ur.master[: ur.numel]).abs() > 3e-5
        assert bad.float().mean().item() < 0.01
        assert torch.allclose(u.exp_avg[: u.numel], ur.exp_avg[: ur.numel], atol=3e-6)


def test_config_presets_and_yaml(tmp_path):
    from rumus_b200.utils import PRESETS, load_config
    assert set(PRESETS) == {"tiny-decoder-cpu", "gpt-1.3b-fsdp", "llama-7b-tp4-pp2", "resnet50-dp-fp16",
                            "llama-7b-int4-serve-tp8"}
    c = load_config("llama-7b-tp4-pp2")
    assert (c.parallel.tp, c.parallel.pp, c.parallel.micro_batches, c.global_batch) == (4, 2, 8, 64)
    p = tmp_path / "c.yaml"
    p.write_text("name: x\nmodel: {family: gpt, kwargs: {d_model: 64}}\nparallel: {tp: 2}\nlr: 0.5\n")
    c = load_config(str(p))
    assert c.model.kwargs["d_model"] == 64 and c.parallel.tp == 2 and c.lr == 0.5


def test_metrics_logger(tmp_path):
    from rumus_b200.utils import DeviceTimer, MetricsLogger, trace_range
    log = MetricsLogger(str(tmp_path), rank=3)
    with trace_range("step"), DeviceTimer() as t:
        time.sleep(0.01)
    log.log(step=1, loss=torch.tensor(2.5), ms=t.ms)
    rec = json.loads(open(tmp_path / "metrics-rank3.jsonl").read().strip())
    assert rec["step"] == 1 and rec["loss"] == 2.5 and rec["rank"] == 3 and rec["ms"] >= 9


def _fault_worker(rank, world):
    """Rank 1 leaves between steps (host-side injection).  Rank 0 learns of it from the heartbeat
    before its next collective and stops cleanly instead of blocking."""
    from rumus_b200.utils import FaultInjector, Heartbeat, PeerLost
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.5).start()
    inj = FaultInjector(rank, "exit:1:2")
    done, detected = 0, False
    for step in range(6):
        if not inj.before_step(step, hb):
            break                               # leaves with nothing in flight
        try:
            if step >= 2:
                time.sleep(0.8)                 # give the heartbeat time to go stale
            hb.check_peers()
        except PeerLost as e:
            detected = e.ranks == [1]
            break
        t = torch.ones(1)
        dist.all_reduce(t)
        done += 1
    hb.stop()
    return done, detected


def test_peer_loss_is_detected_before_the_next_collective():
    out = run_ranks(_fault_worker, 2, timeout=120)
    assert out[1] == (2, False)          # the leaving rank completed steps 0 and 1
    assert out[0] == (2, True)           # the survivor noticed and launched nothing further


def test_flag_protocols_hold_on_every_interleaving():
    """Model check of the fused kernels' epoch-flag protocols (every interleaving of 2 and 3 ranks
    over two steps), and proof that the checker sees the hazard once a wait is taken out."""
    import pytest
    from rumus_b200.utils.protocol_check import (ProtocolViolation, allreduce_programs, explore,
                                                 fsdp_reshard_programs, fsdp_unit_programs,
                                                 tp_sequence_programs)
    assert explore(fsdp_unit_programs(2, 2)) > 100
    assert explore(fsdp_unit_programs(3, 2)) > 1000
    assert explore(allreduce_programs(2, 2)) > 100
    with pytest.raises(ProtocolViolation):
        explore(fsdp_unit_programs(2, 2, wait_param_flags=False))   # shard read before it is written
    with pytest.raises(ProtocolViolation):
        explore(fsdp_unit_programs(2, 2, wait_grad_flags=False))    # gradient read before the write
    with pytest.raises(ProtocolViolation):
        explore(allreduce_programs(2, 2, exit_barrier=False))       # reads a half-reduced bucket
    # parameters resharded between uses: shards are gathered twice per step and overwritten after
    # the gradient exchange; no extra barrier is needed, and each wait is necessary
    assert explore(fsdp_reshard_programs(2, 3)) > 500
    assert explore(fsdp_reshard_programs(3, 2)) > 10000
    with pytest.raises(ProtocolViolation):
        explore(fsdp_reshard_programs(2, 2, wait_param_flags=False))  # gathers a shard before its update
    with pytest.raises(ProtocolViolation):
        explore(fsdp_reshard_programs(2, 2, wait_grad_flags=False))
    # fused tensor-parallel operations on one context: gather (A) and reduce (R) operations may follow
    # each other without a barrier only when they alternate; the context inserts one (b) otherwise
    # push-form reduce-scatter: two sum buffers in turn are enough, one is not
    from rumus_b200.utils.protocol_check import rs_push_programs
    assert explore(rs_push_programs(2, 4)) > 100
    assert explore(rs_push_programs(3, 3)) > 1000
    with pytest.raises(ProtocolViolation):
        explore(rs_push_programs(2, 3, alternate=False))
    assert explore(tp_sequence_programs(2, "ARARAR")) > 100
    assert explore(tp_sequence_programs(3, "RARA")) > 1000
    assert explore(tp_sequence_programs(3, "AbARbR")) > 1000
    for bad in ("AA", "RR", "ARRA"):
        with pytest.raises(ProtocolViolation):
            explore(tp_sequence_programs(2, bad))
    # a rank that never publishes one of its flags: the model deadlocks (on the device the bounded
    # wait turns that into a status code instead)
    progs = fsdp_unit_programs(2, 1)
    progs[1] = [a for a in progs[1] if not (a[0] == "set" and a[1] == "grad_ready[0][1]")]
    with pytest.raises(ProtocolViolation, match="deadlock"):
        explore(progs)


def _elastic_worker(rank, world, generation, root, total_steps):
    """FSDP training on CPU ranks with a checkpoint every 2 steps.  In generation 0 rank 1 leaves
    after step 3 (host-side injection) and the survivors stop on ``PeerLost``; every later
    generation resumes from the newest checkpoint, whatever its world size was."""
    import sys
    from rumus_b200.io.checkpoint import load_checkpoint, save_checkpoint
    from rumus_b200.parallel import FSDP
    from rumus_b200.utils import FaultInjector, Heartbeat, PeerLost
    from rumus_b200.utils.elastic import latest_checkpoint
    os.environ["RB_BACKEND"] = "cpu"
    torch.set_num_threads(1)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval_s=0.05, timeout_s=0.6).start()
    inj = FaultInjector(rank, "exit:1:3" if generation == 0 else "")
    m = _make(); e = FSDP(m, lr=1e-2)
    ck = latest_checkpoint(root)
    if ck is not None:
        load_checkpoint(ck, m, e)
    data = _data()
    rc = 0
    try:
        while e.step_count < total_steps:
            step = e.step_count
            if not inj.before_step(step, hb):
                rc = 17                                   # leaves between steps, nothing in flight
                break
            if generation == 0 and step >= 3:
                time.sleep(0.9)                           # let the lost peer's heartbeat go stale
            hb.check_peers()
            per = 4 // world if 4 % world == 0 else 1
            _step(m, e, data[step % 6][rank * per:(rank + 1) * per])
            if e.step_count % 2 == 0:
                save_checkpoint(os.path.join(root, f"step-{e.step_count}"), m, e)
    except PeerLost:
        rc = 18
    hb.stop()
    if rc == 0:
        dist.barrier()
        if rank == 0:
            with open(os.path.join(root, f"done-gen{generation}.json"), "w") as f:
                json.dump({"steps": e.step_count, "world": world, "resumed_from": ck}, f)
        dist.destroy_process_group()
    # a rank that lost a peer must not run the process-group destructor's collectives
    os._exit(rc)


def test_elastic_supervisor_restarts_smaller_from_last_checkpoint(tmp_path):
    from rumus_b200.utils.elastic import ElasticSupervisor, latest_checkpoint
    root = str(tmp_path)
    sup = ElasticSupervisor(_elastic_worker, world=2, args=(root, 8), max_restarts=2,
                            shrink_on_failure=True)
    hist = sup.run()
    assert len(hist) == 2
    assert hist[0].world == 2 and 1 in hist[0].failed_ranks and hist[0].exit_codes[1] == 17
    assert hist[1].world == 1 and hist[1].exit_codes == [0]
    done = json.load(open(os.path.join(root, "done-gen1.json")))
    # generation 0 saved step-2 (step 4 was never reached: rank 1 left after step 3)
    assert done["steps"] == 8 and done["world"] == 1 and done["resumed_from"].endswith("step-2")
    assert latest_checkpoint(root).endswith("step-8")


def test_corrupted_checkpoint_is_rejected_and_skipped(tmp_path):
    """Host-side fault injection on storage: a flipped byte in an optimizer shard."""
    from rumus_b200.io.checkpoint import CheckpointCorrupt, load_checkpoint, save_checkpoint, verify_checkpoint
    from rumus_b200.parallel import FSDP
    from rumus_b200.utils.elastic import latest_checkpoint
    m = _make(); e = FSDP(m, lr=1e-2)
    data = _data()
    for s in range(4):
        _step(m, e, data[s])
        if e.step_count % 2 == 0:
            save_checkpoint(str(tmp_path / f"step-{e.step_count}"), m, e)
    newest = tmp_path / "step-4"
    assert verify_checkpoint(str(newest)) and latest_checkpoint(str(tmp_path), verify=True).endswith("step-4")
    shard = newest / "optim-rank0.safetensors"
    raw = bytearray(shard.read_bytes())
    raw[len(raw) // 2] ^= 0x40
    shard.write_bytes(bytes(raw))
    assert not verify_checkpoint(str(newest))
    with pytest.raises(CheckpointCorrupt):
        load_checkpoint(str(newest), _make(), FSDP(_make(), lr=1.0))
    assert latest_checkpoint(str(tmp_path), verify=True).endswith("step-2")
    assert latest_checkpoint(str(tmp_path)).endswith("step-4")      # unverified: newest by name


def test_llama_stage_never_issues_two_same_kind_fused_ops_in_a_row():
    """The staging buffers of the fused tensor-parallel kernels are reused without a barrier as long as
    gather (A) and reduce (R) operations alternate.  Under every 1F1B schedule the parallel Llama
    stage issues: forward = ARAR per block (+ A for the head on the last stage), backward = (R for the
    head) + ARAR per block — so the sequence alternates and ``TPContext.order_fused`` never has to
    insert its barrier there."""
    from rumus_b200.parallel.pp import one_f_one_b_order
    for stages in (1, 2, 4):
        for micro in (1, 2, 4, 8):
            for st in range(stages):
                last = st == stages - 1
                seq = ""
                for kind, _mb in one_f_one_b_order(st, stages, micro):
                    seq += ("ARAR" * 2 + ("A" if last else "")) if kind == "F" else (("R" if last else "") + "ARAR" * 2)
                assert all(seq[i] != seq[i - 1] for i in range(1, len(seq))), (stages, micro, st)
