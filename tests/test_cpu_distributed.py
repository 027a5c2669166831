"""Distributed logic on CPU ranks (gloo): FSDP sharding/step, tensor parallel layers, 1F1B pipeline,
TP x PP Llama, data parallel — each compared with the single-process computation."""
import torch
import torch.distributed as dist

from dist_utils import run_ranks


# ------------------------------------------------------------------ FSDP
def _fsdp_worker(rank, world):
    from rumus_b200.models import GPT, GPTConfig
    from rumus_b200.parallel import FSDP
    cfg = GPTConfig(vocab_size=64, seq_len=16, d_model=32, num_heads=2, num_layers=2, ffn_dim=64)
    torch.manual_seed(0)
    model = GPT(cfg)
    eng = FSDP(model, lr=1e-2)
    assert eng.mode == "cpu" and eng.world == world
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, 64, (3, world * 2, 17), generator=g)
    for step in range(3):
        tok = data[step, rank * 2:(rank + 1) * 2]
        eng.zero_grad()
        loss = model(tok[:, :-1], tok[:, 1:])
        loss.backward()
        eng.step()
    return {k: v.clone() for k, v in model.state_dict().items()}


def test_fsdp_matches_single_process():
    from rumus_b200.models import GPT, GPTConfig
    from rumus_b200.optim import Adam
    world = 2
    states = run_ranks(_fsdp_worker, world)
    for k in states[0]:
        assert torch.equal(states[0][k], states[1][k]), k       # replicas agree after all-gather
    cfg = GPTConfig(vocab_size=64, seq_len=16, d_model=32, num_heads=2, num_layers=2, ffn_dim=64)
    torch.manual_seed(0)
    ref = GPT(cfg)
    opt = Adam(ref.parameters(), lr=1e-2)
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, 64, (3, world * 2, 17), generator=g)
    for step in range(3):
        opt.zero_grad()
        ref(data[step][:, :-1], data[step][:, 1:]).backward()
        opt.step()
    rs = ref.state_dict()
    for k in rs:
        if k.endswith("k_proj.bias"):
            continue   # exact gradient is zero (softmax ignores a key bias): Adam amplifies rounding noise
        assert torch.allclose(states[0][k], rs[k], atol=2e-5), k


def _fsdp_reshard_worker(rank, world, ckpt_dir):
    """Same job twice: parameters resident (gathered after each update) and resharded (gathered
    around each block's forward and backward).  Both must produce identical losses and weights."""
    from rumus_b200.io.checkpoint import load_checkpoint, save_checkpoint
    from rumus_b200.models import GPT, GPTConfig
    from rumus_b200.parallel import FSDP
    cfg = GPTConfig(vocab_size=64, seq_len=16, d_model=32, num_heads=2, num_layers=5, ffn_dim=64)
    g = torch.Generator().manual_seed(5)
    data = torch.randint(0, 64, (5, world * 2, 17), generator=g)

    def run(reshard, steps, eng=None, model=None, start=0):
        if eng is None:
            torch.manual_seed(0)
            model = GPT(cfg)
            eng = FSDP(model, lr=1e-2, reshard_after_forward=reshard)
        losses = []
        for step in range(start, start + steps):
            tok = data[step, rank * 2:(rank + 1) * 2]
            eng.zero_grad()
            loss = model(tok[:, :-1], tok[:, 1:])
            loss.backward()
            eng.step()
            losses.append(loss.item())
        return model, eng, losses

    m0, e0, l0 = run(False, 5)
    m1, e1, l1 = run(True, 3)
    assert e1._resharded == [1, 2, 3, 4, 5] and e1.param_bytes() < e0.param_bytes()
    # per step: 5 gathers forward; backward reuses what the two slots still hold (blocks 5 and 4)
    assert e1.gathers_issued == 3 * (2 * 5 - 2)
    save_checkpoint(ckpt_dir, m1, e1)
    # resume into a fresh resharded engine and finish the run
    torch.manual_seed(123)
    m2 = GPT(cfg)
    e2 = FSDP(m2, lr=1.0, reshard_after_forward=True)
    load_checkpoint(ckpt_dir, m2, e2)
    _, _, l2 = run(True, 2, eng=e2, model=m2, start=3)
    with e2.summon_full_params():
        sd2 = {k: v.clone() for k, v in m2.state_dict().items()}
    with torch.no_grad():   # evaluation forward also gathers
        tok = data[0, :2]
        ev = (m0(tok[:, :-1], tok[:, 1:]).item(), m2(tok[:, :-1], tok[:, 1:]).item())
    return l0, l1 + l2, {k: v.clone() for k, v in m0.state_dict().items()}, sd2, ev


def test_fsdp_reshard_after_forward_is_identical_and_resumes(tmp_path):
    out = run_ranks(_fsdp_reshard_worker, 2, str(tmp_path), timeout=240)
    for l_res, l_shard, sd_res, sd_shard, ev in out:
        assert l_res == l_shard
        assert ev[0] == ev[1]
        for k in sd_res:
            assert torch.equal(sd_res[k], sd_shard[k]), k


def _vocab_parallel_worker(rank, world):
    """Vocabulary-parallel embedding (replicated and sequence-parallel output) and cross entropy
    against the dense computation, values and gradients."""
    from rumus_b200.nn import Embedding
    from rumus_b200.parallel.tp import (TPContext, VocabParallelEmbedding, copy_to_region, gather_rows,
                                        vocab_parallel_cross_entropy)
    tp = TPContext(mode="nccl")
    V, d, M = 24, 8, 12
    torch.manual_seed(7)
    dense = Embedding(V, d)
    torch.manual_seed(7)
    emb = VocabParallelEmbedding(V, d, tp)
    torch.manual_seed(7)
    emb_sp = VocabParallelEmbedding(V, d, tp, sequence_parallel=True)
    vloc = V // world
    assert torch.equal(emb.weight, dense.weight[rank * vloc:(rank + 1) * vloc])
    g = torch.Generator().manual_seed(3)
    tok = torch.randint(0, V, (M,), generator=g)
    tgt = torch.randint(0, V, (M,), generator=g)
    head = torch.randn(d, V, generator=g) * 0.3
    # dense reference
    h = dense(tok)
    loss_ref = torch.nn.functional.cross_entropy(h @ head, tgt)
    loss_ref.backward()
    out = {}
    for name, e in (("ar", emb), ("sp", emb_sp)):
        x = e(tok)
        if name == "sp":
            assert x.shape == (M // world, d)
            x = gather_rows(x, tp)
        else:
            x = copy_to_region(x, tp)     # replicated input of a column-parallel product
        assert torch.allclose(x, h.detach(), atol=1e-6)
        hl = head[:, rank * vloc:(rank + 1) * vloc].clone().requires_grad_()
        loss = vocab_parallel_cross_entropy(x @ hl, tgt, tp)
        loss.backward()
        out[name] = (abs(loss.item() - loss_ref.item()),
                     (e.weight.grad - dense.weight.grad[rank * vloc:(rank + 1) * vloc]).abs().max().item())
    return out


def test_vocab_parallel_embedding_and_cross_entropy():
    for res in run_ranks(_vocab_parallel_worker, 2):
        for name, (dl, dg) in res.items():
            assert dl < 1e-5 and dg < 1e-5, (name, dl, dg)


def _async_allreduce_worker(rank, world):
    from rumus_b200.parallel import all_reduce, async_all_reduce
    a = torch.full((1000,), float(rank + 1))
    b = torch.arange(4.0) * (rank + 1)
    ha = async_all_reduce(a)                    # mean, like the reference's barrier
    hb = async_all_reduce(b, average=False)
    c = torch.ones(3) * rank                    # independent work while the collectives run
    c = c * 2
    ra, rb = ha.wait(), hb.wait()
    assert ra is a and ha.is_completed() and ha.wait() is a    # waiting twice is harmless
    return ra[0].item(), rb.tolist(), all_reduce(c.clone()).tolist()


def test_async_all_reduce_handles():
    for ra, rb, rc in run_ranks(_async_allreduce_worker, 3):
        assert ra == 2.0 and rb == [0.0, 6.0, 12.0, 18.0] and rc == [2.0, 2.0, 2.0]


# ------------------------------------------------------------------ TP layers
def _tp_worker(rank, world):
    from rumus_b200.parallel.tp import ColumnParallelLinear, RowParallelLinear, TPContext, scatter_rows, gather_rows
    tp = TPContext(mode="nccl")
    torch.manual_seed(1)
    w1 = torch.randn(16, 32) * 0.2
    w2 = torch.randn(32, 16) * 0.2
    b2 = torch.randn(16) * 0.1
    x = torch.randn(8, 16)
    col = ColumnParallelLinear(16, 32, tp, bias=False)
    row = RowParallelLinear(32, 16, tp, bias=True)
    n = 32 // world
    with torch.no_grad():
        col.weight.copy_(w1[:, rank * n:(rank + 1) * n])
        row.weight.copy_(w2[rank * n:(rank + 1) * n])
        row.bias.copy_(b2)
    xs = x.clone().requires_grad_(True)
    y_local = row(torch.relu(col(scatter_rows(xs, tp))))
    y = gather_rows(y_local, tp)
    (y ** 2).sum().backward()
    xr = x.clone().requires_grad_(True)
    w1r, w2r = w1.clone().requires_grad_(True), w2.clone().requires_grad_(True)
    yr = torch.relu(xr @ w1r) @ w2r + b2
    (yr ** 2).sum().backward()
    assert torch.allclose(y, yr, atol=1e-5)
    # every rank seeds the loss on the full gathered output, so input grads arrive summed T times
    assert torch.allclose(xs.grad, xr.grad * world, atol=1e-4)
    assert torch.allclose(col.weight.grad, w1r.grad[:, rank * n:(rank + 1) * n] * world, atol=1e-4)
    assert torch.allclose(row.weight.grad, w2r.grad[rank * n:(rank + 1) * n] * world, atol=1e-4)
    return True


def test_tensor_parallel_linear_pair():
    assert all(run_ranks(_tp_worker, 2))


# ------------------------------------------------------------------ pipeline
def _pp_worker(rank, world):
    from rumus_b200.parallel.pp import PipelineStage, one_f_one_b_order
    torch.manual_seed(2)
    w = [torch.randn(8, 8) * 0.3 for _ in range(world)]
    mine = w[rank].clone().requires_grad_(True)
    M = 4
    g = torch.Generator().manual_seed(3)
    xs = [torch.randn(5, 8, generator=g) for _ in range(M)]
    ts = [torch.randn(5, 8, generator=g) for _ in range(M)]
    last = rank == world - 1

    def fwd(inp):
        if last:
            x, t = inp
            return ((torch.tanh(x @ mine) - t) ** 2).mean()
        return torch.tanh(inp @ mine)

    st = PipelineStage(fwd, rank, world, rank - 1 if rank > 0 else None, rank + 1 if not last else None,
                       (5, 8), torch.float32, torch.device("cpu"))
    log = []
    loss = st.run(xs if rank == 0 else ts, ops_log=log)
    assert log == one_f_one_b_order(rank, world, M)
    # single-process reference
    ws = [t.clone().requires_grad_(True) for t in w]
    tot = 0
    for x, t in zip(xs, ts):
        h = x
        for wi in ws:
            h = torch.tanh(h @ wi)
        tot = tot + ((h - t) ** 2).mean() / M
    tot.backward()
    assert torch.allclose(mine.grad, ws[rank].grad, atol=1e-6)
    if last:
        assert torch.allclose(loss, tot.detach(), atol=1e-6)
    return True


def test_pipeline_1f1b_matches_sequential():
    assert all(run_ranks(_pp_worker, 3))


def test_bubble_fraction_matches_schedule_length():
    from rumus_b200.parallel.pp import bubble_fraction, one_f_one_b_order
    for P, M in ((2, 8), (4, 8), (4, 4)):
        # stage 0's schedule has M forwards and M backwards; with unit-time slots the step spans
        # M + P - 1 slots per direction, the rest is the bubble
        assert len(one_f_one_b_order(0, P, M)) == 2 * M
        assert abs(bubble_fraction(P, M) - (P - 1) / (M + P - 1)) < 1e-12
    assert bubble_fraction(2, 8) == 1 / 9


def test_1f1b_order_properties():
    from rumus_b200.parallel.pp import one_f_one_b_order
    for P in (2, 4):
        for M in (1, 4, 8):
            for s in range(P):
                ops = one_f_one_b_order(s, P, M)
                assert [m for k, m in ops if k == "F"] == list(range(M))
                assert [m for k, m in ops if k == "B"] == list(range(M))
                live = peak = 0
                for k, _ in ops:
                    live += 1 if k == "F" else -1
                    peak = max(peak, live)
                assert peak <= min(P - s, M)     # bounded activation memory: the point of 1F1B


# ------------------------------------------------------------------ TP x PP Llama
def _tp_pp_worker(rank, world):
    from rumus_b200.models import Llama, LlamaConfig
    from rumus_b200.models.llama_parallel import ParallelLlamaStage
    from rumus_b200.parallel.pp import PipelineStage
    from rumus_b200.parallel.topology import build_topology
    from rumus_b200.parallel.tp import TPContext
    topo = build_topology(tp=2, pp=2)
    cfg = LlamaConfig(vocab_size=64, seq_len=8, d_model=32, num_heads=2, num_kv_heads=2, num_layers=2,
                      ffn_dim=64)
    torch.manual_seed(11)
    dense = Llama(cfg)
    tp = TPContext(group=topo.tp_group, mode="nccl")
    stage = ParallelLlamaStage(cfg, tp, topo.pp_idx, 2)
    stage.load_dense(dense.state_dict())
    B, S, M = 2, 8, 2
    stage.set_microbatch_shape(B, S)
    g = torch.Generator().manual_seed(12)
    toks = [torch.randint(0, 64, (B, S + 1), generator=g) for _ in range(M)]
    first, last = topo.pp_idx == 0, topo.pp_idx == 1
    mbs = [t[:, :-1] for t in toks] if first else [t[:, 1:] for t in toks]
    ps = PipelineStage(stage, topo.pp_idx, 2, topo.prev_stage_rank, topo.next_stage_rank,
                       (B * S // 2, cfg.d_model), torch.float32, torch.device("cpu"))
    loss = ps.run(mbs)
    ref = sum(dense(t[:, :-1], t[:, 1:]) for t in toks) / M
    ref.backward()
    if last:
        assert torch.allclose(loss, ref.detach(), atol=1e-5), (loss, ref)
    # gradient of this rank's shard of the first block's down projection
    per = cfg.num_layers // 2
    gd = dense.blocks[topo.pp_idx * per].mlp.down_proj.weight.grad
    f = cfg.ffn_dim // 2
    mine = stage.blocks[0].down.weight.grad
    assert torch.allclose(mine, gd[topo.tp_idx * f:(topo.tp_idx + 1) * f], atol=1e-5)
    # norm weights are replicated over the tensor-parallel ranks but only see this rank's token
    # slab: after the group sum every copy carries the dense gradient
    from rumus_b200.parallel.tp import sync_replicated_grads
    sync_replicated_grads(stage, tp)
    db = dense.blocks[topo.pp_idx * per]
    assert torch.allclose(stage.blocks[0].ln1.weight.grad, db.ln1.weight.grad, atol=1e-5)
    assert torch.allclose(stage.blocks[0].ln2.weight.grad, db.ln2.weight.grad, atol=1e-5)
    if last:
        assert torch.allclose(stage.ln_final.weight.grad, dense.ln_final.weight.grad, atol=1e-5)
    # shards -> reference-layout dense state dict (TP shards concatenated, stages merged on rank 0)
    full = stage.export_dense()
    if rank == 0:
        ref_sd = dense.state_dict()
        assert set(full) == set(ref_sd), set(ref_sd) ^ set(full)
        for k, v in ref_sd.items():
            assert torch.equal(full[k], v), k
    else:
        assert full is None
    return True


def test_llama_tp2_pp2_matches_dense():
    assert all(run_ranks(_tp_pp_worker, 4))


def _tp_pp_dp_train_worker(rank, world, tp_size, pp_size):
    """Two optimizer steps of the stage engine (flat arenas, deferred update over the micro-batches,
    gradient sums over the tensor-parallel group and averages over the replicas)."""
    from rumus_b200.models import LlamaConfig
    from rumus_b200.models.llama_parallel import ParallelLlamaStage
    from rumus_b200.parallel import FSDP
    from rumus_b200.parallel.pp import PipelineStage
    from rumus_b200.parallel.topology import build_topology
    from rumus_b200.parallel.tp import TPContext
    topo = build_topology(tp=tp_size, pp=pp_size)
    cfg = LlamaConfig(vocab_size=64, seq_len=8, d_model=32, num_heads=2, num_kv_heads=2, num_layers=2,
                      ffn_dim=64)
    tp = TPContext(group=topo.tp_group, mode="nccl")
    stage = ParallelLlamaStage(cfg, tp, topo.pp_idx, pp_size)
    stage.init_weights(0.05, seed=3)
    B, S, M = 2, 8, 2
    stage.set_microbatch_shape(B, S)
    units = [(f"blocks.{i}", [b]) for i, b in enumerate(stage.blocks)]
    rest = [p for n, p in stage.named_parameters() if not n.startswith("blocks.")]
    if rest:
        units.append(("edge", rest))
    opt = FSDP(stage, lr=1e-2, unit_roots=units, local_only=True, defer_update=True)
    ps = PipelineStage(stage, topo.pp_idx, pp_size, topo.prev_stage_rank, topo.next_stage_rank,
                       (B * S // tp_size, cfg.d_model), torch.float32, torch.device("cpu"))
    g = torch.Generator().manual_seed(40 + topo.dp_idx)       # every replica sees its own data
    first = topo.pp_idx == 0
    for _ in range(2):
        toks = [torch.randint(0, 64, (B, S + 1), generator=g) for _ in range(M)]
        mbs = [t[:, :-1] for t in toks] if first else [t[:, 1:] for t in toks]
        opt.zero_grad()
        ps.run(mbs)
        opt.reduce_grads(replicated_group=topo.tp_group, dp_group=topo.dp_group)
        opt.step()
    norms = {n: p.detach().clone() for n, p in stage.named_parameters() if "ln" in n}
    sharded = {n: p.detach().clone() for n, p in stage.named_parameters() if "ln" not in n}
    return {"dp": topo.dp_idx, "pp": topo.pp_idx, "tp": topo.tp_idx, "norms": norms, "sharded": sharded}


def test_llama_stage_engine_keeps_replicated_weights_in_sync():
    # tp2 x pp2: the norm weights of the two tensor-parallel ranks of a stage stay identical and move
    out = run_ranks(_tp_pp_dp_train_worker, 4, 2, 2)
    for pp in (0, 1):
        a, b = [o for o in out if o["pp"] == pp]
        assert a["norms"] and all(torch.equal(a["norms"][k], b["norms"][k]) for k in a["norms"])
        assert any((v - 1.0).abs().max() > 1e-4 for v in a["norms"].values())


def test_llama_tp2_pp2_dp2_replicas_stay_identical():
    out = run_ranks(_tp_pp_dp_train_worker, 8, 2, 2, timeout=400)
    for pp in (0, 1):
        for tp in (0, 1):
            a, b = [o for o in out if o["pp"] == pp and o["tp"] == tp]
            assert a["dp"] != b["dp"]
            for k in a["sharded"]:
                assert torch.equal(a["sharded"][k], b["sharded"][k]), k
            for k in a["norms"]:
                assert torch.equal(a["norms"][k], b["norms"][k]), k


# ------------------------------------------------------------------ DP
def _dp_worker(rank, world):
    from rumus_b200.parallel.dp import DataParallel
    import rumus_b200.nn as rnn
    torch.manual_seed(20 + rank)      # different init per rank: broadcast must sync them
    m = torch.nn.Sequential(rnn.Linear(6, 5), torch.nn.ReLU(), rnn.Linear(5, 2))
    dp = DataParallel(m)
    g = torch.Generator().manual_seed(21)
    x = torch.randn(world * 3, 6, generator=g)
    dp.zero_grad()
    (m(x[rank * 3:(rank + 1) * 3]) ** 2).mean().backward()
    found = dp.all_reduce_grads()
    assert int(found.item()) == 0
    return [p.detach().clone() for p in m.parameters()], [p.grad.clone() for p in m.parameters()], x


def test_data_parallel_mean_gradients():
    outs = run_ranks(_dp_worker, 2)
    (p0, g0, x), (p1, g1, _) = outs
    for a, b in zip(p0, p1):
        assert torch.equal(a, b)
    for a, b in zip(g0, g1):
        assert torch.allclose(a, b, atol=1e-6)
    import rumus_b200.nn as rnn
    m = torch.nn.Sequential(rnn.Linear(6, 5), torch.nn.ReLU(), rnn.Linear(5, 2))
    with torch.no_grad():
        for p, v in zip(m.parameters(), p0):
            p.copy_(v)
    (m(x) ** 2).mean().backward()
    for p, gref in zip(m.parameters(), g0):
        assert torch.allclose(p.grad, gref, atol=1e-6)


def _dp_overlap_worker(rank, world):
    from rumus_b200.parallel.dp import DataParallel
    torch.manual_seed(30)
    m = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 4),
                            torch.nn.Tanh(), torch.nn.Linear(4, 2))
    dp = DataParallel(m, bucket_mb=0)          # one bucket per parameter
    assert len(dp.buckets) == 6
    g = torch.Generator().manual_seed(31)
    x = torch.randn(world * 3, 6, generator=g)
    launched_during_backward = []
    for use_overlap in (True, False):
        dp.zero_grad()
        if use_overlap:
            dp.begin_backward()
        (m(x[rank * 3:(rank + 1) * 3]) ** 2).mean().backward()
        launched_during_backward.append(sum(dp._launched) if use_overlap else 0)
        found = dp.all_reduce_grads()
        assert int(found.item()) == 0
        if use_overlap:
            g_overlap = [p.grad.clone() for p in m.parameters()]
        else:
            g_plain = [p.grad.clone() for p in m.parameters()]
    return g_overlap, g_plain, launched_during_backward[0]


def test_data_parallel_overlapped_buckets_match_plain():
    outs = run_ranks(_dp_overlap_worker, 2)
    for g_overlap, g_plain, n_launched in outs:
        assert n_launched == 6, "every bucket must have been reduced from its hook during backward"
        for a, b in zip(g_overlap, g_plain):
            assert torch.allclose(a, b, atol=1e-6)
    for a, b in zip(outs[0][0], outs[1][0]):
        assert torch.allclose(a, b, atol=1e-6)


def test_topology_groups():
    from rumus_b200.parallel.topology import groups_for
    g = groups_for(8, tp=4, pp=2)
    assert g["tp"] == [[0, 1, 2, 3], [4, 5, 6, 7]] and g["pp"][0] == [0, 4] and g["dp_size"] == 1
    g = groups_for(8, tp=2, pp=2)
    assert g["dp"][0] == [0, 4] and len(g["tp"]) == 4


# ------------------------------------------------------------------ context parallel attention
def _cp_inputs(B=2, S=24, H=4, Hkv=2, D=8):
    g = torch.Generator().manual_seed(11)
    q = torch.randn(B, S, H, D, generator=g)
    k = torch.randn(B, S, Hkv, D, generator=g)
    v = torch.randn(B, S, Hkv, D, generator=g)
    w = torch.randn(B, S, H, D, generator=g)
    return q, k, v, w


def _cp_worker(rank, world, scheme, causal):
    from rumus_b200.parallel.cp import ring_attention, ulysses_attention
    q, k, v, w = _cp_inputs()
    S = q.shape[1]
    sl = slice(rank * S // world, (rank + 1) * S // world)
    ql, kl, vl = (t[:, sl].clone().requires_grad_(True) for t in (q, k, v))
    fn = ulysses_attention if scheme == "ulysses" else ring_attention
    o = fn(ql, kl, vl, causal)
    (o * w[:, sl]).sum().backward()
    return {"o": o.detach(), "dq": ql.grad, "dk": kl.grad, "dv": vl.grad}


def _cp_check(scheme, causal, world):
    from rumus_b200.ops import functional as F
    q, k, v, w = _cp_inputs()
    qr, kr, vr = (t.clone().requires_grad_(True) for t in (q, k, v))
    o_ref = F.sdpa_reference(qr, kr, vr, causal)
    (o_ref * w).sum().backward()
    outs = run_ranks(_cp_worker, world, scheme, causal)
    S = q.shape[1]
    for r in range(world):
        sl = slice(r * S // world, (r + 1) * S // world)
        assert torch.allclose(outs[r]["o"], o_ref[:, sl].detach(), atol=2e-5), (scheme, causal, r)
        assert torch.allclose(outs[r]["dq"], qr.grad[:, sl], atol=5e-5)
        assert torch.allclose(outs[r]["dk"], kr.grad[:, sl], atol=5e-5)
        assert torch.allclose(outs[r]["dv"], vr.grad[:, sl], atol=5e-5)


def test_context_parallel_ulysses_matches_full_attention():
    _cp_check("ulysses", True, 2)
    _cp_check("ulysses", False, 2)


def test_context_parallel_ring_matches_full_attention():
    _cp_check("ring", True, 3)
    _cp_check("ring", False, 2)
