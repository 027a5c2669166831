"""Serving kernels on the GPU: INT4 GEMV / dequant-GEMM, INT8 blocks, paged decode attention,
KV append, argmax, and the engine end to end (GPU results == CPU engine results)."""
import random

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("M", [1, 7, 32, 45, 128, 200])
@pytest.mark.parametrize("K,N", [(4096, 1536), (1000, 264)])
def test_int4_matmul(M, K, N):
    from rumus_b200.nn.quant import QuantizedTensor, qmatmul_int4
    torch.manual_seed(M + K)
    w = torch.randn(K, N) * 0.05
    q = QuantizedTensor.from_f32(w, 128, torch.float16).to("cuda")
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    y = qmatmul_int4(x, q)
    ref = x.detach().float() @ q.dequantize(torch.float32)
    assert _rel(y, ref) < 1e-2
    y.float().sum().backward()
    gref = torch.ones(M, N, device="cuda") @ q.dequantize(torch.float32).t()
    assert _rel(x.grad, gref) < 1e-2


@pytest.mark.parametrize("M", [2, 5, 16, 32, 70])
def test_int4_gemv_all_row_buckets(M, monkeypatch):
    """The streaming GEMV at every row bucket (and chunked above 32 rows), whatever the dispatch
    threshold currently is."""
    from rumus_b200.nn.quant import QuantizedTensor
    from rumus_b200.ops import quant_cuda as Q
    monkeypatch.setattr(Q, "GEMV_CHUNKED_MAX_M", 128)
    torch.manual_seed(M)
    K, N = 1160, 520     # K is not a multiple of the group size, N not of 512
    w = torch.randn(K, N) * 0.05
    q = QuantizedTensor.from_f32(w, 128, torch.float16).to("cuda")
    x = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    y = Q.int4_matmul(x, q, bias)
    ref = x.float() @ q.dequantize(torch.float32) + bias.float()
    assert _rel(y, ref) < 1e-2


def test_q8_roundtrip_and_matmul():
    from rumus_b200.nn.quant import dequantize_q8, matmul_q8, quantize_q8
    torch.manual_seed(0)
    w = torch.randn(256, 48)
    qc = quantize_q8(w, 32)
    qg = quantize_q8(w.cuda(), 32)
    assert torch.equal(qc.data, qg.data.cpu())          # same bytes as the CPU restatement
    assert torch.allclose(dequantize_q8(qg).cpu(), dequantize_q8(qc), atol=1e-6)
    x = torch.randn(9, 256, device="cuda")
    assert _rel(matmul_q8(x, qg), x @ dequantize_q8(qc).cuda()) < 2e-3


def test_paged_decode_attention_and_argmax():
    from rumus_b200.serve.engine import greedy_sample, paged_decode_attention
    torch.manual_seed(1)
    B, H, Hkv, D, bs, nblk = 5, 8, 4, 128, 16, 200
    kc = (torch.randn(nblk, bs, Hkv, D, device="cuda") * 0.5).bfloat16()
    vc = (torch.randn(nblk, bs, Hkv, D, device="cuda") * 0.5).bfloat16()
    ctx = torch.tensor([1, 17, 300, 1000, 64], dtype=torch.int32, device="cuda")
    maxb = 64
    tables = torch.stack([torch.randperm(nblk)[:maxb] for _ in range(B)]).int().cuda()
    q = (torch.randn(B, H, D, device="cuda") * 0.5).bfloat16()
    out = paged_decode_attention(q, kc, vc, tables, ctx, D ** -0.5, 1000)
    ref = paged_decode_attention(q.cpu().float(), kc.cpu().float(), vc.cpu().float(), tables.cpu(),
                                 ctx.cpu(), D ** -0.5, 1000)
    assert _rel(out.cpu(), ref) < 1e-2
    logits = torch.randn(7, 32000, device="cuda").bfloat16()
    ids, vals = greedy_sample(logits)
    assert torch.equal(ids.cpu(), logits.float().argmax(-1).cpu())


def test_engine_gpu_generates_and_frees_blocks():
    from rumus_b200.models.llama import LlamaConfig
    from rumus_b200.serve import Engine, ServeConfig
    mc = LlamaConfig(vocab_size=512, seq_len=512, d_model=256, num_heads=2, num_kv_heads=2, num_layers=2,
                     ffn_dim=512)
    cfg = ServeConfig(model=mc, num_blocks=128, block_size=16, max_batch=8, token_budget=256)
    e = Engine(cfg, torch.device("cuda"))
    r = random.Random(0)
    want = {}
    for i in range(6):
        n = r.randint(4, 12)
        want[i + 1] = n
        e.add_request(i + 1, [r.randrange(512) for _ in range(r.randint(10, 300))], n)
    outs = {}
    while e.has_work():
        for rid in e.step():
            outs[rid] = e.requests.pop(rid).output
    assert {k: len(v) for k, v in outs.items()} == want
    assert e.sched.free_blocks() == 128
    from rumus_b200.ops import native
    assert native.read_status() == 0


def test_engine_decode_graphs_match_eager_decode():
    """Decode steps replayed from captured CUDA graphs (padded batch, static inputs) produce the same
    tokens as launching every kernel eagerly (split-K sums are not ordered, so a near-tie between two
    logits may fall the other way: most sequences, not all, have to agree token for token)."""
    import dataclasses
    from rumus_b200.models.llama import LlamaConfig
    from rumus_b200.ops import native
    from rumus_b200.serve import Engine, ServeConfig
    mc = LlamaConfig(vocab_size=512, seq_len=512, d_model=256, num_heads=2, num_kv_heads=2, num_layers=2,
                     ffn_dim=512)
    base = ServeConfig(model=mc, num_blocks=128, block_size=16, max_batch=8, token_budget=256)
    results = []
    for graphs in (False, True):
        e = Engine(dataclasses.replace(base, cuda_graphs=graphs), torch.device("cuda"), seed=3)
        r = random.Random(1)
        for i in range(7):
            e.add_request(i + 1, [r.randrange(512) for _ in range(r.randint(5, 200))], r.randint(3, 20))
        outs = {}
        while e.has_work():
            for rid in e.step():
                outs[rid] = e.requests.pop(rid).output
        results.append(outs)
        assert (e.graph_replays > 0) == graphs
        assert e.sched.free_blocks() == 128
    assert native.read_status() == 0
    assert results[0].keys() == results[1].keys()
    assert all(len(results[0][k]) == len(results[1][k]) for k in results[0])
    same = sum(results[0][k] == results[1][k] for k in results[0])
    assert same >= 5, (same, results)
