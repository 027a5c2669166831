"""Head-major KV cache on the GPU: the `_hm` append and decode-attention kernels against the
token-major kernels and the CPU restatement, on the same data."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def test_head_major_kernels_match_token_major():
    from rumus_b200.models.llama import LlamaConfig
    from rumus_b200.serve import ServeConfig
    from rumus_b200.serve.engine import PagedKVCache, paged_decode_attention
    torch.manual_seed(1)
    B, H, Hkv, D, bs, nblk = 5, 8, 4, 128, 16, 400     # 5 sequences x 64 distinct blocks each
    mc = LlamaConfig(vocab_size=64, seq_len=2048, d_model=H * D, num_heads=H, num_kv_heads=Hkv, num_layers=1,
                     ffn_dim=64)
    ctx_list = [1000, 17, 512, 333, 64]
    max_blocks = 64
    perm = torch.randperm(nblk)[: B * max_blocks].view(B, max_blocks)
    tables = perm.to(torch.int32).cuda()
    ctx = torch.tensor(ctx_list, dtype=torch.int32, device="cuda")
    q = (torch.randn(B, H, D, device="cuda") * 0.5).bfloat16()
    outs = {}
    caches = {}
    for hm in (False, True):
        cfg = ServeConfig(model=mc, num_blocks=nblk, block_size=bs, max_batch=8, token_budget=2048,
                          dtype=torch.bfloat16, kv_head_major=hm)
        cache = PagedKVCache(cfg, Hkv, D, torch.device("cuda"))
        g = torch.Generator(device="cuda").manual_seed(7)
        for b, n in enumerate(ctx_list):
            # rows are strided views of a wider buffer, like the fused qkv projection output
            wide = (torch.randn(n, 3 * Hkv * D, device="cuda", generator=g) * 0.5).bfloat16()
            k_src, v_src = wide[:, : Hkv * D], wide[:, Hkv * D: 2 * Hkv * D]
            pos = torch.arange(n, device="cuda")
            slots = perm[b].cuda()[pos // bs].to(torch.int64) * bs + pos % bs
            cache.append(0, k_src, v_src, slots)
            kk, vv = cache.gather(0, perm[b].cuda(), pos)
            assert torch.equal(kk.reshape(n, -1), k_src) and torch.equal(vv.reshape(n, -1), v_src)
        outs[hm] = paged_decode_attention(q, cache.k[0], cache.v[0], tables, ctx, D ** -0.5, 1000, head_major=hm)
        caches[hm] = cache
    ref = paged_decode_attention(q.cpu().float(), caches[False].k[0].cpu().float(), caches[False].v[0].cpu().float(),
                                 tables.cpu(), ctx.cpu(), D ** -0.5, 1000)
    assert _rel(outs[False].cpu(), ref) < 1e-2
    assert _rel(outs[True].cpu(), ref) < 1e-2
    assert _rel(outs[True], outs[False]) < 1e-3
