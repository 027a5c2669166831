"""Finite-difference gradient checks in fp64 of every hand-written backward that runs on CPU
tensors (the formulas the CUDA paths are compared against in the GPU suite)."""
import torch
from torch.autograd import gradcheck

from rumus_b200.ops import functional as F


def _r(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g, dtype=torch.float64) * scale).requires_grad_()


def test_composed_attention_and_reference_attention():
    q, k, v = _r(2, 5, 2, 4, seed=1), _r(2, 5, 2, 4, seed=2), _r(2, 5, 2, 4, seed=3)
    for causal in (False, True):
        assert gradcheck(lambda a, b, c: F.sdpa_reference(a, b, c, causal), (q, k, v), atol=1e-6)
        assert gradcheck(lambda a, b, c: F._sdpa_composed(a, b, c, causal, 0.5), (q, k, v), atol=1e-6)
        assert gradcheck(lambda a, b, c: F.flash_attention(a, b, c, causal), (q, k, v), atol=1e-6)


def test_grouped_query_attention_reference():
    q, k, v = _r(1, 6, 4, 4, seed=1), _r(1, 6, 2, 4, seed=2), _r(1, 6, 2, 4, seed=3)
    assert gradcheck(lambda a, b, c: F.sdpa_reference(a, b, c, True), (q, k, v), atol=1e-6)


def test_rope_is_differentiable_and_orthogonal():
    qkv = _r(2, 6, (2 + 2 * 1) * 8, seed=4)
    fn = lambda t: F.rope_qkv(t, 6, 2, 1, 8, 10000.0)
    assert gradcheck(fn, (qkv,), atol=1e-6)
    y = fn(qkv)
    # rotation: q and k parts keep their norms, v is untouched
    assert torch.allclose(y[..., :24].norm(), qkv[..., :24].norm()) and torch.equal(y[..., 24:], qkv[..., 24:])


def test_pointwise_and_fused_blocks():
    x = _r(7, 6, seed=5)
    for fn in (F.relu, F.gelu, F.silu, F.sigmoid, F.tanh, lambda t: F.leaky_relu(t, 0.1)):
        xs = (x.detach() + 0.05).requires_grad_()     # keep away from the ReLU kink
        assert gradcheck(fn, (xs,), atol=1e-6)
    assert gradcheck(F.swiglu, (_r(5, 8, seed=6),), atol=1e-6)
    w1, b1, w2, b2 = _r(6, 10, seed=7, scale=0.3), _r(10, seed=8), _r(10, 6, seed=9, scale=0.3), _r(6, seed=10)
    for act in ("gelu", "relu", "silu"):
        assert gradcheck(lambda a, b, c, d, e: F.mlp(a, b, c, d, e, act=act, residual=a), (x, w1, b1, w2, b2), atol=1e-6)
        assert gradcheck(lambda a, b, c: F.linear(a, b, c, act=act, residual=None), (x, w1, b1), atol=1e-6)


def test_norms_softmax_and_losses():
    x, g, b = _r(5, 12, seed=11), _r(12, seed=12), _r(12, seed=13)
    assert gradcheck(lambda a, c, d: F.layer_norm(a, c, d), (x, g, b), atol=1e-6)
    assert gradcheck(lambda a, c: F.rms_norm(a, c), (x, g), atol=1e-6)
    assert gradcheck(lambda a, c, d: F.layer_norm(a, c, d, residual=a * 0.5), (x, g, b), atol=1e-6)
    assert gradcheck(F.softmax, (x,), atol=1e-6)
    tgt = torch.randint(0, 12, (5,))
    assert gradcheck(lambda a: F.cross_entropy_loss(a, tgt), (x,), atol=1e-6)
    w = _r(12, 9, seed=14, scale=0.3)
    tgt9 = torch.randint(0, 9, (5,))
    assert gradcheck(lambda a, c: F.lm_head_loss(a, c, tgt9), (x, w), atol=1e-6)
    target = x.detach().clone() * 0.3
    assert gradcheck(lambda a: F.mse_loss(a, target), (x,), atol=1e-6)


def test_embedding_with_positions():
    w, pos = _r(10, 4, seed=15), _r(6, 4, seed=16)
    idx = torch.randint(0, 10, (2, 6))
    assert gradcheck(lambda a, p: F.embedding(idx, a, p), (w, pos), atol=1e-6)
    assert gradcheck(lambda a: F.embedding(idx, a), (w,), atol=1e-6)


def test_vocab_parallel_functions_single_rank():
    from rumus_b200.models.llama_parallel import _VocabParallelCE
    from rumus_b200.parallel.tp import TPContext, _VocabParallelEmbedFn
    tp = TPContext(mode="nccl")                      # world 1: the collectives are identities
    logits = _r(6, 10, seed=17)
    tgt = torch.randint(0, 10, (6,))
    assert gradcheck(lambda a: _VocabParallelCE.apply(a, tgt, tp, 0), (logits,), atol=1e-6)
    # a rank that holds rows [4, 9) of a larger vocabulary: targets outside contribute through the sums only
    assert gradcheck(lambda a: _VocabParallelCE.apply(a, tgt, tp, 4), (logits,), atol=1e-6)
    w = _r(5, 3, seed=18)
    tok = torch.tensor([0, 3, 4, 7, 8, 9, 4])
    assert gradcheck(lambda a: _VocabParallelEmbedFn.apply(a, tok, tp, 4, False), (w,), atol=1e-6)


def test_vision_ops():
    x = _r(2, 3, 6, 6, seed=19)
    w = _r(4, 3, 3, 3, seed=20, scale=0.3)
    b = _r(4, seed=21)
    from rumus_b200.ops import vision as V
    assert gradcheck(lambda a, c, d: V.conv2d(a, c, d, stride=2, padding=1), (x, w, b), atol=1e-6)
    assert gradcheck(lambda a: F.adaptive_avg_pool2d(a, 2), (x,), atol=1e-6)
    assert gradcheck(lambda a: F.max_pool2d(a + 0.0, 3, 2, 1), (x,), atol=1e-6)
    rm, rv = torch.zeros(3, dtype=torch.float64), torch.ones(3, dtype=torch.float64)
    g, bb = _r(3, seed=22), _r(3, seed=23)
    assert gradcheck(lambda a, c, d: F.batch_norm_2d(a, c, d, rm.clone(), rv.clone(), True), (x, g, bb), atol=1e-5)


def test_graph_spmm_and_custom_op():
    from rumus_b200.ext import CustomOp, custom_forward
    from rumus_b200.graph import Graph
    g = Graph.new(5, [0, 1, 2, 3, 0], [1, 2, 3, 4, 4], [1., 2., 3., 4., 5.])
    x = _r(5, 3, seed=24)
    assert gradcheck(lambda a: g.spmm(a), (x,), atol=1e-6)
    op = CustomOp("cube", "", "k", 1, output_shape=lambda s: s[0], cpu_fn=lambda a: a ** 3,
                  backward=lambda go, ins, out: (3 * ins[0] ** 2 * go,))
    assert gradcheck(lambda a: custom_forward(op, a), (x,), atol=1e-6)
