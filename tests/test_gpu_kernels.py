"""Numerics of the sm_100a kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu


def _native():
    from rumus_b200.ops import native
    return native


def _rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    if torch.cuda.is_available():
        assert _native().read_status() == 0, "a device-side bounded wait timed out"


# ------------------------------------------------------------------ GEMM
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
@pytest.mark.parametrize("a_t,b_t", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("shape", [(256, 512, 384), (304, 200, 136), (128, 128, 64), (1000, 264, 72)])
def test_gemm_tcgen05_majors(dtype, a_t, b_t, shape):
    native = _native()
    M, N, K = shape
    g = torch.Generator(device="cuda").manual_seed(M * 7 + N * 3 + K)
    a_store = torch.randn((K, M) if a_t else (M, K), device="cuda", generator=g).to(dtype)
    b_store = torch.randn((N, K) if b_t else (K, N), device="cuda", generator=g).to(dtype)
    a = a_store.t() if a_t else a_store
    b = b_store.t() if b_t else b_store
    out = native.gemm(a, b, path=1)
    assert native.gemm.last_path == 1
    ref = a.float() @ b.float()
    tol = 2e-2 if dtype != torch.float32 else 2e-3  # tf32 inputs for fp32
    assert _rel_err(out, ref) < tol, (_rel_err(out, ref), dtype, a_t, b_t, shape)


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_large_persistent(bn):
    native = _native()
    M, N, K = 2048, 1536, 1024
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(K, N, device="cuda").bfloat16()
    out = native.gemm(a, b, path=1, bn=bn)
    ref = a.float() @ b.float()
    assert _rel_err(out, ref) < 1e-2
    # fp32 output
    out32 = native.gemm(a, b, path=1, bn=bn, out_dtype=torch.float32)
    assert out32.dtype == torch.float32
    assert _rel_err(out32, ref) < 5e-3


@pytest.mark.parametrize("split_k", [0, 3, 7])
def test_gemm_split_k_weight_gradient_shape(split_k):
    """Few output tiles, long K (convolution weight gradients): K slices as separate work items."""
    native = _native()
    M, N, K = 200, 136, 12544   # 2 x 2 tiles of 128; K = 196 K-blocks of 64
    x = torch.randn(K, M, device="cuda").half()
    dy = torch.randn(K, N, device="cuda").half()
    ref = x.float().t() @ dy.float()
    out = native.gemm(x.t(), dy, path=1, split_k=split_k)
    assert out.dtype == torch.float16
    assert _rel_err(out, ref) < 5e-3
    acc = torch.randn(M, N, device="cuda").half()
    out2 = native.gemm(x.t(), dy, path=1, split_k=split_k, out=acc.clone(), residual=acc)
    assert _rel_err(out2, ref + acc.float()) < 5e-3


def test_gemm_epilogues():
    native = _native()
    M, N, K = 384, 512, 256
    a = (torch.randn(M, K, device="cuda") * 0.5).bfloat16()
    b = (torch.randn(K, N, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda").bfloat16()
    res = torch.randn(M, N, device="cuda").bfloat16()
    pre_ref = a.float() @ b.float() + bias.float()
    for act, fn in [("relu", torch.relu), ("gelu", lambda t: TF.gelu(t, approximate="tanh")),
                    ("silu", TF.silu)]:
        out, pre = native.gemm(a, b, bias=bias, act=act, residual=res, aux_out=True, path=1)
        assert _rel_err(pre, pre_ref) < 1e-2
        assert _rel_err(out, fn(pre_ref) + res.float()) < 1e-2
    # derivative epilogue: out = (a@b) * gelu'(aux)
    aux = torch.randn(M, N, device="cuda").bfloat16()
    out = native.gemm(a, b, aux_in=aux, dact="gelu", path=1)
    x = aux.float().requires_grad_(True)
    TF.gelu(x, approximate="tanh").sum().backward()
    assert _rel_err(out, (a.float() @ b.float()) * x.grad) < 1.5e-2


@pytest.mark.parametrize("shape", [(5, 3, 7), (64, 10, 33), (130, 70, 257)])
def test_gemm_simt_fallback_odd_shapes(shape):
    native = _native()
    M, N, K = shape
    a = torch.randn(M, K, device="cuda")
    b = torch.randn(K, N, device="cuda")
    bias = torch.randn(N, device="cuda")
    out = native.gemm(a, b, bias=bias, act="relu")
    assert native.gemm.last_path == 2
    assert torch.allclose(out, torch.relu(a @ b + bias), atol=1e-4, rtol=1e-4)
    o2 = native.gemm(a.t().contiguous().t(), b.t().contiguous().t())
    assert torch.allclose(o2, a @ b, atol=1e-4, rtol=1e-4)


def test_bmm():
    native = _native()
    a = torch.randn(6, 33, 17, device="cuda")
    b = torch.randn(6, 17, 29, device="cuda")
    assert torch.allclose(native.bmm(a, b), torch.bmm(a, b), atol=1e-4, rtol=1e-4)
    assert torch.allclose(native.bmm(a, b.transpose(1, 2).contiguous().transpose(1, 2)),
                          torch.bmm(a, b), atol=1e-4, rtol=1e-4)


def test_linear_and_mlp_autograd():
    from rumus_b200.ops import functional as F
    torch.manual_seed(0)
    x = (torch.randn(4, 96, 256, device="cuda") * 0.5).bfloat16().requires_grad_(True)
    w1 = (torch.randn(256, 1024, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b1 = (torch.randn(1024, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    w2 = (torch.randn(1024, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    b2 = (torch.randn(256, device="cuda") * 0.1).bfloat16().requires_grad_(True)
    y = F.mlp(x, w1, b1, w2, b2, act="gelu", residual=x)
    y.float().pow(2).mean().backward()
    ps = [x, w1, b1, w2, b2]
    got = [p.grad.clone() for p in ps]
    refs = [p.detach().float().requires_grad_(True) for p in ps]
    xr, w1r, b1r, w2r, b2r = refs
    yr = TF.gelu(xr @ w1r + b1r, approximate="tanh") @ w2r + b2r + xr
    yr.pow(2).mean().backward()
    assert _rel_err(y, yr) < 1e-2
    for g, r in zip(got, refs):
        assert _rel_err(g, r.grad) < 3e-2
    # plain linear with activation
    for p in ps:
        p.grad = None
    z = F.linear(x, w1, b1, act="relu")
    z.float().sum().backward()
    xr.grad = None; w1r.grad = None; b1r.grad = None
    torch.relu(xr @ w1r + b1r).sum().backward()
    assert _rel_err(x.grad, xr.grad) < 3e-2
    assert _rel_err(w1.grad, w1r.grad) < 3e-2
    assert _rel_err(b1.grad, b1r.grad) < 3e-2


# ------------------------------------------------------------------ norms
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("D", [128, 2048, 100, 4096 + 8])
@pytest.mark.parametrize("rms", [False, True])
def test_norm_fwd_bwd(dtype, D, rms):
    from rumus_b200.ops import functional as F
    rows = 77
    x = torch.randn(rows, D, device="cuda").to(dtype).requires_grad_(True)
    res = torch.randn(rows, D, device="cuda").to(dtype).requires_grad_(True)
    g = (1 + 0.1 * torch.randn(D, device="cuda")).to(dtype).requires_grad_(True)
    b = (0.1 * torch.randn(D, device="cuda")).to(dtype).requires_grad_(True)
    if rms:
        y, h = F.rms_norm(x, g, 1e-6, residual=res)
    else:
        y, h = F.layer_norm(x, g, b, 1e-5, residual=res)
    w = torch.randn_like(y, dtype=torch.float32)
    ((y.float() * w).sum() + h.float().pow(2).sum()).backward()
    xr, rr, gr, br = (t.detach().float().requires_grad_(True) for t in (x, res, g, b))
    hr = xr + rr
    if rms:
        yr = hr * torch.rsqrt(hr.pow(2).mean(-1, keepdim=True) + 1e-6) * gr
    else:
        yr = TF.layer_norm(hr, (D,), gr, br, 1e-5)
    ((yr * w).sum() + hr.pow(2).sum()).backward()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-4
    assert _rel_err(y, yr) < tol
    assert _rel_err(x.grad, xr.grad) < tol
    assert _rel_err(res.grad, rr.grad) < tol
    assert _rel_err(g.grad, gr.grad) < tol
    if not rms:
        assert _rel_err(b.grad, br.grad) < tol


# ------------------------------------------------------------------ softmax / CE
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [7, 1024, 50304 // 8 + 3])
def test_softmax(dtype, n):
    from rumus_b200.ops import functional as F
    x = (torch.randn(19, n, device="cuda") * 3).to(dtype).requires_grad_(True)
    y = F.softmax(x)
    w = torch.randn_like(y)
    (y * w).sum().backward()
    xr = x.detach().float().requires_grad_(True)
    yr = torch.softmax(xr, -1)
    (yr * w.float()).sum().backward()
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    assert _rel_err(y, yr) < tol
    assert _rel_err(x.grad, xr.grad) < (6e-2 if dtype == torch.bfloat16 else 1e-4)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n", [3, 1000, 50304])
def test_cross_entropy(dtype, n):
    from rumus_b200.ops import functional as F
    rows = 33
    x = (torch.randn(rows, n, device="cuda") * 2).to(dtype).requires_grad_(True)
    t = torch.randint(0, n, (rows,), device="cuda")
    loss = F.cross_entropy_loss(x, t)
    loss.backward()
    xr = x.detach().float().requires_grad_(True)
    lr = TF.cross_entropy(xr, t)
    lr.backward()
    assert abs(loss.item() - lr.item()) < (2e-2 if dtype == torch.bfloat16 else 1e-4)
    assert _rel_err(x.grad, xr.grad) < (2e-2 if dtype == torch.bfloat16 else 1e-4)


# ------------------------------------------------------------------ pointwise
@pytest.mark.parametrize("name", ["relu", "gelu", "silu", "sigmoid", "tanh", "leaky_relu"])
def test_activations(name):
    from rumus_b200.ops import functional as F
    x = torch.randn(1000, 37, device="cuda", requires_grad=True)
    y = getattr(F, name)(x)
    y.sum().backward()
    xr = x.detach().cpu().requires_grad_(True)
    yr = getattr(F, name)(xr)
    yr.sum().backward()
    assert torch.allclose(y.cpu(), yr, atol=1e-5, rtol=1e-4)
    assert torch.allclose(x.grad.cpu(), xr.grad, atol=1e-5, rtol=1e-4)


def test_swiglu_rope_embedding_dropout():
    from rumus_b200.ops import functional as F
    gu = torch.randn(50, 2 * 96, device="cuda").bfloat16().requires_grad_(True)
    y = F.swiglu(gu)
    y.float().sum().backward()
    gr = gu.detach().float().requires_grad_(True)
    yr = F.swiglu(gr.cpu()).cuda() if False else TF.silu(gr[:, :96]) * gr[:, 96:]
    yr.sum().backward()
    assert _rel_err(y, yr) < 1e-2 and _rel_err(gu.grad, gr.grad) < 2e-2
    # rope: GPU kernel vs torch formula, forward + backward
    B, S, H, hd = 2, 24, 4, 64
    qkv = torch.randn(B, S, 3 * H * hd, device="cuda", requires_grad=True)
    out = F.rope_qkv(qkv * 1.0, S, H, H, hd)
    w = torch.randn_like(out)
    (out * w).sum().backward()
    qc = qkv.detach().cpu().requires_grad_(True)
    oc = F.rope_qkv(qc * 1.0, S, H, H, hd)
    (oc * w.cpu()).sum().backward()
    assert torch.allclose(out.cpu(), oc, atol=1e-4, rtol=1e-4)
    assert torch.allclose(qkv.grad.cpu(), qc.grad, atol=1e-4, rtol=1e-4)
    # embedding (+pos) forward/backward
    W = torch.randn(100, 64, device="cuda", requires_grad=True)
    P = torch.randn(16, 64, device="cuda", requires_grad=True)
    idx = torch.randint(0, 100, (3, 16), device="cuda")
    e = F.embedding(idx, W, P)
    e.pow(2).sum().backward()
    Wr, Pr = W.detach().cpu().requires_grad_(True), P.detach().cpu().requires_grad_(True)
    er = F.embedding(idx.cpu(), Wr, Pr)
    er.pow(2).sum().backward()
    assert torch.allclose(e.cpu(), er, atol=1e-5)
    assert torch.allclose(W.grad.cpu(), Wr.grad, atol=1e-4)
    assert torch.allclose(P.grad.cpu(), Pr.grad, atol=1e-4)
    # dropout: keep ratio and scaling
    x = torch.ones(1 << 20, device="cuda", requires_grad=True)
    d = F.dropout(x, 0.25, True, seed=1234)
    keep = (d != 0).float().mean().item()
    assert abs(keep - 0.75) < 0.01
    assert torch.allclose(d[d != 0], torch.full_like(d[d != 0], 1 / 0.75))
    d.sum().backward()
    assert torch.equal(x.grad != 0, d != 0)


# ------------------------------------------------------------------ optimizers
def test_fused_adam_and_sgd_match_reference_math():
    native = _native()
    torch.manual_seed(0)
    sizes = [1000, 33, 70000, 5]
    ps = [torch.randn(n, device="cuda") for n in sizes]
    gs = [torch.randn(n, device="cuda") for n in sizes]
    ms = [torch.zeros_like(p) for p in ps]
    vs = [torch.zeros_like(p) for p in ps]
    ref_p = [p.clone() for p in ps]
    ref_m = [torch.zeros_like(p) for p in ps]
    ref_v = [torch.zeros_like(p) for p in ps]
    lr, b1, b2, eps, wd = 1e-2, 0.9, 0.999, 1e-8, 0.1
    for step in range(1, 4):
        native.multi_tensor_adam(gs, ps, ms, vs, None, lr=lr, beta1=b1, beta2=b2, eps=eps,
                                 weight_decay=wd, step=step, adamw=True)
        for p, g, m, v in zip(ref_p, gs, ref_m, ref_v):
            m.mul_(b1).add_(g, alpha=1 - b1)
            v.mul_(b2).addcmul_(g, g, value=1 - b2)
            p.mul_(1 - lr * wd)
            p.sub_(lr * (m / (1 - b1 ** step)) / ((v / (1 - b2 ** step)).sqrt() + eps))
    for p, r in zip(ps, ref_p):
        assert torch.allclose(p, r, atol=1e-5, rtol=1e-5)
    # flat bf16 grads with fp32 master + bf16 model copy
    n = 100003
    master = torch.randn(n, device="cuda")
    model = master.bfloat16()
    g = torch.randn(n, device="cuda").bfloat16()
    m = torch.zeros(n, device="cuda"); v = torch.zeros(n, device="cuda")
    rp = master.clone()
    native.adam_flat(g, master, m, v, model, lr=lr, beta1=b1, beta2=b2, eps=eps, weight_decay=0.0,
                     step=1, adamw=False)
    gf = g.float()
    rm = (1 - b1) * gf; rv = (1 - b2) * gf * gf
    rp -= lr * (rm / (1 - b1)) / ((rv / (1 - b2)).sqrt() + eps)
    assert torch.allclose(master, rp, atol=1e-5)
    assert torch.equal(model, master.bfloat16())
    # SGD momentum
    p = torch.randn(5000, device="cuda"); g2 = torch.randn(5000, device="cuda")
    mom = torch.zeros_like(p); rp2 = p.clone(); rmom = torch.zeros_like(p)
    for _ in range(3):
        native.multi_tensor_sgd([g2], [p], [mom], None, lr=0.1, momentum=0.9, weight_decay=0.0)
        rmom.mul_(0.9).add_(g2); rp2.sub_(0.1 * rmom)
    assert torch.allclose(p, rp2, atol=1e-5)
    # global norm + clip coefficient + inf detection
    ts = [torch.randn(1000, device="cuda"), torch.randn(77777, device="cuda").bfloat16()]
    found = torch.zeros(1, dtype=torch.int32, device="cuda")
    norm, coef = native.global_norm(ts, max_norm=1.0, found_inf=found)
    ref = math.sqrt(sum(t.float().pow(2).sum().item() for t in ts))
    assert abs(norm.item() - ref) / ref < 1e-4
    assert abs(coef.item() - min(1.0, 1.0 / (ref + 1e-6))) < 1e-5
    assert found.item() == 0
    ts[0][5] = float("inf")
    native.global_norm(ts, max_norm=1.0, found_inf=found)
    assert found.item() == 1
