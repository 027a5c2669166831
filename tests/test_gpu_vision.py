"""Vision kernels (implicit-GEMM conv, BatchNorm, pools) against PyTorch fp32 references."""
import pytest
import torch
import torch.nn.functional as TF

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-3), (torch.float16, 1e-2)])
@pytest.mark.parametrize("cfg", [
    dict(B=2, Cin=16, Cout=32, H=14, W=14, k=3, s=1, p=1, d=1),
    dict(B=2, Cin=3, Cout=16, H=33, W=31, k=7, s=2, p=3, d=1),
    dict(B=3, Cin=32, Cout=64, H=8, W=8, k=1, s=1, p=0, d=1),
    dict(B=2, Cin=16, Cout=24, H=9, W=9, k=1, s=2, p=0, d=1),
    dict(B=1, Cin=8, Cout=8, H=12, W=12, k=3, s=2, p=2, d=2),
    dict(B=4, Cin=64, Cout=64, H=28, W=28, k=3, s=1, p=1, d=1),   # vector im2col / col2im, split-K wgrad
])
def test_conv2d_fwd_bwd(dtype, tol, cfg):
    from rumus_b200.ops import vision as V
    torch.manual_seed(0)
    x = torch.randn(cfg["B"], cfg["Cin"], cfg["H"], cfg["W"], device="cuda").to(dtype).requires_grad_(True)
    w = (torch.randn(cfg["Cout"], cfg["Cin"], cfg["k"], cfg["k"], device="cuda") * 0.2).to(dtype).requires_grad_(True)
    b = torch.randn(cfg["Cout"], device="cuda").to(dtype).requires_grad_(True)
    y = V.conv2d(x, w, b, cfg["s"], cfg["p"], cfg["d"])
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = TF.conv2d(xr, wr, br, cfg["s"], cfg["p"], cfg["d"])
    yr.backward(g.float())
    assert y.shape == yr.shape
    assert _rel(y, yr) < tol
    assert _rel(x.grad, xr.grad) < tol and _rel(w.grad, wr.grad) < tol and _rel(b.grad, br.grad) < tol


def test_conv_transpose2d():
    from rumus_b200.ops import vision as V
    torch.manual_seed(1)
    x = torch.randn(2, 8, 5, 6, device="cuda", requires_grad=True)
    w = (torch.randn(8, 4, 4, 4, device="cuda") * 0.2).requires_grad_(True)
    b = torch.randn(4, device="cuda", requires_grad=True)
    y = V.conv_transpose2d(x, w, b, 2, 1)
    g = torch.randn_like(y); y.backward(g)
    xr, wr, br = (t.detach().clone().requires_grad_(True) for t in (x, w, b))
    yr = TF.conv_transpose2d(xr, wr, br, 2, 1); yr.backward(g)
    assert _rel(y, yr) < 3e-3 and _rel(x.grad, xr.grad) < 3e-3 and _rel(w.grad, wr.grad) < 3e-3
    assert _rel(b.grad, br.grad) < 1e-4


@pytest.mark.parametrize("relu,use_res", [(False, False), (True, True)])
def test_batch_norm2d(relu, use_res):
    from rumus_b200.ops import vision as V
    torch.manual_seed(2)
    B, C, H, W = 4, 24, 7, 9
    x = torch.randn(B, C, H, W, device="cuda", requires_grad=True)
    res = torch.randn(B, C, H, W, device="cuda", requires_grad=True) if use_res else None
    w = (1 + 0.1 * torch.randn(C, device="cuda")).requires_grad_(True)
    b = (0.1 * torch.randn(C, device="cuda")).requires_grad_(True)
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    y = V.batch_norm2d(x, w, b, rm, rv, True, 0.1, 1e-5, relu=relu, residual=res)
    g = torch.randn_like(y); y.backward(g)
    xs = [t.detach().cpu().requires_grad_(True) for t in (x, w, b)]
    rc = res.detach().cpu().requires_grad_(True) if use_res else None
    rmc, rvc = torch.zeros(C), torch.ones(C)
    yr = V.batch_norm2d(xs[0], xs[1], xs[2], rmc, rvc, True, 0.1, 1e-5, relu=relu, residual=rc)
    yr.backward(g.cpu())
    assert _rel(y.cpu(), yr) < 1e-4
    assert _rel(x.grad.cpu(), xs[0].grad) < 1e-3
    assert _rel(w.grad.cpu(), xs[1].grad) < 1e-3 and _rel(b.grad.cpu(), xs[2].grad) < 1e-3
    assert _rel(rm.cpu(), rmc) < 1e-4 and _rel(rv.cpu(), rvc) < 1e-4
    if use_res:
        assert _rel(res.grad.cpu(), rc.grad) < 1e-4
    # eval mode uses the running statistics
    ye = V.batch_norm2d(x.detach(), w.detach(), b.detach(), rm, rv, False, 0.1, 1e-5)
    yer = V.batch_norm2d(xs[0].detach(), xs[1].detach(), xs[2].detach(), rmc, rvc, False, 0.1, 1e-5)
    assert _rel(ye.cpu(), yer) < 1e-4


@pytest.mark.parametrize("C,relu,use_res,shape", [
    (64, True, True, (6, 9, 11)), (256, False, False, (6, 9, 11)), (16, True, False, (6, 9, 11)),
    (64, True, True, (8, 100, 100)),      # long enough for the unrolled main loops of all three kernels
    (512, True, False, (4, 41, 40)),      # 32 channel groups per CTA, ragged row count
])
def test_batch_norm2d_half_vector_path(C, relu, use_res, shape):
    """fp16 channels-last batch norm with C % 8 == 0 (16-byte kernels) against the fp32 CPU form."""
    from rumus_b200.ops import vision as V
    torch.manual_seed(5)
    B, H, W = shape
    x32 = torch.randn(B, C, H, W)
    r32 = torch.randn(B, C, H, W) if use_res else None
    w32, b32 = 1 + 0.1 * torch.randn(C), 0.1 * torch.randn(C)
    g32 = torch.randn(B, C, H, W)
    cl = dict(memory_format=torch.channels_last)
    x = x32.cuda().half().contiguous(**cl).requires_grad_(True)
    res = r32.cuda().half().contiguous(**cl).requires_grad_(True) if use_res else None
    w = w32.cuda().half().requires_grad_(True)
    b = b32.cuda().half().requires_grad_(True)
    rm, rv = torch.zeros(C, device="cuda"), torch.ones(C, device="cuda")
    y = V.batch_norm2d(x, w, b, rm, rv, True, 0.1, 1e-5, relu=relu, residual=res)
    y.backward(g32.cuda().half().contiguous(**cl))
    xs = [t.detach().float().cpu().requires_grad_(True) for t in (x, w, b)]
    rc = res.detach().float().cpu().requires_grad_(True) if use_res else None
    yr = V.batch_norm2d(xs[0], xs[1], xs[2], torch.zeros(C), torch.ones(C), True, 0.1, 1e-5,
                        relu=relu, residual=rc)
    yr.backward(g32.half().float())
    assert _rel(y.float().cpu(), yr) < 3e-3
    assert _rel(x.grad.float().cpu(), xs[0].grad) < 1e-2
    assert _rel(w.grad.float().cpu(), xs[1].grad) < 1e-2 and _rel(b.grad.float().cpu(), xs[2].grad) < 1e-2
    if use_res:
        assert _rel(res.grad.float().cpu(), rc.grad) < 3e-3


def test_pools():
    from rumus_b200.ops import vision as V
    torch.manual_seed(3)
    x = torch.randn(2, 6, 13, 15, device="cuda", requires_grad=True)
    y = V.max_pool2d(x, 3, 2, 1)
    g = torch.randn_like(y); y.backward(g)
    xr = x.detach().clone().requires_grad_(True)
    yr = TF.max_pool2d(xr, 3, 2, 1); yr.backward(g)
    assert torch.allclose(y, yr) and torch.allclose(x.grad, xr.grad, atol=1e-6)
    x2 = torch.randn(2, 5, 7, 7, device="cuda", requires_grad=True)
    for out in [(1, 1), (3, 2)]:
        x2.grad = None
        y2 = V.adaptive_avg_pool2d(x2, out)
        g2 = torch.randn_like(y2); y2.backward(g2)
        x2r = x2.detach().clone().requires_grad_(True)
        y2r = TF.adaptive_avg_pool2d(x2r, out); y2r.backward(g2)
        assert torch.allclose(y2, y2r, atol=1e-5) and torch.allclose(x2.grad, x2r.grad, atol=1e-5)


def test_resnet_bottleneck_stack_trains_fp16():
    """Tiny ResNet (bottleneck blocks, BatchNorm) in fp16 with dynamic loss scaling and SGD."""
    from rumus_b200.models import ResNet50
    from rumus_b200.optim import SGD, GradScaler
    from rumus_b200.ops import functional as F
    torch.manual_seed(4)
    m = ResNet50(num_classes=10, layers=(1, 1, 1, 1), width=16, device="cuda", dtype=torch.float16)
    opt = SGD(m.parameters(), lr=0.05, momentum=0.9)
    scaler = GradScaler(init_scale=1024.0)
    x = torch.randn(8, 3, 64, 64, device="cuda").half()
    t = torch.randint(0, 10, (8,), device="cuda")
    losses = []
    for _ in range(12):
        opt.zero_grad()
        loss = F.cross_entropy_loss(m(x), t)
        scaler.scale(loss).backward()
        scaler.unscale_and_check(opt)
        opt.step()
        scaler.update()
        losses.append(loss.item())
    assert losses[-1] < losses[0], losses


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("cfg", [
    dict(B=4, Cin=64, Cout=64, H=28, W=28, k=3, s=1, p=1, d=1),      # 3x3, tiles of 4 x 4 pixels x 8 images
    dict(B=3, Cin=128, Cout=256, H=15, W=13, k=3, s=2, p=1, d=1),    # strided gather, ragged image, data grad in 4 phases
    dict(B=2, Cin=64, Cout=64, H=13, W=11, k=5, s=3, p=2, d=1),      # stride 3: 9 phases with 1..4 taps
    dict(B=2, Cin=256, Cout=128, H=14, W=14, k=1, s=2, p=0, d=1),    # strided 1x1 shortcut
    dict(B=5, Cin=64, Cout=192, H=9, W=20, k=3, s=1, p=2, d=2),      # dilation, Cout not a multiple of 128
    dict(B=2, Cin=192, Cout=64, H=7, W=7, k=5, s=1, p=2, d=1),       # 5x5 taps, three channel blocks
])
def test_conv2d_implicit_gemm(dtype, cfg):
    """Convolutions with 64-channel blocks take the implicit-GEMM kernels (no patch matrix): forward,
    data gradient (stride 1: mirrored gather; strided: one stride-1 gather per phase) and weight gradient
    against fp32."""
    from rumus_b200.ops import native
    from rumus_b200.ops import vision as V
    from rumus_b200.ops import vision_cuda as VC
    torch.manual_seed(1)
    assert VC._igemm_ok(torch.empty(1, device="cuda", dtype=dtype), cfg["Cin"], cfg["Cout"])
    x = torch.randn(cfg["B"], cfg["Cin"], cfg["H"], cfg["W"], device="cuda").to(dtype).requires_grad_(True)
    w = (torch.randn(cfg["Cout"], cfg["Cin"], cfg["k"], cfg["k"], device="cuda") * 0.05).to(dtype).requires_grad_(True)
    b = torch.randn(cfg["Cout"], device="cuda").to(dtype).requires_grad_(True)
    y = V.conv2d(x, w, b, cfg["s"], cfg["p"], cfg["d"])
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_(True) for t in (x, w, b))
    yr = TF.conv2d(xr, wr, br, cfg["s"], cfg["p"], cfg["d"])
    yr.backward(g.float())
    assert native.read_status() == 0
    assert y.shape == yr.shape
    assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2
    assert _rel(b.grad, br.grad) < 1e-2


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,W,bias", [(2, 64, 64, False), (3, 40, 56, True), (1, 224, 224, False), (5, 18, 8, True)])
def test_conv2d_direct_stem(dtype, B, H, W, bias):
    """The 3-channel 7x7 stride-2 stem takes the direct kernels (window in shared memory, tcgen05 product,
    weight gradient accumulated in TMEM): forward and weight / bias gradients against fp32."""
    from rumus_b200.ops import native
    from rumus_b200.ops import vision as V
    from rumus_b200.ops import vision_cuda as VC
    torch.manual_seed(2)
    x = torch.randn(B, 3, H, W, device="cuda").to(dtype)
    w = (torch.randn(64, 3, 7, 7, device="cuda") * 0.1).to(dtype).requires_grad_(True)
    b = torch.randn(64, device="cuda").to(dtype).requires_grad_(True) if bias else None
    assert VC._stem_ok(x, w, 2, 3, 1)
    y = V.conv2d(x, w, b, 2, 3, 1)
    g = torch.randn_like(y)
    y.backward(g)
    wr = w.detach().float().requires_grad_(True)
    br = b.detach().float().requires_grad_(True) if bias else None
    yr = TF.conv2d(x.float(), wr, br, 2, 3, 1)
    yr.backward(g.float())
    assert native.read_status() == 0
    assert y.shape == yr.shape
    assert _rel(y, yr) < 1e-2
    assert _rel(w.grad, wr.grad) < 1e-2
    if bias:
        assert _rel(b.grad, br.grad) < 1e-2
    # an image that needs a gradient keeps the general path
    xg = x.clone().requires_grad_(True)
    V.conv2d(xg, w, b, 2, 3, 1).backward(g)
    xr = x.float().requires_grad_(True)
    TF.conv2d(xr, wr.detach(), br.detach() if bias else None, 2, 3, 1).backward(g.float())
    assert _rel(xg.grad, xr.grad) < 1e-2


def test_pixel_tile_choice_covers_the_grid_with_128_pixels():
    from rumus_b200.ops.vision_cuda import _pixel_tile
    for B, Ho, Wo in ((256, 56, 56), (256, 28, 28), (256, 14, 14), (256, 7, 7), (3, 8, 7), (1, 1, 1)):
        tw, th, tn = _pixel_tile(B, Ho, Wo)
        assert tw * th * tn == 128
    assert _pixel_tile(256, 7, 7) == (1, 1, 128)        # no wasted rows on 7 x 7 images
    assert _pixel_tile(256, 56, 56)[2] <= 2
