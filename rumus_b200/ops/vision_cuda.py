"""CUDA paths of the vision ops: convolution (implicit GEMM: operand tiles gathered from the NHWC
tensor by TMA inside the tcgen05 GEMM, ``csrc/kernels/conv_igemm.cu``; im2col / col2im kernels around
the GEMM remain for the 3-channel stem, fp32 and strided data gradients), BatchNorm2d, max-pool,
adaptive average pool.  Activations are kept channels-last
(NHWC in memory, NCHW in shape) so 1x1 convolutions are plain GEMMs on the activation tensor and
BatchNorm reduces over contiguous channel vectors.  Kernels: ``csrc/kernels/vision.cu``."""
from __future__ import annotations

from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from . import native
from ._lib import check, count_launch, ptr, stream_ptr

P, LL, I, F = c_void_p, c_longlong, c_int, c_float
native.register_signature("rb_im2col_nhwc", [I, P, P] + [I] * 12 + [P])
native.register_signature("rb_col2im_nhwc", [I, P, P] + [I] * 12 + [P])
native.register_signature("rb_conv_igemm", [I, I, P, P, P, P, I] + [I] * 15 + [P])
native.register_signature("rb_conv_igemm_wgrad", [I, P, P, P] + [I] * 12 + [P])
native.register_signature("rb_conv_igemm_dgrad_phase", [I, P, P, P] + [I] * 17 + [P])
native.register_signature("rb_conv_stem_fwd", [I, P, P, P, P, I, I, I, P])
native.register_signature("rb_conv_stem_wgrad", [I, P, P, P, I, I, I, P])
native.register_signature("rb_bn_slabs", [LL])
native.register_signature("rb_bn_fwd", [I, P, P, P, P, P, P, P, P, P, P, LL, I, F, F, I, I, P])
native.register_signature("rb_bn_bwd", [I, P, P, P, P, P, P, P, P, P, P, P, P, LL, I, I, I, P])
native.register_signature("rb_maxpool_fwd", [I, P, P, P] + [I] * 9 + [P])
native.register_signature("rb_maxpool_bwd", [I, P, P, P] + [I] * 9 + [P])
native.register_signature("rb_adaptive_avgpool", [I, I, P, P] + [I] * 6 + [P])


def _nhwc(x: torch.Tensor) -> torch.Tensor:
    """[B,C,H,W] (any layout) -> contiguous [B,H,W,C] tensor sharing memory when already channels-last."""
    return x.permute(0, 2, 3, 1).contiguous()


def _as_nchw(y_nhwc: torch.Tensor) -> torch.Tensor:
    return y_nhwc.permute(0, 3, 1, 2)


def _out(n, k, s, p, d=1):
    return (n + 2 * p - d * (k - 1) - 1) // s + 1


def _pad8(k: int, esz: int) -> int:
    a = 16 // esz
    return (k + a - 1) // a * a


def _im2col(xh, KH, KW, Ho, Wo, stride, pad, dil, Kpad):
    B, H, W, C = xh.shape
    cols = torch.empty((B * Ho * Wo, Kpad), dtype=xh.dtype, device=xh.device)
    check(native.lib().rb_im2col_nhwc(native.dtype_code(xh.dtype), ptr(xh), ptr(cols), B, H, W, C, KH,
                                      KW, Ho, Wo, stride, pad, dil, Kpad, stream_ptr()), "rb_im2col_nhwc")
    count_launch()
    return cols


def _col2im(dcols, B, H, W, C, KH, KW, Ho, Wo, stride, pad, dil, Kpad):
    dx = torch.empty((B, H, W, C), dtype=dcols.dtype, device=dcols.device)
    check(native.lib().rb_col2im_nhwc(native.dtype_code(dcols.dtype), ptr(dcols), ptr(dx), B, H, W, C,
                                      KH, KW, Ho, Wo, stride, pad, dil, Kpad, stream_ptr()), "rb_col2im_nhwc")
    count_launch()
    return dx


def _weight_matrix(weight, Kpad):
    """[Cout, Cin, KH, KW] -> [Cout, Kpad] with K ordered (kh, kw, c) to match NHWC patches."""
    Cout, Cin, KH, KW = weight.shape
    wm = weight.permute(0, 2, 3, 1).reshape(Cout, KH * KW * Cin)
    if Kpad != wm.shape[1]:
        wm = torch.nn.functional.pad(wm, (0, Kpad - wm.shape[1]))
    return wm.contiguous()


def _igemm_ok(x: torch.Tensor, cin: int, cout: int) -> bool:
    """The implicit-GEMM kernels (``csrc/kernels/conv_igemm.cu``) gather 64-channel blocks of a 16-bit
    NHWC tensor; other convolutions (the 3-channel stem, fp32) keep the im2col path."""
    import os
    return (x.dtype in (torch.bfloat16, torch.float16) and cin % 64 == 0 and cout % 8 == 0
            and os.environ.get("RB_CONV_IGEMM", "1") == "1")


def _stem_ok(x: torch.Tensor, weight: torch.Tensor, stride: int, padding: int, dilation: int) -> bool:
    """The direct stem kernels (``csrc/kernels/conv_stem.cu``) cover one layer shape: 3 input channels,
    7x7 taps, stride 2, padding 3, 64 output channels, 16-bit, image width a multiple of 8."""
    import os
    return (x.dtype in (torch.bfloat16, torch.float16) and tuple(weight.shape) == (64, 3, 7, 7)
            and stride == 2 and padding == 3 and dilation == 1 and x.shape[3] % 8 == 0
            and os.environ.get("RB_CONV_STEM", "1") == "1")


STEM_K = 192      # K of the stem's weight matrix: kh*24 + 1 + kw*3 + ci, zero elsewhere


def _stem_weight_matrix(weight: torch.Tensor) -> torch.Tensor:
    """[64, 3, 7, 7] -> [64, 192]: per tap row 24 slots = one zero, the 7 taps x 3 channels, two zeros."""
    w = weight.permute(0, 2, 3, 1).reshape(64, 7, 21)
    w = torch.nn.functional.pad(w, (1, 2)).reshape(64, 168)
    return torch.nn.functional.pad(w, (0, STEM_K - 168)).contiguous()


def conv_stem(xh: torch.Tensor, wk: torch.Tensor, bias=None) -> torch.Tensor:
    """x NHWC ``[B, H, W, 3]`` -> NHWC ``[B, H/2, W/2, 64]`` (7x7, stride 2, padding 3)."""
    B, H, W, _ = xh.shape
    Ho, Wo = _out(H, 7, 2, 3), _out(W, 7, 2, 3)
    y = torch.empty((B, Ho, Wo, 64), dtype=xh.dtype, device=xh.device)
    check(native.lib().rb_conv_stem_fwd(native.dtype_code(xh.dtype), ptr(xh), ptr(wk), ptr(bias), ptr(y), B, H, W,
                                        stream_ptr()), "rb_conv_stem_fwd")
    count_launch()
    return y


def conv_stem_wgrad(xh: torch.Tensor, dyh: torch.Tensor) -> torch.Tensor:
    """x NHWC ``[B, H, W, 3]``, dY NHWC ``[B, Ho, Wo, 64]`` -> weight gradient ``[64, 3, 7, 7]`` in fp32."""
    B, H, W, _ = xh.shape
    dwk = torch.zeros((STEM_K, 64), dtype=torch.float32, device=xh.device)
    check(native.lib().rb_conv_stem_wgrad(native.dtype_code(xh.dtype), ptr(xh), ptr(dyh), ptr(dwk), B, H, W,
                                          stream_ptr()), "rb_conv_stem_wgrad")
    count_launch()
    return dwk[:168].view(7, 24, 64)[:, 1:22].reshape(7, 7, 3, 64).permute(3, 2, 0, 1)


def _pixel_tile(B: int, Ho: int, Wo: int):
    """(tw, th, tn): the patch of 128 output pixels (tw x th pixels of tn images, powers of two) that
    wastes the fewest rows on the edges of the ``B x Ho x Wo`` grid; ties go to the larger patch."""
    best = None
    for lw in range(8):
        for lh in range(8 - lw):
            tw, th, tn = 1 << lw, 1 << lh, 1 << (7 - lw - lh)
            cover = (-(-Wo // tw) * tw) * (-(-Ho // th) * th) * (-(-B // tn) * tn)
            key = (cover, -(tw * th), abs(lw - lh))
            if best is None or key < best[0]:
                best = (key, (tw, th, tn))
    return best[1]


def conv_igemm(mode: int, act: torch.Tensor, wmat: torch.Tensor, Ho: int, Wo: int, KH: int, KW: int,
               stride: int, pad: int, dil: int, bias=None, relu: bool = False) -> torch.Tensor:
    """``act`` NHWC ``[B, H, W, C]``, ``wmat [N, KH*KW*C]`` -> NHWC ``[B, Ho, Wo, N]``; mode 0 forward,
    mode 1 data gradient of a stride-1 convolution (``act`` = dY, taps mirrored)."""
    B, H, W, C = act.shape
    N = wmat.shape[0]
    out = torch.empty((B, Ho, Wo, N), dtype=act.dtype, device=act.device)
    tw, th, tn = _pixel_tile(B, Ho, Wo)
    check(native.lib().rb_conv_igemm(mode, native.dtype_code(act.dtype), ptr(act), ptr(wmat), ptr(out), ptr(bias),
                                     1 if relu else 0, B, H, W, C, Ho, Wo, N, KH, KW, stride, pad, dil, tw, th, tn,
                                     stream_ptr()), "rb_conv_igemm")
    count_launch()
    return out


def conv_igemm_dgrad_strided(dy4: torch.Tensor, wm: torch.Tensor, H: int, W: int, Cin: int, KH: int, KW: int,
                             stride: int, pad: int) -> torch.Tensor:
    """Data gradient of a convolution with stride > 1 (dilation 1) without a patch matrix: the input
    pixels split into stride x stride phases by ``(ih + pad) % stride, (iw + pad) % stride``; a phase
    only ever meets the taps ``kh = phase + stride * a``, so it is a stride-1 gather over dY with those
    taps, written to every stride-th input pixel.  dY NHWC ``[B, Ho, Wo, Cout]``, ``wm [Cout, KH*KW*Cin]``
    (K ordered kh, kw, ci) -> dx NHWC ``[B, H, W, Cin]``."""
    B, Ho, Wo, Cout = dy4.shape
    s = stride
    w4 = wm.view(Cout, KH, KW, Cin)
    every_phase_has_taps = KH >= s and KW >= s
    dx = (torch.empty if every_phase_has_taps else torch.zeros)((B, H, W, Cin), dtype=dy4.dtype, device=dy4.device)
    L = native.lib()
    for rh in range(min(s, KH)):
        for rw in range(min(s, KW)):
            e_h, e_w = (rh - pad) % s, (rw - pad) % s
            if e_h >= H or e_w >= W:
                continue
            c_h, c_w = (e_h + pad - rh) // s, (e_w + pad - rw) // s
            taps = w4[:, rh::s, rw::s, :]                                   # [Cout, KHp, KWp, Cin]
            KHp, KWp = taps.shape[1], taps.shape[2]
            wphase = taps.permute(3, 1, 2, 0).reshape(Cin, KHp * KWp * Cout).contiguous()
            Hu, Wu = -(-(H - e_h) // s), -(-(W - e_w) // s)
            tw, th, tn = _pixel_tile(B, Hu, Wu)
            check(L.rb_conv_igemm_dgrad_phase(native.dtype_code(dy4.dtype), ptr(dy4), ptr(wphase), ptr(dx), B, Ho, Wo,
                                              Cout, H, W, Cin, KHp, KWp, s, c_h, c_w, e_h, e_w, tw, th, tn,
                                              stream_ptr()), "rb_conv_igemm_dgrad_phase")
            count_launch()
    return dx


def conv_igemm_wgrad(dyh: torch.Tensor, xh: torch.Tensor, KH: int, KW: int, stride: int, pad: int, dil: int) -> torch.Tensor:
    """dY NHWC ``[B, Ho, Wo, Cout]``, x NHWC ``[B, H, W, C]`` -> fp32 ``[Cout, KH*KW*C]`` (K ordered kh, kw, c)."""
    B, Ho, Wo, Cout = dyh.shape
    _, H, W, C = xh.shape
    dwm = torch.zeros((Cout, KH * KW * C), dtype=torch.float32, device=xh.device)
    check(native.lib().rb_conv_igemm_wgrad(native.dtype_code(xh.dtype), ptr(dyh), ptr(xh), ptr(dwm), B, H, W, C, Ho, Wo,
                                           Cout, KH, KW, stride, pad, dil, stream_ptr()), "rb_conv_igemm_wgrad")
    count_launch()
    return dwm


class Conv2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding, dilation):
        B, Cin, H, W = x.shape
        Cout, _, KH, KW = weight.shape
        Ho, Wo = _out(H, KH, stride, padding, dilation), _out(W, KW, stride, padding, dilation)
        xh = _nhwc(x)
        esz = x.element_size()
        pointwise = KH == 1 and KW == 1 and stride == 1 and padding == 0 and Cin % (16 // esz) == 0
        if not ctx.needs_input_grad[0] and _stem_ok(x, weight, stride, padding, dilation):
            # the image needs no gradient: direct kernels, no patch matrix
            wk = _stem_weight_matrix(weight)
            b = bias.to(x.dtype).contiguous() if bias is not None else None
            y = conv_stem(xh, wk, b)
            ctx.stem = True
            ctx.geom = (B, H, W, Cin, Cout, KH, KW, Ho, Wo, stride, padding, dilation, 0, False)
            ctx.save_for_backward(xh, wk)
            ctx.has_bias = bias is not None
            ctx.w_dtype = weight.dtype
            return _as_nchw(y)
        ctx.stem = False
        igemm = not pointwise and _igemm_ok(x, Cin, Cout)
        Kpad = Cin if pointwise else (KH * KW * Cin if igemm else _pad8(KH * KW * Cin, esz))
        wm = _weight_matrix(weight, Kpad)
        if igemm:
            # operand tiles come straight out of the NHWC tensor: no patch matrix is written
            y = conv_igemm(0, xh, wm, Ho, Wo, KH, KW, stride, padding, dilation, bias=bias)
        else:
            cols = xh.view(B * H * W, Cin) if pointwise else _im2col(xh, KH, KW, Ho, Wo, stride, padding,
                                                                     dilation, Kpad)
            y = native.gemm(cols, wm.t(), bias=bias)      # [M, Cout] == NHWC output
        ctx.igemm = igemm
        ctx.geom = (B, H, W, Cin, Cout, KH, KW, Ho, Wo, stride, padding, dilation, Kpad, pointwise)
        ctx.save_for_backward(xh, wm)
        ctx.has_bias = bias is not None
        ctx.w_dtype = weight.dtype
        return _as_nchw(y.view(B, Ho, Wo, Cout))

    @staticmethod
    def backward(ctx, dy):
        xh, wm = ctx.saved_tensors
        B, H, W, Cin, Cout, KH, KW, Ho, Wo, stride, padding, dilation, Kpad, pointwise = ctx.geom
        dyh = _nhwc(dy).view(B * Ho * Wo, Cout)
        dx = dw = db = None
        if ctx.stem:
            if ctx.needs_input_grad[1]:
                dw = conv_stem_wgrad(xh, dyh.view(B, Ho, Wo, Cout)).to(ctx.w_dtype).contiguous()
            if ctx.has_bias and ctx.needs_input_grad[2]:
                db = native.colsum(dyh)
            return dx, dw, db, None, None, None
        if ctx.igemm:
            dy4 = dyh.view(B, Ho, Wo, Cout)
            if ctx.needs_input_grad[1]:
                dwm = conv_igemm_wgrad(dy4, xh, KH, KW, stride, padding, dilation)
                dw = dwm.view(Cout, KH, KW, Cin).permute(0, 3, 1, 2).to(ctx.w_dtype).contiguous()
            if ctx.needs_input_grad[0]:
                if stride == 1 and Cout % 64 == 0:
                    # data gradient = the same gather on dY with mirrored taps; weight as [Cin, (kh, kw, co)]
                    wd = wm.view(Cout, KH, KW, Cin).permute(3, 1, 2, 0).reshape(Cin, KH * KW * Cout).contiguous()
                    dx = _as_nchw(conv_igemm(1, dy4, wd, H, W, KH, KW, 1, padding, dilation))
                elif stride > 1 and dilation == 1 and Cout % 64 == 0:
                    dx = _as_nchw(conv_igemm_dgrad_strided(dy4, wm, H, W, Cin, KH, KW, stride, padding))
                else:
                    dcols = native.gemm(dyh, wm)           # [M, K]: strided data gradients scatter through col2im
                    dx = _as_nchw(_col2im(dcols, B, H, W, Cin, KH, KW, Ho, Wo, stride, padding, dilation, Kpad))
            if ctx.has_bias and ctx.needs_input_grad[2]:
                db = native.colsum(dyh)
            return dx, dw, db, None, None, None
        cols = xh.view(B * H * W, Cin) if pointwise else _im2col(xh, KH, KW, Ho, Wo, stride, padding,
                                                                 dilation, Kpad)
        if ctx.needs_input_grad[1]:
            dwm = native.gemm(dyh.t(), cols)               # [Cout, Kpad]
            dw = dwm[:, :KH * KW * Cin].reshape(Cout, KH, KW, Cin).permute(0, 3, 1, 2).contiguous()
        if ctx.needs_input_grad[0]:
            dcols = native.gemm(dyh, wm)                   # [M, Kpad]
            if pointwise:
                dx = _as_nchw(dcols.view(B, H, W, Cin))
            else:
                dx = _as_nchw(_col2im(dcols, B, H, W, Cin, KH, KW, Ho, Wo, stride, padding, dilation, Kpad))
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = native.colsum(dyh)
        return dx, dw, db, None, None, None


class _ConvTranspose2dFn(torch.autograd.Function):
    """y = col2im(x[M, Cin] @ W[Cin, Cout*K*K]) — the data-gradient path of a convolution."""

    @staticmethod
    def forward(ctx, x, weight, bias, stride, padding):
        B, Cin, H, W = x.shape
        _, Cout, KH, KW = weight.shape
        Ho = (H - 1) * stride - 2 * padding + KH
        Wo = (W - 1) * stride - 2 * padding + KW
        esz = x.element_size()
        Kpad = _pad8(KH * KW * Cout, esz)
        xh = _nhwc(x).view(B * H * W, Cin)
        wm = weight.permute(0, 2, 3, 1).reshape(Cin, KH * KW * Cout)    # [Cin, (kh,kw,co)]
        if Kpad != wm.shape[1]:
            wm = torch.nn.functional.pad(wm, (0, Kpad - wm.shape[1]))
        wm = wm.contiguous()
        cols = native.gemm(xh, wm)                                       # [M, Kpad]
        yh = _col2im(cols, B, Ho, Wo, Cout, KH, KW, H, W, stride, padding, 1, Kpad)
        if bias is not None:
            yh = yh + bias
        ctx.geom = (B, H, W, Cin, Cout, KH, KW, Ho, Wo, stride, padding, Kpad)
        ctx.has_bias = bias is not None
        ctx.save_for_backward(xh, wm)
        return _as_nchw(yh)

    @staticmethod
    def backward(ctx, dy):
        xh, wm = ctx.saved_tensors
        B, H, W, Cin, Cout, KH, KW, Ho, Wo, stride, padding, Kpad = ctx.geom
        dyh = _nhwc(dy)
        dcols = _im2col(dyh, KH, KW, H, W, stride, padding, 1, Kpad)     # [B*H*W, Kpad]
        dx = native.gemm(dcols, wm.t()).view(B, H, W, Cin)
        dwm = native.gemm(xh.t(), dcols)                                 # [Cin, Kpad]
        dw = dwm[:, :KH * KW * Cout].reshape(Cin, KH, KW, Cout).permute(0, 3, 1, 2).contiguous()
        db = native.colsum(dyh.view(-1, Cout)) if ctx.has_bias else None
        return _as_nchw(dx), dw, db, None, None


def conv_transpose2d_cuda(x, weight, bias, stride, padding):
    return _ConvTranspose2dFn.apply(x, weight, bias, stride, padding)


class MaxPool2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, stride, pad):
        B, C, H, W = x.shape
        Ho, Wo = _out(H, k, stride, pad), _out(W, k, stride, pad)
        xh = _nhwc(x)
        y = torch.empty((B, Ho, Wo, C), dtype=x.dtype, device=x.device)
        idx = torch.empty((B, Ho, Wo, C), dtype=torch.int8, device=x.device)
        check(native.lib().rb_maxpool_fwd(native.dtype_code(x.dtype), ptr(xh), ptr(y), ptr(idx), B, H, W,
                                          C, k, stride, pad, Ho, Wo, stream_ptr()), "rb_maxpool_fwd")
        count_launch()
        ctx.geom = (B, H, W, C, k, stride, pad, Ho, Wo)
        ctx.save_for_backward(idx)
        return _as_nchw(y)

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        B, H, W, C, k, stride, pad, Ho, Wo = ctx.geom
        dyh = _nhwc(dy)
        dx = torch.empty((B, H, W, C), dtype=dy.dtype, device=dy.device)
        check(native.lib().rb_maxpool_bwd(native.dtype_code(dy.dtype), ptr(dyh), ptr(idx), ptr(dx), B, H,
                                          W, C, k, stride, pad, Ho, Wo, stream_ptr()), "rb_maxpool_bwd")
        count_launch()
        return _as_nchw(dx), None, None, None


class AdaptiveAvgPool2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, out_size):
        B, C, H, W = x.shape
        Ho, Wo = out_size
        xh = _nhwc(x)
        y = torch.empty((B, Ho, Wo, C), dtype=x.dtype, device=x.device)
        check(native.lib().rb_adaptive_avgpool(native.dtype_code(x.dtype), 0, ptr(xh), ptr(y), B, H, W, C,
                                               Ho, Wo, stream_ptr()), "rb_adaptive_avgpool")
        count_launch()
        ctx.geom = (B, H, W, C, Ho, Wo)
        return _as_nchw(y)

    @staticmethod
    def backward(ctx, dy):
        B, H, W, C, Ho, Wo = ctx.geom
        dyh = _nhwc(dy)
        dx = torch.empty((B, H, W, C), dtype=dy.dtype, device=dy.device)
        check(native.lib().rb_adaptive_avgpool(native.dtype_code(dy.dtype), 1, ptr(dyh), ptr(dx), B, H, W,
                                               C, Ho, Wo, stream_ptr()), "rb_adaptive_avgpool")
        count_launch()
        return _as_nchw(dx), None


class BatchNorm2dFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, running_mean, running_var, training, momentum, eps, relu,
                residual):
        B, C, H, W = x.shape
        M = B * H * W
        xh = _nhwc(x)
        rh = _nhwc(residual) if residual is not None else None
        y = torch.empty_like(xh)
        L = native.lib()
        slabs = L.rb_bn_slabs(M)
        scratch = torch.empty((slabs, 2, C), dtype=torch.float32, device=x.device)
        if training:
            mean = torch.empty(C, dtype=torch.float32, device=x.device)
            rstd = torch.empty(C, dtype=torch.float32, device=x.device)
        else:
            mean = running_mean.float().contiguous()
            rstd = torch.rsqrt(running_var.float() + eps)
        w = weight.to(x.dtype).contiguous()
        b = bias.to(x.dtype).contiguous()
        check(L.rb_bn_fwd(native.dtype_code(x.dtype), ptr(xh), ptr(rh), ptr(w), ptr(b), ptr(y), ptr(mean),
                          ptr(rstd), ptr(running_mean) if training else None,
                          ptr(running_var) if training else None, ptr(scratch), M, C, float(eps),
                          float(momentum), 1 if relu else 0, 1 if training else 0, stream_ptr()),
              "rb_bn_fwd")
        count_launch(3 if training else 1)
        ctx.geom = (B, C, H, W, relu, training)
        ctx.has_res = residual is not None
        ctx.param_dtype = weight.dtype
        ctx.save_for_backward(xh, y, w, mean, rstd)
        return _as_nchw(y)

    @staticmethod
    def backward(ctx, dy):
        xh, y, w, mean, rstd = ctx.saved_tensors
        B, C, H, W, relu, training = ctx.geom
        M = B * H * W
        dyh = _nhwc(dy)
        L = native.lib()
        dx = torch.empty_like(xh)
        dres = torch.empty_like(xh) if ctx.has_res else None
        dg = torch.empty(C, dtype=xh.dtype, device=xh.device)
        db = torch.empty(C, dtype=xh.dtype, device=xh.device)
        sums = torch.empty(2 * C, dtype=torch.float32, device=xh.device)
        slabs = L.rb_bn_slabs(M)
        scratch = torch.empty((slabs, 2, C), dtype=torch.float32, device=xh.device)
        check(L.rb_bn_bwd(native.dtype_code(xh.dtype), ptr(xh), ptr(dyh), ptr(y), ptr(w), ptr(mean),
                          ptr(rstd), ptr(dx), ptr(dres), ptr(dg), ptr(db), ptr(sums), ptr(scratch), M, C,
                          1 if relu else 0, 1 if training else 0, stream_ptr()), "rb_bn_bwd")
        count_launch(3)
        return (_as_nchw(dx), dg.to(ctx.param_dtype), db.to(ctx.param_dtype), None, None, None, None,
                None, None, _as_nchw(dres) if dres is not None else None)
