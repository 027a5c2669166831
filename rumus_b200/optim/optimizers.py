"""Optimizers, gradient clipping, LR schedulers, loss scaling.

API follows the reference's ``Optimizer`` trait (rumus/src/optim/mod.rs:24-49:
``step / zero_grad / set_lr / get_lr``) with gradients read from ``param.grad``.
On CUDA, one fused multi-tensor launch updates every parameter (fp32 master
weights + moments; a bf16/fp16 model copy is refreshed in the same pass when the
parameter itself is low precision).  On CPU the same math runs in PyTorch.
"""
from __future__ import annotations

import math
from typing import Iterable, List, Optional

import torch

from ..ops import native
from ..ops._lib import check, ptr, stream_ptr


class Optimizer:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float):
        self.params: List[torch.nn.Parameter] = [p for p in params]
        self.lr = lr
        self.step_count = 0
        # fp32 master copies for low-precision parameters
        self.master = {}
        # device-side knobs shared with GradScaler / clip_grad_norm_
        self.grad_scale: Optional[torch.Tensor] = None   # multiplied into every gradient
        self.skip_flag: Optional[torch.Tensor] = None    # int32: non-zero -> step is a no-op

    # --- reference trait surface -------------------------------------------------------------
    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params:
            if p.grad is not None:
                if set_to_none:
                    p.grad = None
                else:
                    p.grad.zero_()

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def get_lr(self) -> float:
        return self.lr

    def step(self) -> None:  # pragma: no cover - abstract
        raise NotImplementedError

    # --- helpers -------------------------------------------------------------------------------
    def _master_of(self, p: torch.nn.Parameter) -> torch.Tensor:
        if p.dtype == torch.float32:
            return p.data
        m = self.master.get(p)
        if m is None:
            m = p.data.float()
            self.master[p] = m
        return m

    def _active(self):
        return [p for p in self.params if p.grad is not None]

    def state_dict(self) -> dict:
        return {"lr": self.lr, "step_count": self.step_count}

    def load_state_dict(self, sd: dict) -> None:
        self.lr = sd["lr"]
        self.step_count = sd["step_count"]


class SGD(Optimizer):
    """``v = mu*v + g; p -= lr*v`` (rumus/src/optim/sgd.rs:14-129, shaders/optim.wgsl:23)."""

    def __init__(self, params, lr: float, momentum: float = 0.0, weight_decay: float = 0.0):
        super().__init__(params, lr)
        self.momentum, self.weight_decay = momentum, weight_decay
        self.velocity = {}

    def step(self) -> None:
        self.step_count += 1
        act = self._active()
        if not act:
            return
        for p in act:
            if self.momentum != 0.0 and p not in self.velocity:
                self.velocity[p] = torch.zeros_like(p.data, dtype=torch.float32)
        if act[0].is_cuda:
            for dt in {p.grad.dtype for p in act}:
                grp = [p for p in act if p.grad.dtype == dt]
                native.multi_tensor_sgd(
                    [p.grad.contiguous() for p in grp], [self._master_of(p) for p in grp],
                    [self.velocity.get(p) for p in grp] if self.momentum != 0.0 else None,
                    [p.data if p.dtype != torch.float32 else None for p in grp],
                    lr=self.lr, momentum=self.momentum, weight_decay=self.weight_decay,
                    grad_scale=self.grad_scale, skip=self.skip_flag)
            return
        if self.skip_flag is not None and int(self.skip_flag.item()) != 0:
            return
        gs = float(self.grad_scale.item()) if self.grad_scale is not None else 1.0
        # CPU tensors: multi-tensor form of the same update
        gr = [p.grad if (p.grad.dtype == torch.float32 and gs == 1.0) else p.grad.float() * gs for p in act]
        ws = [self._master_of(p) for p in act]
        if self.weight_decay:
            gr = torch._foreach_add(gr, ws, alpha=self.weight_decay)
        if self.momentum != 0.0:
            vs = [self.velocity[p] for p in act]
            torch._foreach_mul_(vs, self.momentum)
            torch._foreach_add_(vs, gr)
            gr = vs
        torch._foreach_add_(ws, gr, alpha=-self.lr)
        for p, w in zip(act, ws):
            if p.dtype != torch.float32:
                p.data.copy_(w)

    def state_dict(self):
        sd = super().state_dict()
        sd["velocity"] = [self.velocity.get(p) for p in self.params]
        sd["master"] = [self.master.get(p) for p in self.params]
        return sd

    def load_state_dict(self, sd):
        super().load_state_dict(sd)
        for p, v in zip(self.params, sd.get("velocity", [])):
            if v is not None:
                self.velocity[p] = v.to(p.device)
        for p, w in zip(self.params, sd.get("master", [])):
            if w is not None:
                self.master[p] = w.to(p.device)


class Adam(Optimizer):
    """Adam with bias correction (rumus/src/optim/adam.rs:14-163, shaders/optim.wgsl:53):
    ``p -= lr * (m/bc1) / (sqrt(v/bc2) + eps)``."""

    _decoupled = False

    def __init__(self, params, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999,
                 epsilon: float = 1e-8, weight_decay: float = 0.0):
        super().__init__(params, lr)
        if weight_decay and not self._decoupled:
            # the reference's Adam has no weight decay (rumus/src/optim/adam.rs:14-40); an L2 term
            # silently dropped would be worse than an error
            raise ValueError("Adam takes no weight_decay; use AdamW for decoupled weight decay")
        self.beta1, self.beta2, self.epsilon, self.weight_decay = beta1, beta2, epsilon, weight_decay
        self.first_moment, self.second_moment = {}, {}
        # set when the last step ran on the device under a skip flag whose value the host has not
        # seen: GradScaler.update() takes the step count back if that step turned out to be skipped
        self._device_skip_pending = False

    def step(self) -> None:
        act = self._active()
        if not act:
            return
        self.step_count += 1
        t = self.step_count
        for p in act:
            if p not in self.first_moment:
                self.first_moment[p] = torch.zeros_like(p.data, dtype=torch.float32)
                self.second_moment[p] = torch.zeros_like(p.data, dtype=torch.float32)
        if act[0].is_cuda:
            for dt in {p.grad.dtype for p in act}:
                grp = [p for p in act if p.grad.dtype == dt]
                native.multi_tensor_adam(
                    [p.grad.contiguous() for p in grp], [self._master_of(p) for p in grp],
                    [self.first_moment[p] for p in grp], [self.second_moment[p] for p in grp],
                    [p.data if p.dtype != torch.float32 else None for p in grp],
                    lr=self.lr, beta1=self.beta1, beta2=self.beta2, eps=self.epsilon,
                    weight_decay=self.weight_decay, step=t, adamw=self._decoupled,
                    grad_scale=self.grad_scale, skip=self.skip_flag)
            self._device_skip_pending = self.skip_flag is not None
            return
        if self.skip_flag is not None and int(self.skip_flag.item()) != 0:
            self.step_count -= 1
            return
        gs = float(self.grad_scale.item()) if self.grad_scale is not None else 1.0
        bc1, bc2 = 1.0 - self.beta1 ** t, 1.0 - self.beta2 ** t
        # CPU tensors: the same update over all parameters at once (multi-tensor ops; one Python
        # call per operation instead of one per operation and parameter)
        gr = [p.grad if (p.grad.dtype == torch.float32 and gs == 1.0) else p.grad.float() * gs for p in act]
        ms = [self.first_moment[p] for p in act]
        vs = [self.second_moment[p] for p in act]
        ws = [self._master_of(p) for p in act]
        torch._foreach_mul_(ms, self.beta1)
        torch._foreach_add_(ms, gr, alpha=1 - self.beta1)
        torch._foreach_mul_(vs, self.beta2)
        torch._foreach_addcmul_(vs, gr, gr, value=1 - self.beta2)
        if self._decoupled:
            torch._foreach_mul_(ws, 1 - self.lr * self.weight_decay)
        den = torch._foreach_div(vs, bc2)
        torch._foreach_sqrt_(den)
        torch._foreach_add_(den, self.epsilon)
        torch._foreach_addcdiv_(ws, ms, den, value=-self.lr / bc1)     # w -= lr * (m / bc1) / den
        for p, w in zip(act, ws):
            if p.dtype != torch.float32:
                p.data.copy_(w)

    def state_dict(self):
        sd = super().state_dict()
        sd["m"] = [self.first_moment.get(p) for p in self.params]
        sd["v"] = [self.second_moment.get(p) for p in self.params]
        sd["master"] = [self.master.get(p) for p in self.params]
        return sd

    def load_state_dict(self, sd):
        super().load_state_dict(sd)
        for p, m, v, w in zip(self.params, sd["m"], sd["v"], sd.get("master", [None] * len(self.params))):
            if m is not None:
                self.first_moment[p] = m.to(p.device)
                self.second_moment[p] = v.to(p.device)
            if w is not None:
                self.master[p] = w.to(p.device)


class AdamW(Adam):
    """Decoupled weight decay applied before the Adam step
    (rumus/src/optim/adamw.rs:15-192, shaders/adamw.wgsl:26)."""

    _decoupled = True

    def __init__(self, params, lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999,
                 epsilon: float = 1e-8, weight_decay: float = 0.01):
        super().__init__(params, lr, beta1, beta2, epsilon, weight_decay)


def clip_grad_norm_(params: Iterable[torch.nn.Parameter], max_norm: float) -> torch.Tensor:
    """Scales gradients so their global L2 norm is at most ``max_norm``; returns the unclipped norm
    (rumus/src/optim/clip.rs:32-190).  On CUDA: per-tensor partial sums, one finalize kernel that
    also produces the clip coefficient on the device, one in-place scale per tensor — no host
    round-trip."""
    assert max_norm > 0
    params = [p for p in params if p.grad is not None]
    for p in params:
        if not p.grad.is_contiguous():
            p.grad = p.grad.contiguous()       # scaled in place below: must be the tensor the optimizer reads
    grads = [p.grad for p in params]
    if not grads:
        return torch.zeros(())
    if grads[0].is_cuda:
        norm, coef = native.global_norm(grads, max_norm=max_norm)
        for g in grads:
            native.scale_check_(g, scale_tensor=coef)
        return norm
    total = math.sqrt(sum(float(g.float().pow(2).sum()) for g in grads))
    if total > max_norm:
        s = max_norm / (total + 1e-6)
        for g in grads:
            g.mul_(s)
    return torch.tensor(total)


class LRScheduler:
    """rumus/src/optim/scheduler.rs:9-18 — schedulers only compute the LR; the caller applies it
    with ``optimizer.set_lr(scheduler.get_lr())``."""

    def step(self) -> None:
        raise NotImplementedError

    def get_lr(self) -> float:
        return self.current_lr

    def state_dict(self):
        return dict(self.__dict__)

    def load_state_dict(self, sd):
        self.__dict__.update(sd)


class StepLR(LRScheduler):
    """``lr *= gamma`` every ``step_size`` epochs (scheduler.rs:22-60)."""

    def __init__(self, initial_lr: float, step_size: int, gamma: float):
        assert step_size > 0
        self.initial_lr, self.step_size, self.gamma = initial_lr, step_size, gamma
        self.current_epoch, self.current_lr = 0, initial_lr

    def step(self):
        self.current_epoch += 1
        if self.current_epoch % self.step_size == 0:
            self.current_lr *= self.gamma

    def set_initial_lr(self, lr: float):
        self.initial_lr = lr
        self.current_lr = lr * self.gamma ** (self.current_epoch // self.step_size)


class CosineAnnealingLR(LRScheduler):
    """``eta_min + 0.5 (lr0 - eta_min)(1 + cos(pi t / t_max))``, clamped at ``eta_min`` after
    ``t_max`` (scheduler.rs:62-124)."""

    def __init__(self, initial_lr: float, t_max: int, eta_min: float = 0.0):
        assert t_max > 0
        self.initial_lr, self.t_max, self.eta_min = initial_lr, t_max, eta_min
        self.current_epoch, self.current_lr = 0, initial_lr

    def _lr(self, base):
        if self.current_epoch >= self.t_max:
            return self.eta_min
        return self.eta_min + 0.5 * (base - self.eta_min) * (
            1.0 + math.cos(math.pi * self.current_epoch / self.t_max))

    def step(self):
        self.current_epoch += 1
        self.current_lr = self._lr(self.initial_lr)

    def set_initial_lr(self, lr: float):
        self.initial_lr = lr
        self.current_lr = self._lr(lr)


class GradScaler:
    """Dynamic loss scaling for fp16 training (no counterpart in the reference).

    ``scale(loss)`` multiplies the loss; ``unscale_and_check(optimizer)`` points the optimizer at
    a device-side ``1/scale`` and a device-side overflow flag, so the fused optimizer kernel
    unscales the gradients while it reads them and skips the whole step on overflow;
    ``update()`` halves the scale after an overflow and doubles it every ``growth_interval``
    clean steps.
    """

    def __init__(self, init_scale: float = 2.0 ** 16, growth_factor: float = 2.0,
                 backoff_factor: float = 0.5, growth_interval: int = 2000, device=None,
                 device_side: bool = False):
        """``device_side``: the scale, its reciprocal and the count of clean steps live on the device and
        ``update()`` is one tiny kernel that reads the overflow flag there — the host never waits for a
        step to finish before it launches the next one.  ``update()`` then returns None, and reading
        ``scale_value`` synchronises."""
        self._scale_host = float(init_scale)
        self.growth_factor, self.backoff_factor = growth_factor, backoff_factor
        self.growth_interval = growth_interval
        self._good_steps = 0
        self.device = device
        self.device_side = device_side
        self.inv_scale: Optional[torch.Tensor] = None
        self.found_inf: Optional[torch.Tensor] = None
        self._scale_dev: Optional[torch.Tensor] = None
        self._good_dev: Optional[torch.Tensor] = None

    @property
    def scale_value(self) -> float:
        if self.device_side and self._scale_dev is not None:
            return float(self._scale_dev.item())
        return self._scale_host

    @scale_value.setter
    def scale_value(self, v: float) -> None:
        self._scale_host = float(v)
        if self._scale_dev is not None:
            self._scale_dev.fill_(float(v))

    def _ensure(self, device):
        if self.inv_scale is None:
            self.inv_scale = torch.full((), 1.0 / self._scale_host, dtype=torch.float32, device=device)
            self.found_inf = torch.zeros(1, dtype=torch.int32, device=device)
            if self.device_side:
                self._scale_dev = torch.full((), self._scale_host, dtype=torch.float32, device=device)
                self._good_dev = torch.full((), self._good_steps, dtype=torch.int32, device=device)

    def scale(self, loss: torch.Tensor) -> torch.Tensor:
        self._ensure(loss.device)
        return loss * (self._scale_dev if self.device_side else self._scale_host)

    def unscale_and_check(self, optimizer: Optimizer) -> None:
        params = optimizer._active()
        if not params:
            return
        self._ensure(params[0].device)
        self.found_inf.zero_()
        grads = [p.grad for p in params]
        if grads[0].is_cuda:
            native.global_norm(grads, found_inf=self.found_inf)
        else:
            bad = any(not torch.isfinite(g).all() for g in grads)
            self.found_inf.fill_(1 if bad else 0)
        optimizer.grad_scale = self.inv_scale
        optimizer.skip_flag = self.found_inf
        self._optimizer = optimizer

    def update(self) -> bool:
        """Returns True when the last step overflowed (and was skipped); None in device-side mode."""
        opt = getattr(self, "_optimizer", None)
        if self.device_side and self._scale_dev is not None and not getattr(opt, "_device_skip_pending", False):
            if self._scale_dev.is_cuda:
                check(native.lib().rb_scaler_update(ptr(self._scale_dev), ptr(self.inv_scale), ptr(self._good_dev),
                                                    ptr(self.found_inf), float(self.growth_factor),
                                                    float(self.backoff_factor), int(self.growth_interval),
                                                    stream_ptr()), "rb_scaler_update")
            else:
                bad = self.found_inf.reshape(()) != 0
                good = torch.where(bad, torch.zeros_like(self._good_dev), self._good_dev + 1)
                grow = (~bad) & (good % max(1, self.growth_interval) == 0)
                s2 = torch.where(bad, self._scale_dev * self.backoff_factor,
                                 torch.where(grow, self._scale_dev * self.growth_factor, self._scale_dev))
                self._scale_dev.copy_(s2)
                self._good_dev.copy_(good)
                self.inv_scale.copy_(1.0 / s2)
            return None
        overflow = bool(int(self.found_inf.item())) if self.found_inf is not None else False
        if opt is not None and getattr(opt, "_device_skip_pending", False):
            # the device-side step counted itself before the flag was known: a skipped step must not
            # advance the bias-correction exponent (the CPU path never counts it)
            if overflow:
                opt.step_count -= 1
            opt._device_skip_pending = False
        if self.device_side and self._scale_dev is not None:      # an optimizer that needs the flag on the host
            self._scale_host = float(self._scale_dev.item())
            self._good_steps = int(self._good_dev.item())
        if overflow:
            self._scale_host *= self.backoff_factor
            self._good_steps = 0
        else:
            self._good_steps += 1
            if self._good_steps % self.growth_interval == 0:
                self._scale_host *= self.growth_factor
        if self._scale_dev is not None:
            self._scale_dev.fill_(self._scale_host)
            self._good_dev.fill_(self._good_steps)
        if self.inv_scale is not None:
            self.inv_scale.fill_(1.0 / self._scale_host)
        return overflow

    def state_dict(self):
        good = int(self._good_dev.item()) if (self.device_side and self._good_dev is not None) else self._good_steps
        return {"scale": self.scale_value, "good_steps": good}

    def load_state_dict(self, sd):
        self.scale_value, self._good_steps = sd["scale"], sd["good_steps"]
        if self._good_dev is not None:
            self._good_dev.fill_(self._good_steps)
        if self.inv_scale is not None:
            self.inv_scale.fill_(1.0 / self._scale_host)
