"""Training loop helper (reference: rumus/src/train.rs:32-96).

``Trainer.train_step(closure)`` runs forward (the closure returns the loss), backward and the
optimizer step, and keeps epoch statistics.  Unlike the reference, the loss value is not read
back every step: it is accumulated on the device and fetched only when statistics are asked for
(``sync_every`` bounds how stale the host copy may get).
"""
from __future__ import annotations

from typing import Callable, Optional

import torch

from .optim import GradScaler, Optimizer, clip_grad_norm_


class Trainer:
    def __init__(self, optimizer: Optimizer, max_grad_norm: Optional[float] = None,
                 grad_scaler: Optional[GradScaler] = None):
        self.optimizer = optimizer
        self.max_grad_norm = max_grad_norm
        self.grad_scaler = grad_scaler
        self._loss_sum: Optional[torch.Tensor] = None
        self._steps = 0
        self.last_loss: Optional[torch.Tensor] = None
        self.skipped_steps = 0

    def train_step(self, forward_fn: Callable[[], torch.Tensor]) -> torch.Tensor:
        """Returns the (device-resident) loss tensor of this step."""
        self.optimizer.zero_grad()
        loss = forward_fn()
        if self.grad_scaler is not None:
            self.grad_scaler.scale(loss).backward()
            self.grad_scaler.unscale_and_check(self.optimizer)
        else:
            loss.backward()
        if self.max_grad_norm is not None:
            clip_grad_norm_(self.optimizer.params, self.max_grad_norm)
        self.optimizer.step()
        if self.grad_scaler is not None and self.grad_scaler.update():
            self.skipped_steps += 1
        d = loss.detach().float()
        self._loss_sum = d if self._loss_sum is None else self._loss_sum + d
        self._steps += 1
        self.last_loss = d
        return d

    def epoch_avg_loss(self) -> float:
        if self._steps == 0:
            return 0.0
        return float(self._loss_sum.item()) / self._steps

    def reset_epoch(self) -> None:
        self._loss_sum, self._steps = None, 0

    def optimizer_mut(self) -> Optimizer:
        return self.optimizer
