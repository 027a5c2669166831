"""Optimizers and schedulers (reference: rumus/src/optim/)."""
from .optimizers import (Optimizer, SGD, Adam, AdamW, clip_grad_norm_, LRScheduler, StepLR,
                         CosineAnnealingLR, GradScaler)
