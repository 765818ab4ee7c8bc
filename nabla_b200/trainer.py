"""The optimizer-facing tail of nabla's training loop, on device buffers.

`TrainerTail.on_backward(params, grads)` is what `Trainer::train_epoch_with_max_steps` does between
`loss.backward()` and the next batch (nabla-train/src/trainer.rs:230-292), in the same order:

    GradScaler::unscale_and_update   (a `false` drops the partial accumulation and skips the step)
    has_non_finite + GradNanPolicy   (Skip -> drop and skip, Stop -> error, None -> carry on)
    accumulate                        buf = buf + g, allocated as zeros on first use
    when `grad_accum` micro-batches are in:
        set_lr(lr_at_step(schedule, base_lr, state.step))      (step counted before the increment)
        clip_grad_norm(buf, max_norm)                            (with_grad_clip maps max_norm <= 0 to off)
        optimizer.step(params, buf)
        buf = zeros ; state.step += 1

Every tensor op is a kernel of libnabla_optim_b200 over the device table; nothing is computed in torch.
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

from . import _lib as L
from .checkpoint import TrainState
from .optim import GradClipper, GradScaler, LrSchedule, Optimizer, _Handle, _check_tensors, _ptrs, lr_at_step


class GradNanPolicy:
    """`enum GradNanPolicy` (trainer.rs)."""
    Skip = "skip"
    Stop = "stop"


class NonFiniteGradient(RuntimeError):
    """TrainError::EvalError("non-finite gradient") (trainer.rs:246-248)."""


class GradAccumulator:
    """Accumulation buffers + the kernel that adds a gradient list into them."""

    def __init__(self, shapes: Sequence, device=None, stream=None):
        self._numel = [int(torch.Size(s).numel()) if not isinstance(s, int) else s for s in shapes]
        self._h = _Handle(device, stream)
        self._h.add_group(L.GroupConfig(kind=L.NBO_SGD, lr=0.0))
        self._h.set_tensors(self._numel, None, L.NBO_F32)

    def add(self, accum: Sequence[torch.Tensor], grads: Sequence[torch.Tensor]) -> None:
        _check_tensors(accum, torch.float32, "accum")
        _check_tensors(grads, torch.float32, "grads")
        self._h.check(self._h.lib.nbo_accumulate_grads(self._h.h, len(accum), _ptrs(accum), _ptrs(grads)))

    def zero(self, accum: Sequence[torch.Tensor]) -> None:
        self._h.check(self._h.lib.nbo_zero_grad(self._h.h, len(accum), _ptrs(accum)))


class TrainerTail:
    def __init__(self, optimizer: Optimizer, shapes: Sequence, *, scaler: bool = False,
                 nan_policy: Optional[str] = None, schedule: Optional[Tuple[LrSchedule, float]] = None,
                 grad_clip: Optional[float] = None, grad_accum: int = 1, device=None):
        self.optimizer = optimizer
        self.shapes = [tuple(s) if not isinstance(s, int) else (s,) for s in shapes]
        self.scaler = GradScaler(self.shapes, device=device) if scaler else None
        self.nan_policy = nan_policy
        self.schedule = schedule
        self.grad_clip = grad_clip if (grad_clip is not None and grad_clip > 0.0) else None   # trainer.rs:137-140
        self.state = TrainState(0, 0, max(1, grad_accum), None)
        self._acc = GradAccumulator(self.shapes, device=device)
        self._clip = GradClipper(self.shapes, device=device)
        self._buf = None
        self._count = 0
        self.last_grad_norm = 0.0

    def _drop(self):
        self._buf, self._count = None, 0

    def on_backward(self, params: Sequence[torch.Tensor], grads: Sequence[torch.Tensor]) -> bool:
        """Returns True when an optimizer step was applied."""
        if self.scaler is not None and not self.scaler.unscale_and_update(grads):
            self._drop()
            return False
        if self.nan_policy is not None:
            _, bad = self._clip.grad_norm(grads)
            if bad:
                if self.nan_policy == GradNanPolicy.Skip:
                    self._drop()
                    return False
                raise NonFiniteGradient("non-finite gradient")
        if self._buf is None:
            self._buf = [torch.zeros_like(g) for g in grads]
        self._acc.add(self._buf, grads)
        self._count += 1
        if self._count < self.state.grad_accum:
            return False
        if self.schedule is not None:
            self.optimizer.set_lr(lr_at_step(self.schedule[0], self.schedule[1], self.state.step))
        if self.grad_clip is not None:
            self.last_grad_norm = self._clip.clip_grad_norm(self._buf, self.grad_clip)
        self.optimizer.step(params, self._buf)
        self._count = 0
        self._acc.zero(self._buf)
        self.state.step += 1
        return True
