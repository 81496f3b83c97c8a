"""Training leftovers of the reference, kept for inventory parity: they are on no inference path.

The reference inherits a cross-entropy loss (on probabilities, with label smoothing), its gradient and an
AdamW step from its seq2seq ancestry (TensorSharp.GGML.Native/ggml_ops_training.cpp:535-611,
TensorSharp.Backends.GGML/GgmlLossOps.cs:14-50, the Adam / RMSProp kernels of TensorSharp.Core).  Here they
are plain PyTorch tensor code, device-agnostic, with the same arithmetic:

* labels: ``1 - s + s / C`` on the target class and ``s / C`` elsewhere (``s`` = label smoothing, ``C`` classes)
* loss: mean over rows of ``- sum(labels * log(probs + smooth))`` (``smooth`` guards log(0); the reference
  takes the log of the probabilities it is handed)
* AdamW: gradient scaled by ``grad_norm_factor``, clamped to ``+-clip``, moments with bias correction
  ``1 / (1 - beta^iter)``, decoupled weight decay ``regc``, gradient zeroed afterwards.
"""
from __future__ import annotations

import torch


def smoothed_labels(targets: torch.Tensor, classes: int, label_smooth: float = 0.0) -> torch.Tensor:
    if not 0.0 <= label_smooth <= 1.0:
        raise ValueError("label_smooth must be in [0, 1]")
    if int(targets.min()) < 0 or int(targets.max()) >= classes:
        raise ValueError("target index out of range")
    base = label_smooth / classes if label_smooth > 0 else 0.0
    lab = torch.full((targets.numel(), classes), base, dtype=torch.float32, device=targets.device)
    lab.scatter_(1, targets.reshape(-1, 1).long(), 1.0 - label_smooth + base)
    return lab


def cross_entropy_loss(probs: torch.Tensor, targets: torch.Tensor, smooth: float = 0.0, label_smooth: float = 0.0) -> float:
    """``probs`` [..., C] are probabilities (already soft-maxed); returns the mean loss over the rows."""
    C = probs.shape[-1]
    p = probs.reshape(-1, C).float()
    lab = smoothed_labels(targets.reshape(-1), C, label_smooth)
    return float(-(lab * torch.log(p + smooth)).sum(-1).mean())


def cross_entropy_loss_backward(probs: torch.Tensor, targets: torch.Tensor, loss_gradient: float = 1.0, smooth: float = 0.0,
                                label_smooth: float = 0.0, grad: torch.Tensor = None, add_grad: bool = False) -> torch.Tensor:
    """Gradient of the mean loss with respect to the *logits* that produced ``probs`` by soft-max:
    ``(probs - labels) * loss_gradient / rows``; accumulated into ``grad`` when ``add_grad``."""
    C = probs.shape[-1]
    p = probs.reshape(-1, C).float()
    lab = smoothed_labels(targets.reshape(-1), C, label_smooth)
    g = ((p - lab) * (loss_gradient / p.shape[0])).reshape(probs.shape)
    if grad is None:
        return g
    if add_grad:
        grad.add_(g)
    else:
        grad.copy_(g)
    return grad


def adam_step(weight: torch.Tensor, gradient: torch.Tensor, v: torch.Tensor, m: torch.Tensor, *, grad_norm_factor: float = 1.0,
              step_size: float = 1e-3, clip_value: float = 5.0, regc: float = 0.0, decay_rate_v: float = 0.999,
              decay_rate_m: float = 0.9, iteration: int = 1, eps: float = 1e-8) -> None:
    """One AdamW update in place; ``gradient`` is zeroed afterwards, as the reference does."""
    g = (gradient * grad_norm_factor).clamp_(-clip_value, clip_value)
    m.mul_(decay_rate_m).add_(g, alpha=1.0 - decay_rate_m)
    v.mul_(decay_rate_v).addcmul_(g, g, value=1.0 - decay_rate_v)
    mh = m * (1.0 / (1.0 - decay_rate_m ** iteration))
    vh = (v * (1.0 / (1.0 - decay_rate_v ** iteration))).sqrt_().add_(eps)
    weight.mul_(1.0 - step_size * regc).addcdiv_(mh, vh, value=-step_size)
    gradient.zero_()


def rmsprop_step(weight: torch.Tensor, gradient: torch.Tensor, cache: torch.Tensor, *, grad_norm_factor: float = 1.0,
                 step_size: float = 1e-3, clip_value: float = 5.0, regc: float = 0.0, decay_rate: float = 0.999,
                 eps: float = 1e-8) -> None:
    """RMSProp with clipping and L2 regularisation, in place; the gradient is zeroed afterwards."""
    g = (gradient * grad_norm_factor).clamp_(-clip_value, clip_value)
    cache.mul_(decay_rate).addcmul_(g, g, value=1.0 - decay_rate)
    weight.sub_(step_size * g / (cache + eps).sqrt() + step_size * regc * weight)
    gradient.zero_()
