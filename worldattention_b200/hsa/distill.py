"""Registry for the HSA-to-dense self-distillation term (reference: wan/modules/hsa/distill.py).

Distillation is a training signal and outside what this package accelerates; the registry is kept
so code that toggles or drains it keeps working.  The CUDA forward does not build an autograd
graph, so recorded terms carry no gradient.
"""
from __future__ import annotations

import torch

_enabled = False
_losses: list = []


def enable_distill(flag: bool = True) -> None:
    global _enabled
    _enabled = bool(flag)
    if not _enabled:
        _losses.clear()


def distill_enabled() -> bool:
    return _enabled


def record_distill_loss(loss: torch.Tensor) -> None:
    if _enabled:
        _losses.append(loss)


def pop_distill_losses() -> list:
    out = list(_losses)
    _losses.clear()
    return out


def dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
    """Full softmax attention over `[B, L, H, D]` tensors (the distillation teacher)."""
    out = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return out.transpose(1, 2)


def record_against_dense(output: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> None:
    if not _enabled:
        return
    with torch.no_grad():
        target = dense_attention(q, k, v)
    record_distill_loss(torch.nn.functional.mse_loss(output.float(), target.float()))
