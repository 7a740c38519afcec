"""HSA parameter helpers used by callers and tests (reference: trainer/hsa_stage.py).

Only the pieces an inference user needs are provided: the block-average initialisation that gives
the linear branch a non-degenerate starting point, the name iterator, and the backend switch.
Training-stage configuration (trainable sets, distillation collection) is out of scope.
"""
from __future__ import annotations

from typing import Iterator, Tuple

import torch
import torch.nn as nn

from .hsa import HSAAttention

__all__ = ["init_hsa_parameters", "hsa_named_parameters", "set_hsa_backend"]

_HSA_ATTR = "hsa_attention"


def init_hsa_parameters(model: nn.Module) -> int:
    """Make every projection row the average of one block of tokens; zero the gate.

    Same result as the reference's `init_hsa_parameters` (trainer/hsa_stage.py:43-88) for
    unsharded parameters.  Returns the number of HSA modules initialised.
    """
    modules = [m for m in model.modules() if isinstance(m, HSAAttention)]
    with torch.no_grad():
        for module in modules:
            rank, seq_len = module.k_proj_mat.shape
            rows = torch.arange(rank).unsqueeze(1)
            cols = torch.arange(seq_len).unsqueeze(0)
            lo = rows * module.block_size
            hi = torch.clamp((rows + 1) * module.block_size, max=seq_len)
            width = (hi - lo).clamp(min=1).float()
            pattern = ((cols >= lo) & (cols < hi)).float() / width
            for proj in (module.k_proj_mat, module.v_proj_mat):
                proj.copy_(pattern.to(device=proj.device, dtype=proj.dtype))
            module.gate_lin.weight.zero_()
            module.gate_lin.bias.zero_()
    return len(modules)


def hsa_named_parameters(model: nn.Module, attr_name: str = _HSA_ATTR) -> Iterator[Tuple[str, nn.Parameter]]:
    """Yield the `(name, parameter)` pairs that belong to HSA submodules."""
    for name, param in model.named_parameters():
        if attr_name in name:
            yield name, param


def set_hsa_backend(model: nn.Module, backend: str = "auto") -> int:
    """Point every HSA module at a backend name; returns how many were set."""
    count = 0
    for module in model.modules():
        if isinstance(module, HSAAttention):
            module.backend = backend
            count += 1
    return count
