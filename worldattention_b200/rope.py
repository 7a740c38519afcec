"""q/k RMSNorm and causal rotary embedding of the DiT self-attention on the GPU.

`causal_rope_apply` keeps the reference's signature (wan/modules/causal_model.py:34-62); `qk_norm_rope` fuses the
RMSNorm in front of it (wan/modules/model.py:70-86), which the reference applies to q and k just before.  One kernel
launch per tensor, no float64 copy of the tokens, no loop over samples.
"""
from __future__ import annotations

import torch

from . import _lib

__all__ = ["causal_rope_apply", "qk_norm_rope"]


def _table(freqs: torch.Tensor, dev: torch.device) -> torch.Tensor:
    """The reference's complex table `[rows, D/2]` as float64 `[rows, D/2, 2]` on the device."""
    if torch.is_complex(freqs):
        freqs = torch.view_as_real(freqs.to(torch.complex128))
    return freqs.to(device=dev, dtype=torch.float64).contiguous()


def _grid(grid_sizes) -> tuple[int, int, int]:
    rows = grid_sizes.tolist() if hasattr(grid_sizes, "tolist") else list(grid_sizes)
    if rows and isinstance(rows[0], (list, tuple)):
        if any(tuple(r) != tuple(rows[0]) for r in rows):
            raise NotImplementedError("samples of one batch must share a (frames, height, width) grid")
        rows = rows[0]
    f, h, w = (int(v) for v in rows)
    return f, h, w


def qk_norm_rope(x: torch.Tensor, norm_weight: torch.Tensor | None, eps: float, grid_sizes, freqs: torch.Tensor | None,
                 start_frame=0, *, heads: int | None = None, table: torch.Tensor | None = None) -> torch.Tensor:
    """RMSNorm over the last axis of `[B, L, H*D]` (or `[B, L, H, D]`), then the causal rotary embedding -> `[B, L, H, D]`.

    `table` is `_table(freqs)` kept by the caller (saves the conversion per call).  `start_frame` may be an int32 device
    tensor of one element: the kernel then reads the position when it runs (for launches replayed from a CUDA graph)."""
    dev = _lib.require_cuda(x)
    if x.dim() == 3:
        if heads is None:
            raise ValueError("heads is needed to split the last axis of a [B, L, H*D] tensor")
        x = x.view(x.shape[0], x.shape[1], heads, -1)
    bsz, length, n_heads, head_dim = x.shape
    x = x if x.stride(-1) == 1 else x.contiguous()
    out = torch.empty((bsz, length, n_heads, head_dim), device=dev, dtype=x.dtype)
    f = h = w = 1
    if freqs is not None or table is not None:
        f, h, w = _grid(grid_sizes)
        if f * h * w != length:
            raise NotImplementedError(f"the grid {f}x{h}x{w} must cover all {length} tokens")
        table = _table(freqs, dev) if table is None else table
    weight = None if norm_weight is None else norm_weight.detach().to(dev).contiguous()
    head = (_lib.t4_blhd(x), _lib.t4_blhd(out), bsz, length, n_heads, head_dim, _lib.ptr(weight),
            _lib.dtype_code(weight.dtype) if weight is not None else 0, float(eps), _lib.ptr(table),
            int(table.shape[0]) if table is not None else 0)
    if isinstance(start_frame, torch.Tensor):
        if start_frame.dtype != torch.int32 or start_frame.numel() != 1 or start_frame.device != dev:
            raise ValueError("a device-resident start_frame must be one int32 on the tensors' device")
        _lib.check(_lib.lib().wa_qk_norm_rope_at(*head, start_frame.data_ptr(), h, w, _lib.stream_ptr(dev)))
    else:
        _lib.check(_lib.lib().wa_qk_norm_rope(*head, int(start_frame), h, w, _lib.stream_ptr(dev)))
    return out


def causal_rope_apply(x: torch.Tensor, grid_sizes, freqs: torch.Tensor, start_frame: int = 0) -> torch.Tensor:
    """Rotary embedding of `[B, L, H, D]` tokens laid out as a (frames, height, width) grid that starts at `start_frame`."""
    return qk_norm_rope(x, None, 0.0, grid_sizes, freqs, start_frame)
