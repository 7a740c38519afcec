"""CPU oracle for the q/k RMSNorm + causal rotary embedding of the DiT self-attention -- TEST INFRASTRUCTURE ONLY.

A numpy restatement of `WanRMSNorm` (wan/modules/model.py:70-86) followed by `causal_rope_apply`
(wan/modules/causal_model.py:34-62), the two steps between the q/k projections and the attention call.
Nothing in the product package imports it.

Parity status: PINNED.  `tests/golden/make_golden.py` executes the reference's own definitions of these
functions (taken out of its source text) on seeded inputs; `tests/test_oracle_golden.py` checks the functions
below against those vectors.
"""
from __future__ import annotations

import numpy as np

from .hsa_oracle import as_dtype

__all__ = ["rms_norm", "causal_rope_apply", "qk_norm_rope"]


def rms_norm(x: np.ndarray, weight: np.ndarray, eps: float, dtype: str = "fp32") -> np.ndarray:
    """model.py:78-86 -- `x * rsqrt(mean(x^2) + eps)` in float32, stored in the input dtype, then times the weight
    (a second store in the input dtype)."""
    x32 = np.asarray(x, np.float32)
    mean_sq = np.mean(x32.astype(np.float64) ** 2, axis=-1, keepdims=True).astype(np.float32)
    normed = as_dtype(x32 * (np.float32(1.0) / np.sqrt(mean_sq + np.float32(eps))), dtype)
    return as_dtype(normed * np.asarray(weight, np.float32), dtype)


def causal_rope_apply(x: np.ndarray, grid, freqs: np.ndarray, start_frame: int = 0, dtype: str = "fp32") -> np.ndarray:
    """causal_model.py:34-62 -- rotate the complex pairs of every head of `[B, L, H, D]`: the first c - 2(c//3) pairs
    by the frame's factor, the next c//3 by the row's, the last c//3 by the column's (c = D / 2); float64 arithmetic,
    stored in the input dtype.  `grid` = (frames, height, width) of the L = f*h*w tokens; `freqs` complex `[rows, c]`."""
    f, h, w = (int(v) for v in grid)
    bsz, length, heads, d = x.shape
    c = d // 2
    ct = c - 2 * (c // 3)
    t = np.arange(f * h * w)
    frame, row, col = start_frame + t // (h * w), (t // w) % h, t % w
    factor = np.concatenate([freqs[frame, :ct], freqs[row, ct:ct + c // 3], freqs[col, ct + c // 3:c]], axis=1)   # [L, c]
    out = np.asarray(x, np.float64).copy()
    z = out[:, :f * h * w].reshape(bsz, f * h * w, heads, c, 2)
    zc = (z[..., 0] + 1j * z[..., 1]) * factor[None, :, None, :]
    out[:, :f * h * w] = np.stack([zc.real, zc.imag], axis=-1).reshape(bsz, f * h * w, heads, d)
    return as_dtype(out.astype(np.float32), dtype)


def qk_norm_rope(x: np.ndarray, weight: np.ndarray, eps: float, grid, freqs: np.ndarray, start_frame: int, heads: int,
                 dtype: str = "fp32") -> np.ndarray:
    """The two steps in sequence: `[B, L, H*D]` -> `[B, L, H, D]`."""
    normed = rms_norm(x, weight, eps, dtype)
    return causal_rope_apply(normed.reshape(*normed.shape[:2], heads, -1), grid, freqs, start_frame, dtype)
