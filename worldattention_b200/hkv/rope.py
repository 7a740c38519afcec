"""Temporal rotary re-rotation for reused KV pages (reference: pipeline/hkv/rope.py).

Moving a token along the frame axis only touches the temporal band of its rotary embedding, i.e.
the first `temporal_complex_dims(D)` complex pairs of every head.  Both operations here are one
launch of the page-copy kernel (csrc/wa_hkv.cu) with a rotation table built on the host in
complex128, the precision the reference keeps its frequency table in.
"""
from __future__ import annotations

import ctypes

import numpy as np
import torch

from .. import _lib

__all__ = ["temporal_complex_dims", "temporal_band", "shift_temporal_rope", "derope_temporal",
           "rotation_table"]


def temporal_complex_dims(head_dim: int) -> int:
    """Complex pairs in the temporal band of a `head_dim` rotary embedding (rope.py:22-25)."""
    half = head_dim // 2
    return half - 2 * (half // 3)


def temporal_band(freqs: torch.Tensor, head_dim: int) -> torch.Tensor:
    """Slice the temporal band out of a `[max_positions, head_dim // 2]` table (rope.py:28-30)."""
    return freqs[:, : temporal_complex_dims(head_dim)]


def _freqs_numpy(temporal_freqs) -> np.ndarray:
    if isinstance(temporal_freqs, torch.Tensor):
        return temporal_freqs.detach().to("cpu").numpy()
    return np.asarray(temporal_freqs)


def rotation_table(temporal_freqs, new_ids, orig_ids, num_temporal: int) -> np.ndarray:
    """`freqs[new] * conj(freqs[orig])` per row, ids clamped to the table (rope.py:40-47).

    Returns float32 `[rows, num_temporal, 2]` (complex64 as re/im pairs), computed in complex128.
    """
    table = _freqs_numpy(temporal_freqs)
    n = table.shape[0]
    new = np.clip(np.asarray(new_ids, dtype=np.int64).reshape(-1), 0, n - 1)
    orig = np.clip(np.asarray(orig_ids, dtype=np.int64).reshape(-1), 0, n - 1)
    factor = (table[new, :num_temporal] * np.conj(table[orig, :num_temporal])).astype(np.complex64)
    return np.ascontiguousarray(factor).view(np.float32).reshape(len(new), num_temporal, 2)


def _run_copies(records, src_like: torch.Tensor, row_elems: int, head_dim: int, rotations: np.ndarray,
                num_temporal: int, max_tokens: int) -> None:
    dev = src_like.device
    arr = (_lib.PageCopy * len(records))(*records)
    host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8)
    dev_records = host.to(dev, non_blocking=False)
    rot = torch.from_numpy(np.ascontiguousarray(rotations)).to(dev) if rotations is not None and rotations.size else None
    _lib.check(_lib.lib().wa_hkv_gather_pages(
        dev_records.data_ptr(), len(records), max_tokens, row_elems, head_dim, _lib.dtype_code(src_like.dtype),
        _lib.ptr(rot), num_temporal, _lib.stream_ptr(dev)))


def shift_temporal_rope(k: torch.Tensor, temporal_freqs, new_frame0: int, orig_frame0: int) -> torch.Tensor:
    """Move a page of `[..., tokens, H, D]` keys from `orig_frame0` to `new_frame0` (rope.py:50-67)."""
    _lib.require_cuda(k)
    head_dim = k.shape[-1]
    nt = temporal_complex_dims(head_dim)
    src = k.contiguous()
    out = torch.empty_like(src)
    rows = src.numel() // (src.shape[-2] * head_dim)
    row_elems = src.shape[-2] * head_dim
    rot = rotation_table(temporal_freqs, [int(new_frame0)], [int(orig_frame0)], nt)
    rec = _lib.PageCopy(src.data_ptr(), out.data_ptr(), row_elems, row_elems, rows, 0)
    _run_copies([rec], src, row_elems, head_dim, rot, nt, rows)
    return out


def derope_temporal(k: torch.Tensor, temporal_freqs, frame_ids: torch.Tensor) -> torch.Tensor:
    """Remove each token's own temporal rotation from `[B, T, H, D]` keys (rope.py:70-82).

    `frame_ids` gives the absolute frame of every token; consecutive tokens of one frame become
    one copy record.
    """
    _lib.require_cuda(k)
    bsz, tokens, heads, head_dim = k.shape
    nt = temporal_complex_dims(head_dim)
    ids = frame_ids.detach().to("cpu").numpy().astype(np.int64).reshape(-1)
    if ids.shape[0] != tokens:
        raise ValueError(f"frame_ids has {ids.shape[0]} entries for {tokens} tokens")
    src = k.contiguous()
    out = torch.empty_like(src)
    row_elems = heads * head_dim
    esize = src.element_size()
    # runs of equal frame id
    starts = np.flatnonzero(np.concatenate([[True], ids[1:] != ids[:-1]]))
    ends = np.concatenate([starts[1:], [tokens]])
    frames, inverse = np.unique(ids[starts], return_inverse=True)
    rot = rotation_table(temporal_freqs, np.zeros_like(frames), frames, nt)
    records, longest = [], 1
    for b in range(bsz):
        for run, (s, e) in enumerate(zip(starts, ends)):
            off = (b * tokens + int(s)) * row_elems * esize
            records.append(_lib.PageCopy(src.data_ptr() + off, out.data_ptr() + off, row_elems, row_elems,
                                         int(e - s), int(inverse[run])))
            longest = max(longest, int(e - s))
    _run_copies(records, src, row_elems, head_dim, rot, nt, longest)
    return out
