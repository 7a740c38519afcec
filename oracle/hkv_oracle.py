"""CPU oracle for Hierarchical KV Cache (HKV) retrieval -- TEST INFRASTRUCTURE ONLY.

A numpy restatement of the reference's page-centroid scoring, top-k page selection and page
install (gather + temporal re-rotation).  Used as the checker in the tests, the smoke test and the
benchmark's CPU baseline; never imported by the product package.

Parity status: PINNED by `tests/golden/` vectors generated from the reference's own functions
(`tests/golden/make_golden.py`) and checked in `tests/test_oracle_golden.py`.

Conventions: arrays are float32 (bf16 tensors are float32 values representable in bf16, tagged by
`dtype`); the temporal frequency table is complex128 `[max_positions, n_temporal]` exactly as the
reference keeps it.  Reductions accumulate in float64 and round once to float32; equal scores are
ordered by the lower index (the reference's `torch.topk` leaves that order unspecified).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np

from .hsa_oracle import as_dtype

__all__ = [
    "temporal_complex_dims", "temporal_band", "rotation_factor", "apply_factor",
    "shift_temporal_rope", "derope_temporal", "prompt_index", "query_index", "page_key_index",
    "score_pages", "topk_lower_index_first", "select_top_chunks", "select_topk_pages",
    "page_spans", "plan_install", "plan_rerope", "install_pages",
]


# --------------------------------------------------------------------------------------------
# pipeline/hkv/rope.py
# --------------------------------------------------------------------------------------------

def temporal_complex_dims(head_dim: int) -> int:
    """rope.py:22-25 -- complex pairs in the temporal band."""
    half = head_dim // 2
    return half - 2 * (half // 3)


def temporal_band(freqs: np.ndarray, head_dim: int) -> np.ndarray:
    """rope.py:28-30."""
    return freqs[:, : temporal_complex_dims(head_dim)]


def rotation_factor(temporal_freqs: np.ndarray, new_ids, orig_ids) -> np.ndarray:
    """rope.py:40-47 -- `freqs[new] * conj(freqs[orig])` with both ids clamped to the table.

    Computed in complex128 and rounded to complex64, as the reference does before multiplying.
    """
    n = temporal_freqs.shape[0]
    new = np.clip(np.asarray(new_ids, dtype=np.int64), 0, n - 1)
    orig = np.clip(np.asarray(orig_ids, dtype=np.int64), 0, n - 1)
    return (temporal_freqs[new] * np.conj(temporal_freqs[orig])).astype(np.complex64)


def apply_factor(k: np.ndarray, factor: np.ndarray, num_temporal: int, dtype: str) -> np.ndarray:
    """rope.py:33-40 -- multiply the first `num_temporal` complex pairs of the last axis by `factor`.

    `factor` broadcasts against `k[..., :num_temporal]` viewed as complex.  The product is formed
    in float32 as `(ac - bd, ad + bc)` with every multiply and add rounded separately, then stored
    in the key dtype.
    """
    k = np.asarray(k, np.float32)
    out = k.copy()
    a = k[..., 0:2 * num_temporal:2]
    b = k[..., 1:2 * num_temporal:2]
    c = np.real(factor).astype(np.float32)
    d = np.imag(factor).astype(np.float32)
    re = ((a * c).astype(np.float32) - (b * d).astype(np.float32)).astype(np.float32)
    im = ((a * d).astype(np.float32) + (b * c).astype(np.float32)).astype(np.float32)
    out[..., 0:2 * num_temporal:2] = re
    out[..., 1:2 * num_temporal:2] = im
    return as_dtype(out, dtype)


def shift_temporal_rope(k, temporal_freqs, new_frame0: int, orig_frame0: int, dtype: str = "fp32"):
    """rope.py:50-67 -- move a page of `[..., tokens, H, D]` keys by a constant frame delta."""
    nt = temporal_complex_dims(k.shape[-1])
    factor = rotation_factor(temporal_freqs, int(new_frame0), int(orig_frame0))
    return apply_factor(k, factor[:nt], nt, dtype)


def derope_temporal(k, temporal_freqs, frame_ids, dtype: str = "fp32"):
    """rope.py:70-82 -- remove each token's own temporal rotation from `[B, T, H, D]` keys."""
    nt = temporal_complex_dims(k.shape[-1])
    frame_ids = np.asarray(frame_ids, dtype=np.int64)
    factor = rotation_factor(temporal_freqs, np.zeros_like(frame_ids), frame_ids)   # [T, nt]
    return apply_factor(k, factor[None, :, None, :nt], nt, dtype)


# --------------------------------------------------------------------------------------------
# pipeline/hkv/retrieval.py
# --------------------------------------------------------------------------------------------

def _mean64(x: np.ndarray, axis: int) -> np.ndarray:
    return np.mean(x.astype(np.float64), axis=axis).astype(np.float32)


def prompt_index(prompt_embeds: np.ndarray) -> np.ndarray:
    """retrieval.py:32-38 -- mean over tokens then batch, L2-normalised (eps 1e-12)."""
    pooled = _mean64(_mean64(np.asarray(prompt_embeds, np.float32), 1), 0)
    norm = np.float32(np.sqrt(np.sum(pooled.astype(np.float64) ** 2)))
    return (pooled / max(norm, np.float32(1e-12))).astype(np.float32)


def query_index(q_tokens: np.ndarray) -> np.ndarray:
    """retrieval.py:41-47 -- `[B, tokens, H*D]` -> `[H*D]` mean query."""
    return _mean64(_mean64(np.asarray(q_tokens, np.float32), 1), 0)


def page_key_index(keys, spans: Sequence[Tuple[int, int]], *, frame_seq_length: int,
                   start_frame: int, temporal_freqs, dtype: str = "fp32") -> Optional[np.ndarray]:
    """retrieval.py:50-72 -- per-page mean of content-space keys, `[pages, H*D]` float32."""
    if not spans:
        return None
    t = keys.shape[1]
    frame_ids = start_frame + np.arange(t) // frame_seq_length
    content = derope_temporal(keys, temporal_freqs, frame_ids, dtype).reshape(keys.shape[0], t, -1)
    return np.stack([_mean64(_mean64(content[:, s:e], 1), 0) for s, e in spans], axis=0)


def score_pages(query_vec, page_index, scale: Optional[float] = None) -> np.ndarray:
    """retrieval.py:75-89 -- `index @ q / sqrt(dim)`."""
    page_index = np.asarray(page_index, np.float32)
    if page_index.size == 0:
        return np.zeros((0,), np.float32)
    q = np.asarray(query_vec, np.float32).reshape(-1)
    scores = (page_index.astype(np.float64) @ q.astype(np.float64)).astype(np.float32)
    if scale is None:
        scale = float(page_index.shape[-1]) ** 0.5
    if scale and scale > 0:
        scores = (scores / np.float32(scale)).astype(np.float32)
    return scores


def topk_lower_index_first(scores: np.ndarray, k: int):
    """Largest `k` entries, highest first, equal scores by ascending index."""
    scores = np.asarray(scores, np.float32)
    order = np.argsort(-scores, kind="stable")[:k]
    return order.astype(np.int32), scores[order]


def select_top_chunks(query_vec, chunk_index, topk: int) -> List[int]:
    """retrieval.py:92-102 -- stage 1, cosine over the prompt bank."""
    chunk_index = np.asarray(chunk_index, np.float32)
    if chunk_index.size == 0 or topk <= 0:
        return []
    scores = (chunk_index.astype(np.float64) @ np.asarray(query_vec, np.float64).reshape(-1)).astype(np.float32)
    ids, _ = topk_lower_index_first(scores, min(int(topk), scores.shape[0]))
    return [int(i) for i in ids]


def select_topk_pages(query_vec, candidates, topk: int, scale: Optional[float] = None):
    """retrieval.py:105-126 -- stage 2, one global top-k over pooled candidate pages."""
    if topk <= 0 or len(candidates) == 0:
        return []
    index = np.stack([np.asarray(c[2], np.float32).reshape(-1) for c in candidates], axis=0)
    scores = score_pages(query_vec, index, scale=scale)
    ids, vals = topk_lower_index_first(scores, min(int(topk), scores.shape[0]))
    return [(int(candidates[i][0]), int(candidates[i][1]), float(s)) for i, s in zip(ids, vals)]


# --------------------------------------------------------------------------------------------
# pipeline/hkv/cache.py
# --------------------------------------------------------------------------------------------

def page_spans(valid_tokens: int, page_tokens: int) -> List[Tuple[int, int]]:
    """cache.py:109-112 -- token spans of a chunk's pages; the last may be partial."""
    return [(s, min(s + page_tokens, valid_tokens)) for s in range(0, valid_tokens, page_tokens)]


def plan_install(entries: Sequence[Tuple[int, int, int]], capacity: int):
    """cache.py:203-211 -- truncate the `(chunk, start, end)` list to the cache capacity."""
    budget, installed = capacity, []
    for chunk_id, start, end in entries:
        if budget <= 0:
            break
        take = min(end - start, budget)
        installed.append((chunk_id, start, start + take))
        budget -= take
    return installed


def plan_rerope(installed, chunk_start_frames, frame_seq_length: int, current_start_frame: int):
    """cache.py:273-287 -- `(orig_frame, new_frame)` of each installed page."""
    total = sum(e - s for _, s, e in installed)
    base = current_start_frame - total // frame_seq_length
    moves, offset = [], 0
    for chunk_id, start, end in installed:
        orig = chunk_start_frames[chunk_id] + start // frame_seq_length
        moves.append((orig, base + offset // frame_seq_length))
        offset += end - start
    return moves


def install_pages(capacity: int, chunk_k, chunk_v, installed, moves, temporal_freqs,
                  dtype: str = "fp32"):
    """cache.py:222-246 -- the K/V cache of one layer after the selected pages are installed.

    `chunk_k[c]`, `chunk_v[c]` are the stored `[B, valid, H, D]` arrays of chunk `c` for this
    layer.  Everything outside the installed span is zero (cache.py:223-224); keys are re-rotated
    per page when `moves` is given (cache.py:232-236), values are copied verbatim.
    """
    first = chunk_k[installed[0][0]]
    b, _, h, d = first.shape
    out_k = np.zeros((b, capacity, h, d), np.float32)
    out_v = np.zeros((b, capacity, h, d), np.float32)
    offset = 0
    for i, (chunk_id, start, end) in enumerate(installed):
        seg_k = np.asarray(chunk_k[chunk_id][:, start:end], np.float32)
        if moves is not None:
            orig, new = moves[i]
            seg_k = shift_temporal_rope(seg_k, temporal_freqs, new, orig, dtype)
        out_k[:, offset:offset + (end - start)] = seg_k
        out_v[:, offset:offset + (end - start)] = np.asarray(chunk_v[chunk_id][:, start:end], np.float32)
        offset += end - start
    return as_dtype(out_k, dtype), as_dtype(out_v, dtype), offset
