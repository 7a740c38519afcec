"""Two-stage retrieval over the hierarchical KV bank (reference: pipeline/hkv/retrieval.py).

Stage 1 ranks chunks by cosine similarity of prompt embeddings; stage 2 pools the pages of the
candidate chunks and takes the global top-K by `alpha = (Qbar . Kbar) / sqrt(dim)`.  Page
centroids, page scores and the top-k run in csrc/wa_hkv.cu; equal scores are ordered by the lower
index.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch
import torch.nn.functional as F

from .. import _lib
from .rope import rotation_table, temporal_complex_dims

__all__ = ["prompt_index", "query_index", "page_key_index", "score_pages", "select_top_chunks",
           "select_topk_pages", "score_and_topk"]


def prompt_index(prompt_embeds: torch.Tensor) -> torch.Tensor:
    """Mean-pool `[B, tokens, dim]` into a unit vector `[dim]` (retrieval.py:32-38)."""
    pooled = prompt_embeds.float().mean(dim=1).mean(dim=0)
    return F.normalize(pooled, dim=0)


def query_index(q_tokens: torch.Tensor) -> torch.Tensor:
    """Mean-pool pre-rotation queries `[B, tokens, H*D]` into `[H*D]` (retrieval.py:41-47)."""
    return q_tokens.float().mean(dim=1).mean(dim=0)


def page_key_index(keys: torch.Tensor, page_spans: Sequence[Tuple[int, int]], *, frame_seq_length: int,
                   start_frame: int, temporal_freqs) -> Optional[torch.Tensor]:
    """Per-page mean key in content space: `[num_pages, H*D]` float32 (retrieval.py:50-72).

    `keys` is `[B, tokens, H, D]` as cached (rotated).  The temporal rotation of every token is
    removed inside the pooling kernel; no de-rotated copy of the keys is materialised.
    """
    if not page_spans:
        return None
    dev = _lib.require_cuda(keys)
    bsz, tokens, heads, head_dim = keys.shape
    nt = temporal_complex_dims(head_dim)
    n_frames = (tokens + frame_seq_length - 1) // frame_seq_length
    frames = start_frame + np.arange(n_frames)
    rot = torch.from_numpy(rotation_table(temporal_freqs, np.zeros_like(frames), frames, nt)).to(dev)
    spans = torch.tensor([[int(s), int(e)] for s, e in page_spans], dtype=torch.int32).to(dev)
    out = torch.empty((len(page_spans), heads * head_dim), device=dev, dtype=torch.float32)
    keys = keys if keys.stride(-1) == 1 else keys.contiguous()
    _lib.check(_lib.lib().wa_hkv_page_centroids(
        _lib.t4_blhd(keys), bsz, tokens, heads, head_dim, spans.data_ptr(), len(page_spans), rot.data_ptr(),
        n_frames, nt, frame_seq_length, out.data_ptr(), _lib.stream_ptr(dev)))
    return out


def score_and_topk(query_vec: torch.Tensor, page_index: torch.Tensor, topk: int, *, groups: int = 1,
                   scale: Optional[float] = None):
    """Scores `[G, P]` plus top-k ids/scores `[G, topk]` in one launch.

    `groups=1` scores whole index vectors (the reference's behaviour); `groups=H` scores each
    head's slice of the vector separately and selects per head.
    """
    dev = _lib.require_cuda(page_index)
    pages, dim = page_index.shape
    if dim % groups:
        raise ValueError(f"index dim {dim} is not divisible into {groups} groups")
    index = page_index.float().contiguous()
    query = query_vec.to(device=dev, dtype=torch.float32).reshape(-1).contiguous()
    if query.shape[0] != dim:
        raise ValueError(f"query dim {query.shape[0]} does not match page index dim {dim}")
    if scale is None:
        scale = float(dim // groups) ** 0.5
    k = max(0, min(int(topk), pages))
    scores = torch.empty((groups, pages), device=dev, dtype=torch.float32)
    ids = torch.empty((groups, max(k, 1)), device=dev, dtype=torch.int32)
    vals = torch.empty((groups, max(k, 1)), device=dev, dtype=torch.float32)
    _lib.check(_lib.lib().wa_hkv_score_topk(
        index.data_ptr(), query.data_ptr(), pages, groups, dim // groups, float(scale or 0.0), k,
        scores.data_ptr(), ids.data_ptr(), vals.data_ptr(), _lib.stream_ptr(dev)))
    return scores, ids[:, :k], vals[:, :k]


def score_and_topk_layers(query_vec: torch.Tensor, page_index: torch.Tensor, topk: int, *, groups: int = 1,
                          scale: Optional[float] = None):
    """`score_and_topk` for a stack of page indexes `[layers, P, dim]` in ONE launch (no host loop).

    `query_vec` is `[dim]` (shared by the layers) or `[layers, dim]`.  Returns scores `[layers, G, P]` and
    top-k ids / scores `[layers, G, topk]`, all on the device.
    """
    dev = _lib.require_cuda(page_index)
    layers, pages, dim = page_index.shape
    if dim % groups:
        raise ValueError(f"index dim {dim} is not divisible into {groups} groups")
    index = page_index.float().contiguous()
    query = query_vec.to(device=dev, dtype=torch.float32).contiguous()
    if tuple(query.shape) not in ((dim,), (layers, dim)):
        raise ValueError(f"query must be [{dim}] or [{layers}, {dim}], got {tuple(query.shape)}")
    stride = dim if query.dim() == 2 else 0
    if scale is None:
        scale = float(dim // groups) ** 0.5
    k = max(0, min(int(topk), pages))
    scores = torch.empty((layers, groups, pages), device=dev, dtype=torch.float32)
    ids = torch.empty((layers, groups, max(k, 1)), device=dev, dtype=torch.int32)
    vals = torch.empty((layers, groups, max(k, 1)), device=dev, dtype=torch.float32)
    _lib.check(_lib.lib().wa_hkv_score_topk_layers(
        index.data_ptr(), query.data_ptr(), layers, pages, groups, dim // groups, stride, float(scale or 0.0), k,
        scores.data_ptr(), ids.data_ptr(), vals.data_ptr(), _lib.stream_ptr(dev)))
    return scores, ids[..., :k], vals[..., :k]


def score_pages(query_vec: torch.Tensor, page_index: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Affinity `alpha_j = (Qbar . Kbar_j) / sqrt(dim)` for every page (retrieval.py:75-89)."""
    if page_index.numel() == 0:
        return page_index.new_zeros((0,))
    scores, _, _ = score_and_topk(query_vec, page_index, 0, scale=scale)
    return scores[0]


def select_top_chunks(query_vec: torch.Tensor, chunk_index: torch.Tensor, topk: int) -> List[int]:
    """Stage 1: chunk ids most cosine-similar to `query_vec` (retrieval.py:92-102)."""
    if chunk_index.numel() == 0 or topk <= 0:
        return []
    _, ids, _ = score_and_topk(query_vec, chunk_index, topk, scale=0.0)
    return [int(i) for i in ids[0].tolist()]


def select_topk_pages(query_vec: torch.Tensor, candidates: Sequence[Tuple[int, int, torch.Tensor]], topk: int,
                      scale: Optional[float] = None) -> List[Tuple[int, int, float]]:
    """Stage 2: global top-`K_p` pages across candidate chunks (retrieval.py:105-126)."""
    if topk <= 0 or len(candidates) == 0:
        return []
    index = torch.stack([c[2].reshape(-1).float() for c in candidates], dim=0)
    _, ids, vals = score_and_topk(query_vec.float(), index, topk, scale=scale)
    ids, vals = ids[0].tolist(), vals[0].tolist()
    return [(int(candidates[i][0]), int(candidates[i][1]), float(s)) for i, s in zip(ids, vals)]
