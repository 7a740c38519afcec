"""Head-adaptive block routing, CUDA implementation.

Same functions and argument meaning as the reference's `wan/modules/hsa/routing.py`; the maths runs
in `libwa_b200.so` (csrc/wa_routing.cu).  Differences from the reference are limited to making the
discrete outcome well defined: reductions accumulate in float64 and equal probabilities are ordered
by the lower block id.
"""
from __future__ import annotations

import math

import torch

from .. import _lib

__all__ = [
    "BlockRouting", "build_block_routing", "block_attention_map", "block_mean_pool", "block_counts",
    "pad_to_len", "variable_block_sizes",
]


class BlockRouting:
    """Which key blocks each query block attends to (reference: routing.py:25-42).

    index: `[B, H, Nq, Nkv]` int32 ids by descending block-attention weight (ties: lower id first);
    num: `[B, H, Nq]` int32 selected count; mask: bool `[B, H, Nq, Nkv]` or None;
    thresholds: `[H]` float32 coverage threshold per head.
    """

    __slots__ = ("index", "num", "mask", "thresholds")

    def __init__(self, index, num, mask, thresholds):
        self.index = index
        self.num = num
        self.mask = mask
        self.thresholds = thresholds


def block_mean_pool(x: torch.Tensor, logical_len: int, num_blocks: int, block_size: int) -> torch.Tensor:
    """Mean-pool `[B, H, num_blocks * block_size, D]` to `[B, H, num_blocks, D]` (routing.py:45-61)."""
    _lib.require_cuda(x)
    bsz, heads, tokens, head_dim = x.shape
    if tokens != num_blocks * block_size:
        raise ValueError(f"expected {num_blocks * block_size} tokens, got {tokens}")
    if math.ceil(logical_len / block_size) != num_blocks:
        raise ValueError("logical_len does not span num_blocks blocks")
    pooled = torch.empty((bsz, heads, num_blocks, head_dim), device=x.device, dtype=torch.float32)
    desc = _lib.t4_bhnd(x)
    _lib.check(_lib.lib().wa_pool_blocks(desc, bsz, logical_len, heads, head_dim, block_size,
                                         pooled.data_ptr(), _lib.stream_ptr(x.device)))
    # the reference returns the input dtype for an aligned length and float32 for a ragged one
    return pooled.to(x.dtype) if logical_len % block_size == 0 else pooled


def block_attention_map(q_pooled: torch.Tensor, k_pooled: torch.Tensor) -> torch.Tensor:
    """Softmax over pooled `q.k^T / sqrt(D)`: float32 `[B, H, Nq, Nkv]` (routing.py:64-68)."""
    _lib.require_cuda(q_pooled, k_pooled)
    bsz, heads, nq, head_dim = q_pooled.shape
    nkv = k_pooled.shape[2]
    qp = q_pooled.float().contiguous()
    kp = k_pooled.float().contiguous()
    attn = torch.empty((bsz, heads, nq, nkv), device=qp.device, dtype=torch.float32)
    _lib.check(_lib.lib().wa_route_scores(qp.data_ptr(), kp.data_ptr(), bsz, heads, nq, nkv, head_dim,
                                          attn.data_ptr(), _lib.stream_ptr(qp.device)))
    return attn


def build_block_routing(block_attn: torch.Tensor, tau_min: float, tau_max: float, *,
                        return_mask: bool = False, topk_per_head: torch.Tensor | None = None) -> BlockRouting:
    """Minimal block set covering mass tau_h per (query block, head) (routing.py:71-118).

    `topk_per_head` (int32 `[H]`, optional, not in the reference signature) replaces the
    cumulative-mass count by a fixed per-head count over the same descending order.
    """
    _lib.require_cuda(block_attn)
    bsz, heads, nq, nkv = block_attn.shape
    attn = block_attn.float().contiguous()
    dev = attn.device
    index = torch.empty((bsz, heads, nq, nkv), device=dev, dtype=torch.int32)
    num = torch.empty((bsz, heads, nq), device=dev, dtype=torch.int32)
    thresholds = torch.empty((heads,), device=dev, dtype=torch.float32)
    gini = torch.empty((bsz * heads * nq,), device=dev, dtype=torch.float32)
    mask = torch.empty((bsz, heads, nq, nkv), device=dev, dtype=torch.bool) if return_mask else None
    fixed = None
    if topk_per_head is not None:
        fixed = topk_per_head.to(device=dev, dtype=torch.int32).contiguous()
        if fixed.numel() != heads:
            raise ValueError(f"topk_per_head must have {heads} entries")
    _lib.check(_lib.lib().wa_route_select(attn.data_ptr(), bsz, heads, nq, nkv, float(tau_min), float(tau_max),
                                          _lib.ptr(fixed), index.data_ptr(), num.data_ptr(), _lib.ptr(mask),
                                          thresholds.data_ptr(), gini.data_ptr(), _lib.stream_ptr(dev)))
    return BlockRouting(index=index, num=num, mask=mask, thresholds=thresholds)


def variable_block_sizes(kv_len: int, kv_len_padded: int, block_size: int, device) -> torch.Tensor:
    """Real token count of each key block; only the trailing one can be short (routing.py:121-126)."""
    kv_blocks = kv_len_padded // block_size
    sizes = torch.full((kv_blocks,), block_size, dtype=torch.int32, device=device)
    sizes[-1] = kv_len - (kv_blocks - 1) * block_size
    return sizes


def pad_to_len(x: torch.Tensor, target_len: int) -> torch.Tensor:
    """Zero-pad `[B, L, H, D]` along the token axis (routing.py:129-135)."""
    pad_len = target_len - x.shape[1]
    if pad_len <= 0:
        return x
    return torch.nn.functional.pad(x, (0, 0, 0, 0, 0, pad_len))


def block_counts(q_len: int, kv_len: int, block_size: int) -> tuple[int, int, int, int]:
    """Padded lengths and block counts (routing.py:138-142)."""
    q_pad = math.ceil(q_len / block_size) * block_size
    kv_pad = math.ceil(kv_len / block_size) * block_size
    return q_pad, kv_pad, q_pad // block_size, kv_pad // block_size
