"""Block-sparse attention with the reference semantics, any shape, on the GPU.

Keeps the name and signature of the reference's `block_sparse_attention_reference`
(wan/modules/hsa/block_sparse_torch.py:16-64) so callers and tests switch over unchanged; the
computation is the shape-generic CUDA kernel in csrc/wa_attention_generic.cu (float32 math, exact
softmax over the selected blocks, trailing partial block masked, empty selection -> zeros).
"""
from __future__ import annotations

import torch

from .. import _lib

__all__ = ["block_sparse_attention_reference"]


def block_sparse_attention_reference(q, k, v, q2k_index, q2k_num, block_sizes, block_size: int,
                                     return_lse: bool = False):
    """Attention over selected blocks for `[B, H, N, D]` inputs padded to `block_size`."""
    dev = _lib.require_cuda(q, k, v, q2k_index, q2k_num, block_sizes)
    bsz, heads, q_tokens, head_dim = q.shape
    kv_tokens = k.shape[2]
    if q_tokens % block_size or kv_tokens % block_size:
        raise ValueError("q and k/v must be padded to a multiple of block_size")
    k = k.to(q.dtype)
    v = v.to(q.dtype)
    out = torch.empty((bsz, heads, q_tokens, head_dim), device=dev, dtype=q.dtype)
    lse = torch.empty((bsz, heads, q_tokens), device=dev, dtype=torch.float32) if return_lse else None
    index = q2k_index.to(torch.int32).contiguous()
    num = q2k_num.to(torch.int32).contiguous()
    sizes = block_sizes.to(torch.int32).contiguous()
    _lib.check(_lib.lib().wa_block_sparse_forward(
        _lib.t4_bhnd(q), _lib.t4_bhnd(k), _lib.t4_bhnd(v), _lib.t4_bhnd(out), bsz, heads, q_tokens, kv_tokens,
        head_dim, block_size, index.data_ptr(), num.data_ptr(), index.shape[-1], sizes.data_ptr(), 0, 0,
        _lib.ptr(lse), _lib.stream_ptr(dev)))
    return (out, lse) if return_lse else out
